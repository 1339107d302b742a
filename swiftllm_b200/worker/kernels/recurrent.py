"""Kernels of recurrent mixers (csrc/recurrent.cu).  Their state is one row per SEQUENCE (the sequence's block-table row) of
fp32 tensors that live as long as the worker; a step's rows are segments of consecutive positions (infer_state.seg_starts /
seq_ids); a segment that starts at position 0 starts from the zero state, whatever its row still holds."""
import torch

from swiftllm_b200 import _lib


def _stride0(x: torch.Tensor) -> int:
    return x.stride(0) if x.shape[0] > 1 else max(x.stride(0), x.shape[1])


def causal_conv(xin: torch.Tensor, w: torch.Tensor, bias, tail: torch.Tensor, infer_state) -> torch.Tensor:
    """xin [T, C] (a column slice is fine), w [C, taps] (last column: the current token), tail [rows, taps - 1, C] -> u [T, C]."""
    T, C = xin.shape
    taps = w.shape[1]
    assert xin.stride(1) == 1 and w.is_contiguous() and w.shape[0] == C and w.dtype == xin.dtype
    assert taps == 1 or (tail.is_contiguous() and tail.shape[1:] == (taps - 1, C) and tail.dtype == xin.dtype)
    _lib.require_device(xin)
    u = torch.empty((T, C), dtype=xin.dtype, device=xin.device)
    _lib.check(_lib.lib().sllm_causal_conv(xin.data_ptr(), _stride0(xin), w.data_ptr(), _lib.ptr(bias), _lib.ptr(tail),
                                           infer_state.token_seq_ids.data_ptr(), infer_state.token_positions.data_ptr(), u.data_ptr(),
                                           T, min(T, max(0, int(getattr(infer_state, "num_prefill_tokens", T)))), C, taps, _lib.dtype_tag_f32(xin.dtype), _lib.stream()), "causal_conv")
    return u


def rglru_scan(u: torch.Tensor, gates: torch.Tensor, ybr: torch.Tensor, rate: torch.Tensor, xin: torch.Tensor, state: torch.Tensor,
               tail: torch.Tensor, infer_state) -> torch.Tensor:
    """u [T, C]; gates [blocks, T, 2 * C / blocks] logits (recurrence gate | input gate); ybr [T, C] pre-activation of the GELU
    branch; rate fp32 [C] (log a = rate * sigmoid(r)); xin [T, C] the convolution's inputs (for the tail); state fp32 [rows, C].
    -> S * gelu(ybr) [T, C]; state and tail move on.  The first infer_state.num_prefill_seqs segments (prompt portions) go
    through the kernel that is parallel over time, the rest (single decoded tokens) through the one-thread-per-channel kernel."""
    T, C = u.shape
    blocks, taps = gates.shape[0], tail.shape[1] + 1
    assert u.is_contiguous() and gates.is_contiguous() and gates.shape == (blocks, T, 2 * C // blocks) and gates.dtype == u.dtype
    assert ybr.stride(1) == 1 and xin.stride(1) == 1 and rate.dtype == torch.float32 and state.dtype == torch.float32
    assert state.is_contiguous() and state.shape[1] == C and tail.is_contiguous() and tail.dtype == u.dtype
    _lib.require_device(u)
    st = infer_state
    out = torch.empty((T, C), dtype=u.dtype, device=u.device)
    _lib.check(_lib.lib().sllm_rglru_scan(u.data_ptr(), gates.data_ptr(), blocks, ybr.data_ptr(), _stride0(ybr), rate.data_ptr(),
                                          xin.data_ptr(), _stride0(xin), state.data_ptr(), tail.data_ptr(), st.seg_starts.data_ptr(),
                                          st.seq_ids.data_ptr(), st.token_positions.data_ptr(), out.data_ptr(), T, st.batch_size,
                                          min(st.batch_size, max(0, int(getattr(st, "num_prefill_seqs", st.batch_size)))), C, taps, _lib.dtype_tag_f32(u.dtype), _lib.stream()), "rglru_scan")
    return out


def linear_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, state: torch.Tensor, infer_state,
                     heads: int, dk: int, dv: int) -> torch.Tensor:
    """q, k [T, H * dk], v [T, H * dv] pre-activation (column slices are fine); decay fp32 [H]; state fp32 [rows, H, dk, dv]
    -> fp32 [T, H * dv]."""
    T = q.shape[0]
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1 and q.shape == k.shape == (T, heads * dk) and v.shape == (T, heads * dv)
    assert decay.dtype == torch.float32 and state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (heads, dk, dv)
    _lib.require_device(q)
    st = infer_state
    out = torch.empty((T, heads * dv), dtype=torch.float32, device=q.device)
    _lib.check(_lib.lib().sllm_linear_attention(q.data_ptr(), _stride0(q), k.data_ptr(), _stride0(k), v.data_ptr(), _stride0(v),
                                                decay.data_ptr(), state.data_ptr(), st.seg_starts.data_ptr(), st.seq_ids.data_ptr(),
                                                st.token_positions.data_ptr(), out.data_ptr(), st.batch_size, heads, dk, dv,
                                                _lib.dtype_tag_f32(q.dtype), _lib.stream()), "linear_attention")
    return out


def gated_rmsnorm(x: torch.Tensor, weight: torch.Tensor, gate, eps: float, out: torch.Tensor, out_scale: float = 1.0):
    """out [T, n] (a column slice is fine) = x / rms(x) * weight * sigmoid(gate) * out_scale; x fp32 [T, n], gate logits or None."""
    T, n = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and weight.dtype == torch.float32 and weight.shape == (n,)
    assert out.shape == (T, n) and out.stride(1) == 1 and (gate is None or (gate.shape == (T, n) and gate.stride(1) == 1 and gate.dtype == out.dtype))
    _lib.require_device(x)
    _lib.check(_lib.lib().sllm_gated_rmsnorm(x.data_ptr(), weight.data_ptr(), _lib.ptr(gate), _stride0(gate) if gate is not None else 0,
                                             eps, out_scale, out.data_ptr(), _stride0(out), T, n, _lib.dtype_tag_f32(out.dtype),
                                             _lib.stream()), "gated_rmsnorm")
