"""Per-channel recurrences with per-sequence state (csrc/scan_ops.cu): a short causal convolution whose last inputs are carried
per sequence, the minGRU scan and the selective state-space scan.  State tensors have one row per SEQUENCE (the sequence's
block-table row); a step's rows are segments of consecutive positions (infer_state.seg_starts / seq_ids); a segment that starts at
position 0 starts from the zero state, whatever its row still holds."""
import torch

from swiftllm_b200 import _lib


def _stride0(x: torch.Tensor) -> int:
    return x.stride(0) if x.shape[0] > 1 else max(x.stride(0), x.shape[1])


def _prefill_segs(st) -> int:
    """Leading segments of the step that are prompt portions (they take the kernels that tile over time)."""
    return min(st.batch_size, max(0, int(getattr(st, "num_prefill_seqs", st.batch_size))))


def short_conv(xin: torch.Tensor, w: torch.Tensor, bias, tail: torch.Tensor, infer_state, out_dtype: torch.dtype,
               add_input: bool = False, silu: bool = False, move_tail: bool = False) -> torch.Tensor:
    """xin [T, C] (fp32 or out_dtype; a column slice is fine), w fp32 [C, taps] (last column: the current token), bias fp32 [C] or
    None, tail [rows, taps - 1, C] of xin's dtype -> [T, C] out_dtype = act(conv(xin)) (+ xin).  move_tail: every sequence's tail
    moves on by the step's inputs - decoded tokens' inside the convolution kernel, prompt portions' in a launch of their own
    behind it; otherwise the tail is only read."""
    T, C = xin.shape
    taps = w.shape[1]
    assert xin.stride(1) == 1 and w.is_contiguous() and w.shape[0] == C and w.dtype == torch.float32
    assert bias is None or (bias.dtype == torch.float32 and bias.shape == (C,))
    assert taps == 1 or (tail.is_contiguous() and tail.shape[1:] == (taps - 1, C) and tail.dtype == xin.dtype)
    _lib.require_device(xin)
    out = torch.empty((T, C), dtype=out_dtype, device=xin.device)
    npre = min(T, max(0, int(getattr(infer_state, "num_prefill_tokens", T))))
    _lib.check(_lib.lib().sllm_short_conv(xin.data_ptr(), _stride0(xin), _lib.dtype_tag_f32(xin.dtype), w.data_ptr(), _lib.ptr(bias),
                                          _lib.ptr(tail), infer_state.token_seq_ids.data_ptr(), infer_state.token_positions.data_ptr(),
                                          out.data_ptr(), _lib.dtype_tag_f32(out_dtype), T, npre, C, taps, 1 if add_input else 0,
                                          1 if silu else 0, 1 if move_tail else 0, _lib.stream()), "short_conv")
    if move_tail and taps > 1 and _prefill_segs(infer_state) > 0:
        conv_tail_update(xin, tail, infer_state, _prefill_segs(infer_state))
    return out


def conv_tail_update(xin: torch.Tensor, tail: torch.Tensor, infer_state, num_segs: int = None):
    """tail [rows, taps - 1, C] <- the sequences' last taps - 1 inputs after the step (xin [T, C], same dtype), for the step's
    first num_segs segments (default: all)."""
    C, taps = xin.shape[1], tail.shape[1] + 1
    assert xin.stride(1) == 1 and tail.is_contiguous() and tail.dtype == xin.dtype and tail.shape[2] == C
    _lib.require_device(xin)
    st = infer_state
    _lib.check(_lib.lib().sllm_conv_tail_update(xin.data_ptr(), _stride0(xin), tail.data_ptr(), st.seg_starts.data_ptr(),
                                                st.seq_ids.data_ptr(), st.token_positions.data_ptr(),
                                                st.batch_size if num_segs is None else num_segs, C, taps,
                                                _lib.dtype_tag_f32(xin.dtype), _lib.stream()), "conv_tail_update")


def mingru_scan(proj: torch.Tensor, state: torch.Tensor, infer_state, channels: int) -> torch.Tensor:
    """proj [T, 3 C] = [z logits | candidate pre-activations | output-gate pre-activations]; state fp32 [rows, C] (moves on)
    -> S * silu(g) [T, C] in proj's dtype."""
    T, C = proj.shape[0], channels
    assert proj.stride(1) == 1 and proj.shape[1] == 3 * C and state.dtype == torch.float32 and state.is_contiguous() and state.shape[1] == C
    _lib.require_device(proj)
    st = infer_state
    out = torch.empty((T, C), dtype=proj.dtype, device=proj.device)
    _lib.check(_lib.lib().sllm_mingru_scan(proj.data_ptr(), _stride0(proj), state.data_ptr(), st.seg_starts.data_ptr(),
                                           st.seq_ids.data_ptr(), st.token_positions.data_ptr(), out.data_ptr(), st.batch_size,
                                           _prefill_segs(st), C, _lib.dtype_tag_f32(proj.dtype), _lib.stream()), "mingru_scan")
    return out


def selective_scan(x: torch.Tensor, dt: torch.Tensor, dt_bias: torch.Tensor, A: torch.Tensor, bc: torch.Tensor, b_off: int,
                   c_off: int, D: torch.Tensor, z: torch.Tensor, state: torch.Tensor, infer_state) -> torch.Tensor:
    """x, z [T, C]; dt [T, C] step logits (fp32 or x's dtype); bc [T, ...] rows with B at column b_off and C at c_off (N each);
    A fp32 [C, N] (negative), D, dt_bias fp32 [C]; state fp32 [rows, C, N] (moves on) -> (y + D x) * silu(z) [T, C]."""
    T, C = x.shape
    N = A.shape[1]
    assert x.stride(1) == 1 and z.stride(1) == 1 and dt.stride(1) == 1 and bc.stride(1) == 1 and z.shape == (T, C) and dt.shape == (T, C)
    assert bc.dtype == x.dtype == z.dtype and dt.dtype in (torch.float32, x.dtype) and max(b_off, c_off) + N <= bc.shape[1]
    assert A.dtype == D.dtype == dt_bias.dtype == torch.float32 and A.is_contiguous() and A.shape == (C, N)
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (C, N)
    _lib.require_device(x)
    st = infer_state
    out = torch.empty((T, C), dtype=x.dtype, device=x.device)
    _lib.check(_lib.lib().sllm_selective_scan(
        x.data_ptr(), _stride0(x), dt.data_ptr(), _stride0(dt), 1 if dt.dtype == torch.float32 else 0, dt_bias.data_ptr(), A.data_ptr(),
        bc.data_ptr(), _stride0(bc), b_off, c_off, D.data_ptr(), z.data_ptr(), _stride0(z), state.data_ptr(), st.seg_starts.data_ptr(),
        st.seq_ids.data_ptr(), st.token_positions.data_ptr(), out.data_ptr(), st.batch_size, _prefill_segs(st), C, N,
        _lib.dtype_tag_f32(x.dtype), _lib.stream()), "selective_scan")
    return out
