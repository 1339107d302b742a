"""Gated sliding-window attention with grouped key/value heads over the paged cache (csrc/window_attn.cu).  Cache layout
[num_blocks, slots, block_size, G * (dk + dv)]: per token and layer ONE row [rotated keys of all G heads | their values].

Options (`AttnOptions`) that other designs switch on: rotary pairs as halves instead of neighbours, unit-RMS queries and keys, a
tanh cap on the scores, values that are stored turned by their position (the output is turned back), a factor on the output, an
RMS norm with weight on every query / key head before it turns, a chunked mask, several key heads (score maps) per value head
with fp32 output, and `diff_combine`, which turns two maps' outputs into one gated head."""
import dataclasses
import torch

from swiftllm_b200 import _lib


@dataclasses.dataclass(frozen=True)
class AttnOptions:
    pair_halves: bool = False       # rotary pairs (i, i + rot_dims / 2) instead of (2i, 2i + 1)
    qk_norm_eps: float = -1.0       # >= 0: rotated queries / keys are divided by sqrt(mean of squares over the head + eps)
    softcap: float = 0.0            # > 0: score <- softcap * tanh(score / softcap)
    out_scale: float = 1.0
    q_norm: object = None           # fp32 [dk] weights of an RMS norm over every query / key head BEFORE rotation (eps: prenorm_eps)
    k_norm: object = None
    prenorm_eps: float = 0.0
    chunk: int = 0                  # > 0: a query at position p sees only positions >= floor(p / chunk) * chunk
    vshare: int = 1                 # this many neighbouring key heads share one value head (cache row: G keys, G / vshare values)
    out_f32: bool = False           # the attention output is fp32 whatever the storage dtype


PLAIN = AttnOptions()


def _stride0(x: torch.Tensor) -> int:
    return x.stride(0) if x.shape[0] > 1 else max(x.stride(0), x.shape[1])


def window_kv_store(k: torch.Tensor, v: torch.Tensor, cache: torch.Tensor, slot: int, block_table: torch.Tensor, infer_state,
                    kv_heads: int, dk: int, dv: int, rot_dims: int, cos: torch.Tensor, sin: torch.Tensor,
                    opt: AttnOptions = PLAIN, vcos: torch.Tensor = None, vsin: torch.Tensor = None):
    """k [T, G * dk], v [T, G * dv] (row-strided slices are fine): rotate the keys, write the tokens' cache rows.
    vcos / vsin fp32 [T, dv / 2]: the values are stored turned by their position."""
    T = k.shape[0]
    gv = kv_heads // opt.vshare
    assert k.dim() == 2 and k.stride(1) == 1 and v.stride(1) == 1 and k.shape[1] == kv_heads * dk and v.shape == (T, gv * dv)
    assert cache.is_contiguous() and cache.dtype == k.dtype == v.dtype and cache.shape[3] == kv_heads * dk + gv * dv
    assert opt.k_norm is None or (opt.k_norm.dtype == torch.float32 and opt.k_norm.shape == (dk,))
    _lib.require_device(k)
    _lib.check(_lib.lib().sllm_window_kv_store(
        k.data_ptr(), _stride0(k), v.data_ptr(), _stride0(v), _lib.ptr(cos), _lib.ptr(sin), infer_state.token_seq_ids.data_ptr(),
        infer_state.token_positions.data_ptr(), block_table.data_ptr(), block_table.shape[1], cache.data_ptr(), cache.shape[1],
        slot, cache.shape[2], T, kv_heads, dk, dv, rot_dims, 1 if opt.pair_halves else 0, opt.qk_norm_eps, _lib.ptr(vcos),
        _lib.ptr(vsin), _lib.ptr(opt.k_norm), opt.prenorm_eps, opt.vshare, _lib.dtype_tag_f32(k.dtype), _lib.stream()),
        "window_kv_store")


def window_attention(q: torch.Tensor, gate, cache: torch.Tensor, slot: int, block_table: torch.Tensor, infer_state,
                     out: torch.Tensor, heads: int, kv_heads: int, dk: int, dv: int, rot_dims: int, window: int, scale: float,
                     sink: bool, cos: torch.Tensor, sin: torch.Tensor, opt: AttnOptions = PLAIN, vcos: torch.Tensor = None,
                     vsin: torch.Tensor = None):
    """q [T, H * dk] (un-rotated), gate [T, H * dv] logits or None, out [T, H * dv] (fp32 with opt.out_f32); row-strided slices
    are fine."""
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.shape == (T, heads * dk) and out.shape == (T, heads * dv)
    assert gate is None or (gate.shape == (T, heads * dv) and gate.stride(1) == 1 and gate.dtype == q.dtype)
    assert cache.shape[3] == kv_heads * dk + kv_heads // opt.vshare * dv and cache.dtype == q.dtype
    assert out.dtype == (torch.float32 if opt.out_f32 else q.dtype)
    assert opt.q_norm is None or (opt.q_norm.dtype == torch.float32 and opt.q_norm.shape == (dk,))
    _lib.require_device(q)
    _lib.check(_lib.lib().sllm_window_attention(
        q.data_ptr(), _stride0(q), _lib.ptr(cos), _lib.ptr(sin), _lib.ptr(gate), _stride0(gate) if gate is not None else 0,
        cache.data_ptr(), cache.shape[1], slot, cache.shape[2], block_table.data_ptr(), block_table.shape[1],
        infer_state.token_seq_ids.data_ptr(), infer_state.token_positions.data_ptr(), out.data_ptr(), _stride0(out), T,
        min(T, max(0, int(getattr(infer_state, "num_prefill_tokens", T)))), heads, kv_heads, dk, dv, rot_dims, window, scale, 1 if sink else 0,
        1 if opt.pair_halves else 0, opt.qk_norm_eps, opt.softcap, _lib.ptr(vcos), _lib.ptr(vsin), opt.out_scale,
        _lib.ptr(opt.q_norm), opt.prenorm_eps, opt.chunk, opt.vshare, 1 if opt.out_f32 else 0, _lib.dtype_tag_f32(q.dtype),
        _lib.stream()),
        "window_attention")


def diff_combine(a: torch.Tensor, gate, out: torch.Tensor, heads: int, kv_heads: int, dv: int, lam: float, eps: float,
                 factor: float):
    """a fp32 [T, 2 * heads * dv] laid out [key/value head][map][head of the group][dv] (window_attention with vshare = 2 and
    out_f32) -> out [T, heads * dv] (heads in their natural order) = o / sqrt(mean(o^2) + eps) * factor * sigmoid(gate) with
    o = map 0 - lam * map 1; gate [T, heads * dv] logits or None; row-strided slices are fine for gate and out."""
    T = a.shape[0]
    assert a.dtype == torch.float32 and a.is_contiguous() and a.shape == (T, 2 * heads * dv)
    assert out.shape == (T, heads * dv) and out.stride(1) == 1
    assert gate is None or (gate.shape == out.shape and gate.stride(1) == 1 and gate.dtype == out.dtype)
    _lib.require_device(a)
    _lib.check(_lib.lib().sllm_diff_combine(a.data_ptr(), _lib.ptr(gate), _stride0(gate) if gate is not None else 0, out.data_ptr(),
                                            _stride0(out), T, heads, kv_heads, dv, lam, eps, factor, _lib.dtype_tag_f32(out.dtype),
                                            _lib.stream()), "diff_combine")


def set_simt(on: bool) -> bool:
    """Force the fp32 CUDA-core attention kernel for every shape (tests compare the two paths); returns the old setting."""
    return bool(_lib.lib().sllm_window_attention_set_simt(1 if on else 0))
