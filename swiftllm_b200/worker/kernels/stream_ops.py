"""Kernels of sequential decoder blocks on an fp32 residual stream whose sublayer outputs are normalised before they are added
(csrc/stream_ops.cu): the embedding with a hashed table of token pairs, the post-norm add with the weighted sum over depth, the
tanh cap, and the sigmoid router with the SiLU-gated expert activation.  The stream, norms and the router are fp32 for every
storage dtype of the projections."""
import torch

from swiftllm_b200 import _lib


def embed_pair_hash(tokens: torch.Tensor, infer_state, last_token: torch.Tensor, embed: torch.Tensor, pairs, buckets: int,
                    mul_prev: int, mul_cur: int, x_copy: torch.Tensor = None):
    """-> (x fp32 [T, W], h [T, W] in embed's dtype).  x = embed[token] + pairs[hash(previous token, token)] (pairs may be None);
    the previous token of a step's first row comes from last_token[sequence row], which is then moved on to the step's last
    token.  x_copy (fp32 [T, W]) receives the same values."""
    _lib.require_device(embed)
    T, W = tokens.shape[0], embed.shape[1]
    assert tokens.dtype == torch.int32 and embed.is_contiguous() and (pairs is None or (pairs.is_contiguous() and pairs.dtype == embed.dtype))
    x = torch.empty((T, W), dtype=torch.float32, device=embed.device)
    h = torch.empty((T, W), dtype=embed.dtype, device=embed.device)
    st = infer_state
    _lib.check(_lib.lib().sllm_embed_pair_hash(
        tokens.data_ptr(), st.token_seq_ids.data_ptr(), st.token_positions.data_ptr(), _lib.ptr(last_token), embed.data_ptr(),
        _lib.ptr(pairs), buckets, mul_prev, mul_cur, x.data_ptr(), _lib.ptr(x_copy), h.data_ptr(), T, W,
        _lib.dtype_tag_f32(embed.dtype), _lib.stream()), "embed_pair_hash")
    if pairs is not None:
        _lib.check(_lib.lib().sllm_store_last_tokens(tokens.data_ptr(), st.seg_starts.data_ptr(), st.seq_ids.data_ptr(),
                                                     last_token.data_ptr(), st.batch_size, _lib.stream()), "store_last_tokens")
    return x, h


def postnorm_add_mix(x: torch.Tensor, y, gain, eps: float, h: torch.Tensor, history: torch.Tensor = None, slot: int = 0,
                     mix: torch.Tensor = None):
    """x (fp32 [T, W], in place) <- x + gain * y / rms(y)  (y None: unchanged); with `history` (fp32 [slots, T, W]) the result is
    kept in history[slot], and with `mix` (fp32 [slot + 1]) x <- sum_j mix[j] * history[j].  h <- x rounded to h's dtype."""
    assert x.dtype == torch.float32 and x.is_contiguous() and h.is_contiguous() and h.shape == x.shape
    assert y is None or (y.dtype == h.dtype and y.is_contiguous() and y.shape == x.shape and gain.dtype == torch.float32)
    assert history is None or (history.dtype == torch.float32 and history.is_contiguous() and history.shape[1:] == x.shape)
    assert mix is None or (history is not None and mix.dtype == torch.float32 and mix.numel() == slot + 1 and slot < history.shape[0])
    _lib.require_device(x)
    _lib.check(_lib.lib().sllm_postnorm_add_mix(x.data_ptr(), _lib.ptr(y), _lib.ptr(gain), eps, _lib.ptr(history), slot, _lib.ptr(mix),
                                                h.data_ptr(), x.shape[0], x.shape[1], _lib.dtype_tag_f32(h.dtype), _lib.stream()),
               "postnorm_add_mix")


def tanh_cap_inplace(x: torch.Tensor, cap: float):
    assert x.is_contiguous()
    _lib.require_device(x)
    _lib.check(_lib.lib().sllm_tanh_cap_inplace(x.data_ptr(), x.numel(), cap, _lib.dtype_tag_f32(x.dtype), _lib.stream()), "tanh_cap_inplace")


def moe_route_sigmoid(logits: torch.Tensor, bias, top: int) -> torch.Tensor:
    """logits fp32 [T, E] -> routing weights fp32 [T, E]: sigmoid scores at the `top` experts with the largest score + bias."""
    assert logits.dtype == torch.float32 and logits.is_contiguous() and (bias is None or bias.dtype == torch.float32)
    _lib.require_device(logits)
    w = torch.empty_like(logits)
    _lib.check(_lib.lib().sllm_moe_route_sigmoid(logits.data_ptr(), _lib.ptr(bias), w.data_ptr(), logits.shape[0], logits.shape[1], top,
                                                 _lib.stream()), "moe_route_sigmoid")
    return w


def moe_silu_glu_scale(u: torch.Tensor, weights: torch.Tensor, experts: int, ff: int) -> torch.Tensor:
    """u [T, experts * 2 * ff] (per expert [gate | up]) -> y [T, experts * ff] = silu(gate) * up * weights[t, expert]."""
    assert u.is_contiguous() and weights.dtype == torch.float32 and weights.is_contiguous()
    _lib.require_device(u)
    T = u.shape[0]
    assert u.shape == (T, 2 * experts * ff) and weights.shape == (T, experts)
    y = torch.empty((T, experts * ff), dtype=u.dtype, device=u.device)
    _lib.check(_lib.lib().sllm_moe_silu_glu_scale(u.data_ptr(), weights.data_ptr(), y.data_ptr(), T, experts, ff,
                                                  _lib.dtype_tag_f32(u.dtype), _lib.stream()), "moe_silu_glu_scale")
    return y
