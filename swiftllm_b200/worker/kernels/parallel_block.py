"""Kernels of parallel decoder blocks with an fp32 residual stream (csrc/parallel_block.cu): fused residual add + RMS norm,
row-strided RMS norm, squared ReLU, and the mixture-of-experts router with its weight-applying activation.  The storage
dtype of activations may be float16, bfloat16 or float32; sums, norms and the router are fp32 in every case."""
import torch

from swiftllm_b200 import _lib


def add_rmsnorm_f32(residual: torch.Tensor, a, b, weight: torch.Tensor, eps: float, out: torch.Tensor = None,
                    out_dtype: torch.dtype = None) -> torch.Tensor:
    """residual (fp32 [T, W], updated in place) += a + b (either may be None); returns rmsnorm(residual) * weight in
    `out_dtype` (default: weight's dtype).  The weight is stored in the output dtype or in fp32."""
    assert residual.dtype == torch.float32 and residual.is_contiguous() and weight.is_contiguous()
    _lib.require_device(residual)
    T, W = residual.shape
    if out is None:
        out = torch.empty((T, W), dtype=out_dtype or weight.dtype, device=residual.device)
    for x in (a, b):
        assert x is None or (x.dtype == out.dtype and x.is_contiguous() and x.shape == residual.shape)
    if weight.dtype == out.dtype:
        fn, what = _lib.lib().sllm_add_rmsnorm_f32, "add_rmsnorm_f32"
    else:
        assert weight.dtype == torch.float32, "norm weights are stored in the activation dtype or in float32"
        fn, what = _lib.lib().sllm_add_rmsnorm_f32w, "add_rmsnorm_f32w"
    _lib.check(fn(residual.data_ptr(), _lib.ptr(a), _lib.ptr(b), weight.data_ptr(), out.data_ptr(), eps, T, W,
                  _lib.dtype_tag_f32(out.dtype), _lib.stream()), what)
    return out


def rmsnorm_strided(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm of x [T, n] (a column slice of a wider matrix is fine) -> new contiguous [T, n]."""
    assert x.dim() == 2 and x.stride(1) == 1 and weight.is_contiguous() and weight.dtype == x.dtype
    _lib.require_device(x)
    T, n = x.shape
    out = torch.empty((T, n), dtype=x.dtype, device=x.device)
    _lib.check(_lib.lib().sllm_rmsnorm_strided(x.data_ptr(), x.stride(0) if T > 1 else max(x.stride(0), n), weight.data_ptr(),
                                               out.data_ptr(), n, eps, T, n, _lib.dtype_tag_f32(x.dtype), _lib.stream()),
               "rmsnorm_strided")
    return out


def relu2_inplace(x: torch.Tensor):
    assert x.is_contiguous()
    _lib.require_device(x)
    _lib.check(_lib.lib().sllm_relu2_inplace(x.data_ptr(), x.numel(), _lib.dtype_tag_f32(x.dtype), _lib.stream()), "relu2_inplace")


def moe_route(logits: torch.Tensor, top: int) -> torch.Tensor:
    """logits fp32 [T, E] -> routing weights fp32 [T, E]: softmax over each row's `top` largest logits, 0 elsewhere."""
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    _lib.require_device(logits)
    w = torch.empty_like(logits)
    _lib.check(_lib.lib().sllm_moe_route(logits.data_ptr(), w.data_ptr(), logits.shape[0], logits.shape[1], top, _lib.stream()),
               "moe_route")
    return w


def moe_relu2_scale_inplace(u: torch.Tensor, weights: torch.Tensor, ff: int):
    """u [T, E * ff] = relu(u)^2 * weights[t, column // ff]."""
    assert u.is_contiguous() and weights.dtype == torch.float32 and weights.is_contiguous()
    _lib.require_device(u)
    T, E = weights.shape
    assert u.shape == (T, E * ff)
    _lib.check(_lib.lib().sllm_moe_relu2_scale_inplace(u.data_ptr(), weights.data_ptr(), T, E, ff, _lib.dtype_tag_f32(u.dtype),
                                                       _lib.stream()), "moe_relu2_scale_inplace")


def moe_route_grouped(logits: torch.Tensor, top: int, groups: int, keep: int, scale: float, norm_eps: float) -> torch.Tensor:
    """logits fp32 [T, E] -> routing weights fp32 [T, E]: scores are a softmax over all experts; only experts of the `keep`
    best of `groups` equal groups (a group's score: its largest score) can be chosen; the `top` largest of those get
    score / (sum of chosen scores + norm_eps) * scale, the others 0."""
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    _lib.require_device(logits)
    w = torch.empty_like(logits)
    _lib.check(_lib.lib().sllm_moe_route_grouped(logits.data_ptr(), w.data_ptr(), logits.shape[0], logits.shape[1], top, groups,
                                                 keep, scale, norm_eps, _lib.stream()), "moe_route_grouped")
    return w


def moe_clamped_glu_scale(u: torch.Tensor, weights, experts: int, ff: int, limit: float, shared_ff: int, shared_limit: float,
                          alpha: float, shared_gated: bool = False) -> torch.Tensor:
    """u [T, 2 * (experts * ff + shared_ff)]: per expert [gate | up], then the shared expert's [gate | up] ->
    y [T, experts * ff + shared_ff] = min(gate, limit) * sigmoid(alpha * .) * (clamp(up, +-limit) + 1) * weights[t, expert]
    (the shared expert: its own limit, weight 1 - or, with shared_gated, the extra last column of weights [T, experts + 1])."""
    assert u.is_contiguous() and (weights is None or (weights.dtype == torch.float32 and weights.is_contiguous()))
    _lib.require_device(u)
    T, cols = u.shape[0], experts * ff + shared_ff
    assert u.shape == (T, 2 * cols) and (weights is None or weights.shape == (T, experts + (1 if shared_gated else 0)))
    assert weights is not None or (experts == 0 and not shared_gated)
    y = torch.empty((T, cols), dtype=u.dtype, device=u.device)
    _lib.check(_lib.lib().sllm_moe_clamped_glu_scale(u.data_ptr(), _lib.ptr(weights), y.data_ptr(), T, experts, ff, limit, shared_ff,
                                                     shared_limit, alpha, 1 if shared_gated else 0, _lib.dtype_tag_f32(u.dtype),
                                                     _lib.stream()),
               "moe_clamped_glu_scale")
    return y
