"""Row-wise kernels of sandwich blocks (csrc/sandwich_ops.cu): x <- x + mult * norm_b(sublayer(norm_a(x))) with RMS norms over
equal consecutive groups of a row, the addition of a saved stream / a row vector, the GELU gated linear unit, and the softmax
router whose weights are the chosen experts' plain scores (with a per-token sigmoid weight for a shared expert).  The stream,
norms and the router are fp32 for every storage dtype of the projections."""
import torch

from swiftllm_b200 import _lib


def group_norm_add_norm(x: torch.Tensor, y, wb, mult: float, wn, eps: float, groups: int, n_out: torch.Tensor = None):
    """x fp32 [T, W] in place.  With y ([T, W], storage dtype) and wb (fp32 [W]): x += mult * y / rms_g(y) * wb.  With wn (fp32
    [W]): returns n = x / rms_g(x) * wn (fp32 [T, W]) of the updated x.  rms_g: per group of W / groups consecutive entries."""
    assert x.dtype == torch.float32 and x.is_contiguous() and x.shape[1] % groups == 0
    assert y is None or (y.is_contiguous() and y.shape == x.shape and wb.dtype == torch.float32 and wb.shape == (x.shape[1],))
    assert wn is None or (wn.dtype == torch.float32 and wn.shape == (x.shape[1],))
    _lib.require_device(x)
    if wn is not None and n_out is None:
        n_out = torch.empty_like(x)
    _lib.check(_lib.lib().sllm_group_norm_add_norm(x.data_ptr(), _lib.ptr(y), _lib.ptr(wb), mult, _lib.ptr(wn), _lib.ptr(n_out), eps,
                                                   x.shape[0], x.shape[1], groups,
                                                   _lib.dtype_tag_f32(y.dtype if y is not None else torch.float32), _lib.stream()),
               "group_norm_add_norm")
    return n_out


def group_norm_cast(x: torch.Tensor, w: torch.Tensor, eps: float, groups: int, out_dtype: torch.dtype) -> torch.Tensor:
    """x fp32 [T, W] -> x / rms_g(x) * w in out_dtype."""
    assert x.dtype == torch.float32 and x.is_contiguous() and w.dtype == torch.float32 and x.shape[1] % groups == 0
    _lib.require_device(x)
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    _lib.check(_lib.lib().sllm_group_norm_cast(x.data_ptr(), w.data_ptr(), out.data_ptr(), eps, x.shape[0], x.shape[1], groups,
                                               _lib.dtype_tag_f32(out_dtype), _lib.stream()), "group_norm_cast")
    return out


def stream_add(x: torch.Tensor, a=None, v=None):
    """x fp32 [T, W] in place += a (fp32 [T, W]) + v (fp32 [W]); either may be None."""
    assert x.dtype == torch.float32 and x.is_contiguous()
    assert a is None or (a.dtype == torch.float32 and a.is_contiguous() and a.shape == x.shape)
    assert v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.shape == (x.shape[1],))
    _lib.require_device(x)
    _lib.check(_lib.lib().sllm_stream_add(x.data_ptr(), _lib.ptr(a), _lib.ptr(v), x.shape[0], x.shape[1], _lib.stream()), "stream_add")


def gelu_glu(u: torch.Tensor) -> torch.Tensor:
    """u [T, 2 F] = [gate | up] -> gelu_tanh(gate) * up [T, F]."""
    assert u.is_contiguous() and u.shape[1] % 2 == 0
    _lib.require_device(u)
    T, F = u.shape[0], u.shape[1] // 2
    y = torch.empty((T, F), dtype=u.dtype, device=u.device)
    _lib.check(_lib.lib().sllm_gelu_glu(u.data_ptr(), y.data_ptr(), T, F, _lib.dtype_tag_f32(u.dtype), _lib.stream()), "gelu_glu")
    return y


def moe_route_softmax(logits: torch.Tensor, experts: int, top: int, gated: bool) -> torch.Tensor:
    """logits fp32 [T, experts (+ 1 when gated)] -> weights of the same shape: softmax scores at the `top` experts with the
    largest scores (not renormalised), 0 at the others; gated: the last column is the sigmoid of its logit."""
    assert logits.dtype == torch.float32 and logits.is_contiguous() and logits.shape[1] == experts + (1 if gated else 0)
    _lib.require_device(logits)
    w = torch.empty_like(logits)
    _lib.check(_lib.lib().sllm_moe_route_softmax(logits.data_ptr(), w.data_ptr(), logits.shape[0], experts, top, 1 if gated else 0,
                                                 _lib.stream()), "moe_route_softmax")
    return w
