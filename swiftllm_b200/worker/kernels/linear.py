"""Reference: swiftllm/worker/kernels/linear.py:3-12.  A plain library GEMM (cuBLAS through torch), exactly as in
the reference; the hot-path scope keeps it a library call."""
import torch


def linear(
    a: torch.Tensor,  # [a, b] (row-strided allowed)
    w: torch.Tensor   # [c, b]
) -> torch.Tensor:    # [a, c]
    return torch.nn.functional.linear(a, w)


def linear_f32_out(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """a [n, k] (row-strided allowed), w [m, k] in a's dtype -> a w^T as fp32 [n, m]: the library GEMM's fp32 accumulator is
    written out unrounded (inputs that feed a recurrence's step size or decay)."""
    if a.dtype == torch.float32:
        return torch.nn.functional.linear(a, w)
    return torch.mm(a, w.t(), out_dtype=torch.float32)
