"""Feed-forward sublayers: dense and mixture-of-experts with the squared-ReLU activation, a dense clamped gated linear unit, a
dense GELU gated linear unit, a mixture of clamped gated-linear-unit experts (group-limited routing with renormalised scores, or
the plain softmax scores of the largest experts) with a shared expert that may have a per-token sigmoid weight, and a mixture of
SiLU-gated experts routed by sigmoid scores with a bias that only takes part in the choice.

Every forward takes the sublayer's input `h` in the storage dtype and, optionally, the same input in fp32 (`x32`: designs whose
sublayers read an fp32 stream hand it to the router, which then sees no rounding).

Mixture of experts.  Router logits are an fp32 GEMM; `moe_route` turns them into a [T, experts] weight matrix (softmax over the
`top` largest logits at their experts, exact zeros elsewhere).  The experts' up projections are ONE GEMM over the row-wise
concatenation of their weights, the activation kernel multiplies every expert's slice by the token's weight for that expert,
and ONE down GEMM over the column-wise concatenation then sums the chosen experts' weighted outputs.  No token permutation,
no host sync, fixed shapes (CUDA-graph friendly); the price is experts / top times the FLOPs of a gathered formulation, which
only matters once the step is compute-bound (a decode step streams every expert's weights anyway as soon as
tokens * top >= experts)."""
import torch

from swiftllm_b200.worker.kernels.linear import linear
from swiftllm_b200.worker.kernels.parallel_block import (moe_clamped_glu_scale, moe_relu2_scale_inplace, moe_route,
                                                         moe_route_grouped, relu2_inplace)
from swiftllm_b200.worker.kernels.sandwich_ops import gelu_glu, moe_route_softmax
from swiftllm_b200.worker.kernels.stream_ops import moe_route_sigmoid, moe_silu_glu_scale

GLU_SIGMOID_SLOPE = 1.702       # the gate's activation is g * sigmoid(1.702 g)
ROUTE_NORM_EPS = 1e-20          # added to the sum of the chosen scores before dividing by it


class Relu2FeedForward:
    def __init__(self, spec, weight):
        self.spec, self.weight = spec, weight

    def forward(self, h: torch.Tensor, x32=None) -> torch.Tensor:
        u = linear(h, self.weight.up)
        relu2_inplace(u)
        return linear(u, self.weight.down)


class Relu2MixtureOfExperts:
    def __init__(self, spec, weight):
        self.spec, self.weight = spec, weight

    def forward(self, h: torch.Tensor, x32=None) -> torch.Tensor:
        w = self.weight
        logits = linear(h.float() if x32 is None else x32, w.router)   # fp32 GEMM (TF32 stays off)
        weights = moe_route(logits, self.spec.top)
        u = linear(h, w.up)                                     # [T, experts * ff]
        moe_relu2_scale_inplace(u, weights, self.spec.ff)
        return linear(u, w.down)


class ClampedGluMixtureOfExperts:
    """Experts y = min(gate, limit) * sigmoid(1.702 .) * (clamp(up, +-limit) + 1) -> down.  Same dense formulation as above:
    ONE [gate | up] GEMM over all experts AND the shared expert (its rows come last), the activation kernel applies the routing
    weight (1 for the shared expert), ONE down GEMM sums everything.  Routing "softmax_grouped": softmax over all experts,
    group-limited top-k, chosen scores renormalised and scaled (fp32).  Routing "softmax_top": softmax over all experts, the
    `top` largest scores as they are; with `shared_gated` the router GEMM has one more row, whose sigmoid weighs the shared expert."""

    def __init__(self, spec, weight):
        self.spec, self.weight = spec, weight

    def forward(self, h: torch.Tensor, x32=None) -> torch.Tensor:
        f, w = self.spec, self.weight
        logits = linear(h.float() if x32 is None else x32, w.router)   # fp32 GEMM (TF32 stays off)
        if f.routing == "softmax_top":
            weights = moe_route_softmax(logits, f.experts, f.top, f.shared_gated)
        else:
            weights = moe_route_grouped(logits, f.top, f.groups, f.keep, f.route_scale, ROUTE_NORM_EPS)
        u = linear(h, w.up)                                     # [T, 2 * (experts * ff + shared_ff)]
        y = moe_clamped_glu_scale(u, weights, f.experts, f.ff, f.limit, f.shared_ff, f.shared_limit, GLU_SIGMOID_SLOPE,
                                  shared_gated=f.shared_gated)
        return linear(y, w.down)


class ClampedGluFeedForward:
    """Dense y = min(gate, limit) * sigmoid(1.702 .) * (clamp(up, +-limit) + 1) -> down: ONE [gate | up] GEMM, the activation
    kernel of the clamped-GLU experts with no routed expert (the dense layer takes the place of the shared one), ONE down GEMM."""

    def __init__(self, spec, weight):
        self.spec, self.weight = spec, weight

    def forward(self, h: torch.Tensor, x32=None) -> torch.Tensor:
        f = self.spec
        u = linear(h, self.weight.up)                           # [T, gate (ff) | up (ff)]
        y = moe_clamped_glu_scale(u, None, 0, 0, 0.0, f.ff, f.limit, GLU_SIGMOID_SLOPE)
        return linear(y, self.weight.down)


class GeluGluFeedForward:
    """Dense gelu_tanh(gate) * up -> down: ONE [gate | up] GEMM, the activation kernel, ONE down GEMM."""

    def __init__(self, spec, weight):
        self.spec, self.weight = spec, weight

    def forward(self, h: torch.Tensor, x32=None) -> torch.Tensor:
        return linear(gelu_glu(linear(h, self.weight.up)), self.weight.down)


class SiluGluMixtureOfExperts:
    """Experts y = silu(gate) * up -> down, no biases.  Routing: scores are sigmoids of fp32 router logits; the `top` experts with
    the largest score + correction are chosen and weighted by their plain scores (not renormalised).  Dense formulation as above:
    ONE [gate | up] GEMM over all experts, the activation kernel applies the routing weight (exact zeros for the others), ONE
    down GEMM sums the chosen experts."""

    def __init__(self, spec, weight):
        self.spec, self.weight = spec, weight

    def forward(self, h: torch.Tensor, x32=None) -> torch.Tensor:
        f, w = self.spec, self.weight
        logits = linear(h.float() if x32 is None else x32, w.router)   # fp32 GEMM (TF32 stays off)
        weights = moe_route_sigmoid(logits, w.correction, f.top)
        u = linear(h, w.up)                                     # [T, experts * 2 * ff]
        y = moe_silu_glu_scale(u, weights, f.experts, f.ff)
        return linear(y, w.down)


def build_feed_forward(spec, weight):
    if spec is None:
        return None
    if spec.activation == "silu_glu":
        assert spec.kind == "moe" and spec.routing == "sigmoid_bias"
        return SiluGluMixtureOfExperts(spec, weight)
    if spec.activation == "gelu_glu":
        assert spec.kind == "dense"
        return GeluGluFeedForward(spec, weight)
    if spec.activation == "clamped_glu" and spec.kind == "dense":
        return ClampedGluFeedForward(spec, weight)
    if spec.activation == "clamped_glu":
        assert spec.kind == "moe" and spec.routing in ("softmax_grouped", "softmax_top")
        return ClampedGluMixtureOfExperts(spec, weight)
    return (Relu2FeedForward if spec.kind == "dense" else Relu2MixtureOfExperts)(spec, weight)
