"""Two mixers side by side on the same input, summed with fixed weights: softmax attention over the paged cache
(worker/layers/window_attention.py) and decayed linear attention with per-sequence state (worker/layers/linear_attention.py).
ONE input GEMM feeds both ([left q ; k ; v ; right q ; k ; v ; g]); both write their (already weighted) outputs into one matrix
[left | right] and ONE output GEMM over [left.o | right.o] adds them."""
import torch

from swiftllm_b200.worker.kernels.linear import linear
from swiftllm_b200.worker.layers.linear_attention import DecayedLinearAttention
from swiftllm_b200.worker.layers.window_attention import WindowAttentionMixer


class ParallelMixer:
    def __init__(self, spec, weight, eps: float, cache_key, layer_id: int):
        self.spec, self.weight = spec, weight
        self.left = WindowAttentionMixer(spec.left, weight, eps, cache_key)
        self.right = DecayedLinearAttention(spec.right, weight, eps, f"l{layer_id}.linear_attention")
        assert not spec.left.gate
        self.widths = self.left.proj_widths + self.right.proj_widths

    def register(self, model):
        self.left.register(model)

    def state_layout(self) -> dict:
        return self.right.state_layout()

    def forward(self, h: torch.Tensor, caches, block_table, states, st) -> torch.Tensor:
        a, b = self.spec.left, self.spec.right
        q, k, v, rq, rk, rv, rg = torch.split(linear(h, self.weight.in_proj), self.widths, dim=1)
        nl = a.heads * a.vdim
        out = torch.empty((h.shape[0], nl + b.heads * b.vdim), dtype=h.dtype, device=h.device)
        self.left.attend(q, k, v, None, out[:, :nl], caches, block_table, st)
        self.right.attend(rq, rk, rv, rg, out[:, nl:], states, st)
        return linear(out, self.weight.o)
