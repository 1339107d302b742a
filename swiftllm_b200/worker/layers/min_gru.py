"""Recurrent mixer whose gates read only the current token (minGRU): ONE input GEMM with bias [z ; x ; g] -> the scan (sigmoid
gate, candidate, state update S <- (1 - z) S + z c, SiLU output gate: one kernel, fp32 state per sequence) -> o GEMM."""
import torch

from swiftllm_b200.worker.kernels.linear import linear
from swiftllm_b200.worker.kernels.scan_ops import mingru_scan


class MinGruMixer:
    def __init__(self, spec, weight, run_id: int):
        self.spec, self.weight = spec, weight
        self.state_name = f"r{run_id}.mingru"

    def register(self, model):
        pass

    def state_layout(self) -> dict:
        return {self.state_name: ((self.spec.width,), torch.float32)}

    def forward(self, h: torch.Tensor, caches, block_table, states, st) -> torch.Tensor:
        w, C = self.weight, self.spec.width
        proj = torch.nn.functional.linear(h, w.in_proj, w.in_bias)          # [T, z (C) | x (C) | g (C)]
        if st.ignore_kvcache:
            return linear(proj[:, :C], w.o)
        return linear(mingru_scan(proj, states[self.state_name], st, C), w.o)
