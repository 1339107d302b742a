"""Recurrent mixer: a real-gated linear recurrent unit behind a short causal convolution, times a GELU branch.
ONE input GEMM with bias [y ; x] -> causal convolution of x over the sequence (its last taps - 1 inputs are per-sequence state)
-> ONE batched GEMM for the two block-diagonal gate projections -> the scan (gates, decay, state update, GELU branch and the
convolution's state: one kernel, fp32) -> o GEMM."""
import torch

from swiftllm_b200.worker.kernels.linear import linear
from swiftllm_b200.worker.kernels.recurrent import causal_conv, rglru_scan


class GatedRecurrenceMixer:
    def __init__(self, spec, weight, layer_id: int):
        self.spec, self.weight = spec, weight
        self.state_name, self.tail_name = f"l{layer_id}.recurrence", f"l{layer_id}.conv_tail"

    def register(self, model):
        pass

    def state_layout(self) -> dict:
        m = self.spec
        return {self.state_name: ((m.width,), torch.float32), self.tail_name: ((m.conv - 1, m.width), self.weight.dtype)}

    def forward(self, h: torch.Tensor, caches, block_table, states, st) -> torch.Tensor:
        m, w = self.spec, self.weight
        T, C = h.shape[0], m.width
        proj = torch.nn.functional.linear(h, w.in_proj, w.in_bias)          # [T, y (C) | x (C)]
        if st.ignore_kvcache:
            return linear(proj[:, :C], w.o)
        ybr, xin = proj[:, :C], proj[:, C:]
        tail = states[self.tail_name]
        u = causal_conv(xin, w.conv, w.conv_b, tail, st)
        ub = u.view(T, m.blocks, C // m.blocks).transpose(0, 1)              # [blocks, T, C / blocks] (strided)
        gates = torch.baddbmm(w.gate_b, ub, w.gate_w)                         # [blocks, T, 2 C / blocks]
        y = rglru_scan(u, gates, ybr, w.rate, xin, states[self.state_name], tail, st)
        return linear(y, w.o)
