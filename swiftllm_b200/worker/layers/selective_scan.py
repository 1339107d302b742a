"""Selective state-space mixer: in GEMM [x ; z] -> causal convolution of x with bias and SiLU (its last taps - 1 inputs are
per-sequence state) -> GEMM [dt ; B ; C] -> step-size GEMM with an fp32 result -> the scan (softplus, decay exp(dt A), state
update, read-out, D skip, SiLU gate of z: one kernel, fp32 state [inner, state] per sequence) -> o GEMM."""
import torch

from swiftllm_b200.worker.kernels.linear import linear, linear_f32_out
from swiftllm_b200.worker.kernels.scan_ops import selective_scan, short_conv


class SelectiveScanMixer:
    def __init__(self, spec, weight, run_id: int):
        self.spec, self.weight = spec, weight
        self.state_name, self.tail_name = f"r{run_id}.ssm", f"r{run_id}.ssm_conv_tail"

    def register(self, model):
        pass

    def state_layout(self) -> dict:
        m = self.spec
        out = {self.state_name: ((m.inner, m.state), torch.float32)}
        if m.conv > 1:
            out[self.tail_name] = ((m.conv - 1, m.inner), self.weight.dtype)
        return out

    def forward(self, h: torch.Tensor, caches, block_table, states, st) -> torch.Tensor:
        m, w = self.spec, self.weight
        C, N, R = m.inner, m.state, m.dt_rank
        xz = linear(h, w.in_proj)                                           # [T, x (C) | z (C)]
        if st.ignore_kvcache:
            return linear(xz[:, :C], w.o)
        xin, z = xz[:, :C], xz[:, C:]
        tail = states[self.tail_name] if m.conv > 1 else None
        x = short_conv(xin, w.conv, w.conv_b, tail, st, h.dtype, silu=True, move_tail=True)
        proj = linear(x, w.x_proj)                                          # [T, dt (R) | B (N) | C (N)]
        dt = linear_f32_out(proj[:, :R], w.dt_proj)                         # step logits, fp32 [T, C]
        y = selective_scan(x, dt, w.dt_bias, w.A, proj, R, R + N, w.D, z, states[self.state_name], st)
        return linear(y, w.o)
