"""Linear attention with a constant decay per head and per-sequence state: q, k, v = silu(projection); S <- decay_h S + k v^T,
out = S^T q (one kernel that walks each sequence's rows of the step and carries S in the sequence's state row, fp32); the heads'
outputs are RMS-normed together, gated by sigmoid(projection g) and scaled (one kernel).  `attend` is the part between the
input and output GEMMs."""
import torch

from swiftllm_b200.worker.kernels.recurrent import gated_rmsnorm, linear_attention


class DecayedLinearAttention:
    def __init__(self, spec, weight, eps: float, state_name: str):
        self.spec, self.weight, self.eps, self.state_name = spec, weight, eps, state_name

    @property
    def proj_widths(self):
        m = self.spec
        return [m.heads * m.dim, m.heads * m.dim, m.heads * m.vdim, m.heads * m.vdim]          # q, k, v, gate

    def state_layout(self) -> dict:
        m = self.spec
        return {self.state_name: ((m.heads, m.dim, m.vdim), torch.float32)}

    def attend(self, q, k, v, gate, out, states, st):
        m, w = self.spec, self.weight
        if st.ignore_kvcache:
            out.zero_()
            return
        o = linear_attention(q, k, v, w.decay, states[self.state_name], st, m.heads, m.dim, m.vdim)
        gated_rmsnorm(o, w.lin_norm, gate, self.eps, out, m.out_scale)
