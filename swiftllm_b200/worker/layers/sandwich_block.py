"""A sequential decoder block with a norm before AND after each sublayer, x <- x + m * norm_b(sublayer(c(norm_a(x)))), where the
norms are RMS norms over equal consecutive groups of the row and c(h) = h + causal per-channel convolution of h over time (its
last taps - 1 inputs are per-sequence state of every run of the block, for both sublayers).  The fp32 stream `x` is updated in
place.  The kernel that adds a sublayer's normed output also computes the NEXT norm of the updated stream (the same groups), so
`forward` takes its first norm's result and returns the first norm of the block that follows."""
import torch

from swiftllm_b200.model_config import MinGruSpec, SelectiveScanSpec
from swiftllm_b200.worker.kernels.sandwich_ops import group_norm_add_norm
from swiftllm_b200.worker.kernels.scan_ops import short_conv
from swiftllm_b200.worker.layers.feed_forward import build_feed_forward
from swiftllm_b200.worker.layers.min_gru import MinGruMixer
from swiftllm_b200.worker.layers.selective_scan import SelectiveScanMixer
from swiftllm_b200.worker.layers.window_attention import DifferentialAttentionMixer


class SandwichBlockLayer:
    def __init__(self, model_config, weight, layer_id: int, run_id: int):
        """run_id: the block's place in the running order (a layer that runs several times has one object, one set of cache rows
        and one set of state tensors per run, and shares its weights)."""
        mc = model_config
        self.layer_id, self.run_id, self.weight = layer_id, run_id, weight
        self.eps, self.groups, self.mult, self.taps = mc.rms_norm_eps, mc.norm_groups, mc.residual_mult, mc.canon_taps
        self.width = mc.hidden_size
        spec = mc.mixers[layer_id]
        if isinstance(spec, MinGruSpec):
            self.mixer = MinGruMixer(spec, weight, run_id)
        elif isinstance(spec, SelectiveScanSpec):
            self.mixer = SelectiveScanMixer(spec, weight, run_id)
        else:
            self.mixer = DifferentialAttentionMixer(spec, weight, self.eps, mc.cache_slot[run_id])
        self.ff = build_feed_forward(mc.ffs[layer_id], weight)
        self.tail_names = (f"r{run_id}.canon1", f"r{run_id}.canon2")

    def state_layout(self) -> dict:
        out = dict(self.mixer.state_layout())
        if self.taps > 1:
            for name in self.tail_names[:1 if self.ff is None else 2]:
                out[name] = ((self.taps - 1, self.width), torch.float32)
        return out

    def _sublayer_input(self, n: torch.Tensor, taps_w: torch.Tensor, tail_name: str, states, st, dtype) -> torch.Tensor:
        """n + conv(n) in the projections' dtype; the sequence's tail moves on."""
        if st.ignore_kvcache:
            return n.to(dtype)
        tail = states[tail_name] if self.taps > 1 else None
        return short_conv(n, taps_w, None, tail, st, dtype, add_input=True, move_tail=True)

    def forward(self, x, n, caches, block_table, states, st, next_norm=None):
        """x fp32 [T, W] (in place); n = norm1(x) fp32; next_norm: weight of the norm that reads the result (or None).
        -> that norm of the result, or None."""
        w, dtype = self.weight, self.weight.dtype
        h = self._sublayer_input(n, w.canon1, self.tail_names[0], states, st, dtype)
        y = self.mixer.forward(h, caches, block_table, states, st)
        if self.ff is None:
            return group_norm_add_norm(x, y, w.norm1b, self.mult, next_norm, self.eps, self.groups)
        n = group_norm_add_norm(x, y, w.norm1b, self.mult, w.norm2, self.eps, self.groups)
        h = self._sublayer_input(n, w.canon2, self.tail_names[1], states, st, dtype)
        y = self.ff.forward(h)
        return group_norm_add_norm(x, y, w.norm2b, self.mult, next_norm, self.eps, self.groups)
