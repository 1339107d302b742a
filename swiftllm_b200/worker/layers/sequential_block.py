"""A sequential decoder block whose sublayers read the residual stream itself and whose OUTPUTS are normalised before they are
added: x <- x + g1 * rms(mixer(x)), then x <- x + g2 * rms(ff(x)) (scalar gains).  The block returns nothing: it updates the
fp32 stream `x` and its rounding `h` (what the projections read) in place; the second update also applies the weighted sum over
the results of all earlier layers when the design has one (worker/kernels/stream_ops.py)."""
from swiftllm_b200.model_config import GatedRecurrenceSpec, ParallelMixerSpec
from swiftllm_b200.worker.kernels.stream_ops import postnorm_add_mix
from swiftllm_b200.worker.layers.feed_forward import build_feed_forward
from swiftllm_b200.worker.layers.gated_recurrence import GatedRecurrenceMixer
from swiftllm_b200.worker.layers.parallel_mixer import ParallelMixer


class PostNormBlockLayer:
    def __init__(self, model_config, weight, layer_id: int):
        self.layer_id, self.weight, self.eps = layer_id, weight, model_config.rms_norm_eps
        spec = model_config.mixers[layer_id]
        if isinstance(spec, GatedRecurrenceSpec):
            self.mixer = GatedRecurrenceMixer(spec, weight, layer_id)
        else:
            assert isinstance(spec, ParallelMixerSpec)
            self.mixer = ParallelMixer(spec, weight, self.eps, model_config.cache_slot[layer_id], layer_id)
        self.ff = build_feed_forward(model_config.ffs[layer_id], weight)

    def forward(self, x, h, caches, block_table, states, st, history=None):
        """x fp32 [T, W] and h (its rounding) are updated in place; history fp32 [layers + 1, T, W] or None."""
        w, i = self.weight, self.layer_id
        mix = w.dwa if history is not None else None
        y = self.mixer.forward(h, caches, block_table, states, st)
        if self.ff is None:
            postnorm_add_mix(x, y, w.norm1, self.eps, h, history, i + 1, mix)
            return
        postnorm_add_mix(x, y, w.norm1, self.eps, h)
        y = self.ff.forward(h, x)
        postnorm_add_mix(x, y, w.norm2, self.eps, h, history, i + 1, mix)
