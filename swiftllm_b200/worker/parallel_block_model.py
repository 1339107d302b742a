"""ParallelBlockModel - worker of designs made of PARALLEL decoder blocks (one RMS norm feeds a mixer and a feed-forward whose
outputs are both added to an fp32 residual stream).  The public surface, the cache, the step's metadata and the CUDA-graph
decode path are the shared token-batch worker's (worker/token_model.py); here are the topology and its layers.  A design
subclasses it with its configuration class, its weight loader and the CUDA sources of its kernels (worker/bupozen_model.py:
latent attention + squared-ReLU feed-forwards; worker/rivudra_model.py: gated sliding-window attention with grouped key/value
heads + clamped gated-linear-unit experts); which mixer and which feed-forward a layer gets is decided per layer from the
configuration (worker/layers/parallel_block.py), so a design may mix them.

What a cache block holds per token: ONE row for every layer that caches (latent attention: [latent | rotated key part], and
layers with `kv_from` read the row of the layer they name; window attention: [rotated keys | values] of all key/value heads)."""
from __future__ import annotations

import torch

from swiftllm_b200.worker.kernels.linear import linear
from swiftllm_b200.worker.kernels.parallel_block import add_rmsnorm_f32

from .infer_state import TokenInferState
from .layers.parallel_block import ParallelBlockLayer
from .token_model import TokenBatchModel


class ParallelBlockModel(TokenBatchModel):
    # CUDA sources this worker's kernels live in (build(only=...) compiles just these in a fresh checkout)
    NATIVE_SOURCES = TokenBatchModel.NATIVE_SOURCES + ("parallel_block.cu",)

    def _build_layers(self) -> list:
        for m in self.model_config.mixers:
            self._register_rotary((m.rot_base, m.rot_dims), m.rot_base, m.rot_dims)
        return [ParallelBlockLayer(self.model_config, self.weight.layers[i], i) for i in range(self.model_config.num_layers)]

    @torch.inference_mode()
    def _forward(self, input_ids: torch.Tensor, st: TokenInferState) -> torch.Tensor:
        """-> logits (engine dtype) of st.output_rows."""
        mc, w = self.model_config, self.weight
        x = torch.embedding(w.wte, input_ids, padding_idx=-1).float()        # the fp32 residual stream
        if mc.embedding_scale != 1.0:
            x.mul_(mc.embedding_scale)
        self._wait_for_swaps()
        block_table = None if st.ignore_kvcache else self.gpu_block_manager.block_table
        keep = [] if self.keep_residuals else None
        h = add_rmsnorm_f32(x, None, None, w.layers[0].norm if self.layers else w.final_norm, mc.rms_norm_eps, out_dtype=self.dtype)
        for i, layer in enumerate(self.layers):
            y_mix, y_ff = layer.forward(h, self.caches, block_table, st)
            next_norm = w.layers[i + 1].norm if i + 1 < len(self.layers) else w.final_norm
            h = add_rmsnorm_f32(x, y_mix, y_ff, next_norm, mc.rms_norm_eps, out=h)
            if keep is not None:
                keep.append(x.clone())
        self.last_residuals = keep
        return linear(h.index_select(0, st.output_rows), w.lm_head)
