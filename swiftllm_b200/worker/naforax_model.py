"""NaforaxModel - worker of the Naforax design: SEQUENTIAL sandwich blocks on an fp32 residual stream (a group RMS norm before
and after every sublayer, a short causal convolution on every sublayer's input), of which a range runs several times in a row
with the same weights (the embedding output and a per-pass vector are added before each pass; every pass has its own cache rows
and state); mixers are differential attention over the paged cache (two score maps per head, chunked causal mask), a minGRU
recurrence or a selective state-space scan; feed-forwards are a GELU gated linear unit or a mixture of clamped-GLU experts with
softmax-score routing and a gated shared expert; the logits are tanh-capped.

The public surface, the paged cache, the per-sequence state rows, the step's metadata and the CUDA-graph decode path are the
shared token-batch worker's (worker/token_model.py).  Per sequence this design keeps, besides the attention runs' cache rows:
every run's input-convolution tails, recurrence states and the scan's convolution tail."""
from __future__ import annotations

import torch

from swiftllm_b200.model_config import NaforaxModelConfig
from swiftllm_b200.worker.kernels.linear import linear
from swiftllm_b200.worker.kernels.sandwich_ops import group_norm_add_norm, group_norm_cast, stream_add
from swiftllm_b200.worker.kernels.stream_ops import embed_pair_hash, tanh_cap_inplace
from swiftllm_b200.worker.weight import load_naforax_weights

from .infer_state import TokenInferState
from .layers.sandwich_block import SandwichBlockLayer
from .token_model import TokenBatchModel


class NaforaxModel(TokenBatchModel):
    NATIVE_SOURCES = TokenBatchModel.NATIVE_SOURCES + ("parallel_block.cu", "stream_ops.cu", "sandwich_ops.cu", "scan_ops.cu",
                                                       "window_attn.cu")
    CONFIG_CLASS = NaforaxModelConfig

    @staticmethod
    def _load_weights(model_config, dtype, model_path, use_dummy, getter, device):
        return load_naforax_weights(model_config, dtype, model_path, use_dummy, getter=getter, device=device)

    def _build_layers(self) -> list:
        """One block object per RUN, in running order."""
        mc = self.model_config
        layers = [SandwichBlockLayer(mc, self.weight.layers[i], i, r) for r, (i, _) in enumerate(mc.runs)]
        for layer in layers:
            layer.mixer.register(self)
        return layers

    def _state_layout(self) -> dict:
        layout = {}
        for layer in self.layers:
            layout.update(layer.state_layout())
        return layout

    @torch.inference_mode()
    def _forward(self, input_ids: torch.Tensor, st: TokenInferState) -> torch.Tensor:
        """-> fp32 logits of st.output_rows."""
        mc, w = self.model_config, self.weight
        loop = mc.loop
        again = loop is not None and loop[2] > 1
        x0 = torch.empty((input_ids.shape[0], mc.hidden_size), dtype=torch.float32, device=self.device) if again else None
        x, _ = embed_pair_hash(input_ids, st, None, w.wte, None, 0, 0, 0, x_copy=x0)
        self._wait_for_swaps()
        block_table = None if st.ignore_kvcache else self.gpu_block_manager.block_table
        keep = [] if self.keep_residuals else None
        eps, groups = mc.rms_norm_eps, mc.norm_groups

        def starts_pass(r):
            return loop is not None and r < len(mc.runs) and mc.runs[r][0] == loop[0]
        n = None
        for r, layer in enumerate(self.layers):
            if starts_pass(r):
                t = mc.runs[r][1]
                stream_add(x, x0 if t > 0 else None, w.loop_step[t])
                n = None
            if n is None:
                n = group_norm_add_norm(x, None, None, 1.0, layer.weight.norm1, eps, groups)
            nxt = None if r + 1 == len(self.layers) or starts_pass(r + 1) else self.layers[r + 1].weight.norm1
            n = layer.forward(x, n, self.caches, block_table, self.seq_states, st, nxt)
            if keep is not None:
                keep.append(x.clone())
        self.last_residuals = keep
        rows = x.index_select(0, st.output_rows)
        logits = linear(group_norm_cast(rows, w.final_norm, eps, groups, self.dtype), w.lm_head).float()
        if mc.logit_softcap > 0:
            tanh_cap_inplace(logits, mc.logit_softcap)
        return logits
