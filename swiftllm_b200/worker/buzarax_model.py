"""BuzaraxModel - worker of the Buzarax design: SEQUENTIAL blocks on an fp32 residual stream whose sublayers read the stream
itself and whose outputs are RMS-normed (one scalar gain) before they are added; mixers are either softmax attention beside
decayed linear attention (worker/layers/parallel_mixer.py) or a gated linear recurrence behind a causal convolution
(worker/layers/gated_recurrence.py); feed-forwards are a clamped gated linear unit or a mixture of SiLU-gated experts with
sigmoid routing; the embedding adds a hashed table of token pairs; after every layer the stream becomes a learned weighted sum
of the embedding output and all layers' results; the logits are tanh-capped.

The public surface, the paged cache, the per-sequence state rows, the step's metadata and the CUDA-graph decode path are the
shared token-batch worker's (worker/token_model.py).  Per sequence this design keeps, besides the attention layers' cache rows:
the previous token, every recurrence's state and convolution tail, every linear attention's state."""
from __future__ import annotations

import torch

from swiftllm_b200.model_config import BuzaraxModelConfig
from swiftllm_b200.worker.kernels.linear import linear
from swiftllm_b200.worker.kernels.parallel_block import add_rmsnorm_f32
from swiftllm_b200.worker.kernels.stream_ops import embed_pair_hash, tanh_cap_inplace
from swiftllm_b200.worker.weight import load_buzarax_weights

from .infer_state import TokenInferState
from .layers.sequential_block import PostNormBlockLayer
from .token_model import TokenBatchModel

LAST_TOKEN = "last_token"


class BuzaraxModel(TokenBatchModel):
    NATIVE_SOURCES = TokenBatchModel.NATIVE_SOURCES + ("parallel_block.cu", "stream_ops.cu", "recurrent.cu", "window_attn.cu")
    CONFIG_CLASS = BuzaraxModelConfig

    @staticmethod
    def _load_weights(model_config, dtype, model_path, use_dummy, getter, device):
        return load_buzarax_weights(model_config, dtype, model_path, use_dummy, getter=getter, device=device)

    def _build_layers(self) -> list:
        layers = [PostNormBlockLayer(self.model_config, self.weight.layers[i], i) for i in range(self.model_config.num_layers)]
        for layer in layers:
            layer.mixer.register(self)
        return layers

    def _state_layout(self) -> dict:
        layout = {}
        if self.model_config.pair_hash is not None:
            layout[LAST_TOKEN] = ((), torch.int32)
        for layer in self.layers:
            layout.update(layer.mixer.state_layout())
        return layout

    @torch.inference_mode()
    def _forward(self, input_ids: torch.Tensor, st: TokenInferState) -> torch.Tensor:
        """-> fp32 logits of st.output_rows."""
        mc, w = self.model_config, self.weight
        T, L = input_ids.shape[0], len(self.layers)
        # the results of all layers (slot 0: the embedding output) for the weighted sums over depth
        history = torch.empty((L + 1, T, mc.hidden_size), dtype=torch.float32, device=self.device)
        pair, states = mc.pair_hash, self.seq_states
        if pair is not None and not st.ignore_kvcache:
            x, h = embed_pair_hash(input_ids, st, states[LAST_TOKEN], w.wte, w.pairs, pair.buckets, pair.mul_prev, pair.mul_cur,
                                   x_copy=history[0])
        else:
            x, h = embed_pair_hash(input_ids, st, None, w.wte, None, 0, 0, 0, x_copy=history[0])
        self._wait_for_swaps()
        block_table = None if st.ignore_kvcache else self.gpu_block_manager.block_table
        keep = [] if self.keep_residuals else None
        for layer in self.layers:
            layer.forward(x, h, self.caches, block_table, states, st, history)
            if keep is not None:
                keep.append(x.clone())
        self.last_residuals = keep
        rows = x.index_select(0, st.output_rows)
        hn = add_rmsnorm_f32(rows, None, None, w.final_norm, mc.rms_norm_eps, out_dtype=self.dtype)
        logits = linear(hn, w.lm_head).float()
        if mc.logit_softcap > 0:
            tanh_cap_inplace(logits, mc.logit_softcap)
        return logits
