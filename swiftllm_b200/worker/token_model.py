"""TokenBatchModel - what every worker shares whose kernels treat each token of a step as a row with its own (sequence row,
position): the public surface of `LlamaModel` (worker/model.py), the paged cache tensors and their block manager, per-sequence
recurrent state (worker/state_manager.py), the step's metadata and angle tables, and the CUDA-graph replay of pure-decode steps.
A topology subclasses it (worker/parallel_block_model.py: parallel blocks; worker/buzarax_model.py: sequential blocks whose
sublayer outputs are normalised, with recurrent mixers; worker/naforax_model.py: sequential blocks with norms on both sides of
every sublayer, of which a range of layers runs several times) and provides `_load_weights`, `_build_layers` and `_forward`.

    Model(engine_config[, model_config]) -> load_weights() -> profile_num_blocks() -> init_kvcache_and_swap(num_blocks)
    forward(input_ids_list, seq_ids_list, decoding_seq_lens_list, ignore_kvcache=False, prefill_prefix_lens_list=None,
            logit_rows=None) -> list[int]                      (greedy token after the last row of every sequence)
    free_seqs_resources(seq_ids_list)

Batch layout: prompt portions first (portion i starts at position prefill_prefix_lens_list[i] of its sequence; earlier
positions are in the cache and in the sequence's state), then one token per decoding sequence (decoding_seq_lens_list[i]
includes it).  Blocks come from the same `BlockManager` as the Llama worker's; what a block holds differs: per token ONE row for
every layer that caches.  Rows of different widths live in different cache tensors that share the block table.  State that does
not grow with the sequence (a recurrence's state, a convolution's last inputs, the previous token) lives in tensors with one
row per block-table row.

Precision: the residual stream, norms, softmax, rotary angles, routers and recurrent state are fp32 for every engine dtype;
projections and the cache are in the engine dtype (float16 / bfloat16 / float32 - with float32 everything is true fp32, TF32
off)."""
from __future__ import annotations

import itertools
import math
from typing import Callable, Optional

import torch

from swiftllm_b200.engine_config import EngineConfig
from swiftllm_b200.utils import GB
from swiftllm_b200.worker.block_manager import BlockManager
from swiftllm_b200.worker.state_manager import SequenceStateManager

from .infer_state import TokenInferState
from .model_base import PagedModelBase

_DTYPES = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}


def rotary_frequencies(base: float, dims: int, scaling: Optional[tuple] = None):
    """-> (frequency of every pair [dims / 2], factor on cos and sin).  Plain: base^(-2i/dims), factor 1.  With scaling =
    (factor, original context, fast, slow): the pair index at which a wavelength makes `turns` turns over the original context is
    d(turns) = dims ln(original / (2 pi turns)) / (2 ln base); pairs up to floor(d(fast)) keep their frequency, pairs from
    ceil(d(slow)) on are slowed by `factor`, linearly blended between; cos and sin are multiplied by 0.1 ln(factor) + 1."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if scaling is None:
        return f, 1.0
    factor, original, fast, slow = scaling

    def pair_at(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo, hi = max(math.floor(pair_at(fast)), 0), min(math.ceil(pair_at(slow)), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


class TokenBatchModel(PagedModelBase):
    # CUDA sources this worker's kernels live in (build(only=...) compiles just these in a fresh checkout)
    NATIVE_SOURCES = ("host.cu", "kvcache.cu")
    DTYPES = tuple(_DTYPES)
    CONFIG_CLASS = None         # the design's configuration class (model_config.py)

    @staticmethod
    def _load_weights(model_config, dtype, model_path, use_dummy, getter, device):
        """-> the design's weight object: wte, lm_head, final_norm, layers[i].norm + what its layers read."""
        raise NotImplementedError

    @torch.inference_mode()
    def __init__(self, engine_config: EngineConfig, model_config=None):
        self.engine_config = engine_config
        self.model_config = model_config if model_config is not None else \
            self.CONFIG_CLASS.load_from_model_path(engine_config.model_path)
        self.dtype = _DTYPES[getattr(engine_config, "dtype", "bfloat16")]
        assert getattr(engine_config, "tp_size", 1) == 1, "parallel-block workers are single-GPU (no tensor-parallel sharding yet)"
        self.tp_size, self.tp_rank = 1, 0
        self.device = torch.device("cuda", torch.cuda.current_device())
        if self.dtype == torch.float32:
            torch.backends.cuda.matmul.allow_tf32 = False       # "float32" means true fp32 products
            torch.backends.cudnn.allow_tf32 = False
        self.weight = None
        self.layers = None
        self.num_blocks = None
        self.caches = None              # row width -> [num_blocks, slots, block_size, width]
        self.k_cache = self.v_cache = None
        self.cpu_block_manager = self.gpu_block_manager = None
        self._rot = {}                  # angle-table key -> (fp64 frequencies on the device, factor on cos and sin)
        self.seq_states = None          # per-sequence state of recurrent mixers (SequenceStateManager), None when no layer has any
        self.last_logits = None         # fp32 logits of the rows named by forward(..., logit_rows=...)
        self.keep_residuals = False     # debugging / tests: keep the residual stream after every block of the last forward
        self.last_residuals = None
        self._graphs = {}               # decode batch size -> captured step (EngineConfig.use_cuda_graph)
        self._graph_pool = None
        self._init_staging()

    # ------------------------------------------------------------------ init
    @torch.inference_mode()
    def load_weights(self, weight_getter: Optional[Callable] = None):
        self.weight = self._load_weights(self.model_config, self.dtype, self.engine_config.model_path,
                                         self.engine_config.use_dummy, weight_getter, self.device)
        self.layers = self._build_layers()

    def _build_layers(self) -> list:
        """-> the layer objects (they call _register_rotary for the angle tables they read)."""
        raise NotImplementedError

    def _register_rotary(self, key, base: float, dims: int, scaling: Optional[tuple] = None):
        """Make TokenInferState.rotary[key] = (cos, sin) fp32 [num_tokens, dims / 2] available in every step."""
        if dims > 0 and key not in self._rot:
            # the frequencies are kept in fp64, a position's angles are rounded once
            f, amp = rotary_frequencies(base, dims, scaling)
            self._rot[key] = (torch.tensor(f, dtype=torch.float64).to(self.device), amp)

    def _state_layout(self) -> dict:
        """name -> (shape of one sequence's state, dtype): what the layers keep per sequence besides cache rows."""
        return {}

    def _kvslot_bytes(self) -> int:
        return self.model_config.get_kvslot_size(self.dtype)

    @torch.inference_mode()
    def profile_num_blocks(self) -> int:
        """Forged maximum-size prompt batch without a cache -> peak memory -> number of blocks that fit in what is left."""
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats()
        num_tokens, batch_size = self.engine_config.max_tokens_in_batch, self.engine_config.max_batch_size
        input_lens = [num_tokens // batch_size] * batch_size
        input_lens[-1] += num_tokens % batch_size
        self.forward([[0] * n for n in input_lens], list(range(batch_size)), [], ignore_kvcache=True)
        torch.cuda.synchronize()
        free_memory, total_memory = torch.cuda.mem_get_info()
        peak_memory = total_memory - free_memory
        useable_memory = total_memory * self.engine_config.gpu_mem_utilization
        if useable_memory < peak_memory:
            raise RuntimeError(f"Peak memory {peak_memory/GB:.2f} GB exceeds usable memory {useable_memory/GB:.2f} GB")
        # a model without caching layers (recurrent mixers only) still needs blocks for the positions' bookkeeping: count them
        # as one byte per token
        num_gpu_blocks = math.floor((useable_memory - peak_memory) / (self.engine_config.block_size * max(1, self._kvslot_bytes())))
        num_gpu_blocks = min(num_gpu_blocks, self.engine_config.max_seqs_in_block_table * self.engine_config.max_blocks_per_seq)
        torch.cuda.empty_cache()
        return num_gpu_blocks

    @torch.inference_mode()
    def init_kvcache_and_swap(self, num_blocks: int):
        ec, mc = self.engine_config, self.model_config
        self.num_blocks = num_blocks
        self.caches = {w: torch.zeros((num_blocks, n, ec.block_size, w), dtype=self.dtype, device=self.device)
                       for w, n in mc.cache_slots_per_width.items()}
        self.k_cache = next(iter(self.caches.values()), None)
        self.gpu_block_manager = BlockManager("GPU", num_blocks, ec.max_seqs_in_block_table, ec.max_blocks_per_seq,
                                              ec.block_size, device=self.device)
        # no swap space for these cache rows yet: the CPU manager exists (empty) so that the shared bookkeeping paths work
        self.cpu_block_manager = BlockManager("CPU", 0, ec.max_seqs_in_block_table, 1, ec.block_size, device=self.device)
        layout = self._state_layout()
        self.seq_states = SequenceStateManager(ec.max_seqs_in_block_table, layout, self.device) if layout else None
        self._graphs = {}

    def swap_in_seqs(self, seq_ids_list: list):
        raise NotImplementedError("parallel-block workers have no CPU swap space")

    swap_out_seqs = swap_in_seqs

    # ------------------------------------------------------------------ forward
    def _rotary_tables(self, positions: torch.Tensor) -> dict:
        p = positions.to(torch.float64)[:, None]
        out = {}
        for key, (inv, amp) in self._rot.items():
            ang = p * inv[None, :]
            out[key] = ((torch.cos(ang) * amp).float().contiguous(), (torch.sin(ang) * amp).float().contiguous())
        return out

    def _forward(self, input_ids: torch.Tensor, st: TokenInferState) -> torch.Tensor:
        """-> logits of st.output_rows."""
        raise NotImplementedError

    @torch.inference_mode()
    def forward(self, input_ids_list: list, seq_ids_list: list, decoding_seq_lens_list: list, ignore_kvcache: bool = False,
                prefill_prefix_lens_list: Optional[list] = None, logit_rows: Optional[list] = None) -> list:
        return self.forward_async(input_ids_list, seq_ids_list, decoding_seq_lens_list, ignore_kvcache,
                                  prefill_prefix_lens_list, logit_rows).tolist()

    @torch.inference_mode()
    def forward_async(self, input_ids_list, seq_ids_list, decoding_seq_lens_list, ignore_kvcache=False,
                      prefill_prefix_lens_list=None, logit_rows=None) -> torch.Tensor:
        """Greedy tokens on the device (no sync).  `logit_rows`: rows of the packed batch whose fp32 logits are kept in
        `self.last_logits` ([len(logit_rows), vocab], same order)."""
        num_prefill_seqs = len(input_ids_list) - len(decoding_seq_lens_list)
        prefill_lens = [len(s) for s in input_ids_list[:num_prefill_seqs]]
        assert all(len(s) == 1 for s in input_ids_list[num_prefill_seqs:]), "decoding sequences bring exactly one token"
        prefix_lens = [int(v) for v in prefill_prefix_lens_list] if prefill_prefix_lens_list is not None else [0] * num_prefill_seqs
        assert len(prefix_lens) == num_prefill_seqs and min(prefix_lens, default=0) >= 0
        flat_ids = list(itertools.chain(*input_ids_list))
        batch_size, num_tokens = len(input_ids_list), len(flat_ids)
        if (getattr(self.engine_config, "use_cuda_graph", False) and num_prefill_seqs == 0 and batch_size > 0
                and not ignore_kvcache and not logit_rows and not self.keep_residuals):
            return self._forward_decode_graph(flat_ids, list(seq_ids_list), list(decoding_seq_lens_list))
        num_prefill_tokens = sum(prefill_lens)
        seq_lengths_list = [p + n for p, n in zip(prefix_lens, prefill_lens)] + list(decoding_seq_lens_list)
        tok_seq = [s for s, n in zip(seq_ids_list, prefill_lens) for _ in range(n)] + list(seq_ids_list[num_prefill_seqs:])
        tok_pos = [p0 + p for p0, n in zip(prefix_lens, prefill_lens) for p in range(n)] + [l - 1 for l in decoding_seq_lens_list]
        starts = list(itertools.accumulate([0] + prefill_lens[:-1])) if prefill_lens else []
        out_rows = [s + n - 1 for s, n in zip(starts, prefill_lens)] + list(range(num_prefill_tokens, num_tokens)) + \
            [int(r) for r in (logit_rows or [])]
        assert all(0 <= r < num_tokens for r in out_rows)

        seg_starts = list(itertools.accumulate([0] + prefill_lens + [1] * (batch_size - num_prefill_seqs)))
        ids, seq_ids, seq_lengths, t_seq, t_pos, rows, seg = self._stage_metadata(
            flat_ids, seq_ids_list, seq_lengths_list, tok_seq, tok_pos, out_rows, seg_starts)
        if not ignore_kvcache:
            self.gpu_block_manager.allocate_blocks_for_seqs(seq_ids, seq_lengths, seq_ids_list=seq_ids_list,
                                                            target_lens_list=seq_lengths_list, want_new_blocks=False)
        st = TokenInferState(
            batch_size=batch_size, num_tokens=num_tokens, seq_ids=seq_ids, num_prefill_seqs=num_prefill_seqs,
            num_decoding_seqs=batch_size - num_prefill_seqs, num_prefill_tokens=num_prefill_tokens, token_seq_ids=t_seq,
            token_positions=t_pos, output_rows=rows, ignore_kvcache=ignore_kvcache, rotary=self._rotary_tables(t_pos),
            seg_starts=seg)
        logits = self._forward(ids, st)
        self.last_logits = logits[batch_size:].float() if logit_rows else None
        return torch.argmax(logits[:batch_size], dim=1)

    # ------------------------------------------------------------------ CUDA-graph decode path
    def _decode_step(self, ids, seq_ids, lens, bm, caches, states=None):
        """One pure-decode step on device-resident metadata (ids / seq_ids / lens int32 [B]): block allocation, rotary tables,
        every layer, head, argmax.  Allocation-free apart from activations, no host sync: capturable."""
        from swiftllm_b200.worker.kernels.block_mgmt import allocate_blocks_for_seqs as alloc_kernel
        B = ids.shape[0]
        alloc_kernel(bm.num_seq_allocated_blocks, bm.block_table, bm.is_block_free, seq_ids, lens, bm.block_size, None, bm._status)
        pos = lens - 1
        rows = torch.arange(B, dtype=torch.int32, device=self.device)
        st = TokenInferState(batch_size=B, num_tokens=B, seq_ids=seq_ids, num_prefill_seqs=0, num_decoding_seqs=B,
                             num_prefill_tokens=0, token_seq_ids=seq_ids, token_positions=pos, output_rows=rows,
                             rotary=self._rotary_tables(pos), seg_starts=torch.arange(B + 1, dtype=torch.int32, device=self.device))
        saved = self.caches, self.gpu_block_manager, self.seq_states
        self.caches, self.gpu_block_manager, self.seq_states = caches, bm, states
        try:
            logits = self._forward(ids, st)
        finally:
            self.caches, self.gpu_block_manager, self.seq_states = saved
        return torch.argmax(logits, dim=1)

    def _forward_decode_graph(self, flat_ids, seq_ids_list, lens_list) -> torch.Tensor:
        """Pure-decode step replayed from a CUDA graph (one graph per batch size; nothing in the step depends on the lengths
        except through device data)."""
        B = len(flat_ids)
        g = self._graphs.pop(B, None)
        if g is None:
            cap = max(1, int(getattr(self.engine_config, "max_cuda_graphs", 16)))
            while len(self._graphs) >= cap:
                self._graphs.pop(next(iter(self._graphs)))
            g = self._capture_decode_graph(B)
        self._graphs[B] = g                      # most recently used last
        self.gpu_block_manager.reserve_on_host(seq_ids_list, lens_list)
        i = g["next"]; g["next"] = (i + 1) % len(g["host"])
        host, ev = g["host"][i]
        ev.synchronize()                         # the copy that last read this pinned buffer has finished
        hv = host.numpy()
        hv[:B] = flat_ids; hv[B:2 * B] = seq_ids_list; hv[2 * B:] = lens_list
        g["meta"].copy_(host, non_blocking=True)
        ev.record()
        self._wait_for_swaps()
        g["graph"].replay()
        return g["tokens"].clone()               # the static output is overwritten by the next replay

    def _capture_decode_graph(self, B: int):
        ec, dev = self.engine_config, self.device
        meta = torch.zeros((3 * B,), dtype=torch.int32, device=dev)
        host = [(torch.zeros((3 * B,), dtype=torch.int32).pin_memory(), torch.cuda.Event()) for _ in range(self._STAGE_SLOTS)]
        ids, seq_ids, lens = meta[:B], meta[B:2 * B], meta[2 * B:]
        # warm-up (library handles, GEMM heuristics) against a scratch cache and block table: B one-token sequences
        scratch_bm = BlockManager("scratch", B, B, 1, ec.block_size, device=dev)
        scratch = {w: torch.zeros((B,) + tuple(c.shape[1:]), dtype=self.dtype, device=dev) for w, c in self.caches.items()}
        scratch_states = self.seq_states.scratch(B) if self.seq_states is not None else None      # live sequences keep theirs
        seq_ids.copy_(torch.arange(B, dtype=torch.int32, device=dev))
        lens.fill_(1)
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                self._decode_step(ids, seq_ids, lens, scratch_bm, scratch, scratch_states)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        del scratch, scratch_bm, scratch_states
        graph = torch.cuda.CUDAGraph()
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        with torch.cuda.graph(graph, pool=self._graph_pool):
            tokens = self._decode_step(ids, seq_ids, lens, self.gpu_block_manager, self.caches, self.seq_states)
        torch.cuda.synchronize()
        return dict(graph=graph, meta=meta, host=host, next=0, tokens=tokens)
