/*
 * swiftllm_b200.h - C ABI of the B200-native (sm_100a) data plane that replaces every kernel in
 * swiftLLM's `swiftllm/worker/kernels/` plus the native `swiftllm_c` module.
 *
 * Drop-in boundary: the reference binds its kernels as Python functions on torch tensors (one wrapper
 * per op, in place / into caller-provided outputs, current CUDA stream).  This library exports exactly
 * one entry point per wrapper, taking raw device pointers, sizes, a dtype tag and the stream; the host
 * package `swiftllm_b200/worker/kernels/*.py` binds them with ctypes under the reference's own names and
 * signatures (see INTEGRATION.md for the stub a swiftLLM maintainer would add).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless the parameter name says `host_`;
 *   - tensors are contiguous in the reference's layouts (cited per function);
 *   - all functions enqueue on `stream` (a cudaStream_t) and return immediately;
 *   - return value: 0 on success, non-zero on error (`sllm_last_error()` gives the message).  Invalid
 *     shapes are rejected before anything is launched (the reference raises AssertionError there);
 *   - no CPU fallback exists: on a non-sm_100 device every launch fails with an error.
 *
 * Reference paths below are relative to the swiftLLM repository root.
 */
#ifndef SWIFTLLM_B200_H
#define SWIFTLLM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SLLM_ABI_VERSION 1

typedef enum { SLLM_F16 = 0, SLLM_BF16 = 1, SLLM_F32 = 2 } sllm_dtype_t; /* F32: only where a function says so */
typedef void* sllm_stream_t; /* cudaStream_t */

/* ---- library ---- */
int sllm_abi_version(void);
const char* sllm_last_error(void);          /* thread-local message of the last failing call */
int sllm_device_check(int device);          /* 0 iff `device` is compute capability 10.x */

/* ---- RMSNorm: swiftllm/worker/kernels/rmsnorm.py:26-37 (rmsnorm_inplace), :67-89 (fused_add_rmsnorm_inplace)
 * x [num_tokens, hidden] in place; weight [hidden].  fused: residual <- x + residual (rounded to dtype),
 * x <- rmsnorm(residual) * weight.  hidden % 8 == 0. */
int sllm_rmsnorm_inplace(void* x, const void* weight, float eps, int64_t num_tokens, int hidden,
                         sllm_dtype_t dtype, sllm_stream_t stream);
int sllm_fused_add_rmsnorm_inplace(void* x, void* residual, const void* weight, float eps, int64_t num_tokens,
                                   int hidden, sllm_dtype_t dtype, sllm_stream_t stream);

/* ---- Rotary embedding: swiftllm/worker/kernels/rotary_emb.py:44-58 (rotary_embedding_inplace)
 * q [T, nq, D], k [T, nkv, D] in place; cos/sin [T, D/2] (infer_state.position_cos/sin).  NeoX half-split.
 * D % 16 == 0.  *_row_stride: elements between consecutive token rows (nq*D / nkv*D when contiguous, as in the
 * reference; larger when q/k/v are column slices of one fused QKV GEMM output); heads stay contiguous within a token. */
int sllm_rotary_embedding_inplace(void* q, void* k, const void* cos, const void* sin, int64_t num_tokens,
                                  int num_q_heads, int num_kv_heads, int head_dim, int64_t q_row_stride,
                                  int64_t k_row_stride, sllm_dtype_t dtype, sllm_stream_t stream);

/* ---- SwiGLU gate: swiftllm/worker/kernels/silu_and_mul.py:25-34 (silu_and_mul_inplace)
 * x [T, 2*ffn_inter_dim] = [up | gate]; x[:, :F] <- up * silu(gate).  F % 8 == 0. */
int sllm_silu_and_mul_inplace(void* x, int64_t num_tokens, int64_t ffn_inter_dim, sllm_dtype_t dtype,
                              sllm_stream_t stream);

/* ---- KV-cache store: swiftllm/worker/kernels/kvcache_mgmt.py:81-122 (store_kvcache)
 * k,v [num_tokens, nkv, D] (prefill tokens first, then one row per decoding seq);
 * caches [num_blocks, num_layers, nkv, block_size, D]; block_table int32 [*, max_blocks_per_seq];
 * seq_ids int32 [num_prefill_seqs + num_decoding_seqs]. */
int sllm_store_kvcache(const void* k, const void* v, void* k_cache, void* v_cache, const int32_t* block_table,
                       const int32_t* seq_ids, const int32_t* prefill_seq_start_locs,
                       const int32_t* prefill_seq_lens, const int32_t* decoding_seq_lens, int num_prefill_seqs,
                       int num_decoding_seqs, int64_t num_prefill_tokens, int max_prefill_len, int cur_layer,
                       int num_layers, int num_kv_heads, int block_size, int head_dim, int max_blocks_per_seq,
                       int64_t k_row_stride, int64_t v_row_stride, sllm_dtype_t dtype, sllm_stream_t stream);

/* ---- Decode-step fusion (new): rotary_embedding_inplace (rotary_emb.py:44-58) + the decode part of store_kvcache
 * (kvcache_mgmt.py:50-79) in ONE launch for a batch of decoding rows only: q [Bd, nq, D] and k [Bd, nkv, D] rotated in place
 * with cos/sin [Bd, D/2]; the rotated k row and the v row of sequence i are written to position decoding_seq_lens[i] - 1 of
 * block-table row seq_ids[i].  Same results, bit for bit, as the two separate calls. */
int sllm_rotary_store_kvcache_decode(void* q, void* k, const void* v, const void* cos, const void* sin, void* k_cache,
                                     void* v_cache, const int32_t* block_table, const int32_t* seq_ids,
                                     const int32_t* decoding_seq_lens, int num_decoding_seqs, int cur_layer,
                                     int num_layers, int num_q_heads, int num_kv_heads, int block_size, int head_dim,
                                     int max_blocks_per_seq, int64_t q_row_stride, int64_t k_row_stride,
                                     int64_t v_row_stride, sllm_dtype_t dtype, sllm_stream_t stream);

/* ---- Paged (decode) attention: swiftllm/worker/kernels/paged_attn.py:152-222 (paged_attention)
 * q [Bd, nq, D]; o [Bd, nq*D]; seq_ids = infer_state.seq_ids[num_prefill_seqs:]; seq_lens = decoding_seq_lens.
 * seq_block_size: tokens per flash-decoding split (multiple of block_size); 0 = let the library choose
 * (v1 single pass when the batch alone fills the GPU, v2 split + merge otherwise).
 * workspace: fp32 scratch for split partials, >= sllm_paged_attention_workspace_bytes(...) bytes
 * (the reference allocates mid_o / mid_o_logexpsum per call, paged_attn.py:170-180). */
int64_t sllm_paged_attention_workspace_bytes(int num_decoding_seqs, int num_q_heads, int head_dim, int max_seq_len,
                                             int seq_block_size, int num_kv_heads);
int sllm_paged_attention(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                         const int32_t* seq_ids, const int32_t* seq_lens, void* o, void* workspace,
                         int64_t workspace_bytes, float softmax_scale, int num_decoding_seqs, int max_seq_len,
                         int seq_block_size, int cur_layer, int num_layers, int num_q_heads, int num_kv_heads,
                         int block_size, int head_dim, int max_blocks_per_seq, int64_t num_blocks,
                         int64_t q_row_stride, sllm_dtype_t dtype, sllm_stream_t stream);

/* ---- Prefill attention: swiftllm/worker/kernels/prefill_attn.py:102-139 (prefill_attention) and the
 * flash_attn_varlen_func call it stands for (swiftllm/worker/layers/transformer_layer.py:86-96).
 * Causal, varlen, packed: q,o [Tp, nq, D]; k,v [Tp, nkv, D]; start_locs/seq_lens int32 [num_prefill_seqs]. */
int sllm_prefill_attention(const void* q, const void* k, const void* v, void* o, const int32_t* prefill_seq_start_locs,
                           const int32_t* prefill_seq_lens, float softmax_scale, int num_prefill_seqs,
                           int max_prefill_len, int64_t num_prefill_tokens, int num_q_heads, int num_kv_heads,
                           int head_dim, int64_t q_row_stride, int64_t k_row_stride, int64_t v_row_stride,
                           sllm_dtype_t dtype, sllm_stream_t stream);

/* ---- Chunked ("prefix-aware") prefill - SURVEY.md §8 f-1.  NEW: the reference's forward cannot express a partial prompt
 * (its prefill attention only sees the packed k/v of the batch: swiftllm/worker/kernels/prefill_attn.py:102-139,
 * swiftllm/worker/layers/transformer_layer.py:86-96; its store always starts at position 0: kvcache_mgmt.py:10-48).
 * Prefill entry i of the batch is the CHUNK of its prompt that covers positions
 * [prefill_prefix_lens[i], prefill_prefix_lens[i] + prefill_seq_lens[i]); earlier positions are already in the cache.
 *   sllm_store_kvcache_chunked   = sllm_store_kvcache with chunk token t written to position prefix + t;
 *   sllm_prefill_attention_paged = causal attention of the chunk's queries (q, o [Tp, nq, D] packed) over positions
 *       0 .. prefix + chunk - 1 read from the paged caches through rows `seq_ids` of the block table (the chunk's own
 *       K/V must have been stored first); query t sees positions <= prefix + t.  With all prefixes 0 it computes
 *       exactly what sllm_prefill_attention computes.  head_dim 64 / 128. */
int sllm_store_kvcache_chunked(const void* k, const void* v, void* k_cache, void* v_cache, const int32_t* block_table,
                               const int32_t* seq_ids, const int32_t* prefill_seq_start_locs,
                               const int32_t* prefill_seq_lens, const int32_t* prefill_prefix_lens,
                               const int32_t* decoding_seq_lens, int num_prefill_seqs, int num_decoding_seqs,
                               int64_t num_prefill_tokens, int max_prefill_len, int cur_layer, int num_layers,
                               int num_kv_heads, int block_size, int head_dim, int max_blocks_per_seq,
                               int64_t k_row_stride, int64_t v_row_stride, sllm_dtype_t dtype, sllm_stream_t stream);
int sllm_prefill_attention_paged(const void* q, const void* k_cache, const void* v_cache, void* o,
                                 const int32_t* block_table, const int32_t* seq_ids,
                                 const int32_t* prefill_seq_start_locs, const int32_t* prefill_seq_lens,
                                 const int32_t* prefill_prefix_lens, float softmax_scale, int num_prefill_seqs,
                                 int max_prefill_len, int64_t num_prefill_tokens, int cur_layer, int num_layers,
                                 int num_q_heads, int num_kv_heads, int block_size, int head_dim,
                                 int max_blocks_per_seq, int64_t num_blocks, int64_t q_row_stride, sllm_dtype_t dtype,
                                 sllm_stream_t stream);

/* ---- Block-table maintenance: swiftllm/worker/kernels/block_mgmt.py:26-46, :66-80, :106-127
 * block_table int32 [max_seqs, max_blocks_per_seq]; num_seq_allocated_blocks int32 [max_seqs];
 * is_block_free uint8/bool [num_blocks]; candidate_blocks int64 [sum(block_needed)];
 * block_needed int32 [batch]; block_needed_cumsum int32 [batch] (inclusive). */
int sllm_set_block_table_and_num_seq_alloc_blocks(int32_t* num_seq_allocated_blocks, int32_t* block_table,
                                                  const int64_t* candidate_blocks, const int32_t* seq_ids,
                                                  const int32_t* block_needed, const int32_t* block_needed_cumsum,
                                                  int batch_size, int max_blocks_per_seq, sllm_stream_t stream);
int sllm_unset_block_table_and_num_seq_alloc_blocks(int32_t* num_seq_allocated_blocks, const int32_t* block_table,
                                                    const int32_t* seq_ids, uint8_t* is_block_free, int batch_size,
                                                    int max_blocks_per_seq, sllm_stream_t stream);
/* allocated_cumsum int32 [batch] (inclusive cumsum of num_seq_allocated_blocks[seq_ids]);
 * gathered_block_ids int32 [allocated_cumsum[batch-1]] */
int sllm_gather_allocated_blocks_and_unset(int32_t* num_seq_allocated_blocks, const int32_t* block_table,
                                           const int32_t* seq_ids, uint8_t* is_block_free,
                                           const int32_t* allocated_cumsum, int32_t* gathered_block_ids,
                                           int batch_size, int max_blocks_per_seq, sllm_stream_t stream);

/* ---- Sync-free block allocation (replaces swiftllm/worker/block_manager.py:43-79: assert + .item() +
 * torch.nonzero).  One launch: for seq i (batch order) needs max(0, cdiv(target_lens[i], block_size) -
 * num_seq_allocated_blocks[seq_ids[i]]) blocks, taken lowest-free-id first - the reference's order - and
 * appended to the block table.  Writes the new ids (int64, batch order) to new_blocks_out (capacity
 * new_blocks_capacity; may be NULL) and {num_new_blocks, error_flag} to status_out (int32[2], error_flag:
 * 1 = not enough free blocks, 2 = a sequence already holds more blocks than its target; on error nothing
 * is modified). */
int sllm_allocate_blocks_for_seqs(int32_t* num_seq_allocated_blocks, int32_t* block_table, uint8_t* is_block_free,
                                  const int32_t* seq_ids, const int32_t* target_lens, int batch_size,
                                  int block_size, int64_t num_blocks, int max_blocks_per_seq,
                                  int64_t* new_blocks_out, int64_t new_blocks_capacity, int32_t* status_out,
                                  sllm_stream_t stream);

/* ---- Tensor-parallel exchange fused with the op that follows it (new; the reference is single-GPU):
 *   residual <- h(sum over ranks of partial) + residual ;  x_out <- rmsnorm(residual) * weight
 * i.e. the all-reduce after o_proj / down_proj merged with fused_add_rmsnorm_inplace (rmsnorm.py:67-89) in one kernel that
 * reads every rank's partial [num_tokens, hidden] directly over NVLink peer memory, in rank order with fp32 accumulation
 * (bit-identical on all ranks).  host_peer_bufs / host_peer_flags: HOST arrays of `nranks` DEVICE pointers: the partial buffer
 * and the flag pad (uint32 [16 slots][8]) of every rank as mapped into this process (e.g. torch symmetric memory);
 * epoch_state: local device memory, 32 uint32, zeroed once; slot: which of the alternating buffers / flag rows is used.
 * weight == NULL skips the norm (x_out unused). */
int sllm_allreduce_add_rmsnorm(const void* const* host_peer_bufs, void* const* host_peer_flags, int rank, int nranks,
                               int slot, void* epoch_state, void* x_out, void* residual, const void* weight, float eps,
                               int64_t num_tokens, int hidden, sllm_dtype_t dtype, sllm_stream_t stream);

/* Two-shot variant for larger TP degrees: token row t is reduced, added to the residual and normalised by rank t % nranks
 * only, which then stores the normalised row into EVERY rank's x_out buffer (host_peer_xout: HOST array of `nranks` DEVICE
 * pointers, symmetric memory like the partial buffers; the result appears in this rank's own buffer when the call's kernel
 * has finished).  Remote traffic per rank 2*(N-1)/N*T*H instead of (N-1)*T*H bytes; two flag barriers (signal-pad rows
 * `slot` and 8 + `slot`, slot < 8).  `residual` is only maintained for the rows this rank owns; weight is required.
 * mc_buf / mc_xout: NVLS multicast addresses (DEVICE pointers) of the partial buffer of this slot and of x_out, or both NULL.
 * When given, the reduction is ONE multimem.ld_reduce per 16 bytes (the NVSwitch sums all ranks' copies, fp32 accumulation)
 * and the broadcast ONE multimem.st, instead of N peer loads / stores. */
int sllm_allreduce_add_rmsnorm_2shot(const void* const* host_peer_bufs, void* const* host_peer_xout,
                                     void* const* host_peer_flags, const void* mc_buf, void* mc_xout, int rank, int nranks,
                                     int slot, void* epoch_state, void* residual, const void* weight, float eps,
                                     int64_t num_tokens, int hidden, sllm_dtype_t dtype, sllm_stream_t stream);

/* Low-latency variant for decode-sized exchanges (csrc/allreduce_ll.cu): same result as the two-shot call (row t reduced, added
 * to the residual and normalised by rank t % nranks, residual maintained for owned rows only), but WITHOUT barriers: partial rows
 * are pushed to their owner and normalised rows to every rank as 16-byte lines {payload, epoch tag, payload, epoch tag} that the
 * receiver polls ("LL" protocol); the complete plain rows appear in x_out (local).  partial: this rank's [num_tokens, hidden]
 * GEMM output (local).  host_peer_rs_recv / host_peer_ag_recv: HOST arrays of `nranks` DEVICE pointers to every rank's receive
 * buffers OF THIS SLOT (symmetric memory, zeroed once): rs_recv [nranks][rows_per_rank][hidden], ag_recv [>= num_tokens][hidden],
 * 4 bytes per element.  mc_ag_recv: NVLS multicast address of ag_recv (one multimem.st per line instead of nranks-1 peer stores)
 * or NULL.  num_tokens <= nranks * rows_per_rank.  epoch_state as above (shared with the other exchange calls of the slot). */
int sllm_allreduce_add_rmsnorm_ll(const void* partial, void* const* host_peer_rs_recv, void* const* host_peer_ag_recv,
                                  void* mc_ag_recv, int rank, int nranks, int slot, void* epoch_state, void* x_out,
                                  void* residual, const void* weight, float eps, int64_t num_tokens, int hidden,
                                  int64_t rows_per_rank, sllm_dtype_t dtype, sllm_stream_t stream);

/* ---- Block swapping: csrc/src/block_swapping.cpp:22-85 (swiftllm_c.swap_blocks, csrc/src/entrypoints.cpp:5-7)
 * host_src_ids/host_dst_ids: HOST arrays of n block ids.  k_swap/v_swap: HOST memory (pinned or pageable),
 * k_cache/v_cache: device.  block_bytes = bytes of one block (all layers/heads) of k_cache.
 * Consecutive (src,dst) runs are coalesced into one copy each, as the reference does. */
int sllm_swap_blocks(const int64_t* host_src_ids, const int64_t* host_dst_ids, int64_t n, int is_swap_in,
                     void* k_cache, void* v_cache, void* host_k_swap, void* host_v_swap, int64_t block_bytes,
                     sllm_stream_t stream);

/* Sync-free variant (new): src_ids / dst_ids are DEVICE arrays (int64) - the gathered source ids and the
 * newly allocated target ids never travel to the host (the reference does `.tolist()` twice per swap, model.py:374-377) - and
 * one kernel moves every block between the cache and the swap space, which must be pinned, device-mapped host memory
 * (cudaHostAlloc / torch pin_memory).  Same data movement as sllm_swap_blocks. */
int sllm_swap_blocks_gathered(const int64_t* src_ids, const int64_t* dst_ids, int64_t n, int is_swap_in, void* k_cache,
                              void* v_cache, void* host_k_swap, void* host_v_swap, int64_t block_bytes,
                              sllm_stream_t stream);

/* ---- Parallel decoder blocks with an fp32 residual stream (new; the reference has no such model).  `dtype` is the storage
 * type of projections / activations and may be SLLM_F32; sums and norms are computed in fp32 for every dtype.
 * add_rmsnorm_f32: residual (fp32 [T, width]) += a + b (dtype, [T, width], either may be NULL), then
 * out = residual / sqrt(mean(residual^2) + eps) * weight (dtype). */
int sllm_add_rmsnorm_f32(void* residual, const void* a, const void* b, const void* weight, void* out, float eps,
                         int64_t num_tokens, int width, sllm_dtype_t dtype, sllm_stream_t stream);
/* The same with the norm weight stored as fp32 [width] whatever dtype is (models whose norm weights stay in 32-bit). */
int sllm_add_rmsnorm_f32w(void* residual, const void* a, const void* b, const void* weight_f32, void* out, float eps,
                          int64_t num_tokens, int width, sllm_dtype_t dtype, sllm_stream_t stream);
/* RMS norm of the first n columns of row-strided matrices (a slice of a fused projection): out = x / rms(x) * weight. */
int sllm_rmsnorm_strided(const void* x, int64_t x_row_stride, const void* weight, void* out, int64_t out_row_stride,
                         float eps, int64_t num_tokens, int n, sllm_dtype_t dtype, sllm_stream_t stream);
/* x = relu(x)^2 over n contiguous elements. */
int sllm_relu2_inplace(void* x, int64_t n, sllm_dtype_t dtype, sllm_stream_t stream);
/* Mixture-of-experts router: logits fp32 [T, experts] -> weights fp32 [T, experts] = softmax over the `top` largest logits of
 * each row at their positions, 0 elsewhere.  top <= 32, experts <= 2048. */
int sllm_moe_route(const void* logits, void* weights, int64_t num_tokens, int experts, int top, sllm_stream_t stream);
/* Group-limited routing on scores s = softmax(logits) over ALL experts: experts form `groups` equal groups of neighbours, a
 * group's score is its largest s, only experts of the `keep` best groups can be chosen; the `top` largest s among those are
 * chosen (equal values: the lower index wins); weights [T, experts] fp32 = s / (sum of the chosen s + norm_eps) * scale at the
 * chosen experts, 0 elsewhere.  groups = keep = 1: plain top-k on a full softmax. */
int sllm_moe_route_grouped(const void* logits, void* weights, int64_t num_tokens, int experts, int top, int groups, int keep,
                           float scale, float norm_eps, sllm_stream_t stream);
/* Clamped gated-linear-unit experts.  u [T, 2 * cols] (dtype): per expert [gate (ff) | up (ff)], then a shared expert's
 * [gate (shared_ff) | up (shared_ff)]; y [T, cols] (dtype), cols = experts * ff + shared_ff.  With g = min(gate, limit),
 * v = clamp(up, -limit, limit): y = g * sigmoid(alpha * g) * (v + 1) * weights[t, e]; the shared expert uses shared_limit and
 * weight 1, or with shared_gated = 1 the weight weights[t, experts] (weights then has experts + 1 columns).  experts or
 * shared_ff may be 0 (weights may then be NULL / no shared part). */
int sllm_moe_clamped_glu_scale(const void* u, const void* weights, void* y, int64_t num_tokens, int experts, int ff, float limit,
                               int shared_ff, float shared_limit, float alpha, int shared_gated, sllm_dtype_t dtype,
                               sllm_stream_t stream);
/* u [T, experts * ff] (dtype) = relu(u)^2 * weights[t, column / ff]: experts a token does not use contribute exact zeros. */
int sllm_moe_relu2_scale_inplace(void* u, const void* weights, int64_t num_tokens, int experts, int ff, sllm_dtype_t dtype,
                                 sllm_stream_t stream);

/* ---- Latent attention over a paged cache of per-token rows [c (r) | k_rot (dr)] shared by all heads (new).
 * cache: [num_blocks, n_slots, block_size, r + dr] (dtype); tok_seq / tok_pos: int32 [T], the block-table row and the position
 * of every token of the step; cos / sin: fp32 [T, rot_dims / 2], the rotary angles of the tokens' positions (pairs (2i, 2i+1)).
 * latent_kv_store: c = rmsnorm(dkv[:, :r]) * norm_weight, k_rot = rotary(dkv[:, r : r + dr]) -> the tokens' cache rows. */
int sllm_latent_kv_store(const void* dkv, int64_t row_stride, const void* norm_weight, const void* cosb, const void* sinb,
                         const void* tok_seq, const void* tok_pos, const void* block_table, int max_blocks_per_seq,
                         void* cache, int n_slots, int slot, int block_size, int64_t num_tokens, int r, int dr, int rot_dims,
                         float eps, sllm_dtype_t dtype, sllm_stream_t stream);
/* latent_attention: per token i at position p and head h, over the cached positions max(0, p - window + 1) .. p (all of 0 .. p
 * when window <= 0): out[i, h, :r] = sigmoid(gate[i, h]) * sum_j softmax_j((q_lat[i,h] . c_j + rotary(q_rot[i,h]) . k_rot_j) * scale) c_j.
 * q_lat / q_rot / out: element strides per token and per head; gate: [T, num_heads] logits (row stride) or NULL.  r <= 1024. */
/* 16-bit dtypes with r % 16 == 0 and dr % 16 == 0 run on tensor cores (mma.sync over the heads of a token); other shapes and
 * SLLM_F32 run the fp32 CUDA-core kernel.  sllm_latent_attention_set_simt(1) forces the latter (returns the old setting). */
int sllm_latent_attention_set_simt(int on);
/* num_splits > 1 with split_workspace (fp32 [T, num_heads, num_splits, r + 2], device) lets the tensor-core kernel share a
 * query's visible keys between num_splits CTAs (steps with few tokens), merged by a second kernel; ignored by the other path. */
int sllm_latent_attention(const void* q_lat, int64_t q_lat_stride_t, int64_t q_lat_stride_h, const void* q_rot,
                          int64_t q_rot_stride_t, int64_t q_rot_stride_h, const void* cosb, const void* sinb,
                          const void* gate, int64_t gate_stride_t, const void* cache, int n_slots, int slot, int block_size,
                          const void* block_table, int max_blocks_per_seq, const void* tok_seq, const void* tok_pos,
                          void* out, int64_t out_stride_t, int64_t out_stride_h, int64_t num_tokens, int num_heads, int r,
                          int dr, int rot_dims, int window, float scale, int num_splits, void* split_workspace,
                          sllm_dtype_t dtype, sllm_stream_t stream);

/* ---- Gated sliding-window attention with grouped key/value heads over a paged cache of per-token rows
 * [k (num_kv_heads x dk, rotary applied) | v (num_kv_heads x dv)] (new).  cache: [num_blocks, n_slots, block_size,
 * num_kv_heads * (dk + dv)] (dtype); tok_seq / tok_pos, cosb / sinb and rot_dims as for latent attention.
 * window_kv_store: k [T, num_kv_heads * dk] and v [T, num_kv_heads * dv] (row strides in elements) -> the tokens' cache rows.
 * Options shared with window_attention: pair_halves = 1 pairs entry i with i + rot_dims / 2 (0: entries 2i and 2i + 1);
 * qk_norm_eps >= 0 divides every rotated key / query head by sqrt(mean of its squares + eps) (< 0: off); vcos / vsin (fp32
 * [T, dv / 2], or NULL) turn the value of every head by the token's position before it is stored, and window_attention turns
 * each head's output back by the query's position.
 * knorm_w / qnorm_w (fp32 [dk], or NULL): every key / query head is first RMS-normed, x / sqrt(mean(x^2) + prenorm_eps) * w,
 * BEFORE it turns.  vshare >= 1: `vshare` neighbouring key heads share one value head (value head = key head / vshare): v is
 * [T, num_kv_heads / vshare * dv] and the cache row [num_kv_heads * dk | num_kv_heads / vshare * dv]. */
int sllm_window_kv_store(const void* k, int64_t k_row_stride, const void* v, int64_t v_row_stride, const void* cosb,
                         const void* sinb, const void* tok_seq, const void* tok_pos, const void* block_table,
                         int max_blocks_per_seq, void* cache, int n_slots, int slot, int block_size, int64_t num_tokens,
                         int num_kv_heads, int dk, int dv, int rot_dims, int pair_halves, float qk_norm_eps, const void* vcos,
                         const void* vsin, const void* knorm_w, float prenorm_eps, int vshare, sllm_dtype_t dtype,
                         sllm_stream_t stream);
/* window_attention: per token i at position p and query head h (key/value head h / (num_heads / num_kv_heads)), over the cached
 * positions max(0, p - window + 1) .. p (all of 0 .. p when window <= 0):
 *   out[i, h, :dv] = sigmoid(gate[i, h, :dv]) * sum_j p_j v_j,   p_j = exp(s_j) / (sink + sum_j' exp(s_j')),
 *   s_j = rotary(q[i, h]) . k_j * scale;  sink = 1: the softmax has a value-less sink of score 0 (one more in the denominator).
 * q [T, num_heads * dk] un-rotated, gate [T, num_heads * dv] logits or NULL, out [T, num_heads * dv]; row strides in elements.
 * dv <= 256.  Rows [0, num_prefill_tokens) of the step are prompt portions, the others single decoded tokens (a hint for how
 * tokens are grouped into CTAs; any value in 0 .. num_tokens gives the same result).
 * 16-bit dtypes with dk, dv multiples of 16 and <= 128 run on tensor cores (mma.sync over tokens x heads of a key/value group);
 * other shapes and SLLM_F32 run the fp32 CUDA-core kernel.  sllm_window_attention_set_simt(1) forces the latter (returns the
 * old setting).  softcap > 0: s_j <- softcap * tanh(s_j / softcap); out_scale multiplies the output.
 * chunk > 0: only keys at positions >= floor(p / chunk) * chunk are seen.  out_f32 = 1: `out` is fp32 for every dtype (its row
 * stride counts floats; no turned values then). */
int sllm_window_attention_set_simt(int on);
int sllm_window_attention(const void* q, int64_t q_stride_t, const void* cosb, const void* sinb, const void* gate,
                          int64_t gate_stride_t, const void* cache, int n_slots, int slot, int block_size,
                          const void* block_table, int max_blocks_per_seq, const void* tok_seq, const void* tok_pos, void* out,
                          int64_t out_stride_t, int64_t num_tokens, int64_t num_prefill_tokens, int num_heads, int num_kv_heads,
                          int dk, int dv, int rot_dims, int window, float scale, int sink, int pair_halves, float qk_norm_eps,
                          float softcap, const void* vcos, const void* vsin, float out_scale, const void* qnorm_w,
                          float prenorm_eps, int chunk, int vshare, int out_f32, sllm_dtype_t dtype, sllm_stream_t stream);
/* diff_combine: a fp32 [T, num_kv_heads, 2, num_heads / num_kv_heads, dv] - the outputs of two score maps per head over the same
 * values (window_attention with vshare = 2, 2 * num_heads queries ordered [key/value head][map][head of the group], out_f32).
 * out[t, h] = o / sqrt(mean(o^2) + eps) * factor * sigmoid(gate[t, h]) with o = a[map 0] - lambda * a[map 1]; gate logits
 * [T, num_heads * dv] or NULL; out [T, num_heads * dv] (dtype), heads in their natural order; row strides in elements. */
int sllm_diff_combine(const void* a, const void* gate, int64_t gate_stride_t, void* out, int64_t out_stride_t, int64_t num_tokens,
                      int num_heads, int num_kv_heads, int dv, float lambda, float eps, float factor, sllm_dtype_t dtype,
                      sllm_stream_t stream);

/* ---- Sequential blocks on an fp32 residual stream whose sublayer OUTPUTS are normalised (new, stream_ops.cu).
 * embed_pair_hash: x[t] (fp32) = embed[tokens[t]] + pairs[row], row = (previous * mul_prev + token * mul_cur) mod buckets with
 * `previous` the token one position earlier (the row above, or last_token[tok_seq[t]] (int32 per sequence row) when the step
 * starts there); a token at position 0 takes row `buckets`.  pairs may be NULL (no pair table).  x_copy (fp32, may be NULL)
 * gets the same values; h gets their rounding to dtype.  store_last_tokens then records every segment's last token. */
int sllm_embed_pair_hash(const void* tokens, const void* tok_seq, const void* tok_pos, const void* last_token, const void* embed,
                         const void* pairs, int buckets, int64_t mul_prev, int64_t mul_cur, void* x, void* x_copy, void* h,
                         int64_t num_tokens, int width, sllm_dtype_t dtype, sllm_stream_t stream);
int sllm_store_last_tokens(const void* tokens, const void* seg_starts, const void* seq_ids, void* last_token, int num_segs,
                           sllm_stream_t stream);
/* postnorm_add_mix: X = x + gain[0] * y / sqrt(mean(y^2) + eps) per row (X = x when y is NULL); history (fp32
 * [slots, T, width], may be NULL) slot `slot` <- X; with mix (fp32 [slot + 1], may be NULL) x <- sum_j mix[j] * history[j], else
 * x <- X; h <- x rounded to dtype.  x fp32 [T, width] in place, y dtype, gain fp32 on the device. */
int sllm_postnorm_add_mix(void* x, const void* y, const void* gain, float eps, void* history, int slot, const void* mix, void* h,
                          int64_t num_tokens, int width, sllm_dtype_t dtype, sllm_stream_t stream);
int sllm_tanh_cap_inplace(void* x, int64_t n, float cap, sllm_dtype_t dtype, sllm_stream_t stream);
/* moe_route_sigmoid: logits fp32 [T, experts] -> weights fp32 [T, experts]: s = sigmoid(logits); the `top` experts with the
 * largest s + bias (fp32 [experts] or NULL) get weight s, the others 0.  moe_silu_glu_scale: u [T, experts * 2 * ff] (per expert
 * [gate | up]) -> y [T, experts * ff] = silu(gate) * up * weights[t, expert]. */
int sllm_moe_route_sigmoid(const void* logits, const void* bias, void* weights, int64_t num_tokens, int experts, int top,
                           sllm_stream_t stream);
int sllm_moe_silu_glu_scale(const void* u, const void* weights, void* y, int64_t num_tokens, int experts, int ff,
                            sllm_dtype_t dtype, sllm_stream_t stream);

/* ---- Recurrent mixers with per-sequence state (new, recurrent.cu).  A step's rows seg_starts[b] .. seg_starts[b + 1] - 1 are
 * consecutive positions of sequence row seq_ids[b]; a segment at position 0 starts from the zero state.
 * causal_conv: u[t, c] = bias[c] + sum_k w[c, taps - 1 - k] * xin[t - k, c] over the sequence (tail: dtype [rows, taps - 1,
 * channels], the sequence's last inputs before this step; xin row stride in elements).
 * rglru_scan: gates dtype [blocks, T, 2 * channels / blocks] (logits of the recurrence gate, then of the input gate, per block);
 * a = exp(rate[c] * sigmoid(r)); S <- a S + sqrt(1 - a^2) sigmoid(i) u; out = S * gelu_tanh(ybr); state fp32 [rows, channels];
 * also moves `tail` on by the segment's inputs xin.  The first num_prefill_segs segments (prompt portions) run parallel over time
 * (tiles of 64 tokens whose eight runs are composed as maps S -> a S + b), the rest one thread per channel. */
int sllm_causal_conv(const void* xin, int64_t xin_stride, const void* w, const void* bias, const void* tail, const void* tok_seq,
                     const void* tok_pos, void* u, int64_t num_tokens, int64_t num_prefill_tokens, int channels, int taps,
                     sllm_dtype_t dtype, sllm_stream_t stream);
int sllm_rglru_scan(const void* u, const void* gates, int blocks, const void* ybr, int64_t y_stride, const void* rate,
                    const void* xin, int64_t xin_stride, void* state, void* tail, const void* seg_starts, const void* seq_ids,
                    const void* tok_pos, void* out, int64_t num_tokens, int num_segs, int num_prefill_segs, int channels, int taps,
                    sllm_dtype_t dtype, sllm_stream_t stream);
/* linear_attention: per head S <- decay[h] S + silu(k) silu(v)^T, out[t, h] (fp32 [T, heads * dv]) = S^T silu(q); q, k
 * [T, heads * dk], v [T, heads * dv] pre-activation (row strides in elements); state fp32 [rows, heads, dk, dv].
 * gated_rmsnorm: out = x / sqrt(mean(x^2) + eps) * weight * sigmoid(gate) * out_scale; x fp32 [T, n], weight fp32 [n], gate
 * dtype logits (may be NULL), out dtype (row strides in elements). */
int sllm_linear_attention(const void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v, int64_t v_stride,
                          const void* decay, void* state, const void* seg_starts, const void* seq_ids, const void* tok_pos,
                          void* out, int num_segs, int num_heads, int dk, int dv, sllm_dtype_t dtype, sllm_stream_t stream);
int sllm_gated_rmsnorm(const void* x, const void* weight, const void* gate, int64_t gate_stride, float eps, float out_scale,
                       void* out, int64_t out_stride, int64_t num_tokens, int n, sllm_dtype_t dtype, sllm_stream_t stream);

/* ---- Sandwich blocks: x <- x + mult * norm_b(sublayer(norm_a(x))) with RMS norms over `groups` equal consecutive parts of a row
 * (new, sandwich_ops.cu).  group_norm_add_norm: with y (dtype [T, width]) x (fp32, in place) += mult * y / rms_g(y) * wb; with
 * wn, n_out (fp32) = x / rms_g(x) * wn of the updated x; either half may be left out (NULL).  group_norm_cast: out (dtype) =
 * x / rms_g(x) * w.  stream_add: x += a (fp32 [T, width] or NULL) + v (fp32 [width] or NULL).
 * gelu_glu: u [T, 2 ff] = [gate | up] -> y [T, ff] = gelu_tanh(gate) * up.
 * moe_route_softmax: logits fp32 [T, experts (+ 1 when gated)] -> weights of the same shape: s = softmax over the experts, the
 * `top` largest s (equal values: the lower index) keep s, the others 0; gated: the last column becomes its sigmoid. */
int sllm_group_norm_add_norm(void* x, const void* y, const void* wb, float mult, const void* wn, void* n_out, float eps,
                             int64_t num_tokens, int width, int groups, sllm_dtype_t dtype, sllm_stream_t stream);
int sllm_group_norm_cast(const void* x, const void* w, void* out, float eps, int64_t num_tokens, int width, int groups,
                         sllm_dtype_t dtype, sllm_stream_t stream);
int sllm_stream_add(void* x, const void* a, const void* v, int64_t num_tokens, int width, sllm_stream_t stream);
int sllm_gelu_glu(const void* u, void* y, int64_t num_tokens, int ff, sllm_dtype_t dtype, sllm_stream_t stream);
int sllm_moe_route_softmax(const void* logits, void* weights, int64_t num_tokens, int experts, int top, int gated,
                           sllm_stream_t stream);

/* ---- Per-channel recurrences with per-sequence state (new, scan_ops.cu); segments as for the recurrent mixers above.
 * short_conv: out[t, c] = act(bias[c] + sum_k w[c, taps - 1 - k] * xin[t - k, c]) (+ xin[t, c] when add_input); w, bias fp32;
 * xin and tail ([rows, taps - 1, channels]) of in_dtype (SLLM_F32 or out_dtype); act_silu = 1: SiLU.  conv_tail_update moves
 * the tail on by the segments' inputs and runs after every reader of the old tail.  move_decode_tails = 1: the rows from
 * num_prefill_tokens on are one-token segments of sequences that appear once in the step; short_conv moves their tails on itself
 * (conv_tail_update then only needs the prompt segments).
 * mingru_scan: proj [T, 3 channels] rows [z logits | candidate pre-activations u | gate pre-activations g] (row stride in
 * elements); z = sigmoid, c = u + 1/2 (u >= 0) | sigmoid(u); S <- (1 - z) S + z c; out = S * silu(g); state fp32 [rows, channels].
 * selective_scan: x, z dtype [T, channels]; dt [T, channels] step logits (fp32 when dt_f32, else dtype); bc rows hold B at
 * column b_off and C at c_off (`states` each); A fp32 [channels, states]; dt = softplus(dt + dt_bias);
 * S[c, n] <- exp(dt A) S + dt x B[n]; out = (sum_n S C[n] + D x) * silu(z); state fp32 [rows, channels, states]; states <= 256.
 * Both scans: the first num_prefill_segs segments (prompt portions) run through kernels that stage or split tiles of tokens
 * (minGRU: 64 tokens as eight composed runs; selective scan: 16 tokens staged in shared memory), the rest (single decoded tokens)
 * one thread per channel (and state slice); any value in 0 .. num_segs gives the same result up to rounding. */
int sllm_short_conv(const void* xin, int64_t xin_stride, sllm_dtype_t in_dtype, const void* w, const void* bias, const void* tail,
                    const void* tok_seq, const void* tok_pos, void* out, sllm_dtype_t out_dtype, int64_t num_tokens,
                    int64_t num_prefill_tokens, int channels, int taps, int add_input, int act_silu, int move_decode_tails,
                    sllm_stream_t stream);
int sllm_conv_tail_update(const void* xin, int64_t xin_stride, void* tail, const void* seg_starts, const void* seq_ids,
                          const void* tok_pos, int num_segs, int channels, int taps, sllm_dtype_t dtype, sllm_stream_t stream);
int sllm_mingru_scan(const void* proj, int64_t proj_stride, void* state, const void* seg_starts, const void* seq_ids,
                     const void* tok_pos, void* out, int num_segs, int num_prefill_segs, int channels, sllm_dtype_t dtype,
                     sllm_stream_t stream);
int sllm_selective_scan(const void* x, int64_t x_stride, const void* dt, int64_t dt_stride, int dt_f32, const void* dt_bias,
                        const void* A, const void* bc, int64_t bc_stride, int b_off, int c_off, const void* D, const void* z,
                        int64_t z_stride, void* state, const void* seg_starts, const void* seq_ids, const void* tok_pos, void* out,
                        int num_segs, int num_prefill_segs, int channels, int states, sllm_dtype_t dtype, sllm_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* SWIFTLLM_B200_H */
