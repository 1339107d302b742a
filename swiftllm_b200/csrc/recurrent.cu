// Recurrent mixers: their state lives per SEQUENCE (row `seq` of a state tensor, the block-table row of the sequence), in fp32,
// and is carried from step to step.  A step brings SEGMENTS: rows seg_starts[b] .. seg_starts[b+1] - 1 of the packed batch are
// consecutive positions of sequence seq_ids[b] (a prompt portion, or one decoded token).  A segment that starts at position 0
// starts from the zero state whatever its row of the state tensor holds (rows are used again without being cleared).
//
//   causal_conv        u[t, c] = b[c] + sum_k w[c, K-1-k] * x[t-k, c]; inputs before the segment come from the sequence's tail
//                      (its last K-1 inputs), inputs before position 0 are zero
//   rglru_scan         per channel: a = exp(rate[c] * sigmoid(r)), S <- a S + sqrt(1 - a^2) * sigmoid(i) * u;
//                      out = S * gelu_tanh(y); also moves the convolution tail on
//   linear_attention   per head: S <- decay_h S + silu(k) silu(v)^T (S: dk x dv), out = S^T silu(q)
//   gated_rmsnorm      out = x / rms(x) * weight * sigmoid(gate) * out_scale
// Gates, decays, the states and the norm run in fp32 for every storage type T of the projections.
#include <type_traits>

#include "mma_helpers.cuh"
#include "typed_io.cuh"

namespace sllm {

constexpr int CONV_MAX_TAPS = 8;

// grid (ceil(T / CONV_TOKENS), ceil(C / 128)).  tail: [rows, K-1, C] (slot i: the input K-1-i positions before the next one).
// A thread walks CONV_TOKENS consecutive rows of one channel and keeps the last K-1 inputs in registers; where a row does not
// continue the row above (another sequence, or the first row of the tile) the window is filled again: from the rows above as far
// as they are the sequence's previous positions, from the sequence's tail before that, zeros before position 0.
// Rows [row0, row_end) of the batch; CONV_TOKENS = 16 for prompt portions, 1 for single decoded tokens (whose window is filled
// from the tail for every row, all rows at once).
template <typename T, int CONV_TOKENS>
__global__ void __launch_bounds__(128) causal_conv_kernel(const T* __restrict__ xin, int64_t xin_stride, const T* __restrict__ w,
                                                          const T* __restrict__ bias, const T* __restrict__ tail,
                                                          const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                                          T* __restrict__ u, int64_t row0, int64_t row_end, int C, int K) {
    const int64_t tile0 = row0 + (int64_t)blockIdx.x * CONV_TOKENS;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float wk[CONV_MAX_TAPS], hist[CONV_MAX_TAPS];       // wk[k]: weight of the input k positions back; hist[k - 1]: that input
#pragma unroll
    for (int k = 0; k < CONV_MAX_TAPS; k++) { wk[k] = k < K ? ldf(w + (int64_t)c * K + (K - 1 - k)) : 0.f; hist[k] = 0.f; }
    const float b0 = bias != nullptr ? ldf(bias + c) : 0.f;
    const int nrows = (int)min((int64_t)CONV_TOKENS, row_end - tile0);
    float xv[CONV_TOKENS];
#pragma unroll
    for (int i = 0; i < CONV_TOKENS; i++) xv[i] = i < nrows ? ldf(xin + (tile0 + i) * xin_stride + c) : 0.f;
    int prev_seq = -1, prev_pos = -2;
#pragma unroll
    for (int i = 0; i < CONV_TOKENS; i++) {
        if (i >= nrows) break;
        const int64_t t = tile0 + i;
        const int seq = tok_seq[t], pos = tok_pos[t];
        if (i == 0 || seq != prev_seq || pos != prev_pos + 1) {
            int above = 0;                              // rows above this one that are the sequence's previous positions
            while (above < K - 1 && t - above - 1 >= 0 && tok_seq[t - above - 1] == seq && tok_pos[t - above - 1] == pos - above - 1) above++;
#pragma unroll
            for (int k = 1; k < CONV_MAX_TAPS; k++) {
                float v = 0.f;
                if (k < K && pos - k >= 0)
                    v = k <= above ? ldf(xin + (t - k) * xin_stride + c)
                                   : ldf(tail + ((int64_t)seq * (K - 1) + (K - 1 - (k - above))) * C + c);
                hist[k - 1] = v;
            }
        }
        float acc = b0 + wk[0] * xv[i];
#pragma unroll
        for (int k = 1; k < CONV_MAX_TAPS; k++) acc += wk[k] * hist[k - 1];
        stf(u + t * C + c, acc);
#pragma unroll
        for (int k = CONV_MAX_TAPS - 1; k >= 1; k--) hist[k] = hist[k - 1];
        hist[0] = xv[i];
        prev_seq = seq; prev_pos = pos;
    }
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }

// grid (segments, ceil(C / 128)): one thread per (segment, channel) walks the segment's tokens.
// gates: [blocks, T, 2 * cb] (cb = C / blocks): per block the logits of the recurrence gate, then of the input gate.
template <typename T>
__global__ void __launch_bounds__(128) rglru_scan_kernel(
    const T* __restrict__ u, const T* __restrict__ gates, int cb, const T* __restrict__ ybr, int64_t y_stride,
    const float* __restrict__ rate, const T* __restrict__ xin, int64_t xin_stride, float* __restrict__ state,
    T* __restrict__ tail, const int* __restrict__ seg_starts, const int* __restrict__ seq_ids, const int* __restrict__ tok_pos,
    T* __restrict__ out, int64_t num_tokens, int C, int K) {
    const int b = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int t0 = seg_starts[b], n = seg_starts[b + 1] - t0;
    if (c >= C || n <= 0) return;
    const int seq = seq_ids[b], p0 = tok_pos[t0];
    const int blk = c / cb, cc = c - blk * cb;
    const float rt = rate[c];
    float S = p0 > 0 ? state[(int64_t)seq * C + c] : 0.f;
    const T* gr = gates + ((int64_t)blk * num_tokens + t0) * 2 * cb + cc;
    for (int i = 0; i < n; i++) {
        const int64_t t = t0 + i;
        const float x = ldf(u + t * C + c);
        const float r = sigmoid_f(ldf(gr + (int64_t)i * 2 * cb)), g = sigmoid_f(ldf(gr + (int64_t)i * 2 * cb + cb));
        const float log_a = rt * r;
        const float a = expf(log_a);
        S = a * S + sqrtf(-expm1f(2.f * log_a)) * (g * x);              // 1 - a^2 without cancellation near a = 1
        stf(out + t * C + c, S * gelu_tanh_f(ldf(ybr + t * y_stride + c)));
    }
    state[(int64_t)seq * C + c] = S;
    // the convolution tail: slot i <- the input at position p0 + n - (K-1) + i
    float old[CONV_MAX_TAPS];
    T* tl = tail + (int64_t)seq * (K - 1) * C + c;
    for (int i = 0; i < K - 1; i++) old[i] = p0 > 0 ? ldf(tl + (int64_t)i * C) : 0.f;
    for (int i = 0; i < K - 1; i++) {
        const int rel = n - (K - 1) + i;               // position relative to the segment's start
        float v = 0.f;
        if (rel >= 0) v = ldf(xin + (int64_t)(t0 + rel) * xin_stride + c);
        else if (p0 + rel >= 0 && rel + K - 1 >= 0) v = old[rel + K - 1];
        stf(tl + (int64_t)i * C, v);
    }
}

// The same recurrence for PROMPT PORTIONS, parallel over time as well: grid (segments, ceil(C / 32)), 8 warps.  Lane: channel;
// warp w: tokens w TT .. w TT + TT - 1 of the current tile of 8 TT tokens.  Every thread turns its tokens' gates into the pairs
// (a, b) of S <- a S + b (the sigmoids, exponentials, root and the GELU branch are the expensive part and run for 8 TT tokens at
// once), folds them into one pair for its run, the eight pairs of a tile meet in shared memory, every thread composes the state
// at its run's start (and the state after the tile) from them and replays its run.  Composition of the maps S -> a S + b is exact
// algebra; in floating point the result differs from the token-by-token loop by rounding only.
constexpr int SCAN_WARPS = 8;

template <typename T, int TT>
__global__ void __launch_bounds__(SCAN_WARPS * 32) rglru_scan_tiled_kernel(
    const T* __restrict__ u, const T* __restrict__ gates, int cb, const T* __restrict__ ybr, int64_t y_stride,
    const float* __restrict__ rate, const T* __restrict__ xin, int64_t xin_stride, float* __restrict__ state,
    T* __restrict__ tail, const int* __restrict__ seg_starts, const int* __restrict__ seq_ids, const int* __restrict__ tok_pos,
    T* __restrict__ out, int64_t num_tokens, int C, int K) {
    __shared__ float sA[SCAN_WARPS][32], sB[SCAN_WARPS][32];
    const int b = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = blockIdx.y * 32 + lane;
    const int t0 = seg_starts[b], n = seg_starts[b + 1] - t0;
    if (n <= 0) return;
    const bool ok = c < C;
    const int cs = ok ? c : 0;                          // dead lanes walk channel 0 and store nothing
    const int seq = seq_ids[b], p0 = tok_pos[t0];
    const int blk = cs / cb, cc = cs - blk * cb;
    const float rt = rate[cs];
    float carry = p0 > 0 ? state[(int64_t)seq * C + cs] : 0.f;
    const T* gr = gates + ((int64_t)blk * num_tokens + t0) * 2 * cb + cc;
    for (int tile0 = 0; tile0 < n; tile0 += SCAN_WARPS * TT) {
        const int i0 = tile0 + warp * TT;
        float a[TT], bb[TT], gy[TT];
        float A = 1.f, B = 0.f;
        // every load of the run is issued before the first result is needed (rows past the segment's end re-read its last row)
#pragma unroll
        for (int j = 0; j < TT; j++) {
            const int64_t i = min(i0 + j, n - 1), t = t0 + i;
            a[j] = ldf(gr + i * 2 * cb);
            bb[j] = ldf(gr + i * 2 * cb + cb);
            gy[j] = ldf(ybr + t * y_stride + cs);
        }
        float xr[TT];
#pragma unroll
        for (int j = 0; j < TT; j++) xr[j] = ldf(u + (int64_t)(t0 + min(i0 + j, n - 1)) * C + cs);
#pragma unroll
        for (int j = 0; j < TT; j++) {
            if (i0 + j < n) {
                const float r = sigmoid_f(a[j]), g = sigmoid_f(bb[j]);
                const float log_a = rt * r;
                a[j] = expf(log_a);
                bb[j] = sqrtf(-expm1f(2.f * log_a)) * (g * xr[j]);              // 1 - a^2 without cancellation near a = 1
                gy[j] = gelu_tanh_f(gy[j]);
                B = a[j] * B + bb[j];
                A *= a[j];
            } else {
                a[j] = 1.f; bb[j] = 0.f; gy[j] = 0.f;
            }
        }
        sA[warp][lane] = A;
        sB[warp][lane] = B;
        __syncthreads();
        float S = carry;
        for (int w = 0; w < warp; w++) S = sA[w][lane] * S + sB[w][lane];
        float E = S;                                    // every warp composes the state after the tile in the same order
        for (int w = warp; w < SCAN_WARPS; w++) E = sA[w][lane] * E + sB[w][lane];
        carry = E;
#pragma unroll
        for (int j = 0; j < TT; j++) {
            if (i0 + j < n) {
                S = a[j] * S + bb[j];
                if (ok) stf(out + (int64_t)(t0 + i0 + j) * C + c, S * gy[j]);
            }
        }
        __syncthreads();                                // sA / sB are rewritten by the next tile
    }
    if (warp != 0 || !ok) return;
    state[(int64_t)seq * C + c] = carry;
    float old[CONV_MAX_TAPS];
    T* tl = tail + (int64_t)seq * (K - 1) * C + c;
    for (int i = 0; i < K - 1; i++) old[i] = p0 > 0 ? ldf(tl + (int64_t)i * C) : 0.f;
    for (int i = 0; i < K - 1; i++) {
        const int rel = n - (K - 1) + i;
        float v = 0.f;
        if (rel >= 0) v = ldf(xin + (int64_t)(t0 + rel) * xin_stride + c);
        else if (p0 + rel >= 0 && rel + K - 1 >= 0) v = old[rel + K - 1];
        stf(tl + (int64_t)i * C, v);
    }
}

// A read-only global load that stays where it is written (a volatile asm is not moved across other volatile asm or barriers): the
// prefetch of the next token batch must be ISSUED before the current batch is multiplied, not sunk to its first use.
template <typename T>
__device__ __forceinline__ float ldf_pinned(const T* p) {
    if constexpr (sizeof(T) == 4) {
        float f;
        asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(f) : "l"(p));
        return f;
    } else {
        unsigned short u;
        asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(u) : "l"(p));
        if constexpr (std::is_same<T, __nv_bfloat16>::value) return __uint_as_float((unsigned)u << 16);
        else return __half2float(__ushort_as_half(u));
    }
}

// silu of a projection's output.  With 16-bit storage the activation only has to be good to that type's rounding: fast exponential
// and division; with fp32 storage the accurate ones.
template <typename T>
__device__ __forceinline__ float silu_act(float z) {
    if constexpr (sizeof(T) == 4) return z * sigmoid_f(z);
    else return __fdividef(z, 1.f + __expf(-z));
}

// Linear attention with a constant decay per head.  The columns of a head's state S [dk, dv] never mix (out[j] = sum_d S[d, j] q[d],
// S[d, j] <- decay S[d, j] + k[d] v[j]), so a CTA owns 32 CPT columns of one (segment, head): grid (segments, heads,
// ceil(dv / (32 CPT))), 8 warps.  Lane j: columns j, j + 32, .. (CPT of them); warp w: rows w R .. w R + R - 1 of the state, in
// registers for the whole segment.  Tokens are staged LA_TOKENS at a time (silu applied once, rows padded with zeros to 8 R);
// every warp walks them without a barrier and keeps its partial dot products in registers; the eight partial sums per (token,
// column) meet in shared memory once per batch.  k and q reach the threads as broadcast reads of shared memory, four rows a read;
// every read serves 4 CPT fused multiply-adds per lane, and CPT = 4 is where the shared-memory pipe and the FMA pipe balance.
// Inside a batch the decay is folded into the staged vectors: with U_i = S_start + sum_{j <= i} decay^-(j+1) k_j v_j^T the state
// after token i is decay^(i+1) U_i, so k_j is staged times decay^-(j+1), q_i times decay^(i+1), the update is ONE fused
// multiply-add per state entry (plus one for the dot product), and the state is scaled by decay^tokens once per batch.  Eight
// tokens keep the factors within 2^32 for decay >= 1/16; a smaller decay takes the direct form (decay * S + k v).
constexpr int LA_TOKENS = 8;
constexpr int LA_WARPS = 8;
constexpr float LA_MIN_FOLDED_DECAY = 0.0625f;

// ASYNC: the next batch's raw q / k / v rows travel to shared memory by cp.async (16-byte pieces: needs 16-byte aligned rows, see
// the launcher) while the current batch is multiplied; otherwise they are prefetched into registers by plain loads.
template <typename T, int R, int CPT, bool ASYNC>
__global__ void __launch_bounds__(LA_WARPS * 32) linear_attention_kernel(
    const T* __restrict__ q, int64_t q_stride, const T* __restrict__ k, int64_t k_stride, const T* __restrict__ v, int64_t v_stride,
    const float* __restrict__ decay, float* __restrict__ state, const int* __restrict__ seg_starts, const int* __restrict__ seq_ids,
    const int* __restrict__ tok_pos, float* __restrict__ out, int H, int dk, int dv) {
    constexpr int DKP = LA_WARPS * R;                                   // padded rows
    constexpr int COLS = 32 * CPT;
    extern __shared__ __align__(16) unsigned char la_smem[];
    float (*qs)[DKP] = reinterpret_cast<float (*)[DKP]>(la_smem);                                   // [LA_TOKENS][DKP]
    float (*ks)[DKP] = qs + LA_TOKENS;                                                               // [LA_TOKENS][DKP]
    float (*vs)[COLS] = reinterpret_cast<float (*)[COLS]>(ks + LA_TOKENS);                           // [LA_TOKENS][COLS]
    float (*red)[LA_TOKENS][COLS] = reinterpret_cast<float (*)[LA_TOKENS][COLS]>(vs + LA_TOKENS);    // [LA_WARPS][LA_TOKENS][COLS]
    float* fq = reinterpret_cast<float*>(red + LA_WARPS);               // decay^(i+1) ...
    float* fk = fq + LA_TOKENS;                                         // ... and its inverse (1 in the direct form)
    T* rawq = reinterpret_cast<T*>(fk + LA_TOKENS);                     // ASYNC only: [LA_TOKENS][dk], [LA_TOKENS][dk], [LA_TOKENS][COLS]
    T* rawk = rawq + LA_TOKENS * dk;
    T* rawv = rawk + LA_TOKENS * dk;
    const int b = blockIdx.x, h = blockIdx.y;
    const int t0 = seg_starts[b], n = seg_starts[b + 1] - t0;
    if (n <= 0) return;
    const int seq = seq_ids[b], p0 = tok_pos[t0];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int col0 = blockIdx.z * COLS + lane;                          // this thread's columns: col0 + 32 c
    const float lam = decay[h];
    const bool folded = lam >= LA_MIN_FOLDED_DECAY;
    if (tid < LA_TOKENS) {
        const float pw = folded ? powf(lam, (float)(tid + 1)) : 1.f;
        fq[tid] = pw;
        fk[tid] = 1.f / pw;
    }
    float* st = state + ((int64_t)seq * H + h) * dk * dv;
    float S[R][CPT];
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int d = warp * R + r;
#pragma unroll
        for (int c = 0; c < CPT; c++)
            S[r][c] = (col0 + 32 * c < dv && d < dk && p0 > 0) ? st[(int64_t)d * dv + col0 + 32 * c] : 0.f;
    }
    __syncthreads();                                                    // fq / fk
    // raw inputs of one batch, as this thread stages them: NQ entries of q and of k (entry idx = tid + e * 256 of the padded
    // [LA_TOKENS][DKP] tile), CPT of v (warp i stages token i's columns)
    constexpr int NQ = LA_TOKENS * DKP / (LA_WARPS * 32);
    float rq[NQ], rk[NQ], rv[CPT];
    auto fetch = [&](int i0) {
        const int nt = min(LA_TOKENS, n - i0);
#pragma unroll
        for (int e = 0; e < NQ; e++) {
            const int idx = tid + e * (LA_WARPS * 32);
            const int i = idx / DKP, d = idx - i * DKP;
            rq[e] = 0.f; rk[e] = 0.f;
            if (i < nt && d < dk) {
                const int64_t t = t0 + i0 + i;
                rq[e] = ldf_pinned(q + t * q_stride + (int64_t)h * dk + d);
                rk[e] = ldf_pinned(k + t * k_stride + (int64_t)h * dk + d);
            }
        }
#pragma unroll
        for (int c = 0; c < CPT; c++)
            rv[c] = (warp < nt && col0 + 32 * c < dv) ? ldf_pinned(v + (int64_t)(t0 + i0 + warp) * v_stride + (int64_t)h * dv + col0 + 32 * c) : 0.f;
    };
    // ASYNC: 16-byte pieces of the batch's rows, round-robin over the threads
    constexpr int PIECE = 16 / (int)sizeof(T);                          // elements per piece
    auto issue = [&](int i0) {
        const int nt = min(LA_TOKENS, n - i0);
        const int cq = dk / PIECE;
        for (int idx = tid; idx < nt * cq; idx += LA_WARPS * 32) {
            const int i = idx / cq, ch = idx - i * cq;
            const int64_t t = t0 + i0 + i;
            cp_async16(smem_u32(rawq + i * dk + ch * PIECE), q + t * q_stride + (int64_t)h * dk + ch * PIECE);
            cp_async16(smem_u32(rawk + i * dk + ch * PIECE), k + t * k_stride + (int64_t)h * dk + ch * PIECE);
        }
        constexpr int CV = COLS / PIECE;
        for (int idx = tid; idx < nt * CV; idx += LA_WARPS * 32) {
            const int i = idx / CV, ch = idx - i * CV;
            const int c0 = blockIdx.z * COLS + ch * PIECE;
            if (c0 < dv)                                                // dv is a multiple of PIECE: the piece is inside the row
                cp_async16(smem_u32(rawv + i * COLS + ch * PIECE), v + (int64_t)(t0 + i0 + i) * v_stride + (int64_t)h * dv + c0);
        }
        cp_async_commit();
    };
    if constexpr (ASYNC) issue(0); else fetch(0);
    for (int i0 = 0; i0 < n; i0 += LA_TOKENS) {
        const int nt = min(LA_TOKENS, n - i0);
        // stage the batch: silu(q), silu(k) (zeros from dk on), silu(v) of this CTA's columns (silu(0) = 0 keeps the padding)
        if constexpr (ASYNC) {
            cp_async_wait<0>();
            __syncthreads();                                            // the raw rows have landed (every thread's pieces)
#pragma unroll
            for (int e = 0; e < NQ; e++) {
                const int idx = tid + e * (LA_WARPS * 32);
                const int i = idx / DKP, d = idx - i * DKP;
                const bool live = i < nt && d < dk;
                qs[i][d] = live ? silu_act<T>(ldf(rawq + i * dk + d)) * fq[i] : 0.f;
                ks[i][d] = live ? silu_act<T>(ldf(rawk + i * dk + d)) * fk[i] : 0.f;
            }
#pragma unroll
            for (int c = 0; c < CPT; c++)
                vs[warp][lane + 32 * c] = (warp < nt && col0 + 32 * c < dv) ? silu_act<T>(ldf(rawv + warp * COLS + lane + 32 * c)) : 0.f;
            __syncthreads();                                            // staged; the raw rows may be overwritten
            if (i0 + LA_TOKENS < n) issue(i0 + LA_TOKENS);              // in flight while this batch is multiplied
        } else {
#pragma unroll
            for (int e = 0; e < NQ; e++) {
                const int idx = tid + e * (LA_WARPS * 32);
                const int i = idx / DKP, d = idx - i * DKP;
                qs[i][d] = silu_act<T>(rq[e]) * fq[i];
                ks[i][d] = silu_act<T>(rk[e]) * fk[i];
            }
#pragma unroll
            for (int c = 0; c < CPT; c++) vs[warp][lane + 32 * c] = silu_act<T>(rv[c]);
            if (i0 + LA_TOKENS < n) fetch(i0 + LA_TOKENS);    // in flight while this batch is multiplied
            __syncthreads();
        }
        // one token after the other; `fold` is a compile-time flag so that the loops hold fused multiply-adds only
        auto multiply = [&](auto fold) {
            constexpr bool FOLD = decltype(fold)::value;
#pragma unroll
            for (int i = 0; i < LA_TOKENS; i++) {
                float part[CPT];
#pragma unroll
                for (int c = 0; c < CPT; c++) part[c] = 0.f;
                if (i < nt) {                                           // uniform over the CTA
                    float vj[CPT];
#pragma unroll
                    for (int c = 0; c < CPT; c++) vj[c] = vs[i][lane + 32 * c];
#pragma unroll
                    for (int r = 0; r < R; r += 4) {
                        const float4 k4 = *reinterpret_cast<const float4*>(&ks[i][warp * R + r]);
                        const float4 q4 = *reinterpret_cast<const float4*>(&qs[i][warp * R + r]);
                        const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
                        for (int e = 0; e < 4; e++) {
#pragma unroll
                            for (int c = 0; c < CPT; c++) {
                                if constexpr (FOLD) S[r + e][c] = fmaf(kk[e], vj[c], S[r + e][c]);
                                else S[r + e][c] = fmaf(lam, S[r + e][c], kk[e] * vj[c]);
                                part[c] = fmaf(S[r + e][c], qq[e], part[c]);
                            }
                        }
                    }
                }
#pragma unroll
                for (int c = 0; c < CPT; c++) red[warp][i][lane + 32 * c] = part[c];
            }
            if constexpr (FOLD) {
                const float back = fq[nt - 1];                          // U -> S = decay^tokens U
#pragma unroll
                for (int r = 0; r < R; r++)
#pragma unroll
                    for (int c = 0; c < CPT; c++) S[r][c] *= back;
            }
        };
        if (folded) multiply(std::true_type{});                         // uniform over the CTA
        else multiply(std::false_type{});
        __syncthreads();                    // partial sums visible; qs / ks / vs are done with and may be staged again
        {
            const int i = warp;                                         // warp i adds up token i
            if (i < nt) {
#pragma unroll
                for (int c = 0; c < CPT; c++) {
                    if (col0 + 32 * c < dv) {
                        float o = 0.f;
#pragma unroll
                        for (int w = 0; w < LA_WARPS; w++) o += red[w][i][lane + 32 * c];
                        out[(int64_t)(t0 + i0 + i) * ((int64_t)H * dv) + (int64_t)h * dv + col0 + 32 * c] = o;
                    }
                }
            }
        }
        // the next batch writes `red` only after its own first barrier, which every warp reaches after this read
    }
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int d = warp * R + r;
#pragma unroll
        for (int c = 0; c < CPT; c++)
            if (col0 + 32 * c < dv && d < dk) st[(int64_t)d * dv + col0 + 32 * c] = S[r][c];
    }
}

// out[t] = x[t] / sqrt(mean(x[t]^2) + eps) * weight * sigmoid(gate[t]) * out_scale; x fp32 [T, n].  One CTA per token.
template <typename T>
__global__ void __launch_bounds__(256) gated_rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ weight,
                                                            const T* __restrict__ gate, int64_t gate_stride, float eps,
                                                            float out_scale, T* __restrict__ out, int64_t out_stride, int n) {
    __shared__ float red[32];
    const int64_t t = blockIdx.x;
    const float* xr = x + t * n;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss += xr[i] * xr[i];
    const float f = out_scale / sqrtf(block_sum(ss, red) / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float y = xr[i] * f * weight[i];
        if (gate != nullptr) y *= sigmoid_f(ldf(gate + t * gate_stride + i));
        stf(out + t * out_stride + i, y);
    }
}

template <typename T, int R, int CPT, bool ASYNC>
static void launch_linear_attention_as(const void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v,
                                       int64_t v_stride, const void* decay, void* state, const void* seg_starts, const void* seq_ids,
                                       const void* tok_pos, void* out, int num_segs, int H, int dk, int dv, cudaStream_t stream) {
    static unsigned long long attr_mask = 0;
    auto kern = linear_attention_kernel<T, R, CPT, ASYNC>;
    if (first_use_on_this_device(attr_mask)) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    constexpr int DKP = LA_WARPS * R, COLS = 32 * CPT;
    size_t smem = sizeof(float) * (2 * LA_TOKENS * DKP + LA_TOKENS * COLS + LA_WARPS * LA_TOKENS * COLS + 2 * LA_TOKENS);
    if (ASYNC) smem += sizeof(T) * (size_t)LA_TOKENS * (2 * dk + COLS);
    kern<<<dim3((unsigned)num_segs, (unsigned)H, (unsigned)cdiv(dv, COLS)), LA_WARPS * 32, smem, stream>>>(
        (const T*)q, q_stride, (const T*)k, k_stride, (const T*)v, v_stride, (const float*)decay, (float*)state,
        (const int*)seg_starts, (const int*)seq_ids, (const int*)tok_pos, (float*)out, H, dk, dv);
}

template <typename T>
static int launch_linear_attention(const void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v, int64_t v_stride,
                                   const void* decay, void* state, const void* seg_starts, const void* seq_ids, const void* tok_pos,
                                   void* out, int num_segs, int H, int dk, int dv, cudaStream_t stream) {
    const int rows = cdiv(dk, LA_WARPS);                                // state rows per warp, rounded up to 4, 8, 16, 32 or 64
    // cp.async moves 16-byte pieces: every head's row of q, k and v must start on a 16-byte boundary and be whole pieces
    const int piece = 16 / (int)sizeof(T);
    const bool aligned = dk % piece == 0 && dv % piece == 0 && q_stride % piece == 0 && k_stride % piece == 0 &&
                         v_stride % piece == 0 && (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15) == 0;
    // columns per thread (CPT): more columns make every broadcast read of k and q serve more multiply-adds, but leave fewer
    // CTAs; take the widest slice that still gives every SM a CTA (R * CPT state registers and the shared memory allowing)
    int num_sms = 0;
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, current_device());
    int cpt = 1;
    const int64_t units = (int64_t)num_segs * H;
    if (dv > 64 && units * cdiv(dv, 128) >= num_sms) cpt = 4;
    else if (dv > 32 && units * cdiv(dv, 64) >= num_sms) cpt = 2;
#define LA(R, CPT)                                                                                                             \
    do {                                                                                                                       \
        if (aligned) launch_linear_attention_as<T, R, CPT, true>(q, q_stride, k, k_stride, v, v_stride, decay, state, seg_starts, \
                                                                 seq_ids, tok_pos, out, num_segs, H, dk, dv, stream);           \
        else launch_linear_attention_as<T, R, CPT, false>(q, q_stride, k, k_stride, v, v_stride, decay, state, seg_starts,       \
                                                          seq_ids, tok_pos, out, num_segs, H, dk, dv, stream);                  \
    } while (0)
#define LA_BY_CPT(R, MAXC)                                                                                                     \
    do { if (cpt >= 4 && MAXC >= 4) LA(R, (MAXC >= 4 ? 4 : MAXC)); else if (cpt >= 2 && MAXC >= 2) LA(R, 2); else LA(R, 1); } while (0)
    if (rows <= 4) LA_BY_CPT(4, 4);
    else if (rows <= 8) LA_BY_CPT(8, 4);
    else if (rows <= 16) LA_BY_CPT(16, 4);
    else if (rows <= 32) LA_BY_CPT(32, 2);
    else LA_BY_CPT(64, 1);
#undef LA_BY_CPT
#undef LA
    return check_launch("linear_attention");
}

}  // namespace sllm

using namespace sllm;

extern "C" {

int sllm_causal_conv(const void* xin, int64_t xin_stride, const void* w, const void* bias, const void* tail, const void* tok_seq,
                     const void* tok_pos, void* u, int64_t num_tokens, int64_t num_prefill_tokens, int channels, int taps,
                     sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && channels > 0 && taps >= 1 && taps <= CONV_MAX_TAPS, "causal_conv: 1 <= taps <= %d (got %d)",
                 CONV_MAX_TAPS, taps);
    SLLM_REQUIRE(num_prefill_tokens >= 0 && num_prefill_tokens <= num_tokens, "causal_conv: bad number of prompt rows");
    if (num_tokens == 0) return 0;
    SLLM_REQUIRE(xin && w && tok_seq && tok_pos && u && (taps == 1 || tail), "causal_conv: null pointer");
    if (num_prefill_tokens > 0) {
        const dim3 grid((unsigned)cdiv(num_prefill_tokens, 16), (unsigned)cdiv(channels, 128));
        SLLM_DISPATCH_DTYPE_F32(dtype, (causal_conv_kernel<T, 16><<<grid, 128, 0, (cudaStream_t)stream>>>(
            (const T*)xin, xin_stride, (const T*)w, (const T*)bias, (const T*)tail, (const int*)tok_seq, (const int*)tok_pos, (T*)u,
            (int64_t)0, num_prefill_tokens, channels, taps)));
        if (check_launch("causal_conv (prompt portions)")) return 1;
    }
    if (num_tokens > num_prefill_tokens) {
        const dim3 grid((unsigned)(num_tokens - num_prefill_tokens), (unsigned)cdiv(channels, 128));
        SLLM_DISPATCH_DTYPE_F32(dtype, (causal_conv_kernel<T, 1><<<grid, 128, 0, (cudaStream_t)stream>>>(
            (const T*)xin, xin_stride, (const T*)w, (const T*)bias, (const T*)tail, (const int*)tok_seq, (const int*)tok_pos, (T*)u,
            num_prefill_tokens, num_tokens, channels, taps)));
    }
    return check_launch("causal_conv");
}

int sllm_rglru_scan(const void* u, const void* gates, int blocks, const void* ybr, int64_t y_stride, const void* rate,
                    const void* xin, int64_t xin_stride, void* state, void* tail, const void* seg_starts, const void* seq_ids,
                    const void* tok_pos, void* out, int64_t num_tokens, int num_segs, int num_prefill_segs, int channels, int taps,
                    sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && num_segs >= 0 && channels > 0 && blocks > 0 && channels % blocks == 0 && taps >= 1 &&
                 taps <= CONV_MAX_TAPS, "rglru_scan: bad shape (channels %d in %d blocks, %d taps)", channels, blocks, taps);
    SLLM_REQUIRE(num_prefill_segs >= 0 && num_prefill_segs <= num_segs, "rglru_scan: %d prompt segments of %d", num_prefill_segs,
                 num_segs);
    if (num_tokens == 0 || num_segs == 0) return 0;
    SLLM_REQUIRE(u && gates && ybr && rate && xin && state && (taps == 1 || tail) && seg_starts && seq_ids && tok_pos && out,
                 "rglru_scan: null pointer");
    // prompt portions (the first segments): parallel over time; single decoded tokens: one thread per channel
    if (num_prefill_segs > 0) {
        const dim3 grid((unsigned)num_prefill_segs, (unsigned)cdiv(channels, 32));
        SLLM_DISPATCH_DTYPE_F32(dtype, (rglru_scan_tiled_kernel<T, 8><<<grid, SCAN_WARPS * 32, 0, (cudaStream_t)stream>>>(
            (const T*)u, (const T*)gates, channels / blocks, (const T*)ybr, y_stride, (const float*)rate, (const T*)xin, xin_stride,
            (float*)state, (T*)tail, (const int*)seg_starts, (const int*)seq_ids, (const int*)tok_pos, (T*)out, num_tokens,
            channels, taps)));
        if (check_launch("rglru_scan (prompt portions)")) return 1;
    }
    if (num_segs > num_prefill_segs) {
        const dim3 grid((unsigned)(num_segs - num_prefill_segs), (unsigned)cdiv(channels, 128));
        SLLM_DISPATCH_DTYPE_F32(dtype, (rglru_scan_kernel<T><<<grid, 128, 0, (cudaStream_t)stream>>>(
            (const T*)u, (const T*)gates, channels / blocks, (const T*)ybr, y_stride, (const float*)rate, (const T*)xin, xin_stride,
            (float*)state, (T*)tail, (const int*)seg_starts + num_prefill_segs, (const int*)seq_ids + num_prefill_segs,
            (const int*)tok_pos, (T*)out, num_tokens, channels, taps)));
    }
    return check_launch("rglru_scan");
}

int sllm_linear_attention(const void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v, int64_t v_stride,
                          const void* decay, void* state, const void* seg_starts, const void* seq_ids, const void* tok_pos,
                          void* out, int num_segs, int num_heads, int dk, int dv, sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(num_segs >= 0 && num_heads > 0 && dk > 0 && dv > 0 && dk <= 64 * LA_WARPS && cdiv(dv, 32) <= 65535,
                 "linear_attention: bad shape (dk %d <= %d, dv %d)", dk, 64 * LA_WARPS, dv);
    if (num_segs == 0) return 0;
    SLLM_REQUIRE(q && k && v && decay && state && seg_starts && seq_ids && tok_pos && out, "linear_attention: null pointer");
    SLLM_DISPATCH_DTYPE_F32(dtype, return (launch_linear_attention<T>(q, q_stride, k, k_stride, v, v_stride, decay, state, seg_starts,
                                                                       seq_ids, tok_pos, out, num_segs, num_heads, dk, dv,
                                                                       (cudaStream_t)stream)));
    return 0;
}

int sllm_gated_rmsnorm(const void* x, const void* weight, const void* gate, int64_t gate_stride, float eps, float out_scale,
                       void* out, int64_t out_stride, int64_t num_tokens, int n, sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && n > 0, "gated_rmsnorm: bad shape");
    if (num_tokens == 0) return 0;
    SLLM_REQUIRE(x && weight && out, "gated_rmsnorm: null pointer");
    SLLM_DISPATCH_DTYPE_F32(dtype, (gated_rmsnorm_kernel<T><<<(unsigned)num_tokens, 256, 0, (cudaStream_t)stream>>>(
        (const float*)x, (const float*)weight, (const T*)gate, gate_stride, eps, out_scale, (T*)out, out_stride, n)));
    return check_launch("gated_rmsnorm");
}

}  // extern "C"
