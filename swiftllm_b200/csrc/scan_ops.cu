// Per-channel recurrences over a sequence with per-SEQUENCE state (row `seq` of a state tensor: the sequence's block-table row),
// carried from step to step.  A step brings SEGMENTS: rows seg_starts[b] .. seg_starts[b+1] - 1 of the packed batch are
// consecutive positions of sequence seq_ids[b] (a prompt portion, or one decoded token).  A segment that starts at position 0
// starts from the zero state whatever its row of the state tensor holds (rows are used again without being cleared).
//
//   short_conv         out[t, c] = act(b[c] + sum_k w[c, K-1-k] * x[t-k, c]) (+ x[t, c]); inputs before the segment come from the
//                      sequence's tail (its last K-1 inputs), inputs before position 0 are zero.  Input fp32 or T, output T.
//   conv_tail_update   moves a sequence's tail on by the segment's inputs (runs after every reader of the old tail); a decoded
//                      token's row is the only reader and writer of its sequence's tail, so short_conv moves that tail on itself
//   mingru_scan        z = sigmoid(zl); c = u + 1/2 (u >= 0) | sigmoid(u) (u < 0); S <- (1 - z) S + z c; out = S * silu(g)
//   selective_scan     dt = softplus(dtl + bias); S[c, n] <- exp(dt A[c, n]) S[c, n] + dt x B[n]; y = sum_n S C[n] + D x;
//                      out = y * silu(z)
// Gates, step sizes, decays and the states run in fp32 for every storage type T of the projections.
#include "typed_io.cuh"

namespace sllm {

constexpr int SC_MAX_TAPS = 8;

__device__ __forceinline__ float sigmoid_fn(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float silu_fn(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_fn(float z) { return z > 20.f ? z : log1pf(expf(z)); }
// 2^x for x <= 0 on the special-function unit (relative error about 2^-22; results below the normal range become 0)
__device__ __forceinline__ float exp2_neg(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float cvt_f(float v) { return v; }
__device__ __forceinline__ float cvt_f(__half v) { return __half2float(v); }
__device__ __forceinline__ float cvt_f(__nv_bfloat16 v) { return __bfloat162float(v); }

// grid (ceil(rows / TOKENS), ceil(C / 128)).  tail: TI [rows, K-1, C] (slot i: the input K-1-i positions before the next one).
// A thread walks TOKENS consecutive rows of one channel with the last K-1 inputs in registers; where a row does not continue the
// row above (another sequence, or the tile's first row) the window is filled again: from the rows above as far as they are the
// sequence's previous positions, from the sequence's tail before that, zeros before position 0.
// TOKENS = 1 with move_tail: every row is a one-token segment of its own sequence; its thread then writes the sequence's new tail.
template <typename TI, typename TO, int TOKENS>
__global__ void __launch_bounds__(128) short_conv_kernel(const TI* __restrict__ xin, int64_t xin_stride, const float* __restrict__ w,
                                                         const float* __restrict__ bias, TI* tail,
                                                         const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                                         TO* __restrict__ out, int64_t row0, int64_t row_end, int C, int K,
                                                         int add_input, int act_silu, int move_tail) {
    const int64_t tile0 = row0 + (int64_t)blockIdx.x * TOKENS;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float wk[SC_MAX_TAPS], hist[SC_MAX_TAPS];           // wk[k]: weight of the input k positions back; hist[k - 1]: that input
#pragma unroll
    for (int k = 0; k < SC_MAX_TAPS; k++) { wk[k] = k < K ? w[(int64_t)c * K + (K - 1 - k)] : 0.f; hist[k] = 0.f; }
    const float b0 = bias != nullptr ? bias[c] : 0.f;
    const int nrows = (int)min((int64_t)TOKENS, row_end - tile0);
    float xv[TOKENS];
#pragma unroll
    for (int i = 0; i < TOKENS; i++) xv[i] = i < nrows ? ldf(xin + (tile0 + i) * xin_stride + c) : 0.f;
    int prev_seq = -1, prev_pos = -2;
#pragma unroll
    for (int i = 0; i < TOKENS; i++) {
        if (i >= nrows) break;
        const int64_t t = tile0 + i;
        const int seq = tok_seq[t], pos = tok_pos[t];
        if (i == 0 || seq != prev_seq || pos != prev_pos + 1) {
            int above = 0;                              // rows above this one that are the sequence's previous positions
            while (above < K - 1 && t - above - 1 >= 0 && tok_seq[t - above - 1] == seq && tok_pos[t - above - 1] == pos - above - 1) above++;
#pragma unroll
            for (int k = 1; k < SC_MAX_TAPS; k++) {
                float v = 0.f;
                if (k < K && pos - k >= 0)
                    v = k <= above ? ldf(xin + (t - k) * xin_stride + c)
                                   : ldf(tail + ((int64_t)seq * (K - 1) + (K - 1 - (k - above))) * C + c);
                hist[k - 1] = v;
            }
        }
        float acc = b0 + wk[0] * xv[i];
#pragma unroll
        for (int k = 1; k < SC_MAX_TAPS; k++) acc += wk[k] * hist[k - 1];
        if (act_silu) acc = silu_fn(acc);
        if (add_input) acc += xv[i];
        stf(out + t * C + c, acc);
#pragma unroll
        for (int k = SC_MAX_TAPS - 1; k >= 1; k--) hist[k] = hist[k - 1];
        hist[0] = xv[i];
        prev_seq = seq; prev_pos = pos;
        if (TOKENS == 1 && move_tail) {                 // slot i <- the input K - 2 - i positions back (zeros before position 0)
            TI* tl = tail + (int64_t)seq * (K - 1) * C + c;
#pragma unroll
            for (int k = 0; k < SC_MAX_TAPS - 1; k++)
                if (k < K - 1) stf(tl + (int64_t)(K - 2 - k) * C, hist[k]);
        }
    }
}

// One thread per (segment, channel): tail slot i <- the input at position p0 + n - (K-1) + i, taken from the segment's rows, from
// the old tail, or zero before position 0.
template <typename TI>
__global__ void __launch_bounds__(128) conv_tail_update_kernel(const TI* __restrict__ xin, int64_t xin_stride, TI* __restrict__ tail,
                                                               const int* __restrict__ seg_starts, const int* __restrict__ seq_ids,
                                                               const int* __restrict__ tok_pos, int C, int K) {
    const int b = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int t0 = seg_starts[b], n = seg_starts[b + 1] - t0;
    if (c >= C || n <= 0) return;
    const int seq = seq_ids[b], p0 = tok_pos[t0];
    float old[SC_MAX_TAPS];
    TI* tl = tail + (int64_t)seq * (K - 1) * C + c;
    for (int i = 0; i < K - 1; i++) old[i] = p0 > 0 ? ldf(tl + (int64_t)i * C) : 0.f;
    for (int i = 0; i < K - 1; i++) {
        const int rel = n - (K - 1) + i;                // position relative to the segment's start
        float v = 0.f;
        if (rel >= 0) v = ldf(xin + (int64_t)(t0 + rel) * xin_stride + c);
        else if (p0 + rel >= 0) v = old[rel + K - 1];
        stf(tl + (int64_t)i * C, v);
    }
}

// grid (segments, ceil(C / 128)): one thread per (segment, channel) walks the segment's rows.
// proj: [T, >= 3 C] rows [z logits | candidate pre-activations | output-gate pre-activations] (biases already added).
template <typename T>
__global__ void __launch_bounds__(128) mingru_scan_kernel(const T* __restrict__ proj, int64_t stride, float* __restrict__ state,
                                                          const int* __restrict__ seg_starts, const int* __restrict__ seq_ids,
                                                          const int* __restrict__ tok_pos, T* __restrict__ out, int C) {
    const int b = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int t0 = seg_starts[b], n = seg_starts[b + 1] - t0;
    if (c >= C || n <= 0) return;
    const int seq = seq_ids[b];
    float S = tok_pos[t0] > 0 ? state[(int64_t)seq * C + c] : 0.f;
    const T* pr = proj + (int64_t)t0 * stride + c;
    // the loads of the next row are issued before this row's arithmetic
    float zl = ldf(pr), u = ldf(pr + C), g = ldf(pr + 2 * C);
    for (int i = 0; i < n; i++) {
        float zl2 = 0.f, u2 = 0.f, g2 = 0.f;
        if (i + 1 < n) {
            const T* nx = pr + (int64_t)(i + 1) * stride;
            zl2 = ldf(nx); u2 = ldf(nx + C); g2 = ldf(nx + 2 * C);
        }
        const float z = sigmoid_fn(zl);
        const float cand = u >= 0.f ? u + 0.5f : sigmoid_fn(u);
        S = (1.f - z) * S + z * cand;
        stf(out + (int64_t)(t0 + i) * C + c, S * silu_fn(g));
        zl = zl2; u = u2; g = g2;
    }
    state[(int64_t)seq * C + c] = S;
}

// The same recurrence for PROMPT PORTIONS, parallel over time as well: grid (segments, ceil(C / 32)), 8 warps.  Lane: channel;
// warp w: tokens 8 w .. 8 w + 7 of the current tile of 64 tokens.  Every thread turns its tokens' logits into the pairs (a, b) of
// S -> a S + b (all loads of a run are issued before its sigmoids), composes its run into one such map, the eight maps of a tile
// meet in shared memory, every warp takes the state at its run's start from the maps before it and replays its run.
template <typename T>
__global__ void __launch_bounds__(256) mingru_scan_tiled_kernel(const T* __restrict__ proj, int64_t stride, float* __restrict__ state,
                                                                const int* __restrict__ seg_starts, const int* __restrict__ seq_ids,
                                                                const int* __restrict__ tok_pos, T* __restrict__ out, int C) {
    __shared__ float sa[8][32], sb[8][32], s0[32];
    const int b = blockIdx.x, lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int c = blockIdx.y * 32 + lane;
    const int t0 = seg_starts[b], n = seg_starts[b + 1] - t0;
    if (n <= 0) return;                                 // the whole CTA
    const bool live = c < C;
    const int seq = seq_ids[b];
    if (w == 0) s0[lane] = (live && tok_pos[t0] > 0) ? state[(int64_t)seq * C + c] : 0.f;
    float S = 0.f;
    for (int tile0 = 0; tile0 < n; tile0 += 64) {
        const int j0 = tile0 + w * 8;
        float a[8], bb[8], g[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {                   // raw logits first: 24 loads in flight
            const bool ok = live && j0 + j < n;
            const T* pr = proj + (int64_t)(t0 + j0 + j) * stride + c;
            a[j] = ok ? ldf(pr) : 0.f;
            bb[j] = ok ? ldf(pr + C) : 0.f;
            g[j] = ok ? ldf(pr + 2 * C) : 0.f;
        }
        float A = 1.f, B = 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            if (live && j0 + j < n) {
                const float z = sigmoid_fn(a[j]), u = bb[j];
                a[j] = 1.f - z;
                bb[j] = z * (u >= 0.f ? u + 0.5f : sigmoid_fn(u));
                g[j] = silu_fn(g[j]);
            } else {
                a[j] = 1.f; bb[j] = 0.f;                // past the segment's end: the identity map
            }
            B = a[j] * B + bb[j];
            A *= a[j];
        }
        sa[w][lane] = A; sb[w][lane] = B;
        __syncthreads();
        S = s0[lane];
        for (int k = 0; k < w; k++) S = sa[k][lane] * S + sb[k][lane];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            S = a[j] * S + bb[j];
            if (live && j0 + j < n) stf(out + (int64_t)(t0 + j0 + j) * C + c, S * g[j]);
        }
        __syncthreads();                                // s0 and the maps have been read
        if (w == 7) s0[lane] = S;                       // the tile's last run ends at the tile's end state
    }
    if (w == 7 && live) state[(int64_t)seq * C + c] = S;
}

// Block: 128 threads = (128 / NS) channels x NS lanes per channel; lane s of a channel holds the RE = ceil(N / NS) <= SS_R
// consecutive states n = s RE + r of its channel in registers.  grid (segments, ceil(C / (128 / NS))).  x, z: T [T, C] (row strides); dtl: TD [T, C] step logits (without
// bias); bc: T [T, ...] rows with B at column b_off and C at column c_off (N each); A fp32 [C, N] (negative); state fp32
// [rows, C, N].
constexpr int SS_R = 8;

template <typename T, typename TD>
__global__ void __launch_bounds__(128) selective_scan_kernel(
    const T* __restrict__ x, int64_t x_stride, const TD* __restrict__ dtl, int64_t dt_stride, const float* __restrict__ dt_bias,
    const float* __restrict__ A, const T* __restrict__ bc, int64_t bc_stride, int b_off, int c_off, const float* __restrict__ D,
    const T* __restrict__ z, int64_t z_stride, float* __restrict__ state, const int* __restrict__ seg_starts,
    const int* __restrict__ seq_ids, const int* __restrict__ tok_pos, T* __restrict__ out, int C, int N, int ns_log2) {
    const int NS = 1 << ns_log2, RE = (N + NS - 1) >> ns_log2;
    const int b = blockIdx.x;
    const int s = threadIdx.x & (NS - 1);
    const int c = blockIdx.y * (blockDim.x >> ns_log2) + (threadIdx.x >> ns_log2);
    const int t0 = seg_starts[b], n = seg_starts[b + 1] - t0;
    if (n <= 0) return;
    const bool live = c < C;                            // dead threads still take part in the shuffles
    const int cc = live ? c : 0;
    const int seq = seq_ids[b];
    const bool fresh = tok_pos[t0] == 0;
    float S[SS_R], a[SS_R];
    float* sp = state + ((int64_t)seq * C + cc) * N;
#pragma unroll
    for (int r = 0; r < SS_R; r++) {
        const int k = s * RE + r;
        const bool ok = r < RE && k < N;
        a[r] = ok ? A[(int64_t)cc * N + k] * 1.4426950408889634f : 0.f;       // exp(dt A) = 2^(dt A log2 e)
        S[r] = (ok && !fresh) ? sp[k] : 0.f;
    }
    const float bias = dt_bias[cc], dd = D[cc];
    for (int i = 0; i < n; i++) {
        const int64_t t = t0 + i;
        const float dt = softplus_fn(ldf(dtl + t * dt_stride + cc) + bias);
        const float xv = ldf(x + t * x_stride + cc);
        const float dx = dt * xv;
        const T* br = bc + t * bc_stride;
        float y = 0.f;
#pragma unroll
        for (int r = 0; r < SS_R; r++) {
            const int k = s * RE + r;
            if (r < RE && k < N) {
                S[r] = exp2_neg(dt * a[r]) * S[r] + dx * ldf(br + b_off + k);
                y += S[r] * ldf(br + c_off + k);
            }
        }
        for (int o = NS >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
        if (s == 0 && live) stf(out + t * C + c, (y + dd * xv) * silu_fn(ldf(z + t * z_stride + c)));
    }
    if (live) {
#pragma unroll
        for (int r = 0; r < SS_R; r++) {
            const int k = s * RE + r;
            if (r < RE && k < N) sp[k] = S[r];
        }
    }
}

// The same scan for PROMPT PORTIONS with staged tiles of `tt` tokens (tt * (128 / NS) <= 128 SS_ITEMS: 8 tokens for NS = 1, 16 for
// NS = 2, 32 from NS = 4 on, fewer when the B / C rows of very wide states would not fit): all threads first bring the tile's x, step sizes (softplus
// applied), SiLU gates and B / C rows into shared memory with coalesced loads (one exposed load latency per tile instead of one
// per token), the sequential part then reads shared memory only, and the tile's outputs leave coalesced.  The raw values of the
// NEXT tile are loaded into registers before the sequential part of the current one and are only touched after it, so their
// latency hides behind the arithmetic (B / C rows: the first SS_BCR x 128 entries of a tile; wider states load the rest when
// they stage).  Same thread layout, same arithmetic per step.  Dynamic shared memory: (4 tt (128 / NS) + 2 tt N) floats.
constexpr int SS_ITEMS = 8;
constexpr int SS_BCR = 4;

template <typename T, typename TD>
__global__ void __launch_bounds__(128) selective_scan_tiled_kernel(
    const T* __restrict__ x, int64_t x_stride, const TD* __restrict__ dtl, int64_t dt_stride, const float* __restrict__ dt_bias,
    const float* __restrict__ A, const T* __restrict__ bc, int64_t bc_stride, int b_off, int c_off, const float* __restrict__ D,
    const T* __restrict__ z, int64_t z_stride, float* __restrict__ state, const int* __restrict__ seg_starts,
    const int* __restrict__ seq_ids, const int* __restrict__ tok_pos, T* __restrict__ out, int C, int N, int ns_log2, int tt) {
    extern __shared__ __align__(16) float ssm[];
    const int NS = 1 << ns_log2, ch_log2 = 7 - ns_log2, CH = 1 << ch_log2, RE = (N + NS - 1) >> ns_log2;
    // whole groups of four states per lane, on 16-byte boundaries of the staged rows: B and C are read four at a time
    const bool vec = (N & 3) == 0 && (RE & 3) == 0;
    float* xs = ssm;                                    // [tt][CH]
    float* ds = xs + tt * CH;
    float* zs = ds + tt * CH;
    float* ys = zs + tt * CH;
    float* bs = ys + tt * CH;                           // [tt][N]
    float* cs = bs + tt * N;
    const int b = blockIdx.x, tid = threadIdx.x;
    const int s = tid & (NS - 1), cl = tid >> ns_log2;
    const int cbase = blockIdx.y * CH, c = cbase + cl;
    const int t0 = seg_starts[b], n = seg_starts[b + 1] - t0;
    if (n <= 0) return;
    const bool live = c < C;
    const int cc = live ? c : 0;
    const int seq = seq_ids[b];
    const bool fresh = tok_pos[t0] == 0;
    float S[SS_R], a[SS_R];
    float* sp = state + ((int64_t)seq * C + cc) * N;
#pragma unroll
    for (int r = 0; r < SS_R; r++) {
        const int k = s * RE + r;
        const bool ok = r < RE && k < N;
        a[r] = ok ? A[(int64_t)cc * N + k] * 1.4426950408889634f : 0.f;       // exp(dt A) = 2^(dt A log2 e)
        S[r] = (ok && !fresh) ? sp[k] : 0.f;
    }
    const float dd = D[cc];
    // item i of a thread: entry tid + 128 i of the tile.  Kept as loaded: a conversion right behind a load would make the warp wait
    // for it before the sequential part instead of after
    T rx[SS_ITEMS], rz[SS_ITEMS], rb[SS_BCR], rc[SS_BCR];
    TD rd[SS_ITEMS];
    auto fetch = [&](int tile0) {
        const int nt = min(tt, n - tile0);                              // <= 0 past the end: nothing is loaded
        const int64_t tb = t0 + tile0;
#pragma unroll
        for (int i = 0; i < SS_ITEMS; i++) {
            const int idx = tid + 128 * i, j = idx >> ch_log2, cg = cbase + (idx & (CH - 1));
            if (idx < (nt << ch_log2) && cg < C) {
                rx[i] = x[(tb + j) * x_stride + cg];
                rd[i] = dtl[(tb + j) * dt_stride + cg];
                rz[i] = z[(tb + j) * z_stride + cg];
            }
        }
#pragma unroll
        for (int i = 0; i < SS_BCR; i++) {
            const int idx = tid + 128 * i;
            if (idx < nt * N) {
                const int j = idx / N, k = idx - j * N;
                const T* br = bc + (tb + j) * bc_stride;
                rb[i] = br[b_off + k];
                rc[i] = br[c_off + k];
            }
        }
    };
    fetch(0);
    for (int tile0 = 0; tile0 < n; tile0 += tt) {
        const int nt = min(tt, n - tile0);
        const int64_t tb = t0 + tile0;
#pragma unroll
        for (int i = 0; i < SS_ITEMS; i++) {
            const int idx = tid + 128 * i, cg = cbase + (idx & (CH - 1));
            if (idx < (nt << ch_log2) && cg < C) {
                xs[idx] = cvt_f(rx[i]);
                ds[idx] = softplus_fn(cvt_f(rd[i]) + dt_bias[cg]);
                zs[idx] = silu_fn(cvt_f(rz[i]));
            }
        }
#pragma unroll
        for (int i = 0; i < SS_BCR; i++) {
            const int idx = tid + 128 * i;
            if (idx < nt * N) { bs[idx] = cvt_f(rb[i]); cs[idx] = cvt_f(rc[i]); }
        }
        for (int idx = tid + 128 * SS_BCR; idx < nt * N; idx += 128) {
            const int j = idx / N, k = idx - j * N;
            const T* br = bc + (tb + j) * bc_stride;
            bs[idx] = ldf(br + b_off + k);
            cs[idx] = ldf(br + c_off + k);
        }
        __syncthreads();
        fetch(tile0 + tt);                              // in flight during the sequential part below
        const float* bp = bs + s * RE;
        const float* cp = cs + s * RE;
        const bool lane_live = s * RE < N;
        for (int j = 0; j < nt; j++, bp += N, cp += N) {
            const float dt = ds[(j << ch_log2) + cl], xv = xs[(j << ch_log2) + cl];
            const float dx = dt * xv;
            float y = 0.f;
            if (vec) {
#pragma unroll
                for (int q = 0; q < SS_R / 4; q++) {
                    if (4 * q < RE && lane_live) {
                        const float4 b4 = reinterpret_cast<const float4*>(bp)[q], c4 = reinterpret_cast<const float4*>(cp)[q];
                        S[4 * q + 0] = exp2_neg(dt * a[4 * q + 0]) * S[4 * q + 0] + dx * b4.x;
                        S[4 * q + 1] = exp2_neg(dt * a[4 * q + 1]) * S[4 * q + 1] + dx * b4.y;
                        S[4 * q + 2] = exp2_neg(dt * a[4 * q + 2]) * S[4 * q + 2] + dx * b4.z;
                        S[4 * q + 3] = exp2_neg(dt * a[4 * q + 3]) * S[4 * q + 3] + dx * b4.w;
                        y += S[4 * q + 0] * c4.x + S[4 * q + 1] * c4.y + S[4 * q + 2] * c4.z + S[4 * q + 3] * c4.w;
                    }
                }
            } else {
#pragma unroll
                for (int r = 0; r < SS_R; r++) {
                    if (r < RE && s * RE + r < N) {
                        S[r] = exp2_neg(dt * a[r]) * S[r] + dx * bp[r];
                        y += S[r] * cp[r];
                    }
                }
            }
            for (int o = NS >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
            if (s == 0) ys[(j << ch_log2) + cl] = (y + dd * xv) * zs[(j << ch_log2) + cl];
        }
        __syncthreads();
        for (int idx = tid; idx < (nt << ch_log2); idx += 128) {
            const int j = idx >> ch_log2, cg = cbase + (idx & (CH - 1));
            if (cg < C) stf(out + (tb + j) * C + cg, ys[idx]);
        }
        // the next tile's staging writes xs / ds / zs / bs / cs, which nobody reads any more; ys is written again only after
        // the next barrier
    }
    if (live) {
#pragma unroll
        for (int r = 0; r < SS_R; r++) {
            const int k = s * RE + r;
            if (r < RE && k < N) sp[k] = S[r];
        }
    }
}

}  // namespace sllm

using namespace sllm;

extern "C" {

int sllm_short_conv(const void* xin, int64_t xin_stride, sllm_dtype_t in_dtype, const void* w, const void* bias, const void* tail,
                    const void* tok_seq, const void* tok_pos, void* out, sllm_dtype_t out_dtype, int64_t num_tokens,
                    int64_t num_prefill_tokens, int channels, int taps, int add_input, int act_silu, int move_decode_tails,
                    sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && channels > 0 && taps >= 1 && taps <= SC_MAX_TAPS, "short_conv: 1 <= taps <= %d (got %d)",
                 SC_MAX_TAPS, taps);
    SLLM_REQUIRE(num_prefill_tokens >= 0 && num_prefill_tokens <= num_tokens, "short_conv: bad number of prompt rows");
    SLLM_REQUIRE(in_dtype == out_dtype || in_dtype == SLLM_F32, "short_conv: the input is fp32 or of the output's type");
    if (num_tokens == 0) return 0;
    SLLM_REQUIRE(xin && w && tok_seq && tok_pos && out && (taps == 1 || tail), "short_conv: null pointer");
    const cudaStream_t st = (cudaStream_t)stream;
#define SC_LAUNCH(TI, TOKENS, r0, r1)                                                                                          \
    short_conv_kernel<TI, T, TOKENS><<<dim3((unsigned)cdiv((r1) - (r0), TOKENS), (unsigned)cdiv(channels, 128)), 128, 0, st>>>(   \
        (const TI*)xin, xin_stride, (const float*)w, (const float*)bias, (TI*)tail, (const int*)tok_seq,                        \
        (const int*)tok_pos, (T*)out, (int64_t)(r0), (int64_t)(r1), channels, taps, add_input, act_silu,                        \
        (TOKENS == 1 && move_decode_tails && taps > 1) ? 1 : 0)
    if (num_prefill_tokens > 0) {
        if (in_dtype == SLLM_F32) { SLLM_DISPATCH_DTYPE_F32(out_dtype, (SC_LAUNCH(float, 16, 0, num_prefill_tokens))); }
        else { SLLM_DISPATCH_DTYPE_F32(out_dtype, (SC_LAUNCH(T, 16, 0, num_prefill_tokens))); }
        if (check_launch("short_conv (prompt portions)")) return 1;
    }
    if (num_tokens > num_prefill_tokens) {
        if (in_dtype == SLLM_F32) { SLLM_DISPATCH_DTYPE_F32(out_dtype, (SC_LAUNCH(float, 1, num_prefill_tokens, num_tokens))); }
        else { SLLM_DISPATCH_DTYPE_F32(out_dtype, (SC_LAUNCH(T, 1, num_prefill_tokens, num_tokens))); }
    }
#undef SC_LAUNCH
    return check_launch("short_conv");
}

int sllm_conv_tail_update(const void* xin, int64_t xin_stride, void* tail, const void* seg_starts, const void* seq_ids,
                          const void* tok_pos, int num_segs, int channels, int taps, sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(num_segs >= 0 && channels > 0 && taps >= 1 && taps <= SC_MAX_TAPS, "conv_tail_update: bad shape");
    if (num_segs == 0 || taps == 1) return 0;
    SLLM_REQUIRE(xin && tail && seg_starts && seq_ids && tok_pos, "conv_tail_update: null pointer");
    const dim3 grid((unsigned)num_segs, (unsigned)cdiv(channels, 128));
    SLLM_DISPATCH_DTYPE_F32(dtype, (conv_tail_update_kernel<T><<<grid, 128, 0, (cudaStream_t)stream>>>(
        (const T*)xin, xin_stride, (T*)tail, (const int*)seg_starts, (const int*)seq_ids, (const int*)tok_pos, channels, taps)));
    return check_launch("conv_tail_update");
}

int sllm_mingru_scan(const void* proj, int64_t proj_stride, void* state, const void* seg_starts, const void* seq_ids,
                     const void* tok_pos, void* out, int num_segs, int num_prefill_segs, int channels, sllm_dtype_t dtype,
                     sllm_stream_t stream) {
    SLLM_REQUIRE(num_segs >= 0 && channels > 0 && proj_stride >= 3 * (int64_t)channels, "mingru_scan: bad shape");
    SLLM_REQUIRE(num_prefill_segs >= 0 && num_prefill_segs <= num_segs, "mingru_scan: bad number of prompt segments");
    if (num_segs == 0) return 0;
    SLLM_REQUIRE(proj && state && seg_starts && seq_ids && tok_pos && out, "mingru_scan: null pointer");
    if (num_prefill_segs > 0) {
        const dim3 grid((unsigned)num_prefill_segs, (unsigned)cdiv(channels, 32));
        SLLM_DISPATCH_DTYPE_F32(dtype, (mingru_scan_tiled_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>(
            (const T*)proj, proj_stride, (float*)state, (const int*)seg_starts, (const int*)seq_ids, (const int*)tok_pos, (T*)out,
            channels)));
        if (check_launch("mingru_scan (prompt portions)")) return 1;
    }
    if (num_segs > num_prefill_segs) {
        const dim3 grid((unsigned)(num_segs - num_prefill_segs), (unsigned)cdiv(channels, 128));
        SLLM_DISPATCH_DTYPE_F32(dtype, (mingru_scan_kernel<T><<<grid, 128, 0, (cudaStream_t)stream>>>(
            (const T*)proj, proj_stride, (float*)state, (const int*)seg_starts + num_prefill_segs,
            (const int*)seq_ids + num_prefill_segs, (const int*)tok_pos, (T*)out, channels)));
    }
    return check_launch("mingru_scan");
}

int sllm_selective_scan(const void* x, int64_t x_stride, const void* dt, int64_t dt_stride, int dt_f32, const void* dt_bias,
                        const void* A, const void* bc, int64_t bc_stride, int b_off, int c_off, const void* D, const void* z,
                        int64_t z_stride, void* state, const void* seg_starts, const void* seq_ids, const void* tok_pos, void* out,
                        int num_segs, int num_prefill_segs, int channels, int states, sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(num_prefill_segs >= 0 && num_prefill_segs <= num_segs, "selective_scan: bad number of prompt segments");
    SLLM_REQUIRE(num_segs >= 0 && channels > 0 && states > 0 && states <= 32 * SS_R, "selective_scan: 1 <= states <= %d (got %d)",
                 32 * SS_R, states);
    if (num_segs == 0) return 0;
    SLLM_REQUIRE(x && dt && dt_bias && A && bc && D && z && state && seg_starts && seq_ids && tok_pos && out,
                 "selective_scan: null pointer");
    int ns_plain = 0;                                  // lanes per channel (log2): the fewest that hold all states
    while ((SS_R << ns_plain) < states) ns_plain++;
    int ns_tiled = ns_plain;
    if (num_prefill_segs > 0) {
        // prompt portions walk their tokens one after the other: with few (segment, channel) pairs more lanes per channel (fewer
        // states per thread) put more warps on the SMs
        int sms = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, current_device());
        while (ns_tiled < 5 && (2 << ns_tiled) <= states &&
               (((int64_t)num_prefill_segs * channels) << ns_tiled) / 32 < 8 * (int64_t)sms) ns_tiled++;
    }
    int tt = SS_ITEMS << ns_tiled;                     // tt * (128 >> ns_tiled) = 128 SS_ITEMS entries per staged array ...
    if (tt > 32) tt = 32;
    while (tt > 1 && (size_t)2 * tt * states * sizeof(float) > 24 * 1024) tt >>= 1;                    // ... and B / C rows within 24 KB
    const size_t smem = ((size_t)4 * tt * (128 >> ns_tiled) + (size_t)2 * tt * states) * sizeof(float);   // <= 40 KB
#define SS_GRID(NSEG, NSL) dim3((unsigned)(NSEG), (unsigned)cdiv(channels, 128 >> (NSL))), 128
#define SS_ARGS(TD, SEG0, NSL)                                                                                                 \
    (const T*)x, x_stride, (const TD*)dt, dt_stride, (const float*)dt_bias, (const float*)A, (const T*)bc, bc_stride, b_off,     \
        c_off, (const float*)D, (const T*)z, z_stride, (float*)state, (const int*)seg_starts + (SEG0),                          \
        (const int*)seq_ids + (SEG0), (const int*)tok_pos, (T*)out, channels, states, (NSL)
    const cudaStream_t st = (cudaStream_t)stream;
    if (num_prefill_segs > 0) {
        if (dt_f32) {
            SLLM_DISPATCH_DTYPE_F32(dtype, (selective_scan_tiled_kernel<T, float><<<SS_GRID(num_prefill_segs, ns_tiled), smem, st>>>(
                SS_ARGS(float, 0, ns_tiled), tt)));
        } else {
            SLLM_DISPATCH_DTYPE_F32(dtype, (selective_scan_tiled_kernel<T, T><<<SS_GRID(num_prefill_segs, ns_tiled), smem, st>>>(
                SS_ARGS(T, 0, ns_tiled), tt)));
        }
        if (check_launch("selective_scan (prompt portions)")) return 1;
    }
    if (num_segs > num_prefill_segs) {
        const int rest = num_segs - num_prefill_segs;
        if (dt_f32) {
            SLLM_DISPATCH_DTYPE_F32(dtype, (selective_scan_kernel<T, float><<<SS_GRID(rest, ns_plain), 0, st>>>(
                SS_ARGS(float, num_prefill_segs, ns_plain))));
        } else {
            SLLM_DISPATCH_DTYPE_F32(dtype, (selective_scan_kernel<T, T><<<SS_GRID(rest, ns_plain), 0, st>>>(
                SS_ARGS(T, num_prefill_segs, ns_plain))));
        }
    }
#undef SS_ARGS
#undef SS_GRID
    return check_launch("selective_scan");
}

}  // extern "C"
