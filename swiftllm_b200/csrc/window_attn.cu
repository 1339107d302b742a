// Gated sliding-window attention with grouped key/value heads and an optional softmax sink, over a paged cache that holds per
// token and layer ONE row [ k (G heads x dk, rotary applied) | v (G heads x dv) ].
//   score(i, j) = rope(q[i,h]) . k[j, g(h)] * scale          g(h) = h / (H / G)
//   p(i, j)     = exp(score) / (sink + sum_j' exp(score))     sink = 1 when the softmax has a value-less sink of score 0, else 0
//   out[i, h]   = sigmoid(gate[i, h, :]) * sum_j p(i, j) v[j, g(h)]          (element-wise gate; no gate when null)
// Every token of the step is a query with its own (block-table row, position): prompt portions and single decoded tokens go
// through the same kernel, so the result at a position does not depend on how its sequence was cut into steps.  A query at
// position p sees the positions max(0, p - window + 1) .. p (window <= 0: all of 0 .. p).  Rotary pairs are interleaved
// ((2i, 2i+1)) or halves ((i, i + rot_dims/2)) of the first rot_dims entries of a head; the rest pass through; the caller's
// cos / sin tables carry the frequencies (and any common factor on both).  Softmax, rotation and the weighted sum of values
// run in fp32 for every storage type.
// Options that other designs use (all off for the plain gated window attention):
//   qk_norm_eps >= 0   rotated queries and keys are divided by sqrt(mean over the head + eps)
//   softcap > 0        score <- softcap * tanh(score / softcap) after the scale
//   vcos / vsin        the value at position j is stored turned by j (pairs (m, m + dv/2) when `halves`, else (2m, 2m+1), angle
//                      tables [T, dv/2]) and the head's output at position i is turned back by -i
//   out_scale          factor on the output (a mixer that is summed with another one folds its weight here)
//   pre-norm weights   queries / keys are RMS-normed over the head (x / sqrt(mean + prenorm_eps) * weight[dk]) BEFORE they turn
//   chunk > 0          a query at position p sees only keys of its own chunk: positions >= floor(p / chunk) * chunk
//   vshare > 1         `vshare` neighbouring key heads share ONE value head (value head = key head / vshare; the cache row holds
//                      G keys and G / vshare values): several score maps over the same values, each its own query head
//   out_f32            the output is written as fp32 whatever the storage type (a combine step follows)
// diff_combine: per token and head, o = a1 - lambda * a2 of two maps' outputs, o / sqrt(mean(o^2) + eps) * factor * sigmoid(gate).
#include "mma_helpers.cuh"
#include "typed_io.cuh"

namespace sllm {

// entry j of a head row x turned by the token's angles (cs / sn: the token's table rows); entries from rot_dims on pass through
// nw: weight of a norm over the head that comes BEFORE the turn (entry j is x[j] * inv * nw[j]), or null
template <typename T>
__device__ __forceinline__ float pre_entry(const T* __restrict__ x, int j, float inv, const float* __restrict__ nw) {
    const float v = ldf(x + j);
    return nw != nullptr ? v * inv * nw[j] : v;
}
template <typename T>
__device__ __forceinline__ float rot_entry(const T* __restrict__ x, int j, int rot_dims, int halves, const float* __restrict__ cs,
                                           const float* __restrict__ sn, float inv = 1.f, const float* __restrict__ nw = nullptr) {
    if (j >= rot_dims) return pre_entry(x, j, inv, nw);
    if (halves) {
        const int half = rot_dims >> 1;
        if (j < half) return pre_entry(x, j, inv, nw) * cs[j] - pre_entry(x, j + half, inv, nw) * sn[j];
        return pre_entry(x, j, inv, nw) * cs[j - half] + pre_entry(x, j - half, inv, nw) * sn[j - half];
    }
    const int i = j >> 1;
    const float a = pre_entry(x, 2 * i, inv, nw), b = pre_entry(x, 2 * i + 1, inv, nw);
    return (j & 1) ? b * cs[i] + a * sn[i] : a * cs[i] - b * sn[i];
}

// ------------------------------------------------------------------ cache store
// One CTA per token, one warp per key/value head at a time: rotate k (and divide it by its root mean square), rotate or copy v,
// write the token's row of cache slot `slot`.
template <typename T>
__global__ void __launch_bounds__(128) window_kv_store_kernel(
    const T* __restrict__ k, int64_t k_stride, const T* __restrict__ v, int64_t v_stride, const float* __restrict__ cosb,
    const float* __restrict__ sinb, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
    const int* __restrict__ block_table, int max_blocks_per_seq, T* __restrict__ cache, int n_slots, int slot, int block_size,
    int G, int dk, int dv, int rot_dims, int halves, float qk_norm_eps, const float* __restrict__ vcos,
    const float* __restrict__ vsin, const float* __restrict__ knorm_w, float prenorm_eps, int vshare) {
    const int64_t t = blockIdx.x;
    const int pos = tok_pos[t];
    const int blk = block_table[(int64_t)tok_seq[t] * max_blocks_per_seq + pos / block_size];
    const int GV = G / vshare;
    const int kw = G * dk, vw = GV * dv;
    T* dst = cache + (((int64_t)blk * n_slots + slot) * block_size + pos % block_size) * (kw + vw);
    const T* kr = k + t * k_stride;
    const T* vr = v + t * v_stride;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const float* cs = cosb != nullptr ? cosb + t * (rot_dims >> 1) : nullptr;
    const float* sn = sinb != nullptr ? sinb + t * (rot_dims >> 1) : nullptr;
    for (int g = warp; g < G; g += nwarps) {
        const T* x = kr + g * dk;
        float pinv = 1.f;
        if (knorm_w != nullptr) {
            float ss = 0.f;
            for (int j = lane; j < dk; j += 32) { const float o = ldf(x + j); ss += o * o; }
            pinv = 1.f / sqrtf(warp_sum(ss) / (float)dk + prenorm_eps);
        }
        float inv = 1.f;
        if (qk_norm_eps >= 0.f) {
            float ss = 0.f;
            for (int j = lane; j < dk; j += 32) { const float o = rot_entry(x, j, rot_dims, halves, cs, sn, pinv, knorm_w); ss += o * o; }
            inv = 1.f / sqrtf(warp_sum(ss) / (float)dk + qk_norm_eps);
        }
        for (int j = lane; j < dk; j += 32) stf(dst + g * dk + j, rot_entry(x, j, rot_dims, halves, cs, sn, pinv, knorm_w) * inv);
        if (g >= GV) continue;                          // value heads: the first G / vshare turns of this loop
        const T* y = vr + g * dv;
        if (vcos != nullptr) {
            const float* vc = vcos + t * (dv >> 1);
            const float* vs = vsin + t * (dv >> 1);
            for (int j = lane; j < dv; j += 32) stf(dst + kw + g * dv + j, rot_entry(y, j, dv, halves, vc, vs));
        } else {
            for (int j = lane; j < dv; j += 32) dst[kw + g * dv + j] = y[j];
        }
    }
}

// ------------------------------------------------------------------ attention (fp32 CUDA cores)
constexpr int WA_TILE = 32;        // keys per tile: one per lane in the score phase
constexpr int WA_MAX_HPB = 8;      // query heads (warps) per CTA: heads of ONE key/value group, they share the staged tile

// grid (tokens, H / hpb), hpb warps; hpb divides H / G.  KR: per-lane accumulator registers, dv <= 32 * KR.
template <typename T, int KR>
__global__ void __launch_bounds__(WA_MAX_HPB * 32) window_attn_kernel(
    const T* __restrict__ q, int64_t q_stride_t,                                 // [T, H, dk] (un-rotated; rotated here)
    const float* __restrict__ cosb, const float* __restrict__ sinb,            // [T, rot_dims / 2]
    const T* __restrict__ gate, int64_t gate_stride_t,                          // [T, H, dv] gate logits, or null
    const T* __restrict__ cache, int n_slots, int slot, int block_size,
    const int* __restrict__ block_table, int max_blocks_per_seq, const int* __restrict__ tok_seq,
    const int* __restrict__ tok_pos, T* __restrict__ out, int64_t out_stride_t,  // [T, H, dv]
    int H, int G, int dk, int dv, int rot_dims, int window, float scale, float sink, int halves, float qk_norm_eps,
    float softcap, const float* __restrict__ vcos, const float* __restrict__ vsin, float out_scale,
    const float* __restrict__ qnorm_w, float prenorm_eps, int chunk, int vshare, int out_f32) {
    extern __shared__ float smem[];
    const int KP = dk + 1;
    const int hpb = blockDim.x >> 5;
    float* qs = smem;                          // [hpb][dk]
    float* kt = qs + hpb * dk;                 // [WA_TILE][dk + 1]
    float* vt = kt + WA_TILE * KP;             // [WA_TILE][dv]
    float* os = vt + WA_TILE * dv;             // [hpb][dv]: the head's output before it is turned back (vcos only)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t t = blockIdx.x;
    const int h = blockIdx.y * hpb + warp;
    const int g = (blockIdx.y * hpb) / (H / G);
    const int pos = tok_pos[t];
    const int* bt = block_table + (int64_t)tok_seq[t] * max_blocks_per_seq;
    const int row = G * dk + (G / vshare) * dv;

    {
        float* qw = qs + warp * dk;
        const T* qr = q + t * q_stride_t + (int64_t)h * dk;
        const float* cs = cosb != nullptr ? cosb + t * (rot_dims >> 1) : nullptr;
        const float* sn = sinb != nullptr ? sinb + t * (rot_dims >> 1) : nullptr;
        float pinv = 1.f;
        if (qnorm_w != nullptr) {
            float s0 = 0.f;
            for (int j = lane; j < dk; j += 32) { const float o = ldf(qr + j); s0 += o * o; }
            pinv = 1.f / sqrtf(warp_sum(s0) / (float)dk + prenorm_eps);
        }
        float ss = 0.f;
        for (int j = lane; j < dk; j += 32) {
            const float o = rot_entry(qr, j, rot_dims, halves, cs, sn, pinv, qnorm_w);
            qw[j] = o;
            ss += o * o;
        }
        const float f = qk_norm_eps >= 0.f ? scale / sqrtf(warp_sum(ss) / (float)dk + qk_norm_eps) : scale;
        for (int j = lane; j < dk; j += 32) qw[j] *= f;            // every lane rescales what it wrote itself
    }

    // a sink takes part in the normalisation only: it enters the running (maximum, sum) as a key of score 0 without a value
    float m = sink > 0.f ? 0.f : -INFINITY, l = sink;
    float acc[KR];
#pragma unroll
    for (int k = 0; k < KR; k++) acc[k] = 0.f;

    int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    if (chunk > 0) lo = max(lo, pos / chunk * chunk);
    for (int base = lo; base <= pos; base += WA_TILE) {
        __syncthreads();                       // the previous tile is no longer read (and qs is written, first time round)
        const int nkeys = min(WA_TILE, pos - base + 1);
        for (int jj = warp; jj < nkeys; jj += hpb) {
            const int kp = base + jj;
            const T* src = cache + (((int64_t)bt[kp / block_size] * n_slots + slot) * block_size + kp % block_size) * row;
            const T* ks = src + g * dk;
            const T* vs = src + G * dk + (g / vshare) * dv;
            for (int d = lane; d < dk; d += 32) kt[jj * KP + d] = ldf(ks + d);
            for (int d = lane; d < dv; d += 32) vt[jj * dv + d] = ldf(vs + d);
        }
        __syncthreads();
        const float* qw = qs + warp * dk;
        float s = -INFINITY;
        if (lane < nkeys) {
            const float* kr = kt + lane * KP;
            float a = 0.f;
            for (int d = 0; d < dk; d++) a += qw[d] * kr[d];
            s = softcap > 0.f ? softcap * tanhf(a / softcap) : a;
        }
        const float m_new = fmaxf(m, warp_max(s));          // finite: key `base` is always visible
        const float alpha = expf(m - m_new);                // 0 on the first tile without a sink (m = -inf)
        const float p = lane < nkeys ? expf(s - m_new) : 0.f;
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int k = 0; k < KR; k++) acc[k] *= alpha;
        for (int jj = 0; jj < nkeys; jj++) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const float* vr = vt + jj * dv;
#pragma unroll
            for (int k = 0; k < KR; k++) {
                const int d = lane + 32 * k;
                if (d < dv) acc[k] += pj * vr[d];
            }
        }
        m = m_new;
    }
    float denom = l;
    T* o = out + t * out_stride_t + (int64_t)h * dv;
    const T* gr = gate != nullptr ? gate + t * gate_stride_t + (int64_t)h * dv : nullptr;
    if (vcos != nullptr) {
        // the sum of turned values is turned back by the query's own position: pair (a, b) -> (a c + b s, b c - a s)
        float* ow = os + warp * dv;
#pragma unroll
        for (int k = 0; k < KR; k++) {
            const int d = lane + 32 * k;
            if (d < dv) ow[d] = acc[k] / denom;
        }
        __syncwarp();
        const int hv = dv >> 1;
        const float* vc = vcos + t * hv;
        const float* vs = vsin + t * hv;
#pragma unroll
        for (int k = 0; k < KR; k++) {
            const int d = lane + 32 * k;
            if (d < dv) {
                int m, second;
                if (halves) { second = d >= hv; m = second ? d - hv : d; } else { second = d & 1; m = d >> 1; }
                const float a = halves ? ow[m] : ow[2 * m], b = halves ? ow[m + hv] : ow[2 * m + 1];
                acc[k] = second ? b * vc[m] - a * vs[m] : a * vc[m] + b * vs[m];
            }
        }
        denom = 1.f;
    }
#pragma unroll
    for (int k = 0; k < KR; k++) {
        const int d = lane + 32 * k;
        if (d < dv) {
            float y = acc[k] / denom * out_scale;
            if (gr != nullptr) y *= 1.f / (1.f + expf(-ldf(gr + d)));
            if (out_f32) reinterpret_cast<float*>(out)[t * out_stride_t + (int64_t)h * dv + d] = y;
            else stf(o + d, y);
        }
    }
}


// ------------------------------------------------------------------ attention (tensor cores, 16-bit storage)
// One CTA = up to 64 query ROWS of one key/value group: row r is (token r / hqp of the CTA's token range, head r % hqp of the
// group), hqp = heads per group rounded up to a power of two.  The CTA walks its tokens in SEGMENTS (runs of one sequence at
// consecutive positions - a prompt portion; a decoded token is a segment of one), and a segment's rows share every staged key
// tile: WT_KEYS keys x (dk + dv), gathered through the block table with cp.async into a two-stage ring while the previous tile is
// multiplied (32-key tiles for prompt portions and large decode batches, see the launcher).  Warp w owns rows 16 w .. 16 w + 15: S = Q K^T (mma.sync m16n8k16, fp32 accumulate), per-row window mask, online
// softmax in fp32 (base 2, the sink enters as a key of score 0), P rounded to the storage type and fed from registers into
// O += P V.  dk, dv multiples of 16, at most DMAX.  Rows of 16-bit tiles are padded by 16 bytes: the eight rows an ldmatrix
// reads then fall into eight different bank groups for every dk / dv.
constexpr int WT_ROWS = 64;

// WT_KEYS: keys per tile (32 or 64).  Smaller tiles leave room for more CTAs per SM (prompt portions: many CTAs, latency-bound);
// larger ones keep more bytes in flight per CTA (decoded tokens: few CTAs that walk their window alone).
template <typename T, int DMAX, int WT_KEYS>
__global__ void __launch_bounds__(128, WT_KEYS == 32 ? 3 : 2) window_attn_mma_kernel(
    const T* __restrict__ q, int64_t q_stride_t, const float* __restrict__ cosb, const float* __restrict__ sinb,
    const T* __restrict__ gate, int64_t gate_stride_t, const T* __restrict__ cache, int n_slots, int slot, int block_size,
    const int* __restrict__ block_table, int max_blocks_per_seq, const int* __restrict__ tok_seq,
    const int* __restrict__ tok_pos, T* __restrict__ out, int64_t out_stride_t, int row0, int nrows, int qt, int hq, int hqp_log2,
    int H, int G, int dk, int dv, int rot_dims, int window, float scale_log2, float sink, int halves, float qk_norm_eps,
    float softcap, const float* __restrict__ vcos, const float* __restrict__ vsin, float out_scale,
    const float* __restrict__ qnorm_w, float prenorm_eps, int chunk, int vshare, int out_f32) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int PQ = dk * 2 + 16, PK = dk * 2 + 16, PV = dv * 2 + 16;            // row pitches in bytes
    unsigned char* Qs = smem_raw;                                              // [64][PQ]
    unsigned char* Ks = Qs + WT_ROWS * PQ;                                     // [2][64][PK]
    unsigned char* Vs = Ks + 2 * WT_KEYS * PK;                                 // [2][64][PV]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = blockIdx.y;
    const int hqp = 1 << hqp_log2;
    const int t_first = row0 + blockIdx.x * qt;
    const int ntok = min(qt, row0 + nrows - t_first);
    const int row_elems = G * dk + (G / vshare) * dv;
    const int ck = dk >> 3, cv = dv >> 3;                                      // 16-byte chunks per key / value row
    const int half = rot_dims >> 1;
    // with a score cap: cap * tanh(s * scale / cap), then to base 2
    const float cap_in = softcap > 0.f ? scale_log2 * 0.6931471805599453f / softcap : 0.f;
    const float cap_out = softcap * 1.4426950408889634f;

    for (int i0 = 0; i0 < ntok;) {
        // ---- the segment: tokens t_first + i0 .. + n - 1 of one sequence at consecutive positions
        const int ts = t_first + i0;
        const int seq = tok_seq[ts], pos0 = tok_pos[ts];
        int n = 1;
        while (i0 + n < ntok && tok_seq[ts + n] == seq && tok_pos[ts + n] == pos0 + n) n++;
        const int* bt = block_table + (int64_t)seq * max_blocks_per_seq;
        int lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
        if (chunk > 0) lo = max(lo, pos0 / chunk * chunk);
        const int hi = pos0 + n - 1;
        const int ntiles = (hi - lo) / WT_KEYS + 1;
        __syncthreads();                                                       // the previous segment's tiles and queries are done with

        // two threads per key row, alternating 16-byte chunks: ONE block-table lookup and address per thread and tile
        auto load_tile = [&](int it) {
            constexpr int TPR = 128 / WT_KEYS;                                 // threads per key row
            const int st = it & 1, jj = tid / TPR, part = tid % TPR;
            const int kp = lo + it * WT_KEYS + jj;
            const bool ok = kp <= hi;
            const T* krow = cache;
            const T* vrow = cache;
            if (ok) {
                const int b = kp / block_size;
                const int64_t rowi = ((int64_t)bt[b] * n_slots + slot) * block_size + (kp - b * block_size);
                krow = cache + rowi * row_elems + g * dk;
                vrow = cache + rowi * row_elems + G * dk + (g / vshare) * dv;
            }
            const int nb = ok ? 16 : 0;
            const uint32_t kd = smem_u32(Ks + (st * WT_KEYS + jj) * PK), vd = smem_u32(Vs + (st * WT_KEYS + jj) * PV);
            for (int ch = part; ch < ck; ch += TPR) cp_async16(kd + ch * 16, ok ? krow + ch * 8 : krow, nb);
            for (int ch = part; ch < cv; ch += TPR) cp_async16(vd + ch * 16, ok ? vrow + ch * 8 : vrow, nb);
            cp_async_commit();
        };
        load_tile(0);

        // ---- queries of the segment: rotated (and divided by their root mean square) in fp32, rounded to the storage type;
        // dead rows are zeros.  Two threads per row (neighbouring lanes), each takes every other pair of entries.
        {
            const int r = tid >> 1;                                            // 128 threads, 64 rows: one row per thread pair
            const int j = r >> hqp_log2, hh = r & (hqp - 1);
            const bool live = j < n && hh < hq;
            const int64_t t = ts + j;
            const T* qr = q + t * q_stride_t + (int64_t)(g * hq + hh) * dk;
            const float* cs = cosb != nullptr ? cosb + t * half : nullptr;
            const float* sn = sinb != nullptr ? sinb + t * half : nullptr;
            float pinv = 1.f;
            if (qnorm_w != nullptr) {
                float s0 = 0.f;
                if (live)
                    for (int i = tid & 1; i < (dk >> 1); i += 2) {
                        const float a = ldf(qr + 2 * i), b = ldf(qr + 2 * i + 1);
                        s0 += a * a + b * b;
                    }
                s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
                pinv = 1.f / sqrtf(s0 / (float)dk + prenorm_eps);
            }
            float inv = 1.f;
            if (qk_norm_eps >= 0.f) {
                float ss = 0.f;
                if (live)
                    for (int i = tid & 1; i < (dk >> 1); i += 2) {
                        const float a = rot_entry(qr, 2 * i, rot_dims, halves, cs, sn, pinv, qnorm_w),
                                    b = rot_entry(qr, 2 * i + 1, rot_dims, halves, cs, sn, pinv, qnorm_w);
                        ss += a * a + b * b;
                    }
                ss += __shfl_xor_sync(0xffffffffu, ss, 1);
                inv = 1.f / sqrtf(ss / (float)dk + qk_norm_eps);
            }
            for (int i = tid & 1; i < (dk >> 1); i += 2) {
                float a = 0.f, b = 0.f;
                if (live) {
                    a = rot_entry(qr, 2 * i, rot_dims, halves, cs, sn, pinv, qnorm_w) * inv;
                    b = rot_entry(qr, 2 * i + 1, rot_dims, halves, cs, sn, pinv, qnorm_w) * inv;
                }
                *reinterpret_cast<uint32_t*>(Qs + r * PQ + i * 4) = pack2<T>(a, b);
            }
        }

        // ---- per-thread state: rows (lane / 4) and (lane / 4) + 8 of the warp's 16
        const int r_a = warp * 16 + (lane >> 2), r_b = r_a + 8;
        const int j_a = r_a >> hqp_log2, j_b = r_b >> hqp_log2;
        const bool live_a = j_a < n && (r_a & (hqp - 1)) < hq, live_b = j_b < n && (r_b & (hqp - 1)) < hq;
        const int pos_a = pos0 + j_a, pos_b = pos0 + j_b;
        int lo_a = window > 0 ? pos_a - window + 1 : 0, lo_b = window > 0 ? pos_b - window + 1 : 0;
        if (chunk > 0) { lo_a = max(lo_a, pos_a / chunk * chunk); lo_b = max(lo_b, pos_b / chunk * chunk); }
        // keys any row of this warp can see (warp-uniform): tiles outside are skipped
        const int wj_min = (warp * 16) >> hqp_log2, wj_max = min((warp * 16 + 15) >> hqp_log2, n - 1);
        const bool warp_live = wj_min < n;
        int w_lo = window > 0 ? max(0, pos0 + wj_min - window + 1) : 0;
        if (chunk > 0) w_lo = max(w_lo, (pos0 + wj_min) / chunk * chunk);
        const int w_hi = pos0 + wj_max;
        float m_a = sink > 0.f ? 0.f : -INFINITY, m_b = m_a;
        float l_a = (lane & 3) == 0 ? sink : 0.f, l_b = l_a;
        float o[DMAX / 8][4];
#pragma unroll
        for (int nt = 0; nt < DMAX / 8; nt++) { o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f; }

        for (int it = 0; it < ntiles; it++) {
            if (it + 1 < ntiles) { load_tile(it + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
            __syncthreads();                                                   // tile `it` (and, first time, the queries) visible
            const int base = lo + it * WT_KEYS;
            if (warp_live && base <= w_hi && base + WT_KEYS - 1 >= w_lo) {
                const unsigned char* Kt = Ks + (it & 1) * WT_KEYS * PK;
                const unsigned char* Vt = Vs + (it & 1) * WT_KEYS * PV;
                float sc[WT_KEYS / 8][4];
#pragma unroll
                for (int nt = 0; nt < WT_KEYS / 8; nt++) { sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f; }
#pragma unroll
                for (int kk = 0; kk < DMAX / 16; kk++) {
                    if (kk * 16 < dk) {
                        uint32_t a[4];
                        ldmatrix_x4(smem_u32(Qs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * PQ + (kk * 16 + (lane >> 4) * 8) * 2),
                                    a[0], a[1], a[2], a[3]);
#pragma unroll
                        for (int np = 0; np < WT_KEYS / 16; np++) {
                            uint32_t b0, b1, b2, b3;
                            ldmatrix_x4(smem_u32(Kt + (np * 16 + (lane >> 4) * 8 + (lane & 7)) * PK + (kk * 16 + ((lane >> 3) & 1) * 8) * 2),
                                        b0, b1, b2, b3);
                            mma_16816<T>(sc[2 * np], a, b0, b1);
                            mma_16816<T>(sc[2 * np + 1], a, b2, b3);
                        }
                    }
                }
                // mask, running maximum
                float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
                for (int nt = 0; nt < WT_KEYS / 8; nt++) {
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const int kp = base + nt * 8 + (lane & 3) * 2 + e;
                        const bool va = live_a && kp <= pos_a && kp >= lo_a, vb = live_b && kp <= pos_b && kp >= lo_b;
                        const float sa = softcap > 0.f ? cap_out * tanhf(sc[nt][e] * cap_in) : sc[nt][e] * scale_log2;
                        const float sb = softcap > 0.f ? cap_out * tanhf(sc[nt][2 + e] * cap_in) : sc[nt][2 + e] * scale_log2;
                        sc[nt][e] = va ? sa : -INFINITY;
                        sc[nt][2 + e] = vb ? sb : -INFINITY;
                        mx_a = fmaxf(mx_a, sc[nt][e]);
                        mx_b = fmaxf(mx_b, sc[nt][2 + e]);
                    }
                }
                mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1)); mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
                mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1)); mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
                const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
                const float ref_a = mn_a == -INFINITY ? 0.f : mn_a, ref_b = mn_b == -INFINITY ? 0.f : mn_b;   // nothing seen yet
                const float al_a = exp2f(m_a - ref_a), al_b = exp2f(m_b - ref_b);                             // exp2(-inf) = 0
                m_a = mn_a; m_b = mn_b;
                l_a *= al_a; l_b *= al_b;
#pragma unroll
                for (int nt = 0; nt < DMAX / 8; nt++) { o[nt][0] *= al_a; o[nt][1] *= al_a; o[nt][2] *= al_b; o[nt][3] *= al_b; }
                uint32_t pa[WT_KEYS / 16][4];
#pragma unroll
                for (int nt = 0; nt < WT_KEYS / 8; nt++) {
                    const float p0 = exp2f(sc[nt][0] - ref_a), p1 = exp2f(sc[nt][1] - ref_a);
                    const float p2 = exp2f(sc[nt][2] - ref_b), p3 = exp2f(sc[nt][3] - ref_b);
                    l_a += p0 + p1; l_b += p2 + p3;
                    pa[nt >> 1][(nt & 1) * 2] = pack2<T>(p0, p1);
                    pa[nt >> 1][(nt & 1) * 2 + 1] = pack2<T>(p2, p3);
                }
#pragma unroll
                for (int kk = 0; kk < WT_KEYS / 16; kk++) {                    // 16 keys per step
#pragma unroll
                    for (int np = 0; np < DMAX / 16; np++) {
                        if (np * 16 < dv) {
                            uint32_t b0, b1, b2, b3;
                            ldmatrix_x4_trans(smem_u32(Vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * PV + (np * 16 + (lane >> 4) * 8) * 2),
                                              b0, b1, b2, b3);
                            mma_16816<T>(o[2 * np], pa[kk], b0, b1);
                            mma_16816<T>(o[2 * np + 1], pa[kk], b2, b3);
                        }
                    }
                }
            }
            __syncthreads();                                                   // stage it & 1 may be overwritten by tile it + 2
        }

        // ---- normalise, (turn back,) gate, store
        l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
        l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
        if (vcos != nullptr) {
            // values were stored turned by their own position: the normalised sums go through shared memory (the tiles are done
            // with: the loop ended on a barrier), where every pair is turned back by the query's position
            float* Os = reinterpret_cast<float*>(smem_raw);                    // [64][dv]
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int r = e ? r_b : r_a;
                const float inv = 1.f / (e ? l_b : l_a);
#pragma unroll
                for (int nt = 0; nt < DMAX / 8; nt++) {
                    const int d = nt * 8 + (lane & 3) * 2;
                    if (d < dv) { Os[r * dv + d] = o[nt][2 * e] * inv; Os[r * dv + d + 1] = o[nt][2 * e + 1] * inv; }
                }
            }
            __syncthreads();
            const int hv = dv >> 1;
            for (int idx = tid; idx < WT_ROWS * hv; idx += 128) {
                const int r = idx / hv, m = idx - r * hv;
                const int j = r >> hqp_log2, hh = r & (hqp - 1);
                if (j >= n || hh >= hq) continue;
                const int64_t t = ts + j;
                const int da = halves ? m : 2 * m, db = halves ? m + hv : 2 * m + 1;
                const float a = Os[r * dv + da], b = Os[r * dv + db];
                const float c = vcos[t * hv + m], sn = vsin[t * hv + m];
                float ya = (a * c + b * sn) * out_scale, yb = (b * c - a * sn) * out_scale;
                T* orow = out + t * out_stride_t + (int64_t)(g * hq + hh) * dv;
                if (gate != nullptr) {
                    const T* grow = gate + t * gate_stride_t + (int64_t)(g * hq + hh) * dv;
                    ya *= 1.f / (1.f + __expf(-ldf(grow + da)));
                    yb *= 1.f / (1.f + __expf(-ldf(grow + db)));
                }
                stf(orow + da, ya);
                stf(orow + db, yb);
            }
            i0 += n;
            continue;                                                          // the next segment starts with a barrier
        }
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const bool live = e ? live_b : live_a;
            if (!live) continue;
            const int r = e ? r_b : r_a;
            const int64_t t = ts + (r >> hqp_log2);
            const int h = g * hq + (r & (hqp - 1));
            const float inv = out_scale / (e ? l_b : l_a);
            T* orow = out + t * out_stride_t + (int64_t)h * dv;
            const T* grow = gate != nullptr ? gate + t * gate_stride_t + (int64_t)h * dv : nullptr;
#pragma unroll
            for (int nt = 0; nt < DMAX / 8; nt++) {
                const int d = nt * 8 + (lane & 3) * 2;
                if (d < dv) {
                    float y0 = o[nt][2 * e] * inv, y1 = o[nt][2 * e + 1] * inv;
                    if (grow != nullptr) {
                        y0 *= 1.f / (1.f + __expf(-ldf(grow + d)));
                        y1 *= 1.f / (1.f + __expf(-ldf(grow + d + 1)));
                    }
                    if (out_f32) {
                        float* o32 = reinterpret_cast<float*>(out) + t * out_stride_t + (int64_t)h * dv + d;
                        o32[0] = y0; o32[1] = y1;
                    } else {
                        *reinterpret_cast<uint32_t*>(orow + d) = pack2<T>(y0, y1);
                    }
                }
            }
        }
        i0 += n;
    }
}

// ------------------------------------------------------------------ two maps -> one head
// a: fp32 [T, G, 2, hq, dv] (the attention above with vshare = 2 and queries ordered [key/value head][map][head of the group]).
// One warp per (token, head h = g hq + hh): o = a[g, 0, hh] - lambda a[g, 1, hh]; out = o / sqrt(mean(o^2) + eps) * factor *
// sigmoid(gate[t, h]) in the storage type, heads in their natural order.  KR: registers per lane, dv <= 32 KR.
template <typename T, int KR>
__global__ void __launch_bounds__(256) diff_combine_kernel(const float* __restrict__ a, const T* __restrict__ gate,
                                                           int64_t gate_stride_t, T* __restrict__ out, int64_t out_stride_t,
                                                           int64_t units, int H, int hq, int dv, float lambda, float eps,
                                                           float factor) {
    const int lane = threadIdx.x & 31;
    const int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= units) return;
    const int64_t t = unit / H;
    const int h = (int)(unit - t * H), g = h / hq, hh = h - g * hq;
    const float* a1 = a + (t * 2 * H + (int64_t)(g * 2 * hq + hh)) * dv;
    const float* a2 = a1 + (int64_t)hq * dv;
    float o[KR], ss = 0.f;
#pragma unroll
    for (int k = 0; k < KR; k++) {
        const int d = lane + 32 * k;
        o[k] = d < dv ? a1[d] - lambda * a2[d] : 0.f;
        ss += o[k] * o[k];
    }
    const float f = factor / sqrtf(warp_sum(ss) / (float)dv + eps);
    const T* gr = gate != nullptr ? gate + t * gate_stride_t + (int64_t)h * dv : nullptr;
    T* orow = out + t * out_stride_t + (int64_t)h * dv;
#pragma unroll
    for (int k = 0; k < KR; k++) {
        const int d = lane + 32 * k;
        if (d < dv) {
            float y = o[k] * f;
            if (gr != nullptr) y *= 1.f / (1.f + expf(-ldf(gr + d)));
            stf(orow + d, y);
        }
    }
}

static bool g_window_simt = false;

// rows [0, num_prefill) are prompt portions (many consecutive tokens of a sequence share a CTA), the rest single decoded tokens
template <typename T, int DMAX>
static int launch_window_attn_mma(const void* q, int64_t q_stride_t, const void* cosb, const void* sinb, const void* gate,
                                  int64_t gate_stride_t, const void* cache, int n_slots, int slot, int block_size,
                                  const void* block_table, int max_blocks_per_seq, const void* tok_seq, const void* tok_pos,
                                  void* out, int64_t out_stride_t, int64_t num_tokens, int64_t num_prefill, int H, int G, int dk,
                                  int dv, int rot_dims, int window, float scale, float sink, int halves, float qk_norm_eps,
                                  float softcap, const void* vcos, const void* vsin, float out_scale, const void* qnorm_w,
                                  float prenorm_eps, int chunk, int vshare, int out_f32, cudaStream_t stream) {
    static unsigned long long attr_mask = 0;
    const int hq = H / G;
    int hqp_log2 = 0;
    while ((1 << hqp_log2) < hq) hqp_log2++;
    auto kern_prompt = window_attn_mma_kernel<T, DMAX, 32>;
    auto kern_decode = window_attn_mma_kernel<T, DMAX, 64>;
    if (first_use_on_this_device(attr_mask)) {
        cudaFuncSetAttribute(kern_prompt, cudaFuncAttributeMaxDynamicSharedMemorySize, 120 * 1024);
        cudaFuncSetAttribute(kern_decode, cudaFuncAttributeMaxDynamicSharedMemorySize, 120 * 1024);
    }
    int num_sms = 0;
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, current_device());
    const float scale_log2 = scale * 1.4426950408889634f;
    const int64_t parts[2][2] = {{0, num_prefill}, {num_prefill, num_tokens - num_prefill}};
    for (int k = 0; k < 2; k++) {
        const int64_t first = parts[k][0], count = parts[k][1];
        if (count <= 0) continue;
        const int qt = k == 0 ? WT_ROWS >> hqp_log2 : 1;
        // measured on B200 (128 + 128 per head): prompt portions 24 - 26 % faster with 32-key tiles (three CTAs per SM instead of
        // two); decoded tokens faster with 64-key tiles at 512 CTAs (357 vs 385 us), with 32-key tiles at 2048 CTAs (950 vs 1220 us)
        const int keys = (k == 0 || count * G >= 7 * (int64_t)num_sms) ? 32 : 64;
        size_t smem = (size_t)WT_ROWS * (dk * 2 + 16) + 2 * (size_t)keys * ((dk * 2 + 16) + (dv * 2 + 16));
        if (vcos != nullptr && smem < (size_t)WT_ROWS * dv * sizeof(float)) smem = (size_t)WT_ROWS * dv * sizeof(float);
        (keys == 32 ? kern_prompt : kern_decode)<<<dim3((unsigned)cdiv(count, qt), (unsigned)G), 128, smem, stream>>>(
            (const T*)q, q_stride_t, (const float*)cosb, (const float*)sinb, (const T*)gate, gate_stride_t, (const T*)cache,
            n_slots, slot, block_size, (const int*)block_table, max_blocks_per_seq, (const int*)tok_seq, (const int*)tok_pos,
            (T*)out, out_stride_t, (int)first, (int)count, qt, hq, hqp_log2, H, G, dk, dv, rot_dims, window, scale_log2, sink,
            halves, qk_norm_eps, softcap, (const float*)vcos, (const float*)vsin, out_scale, (const float*)qnorm_w, prenorm_eps,
            chunk, vshare, out_f32);
    }
    return check_launch("window_attention (tensor cores)");
}

static int heads_per_cta(int hq) {
    for (int n = WA_MAX_HPB; n > 1; n--)
        if (hq % n == 0) return n;
    return 1;
}

template <typename T, int KR>
static int launch_window_attn(const void* q, int64_t q_stride_t, const void* cosb, const void* sinb, const void* gate,
                              int64_t gate_stride_t, const void* cache, int n_slots, int slot, int block_size,
                              const void* block_table, int max_blocks_per_seq, const void* tok_seq, const void* tok_pos, void* out,
                              int64_t out_stride_t, int64_t num_tokens, int H, int G, int dk, int dv, int rot_dims, int window,
                              float scale, float sink, int halves, float qk_norm_eps, float softcap, const void* vcos,
                              const void* vsin, float out_scale, const void* qnorm_w, float prenorm_eps, int chunk, int vshare,
                              int out_f32, cudaStream_t stream) {
    static unsigned long long attr_mask = 0;
    const int hpb = heads_per_cta(H / G);
    const size_t smem = ((size_t)hpb * dk + (size_t)WA_TILE * (dk + 1) + (size_t)WA_TILE * dv + (size_t)hpb * dv) * sizeof(float);
    SLLM_REQUIRE(smem <= 200 * 1024, "window_attention: head sizes %d / %d need %zu bytes of shared memory", dk, dv, smem);
    auto kern = window_attn_kernel<T, KR>;
    if (first_use_on_this_device(attr_mask))
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    kern<<<dim3((unsigned)num_tokens, (unsigned)(H / hpb)), hpb * 32, smem, stream>>>(
        (const T*)q, q_stride_t, (const float*)cosb, (const float*)sinb, (const T*)gate, gate_stride_t, (const T*)cache, n_slots,
        slot, block_size, (const int*)block_table, max_blocks_per_seq, (const int*)tok_seq, (const int*)tok_pos, (T*)out,
        out_stride_t, H, G, dk, dv, rot_dims, window, scale, sink, halves, qk_norm_eps, softcap, (const float*)vcos,
        (const float*)vsin, out_scale, (const float*)qnorm_w, prenorm_eps, chunk, vshare, out_f32);
    return check_launch("window_attention");
}

}  // namespace sllm

using namespace sllm;

extern "C" {

int sllm_window_kv_store(const void* k, int64_t k_row_stride, const void* v, int64_t v_row_stride, const void* cosb,
                         const void* sinb, const void* tok_seq, const void* tok_pos, const void* block_table,
                         int max_blocks_per_seq, void* cache, int n_slots, int slot, int block_size, int64_t num_tokens,
                         int num_kv_heads, int dk, int dv, int rot_dims, int pair_halves, float qk_norm_eps, const void* vcos,
                         const void* vsin, const void* knorm_w, float prenorm_eps, int vshare, sllm_dtype_t dtype,
                         sllm_stream_t stream) {
    SLLM_REQUIRE(vshare >= 1 && num_kv_heads % vshare == 0, "window_kv_store: %d key heads cannot share values in runs of %d",
                 num_kv_heads, vshare);
    SLLM_REQUIRE(num_tokens >= 0 && num_kv_heads > 0 && dk > 0 && dv > 0 && rot_dims >= 0 && rot_dims <= dk && rot_dims % 2 == 0,
                 "window_kv_store: bad shape (kv heads %d, dk %d, dv %d, rot_dims %d)", num_kv_heads, dk, dv, rot_dims);
    SLLM_REQUIRE((vcos == nullptr) == (vsin == nullptr) && (vcos == nullptr || dv % 2 == 0),
                 "window_kv_store: turned values need both angle tables and an even value size (dv %d)", dv);
    SLLM_REQUIRE(slot >= 0 && slot < n_slots && block_size > 0, "window_kv_store: bad cache slot %d of %d", slot, n_slots);
    if (num_tokens == 0) return 0;
    SLLM_REQUIRE(k && v && tok_seq && tok_pos && block_table && cache && (rot_dims == 0 || (cosb && sinb)),
                 "window_kv_store: null pointer");
    SLLM_DISPATCH_DTYPE_F32(dtype, (window_kv_store_kernel<T><<<(unsigned)num_tokens, 128, 0, (cudaStream_t)stream>>>(
        (const T*)k, k_row_stride, (const T*)v, v_row_stride, (const float*)cosb, (const float*)sinb, (const int*)tok_seq,
        (const int*)tok_pos, (const int*)block_table, max_blocks_per_seq, (T*)cache, n_slots, slot, block_size, num_kv_heads,
        dk, dv, rot_dims, pair_halves, qk_norm_eps, (const float*)vcos, (const float*)vsin, (const float*)knorm_w, prenorm_eps,
        vshare)));
    return check_launch("window_kv_store");
}

int sllm_window_attention_set_simt(int on) {
    const int old = g_window_simt ? 1 : 0;
    g_window_simt = on != 0;
    return old;
}

int sllm_window_attention(const void* q, int64_t q_stride_t, const void* cosb, const void* sinb, const void* gate,
                          int64_t gate_stride_t, const void* cache, int n_slots, int slot, int block_size,
                          const void* block_table, int max_blocks_per_seq, const void* tok_seq, const void* tok_pos, void* out,
                          int64_t out_stride_t, int64_t num_tokens, int64_t num_prefill_tokens, int num_heads, int num_kv_heads,
                          int dk, int dv, int rot_dims, int window, float scale, int sink, int pair_halves, float qk_norm_eps,
                          float softcap, const void* vcos, const void* vsin, float out_scale, const void* qnorm_w,
                          float prenorm_eps, int chunk, int vshare, int out_f32, sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(vshare >= 1 && num_kv_heads % vshare == 0 && chunk >= 0 && (!out_f32 || vcos == nullptr),
                 "window_attention: %d key heads in runs of %d; chunk %d >= 0; fp32 output excludes turned values", num_kv_heads,
                 vshare, chunk);
    SLLM_REQUIRE((vcos == nullptr) == (vsin == nullptr) && (vcos == nullptr || dv % 2 == 0) && softcap >= 0.f,
                 "window_attention: turned values need both angle tables and an even value size (dv %d); softcap >= 0", dv);
    SLLM_REQUIRE(num_tokens >= 0 && num_heads > 0 && num_kv_heads > 0 && num_heads % num_kv_heads == 0 && dk > 0 && dv > 0 &&
                 dv <= 256 && rot_dims >= 0 && rot_dims <= dk && rot_dims % 2 == 0,
                 "window_attention: bad shape (heads %d / %d, dk %d, dv %d <= 256, rot_dims %d)", num_heads, num_kv_heads, dk,
                 dv, rot_dims);
    SLLM_REQUIRE(slot >= 0 && slot < n_slots && block_size > 0, "window_attention: bad cache slot %d of %d", slot, n_slots);
    if (num_tokens == 0) return 0;
    SLLM_REQUIRE(q && tok_seq && tok_pos && block_table && cache && out && (rot_dims == 0 || (cosb && sinb)),
                 "window_attention: null pointer");
    SLLM_REQUIRE(num_prefill_tokens >= 0 && num_prefill_tokens <= num_tokens, "window_attention: bad number of prompt rows");
    const float sinkw = sink ? 1.f : 0.f;
    const int hq = num_heads / num_kv_heads;
    if (!g_window_simt && dtype != SLLM_F32 && dk % 16 == 0 && dv % 16 == 0 && dk <= 128 && dv <= 128 && hq <= WT_ROWS &&
        num_tokens < (1ll << 31)) {
#define WA_MMA(DMAX)                                                                                                        \
    SLLM_DISPATCH_DTYPE(dtype, return (launch_window_attn_mma<T, DMAX>(q, q_stride_t, cosb, sinb, gate, gate_stride_t, cache,  \
        n_slots, slot, block_size, block_table, max_blocks_per_seq, tok_seq, tok_pos, out, out_stride_t, num_tokens,         \
        num_prefill_tokens, num_heads, num_kv_heads, dk, dv, rot_dims, window, scale, sinkw, pair_halves, qk_norm_eps, softcap, \
        vcos, vsin, out_scale, qnorm_w, prenorm_eps, chunk, vshare, out_f32, (cudaStream_t)stream)))
        if (dk <= 64 && dv <= 64) { WA_MMA(64); }
        else { WA_MMA(128); }
#undef WA_MMA
    }
#define WA_LAUNCH(KR)                                                                                                      \
    SLLM_DISPATCH_DTYPE_F32(dtype, return (launch_window_attn<T, KR>(q, q_stride_t, cosb, sinb, gate, gate_stride_t, cache,   \
        n_slots, slot, block_size, block_table, max_blocks_per_seq, tok_seq, tok_pos, out, out_stride_t, num_tokens,        \
        num_heads, num_kv_heads, dk, dv, rot_dims, window, scale, sinkw, pair_halves, qk_norm_eps, softcap, vcos, vsin,      \
        out_scale, qnorm_w, prenorm_eps, chunk, vshare, out_f32, (cudaStream_t)stream)))
    if (dv <= 32) { WA_LAUNCH(1); }
    else if (dv <= 64) { WA_LAUNCH(2); }
    else if (dv <= 128) { WA_LAUNCH(4); }
    else { WA_LAUNCH(8); }
#undef WA_LAUNCH
    return 0;
}

int sllm_diff_combine(const void* a, const void* gate, int64_t gate_stride_t, void* out, int64_t out_stride_t, int64_t num_tokens,
                      int num_heads, int num_kv_heads, int dv, float lambda, float eps, float factor, sllm_dtype_t dtype,
                      sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && num_heads > 0 && num_kv_heads > 0 && num_heads % num_kv_heads == 0 && dv > 0 && dv <= 256,
                 "diff_combine: bad shape (heads %d / %d, dv %d <= 256)", num_heads, num_kv_heads, dv);
    if (num_tokens == 0) return 0;
    SLLM_REQUIRE(a && out, "diff_combine: null pointer");
    const int64_t units = num_tokens * num_heads;
    const int hq = num_heads / num_kv_heads;
#define DC_LAUNCH(KR)                                                                                                       \
    SLLM_DISPATCH_DTYPE_F32(dtype, (diff_combine_kernel<T, KR><<<(unsigned)cdiv(units, 8), 256, 0, (cudaStream_t)stream>>>(   \
        (const float*)a, (const T*)gate, gate_stride_t, (T*)out, out_stride_t, units, num_heads, hq, dv, lambda, eps, factor)))
    if (dv <= 32) { DC_LAUNCH(1); }
    else if (dv <= 64) { DC_LAUNCH(2); }
    else if (dv <= 128) { DC_LAUNCH(4); }
    else { DC_LAUNCH(8); }
#undef DC_LAUNCH
    return check_launch("diff_combine");
}

}  // extern "C"
