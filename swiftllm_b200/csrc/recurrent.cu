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
#include "typed_io.cuh"

namespace sllm {

constexpr int CONV_MAX_TAPS = 8;

// grid (T, ceil(C / 256)).  tail: [rows, K-1, C] (slot i: the input K-1-i positions before the next one).
template <typename T>
__global__ void __launch_bounds__(256) causal_conv_kernel(const T* __restrict__ xin, int64_t xin_stride, const T* __restrict__ w,
                                                          const T* __restrict__ bias, const T* __restrict__ tail,
                                                          const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                                          T* __restrict__ u, int C, int K) {
    const int64_t t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int seq = tok_seq[t], pos = tok_pos[t];
    // rows above this one that are the sequence's previous positions
    int above = 0;
    while (above < K - 1 && t - above - 1 >= 0 && tok_seq[t - above - 1] == seq && tok_pos[t - above - 1] == pos - above - 1) above++;
    float acc = bias != nullptr ? ldf(bias + c) : 0.f;
    for (int k = 0; k < K; k++) {
        if (pos - k < 0) break;
        float v;
        if (k <= above) {
            v = ldf(xin + (t - k) * xin_stride + c);
        } else {
            // position pos - k lies before the segment, which starts at pos - above: tail slot K-1 - (k - above)
            v = ldf(tail + ((int64_t)seq * (K - 1) + (K - 1 - (k - above))) * C + c);
        }
        acc += ldf(w + (int64_t)c * K + (K - 1 - k)) * v;
    }
    stf(u + t * C + c, acc);
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
        S = a * S + sqrtf(fmaxf(1.f - expf(2.f * log_a), 0.f)) * (g * x);
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

// grid (segments, heads), 256 threads.  Thread (sl, j): column j of the state, rows sl, sl + nsl, ... (at most R of them).
template <typename T, int R>
__global__ void __launch_bounds__(256) linear_attention_kernel(
    const T* __restrict__ q, int64_t q_stride, const T* __restrict__ k, int64_t k_stride, const T* __restrict__ v, int64_t v_stride,
    const float* __restrict__ decay, float* __restrict__ state, const int* __restrict__ seg_starts, const int* __restrict__ seq_ids,
    const int* __restrict__ tok_pos, float* __restrict__ out, int H, int dk, int dv, int nsl) {
    extern __shared__ float sm[];
    float* qs = sm;                 // [dk]
    float* ks = qs + dk;            // [dk]
    float* vs = ks + dk;            // [dv]
    float* red = vs + dv;           // [nsl][dv]
    const int b = blockIdx.x, h = blockIdx.y;
    const int t0 = seg_starts[b], n = seg_starts[b + 1] - t0;
    if (n <= 0) return;
    const int seq = seq_ids[b], p0 = tok_pos[t0];
    const int tid = threadIdx.x;
    const bool active = tid < nsl * dv;
    const int j = tid % dv, sl = tid / dv;
    const float lam = decay[h];
    float* st = state + ((int64_t)seq * H + h) * dk * dv;
    float S[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int d = sl + r * nsl;
        S[r] = (active && d < dk && p0 > 0) ? st[(int64_t)d * dv + j] : 0.f;
    }
    for (int i = 0; i < n; i++) {
        const int64_t t = t0 + i;
        __syncthreads();                    // the previous token's vectors and partial sums are done with
        for (int d = tid; d < dk; d += blockDim.x) {
            const float a = ldf(q + t * q_stride + (int64_t)h * dk + d), c = ldf(k + t * k_stride + (int64_t)h * dk + d);
            qs[d] = a * sigmoid_f(a);
            ks[d] = c * sigmoid_f(c);
        }
        for (int d = tid; d < dv; d += blockDim.x) { const float a = ldf(v + t * v_stride + (int64_t)h * dv + d); vs[d] = a * sigmoid_f(a); }
        __syncthreads();
        if (active) {
            const float vj = vs[j];
            float part = 0.f;
#pragma unroll
            for (int r = 0; r < R; r++) {
                const int d = sl + r * nsl;
                if (d < dk) {
                    S[r] = lam * S[r] + ks[d] * vj;
                    part += S[r] * qs[d];
                }
            }
            red[sl * dv + j] = part;
        }
        __syncthreads();
        if (tid < dv) {
            float o = 0.f;
            for (int s = 0; s < nsl; s++) o += red[s * dv + tid];
            out[t * ((int64_t)H * dv) + (int64_t)h * dv + tid] = o;
        }
    }
    if (active) {
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int d = sl + r * nsl;
            if (d < dk) st[(int64_t)d * dv + j] = S[r];
        }
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

template <typename T>
static int launch_linear_attention(const void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v, int64_t v_stride,
                                   const void* decay, void* state, const void* seg_starts, const void* seq_ids, const void* tok_pos,
                                   void* out, int num_segs, int H, int dk, int dv, cudaStream_t stream) {
    int nsl = 256 / dv;
    if (nsl > dk) nsl = dk;
    const int rows = (dk + nsl - 1) / nsl;
    const size_t smem = (size_t)(2 * dk + dv + nsl * dv) * sizeof(float);
    const dim3 grid((unsigned)num_segs, (unsigned)H);
#define LA(R)                                                                                                                  \
    linear_attention_kernel<T, R><<<grid, 256, smem, stream>>>((const T*)q, q_stride, (const T*)k, k_stride, (const T*)v, v_stride, \
        (const float*)decay, (float*)state, (const int*)seg_starts, (const int*)seq_ids, (const int*)tok_pos, (float*)out, H, dk,  \
        dv, nsl)
    if (rows <= 4) LA(4);
    else if (rows <= 8) LA(8);
    else if (rows <= 16) LA(16);
    else if (rows <= 32) LA(32);
    else if (rows <= 64) LA(64);
    else LA(128);
#undef LA
    return check_launch("linear_attention");
}

}  // namespace sllm

using namespace sllm;

extern "C" {

int sllm_causal_conv(const void* xin, int64_t xin_stride, const void* w, const void* bias, const void* tail, const void* tok_seq,
                     const void* tok_pos, void* u, int64_t num_tokens, int channels, int taps, sllm_dtype_t dtype,
                     sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && channels > 0 && taps >= 1 && taps <= CONV_MAX_TAPS, "causal_conv: 1 <= taps <= %d (got %d)",
                 CONV_MAX_TAPS, taps);
    if (num_tokens == 0) return 0;
    SLLM_REQUIRE(xin && w && tok_seq && tok_pos && u && (taps == 1 || tail), "causal_conv: null pointer");
    const dim3 grid((unsigned)num_tokens, (unsigned)cdiv(channels, 256));
    SLLM_DISPATCH_DTYPE_F32(dtype, (causal_conv_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>(
        (const T*)xin, xin_stride, (const T*)w, (const T*)bias, (const T*)tail, (const int*)tok_seq, (const int*)tok_pos, (T*)u,
        channels, taps)));
    return check_launch("causal_conv");
}

int sllm_rglru_scan(const void* u, const void* gates, int blocks, const void* ybr, int64_t y_stride, const void* rate,
                    const void* xin, int64_t xin_stride, void* state, void* tail, const void* seg_starts, const void* seq_ids,
                    const void* tok_pos, void* out, int64_t num_tokens, int num_segs, int channels, int taps, sllm_dtype_t dtype,
                    sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && num_segs >= 0 && channels > 0 && blocks > 0 && channels % blocks == 0 && taps >= 1 &&
                 taps <= CONV_MAX_TAPS, "rglru_scan: bad shape (channels %d in %d blocks, %d taps)", channels, blocks, taps);
    if (num_tokens == 0 || num_segs == 0) return 0;
    SLLM_REQUIRE(u && gates && ybr && rate && xin && state && (taps == 1 || tail) && seg_starts && seq_ids && tok_pos && out,
                 "rglru_scan: null pointer");
    const dim3 grid((unsigned)num_segs, (unsigned)cdiv(channels, 128));
    SLLM_DISPATCH_DTYPE_F32(dtype, (rglru_scan_kernel<T><<<grid, 128, 0, (cudaStream_t)stream>>>(
        (const T*)u, (const T*)gates, channels / blocks, (const T*)ybr, y_stride, (const float*)rate, (const T*)xin, xin_stride,
        (float*)state, (T*)tail, (const int*)seg_starts, (const int*)seq_ids, (const int*)tok_pos, (T*)out, num_tokens, channels,
        taps)));
    return check_launch("rglru_scan");
}

int sllm_linear_attention(const void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v, int64_t v_stride,
                          const void* decay, void* state, const void* seg_starts, const void* seq_ids, const void* tok_pos,
                          void* out, int num_segs, int num_heads, int dk, int dv, sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(num_segs >= 0 && num_heads > 0 && dk > 0 && dv > 0 && dv <= 256, "linear_attention: bad shape (dk %d, dv %d <= 256)",
                 dk, dv);
    {
        int nsl = 256 / dv;
        if (nsl > dk) nsl = dk;
        SLLM_REQUIRE((dk + nsl - 1) / nsl <= 128, "linear_attention: a %d x %d state does not fit one CTA's registers", dk, dv);
    }
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
