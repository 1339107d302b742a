// Row-wise kernels of SEQUENTIAL decoder blocks whose sublayers read the fp32 residual stream itself and whose OUTPUT is
// normalised before it is added (x <- x + gain * y / rms(y), one scalar gain per norm), with an optional learned weighted sum
// over the results of all earlier layers ("depth mix"), plus the embedding with a hashed table of token pairs, the tanh cap
// of logits, and the router / activation of a mixture of SiLU-gated experts with sigmoid scores.
// The stream, sums, norms and the router are fp32 whatever the storage type T (half, bf16 or float) of the projections is; every
// kernel that updates the stream also writes its rounding to T, which is what the next projections read.
// Algorithmic bytes (s = sizeof(T)): postnorm_add_mix  T*W*(8 + 2s) + 4*T*W*(1 + mixed layers).
#include "typed_io.cuh"

namespace sllm {

// x[t] = embed[token] + pairs[row]; row = (previous * mul_prev + token * mul_cur) mod buckets, where `previous` is the token
// before it: the row above when that is the same sequence's previous position, else the sequence's stored last token; a
// sequence's first token (position 0) takes row `buckets`.  One CTA per token.
template <typename T>
__global__ void __launch_bounds__(256) embed_pair_hash_kernel(
    const int* __restrict__ tokens, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
    const int* __restrict__ last_token, const T* __restrict__ embed, const T* __restrict__ pairs, int buckets, int64_t mul_prev,
    int64_t mul_cur, float* __restrict__ x, float* __restrict__ x_copy, T* __restrict__ h, int width) {
    const int64_t t = blockIdx.x;
    const int tok = tokens[t], pos = tok_pos[t], seq = tok_seq[t];
    const T* er = embed + (int64_t)tok * width;
    const T* pr = nullptr;
    if (pairs != nullptr) {
        int64_t row = buckets;
        if (pos > 0) {
            const bool above = t > 0 && tok_seq[t - 1] == seq && tok_pos[t - 1] == pos - 1;
            const int64_t prev = above ? tokens[t - 1] : last_token[seq];
            row = (prev * mul_prev + (int64_t)tok * mul_cur) % buckets;
            if (row < 0) row += buckets;
        }
        pr = pairs + row * width;
    }
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = ldf(er + i);
        if (pr != nullptr) v += ldf(pr + i);
        x[t * width + i] = v;
        if (x_copy != nullptr) x_copy[t * width + i] = v;
        stf(h + t * width + i, v);
    }
}

// last_token[seq of segment b] = the segment's last token.  Runs after the embedding has read the old values.
__global__ void store_last_tokens_kernel(const int* __restrict__ tokens, const int* __restrict__ seg_starts,
                                         const int* __restrict__ seq_ids, int* __restrict__ last_token, int num_segs) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < num_segs && seg_starts[b + 1] > seg_starts[b]) last_token[seq_ids[b]] = tokens[seg_starts[b + 1] - 1];
}

// X = x[t] + gain * y[t] / sqrt(mean(y[t]^2) + eps)     (X = x[t] when y is null)
// history[slot][t] = X (when history is given); x[t] <- sum_{j <= slot} mix[j] * history[j][t] (when mix is given), else X;
// h[t] = T(x[t]).  One CTA per token.
template <typename T>
__global__ void __launch_bounds__(256) postnorm_add_mix_kernel(
    float* __restrict__ x, const T* __restrict__ y, const float* __restrict__ gain, float eps, float* __restrict__ history,
    int slot, int64_t hist_stride, const float* __restrict__ mix, T* __restrict__ h, int width) {
    __shared__ float red[32];
    const int64_t t = blockIdx.x;
    float f = 0.f;
    if (y != nullptr) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < width; i += blockDim.x) { const float v = ldf(y + t * width + i); ss += v * v; }
        f = gain[0] / sqrtf(block_sum(ss, red) / (float)width + eps);
    }
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = x[t * width + i];
        if (y != nullptr) v += ldf(y + t * width + i) * f;
        if (history != nullptr) history[slot * hist_stride + t * width + i] = v;
        if (mix != nullptr) {
            float acc = mix[slot] * v;
            for (int j = 0; j < slot; j++) acc += mix[j] * history[j * hist_stride + t * width + i];
            v = acc;
        }
        x[t * width + i] = v;
        stf(h + t * width + i, v);
    }
}

template <typename T>
__global__ void tanh_cap_kernel(T* __restrict__ x, int64_t n, float cap) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) stf(x + i, cap * tanhf(ldf(x + i) / cap));
}

// One warp per token.  s = sigmoid(logits); the `top` experts with the largest s + bias are chosen (equal values: the lower
// expert index wins); weights[t, e] = s_e at the chosen experts (not renormalised), 0 elsewhere.
// Dynamic shared memory: warps * 2 * experts floats.
__global__ void __launch_bounds__(128) moe_route_sigmoid_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                                                float* __restrict__ weights, int64_t num_tokens, int experts,
                                                                int top) {
    extern __shared__ float vals[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= num_tokens) return;
    float* s = vals + warp * 2 * experts;     // scores
    float* c = s + experts;                   // choice scores
    for (int e = lane; e < experts; e += 32) {
        s[e] = 1.f / (1.f + expf(-logits[t * experts + e]));
        c[e] = s[e] + (bias != nullptr ? bias[e] : 0.f);
        weights[t * experts + e] = 0.f;
    }
    __syncwarp();
    for (int k = 0; k < top; k++) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            const float v = c[e];
            if (v > best) { best = v; bi = e; }
        }
        if (best == -INFINITY) bi = 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (lane == 0 && bi != 0x7fffffff) { weights[t * experts + bi] = s[bi]; c[bi] = -INFINITY; }
        __syncwarp();
    }
}

// u [T, experts * 2 * ff] holds per expert e the rows [gate_e (ff) | up_e (ff)]; y[t, e * ff + f] = silu(gate) * up * w[t, e]:
// exact zeros for the experts a token does not use, so ONE down projection over the concatenated experts sums the chosen ones.
template <typename T>
__global__ void moe_silu_glu_scale_kernel(const T* __restrict__ u, const float* __restrict__ w, T* __restrict__ y, int64_t n,
                                          int experts, int ff) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t cols = (int64_t)experts * ff;
    const int64_t t = i / cols;
    const int64_t c = i - t * cols;
    const int e = (int)(c / ff), f = (int)(c - (int64_t)e * ff);
    const float wt = w[t * experts + e];
    if (wt == 0.f) { stf(y + i, 0.f); return; }
    const T* ur = u + t * 2 * cols + (int64_t)e * 2 * ff;
    const float g = ldf(ur + f), v = ldf(ur + ff + f);
    stf(y + i, g / (1.f + expf(-g)) * v * wt);
}

}  // namespace sllm

using namespace sllm;

extern "C" {

int sllm_embed_pair_hash(const void* tokens, const void* tok_seq, const void* tok_pos, const void* last_token, const void* embed,
                         const void* pairs, int buckets, int64_t mul_prev, int64_t mul_cur, void* x, void* x_copy, void* h,
                         int64_t num_tokens, int width, sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && width > 0 && (pairs == nullptr || buckets > 0), "embed_pair_hash: bad shape");
    if (num_tokens == 0) return 0;
    SLLM_REQUIRE(tokens && tok_seq && tok_pos && embed && x && h && (pairs == nullptr || last_token), "embed_pair_hash: null pointer");
    SLLM_DISPATCH_DTYPE_F32(dtype, (embed_pair_hash_kernel<T><<<(unsigned)num_tokens, 256, 0, (cudaStream_t)stream>>>(
        (const int*)tokens, (const int*)tok_seq, (const int*)tok_pos, (const int*)last_token, (const T*)embed, (const T*)pairs,
        buckets, mul_prev, mul_cur, (float*)x, (float*)x_copy, (T*)h, width)));
    return check_launch("embed_pair_hash");
}

int sllm_store_last_tokens(const void* tokens, const void* seg_starts, const void* seq_ids, void* last_token, int num_segs,
                           sllm_stream_t stream) {
    if (num_segs <= 0) return 0;
    SLLM_REQUIRE(tokens && seg_starts && seq_ids && last_token, "store_last_tokens: null pointer");
    store_last_tokens_kernel<<<(unsigned)cdiv(num_segs, 128), 128, 0, (cudaStream_t)stream>>>(
        (const int*)tokens, (const int*)seg_starts, (const int*)seq_ids, (int*)last_token, num_segs);
    return check_launch("store_last_tokens");
}

int sllm_postnorm_add_mix(void* x, const void* y, const void* gain, float eps, void* history, int slot, const void* mix, void* h,
                          int64_t num_tokens, int width, sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && width > 0 && slot >= 0, "postnorm_add_mix: bad shape");
    if (num_tokens == 0) return 0;
    SLLM_REQUIRE(x && h && (y == nullptr || gain) && (mix == nullptr || history), "postnorm_add_mix: null pointer");
    SLLM_DISPATCH_DTYPE_F32(dtype, (postnorm_add_mix_kernel<T><<<(unsigned)num_tokens, 256, 0, (cudaStream_t)stream>>>(
        (float*)x, (const T*)y, (const float*)gain, eps, (float*)history, slot, num_tokens * (int64_t)width, (const float*)mix,
        (T*)h, width)));
    return check_launch("postnorm_add_mix");
}

int sllm_tanh_cap_inplace(void* x, int64_t n, float cap, sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(n >= 0 && cap > 0.f, "tanh_cap_inplace: need a positive cap");
    if (n == 0) return 0;
    SLLM_REQUIRE(x, "tanh_cap_inplace: null pointer");
    SLLM_DISPATCH_DTYPE_F32(dtype, (tanh_cap_kernel<T><<<(unsigned)cdiv(n, 256), 256, 0, (cudaStream_t)stream>>>((T*)x, n, cap)));
    return check_launch("tanh_cap_inplace");
}

int sllm_moe_route_sigmoid(const void* logits, const void* bias, void* weights, int64_t num_tokens, int experts, int top,
                           sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && experts > 0 && top > 0 && top <= experts && experts <= 2048,
                 "moe_route_sigmoid: need 0 < top <= experts <= 2048 (got top %d, experts %d)", top, experts);
    if (num_tokens == 0) return 0;
    SLLM_REQUIRE(logits && weights, "moe_route_sigmoid: null pointer");
    moe_route_sigmoid_kernel<<<(unsigned)cdiv(num_tokens, 4), 128, 4 * 2 * experts * sizeof(float), (cudaStream_t)stream>>>(
        (const float*)logits, (const float*)bias, (float*)weights, num_tokens, experts, top);
    return check_launch("moe_route_sigmoid");
}

int sllm_moe_silu_glu_scale(const void* u, const void* weights, void* y, int64_t num_tokens, int experts, int ff,
                            sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && experts > 0 && ff > 0, "moe_silu_glu_scale: bad shape");
    const int64_t n = num_tokens * (int64_t)experts * ff;
    if (n == 0) return 0;
    SLLM_REQUIRE(u && y && weights, "moe_silu_glu_scale: null pointer");
    SLLM_DISPATCH_DTYPE_F32(dtype, (moe_silu_glu_scale_kernel<T><<<(unsigned)cdiv(n, 256), 256, 0, (cudaStream_t)stream>>>(
        (const T*)u, (const float*)weights, (T*)y, n, experts, ff)));
    return check_launch("moe_silu_glu_scale");
}

}  // extern "C"
