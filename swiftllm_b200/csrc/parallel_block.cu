// Element-wise and row-wise kernels of PARALLEL decoder blocks (one norm feeds the mixer and the feed-forward, both are added
// to the residual): an fp32 residual stream with the add fused into the next RMS norm, a row-strided RMS norm for the slices
// of a fused projection, the squared-ReLU activation, and the router of a mixture of experts (top-k + softmax over the
// chosen logits) with the activation that applies the routing weight.  Sums, norms and the router run in fp32 whatever the
// storage type T (half, bf16 or float) of the projections is.
// Algorithmic bytes (s = sizeof(T)): add_rmsnorm 8*T*W + 3*T*W*s (residual read + write, two addends, one output).
#include "typed_io.cuh"

namespace sllm {

// residual[t] += a[t] + b[t] (either may be null); out[t] = residual[t] / sqrt(mean(residual[t]^2) + eps) * weight
// (WT: storage type of the weight - T, or float for models whose norm weights are kept in 32-bit)
template <typename T, typename WT>
__global__ void __launch_bounds__(256) add_rmsnorm_f32_kernel(float* __restrict__ residual, const T* __restrict__ a,
                                                              const T* __restrict__ b, const WT* __restrict__ weight,
                                                              T* __restrict__ out, float eps, int width) {
    __shared__ float red[32];
    const int64_t t = blockIdx.x;
    float* xr = residual + t * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float x = xr[i];
        if (a != nullptr || b != nullptr) {
            float y = a != nullptr ? ldf(a + t * width + i) : 0.f;
            if (b != nullptr) y += ldf(b + t * width + i);
            x += y;
            xr[i] = x;
        }
        ss += x * x;
    }
    const float denom = sqrtf(block_sum(ss, red) / (float)width + eps);
    // every thread re-reads only the elements it wrote itself
    for (int i = threadIdx.x; i < width; i += blockDim.x) stf(out + t * width + i, xr[i] / denom * ldf(weight + i));
}

// out[t, :n] = x[t, :n] / sqrt(mean(x[t, :n]^2) + eps) * weight ; rows of x and out may be slices of wider matrices
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_strided_kernel(const T* __restrict__ x, int64_t x_stride,
                                                              const T* __restrict__ weight, T* __restrict__ out,
                                                              int64_t out_stride, float eps, int n) {
    __shared__ float red[32];
    const T* xr = x + (int64_t)blockIdx.x * x_stride;
    T* orow = out + (int64_t)blockIdx.x * out_stride;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) { const float v = ldf(xr + i); ss += v * v; }
    const float denom = sqrtf(block_sum(ss, red) / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) stf(orow + i, ldf(xr + i) / denom * ldf(weight + i));
}

template <typename T>
__global__ void relu2_kernel(T* __restrict__ x, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) { const float v = fmaxf(ldf(x + i), 0.f); stf(x + i, v * v); }
}

// u[t, e * ff + f] = relu(u)^2 * w[t, e]: the activations of experts a token does not use become exact zeros, so ONE down
// projection over the concatenated experts yields the weighted sum of the chosen experts' outputs
template <typename T>
__global__ void moe_relu2_scale_kernel(T* __restrict__ u, const float* __restrict__ w, int64_t n, int experts, int ff) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t cols = (int64_t)experts * ff;
    const int64_t t = i / cols;
    const int e = (int)((i - t * cols) / ff);
    const float g = w[t * experts + e];
    const float v = fmaxf(ldf(u + i), 0.f);
    stf(u + i, g == 0.f ? 0.f : v * v * g);
}

// u [T, 2 * cols] holds per expert e the rows [gate_e (ff) | up_e (ff)], then the shared expert's [gate (sff) | up (sff)];
// y [T, cols], cols = experts * ff + sff.  With g = min(gate, limit), v = clamp(up, -limit, limit):
//     y = g * sigmoid(alpha * g) * (v + 1) * w[t, e]        (the shared expert has its own limit and weight 1)
// so that ONE down projection over the concatenated experts yields the weighted sum of the chosen experts plus the shared one.
template <typename T>
__global__ void moe_clamped_glu_scale_kernel(const T* __restrict__ u, const float* __restrict__ w, T* __restrict__ y, int64_t n,
                                             int experts, int ff, float limit, int sff, float shared_limit, float alpha,
                                             int shared_gated) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t cols = (int64_t)experts * ff + sff;
    const int64_t t = i / cols;
    const int64_t c = i - t * cols;
    const T* ur = u + t * 2 * cols;
    float wt, lim, g, v;
    if (c < (int64_t)experts * ff) {
        const int e = (int)(c / ff), f = (int)(c - (int64_t)e * ff);
        wt = w[t * (experts + shared_gated) + e];
        if (wt == 0.f) { stf(y + i, 0.f); return; }
        lim = limit;
        g = ldf(ur + (int64_t)e * 2 * ff + f);
        v = ldf(ur + (int64_t)e * 2 * ff + ff + f);
    } else {
        const int f = (int)(c - (int64_t)experts * ff);
        wt = shared_gated ? w[t * (experts + 1) + experts] : 1.f;      // a gated shared expert: the weights' extra last column
        lim = shared_limit;
        g = ldf(ur + (int64_t)experts * 2 * ff + f);
        v = ldf(ur + (int64_t)experts * 2 * ff + sff + f);
    }
    g = fminf(g, lim);
    v = fminf(fmaxf(v, -lim), lim);
    stf(y + i, g / (1.f + expf(-alpha * g)) * (v + 1.f) * wt);
}

// One warp per token, group-limited routing on scores that are a softmax over ALL experts:
//   s = softmax(logits);  experts form `groups` equal groups of neighbours, a group's score is its largest s, only experts of
//   the `keep` best groups can be chosen;  the `top` largest s among those are chosen (equal values: the lower index wins);
//   weights[t, e] = s_e / (sum of the chosen s + norm_eps) * scale at the chosen experts, 0 elsewhere.
// Dynamic shared memory: warps * (2 * experts + groups) floats.
__global__ void __launch_bounds__(128) moe_route_grouped_kernel(const float* __restrict__ logits, float* __restrict__ weights,
                                                                int64_t num_tokens, int experts, int top, int groups, int keep,
                                                                float scale, float norm_eps) {
    extern __shared__ float vals[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= num_tokens) return;
    float* s = vals + warp * (2 * experts + groups);      // scores
    float* c = s + experts;                               // choice scores (-inf: may not be chosen)
    float* gs = c + experts;                              // group scores
    float mx = -INFINITY;
    for (int e = lane; e < experts; e += 32) { s[e] = logits[t * experts + e]; mx = fmaxf(mx, s[e]); weights[t * experts + e] = 0.f; }
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < experts; e += 32) { s[e] = expf(s[e] - mx); sum += s[e]; }
    sum = warp_sum(sum);
    for (int e = lane; e < experts; e += 32) { s[e] /= sum; c[e] = -INFINITY; }
    __syncwarp();
    const int per = experts / groups;
    for (int g = lane; g < groups; g += 32) {
        float b = -INFINITY;
        for (int e = g * per; e < (g + 1) * per; e++) b = fmaxf(b, s[e]);
        gs[g] = b;
    }
    __syncwarp();
    for (int k = 0; k < keep; k++) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int g = lane; g < groups; g += 32)
            if (gs[g] > best) { best = gs[g]; bi = g; }
        if (best == -INFINITY) bi = 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (bi != 0x7fffffff) {
            for (int e = bi * per + lane; e < (bi + 1) * per; e += 32) c[e] = s[e];
            if (lane == 0) gs[bi] = -INFINITY;
        }
        __syncwarp();
    }
    float my_val = 0.f;            // lane k keeps the k-th choice
    int my_idx = -1;
    for (int k = 0; k < top; k++) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < experts; e += 32)
            if (c[e] > best) { best = c[e]; bi = e; }
        if (best == -INFINITY) bi = 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (lane == k && bi != 0x7fffffff) { my_val = s[bi]; my_idx = bi; }
        __syncwarp();
        if (lane == 0 && bi != 0x7fffffff) c[bi] = -INFINITY;
        __syncwarp();
    }
    const float total = warp_sum(my_idx >= 0 ? my_val : 0.f);
    if (my_idx >= 0) weights[t * experts + my_idx] = my_val / (total + norm_eps) * scale;
}

// One warp per token.  weights[t, e] = softmax over the `top` largest logits of row t at their experts, 0 elsewhere
// (equal logits: the lower expert index wins).  Dynamic shared memory: warps * experts floats.
__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, float* __restrict__ weights,
                                                        int64_t num_tokens, int experts, int top) {
    extern __shared__ float vals[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= num_tokens) return;
    float* v = vals + warp * experts;
    for (int e = lane; e < experts; e += 32) { v[e] = logits[t * experts + e]; weights[t * experts + e] = 0.f; }
    __syncwarp();
    float my_val = -INFINITY;      // lane k keeps the k-th choice
    int my_idx = -1;
    for (int k = 0; k < top; k++) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            const float x = v[e];
            if (x > best) { best = x; bi = e; }          // ascending e: the first of equal values stays
        }
        if (best == -INFINITY) bi = 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (lane == k) { my_val = best; my_idx = bi; }
        if (lane == 0 && bi != 0x7fffffff) v[bi] = -INFINITY;
        __syncwarp();
    }
    const float m = __shfl_sync(0xffffffffu, my_val, 0);       // the first choice is the largest
    const float p = (lane < top && my_idx != 0x7fffffff) ? expf(my_val - m) : 0.f;
    const float sum = warp_sum(p);
    __syncwarp();
    if (lane < top && my_idx != 0x7fffffff) weights[t * experts + my_idx] = p / sum;
}

}  // namespace sllm

using namespace sllm;

extern "C" {

int sllm_add_rmsnorm_f32(void* residual, const void* a, const void* b, const void* weight, void* out, float eps,
                         int64_t num_tokens, int width, sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && width > 0, "add_rmsnorm_f32: bad shape");
    if (num_tokens == 0) return 0;
    SLLM_REQUIRE(residual && weight && out, "add_rmsnorm_f32: null pointer");
    SLLM_DISPATCH_DTYPE_F32(dtype, (add_rmsnorm_f32_kernel<T, T><<<(unsigned)num_tokens, 256, 0, (cudaStream_t)stream>>>(
        (float*)residual, (const T*)a, (const T*)b, (const T*)weight, (T*)out, eps, width)));
    return check_launch("add_rmsnorm_f32");
}

int sllm_add_rmsnorm_f32w(void* residual, const void* a, const void* b, const void* weight_f32, void* out, float eps,
                          int64_t num_tokens, int width, sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && width > 0, "add_rmsnorm_f32w: bad shape");
    if (num_tokens == 0) return 0;
    SLLM_REQUIRE(residual && weight_f32 && out, "add_rmsnorm_f32w: null pointer");
    SLLM_DISPATCH_DTYPE_F32(dtype, (add_rmsnorm_f32_kernel<T, float><<<(unsigned)num_tokens, 256, 0, (cudaStream_t)stream>>>(
        (float*)residual, (const T*)a, (const T*)b, (const float*)weight_f32, (T*)out, eps, width)));
    return check_launch("add_rmsnorm_f32w");
}

int sllm_rmsnorm_strided(const void* x, int64_t x_row_stride, const void* weight, void* out, int64_t out_row_stride,
                         float eps, int64_t num_tokens, int n, sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && n > 0 && x_row_stride >= n && out_row_stride >= n, "rmsnorm_strided: bad shape");
    if (num_tokens == 0) return 0;
    SLLM_REQUIRE(x && weight && out, "rmsnorm_strided: null pointer");
    SLLM_DISPATCH_DTYPE_F32(dtype, (rmsnorm_strided_kernel<T><<<(unsigned)num_tokens, n >= 256 ? 256 : 64, 0, (cudaStream_t)stream>>>(
        (const T*)x, x_row_stride, (const T*)weight, (T*)out, out_row_stride, eps, n)));
    return check_launch("rmsnorm_strided");
}

int sllm_relu2_inplace(void* x, int64_t n, sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(n >= 0, "relu2: bad size");
    if (n == 0) return 0;
    SLLM_REQUIRE(x, "relu2: null pointer");
    SLLM_DISPATCH_DTYPE_F32(dtype, (relu2_kernel<T><<<(unsigned)cdiv(n, 256), 256, 0, (cudaStream_t)stream>>>((T*)x, n)));
    return check_launch("relu2_inplace");
}

int sllm_moe_route(const void* logits, void* weights, int64_t num_tokens, int experts, int top, sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && experts > 0 && top > 0 && top <= experts && top <= 32 && experts <= 2048,
                 "moe_route: need 0 < top <= min(experts, 32) and experts <= 2048 (got top %d, experts %d)", top, experts);
    if (num_tokens == 0) return 0;
    SLLM_REQUIRE(logits && weights, "moe_route: null pointer");
    moe_route_kernel<<<(unsigned)cdiv(num_tokens, 4), 128, 4 * experts * sizeof(float), (cudaStream_t)stream>>>(
        (const float*)logits, (float*)weights, num_tokens, experts, top);
    return check_launch("moe_route");
}

int sllm_moe_route_grouped(const void* logits, void* weights, int64_t num_tokens, int experts, int top, int groups, int keep,
                           float scale, float norm_eps, sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && experts > 0 && top > 0 && top <= experts && top <= 32 && experts <= 2048 && groups > 0 &&
                 experts % groups == 0 && keep > 0 && keep <= groups && top <= keep * (experts / groups),
                 "moe_route_grouped: need 0 < top <= min(32, keep * experts / groups), experts <= 2048 in equal groups "
                 "(got top %d, experts %d, groups %d, keep %d)", top, experts, groups, keep);
    if (num_tokens == 0) return 0;
    SLLM_REQUIRE(logits && weights, "moe_route_grouped: null pointer");
    moe_route_grouped_kernel<<<(unsigned)cdiv(num_tokens, 4), 128, 4 * (2 * experts + groups) * sizeof(float),
                               (cudaStream_t)stream>>>((const float*)logits, (float*)weights, num_tokens, experts, top, groups,
                                                       keep, scale, norm_eps);
    return check_launch("moe_route_grouped");
}

int sllm_moe_clamped_glu_scale(const void* u, const void* weights, void* y, int64_t num_tokens, int experts, int ff, float limit,
                               int shared_ff, float shared_limit, float alpha, int shared_gated, sllm_dtype_t dtype,
                               sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && experts >= 0 && ff >= 0 && shared_ff >= 0 && (int64_t)experts * ff + shared_ff > 0,
                 "moe_clamped_glu_scale: bad shape");
    const int64_t n = num_tokens * ((int64_t)experts * ff + shared_ff);
    if (n == 0) return 0;
    SLLM_REQUIRE(u && y && (weights || (experts == 0 && !shared_gated)), "moe_clamped_glu_scale: null pointer");
    shared_gated = shared_gated ? 1 : 0;
    SLLM_DISPATCH_DTYPE_F32(dtype, (moe_clamped_glu_scale_kernel<T><<<(unsigned)cdiv(n, 256), 256, 0, (cudaStream_t)stream>>>(
        (const T*)u, (const float*)weights, (T*)y, n, experts, ff, limit, shared_ff, shared_limit, alpha, shared_gated)));
    return check_launch("moe_clamped_glu_scale");
}

int sllm_moe_relu2_scale_inplace(void* u, const void* weights, int64_t num_tokens, int experts, int ff, sllm_dtype_t dtype,
                                 sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && experts > 0 && ff > 0, "moe_relu2_scale: bad shape");
    const int64_t n = num_tokens * experts * ff;
    if (n == 0) return 0;
    SLLM_REQUIRE(u && weights, "moe_relu2_scale: null pointer");
    SLLM_DISPATCH_DTYPE_F32(dtype, (moe_relu2_scale_kernel<T><<<(unsigned)cdiv(n, 256), 256, 0, (cudaStream_t)stream>>>(
        (T*)u, (const float*)weights, n, experts, ff)));
    return check_launch("moe_relu2_scale_inplace");
}

}  // extern "C"
