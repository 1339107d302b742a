// Row-wise kernels of SANDWICH decoder blocks: a sublayer reads norm_a(x) and its output goes through a second norm before it is
// added, x <- x + mult * norm_b(sublayer(norm_a(x))).  Every norm is an RMS norm over `groups` equal consecutive parts of the row
// (each part divided by its own sqrt(mean of squares + eps)) times one weight vector.  Also here: adding a saved stream and a row
// vector to the stream (repeated passes over a range of layers), the GELU (tanh form) gated linear unit, and the router of a
// mixture of experts whose weights are plain softmax scores of the chosen experts with an optional per-token sigmoid weight for
// a shared expert.
// The stream, norms and the router are fp32 whatever the storage type T (half, bf16 or float) of the projections is.
// Algorithmic bytes (s = sizeof(T)): group_norm_add_norm  T*W*(s + 8 + 4) ; gelu_glu  T*F*3s.
#include "typed_io.cuh"

namespace sllm {

// One warp per (token, group).  With y: x <- x + mult * y / rms_g(y) * wb.  With wn: n = x / rms_g(x) * wn (fp32).
template <typename T>
__global__ void __launch_bounds__(256) group_norm_add_norm_kernel(float* __restrict__ x, const T* __restrict__ y,
                                                                  const float* __restrict__ wb, float mult,
                                                                  const float* __restrict__ wn, float* __restrict__ n_out,
                                                                  float eps, int64_t rows, int width, int groups) {
    const int lane = threadIdx.x & 31;
    const int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= rows * groups) return;
    const int64_t t = unit / groups;
    const int g = (int)(unit - t * groups), gw = width / groups;
    const int64_t base = t * width + (int64_t)g * gw;
    const int c0 = g * gw;
    float ssx = 0.f;
    if (y != nullptr) {
        float ss = 0.f;
        for (int i = lane; i < gw; i += 32) { const float v = ldf(y + base + i); ss += v * v; }
        const float f = mult / sqrtf(warp_sum(ss) / (float)gw + eps);
        for (int i = lane; i < gw; i += 32) {
            const float v = x[base + i] + f * ldf(y + base + i) * wb[c0 + i];
            x[base + i] = v;
            ssx += v * v;
        }
    } else if (wn != nullptr) {
        for (int i = lane; i < gw; i += 32) { const float v = x[base + i]; ssx += v * v; }
    }
    if (wn == nullptr) return;
    const float inv = 1.f / sqrtf(warp_sum(ssx) / (float)gw + eps);
    for (int i = lane; i < gw; i += 32) n_out[base + i] = x[base + i] * inv * wn[c0 + i];     // each lane re-reads what it wrote
}

// The same norm with the result in the storage type (the head's input).
template <typename T>
__global__ void __launch_bounds__(256) group_norm_cast_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                              T* __restrict__ out, float eps, int64_t rows, int width, int groups) {
    const int lane = threadIdx.x & 31;
    const int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= rows * groups) return;
    const int64_t t = unit / groups;
    const int g = (int)(unit - t * groups), gw = width / groups;
    const int64_t base = t * width + (int64_t)g * gw;
    float ss = 0.f;
    for (int i = lane; i < gw; i += 32) { const float v = x[base + i]; ss += v * v; }
    const float inv = 1.f / sqrtf(warp_sum(ss) / (float)gw + eps);
    for (int i = lane; i < gw; i += 32) stf(out + base + i, x[base + i] * inv * w[g * gw + i]);
}

// x[t] += a[t] (when given) + v (when given)
__global__ void stream_add_kernel(float* __restrict__ x, const float* __restrict__ a, const float* __restrict__ v, int64_t n, int width) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float s = x[i];
    if (a != nullptr) s += a[i];
    if (v != nullptr) s += v[i % width];
    x[i] = s;
}

__device__ __forceinline__ float gelu_tanh_fn(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// u [T, 2 F] = [gate | up] -> y [T, F] = gelu_tanh(gate) * up
template <typename T>
__global__ void gelu_glu_kernel(const T* __restrict__ u, T* __restrict__ y, int64_t n, int ff) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t t = i / ff;
    const int f = (int)(i - t * ff);
    const T* ur = u + t * 2 * ff;
    stf(y + i, gelu_tanh_fn(ldf(ur + f)) * ldf(ur + ff + f));
}

// One warp per token.  logits [T, experts (+ 1)]: s = softmax over the experts; the `top` experts with the largest s (equal
// values: the lower index) get weight s, the others 0; with `gated` the extra last column becomes its sigmoid.
// Dynamic shared memory: warps * experts floats.
__global__ void __launch_bounds__(128) moe_route_softmax_kernel(const float* __restrict__ logits, float* __restrict__ weights,
                                                                int64_t num_tokens, int experts, int top, int gated) {
    extern __shared__ float vals[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= num_tokens) return;
    const int cols = experts + (gated ? 1 : 0);
    float* s = vals + warp * experts;
    const float* lr = logits + t * cols;
    float* wr = weights + t * cols;
    float mx = -INFINITY;
    for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, lr[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < experts; e += 32) { const float p = expf(lr[e] - mx); s[e] = p; sum += p; }
    sum = warp_sum(sum);
    for (int e = lane; e < experts; e += 32) { s[e] = s[e] / sum; wr[e] = 0.f; }
    if (gated && lane == 0) wr[experts] = 1.f / (1.f + expf(-lr[experts]));
    __syncwarp();
    for (int k = 0; k < top; k++) {
        float best = -1.f;
        int arg = 0x7fffffff;
        for (int e = lane; e < experts; e += 32)
            if (s[e] > best) { best = s[e]; arg = e; }       // strictly larger: the lowest index of equal values stays
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (lane == 0) { wr[arg] = best; s[arg] = -2.f; }
        __syncwarp();
    }
}

}  // namespace sllm

using namespace sllm;

extern "C" {

int sllm_group_norm_add_norm(void* x, const void* y, const void* wb, float mult, const void* wn, void* n_out, float eps,
                             int64_t num_tokens, int width, int groups, sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && width > 0 && groups > 0 && width % groups == 0, "group_norm_add_norm: width %d in %d groups",
                 width, groups);
    if (num_tokens == 0) return 0;
    SLLM_REQUIRE(x && (y == nullptr || wb) && (wn == nullptr || n_out) && (y || wn), "group_norm_add_norm: null pointer");
    const int64_t units = num_tokens * groups;
    SLLM_DISPATCH_DTYPE_F32(dtype, (group_norm_add_norm_kernel<T><<<(unsigned)cdiv(units, 8), 256, 0, (cudaStream_t)stream>>>(
        (float*)x, (const T*)y, (const float*)wb, mult, (const float*)wn, (float*)n_out, eps, num_tokens, width, groups)));
    return check_launch("group_norm_add_norm");
}

int sllm_group_norm_cast(const void* x, const void* w, void* out, float eps, int64_t num_tokens, int width, int groups,
                         sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && width > 0 && groups > 0 && width % groups == 0, "group_norm_cast: width %d in %d groups", width,
                 groups);
    if (num_tokens == 0) return 0;
    SLLM_REQUIRE(x && w && out, "group_norm_cast: null pointer");
    const int64_t units = num_tokens * groups;
    SLLM_DISPATCH_DTYPE_F32(dtype, (group_norm_cast_kernel<T><<<(unsigned)cdiv(units, 8), 256, 0, (cudaStream_t)stream>>>(
        (const float*)x, (const float*)w, (T*)out, eps, num_tokens, width, groups)));
    return check_launch("group_norm_cast");
}

int sllm_stream_add(void* x, const void* a, const void* v, int64_t num_tokens, int width, sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && width > 0, "stream_add: bad shape");
    const int64_t n = num_tokens * width;
    if (n == 0 || (a == nullptr && v == nullptr)) return 0;
    SLLM_REQUIRE(x, "stream_add: null pointer");
    stream_add_kernel<<<(unsigned)cdiv(n, 256), 256, 0, (cudaStream_t)stream>>>((float*)x, (const float*)a, (const float*)v, n, width);
    return check_launch("stream_add");
}

int sllm_gelu_glu(const void* u, void* y, int64_t num_tokens, int ff, sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && ff > 0, "gelu_glu: bad shape");
    const int64_t n = num_tokens * ff;
    if (n == 0) return 0;
    SLLM_REQUIRE(u && y, "gelu_glu: null pointer");
    SLLM_DISPATCH_DTYPE_F32(dtype, (gelu_glu_kernel<T><<<(unsigned)cdiv(n, 256), 256, 0, (cudaStream_t)stream>>>(
        (const T*)u, (T*)y, n, ff)));
    return check_launch("gelu_glu");
}

int sllm_moe_route_softmax(const void* logits, void* weights, int64_t num_tokens, int experts, int top, int gated,
                           sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && experts > 0 && top > 0 && top <= experts && experts <= 4096,
                 "moe_route_softmax: %d of %d experts", top, experts);
    if (num_tokens == 0) return 0;
    SLLM_REQUIRE(logits && weights, "moe_route_softmax: null pointer");
    moe_route_softmax_kernel<<<(unsigned)cdiv(num_tokens, 4), 128, 4 * (size_t)experts * sizeof(float), (cudaStream_t)stream>>>(
        (const float*)logits, (float*)weights, num_tokens, experts, top, gated);
    return check_launch("moe_route_softmax");
}

}  // extern "C"
