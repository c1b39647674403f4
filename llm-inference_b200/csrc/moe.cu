// Mixture-of-experts plumbing around b200_gemm_grouped: routers (softmax over all outputs with a corrected choice and
// identity experts; or a choice on the biased logits with a softmax over the chosen ones), counting sort of the (token, choice) pairs by expert, and the fp32 residual update that gathers every
// token's expert rows back in a fixed order (no atomics: a token's sum does not depend on the batch around it).
#include "b200_serve.h"
#include "common.cuh"
#include "launch_count.h"

namespace b200 {

// one CTA per token: 16 warps compute the router outputs (fp32 dot over the width, eight loads in flight per lane),
// thread 0 the softmax and the choice
template <typename T>
__global__ void __launch_bounds__(512) moe_route_kernel(const T* __restrict__ h, const float* __restrict__ wr,
                                                        const float* __restrict__ corr, const float* __restrict__ bias,
                                                        int on_logits, int width, int n_out, int top,
                                                        float scale, int* __restrict__ chosen, float* __restrict__ weight) {
    extern __shared__ float z[];   // z[n_out] | pick[n_out] | x[width]
    float* pick = z + n_out;
    float* xs = pick + n_out;
    const int t = blockIdx.x, warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const T* x = h + (size_t)t * width;
    // the token's input once in shared memory as fp32, then four independent partial sums per lane
    for (int i = threadIdx.x; i < width; i += blockDim.x) xs[i] = DT<T>::to_f(x[i]);
    __syncthreads();
    const int nw = blockDim.x / 32;
    for (int o = warp; o < n_out; o += nw) {
        const float* w = wr + (size_t)o * width;
        float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
        int i = lane;
        for (; i + 224 < width; i += 256) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = w[i + 32 * u];
            d0 = fmaf(xs[i], v[0], d0);
            d1 = fmaf(xs[i + 32], v[1], d1);
            d2 = fmaf(xs[i + 64], v[2], d2);
            d3 = fmaf(xs[i + 96], v[3], d3);
            d0 = fmaf(xs[i + 128], v[4], d0);
            d1 = fmaf(xs[i + 160], v[5], d1);
            d2 = fmaf(xs[i + 192], v[6], d2);
            d3 = fmaf(xs[i + 224], v[7], d3);
        }
        for (; i < width; i += 32) d0 = fmaf(xs[i], w[i], d0);
        float d = (d0 + d1) + (d2 + d3);
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) d += __shfl_xor_sync(0xffffffffu, d, s);
        if (lane == 0) z[o] = d + (bias ? bias[o] : 0.f);
    }
    __syncthreads();
    if (threadIdx.x == 0 && on_logits) {   // the `top` largest logits, then a softmax over those alone
        float m = -INFINITY, den = 0.f;
        for (int k = 0; k < top; ++k) {
            int best = 0;
            float bv = -INFINITY;
            for (int o = 0; o < n_out; ++o)
                if (z[o] > bv) { bv = z[o]; best = o; }   // ties: lower index
            z[best] = -INFINITY;
            if (k == 0) m = bv;                            // the first pick is the largest
            chosen[(size_t)t * top + k] = best;
            pick[k] = expf(bv - m);
            den += pick[k];
        }
        for (int k = 0; k < top; ++k) weight[(size_t)t * top + k] = pick[k] / den;
    } else if (threadIdx.x == 0) {
        float m = -INFINITY, den = 0.f;
        for (int o = 0; o < n_out; ++o) m = fmaxf(m, z[o]);
        for (int o = 0; o < n_out; ++o) { z[o] = expf(z[o] - m); den += z[o]; }
        const float inv = 1.0f / den;
        for (int o = 0; o < n_out; ++o) { z[o] *= inv; pick[o] = z[o] + corr[o]; }
        for (int k = 0; k < top; ++k) {
            int best = 0;
            float bv = -INFINITY;
            for (int o = 0; o < n_out; ++o)
                if (pick[o] > bv) { bv = pick[o]; best = o; }   // ties: lower index
            pick[best] = -INFINITY;
            chosen[(size_t)t * top + k] = best;
            weight[(size_t)t * top + k] = z[best] * scale;
        }
    }
}

// single CTA: counts -> exclusive offsets -> placement. Row order inside a group is arbitrary; every row's result is
// computed independently of its neighbours, so the order does not reach the output.
__global__ void __launch_bounds__(1024) moe_dispatch_kernel(const int* __restrict__ chosen, int n_pairs, int n_experts,
                                                            int top, int* __restrict__ group_off, int* __restrict__ src_row,
                                                            int* __restrict__ dest) {
    extern __shared__ int cnt[];   // count[n_experts] | cursor[n_experts]
    int* cursor = cnt + n_experts;
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int e = chosen[i];
        if (e < n_experts) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int e = 0; e < n_experts; ++e) {
            group_off[e] = acc;
            cursor[e] = acc;
            acc += cnt[e];
        }
        group_off[n_experts] = acc;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int e = chosen[i];
        int d = -1;
        if (e < n_experts) {
            d = atomicAdd(&cursor[e], 1);
            src_row[d] = i / top;
        }
        dest[i] = d;
    }
}

template <typename T>
__global__ void __launch_bounds__(256) residual_combine_kernel(float* __restrict__ x, const float* __restrict__ mix,
                                                               const float* __restrict__ shared, const float* __restrict__ eo,
                                                               const int* __restrict__ dest, const float* __restrict__ weight,
                                                               const T* __restrict__ h, int width, int top) {
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const size_t i = (size_t)t * width + c;
        float y = mix ? mix[i] : 0.f;
        if (dest) {
            float r = 0.f;
            for (int k = 0; k < top; ++k) {
                const int d = dest[(size_t)t * top + k];
                const float v = d >= 0 ? eo[(size_t)d * width + c] : DT<T>::to_f(h[i]);
                r = fmaf(weight[(size_t)t * top + k], v, r);
            }
            y += r;
        }
        if (shared) y += shared[i];
        x[i] += y;
    }
}

// dst[i, :] = src[rows[i], :]: the rows of every expert's group side by side, so that a dense GEMM can read a group
__global__ void __launch_bounds__(256) gather_rows_kernel(const unsigned char* __restrict__ src, const int* __restrict__ rows,
                                                         unsigned char* __restrict__ dst, size_t row_bytes, int vec) {
    const unsigned char* s = src + (size_t)rows[blockIdx.x] * row_bytes;
    unsigned char* d = dst + (size_t)blockIdx.x * row_bytes;
    if (vec) {
        for (size_t i = (size_t)threadIdx.x * 16; i < row_bytes; i += (size_t)blockDim.x * 16) st16(d + i, ld16(s + i));
    } else {
        for (size_t i = threadIdx.x; i < row_bytes; i += blockDim.x) d[i] = s[i];
    }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_gather_rows(const void* src, const int* rows, void* dst, int n_rows, int width, int dtype, void* stream) {
    if (!src || !rows || !dst || n_rows < 0 || width < 1 || (dtype != B200_BF16 && dtype != B200_F32)) return B200_EINVAL;
    if (n_rows == 0) return B200_OK;
    const size_t row_bytes = (size_t)width * (dtype == B200_BF16 ? 2 : 4);
    const int vec = row_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0;
    gather_rows_kernel<<<n_rows, 256, 0, (cudaStream_t)stream>>>((const unsigned char*)src, rows, (unsigned char*)dst, row_bytes, vec);
    count_launch();
    return (int)cudaGetLastError();
}

extern "C" int b200_moe_route(const void* h, int h_dtype, const float* w_router, const float* correction, int n_tokens,
                              int width, int n_out, int top, float scale, int* chosen, float* weight, void* stream) {
    if (!h || !w_router || !correction || !chosen || !weight || n_tokens < 0 || width < 1 || n_out < 1 || top < 1 || top > n_out)
        return B200_EINVAL;
    if (n_out > 4096) return B200_EUNSUPPORTED;
    if (n_tokens == 0) return B200_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = ((size_t)2 * n_out + width) * sizeof(float);
    if (smem > 48 * 1024) return B200_EUNSUPPORTED;
    if (h_dtype == B200_BF16)
        moe_route_kernel<__nv_bfloat16><<<n_tokens, 512, smem, s>>>((const __nv_bfloat16*)h, w_router, correction, nullptr, 0, width, n_out, top,
                                                                   scale, chosen, weight);
    else if (h_dtype == B200_F32)
        moe_route_kernel<float><<<n_tokens, 512, smem, s>>>((const float*)h, w_router, correction, nullptr, 0, width, n_out, top, scale, chosen,
                                                           weight);
    else
        return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}

extern "C" int b200_moe_route_logits(const void* h, int h_dtype, const float* w_router, const float* bias, int n_tokens, int width,
                                     int n_out, int top, int* chosen, float* weight, void* stream) {
    if (!h || !w_router || !chosen || !weight || n_tokens < 0 || width < 1 || n_out < 1 || top < 1 || top > n_out) return B200_EINVAL;
    if (n_out > 4096) return B200_EUNSUPPORTED;
    if (n_tokens == 0) return B200_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = ((size_t)2 * n_out + width) * sizeof(float);
    if (smem > 48 * 1024) return B200_EUNSUPPORTED;
    if (h_dtype == B200_BF16)
        moe_route_kernel<__nv_bfloat16><<<n_tokens, 512, smem, s>>>((const __nv_bfloat16*)h, w_router, nullptr, bias, 1, width, n_out, top, 1.f,
                                                                   chosen, weight);
    else if (h_dtype == B200_F32)
        moe_route_kernel<float><<<n_tokens, 512, smem, s>>>((const float*)h, w_router, nullptr, bias, 1, width, n_out, top, 1.f, chosen, weight);
    else
        return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}

extern "C" int b200_moe_dispatch(const int* chosen, int n_tokens, int top, int n_experts, int* group_off, int* src_row,
                                 int* dest, void* stream) {
    if (!chosen || !group_off || !src_row || !dest || n_tokens < 0 || top < 1 || n_experts < 0) return B200_EINVAL;
    if (n_experts > 4096) return B200_EUNSUPPORTED;
    moe_dispatch_kernel<<<1, 1024, (size_t)2 * (n_experts + 1) * sizeof(int), (cudaStream_t)stream>>>(
        chosen, n_tokens * top, n_experts, top, group_off, src_row, dest);
    count_launch();
    return (int)cudaGetLastError();
}

extern "C" int b200_residual_combine(float* x, const float* mix, const float* shared, const float* expert_out, const int* dest,
                                     const float* weight, const void* h, int h_dtype, int n_tokens, int width, int top,
                                     void* stream) {
    if (!x || n_tokens < 0 || width < 1) return B200_EINVAL;
    if (dest && (!weight || !h || top < 1)) return B200_EINVAL;
    if (n_tokens == 0) return B200_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (h_dtype == B200_BF16)
        residual_combine_kernel<__nv_bfloat16><<<n_tokens, 256, 0, s>>>(x, mix, shared, expert_out, dest, weight,
                                                                       (const __nv_bfloat16*)h, width, top);
    else if (h_dtype == B200_F32)
        residual_combine_kernel<float><<<n_tokens, 256, 0, s>>>(x, mix, shared, expert_out, dest, weight, (const float*)h, width, top);
    else
        return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}
