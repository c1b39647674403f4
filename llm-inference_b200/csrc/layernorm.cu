// Embedding (with or without learned positions), layer norm (weight + bias) before a sublayer, and the sandwich form
// (norm of the sublayer's output added to the residual, then the next sublayer's input norm), beside norm.cu's RMS norms.
// The residual stream these kernels read and write is fp32; their outputs feed GEMMs and take the serving dtype.
#include "b200_serve.h"
#include "common.cuh"
#include "launch_count.h"

namespace b200 {

template <typename T>
__global__ void embed_positions_kernel(const int* __restrict__ ids, const int* __restrict__ pos, const T* __restrict__ table,
                                       const T* __restrict__ pos_table, float* __restrict__ out, int width) {
    const int t = blockIdx.x;
    const T* e = table + (size_t)ids[t] * width;
    if (!pos_table) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) out[(size_t)t * width + i] = DT<T>::to_f(e[i]);
        return;
    }
    const T* p = pos_table + (size_t)pos[t] * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) out[(size_t)t * width + i] = DT<T>::to_f(e[i]) + DT<T>::to_f(p[i]);
}

__device__ __forceinline__ float ln_block_sum(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, nw = blockDim.x / 32;
    __syncthreads();   // red may still be read from the previous call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float s = 0.f;
    for (int i = 0; i < nw; ++i) s += red[i];   // same order in every thread: one value per block
    return s;
}

// one CTA per row; the row is kept in shared memory between the passes (mean, then squared deviations, then output)
template <typename T>
__global__ void __launch_bounds__(256) layernorm_pair_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                                             int width, float eps, const float* __restrict__ w1,
                                                             const float* __restrict__ b1, T* __restrict__ out1,
                                                             const float* __restrict__ w2, const float* __restrict__ b2,
                                                             T* __restrict__ out2) {
    extern __shared__ float row[];
    __shared__ float red[8];
    const int i = blockIdx.x;
    const float* src = x + (size_t)(rows ? rows[i] : i) * width;
    float s = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = src[c];
        row[c] = v;
        s += v;
    }
    const float mean = ln_block_sum(s, red) / (float)width;
    float q = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float d = row[c] - mean;
        q += d * d;
    }
    const float rstd = 1.0f / sqrtf(ln_block_sum(q, red) / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float n = (row[c] - mean) * rstd;
        out1[(size_t)i * width + c] = DT<T>::from_f(n * w1[c] + b1[c]);
        if (out2) out2[(size_t)i * width + c] = DT<T>::from_f(n * w2[c] + b2[c]);
    }
}

// x += mult * LN(y; w, b); out2 = LN(x; w2, b2). One CTA per row; the row of y, then the new row of x, stay in shared memory.
template <typename T>
__global__ void __launch_bounds__(256) layernorm_residual_kernel(float* __restrict__ x, const float* __restrict__ y, int width,
                                                                 float eps, float mult, const float* __restrict__ w,
                                                                 const float* __restrict__ b, const float* __restrict__ w2,
                                                                 const float* __restrict__ b2, T* __restrict__ out2) {
    extern __shared__ float row[];
    __shared__ float red[8];
    const size_t base = (size_t)blockIdx.x * width;
    float s = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = y[base + c];
        row[c] = v;
        s += v;
    }
    float mean = ln_block_sum(s, red) / (float)width;
    float q = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float d = row[c] - mean;
        q += d * d;
    }
    float rstd = 1.0f / sqrtf(ln_block_sum(q, red) / (float)width + eps);
    s = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = x[base + c] + mult * ((row[c] - mean) * rstd * w[c] + b[c]);
        x[base + c] = v;
        row[c] = v;
        s += v;
    }
    if (!out2) return;
    mean = ln_block_sum(s, red) / (float)width;
    q = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float d = row[c] - mean;
        q += d * d;
    }
    rstd = 1.0f / sqrtf(ln_block_sum(q, red) / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) out2[base + c] = DT<T>::from_f((row[c] - mean) * rstd * w2[c] + b2[c]);
}

// the same for rows of at most 256 * kLnPerThread values: the row and every weight are loaded up front (one round trip to
// memory instead of three) and live in registers
constexpr int kLnPerThread = 8;
template <typename T>
__global__ void __launch_bounds__(256) layernorm_residual_reg_kernel(float* __restrict__ x, const float* __restrict__ y, int width,
                                                                     float eps, float mult, const float* __restrict__ w,
                                                                     const float* __restrict__ b, const float* __restrict__ w2,
                                                                     const float* __restrict__ b2, T* __restrict__ out2) {
    __shared__ float red[8];
    const size_t base = (size_t)blockIdx.x * width;
    float xv[kLnPerThread], yv[kLnPerThread], wv[kLnPerThread], bv[kLnPerThread], w2v[kLnPerThread], b2v[kLnPerThread];
#pragma unroll
    for (int k = 0; k < kLnPerThread; ++k) {
        const int c = threadIdx.x + 256 * k;
        const bool in = c < width;
        yv[k] = in ? y[base + c] : 0.f;
        xv[k] = in ? x[base + c] : 0.f;
        wv[k] = in ? w[c] : 0.f;
        bv[k] = in ? b[c] : 0.f;
        w2v[k] = in && out2 ? w2[c] : 0.f;
        b2v[k] = in && out2 ? b2[c] : 0.f;
    }
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < kLnPerThread; ++k) s += yv[k];
    float mean = ln_block_sum(s, red) / (float)width;
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < kLnPerThread; ++k) {
        const float d = threadIdx.x + 256 * k < width ? yv[k] - mean : 0.f;
        q += d * d;
    }
    float rstd = 1.0f / sqrtf(ln_block_sum(q, red) / (float)width + eps);
    s = 0.f;
#pragma unroll
    for (int k = 0; k < kLnPerThread; ++k) {
        const int c = threadIdx.x + 256 * k;
        if (c < width) {
            xv[k] += mult * ((yv[k] - mean) * rstd * wv[k] + bv[k]);
            x[base + c] = xv[k];
            s += xv[k];
        }
    }
    if (!out2) return;
    mean = ln_block_sum(s, red) / (float)width;
    q = 0.f;
#pragma unroll
    for (int k = 0; k < kLnPerThread; ++k) {
        const float d = threadIdx.x + 256 * k < width ? xv[k] - mean : 0.f;
        q += d * d;
    }
    rstd = 1.0f / sqrtf(ln_block_sum(q, red) / (float)width + eps);
#pragma unroll
    for (int k = 0; k < kLnPerThread; ++k) {
        const int c = threadIdx.x + 256 * k;
        if (c < width) out2[base + c] = DT<T>::from_f((xv[k] - mean) * rstd * w2v[k] + b2v[k]);
    }
}

template <typename T>
__global__ void concat_cast_kernel(const float* __restrict__ a, const float* __restrict__ b, T* __restrict__ out, int width) {
    const size_t t = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        out[t * 2 * width + c] = DT<T>::from_f(a[t * width + c]);
        out[t * 2 * width + width + c] = DT<T>::from_f(b[t * width + c]);
    }
}

// out[t, j] = act(gu[t, j]) * gu[t, n + j] (act: silu or gelu in its tanh form): the GLU of a [gate | up] product that was
// computed without the fused epilogue (small batches stream the stacked weight once through the split-K GEMM)
template <typename T>
__global__ void glu_act_kernel(const float* __restrict__ gu, T* __restrict__ out, int n, size_t total, int gelu) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / n, j = i - t * n;
    const float g = gu[t * 2 * n + j], u = gu[t * 2 * n + n + j];
    out[i] = DT<T>::from_f((gelu ? gelu_tanh_f(g) : g / (1.f + expf(-g))) * u);
}

template <typename T>
__global__ void glu_act_clamped_kernel(const float* __restrict__ gu, T* __restrict__ out, int n, size_t total, float limit) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / n, j = i - t * n;
    out[i] = DT<T>::from_f(glu_clamp_f(gu[t * 2 * n + j], gu[t * 2 * n + n + j], limit));
}

__global__ void scale_kernel(float* __restrict__ v, size_t n, float f) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) v[i] *= f;
}

// scaled token row plus the row of a hashed (previous token, token) table; a sequence's first token takes the table's last row
template <typename T>
__global__ void embed_pair_hash_kernel(const int* __restrict__ ids, const int* __restrict__ prev, const T* __restrict__ table, float scale,
                                       const T* __restrict__ pair_table, int buckets, int mul_prev, int mul_cur, float* __restrict__ out,
                                       T* __restrict__ out_cast, int width) {
    const int t = blockIdx.x;
    const T* e = table + (size_t)ids[t] * width;
    if (!pair_table) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float v = DT<T>::to_f(e[i]) * scale;
            out[(size_t)t * width + i] = v;
            if (out_cast) out_cast[(size_t)t * width + i] = DT<T>::from_f(v);
        }
        return;
    }
    long long row = buckets;
    if (prev[t] >= 0) {
        row = ((long long)prev[t] * mul_prev + (long long)ids[t] * mul_cur) % buckets;
        if (row < 0) row += buckets;
    }
    const T* p = pair_table + (size_t)row * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = DT<T>::to_f(e[i]) * scale + DT<T>::to_f(p[i]);
        out[(size_t)t * width + i] = v;
        if (out_cast) out_cast[(size_t)t * width + i] = DT<T>::from_f(v);
    }
}

__global__ void softcap_kernel(float* __restrict__ v, size_t n, float cap) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) v[i] = cap * tanhf(v[i] / cap);
}

}  // namespace b200

using namespace b200;

extern "C" int b200_layernorm_residual(float* x, const float* y, int n_rows, int width, float eps, float mult, const float* w,
                                       const float* b, const float* w2, const float* b2, void* out2, int out_dtype, void* stream) {
    if (!x || !y || !w || !b || n_rows < 0 || width < 1) return B200_EINVAL;
    if (out2 && (!w2 || !b2)) return B200_EINVAL;
    if (n_rows == 0) return B200_OK;
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return B200_EUNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (width <= 256 * kLnPerThread && (out_dtype == B200_BF16 || out_dtype == B200_F32)) {
        if (out_dtype == B200_BF16)
            layernorm_residual_reg_kernel<__nv_bfloat16><<<n_rows, 256, 0, s>>>(x, y, width, eps, mult, w, b, w2, b2, (__nv_bfloat16*)out2);
        else
            layernorm_residual_reg_kernel<float><<<n_rows, 256, 0, s>>>(x, y, width, eps, mult, w, b, w2, b2, (float*)out2);
        count_launch();
        return (int)cudaGetLastError();
    }
    if (out_dtype == B200_BF16) {
        static unsigned long long done = 0;
        if (smem > 48 * 1024) ensure_max_dynamic_smem((const void*)layernorm_residual_kernel<__nv_bfloat16>, 200 * 1024, done);
        layernorm_residual_kernel<__nv_bfloat16><<<n_rows, 256, smem, s>>>(x, y, width, eps, mult, w, b, w2, b2, (__nv_bfloat16*)out2);
    } else if (out_dtype == B200_F32) {
        static unsigned long long done = 0;
        if (smem > 48 * 1024) ensure_max_dynamic_smem((const void*)layernorm_residual_kernel<float>, 200 * 1024, done);
        layernorm_residual_kernel<float><<<n_rows, 256, smem, s>>>(x, y, width, eps, mult, w, b, w2, b2, (float*)out2);
    } else
        return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}

extern "C" int b200_concat_cast(const float* a, const float* b, void* out, int n_rows, int width, int out_dtype, void* stream) {
    if (!a || !b || !out || n_rows < 0 || width < 1) return B200_EINVAL;
    if (n_rows == 0) return B200_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == B200_BF16) concat_cast_kernel<__nv_bfloat16><<<n_rows, 256, 0, s>>>(a, b, (__nv_bfloat16*)out, width);
    else if (out_dtype == B200_F32) concat_cast_kernel<float><<<n_rows, 256, 0, s>>>(a, b, (float*)out, width);
    else return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}

extern "C" int b200_glu_act(const float* gu, void* out, int n_rows, int n, int epi, int out_dtype, void* stream) {
    if (!gu || !out || n_rows < 0 || n < 1 || (epi != B200_GG_GLU && epi != B200_GG_GLU_GELU)) return B200_EINVAL;
    if (n_rows == 0) return B200_OK;
    const size_t total = (size_t)n_rows * n;
    const unsigned grid = (unsigned)((total + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == B200_BF16) glu_act_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(gu, (__nv_bfloat16*)out, n, total, epi == B200_GG_GLU_GELU);
    else if (out_dtype == B200_F32) glu_act_kernel<float><<<grid, 256, 0, s>>>(gu, (float*)out, n, total, epi == B200_GG_GLU_GELU);
    else return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}

extern "C" int b200_glu_act_clamped(const float* gu, void* out, int n_rows, int n, float limit, int out_dtype, void* stream) {
    if (!gu || !out || n_rows < 0 || n < 1 || !(limit > 0.f)) return B200_EINVAL;
    if (n_rows == 0) return B200_OK;
    const size_t total = (size_t)n_rows * n;
    const unsigned grid = (unsigned)((total + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == B200_BF16) glu_act_clamped_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(gu, (__nv_bfloat16*)out, n, total, limit);
    else if (out_dtype == B200_F32) glu_act_clamped_kernel<float><<<grid, 256, 0, s>>>(gu, (float*)out, n, total, limit);
    else return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}

extern "C" int b200_scale(float* v, size_t n, float f, void* stream) {
    if (!v) return B200_EINVAL;
    if (n == 0) return B200_OK;
    scale_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(v, n, f);
    count_launch();
    return (int)cudaGetLastError();
}

extern "C" int b200_embed_pair_hash(const int* ids, const int* prev, const void* table, float scale, const void* pair_table, int buckets,
                                    int mul_prev, int mul_cur, float* out, void* out_cast, int n_tokens, int width, int dtype, void* stream) {
    if (!ids || !table || !out || n_tokens < 0 || width < 1 || (pair_table && (!prev || buckets < 1))) return B200_EINVAL;
    if (n_tokens == 0) return B200_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == B200_BF16)
        embed_pair_hash_kernel<__nv_bfloat16><<<n_tokens, 128, 0, s>>>(ids, prev, (const __nv_bfloat16*)table, scale, (const __nv_bfloat16*)pair_table,
                                                                      buckets, mul_prev, mul_cur, out, (__nv_bfloat16*)out_cast, width);
    else if (dtype == B200_F32)
        embed_pair_hash_kernel<float><<<n_tokens, 128, 0, s>>>(ids, prev, (const float*)table, scale, (const float*)pair_table, buckets, mul_prev,
                                                              mul_cur, out, (float*)out_cast, width);
    else
        return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}

extern "C" int b200_softcap(float* v, size_t n, float cap, void* stream) {
    if (!v || !(cap > 0.f)) return B200_EINVAL;
    if (n == 0) return B200_OK;
    softcap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(v, n, cap);
    count_launch();
    return (int)cudaGetLastError();
}

extern "C" int b200_embed_positions(const int* ids, const int* pos, const void* table, const void* pos_table, float* out,
                                    int n_tokens, int width, int dtype, void* stream) {
    if (!ids || !table || !out || (pos_table && !pos) || n_tokens < 0 || width < 1) return B200_EINVAL;
    if (n_tokens == 0) return B200_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == B200_BF16)
        embed_positions_kernel<__nv_bfloat16><<<n_tokens, 128, 0, s>>>(ids, pos, (const __nv_bfloat16*)table,
                                                                      (const __nv_bfloat16*)pos_table, out, width);
    else if (dtype == B200_F32)
        embed_positions_kernel<float><<<n_tokens, 128, 0, s>>>(ids, pos, (const float*)table, (const float*)pos_table, out, width);
    else
        return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}

extern "C" int b200_layernorm_pair(const float* x, const int* rows, int n_rows, int width, float eps, const float* w1,
                                   const float* b1, void* out1, const float* w2, const float* b2, void* out2, int out_dtype,
                                   void* stream) {
    if (!x || !w1 || !b1 || !out1 || n_rows < 0 || width < 1) return B200_EINVAL;
    if (out2 && (!w2 || !b2)) return B200_EINVAL;
    if (n_rows == 0) return B200_OK;
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return B200_EUNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == B200_BF16) {
        static unsigned long long done = 0;
        if (smem > 48 * 1024) ensure_max_dynamic_smem((const void*)layernorm_pair_kernel<__nv_bfloat16>, (int)smem, done);
        layernorm_pair_kernel<__nv_bfloat16><<<n_rows, 256, smem, s>>>(x, rows, width, eps, w1, b1, (__nv_bfloat16*)out1, w2, b2,
                                                                      (__nv_bfloat16*)out2);
    } else if (out_dtype == B200_F32) {
        static unsigned long long done = 0;
        if (smem > 48 * 1024) ensure_max_dynamic_smem((const void*)layernorm_pair_kernel<float>, (int)smem, done);
        layernorm_pair_kernel<float><<<n_rows, 256, smem, s>>>(x, rows, width, eps, w1, b1, (float*)out1, w2, b2, (float*)out2);
    } else
        return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}
