// b200_rmsnorm_residual: the fp32 residual update of a pre-norm layer (up to two scaled sublayer outputs, the weighted
// rows of routed experts, a vector shared by all rows) fused with the RMS norm of whatever reads the residual next, so a
// sublayer boundary is one launch. One CTA per row; the new row stays in shared memory between the sum of squares and
// the output. With a row list the kernel only norms the listed rows (the final norm before the vocabulary projection).
// Layers whose norm sits on the sublayer's OUTPUT take the other order (norm_addend): the sublayer's row (plus a bias) is
// normed, added to the residual, and the new residual row leaves in the serving dtype for the next sublayer to read.
#include "b200_serve.h"
#include "common.cuh"
#include "launch_count.h"

namespace b200 {

struct RnArgs {
    float* x;
    const float* y1; float s1;
    const float* y2; float s2;
    const float* eo; const int* dest; const float* weight; int top;
    const float* bcast;
    const int* rows;
    const float* w; float w_offset, eps;
    void* out;
    int width;
};

constexpr int kRnThreads = 256, kRnMaxTop = 16;

template <typename T>
__global__ void __launch_bounds__(kRnThreads) rmsnorm_residual_kernel(const RnArgs a) {
    extern __shared__ float rn_row[];
    __shared__ float red[kRnThreads / 32];
    __shared__ int e_dest[kRnMaxTop];
    __shared__ float e_w[kRnMaxTop];
    const int i = blockIdx.x, width = a.width;
    const size_t src = (size_t)(a.rows ? a.rows[i] : i) * width;
    const bool adds = !a.rows && (a.y1 || a.y2 || a.eo || a.bcast);
    if (a.eo && threadIdx.x < a.top) {
        e_dest[threadIdx.x] = a.dest[(size_t)i * a.top + threadIdx.x];
        e_w[threadIdx.x] = a.weight[(size_t)i * a.top + threadIdx.x];
    }
    if (a.eo) __syncthreads();
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += kRnThreads) {
        float v = a.x[src + c];
        if (adds) {
            if (a.y1) v += a.s1 * a.y1[src + c];
            if (a.y2) v += a.s2 * a.y2[src + c];
            if (a.eo) {
                float r = 0.f;
                for (int k = 0; k < a.top; ++k)
                    if (e_dest[k] >= 0) r = fmaf(e_w[k], a.eo[(size_t)e_dest[k] * width + c], r);
                v += r;
            }
            if (a.bcast) v += a.bcast[c];
            a.x[src + c] = v;
        }
        rn_row[c] = v;
        ss += v * v;
    }
    if (!a.w) return;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (threadIdx.x % 32 == 0) red[threadIdx.x / 32] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int k = 0; k < kRnThreads / 32; ++k) tot += red[k];   // the same order in every thread
    const float rinv = 1.0f / sqrtf(tot / (float)width + a.eps);
    T* out = reinterpret_cast<T*>(a.out) + (size_t)i * width;
    for (int c = threadIdx.x; c < width; c += kRnThreads) out[c] = DT<T>::from_f(rn_row[c] * rinv * (a.w_offset + a.w[c]));
}

// The same for rows of at most 8 values per thread: every operand of the row is loaded up front (one round trip to memory
// instead of a dependent chain per column) and the row lives in registers.
constexpr int kRnPer = 8;
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS) rmsnorm_residual_reg_kernel(const RnArgs a) {
    __shared__ float red[THREADS / 32];
    __shared__ int e_dest[kRnMaxTop];
    __shared__ float e_w[kRnMaxTop];
    const int i = blockIdx.x, width = a.width;
    const size_t src = (size_t)(a.rows ? a.rows[i] : i) * width;
    const bool adds = !a.rows && (a.y1 || a.y2 || a.eo || a.bcast);
    if (a.eo && threadIdx.x < a.top) {
        e_dest[threadIdx.x] = a.dest[(size_t)i * a.top + threadIdx.x];
        e_w[threadIdx.x] = a.weight[(size_t)i * a.top + threadIdx.x];
    }
    if (a.eo) __syncthreads();
    float v[kRnPer], p1[kRnPer], p2[kRnPer], pb[kRnPer], wv[kRnPer];
#pragma unroll
    for (int k = 0; k < kRnPer; ++k) {
        const int c = threadIdx.x + THREADS * k;
        const bool in = c < width;
        v[k] = in ? a.x[src + c] : 0.f;
        p1[k] = (in && adds && a.y1) ? a.y1[src + c] : 0.f;
        p2[k] = (in && adds && a.y2) ? a.y2[src + c] : 0.f;
        pb[k] = (in && adds && a.bcast) ? a.bcast[c] : 0.f;
        wv[k] = (in && a.w) ? a.w[c] : 0.f;
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < kRnPer; ++k) {
        const int c = threadIdx.x + THREADS * k;
        if (adds && c < width) {
            // the order of the plain kernel: y1, y2, experts, the shared vector
            if (a.y1) v[k] += a.s1 * p1[k];
            if (a.y2) v[k] += a.s2 * p2[k];
            if (a.eo) {
                float r = 0.f;
                for (int j = 0; j < a.top; ++j)
                    if (e_dest[j] >= 0) r = fmaf(e_w[j], a.eo[(size_t)e_dest[j] * width + c], r);
                v[k] += r;
            }
            if (a.bcast) v[k] += pb[k];
            a.x[src + c] = v[k];
        }
        ss += v[k] * v[k];
    }
    if (!a.w) return;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (threadIdx.x % 32 == 0) red[threadIdx.x / 32] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int k = 0; k < THREADS / 32; ++k) tot += red[k];
    const float rinv = 1.0f / sqrtf(tot / (float)width + a.eps);
    T* out = reinterpret_cast<T*>(a.out) + (size_t)i * width;
#pragma unroll
    for (int k = 0; k < kRnPer; ++k) {
        const int c = threadIdx.x + THREADS * k;
        if (c < width) out[c] = DT<T>::from_f(v[k] * rinv * (a.w_offset + wv[k]));
    }
}

// x += norm(y1 + y_bias) * (w_offset + w); out = x. Rows of at most kRnPer values per thread live in registers (REG), longer
// ones in shared memory.
template <typename T, int THREADS, bool REG>
__global__ void __launch_bounds__(THREADS) rmsnorm_addend_kernel(const RnArgs a, const float* __restrict__ y_bias) {
    extern __shared__ float rn_row[];
    __shared__ float red[THREADS / 32];
    const int i = blockIdx.x, width = a.width;
    const size_t src = (size_t)i * width;
    float v[kRnPer], xv[kRnPer], wv[kRnPer];
    float ss = 0.f;
    if (REG) {
#pragma unroll
        for (int k = 0; k < kRnPer; ++k) {
            const int c = threadIdx.x + THREADS * k;
            const bool in = c < width;
            v[k] = in ? a.y1[src + c] + (y_bias ? y_bias[c] : 0.f) : 0.f;
            xv[k] = in ? a.x[src + c] : 0.f;
            wv[k] = in ? a.w[c] : 0.f;
            ss += v[k] * v[k];
        }
    } else {
        for (int c = threadIdx.x; c < width; c += THREADS) {
            const float y = a.y1[src + c] + (y_bias ? y_bias[c] : 0.f);
            rn_row[c] = y;
            ss += y * y;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (threadIdx.x % 32 == 0) red[threadIdx.x / 32] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int k = 0; k < THREADS / 32; ++k) tot += red[k];   // the same order in every thread
    const float rinv = 1.0f / sqrtf(tot / (float)width + a.eps);
    T* out = a.out ? reinterpret_cast<T*>(a.out) + src : nullptr;
    if (REG) {
#pragma unroll
        for (int k = 0; k < kRnPer; ++k) {
            const int c = threadIdx.x + THREADS * k;
            if (c >= width) continue;
            const float nx = xv[k] + v[k] * rinv * (a.w_offset + wv[k]);
            a.x[src + c] = nx;
            if (out) out[c] = DT<T>::from_f(nx);
        }
    } else {
        for (int c = threadIdx.x; c < width; c += THREADS) {
            const float nx = a.x[src + c] + rn_row[c] * rinv * (a.w_offset + a.w[c]);
            a.x[src + c] = nx;
            if (out) out[c] = DT<T>::from_f(nx);
        }
    }
}

template <typename T>
static void launch_addend(const RnArgs& a, const float* y_bias, int n_rows, size_t smem, cudaStream_t s) {
    if (a.width <= 256 * kRnPer) rmsnorm_addend_kernel<T, 256, true><<<n_rows, 256, 0, s>>>(a, y_bias);
    else if (a.width <= 1024 * kRnPer) rmsnorm_addend_kernel<T, 1024, true><<<n_rows, 1024, 0, s>>>(a, y_bias);
    else {
        static unsigned long long done = 0;
        if (smem > 48 * 1024) ensure_max_dynamic_smem((const void*)rmsnorm_addend_kernel<T, kRnThreads, false>, 200 * 1024, done);
        rmsnorm_addend_kernel<T, kRnThreads, false><<<n_rows, kRnThreads, smem, s>>>(a, y_bias);
    }
}

template <typename T>
static void launch_rn(const RnArgs& a, int n_rows, size_t smem, cudaStream_t s) {
    if (a.width <= 256 * kRnPer) rmsnorm_residual_reg_kernel<T, 256><<<n_rows, 256, 0, s>>>(a);
    else if (a.width <= 1024 * kRnPer) rmsnorm_residual_reg_kernel<T, 1024><<<n_rows, 1024, 0, s>>>(a);
    else {
        static unsigned long long done = 0;
        if (smem > 48 * 1024) ensure_max_dynamic_smem((const void*)rmsnorm_residual_kernel<T>, 200 * 1024, done);
        rmsnorm_residual_kernel<T><<<n_rows, kRnThreads, smem, s>>>(a);
    }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_rmsnorm_residual(const b200_rmsnorm_residual_args* p, void* stream) {
    if (!p || !p->x || p->n_rows < 0 || p->width < 1) return B200_EINVAL;
    if (p->w && !p->out && !p->norm_addend) return B200_EINVAL;
    if (p->expert_out && (!p->dest || !p->weight || p->top < 1)) return B200_EINVAL;
    if (p->expert_out && p->top > kRnMaxTop) return B200_EUNSUPPORTED;
    if (p->rows && (p->y1 || p->y2 || p->expert_out || p->bcast)) return B200_EINVAL;
    if (p->n_rows == 0) return B200_OK;
    const size_t smem = (size_t)p->width * sizeof(float);
    if (smem > 200 * 1024) return B200_EUNSUPPORTED;
    RnArgs a{p->x, p->y1, p->s1, p->y2, p->s2, p->expert_out, p->dest, p->weight, p->top, p->bcast, p->rows, p->w, p->w_offset, p->eps,
             p->out, p->width};
    cudaStream_t s = (cudaStream_t)stream;
    if (p->norm_addend) {
        if (!p->y1 || !p->w || p->y2 || p->expert_out || p->bcast || p->rows) return B200_EINVAL;
        if (p->out_dtype == B200_BF16 || !p->out) launch_addend<__nv_bfloat16>(a, p->y_bias, p->n_rows, smem, s);
        else if (p->out_dtype == B200_F32) launch_addend<float>(a, p->y_bias, p->n_rows, smem, s);
        else return B200_EINVAL;
        count_launch();
        return (int)cudaGetLastError();
    }
    if (p->out_dtype == B200_BF16 || !p->w) launch_rn<__nv_bfloat16>(a, p->n_rows, smem, s);
    else if (p->out_dtype == B200_F32) launch_rn<float>(a, p->n_rows, smem, s);
    else return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}
