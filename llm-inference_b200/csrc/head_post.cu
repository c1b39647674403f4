// What lies between an attention kernel's fp32 output and the output projection in designs that post-process heads:
// the differential combination of two score maps (a1 - lambda a2, unit RMS per head, a constant factor), an
// element-wise sigmoid gate, and the turn back of outputs whose values were rotated by their own position, with one gate
// per head. fp32 arithmetic; only the store takes the serving dtype.
#include "b200_serve.h"
#include "common.cuh"
#include "launch_count.h"

namespace b200 {

// one warp per (token, head): a [units, 2, vdim]
template <typename T>
__global__ void diff_combine_kernel(const float* __restrict__ a, float lambda, float eps, float out_scale, T* __restrict__ out,
                                    int units, int vdim) {
    const int u = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32, lane = threadIdx.x % 32;
    if (u >= units) return;
    const float* a1 = a + (size_t)u * 2 * vdim;
    const float* a2 = a1 + vdim;
    float ss = 0.f;
    for (int i = lane; i < vdim; i += 32) {
        const float d = a1[i] - lambda * a2[i];
        ss += d * d;
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
    const float f = out_scale / sqrtf(ss / (float)vdim + eps);
    for (int i = lane; i < vdim; i += 32) out[(size_t)u * vdim + i] = DT<T>::from_f((a1[i] - lambda * a2[i]) * f);
}

template <typename T>
__global__ void sigmoid_gate_kernel(const float* __restrict__ o, const float* __restrict__ gate, long long ld_gate, T* __restrict__ out,
                                    int n, size_t total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / n, c = i % n;
    const float z = gate[t * ld_gate + c];
    out[i] = DT<T>::from_f(o[i] / (1.f + expf(-z)));
}

// A thread per rotation pair of one (token, head): (u, v) turned by minus the token's angle, (u c + v s, v c - u s), times the
// head's gate. With an odd vdim the last dimension has no partner and passes unrotated.
template <typename T>
__global__ void unrotate_gate_kernel(const float* __restrict__ o, const float* __restrict__ cs, const float* __restrict__ sn, int layout,
                                     const float* __restrict__ gate, long long ld_gate, T* __restrict__ out, int heads, int vdim,
                                     size_t total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int half = vdim / 2, per = half + (vdim & 1);
    const int m = (int)(i % per);
    const size_t unit = i / per, t = unit / heads;
    const int h = (int)(unit % heads);
    const float gv = gate ? 1.f / (1.f + expf(-gate[t * ld_gate + h])) : 1.f;
    const float* src = o + unit * vdim;
    T* dst = out + unit * vdim;
    if (m >= half) { dst[vdim - 1] = DT<T>::from_f(src[vdim - 1] * gv); return; }
    const int lo = layout == B200_ROPE_HALF ? m : 2 * m, hi = layout == B200_ROPE_HALF ? m + half : 2 * m + 1;
    const float u = src[lo], v = src[hi], c = cs[t * half + m], s = sn[t * half + m];
    dst[lo] = DT<T>::from_f((u * c + v * s) * gv);
    dst[hi] = DT<T>::from_f((v * c - u * s) * gv);
}

}  // namespace b200

using namespace b200;

extern "C" int b200_unrotate_gate(const float* o, const float* cos, const float* sin, int rot_layout, const float* gate, long long ld_gate,
                                  void* out, int n_tokens, int heads, int vdim, int out_dtype, void* stream) {
    if (!o || !cos || !sin || !out || n_tokens < 0 || heads < 1 || vdim < 1 || (gate && ld_gate < heads)) return B200_EINVAL;
    if (rot_layout != B200_ROPE_HALF && rot_layout != B200_ROPE_INTERLEAVED) return B200_EINVAL;
    if (n_tokens == 0) return B200_OK;
    const size_t total = (size_t)n_tokens * heads * (vdim / 2 + (vdim & 1));
    const unsigned grid = (unsigned)((total + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == B200_BF16) unrotate_gate_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(o, cos, sin, rot_layout, gate, ld_gate, (__nv_bfloat16*)out, heads, vdim, total);
    else if (out_dtype == B200_F32) unrotate_gate_kernel<float><<<grid, 256, 0, s>>>(o, cos, sin, rot_layout, gate, ld_gate, (float*)out, heads, vdim, total);
    else return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}

extern "C" int b200_diff_combine(const float* a, float lambda, float eps, float out_scale, void* out, int n_tokens, int heads, int vdim,
                                 int out_dtype, void* stream) {
    if (!a || !out || n_tokens < 0 || heads < 1 || vdim < 1) return B200_EINVAL;
    if (n_tokens == 0) return B200_OK;
    const int units = n_tokens * heads;
    const dim3 grid((units + 3) / 4);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == B200_BF16) diff_combine_kernel<__nv_bfloat16><<<grid, 128, 0, s>>>(a, lambda, eps, out_scale, (__nv_bfloat16*)out, units, vdim);
    else if (out_dtype == B200_F32) diff_combine_kernel<float><<<grid, 128, 0, s>>>(a, lambda, eps, out_scale, (float*)out, units, vdim);
    else return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}

extern "C" int b200_sigmoid_gate(const float* o, const float* gate, long long ld_gate, void* out, int n_tokens, int n, int out_dtype,
                                 void* stream) {
    if (!o || !gate || !out || n_tokens < 0 || n < 1 || ld_gate < n) return B200_EINVAL;
    if (n_tokens == 0) return B200_OK;
    const size_t total = (size_t)n_tokens * n;
    const unsigned grid = (unsigned)((total + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == B200_BF16) sigmoid_gate_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(o, gate, ld_gate, (__nv_bfloat16*)out, n, total);
    else if (out_dtype == B200_F32) sigmoid_gate_kernel<float><<<grid, 256, 0, s>>>(o, gate, ld_gate, (float*)out, n, total);
    else return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}
