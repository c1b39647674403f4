// Between the q / k projection and the cache of an attention layer: rotary angles of a step (double-precision angle,
// one table per frequency set), the short causal convolution over time with its carried inputs, the per-head RMS norm,
// the rotation in either pairing, and the store of q, k (and of the convolved keys as values) — b200_qk_prepare — plus
// the update of the convolution's ring of carried inputs. All arithmetic fp32; only the stores take the serving dtype.
#include <cuda_bf16.h>

#include "b200_serve.h"
#include "common.cuh"
#include "launch_count.h"
#include "rotary.cuh"

namespace b200 {

__global__ void rope_angles_kernel(const int* __restrict__ pos, const double* __restrict__ freq, int n_freq, int total,
                                   double amplitude, float* __restrict__ cos_out, float* __restrict__ sin_out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const double a = (double)pos[i / n_freq] * freq[i % n_freq];
    double s, c;
    sincos(a, &s, &c);
    cos_out[i] = (float)(amplitude * c);
    sin_out[i] = (float)(amplitude * s);
}

struct QkPrep {
    const float* proj; long long ld_proj;
    const float* conv_w; int taps; const float* conv_state;
    const float* q_norm; const float* k_norm; float eps;
    const float* cos; const float* sin; int rot_dims, rot_layout;
    void* q_out; void* k_pool; void* v_pool; int v_from_conv;
    float* ring_out;   // non-NULL: every entry of the batch is one token, and the warp files its own inputs in the ring
    const int* pages; int max_pages, page_rows;
    const int* slot; const int* pos; const int* start;
    int heads, kv_heads, dim;
    int v_heads, vdim; long long v_off;
    const float* bias; const float* v_cos; const float* v_sin; int v_layout;
    int vals_per_warp;   // floats of shared memory per warp: max(dim, vdim)
};

// One warp per (token, head unit): units [0, heads) are query heads, [heads, heads + kv_heads) key heads; a lane owns the
// dimensions lane, lane + 32, ... (coalesced loads and stores); the head's sum of squares is a warp reduction and the
// rotation reads its partner through the warp's slice of shared memory, so no CTA-wide barrier is needed.
constexpr int kPrepWarps = 4, kMaxTapsUnrolled = 4;   // longer filters take the plain loop
template <typename T>
__global__ void __launch_bounds__(kPrepWarps * 32) qk_prepare_kernel(const QkPrep a, int n_units) {
    extern __shared__ float prep_sm[];
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, dim = a.dim;
    const int unit = blockIdx.x * kPrepWarps + warp, per_token = a.heads + a.kv_heads;
    if (unit >= n_units) return;
    float* vals = prep_sm + warp * a.vals_per_warp;   // the normed head before rotation
    const int t = unit / (per_token + a.v_heads), u = unit % (per_token + a.v_heads);
    if (u >= per_token) {   // a projected value head: to its cache row, with its bias and turned by its own position if asked
        const int g = u - per_token, pv = a.pos[t];
        const size_t vrow = ((size_t)a.pages[(size_t)a.slot[t] * a.max_pages + pv / a.page_rows] * a.page_rows + pv % a.page_rows) * a.v_heads + g;
        const size_t col0 = (size_t)a.v_off + (size_t)g * a.vdim;
        const float* src = a.proj + (size_t)t * a.ld_proj + col0;
        T* vd = reinterpret_cast<T*>(a.v_pool) + vrow * a.vdim;
        if (!a.v_cos) {
            for (int i = lane; i < a.vdim; i += 32) vd[i] = DT<T>::from_f(src[i] + (a.bias ? a.bias[col0 + i] : 0.f));
            return;
        }
        for (int i = lane; i < a.vdim; i += 32) vals[i] = src[i] + (a.bias ? a.bias[col0 + i] : 0.f);
        __syncwarp();
        const int vf = a.vdim / 2;
        for (int i = lane; i < a.vdim; i += 32)
            vd[i] = DT<T>::from_f(rotary_component(vals, i, 2 * vf, a.v_layout, a.v_cos + (size_t)t * vf, a.v_sin + (size_t)t * vf));
        return;
    }
    const bool is_k = u >= a.heads;
    const int ch0 = u * dim;          // first channel of this head in [q channels | k channels]
    const int channels = per_token * dim;
    const int p = a.pos[t], b = a.slot[t];
    size_t cache_row = 0;
    if (is_k) cache_row = ((size_t)a.pages[(size_t)b * a.max_pages + p / a.page_rows] * a.page_rows + p % a.page_rows) * a.kv_heads + (u - a.heads);
    const int first = a.conv_w ? a.start[t] : 0, taps = a.taps;
    float ss = 0.f;
    if (a.conv_w && taps <= kMaxTapsUnrolled) {
        // The rows that hold the taps' inputs (this step's batch, the slot's ring, or nothing before position 0) are found
        // once per warp; then four dimensions per lane and all their taps at once: every load of the group is in flight
        // before the first sum. A four-tap filter is one 16-byte load per channel.
        const float* rows[kMaxTapsUnrolled];
        bool ok[kMaxTapsUnrolled];
#pragma unroll
        for (int j = 0; j < kMaxTapsUnrolled; ++j) {
            const int back = taps - 1 - j, src = p - back;
            ok[j] = j < taps && src >= 0;
            rows[j] = !ok[j] ? a.proj
                      : src >= first ? a.proj + (size_t)(t - back) * a.ld_proj + ch0
                                     : a.conv_state + ((size_t)b * (taps - 1) + src % (taps - 1)) * channels + ch0;
        }
        const float* cw = a.conv_w + (size_t)ch0 * taps;
        const bool w4 = taps == 4 && (reinterpret_cast<uintptr_t>(a.conv_w) & 15u) == 0;
        float* ring = (a.ring_out && taps > 1) ? a.ring_out + ((size_t)b * (taps - 1) + p % (taps - 1)) * channels + ch0 : nullptr;
        T* vdst = (is_k && a.v_from_conv) ? reinterpret_cast<T*>(a.v_pool) + cache_row * dim : nullptr;
        for (int i0 = lane; i0 < dim; i0 += 128) {
            float xin[4][kMaxTapsUnrolled], w[4][kMaxTapsUnrolled];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = i0 + 32 * k;
                const bool in = i < dim;
#pragma unroll
                for (int j = 0; j < kMaxTapsUnrolled; ++j) xin[k][j] = in && ok[j] ? rows[j][i] : 0.f;
                if (w4) {
                    const float4 w4v = in ? *reinterpret_cast<const float4*>(cw + (size_t)i * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
                    w[k][0] = w4v.x; w[k][1] = w4v.y; w[k][2] = w4v.z; w[k][3] = w4v.w;
                } else {
#pragma unroll
                    for (int j = 0; j < kMaxTapsUnrolled; ++j) w[k][j] = in && j < taps ? cw[(size_t)i * taps + j] : 0.f;
                }
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = i0 + 32 * k;
                if (i >= dim) continue;
                float y = 0.f;
#pragma unroll
                for (int j = 0; j < kMaxTapsUnrolled; ++j) y = fmaf(w[k][j], xin[k][j], y);
                if (ring) ring[i] = a.proj[(size_t)t * a.ld_proj + ch0 + i];   // the token's own input (the last tap)
                if (vdst) vdst[i] = DT<T>::from_f(y);
                vals[i] = y;
                ss += y * y;
            }
        }
    } else
    for (int i = lane; i < dim; i += 32) {
        const int c = ch0 + i;
        float y;
        if (a.conv_w) {
            y = 0.f;
            for (int j = 0; j < taps; ++j) {
                const int back = taps - 1 - j, src = p - back;
                if (src < 0) continue;
                const float uin = src >= first ? a.proj[(size_t)(t - back) * a.ld_proj + c]
                                               : a.conv_state[((size_t)b * (taps - 1) + src % (taps - 1)) * channels + c];
                y = fmaf(a.conv_w[(size_t)c * taps + j], uin, y);
            }
            // a one-token entry: nobody else reads this sequence's ring in this launch, and this lane has read its own places
            if (a.ring_out && taps > 1) a.ring_out[((size_t)b * (taps - 1) + p % (taps - 1)) * channels + c] = a.proj[(size_t)t * a.ld_proj + c];
        } else
            y = a.proj[(size_t)t * a.ld_proj + c] + (a.bias ? a.bias[c] : 0.f);
        if (is_k && a.v_from_conv) reinterpret_cast<T*>(a.v_pool)[cache_row * dim + i] = DT<T>::from_f(y);
        vals[i] = y;
        ss += y * y;
    }
    const float* nw = is_k ? a.k_norm : a.q_norm;
    if (nw) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float rinv = 1.0f / sqrtf(ss / (float)dim + a.eps);
        for (int i = lane; i < dim; i += 32) vals[i] = vals[i] * rinv * nw[i];
    }
    __syncwarp();
    const int nf = a.rot_dims / 2;
    T* dst = is_k ? reinterpret_cast<T*>(a.k_pool) + cache_row * dim : reinterpret_cast<T*>(a.q_out) + ((size_t)t * a.heads + u) * dim;
    for (int i = lane; i < dim; i += 32)
        dst[i] = DT<T>::from_f(rotary_component(vals, i, a.rot_dims, a.rot_layout, a.cos + (size_t)t * nf, a.sin + (size_t)t * nf));
}

// Without convolution and head norm the preparation is a rotation and three scatters: a thread per four consecutive
// dimensions of one head (or value head) of one token. It loads its own four values and, inside the rotated part, the
// four of its rotate-half partner with 16-byte loads, and stores four values of the serving dtype at once.
template <typename T>
__global__ void __launch_bounds__(256) qk_rotate_store_kernel(const QkPrep a, long long total, int quads_per_token) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int t = (int)(idx / quads_per_token), qd = (int)(idx % quads_per_token);
    const int dim = a.dim, qk_quads = (a.heads + a.kv_heads) * (dim / 4);
    const float* row = a.proj + (size_t)t * a.ld_proj;
    float4 v;
    T* dst;
    if (qd < qk_quads) {
        const int u = qd / (dim / 4), i0 = (qd % (dim / 4)) * 4, half = a.rot_dims / 2;
        v = *reinterpret_cast<const float4*>(row + (size_t)u * dim + i0);
        if (i0 < a.rot_dims) {
            const bool low = i0 < half;
            const float4 w = *reinterpret_cast<const float4*>(row + (size_t)u * dim + (low ? i0 + half : i0 - half));
            const float* cs = a.cos + (size_t)t * half + (low ? i0 : i0 - half);
            const float* sn = a.sin + (size_t)t * half + (low ? i0 : i0 - half);
            // the pair (lo, hi) becomes (lo c - hi s, hi c + lo s)
            if (low) v = make_float4(v.x * cs[0] - w.x * sn[0], v.y * cs[1] - w.y * sn[1], v.z * cs[2] - w.z * sn[2], v.w * cs[3] - w.w * sn[3]);
            else v = make_float4(v.x * cs[0] + w.x * sn[0], v.y * cs[1] + w.y * sn[1], v.z * cs[2] + w.z * sn[2], v.w * cs[3] + w.w * sn[3]);
        }
        if (u < a.heads) dst = reinterpret_cast<T*>(a.q_out) + ((size_t)t * a.heads + u) * dim + i0;
        else {
            const int p = a.pos[t];
            const size_t prow = (size_t)a.pages[(size_t)a.slot[t] * a.max_pages + p / a.page_rows] * a.page_rows + p % a.page_rows;
            dst = reinterpret_cast<T*>(a.k_pool) + (prow * a.kv_heads + (u - a.heads)) * dim + i0;
        }
    } else {
        const int c0 = (qd - qk_quads) * 4, p = a.pos[t];   // value column (head g, dimension c0 % vdim)
        v = *reinterpret_cast<const float4*>(row + a.v_off + c0);
        const size_t prow = (size_t)a.pages[(size_t)a.slot[t] * a.max_pages + p / a.page_rows] * a.page_rows + p % a.page_rows;
        dst = reinterpret_cast<T*>(a.v_pool) + prow * a.v_heads * a.vdim + c0;
    }
    if constexpr (sizeof(T) == 4) *reinterpret_cast<float4*>(dst) = v;
    else {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    }
}

// the rotated part of every head's query, placed behind the head's absorbed part: a thread per (token, head, dimension)
__global__ void rotate_part_kernel(const float* __restrict__ src, long long ld_src, long long src_off, long long src_stride,
                                   float* __restrict__ dst, long long ld_dst, long long dst_off, long long dst_stride,
                                   const float* __restrict__ cs, const float* __restrict__ sn, int layout, int heads, int dims, size_t total) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int i = (int)(idx % dims), h = (int)((idx / dims) % heads);
    const size_t t = idx / ((size_t)dims * heads);
    const int nf = dims / 2;
    dst[t * ld_dst + dst_off + h * dst_stride + i] =
        rotary_component(src + t * ld_src + src_off + h * src_stride, i, 2 * nf, layout, cs + t * nf, sn + t * nf);
}

__global__ void conv_state_update_kernel(const float* __restrict__ proj, long long ld_proj, float* __restrict__ state,
                                         const int* __restrict__ slot, const int* __restrict__ pos, const int* __restrict__ end,
                                         int channels, int taps) {
    const int t = blockIdx.x, p = pos[t];
    if (p < end[t] - (taps - 1)) return;   // only the last taps-1 inputs of a sequence are carried
    float* dst = state + ((size_t)slot[t] * (taps - 1) + p % (taps - 1)) * channels;
    for (int c = threadIdx.x; c < channels; c += blockDim.x) dst[c] = proj[(size_t)t * ld_proj + c];
}

}  // namespace b200

using namespace b200;

extern "C" int b200_rope_angles_amp(const int* pos, int n_tokens, const double* freq, int n_freq, double amplitude, float* cos_out,
                                    float* sin_out, void* stream) {
    if (!pos || !freq || !cos_out || !sin_out || n_tokens < 0 || n_freq < 0) return B200_EINVAL;
    const int total = n_tokens * n_freq;
    if (total == 0) return B200_OK;
    rope_angles_kernel<<<(total + 255) / 256, 256, 0, (cudaStream_t)stream>>>(pos, freq, n_freq, total, amplitude, cos_out, sin_out);
    count_launch();
    return (int)cudaGetLastError();
}
extern "C" int b200_rope_angles(const int* pos, int n_tokens, const double* freq, int n_freq, float* cos_out, float* sin_out,
                                void* stream) {
    return b200_rope_angles_amp(pos, n_tokens, freq, n_freq, 1.0, cos_out, sin_out, stream);
}

extern "C" int b200_qk_prepare(const b200_qk_prepare_args* p, void* stream) {
    if (!p || !p->proj || !p->q_out || !p->k_pool || !p->pages || !p->slot || !p->pos || p->n_tokens < 0 || p->heads < 1 ||
        p->kv_heads < 1 || p->dim < 1 || p->page_rows < 1)
        return B200_EINVAL;
    if (p->conv_w && (p->taps < 1 || !p->start || (p->taps > 1 && !p->conv_state))) return B200_EINVAL;
    if (p->v_from_conv && !p->v_pool) return B200_EINVAL;
    if (p->v_heads < 0 || (p->v_heads > 0 && (!p->v_pool || p->vdim < 1 || p->v_from_conv || p->v_off < 0))) return B200_EINVAL;
    if (p->rot_dims < 0 || (p->rot_dims & 1) || p->rot_dims > p->dim || (p->rot_dims && (!p->cos || !p->sin))) return B200_EINVAL;
    if (p->rot_layout != B200_ROPE_HALF && p->rot_layout != B200_ROPE_INTERLEAVED) return B200_EINVAL;
    if (p->bias && p->conv_w) return B200_EINVAL;   // carried convolution inputs are raw projections
    if ((p->v_cos || p->v_sin) && (!p->v_cos || !p->v_sin || p->v_heads < 1 ||
                                   (p->v_rot_layout != B200_ROPE_HALF && p->v_rot_layout != B200_ROPE_INTERLEAVED)))
        return B200_EINVAL;
    if (p->n_tokens == 0) return B200_OK;
    QkPrep a{p->proj, p->ld_proj, p->conv_w, p->taps, p->conv_state, p->q_norm, p->k_norm, p->eps, p->cos, p->sin, p->rot_dims,
             p->rot_layout, p->q_out, p->k_pool, p->v_pool, p->v_from_conv, p->update_state_inline ? const_cast<float*>(p->conv_state) : nullptr, p->pages, p->max_pages, p->page_rows, p->slot, p->pos,
             p->start, p->heads, p->kv_heads, p->dim, p->v_heads, p->vdim, p->v_off, p->bias, p->v_cos, p->v_sin, p->v_rot_layout,
             p->v_heads > 0 && p->vdim > p->dim ? p->vdim : p->dim};
    if (a.conv_w && a.taps == 1) a.conv_state = a.proj;   // never read: every input of a one-tap filter is the token's own
    cudaStream_t s = (cudaStream_t)stream;
    {   // rotation and scatters only, everything in whole groups of four: the vector kernel
        auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
        const bool plain = !p->conv_w && !p->q_norm && !p->k_norm && !p->bias && !p->v_cos && p->rot_layout == B200_ROPE_HALF && p->dim % 4 == 0 && p->rot_dims % 8 == 0 &&
                           p->ld_proj % 4 == 0 && al16(p->proj) && al16(p->q_out) && al16(p->k_pool) &&
                           (p->v_heads == 0 || (p->vdim % 4 == 0 && p->v_off % 4 == 0 && al16(p->v_pool))) &&
                           (p->dtype == B200_BF16 || p->dtype == B200_F32);
        if (plain) {
            const int quads = (p->heads + p->kv_heads) * (p->dim / 4) + p->v_heads * (p->vdim / 4);
            const long long total = (long long)p->n_tokens * quads;
            const unsigned grid = (unsigned)((total + 255) / 256);
            if (p->dtype == B200_BF16) qk_rotate_store_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(a, total, quads);
            else qk_rotate_store_kernel<float><<<grid, 256, 0, s>>>(a, total, quads);
            count_launch();
            return (int)cudaGetLastError();
        }
    }
    const long long units = (long long)p->n_tokens * (p->heads + p->kv_heads + p->v_heads);
    if (units > 0x7fffffffll) return B200_EUNSUPPORTED;
    const unsigned grid = (unsigned)((units + kPrepWarps - 1) / kPrepWarps);
    const size_t smem = (size_t)kPrepWarps * a.vals_per_warp * sizeof(float);
    if (smem > 48 * 1024) return B200_EUNSUPPORTED;
    if (p->dtype == B200_BF16) qk_prepare_kernel<__nv_bfloat16><<<grid, kPrepWarps * 32, smem, s>>>(a, (int)units);
    else if (p->dtype == B200_F32) qk_prepare_kernel<float><<<grid, kPrepWarps * 32, smem, s>>>(a, (int)units);
    else return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}

extern "C" int b200_rotate_part(const float* src, long long ld_src, long long src_off, long long src_stride, float* dst, long long ld_dst,
                                long long dst_off, long long dst_stride, const float* cos, const float* sin, int rot_layout, int n_tokens,
                                int heads, int dims, void* stream) {
    if (!src || !dst || !cos || !sin || n_tokens < 0 || heads < 1 || dims < 1) return B200_EINVAL;
    if (rot_layout != B200_ROPE_HALF && rot_layout != B200_ROPE_INTERLEAVED) return B200_EINVAL;
    if (n_tokens == 0) return B200_OK;
    const size_t total = (size_t)n_tokens * heads * dims;
    rotate_part_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(src, ld_src, src_off, src_stride, dst, ld_dst, dst_off,
                                                                                         dst_stride, cos, sin, rot_layout, heads, dims, total);
    count_launch();
    return (int)cudaGetLastError();
}

extern "C" int b200_conv_state_update(const float* proj, long long ld_proj, float* conv_state, const int* slot, const int* pos,
                                      const int* end, int n_tokens, int channels, int taps, void* stream) {
    if (!proj || !slot || !pos || !end || n_tokens < 0 || channels < 1 || taps < 1) return B200_EINVAL;
    if (n_tokens == 0 || taps == 1) return B200_OK;
    if (!conv_state) return B200_EINVAL;
    conv_state_update_kernel<<<n_tokens, 128, 0, (cudaStream_t)stream>>>(proj, ld_proj, conv_state, slot, pos, end, channels, taps);
    count_launch();
    return (int)cudaGetLastError();
}
