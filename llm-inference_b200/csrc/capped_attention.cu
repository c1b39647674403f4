// b200_paged_attention: causal attention over paged per-head keys and values with grouped query heads, a tanh cap on
// the scores and a constant added to the softmax denominator (a sink of score 0 that owns no value). Prompt portions,
// single decoded tokens and mixed batches run through the same launch: every token carries its sequence slot and
// position, and only sees its own sequence's pages. Two more masks and layouts are arguments: a block mask (a position
// only sees the keys of its own block of `chunk` positions) and several score maps per head over shared values (`maps`:
// query unit (h, m) scores against key unit (h / group, m) and weights the values of key head h / group). A sliding window
// (a position sees itself and the window - 1 positions before it) is a third mask, and the weights can be sigmoids of the
// score plus a number per head instead of a softmax: then nothing is normalised over the keys, which in the running
// (maximum, denominator, output) form is a maximum held at 0 and a denominator held at 1.
//
//   paged_attn_row_kernel   one CTA per (token, query head), fp32 arithmetic on caches of either dtype: each warp
//                           takes blocks of 32 keys (a lane scores one key; the weighted value sum runs with a lane per
//                           output column), keeps its own running maximum / denominator / output and the warps merge at
//                           the end. The sink is the initial state of warp 0 (m = 0, l = denom_bias).
//   paged_attn_tile_kernel  bfloat16 prompt portions on mma.sync tiles (further down).
#include <cuda_bf16.h>
#include <math.h>
#include <stdlib.h>

#include <algorithm>

#include "b200_serve.h"
#include "common.cuh"
#include "launch_count.h"

namespace b200 {

struct PA {
    const void* q; void* out; const void* k_pool; const void* v_pool;
    const int* pages; int max_pages, page_rows;
    const int* slot; const int* pos;
    int n_tokens, heads, kv_heads, dim, vdim;
    float scale, softcap, denom_bias;
    int splits; float* part;   // row kernel: shares of a context split over gridDim.z CTAs, [token, head, split, 2 + vdim]
    int chunk, maps, out_f32;
    int window, sigmoid; const float* head_bias;
};
// first key that position p sees
__device__ __forceinline__ int pa_first_key(const PA& a, int p) {
    const int f = a.chunk > 0 ? (p / a.chunk) * a.chunk : 0;
    return a.window > 0 ? max(f, p - a.window + 1) : f;
}
__device__ __forceinline__ float pa_sigmoid(float v) { return 1.f / (1.f + expf(-v)); }
template <typename T>
__device__ __forceinline__ void pa_store(const PA& a, size_t idx, float v) {
    if (a.out_f32) reinterpret_cast<float*>(a.out)[idx] = v;
    else reinterpret_cast<T*>(a.out)[idx] = DT<T>::from_f(v);
}

constexpr int kRowWarps = 4;
constexpr int kMaxSplits = 16;
constexpr int kMaxVPerLane = 8;   // vdim <= 256

template <typename T>
__device__ __forceinline__ float dot_row(const float* q, const T* k, int dim) {
    float acc = 0.f;
    if ((dim % DT<T>::kPer16B) == 0 && (reinterpret_cast<uintptr_t>(k) & 15u) == 0) {
        for (int i = 0; i < dim; i += DT<T>::kPer16B) {
            float f[DT<T>::kPer16B];
            const Pack16 pk = ld16(k + i);
            if constexpr (sizeof(T) == 4) {
#pragma unroll
                for (int e = 0; e < 4; ++e) f[e] = __uint_as_float(pk.w[e]);
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pk.w[e]));
                    f[2 * e] = v.x;
                    f[2 * e + 1] = v.y;
                }
            }
#pragma unroll
            for (int e = 0; e < DT<T>::kPer16B; ++e) acc = fmaf(q[i + e], f[e], acc);
        }
    } else {
        for (int i = 0; i < dim; ++i) acc = fmaf(q[i], DT<T>::to_f(k[i]), acc);
    }
    return acc;
}

template <typename T>
__global__ void __launch_bounds__(kRowWarps * 32) paged_attn_row_kernel(const PA a) {
    extern __shared__ float sm[];
    float* qs = sm;                                   // [dim]
    float* om = sm + a.dim;                           // [kRowWarps][vdim]
    __shared__ float ms[kRowWarps], ls[kRowWarps];
    // h counts query units (head, map); ku is the key unit it scores against, g the key head whose values it weights
    const int t = blockIdx.x, h = blockIdx.y, warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int g = (h / a.maps) / (a.heads / a.kv_heads), ku = g * a.maps + h % a.maps, p = a.pos[t];
    const int k_units = a.kv_heads * a.maps, q_units = a.heads * a.maps;
    const int* plist = a.pages + (size_t)a.slot[t] * a.max_pages;
    const T* q = reinterpret_cast<const T*>(a.q) + ((size_t)t * q_units + h) * a.dim;
    for (int i = threadIdx.x; i < a.dim; i += blockDim.x) qs[i] = DT<T>::to_f(q[i]);
    __syncthreads();
    const T* K = reinterpret_cast<const T*>(a.k_pool);
    const T* V = reinterpret_cast<const T*>(a.v_pool);
    float m = -INFINITY, l = 0.f, o[kMaxVPerLane];
#pragma unroll
    for (int c = 0; c < kMaxVPerLane; ++c) o[c] = 0.f;
    // this CTA's share of the keys: whole blocks of 32, the sink with the first share
    const int j_lo = pa_first_key(a, p);
    const int per = ((p - j_lo + a.splits) / a.splits + 31) & ~31;
    const int j_begin = j_lo + blockIdx.z * per, j_end = min(p + 1, j_begin + per);
    if (warp == 0 && blockIdx.z == 0 && a.denom_bias > 0.f) { m = 0.f; l = a.denom_bias; }
    const float hb = (a.sigmoid && a.head_bias) ? a.head_bias[h / a.maps] : 0.f;
    if (a.sigmoid) { m = 0.f; l = (warp == 0 && blockIdx.z == 0) ? 1.f : 0.f; }
    for (int j0 = j_begin + warp * 32; j0 < j_end; j0 += kRowWarps * 32) {
        const int j = j0 + lane;
        const bool ok = j < j_end;
        size_t row = 0;   // the key's row in the page pool
        float s = -INFINITY;
        if (ok) {
            row = (size_t)plist[j / a.page_rows] * a.page_rows + j % a.page_rows;
            s = dot_row<T>(qs, K + (row * k_units + ku) * a.dim, a.dim) * a.scale;
            if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
        }
        float bm = s;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, d));
        const float mn = a.sigmoid ? 0.f : fmaxf(m, bm);
        const float corr = expf(m - mn);   // m = -inf: 0
        const float pj = !ok ? 0.f : a.sigmoid ? pa_sigmoid(s + hb) : expf(s - mn);
        float ps = a.sigmoid ? 0.f : pj;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, d);
        l = l * corr + ps;
        m = mn;
#pragma unroll
        for (int c = 0; c < kMaxVPerLane; ++c) o[c] *= corr;
        const int n = min(32, j_end - j0);
        for (int kk = 0; kk < n; ++kk) {
            const float pk = __shfl_sync(0xffffffffu, pj, kk);
            const size_t r = __shfl_sync(0xffffffffu, (unsigned long long)row, kk);
            const T* vr = V + (r * a.kv_heads + g) * a.vdim;
#pragma unroll
            for (int c = 0; c < kMaxVPerLane; ++c)
                if (lane + 32 * c < a.vdim) o[c] = fmaf(pk, DT<T>::to_f(vr[lane + 32 * c]), o[c]);
        }
    }
    if (lane == 0) { ms[warp] = m; ls[warp] = l; }
#pragma unroll
    for (int c = 0; c < kMaxVPerLane; ++c)
        if (lane + 32 * c < a.vdim) om[warp * a.vdim + lane + 32 * c] = o[c];
    __syncthreads();
    float M = ms[0];
    for (int w = 1; w < kRowWarps; ++w) M = fmaxf(M, ms[w]);
    float L = 0.f;
    for (int w = 0; w < kRowWarps; ++w) L += M == -INFINITY ? 0.f : ls[w] * expf(ms[w] - M);
    if (a.splits > 1) {   // an unnormalised share: (m, l, o); an empty share is (-inf, 0, 0)
        float* pr = a.part + (((size_t)t * q_units + h) * a.splits + blockIdx.z) * (a.vdim + 2);
        if (threadIdx.x == 0) { pr[0] = M; pr[1] = L; }
        for (int c = threadIdx.x; c < a.vdim; c += blockDim.x) {
            float v = 0.f;
            for (int w = 0; w < kRowWarps; ++w) v += M == -INFINITY ? 0.f : om[w * a.vdim + c] * expf(ms[w] - M);
            pr[2 + c] = v;
        }
        return;
    }
    const size_t dst = ((size_t)t * q_units + h) * a.vdim;
    for (int c = threadIdx.x; c < a.vdim; c += blockDim.x) {
        float v = 0.f;
        for (int w = 0; w < kRowWarps; ++w) v += om[w * a.vdim + c] * expf(ms[w] - M);
        pa_store<T>(a, dst + c, v / L);
    }
}

// Decode batches (few rows, long contexts): one CTA per (token, key head, share of the context) serves ALL query heads of
// the group from one pass over the keys and values. Eight lanes share a key row (16-byte loads, a row is read once,
// whole sectors), four keys per warp step; the scores of 32 keys go through shared memory to the softmax (a lane per
// key) and on to the weighted value sum (a lane per pair of output columns). fp32 arithmetic on caches of either dtype.
template <typename T> struct Pair;
template <> struct Pair<float> {
    static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
};
template <> struct Pair<__nv_bfloat16> {
    static __device__ __forceinline__ float2 load(const __nv_bfloat16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }
};

template <typename T, int R>   // R query heads per key head
__global__ void __launch_bounds__(kRowWarps * 32) paged_attn_group_kernel(const PA a) {
    extern __shared__ float sm[];
    float* qs = sm;                                        // [R][dim]
    float* sc = qs + R * a.dim;                            // [warps][R][32]
    float* om = sc + kRowWarps * R * 32;                   // [warps][R][vdim]
    __shared__ float ms[kRowWarps][R], ls[kRowWarps][R];
    __shared__ unsigned long long rows[kRowWarps][32];
    // blockIdx.y counts key units (key head g, map mp); query head g * R + r holds its map mp at unit (g * R + r) * maps + mp
    const int t = blockIdx.x, ku = blockIdx.y, g = ku / a.maps, mp = ku % a.maps, warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int p = a.pos[t], dim = a.dim, vdim = a.vdim, k_units = a.kv_heads * a.maps, q_units = a.heads * a.maps;
    const int* plist = a.pages + (size_t)a.slot[t] * a.max_pages;
    const T* q = reinterpret_cast<const T*>(a.q) + (size_t)t * q_units * dim;
    for (int i = threadIdx.x; i < R * dim; i += blockDim.x) qs[i] = DT<T>::to_f(q[(size_t)((g * R + i / dim) * a.maps + mp) * dim + i % dim]);
    __syncthreads();
    const T* K = reinterpret_cast<const T*>(a.k_pool);
    const T* V = reinterpret_cast<const T*>(a.v_pool);
    float m[R], l[R], o[R][4][2];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const bool sink = warp == 0 && blockIdx.z == 0 && a.denom_bias > 0.f;
        m[r] = (sink || a.sigmoid) ? 0.f : -INFINITY;
        l[r] = sink ? a.denom_bias : (a.sigmoid && warp == 0 && blockIdx.z == 0) ? 1.f : 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) o[r][c][0] = o[r][c][1] = 0.f;
    }
    const int j_lo = pa_first_key(a, p);
    const int per = ((p - j_lo + a.splits) / a.splits + 31) & ~31;
    const int j_begin = j_lo + blockIdx.z * per, j_end = min(p + 1, j_begin + per);
    float* scw = sc + warp * R * 32;
    const int l8 = lane & 7;
    for (int j0 = j_begin + warp * 32; j0 < j_end; j0 += kRowWarps * 32) {
#pragma unroll
        for (int it = 0; it < 8; ++it) {   // scores of keys j0 + 4 it + (lane / 8); unrolled: the loads of all steps are in flight together
            const int kk = it * 4 + (lane >> 3), j = j0 + kk;
            float acc[R];
#pragma unroll
            for (int r = 0; r < R; ++r) acc[r] = 0.f;
            size_t row = 0;
            if (j < j_end) {
                row = (size_t)plist[j / a.page_rows] * a.page_rows + j % a.page_rows;
                const T* kr = K + (row * k_units + ku) * dim;
                for (int i = l8 * 8; i < dim; i += 64) {
                    float f[8];
                    if constexpr (sizeof(T) == 2) {   // eight bfloat16 in one 16-byte load
                        const Pack16 pk = ld16(kr + i);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pk.w[e]));
                            f[2 * e] = v.x;
                            f[2 * e + 1] = v.y;
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; e += 4) {
                            const Pack16 pk = ld16(kr + i + e);
#pragma unroll
                            for (int x = 0; x < 4; ++x) f[e + x] = __uint_as_float(pk.w[x]);
                        }
                    }
#pragma unroll
                    for (int r = 0; r < R; ++r)
#pragma unroll
                        for (int e = 0; e < 8; ++e) acc[r] = fmaf(qs[r * dim + i + e], f[e], acc[r]);
                }
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], 1);
                acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], 2);
                acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], 4);
            }
            if (l8 == 0) {
                rows[warp][kk] = row;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    float sv = acc[r] * a.scale;
                    if (a.softcap > 0.f) sv = a.softcap * tanhf(sv / a.softcap);
                    scw[r * 32 + kk] = j < j_end ? sv : -INFINITY;
                }
            }
        }
        __syncwarp();
#pragma unroll
        for (int r = 0; r < R; ++r) {   // softmax step, a lane per key
            const float sv = scw[r * 32 + lane];
            float bm = sv;
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, d));
            const float mn = a.sigmoid ? 0.f : fmaxf(m[r], bm);          // finite: the block holds at least one key
            const float corr = expf(m[r] - mn);
            // a masked key: exp(-inf) = 0
            const float pj = !a.sigmoid ? expf(sv - mn) : sv == -INFINITY ? 0.f : pa_sigmoid(sv + (a.head_bias ? a.head_bias[g * R + r] : 0.f));
            float ps = a.sigmoid ? 0.f : pj;
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, d);
            l[r] = l[r] * corr + ps;
            m[r] = mn;
#pragma unroll
            for (int c = 0; c < 4; ++c) { o[r][c][0] *= corr; o[r][c][1] *= corr; }
            scw[r * 32 + lane] = pj;
        }
        __syncwarp();
        const int n = min(32, j_end - j0);
#pragma unroll 4
        for (int kk = 0; kk < n; ++kk) {   // weighted values, a lane per pair of columns
            const T* vr = V + (rows[warp][kk] * a.kv_heads + g) * vdim;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int col = 2 * lane + 64 * c;
                if (col < vdim) {
                    const float2 v = Pair<T>::load(vr + col);
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const float pk = scw[r * 32 + kk];
                        o[r][c][0] = fmaf(pk, v.x, o[r][c][0]);
                        o[r][c][1] = fmaf(pk, v.y, o[r][c][1]);
                    }
                }
            }
        }
        __syncwarp();
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        if (lane == 0) { ms[warp][r] = m[r]; ls[warp][r] = l[r]; }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int col = 2 * lane + 64 * c;
            if (col < vdim) { om[(warp * R + r) * vdim + col] = o[r][c][0]; om[(warp * R + r) * vdim + col + 1] = o[r][c][1]; }
        }
    }
    __syncthreads();
    for (int r = 0; r < R; ++r) {
        const int h = (g * R + r) * a.maps + mp;   // query unit
        float M = ms[0][r];
        for (int w = 1; w < kRowWarps; ++w) M = fmaxf(M, ms[w][r]);
        float L = 0.f;
        for (int w = 0; w < kRowWarps; ++w) L += M == -INFINITY ? 0.f : ls[w][r] * expf(ms[w][r] - M);
        float* pr = a.splits > 1 ? a.part + (((size_t)t * q_units + h) * a.splits + blockIdx.z) * (vdim + 2) : nullptr;
        if (pr && threadIdx.x == 0) { pr[0] = M; pr[1] = L; }
        const size_t dst = ((size_t)t * q_units + h) * vdim;
        for (int c = threadIdx.x; c < vdim; c += blockDim.x) {
            float v = 0.f;
            for (int w = 0; w < kRowWarps; ++w) v += M == -INFINITY ? 0.f : om[(w * R + r) * vdim + c] * expf(ms[w][r] - M);
            if (pr) pr[2 + c] = v;
            else pa_store<T>(a, dst + c, v / L);
        }
    }
}

template <typename T>
static bool launch_group(const PA& a, dim3 grid, cudaStream_t s) {
    const int R = a.heads / a.kv_heads;
    const size_t smem = ((size_t)R * a.dim + (size_t)kRowWarps * R * 32 + (size_t)kRowWarps * R * a.vdim) * sizeof(float);
    if (smem > 48 * 1024) return false;
    switch (R) {
        case 1: paged_attn_group_kernel<T, 1><<<grid, kRowWarps * 32, smem, s>>>(a); return true;
        case 2: paged_attn_group_kernel<T, 2><<<grid, kRowWarps * 32, smem, s>>>(a); return true;
        case 4: paged_attn_group_kernel<T, 4><<<grid, kRowWarps * 32, smem, s>>>(a); return true;
        case 8: paged_attn_group_kernel<T, 8><<<grid, kRowWarps * 32, smem, s>>>(a); return true;
    }
    return false;
}

// merges the shares of split contexts: one CTA per (token, head)
template <typename T>
__global__ void __launch_bounds__(128) paged_attn_combine_kernel(const float* __restrict__ part, T* __restrict__ out, int splits, int vdim) {
    const float* pr = part + (size_t)blockIdx.x * splits * (vdim + 2);
    float M = -INFINITY;
    for (int z = 0; z < splits; ++z) M = fmaxf(M, pr[(size_t)z * (vdim + 2)]);
    float L = 0.f, wz[kMaxSplits];
    for (int z = 0; z < splits; ++z) {
        const float mz = pr[(size_t)z * (vdim + 2)];
        wz[z] = mz == -INFINITY ? 0.f : expf(mz - M);
        L += pr[(size_t)z * (vdim + 2) + 1] * wz[z];
    }
    for (int c = threadIdx.x; c < vdim; c += blockDim.x) {
        float v = 0.f;
        for (int z = 0; z < splits; ++z) v += pr[(size_t)z * (vdim + 2) + 2 + c] * wz[z];
        out[(size_t)blockIdx.x * vdim + c] = DT<T>::from_f(v / L);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// bfloat16 prompt portions on tensor-core tiles (mma.sync m16n8k16, fp32 accumulation): a CTA of four warps owns 64
// consecutive rows of the packed batch for one query head; each warp keeps its 16 rows' Q fragments and output
// accumulators in registers and walks the keys in tiles of 64 that land in shared memory by cp.async (two buffers, the
// next tile in flight while this one is multiplied). Scores, cap, mask and the online softmax stay in fp32 registers;
// the probabilities are rounded to bfloat16 only as the operand of the second product. Rows of the tile that belong
// to different sequences are handled segment by segment (the other rows masked), so prompt portions, single tokens and
// mixed batches share the launch. The sink is the initial state of every row (m = 0, l = denom_bias).
// ---------------------------------------------------------------------------------------------------------------
constexpr int kTileM = 64, kTileN = 64;

__device__ __forceinline__ void pa_ldsm_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void pa_ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
// (not volatile: a pure function of its registers, so the compiler may interleave independent accumulators)
__device__ __forceinline__ void pa_mma(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ uint32_t pa_pack(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

template <int D, int DV, bool BLOCKS>   // dim == D (a multiple of 32), vdim == DV (a multiple of 16); BLOCKS: a block mask or a window
__global__ void __launch_bounds__(128, DV <= 128 ? 3 : 2) paged_attn_tile_kernel(const PA a) {
    using bf = __nv_bfloat16;
    constexpr int RS = D + 8;                 // row stride in elements: 16-byte aligned, conflict-free fragment loads
    constexpr int CH = D / 8;                 // 16-byte chunks per row
    constexpr int RSV = DV + 8;               // the same for value rows
    extern __shared__ __align__(16) unsigned char pa_smem[];
    bf* Ks = reinterpret_cast<bf*>(pa_smem);                  // [2][64][RS]
    bf* Vs = Ks + 2 * kTileN * RS;                            // [2][64][RSV]
    bf* Qs = Ks + kTileN * RS;                                // [64][RS]: the Q tile borrows the second K buffer until its
                                                              // fragments are in registers (three CTAs fit an SM this way)
    int* row_pos = reinterpret_cast<int*>(Vs + 2 * kTileN * RSV);   // [64], -1: no such row
    int* row_slot = row_pos + kTileM;
    // the last rows of a prompt see the most keys: those tiles are scheduled first, the short ones fill the tail
    const int t0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * kTileM, h = blockIdx.y;   // h: query unit (head, map)
    const int g = (h / a.maps) / (a.heads / a.kv_heads), ku = g * a.maps + h % a.maps;
    const int k_units = a.kv_heads * a.maps, q_units = a.heads * a.maps;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, gid = lane >> 2, tig = lane & 3;
    const int rows = min(kTileM, a.n_tokens - t0);
    for (int r = threadIdx.x; r < kTileM; r += blockDim.x) {
        row_pos[r] = r < rows ? a.pos[t0 + r] : -1;
        row_slot[r] = r < rows ? a.slot[t0 + r] : -1;
    }
    const bf* Q = reinterpret_cast<const bf*>(a.q);
    for (int i = threadIdx.x; i < kTileM * CH; i += blockDim.x) {
        const int r = i / CH, c = i % CH;
        Pack16 v{{0u, 0u, 0u, 0u}};
        if (r < rows) v = ld16(Q + ((size_t)(t0 + r) * q_units + h) * D + c * 8);
        st16(Qs + r * RS + c * 8, v);
    }
    __syncthreads();
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
        pa_ldsm_x4(qf[ks], Qs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * RS + ks * 16 + (lane >> 4) * 8);
    float o[DV / 8][4];
#pragma unroll
    for (int nt = 0; nt < DV / 8; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
    const bool sig = a.sigmoid != 0;
    const float m0 = (a.denom_bias > 0.f || sig) ? 0.f : -1e30f, l0 = sig ? 1.f : a.denom_bias;
    float m_run[2] = {m0, m0}, l_run[2] = {l0, l0};
    const float hb = (sig && a.head_bias) ? a.head_bias[h / a.maps] : 0.f;
    const int r_lo = warp * 16 + gid, r_hi = r_lo + 8;
    const float scale_over_cap = a.softcap > 0.f ? a.scale / a.softcap : 0.f;
    const bf* Kp = reinterpret_cast<const bf*>(a.k_pool);
    const bf* Vp = reinterpret_cast<const bf*>(a.v_pool);

    for (int seg = 0; seg < rows;) {
        const int b = row_slot[seg];
        int seg_end = seg + 1;
        while (seg_end < rows && row_slot[seg_end] == b) ++seg_end;
        const int n_keys = row_pos[seg_end - 1] + 1;            // positions grow along an entry
        const int first_key = BLOCKS ? pa_first_key(a, row_pos[seg]) : 0;    // with a block mask the first row's block starts the walk
        const int* plist = a.pages + (size_t)b * a.max_pages;
        // this thread's two rows in this segment (last and first key each sees), and the keys any row of the warp sees
        const int p_lo = (r_lo >= seg && r_lo < seg_end) ? row_pos[r_lo] : -1;
        const int p_hi = (r_hi >= seg && r_hi < seg_end) ? row_pos[r_hi] : -1;
        const int f_lo = (BLOCKS && p_lo >= 0) ? pa_first_key(a, p_lo) : 0, f_hi = (BLOCKS && p_hi >= 0) ? pa_first_key(a, p_hi) : 0;
        const int w_first = max(seg, warp * 16), w_last = min(seg_end, warp * 16 + 16) - 1;
        const int warp_keys = w_last >= w_first ? row_pos[w_last] + 1 : 0;
        const int warp_first = (BLOCKS && w_last >= w_first) ? pa_first_key(a, row_pos[w_first]) : 0;
        auto load_tile = [&](int k0, int buf) {
            bf* kd = Ks + buf * kTileN * RS;
            bf* vd = Vs + buf * kTileN * RSV;
            // a thread brings chunk c of key row kr, and the DV / D value chunks that go with it (one page lookup for all)
            for (int i = threadIdx.x; i < kTileN * CH; i += blockDim.x) {
                const int kr = i / CH, c = i % CH, j = k0 + kr;
                const bool ok = j < n_keys;
                const size_t row = ok ? (size_t)plist[j / a.page_rows] * a.page_rows + j % a.page_rows : 0;
                const uint32_t bytes = ok ? 16u : 0u;                 // beyond the sequence: zeros, nothing is read
                const uint32_t kdst = (uint32_t)__cvta_generic_to_shared(kd + kr * RS + c * 8);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(kdst), "l"(Kp + (row * k_units + ku) * D + c * 8), "r"(bytes) : "memory");
#pragma unroll
                for (int e = 0; e < DV / D; ++e) {
                    const uint32_t vdst = (uint32_t)__cvta_generic_to_shared(vd + kr * RSV + (c + e * CH) * 8);
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(vdst), "l"(Vp + (row * a.kv_heads + g) * DV + (c + e * CH) * 8), "r"(bytes) : "memory");
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        __syncthreads();   // the buffers of the previous segment are no longer read
        load_tile(first_key, 0);
        int buf = 0;
        for (int k0 = first_key; k0 < n_keys; k0 += kTileN, buf ^= 1) {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();   // tile k0 has landed for everybody; the other buffer is no longer read
            if (k0 + kTileN < n_keys) load_tile(k0 + kTileN, buf ^ 1);
            if (k0 >= warp_keys || (BLOCKS && k0 + kTileN <= warp_first)) continue;   // nothing for this warp's rows in this tile (it keeps the barriers)
            const bf* Kb = Ks + buf * kTileN * RS;
            const bf* Vb = Vs + buf * kTileN * RSV;
            float s[kTileN / 8][4];
#pragma unroll
            for (int nt = 0; nt < kTileN / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
            // k steps outside, key columns inside: consecutive MMAs feed different accumulators. One ldmatrix.x4 brings the
            // K fragments of two k steps: matrices (k 0-7 | 8-15 | 16-23 | 24-31) of 8 keys
#pragma unroll
            for (int ks = 0; ks < D / 16; ks += 2) {
                uint32_t b4[kTileN / 8][4];
#pragma unroll
                for (int nt = 0; nt < kTileN / 8; ++nt)
                    pa_ldsm_x4(b4[nt], Kb + (nt * 8 + (lane & 7)) * RS + (lane >> 3) * 8 + ks * 16);
#pragma unroll
                for (int nt = 0; nt < kTileN / 8; ++nt) {
                    const uint32_t b0[2] = {b4[nt][0], b4[nt][1]};
                    pa_mma(s[nt], qf[ks], b0);
                }
#pragma unroll
                for (int nt = 0; nt < kTileN / 8; ++nt) {
                    const uint32_t b1[2] = {b4[nt][2], b4[nt][3]};
                    pa_mma(s[nt], qf[ks + 1], b1);
                }
            }
            // cap * tanh(v / cap): when every score of this thread's tile is small against the cap (the usual case) the odd
            // series x - x^3/3 + 2x^5/15 - 17x^7/315 is exact to fp32 rounding below |x| = 0.25 and costs no special-function
            // unit; otherwise (t - 1) / (t + 1) with t = e^(2x) (absolute error ~1e-7 * cap)
            if (a.softcap > 0.f) {
                float big = 0.f;
#pragma unroll
                for (int nt = 0; nt < kTileN / 8; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) { s[nt][e] *= scale_over_cap; big = fmaxf(big, fabsf(s[nt][e])); }
                if (__all_sync(0xffffffffu, big < 0.25f)) {
#pragma unroll
                    for (int nt = 0; nt < kTileN / 8; ++nt)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float x = s[nt][e], x2 = x * x;
                            s[nt][e] = a.softcap * x * fmaf(x2, fmaf(x2, fmaf(x2, -17.f / 315.f, 2.f / 15.f), -1.f / 3.f), 1.f);
                        }
                } else {
#pragma unroll
                    for (int nt = 0; nt < kTileN / 8; ++nt)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float t = __expf(fminf(fmaxf(2.f * s[nt][e], -30.f), 30.f));
                            s[nt][e] = a.softcap * __fdividef(t - 1.f, t + 1.f);
                        }
                }
            } else {
#pragma unroll
                for (int nt = 0; nt < kTileN / 8; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[nt][e] *= a.scale;
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < kTileN / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = k0 + nt * 8 + tig * 2 + (e & 1);
                    const float v = (j <= ((e & 2) ? p_hi : p_lo) && (!BLOCKS || j >= ((e & 2) ? f_hi : f_lo))) ? s[nt][e] : -INFINITY;
                    s[nt][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            if (sig) {   // weights that are not normalised over the keys: nothing runs along the row
#pragma unroll
                for (int nt = 0; nt < kTileN / 8; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[nt][e] = s[nt][e] == -INFINITY ? 0.f : 1.f / (1.f + __expf(-(s[nt][e] + hb)));
            } else {
            float alpha[2];
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                mx[hrow] = fmaxf(mx[hrow], __shfl_xor_sync(0xffffffffu, mx[hrow], 1));
                mx[hrow] = fmaxf(mx[hrow], __shfl_xor_sync(0xffffffffu, mx[hrow], 2));
                const float mn = fmaxf(m_run[hrow], mx[hrow]);   // finite: m starts at 0 (the sink) or at -1e30
                alpha[hrow] = __expf(m_run[hrow] - mn);
                m_run[hrow] = mn;
            }
            float sum[2] = {0.f, 0.f};
#pragma unroll
            for (int nt = 0; nt < kTileN / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float pv = __expf(s[nt][e] - m_run[e >> 1]);   // masked: exp(-inf) = 0
                    s[nt][e] = pv;
                    sum[e >> 1] += pv;
                }
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                sum[hrow] += __shfl_xor_sync(0xffffffffu, sum[hrow], 1);
                sum[hrow] += __shfl_xor_sync(0xffffffffu, sum[hrow], 2);
                l_run[hrow] = l_run[hrow] * alpha[hrow] + sum[hrow];
            }
#pragma unroll
            for (int nt = 0; nt < DV / 8; ++nt) { o[nt][0] *= alpha[0]; o[nt][1] *= alpha[0]; o[nt][2] *= alpha[1]; o[nt][3] *= alpha[1]; }
            }
#pragma unroll
            for (int kk = 0; kk < kTileN / 16; ++kk) {
                uint32_t pf[4];
                pf[0] = pa_pack(s[2 * kk][0], s[2 * kk][1]);
                pf[1] = pa_pack(s[2 * kk][2], s[2 * kk][3]);
                pf[2] = pa_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pf[3] = pa_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int nt = 0; nt < DV / 8; nt += 2) {   // one transposed ldmatrix.x4: the V fragments of two column tiles
                    uint32_t b4[4];
                    pa_ldsm_x4_trans(b4, Vb + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * RSV + (nt + (lane >> 4)) * 8);
                    const uint32_t b0[2] = {b4[0], b4[1]}, b1[2] = {b4[2], b4[3]};
                    pa_mma(o[nt], pf, b0);
                    pa_mma(o[nt + 1], pf, b1);
                }
            }
        }
        seg = seg_end;
    }
#pragma unroll
    for (int hrow = 0; hrow < 2; ++hrow) {
        const int r = hrow ? r_hi : r_lo;
        if (r >= rows) continue;
        const float inv = 1.0f / l_run[hrow];
        const size_t dst = ((size_t)(t0 + r) * q_units + h) * DV + tig * 2;
        if (a.out_f32) {
#pragma unroll
            for (int nt = 0; nt < DV / 8; ++nt)
                *reinterpret_cast<float2*>(reinterpret_cast<float*>(a.out) + dst + nt * 8) = make_float2(o[nt][hrow * 2] * inv, o[nt][hrow * 2 + 1] * inv);
        } else {
#pragma unroll
            for (int nt = 0; nt < DV / 8; ++nt)
                *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<bf*>(a.out) + dst + nt * 8) = __floats2bfloat162_rn(o[nt][hrow * 2] * inv, o[nt][hrow * 2 + 1] * inv);
        }
    }
}

template <int D, int DV>
static int launch_tile(const PA& a, cudaStream_t s) {
    static_assert(kTileM == kTileN, "the Q tile borrows a K buffer");
    constexpr int smem = 2 * kTileN * (D + 8) * 2 + 2 * kTileN * (DV + 8) * 2 + 2 * kTileM * 4;
    static unsigned long long done = 0;
    static_assert(DV % D == 0, "a thread brings DV / D value chunks with every key chunk");
    const dim3 grid((a.n_tokens + kTileM - 1) / kTileM, a.heads * a.maps);
    if (a.chunk > 0 || a.window > 0) {
        static unsigned long long done_b = 0;
        const cudaError_t e = ensure_max_dynamic_smem((const void*)paged_attn_tile_kernel<D, DV, true>, smem, done_b);
        if (e != cudaSuccess) return (int)e;
        paged_attn_tile_kernel<D, DV, true><<<grid, 128, smem, s>>>(a);
        return (int)cudaGetLastError();
    }
    const cudaError_t e = ensure_max_dynamic_smem((const void*)paged_attn_tile_kernel<D, DV, false>, smem, done);
    if (e != cudaSuccess) return (int)e;
    paged_attn_tile_kernel<D, DV, false><<<grid, 128, smem, s>>>(a);
    return (int)cudaGetLastError();
}
// the (dim, vdim) pairs the tile kernel is built for: equal sizes, and values twice as wide as the keys
static int launch_tile_for(const PA& a, cudaStream_t s) {
    if (a.dim == a.vdim) return a.dim == 128 ? launch_tile<128, 128>(a, s) : a.dim == 64 ? launch_tile<64, 64>(a, s) : a.dim == 32 ? launch_tile<32, 32>(a, s) : -1;
    if (a.vdim == 2 * a.dim) return a.dim == 128 ? launch_tile<128, 256>(a, s) : a.dim == 64 ? launch_tile<64, 128>(a, s) : a.dim == 32 ? launch_tile<32, 64>(a, s) : -1;
    return -1;
}

}  // namespace b200

using namespace b200;

extern "C" size_t b200_paged_attention_workspace_bytes(int n_tokens, int heads, int vdim) {
    if (n_tokens < 1 || heads < 1 || vdim < 1 || (long long)n_tokens * heads >= 2 * sm_count()) return 0;
    return (size_t)n_tokens * heads * kMaxSplits * (vdim + 2) * sizeof(float);
}

extern "C" int b200_paged_attention(const b200_paged_attention_args* p, void* stream) {
    if (!p || !p->q || !p->out || !p->k_pool || !p->v_pool || !p->pages || !p->slot || !p->pos || p->n_tokens < 0 || p->heads < 1 ||
        p->kv_heads < 1 || p->heads % p->kv_heads || p->dim < 1 || p->vdim < 1 || p->page_rows < 1 || p->denom_bias < 0.f ||
        p->chunk < 0 || p->maps < 0 || p->window < 0)
        return B200_EINVAL;
    if (p->sigmoid_weights && (p->softcap > 0.f || p->denom_bias > 0.f || p->maps > 1)) return B200_EINVAL;
    const int maps = p->maps > 0 ? p->maps : 1, units = p->heads * maps;
    if (p->vdim > 32 * kMaxVPerLane) return B200_EUNSUPPORTED;
    if (p->n_tokens == 0) return B200_OK;
    PA a{p->q, p->out, p->k_pool, p->v_pool, p->pages, p->max_pages, p->page_rows, p->slot, p->pos, p->n_tokens, p->heads,
         p->kv_heads, p->dim, p->vdim, p->scale, p->softcap, p->denom_bias, 1, nullptr, p->chunk, maps, p->out_f32,
         p->window, p->sigmoid_weights != 0, p->head_bias};
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = ((size_t)p->dim + (size_t)kRowWarps * p->vdim) * sizeof(float);
    if (smem > 48 * 1024) return B200_EUNSUPPORTED;
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    const char* env = getenv("B200_ATTN_ROWS");   // 1: every batch on the row kernel (debugging aid)
    if (p->dtype == B200_BF16 && p->longest_entry != 1 && (p->dim == p->vdim || p->vdim == 2 * p->dim) &&
        (p->dim == 64 || p->dim == 128 || p->dim == 32) && al16(p->q) && al16(p->out) && al16(p->k_pool) && al16(p->v_pool) &&
        !(env && env[0] == '1')) {
        const int rc = launch_tile_for(a, s);
        if (rc == 0) count_launch();
        if (rc >= 0) return rc;
    }
    // single tokens whose heads come in groups of 1, 2, 4 or 8 per key head: one pass over K / V serves the whole group
    const int R = p->heads / p->kv_heads;
    const bool group = p->longest_entry == 1 && (R == 1 || R == 2 || R == 4 || R == 8) && p->dim % 8 == 0 && p->vdim % 2 == 0 &&
                       al16(p->k_pool) && al16(p->v_pool) && !(env && env[0] == '1') &&
                       ((size_t)R * p->dim + (size_t)kRowWarps * R * (32 + p->vdim)) * sizeof(float) <= 48 * 1024;
    const long long ctas = (long long)p->n_tokens * (group ? p->kv_heads * maps : units);
    // few rows with long contexts (decode batches): split every context over several CTAs and merge the shares
    int longest_seen = p->chunk > 0 ? std::min(p->longest_context, p->chunk) : p->longest_context;
    if (p->window > 0) longest_seen = std::min(longest_seen, p->window);
    if (longest_seen > 256 && p->workspace && (long long)p->n_tokens * units < 2 * sm_count()) {
        int splits = (int)((4ll * sm_count() + ctas - 1) / ctas);
        splits = std::min(std::min(splits, kMaxSplits), (longest_seen + 127) / 128);
        if (splits > 1 && p->workspace_bytes >= (size_t)p->n_tokens * units * splits * (p->vdim + 2) * sizeof(float)) {
            a.splits = splits;
            a.part = reinterpret_cast<float*>(p->workspace);
        }
    }
    const dim3 grid3(p->n_tokens, units, a.splits);
    bool done = false;
    if (group) {
        const dim3 gridg(p->n_tokens, p->kv_heads * maps, a.splits);
        done = p->dtype == B200_BF16 ? launch_group<__nv_bfloat16>(a, gridg, s) : p->dtype == B200_F32 ? launch_group<float>(a, gridg, s) : false;
    }
    if (done) {
    } else if (p->dtype == B200_BF16) paged_attn_row_kernel<__nv_bfloat16><<<grid3, kRowWarps * 32, smem, s>>>(a);
    else if (p->dtype == B200_F32) paged_attn_row_kernel<float><<<grid3, kRowWarps * 32, smem, s>>>(a);
    else return B200_EINVAL;
    count_launch();
    if (a.splits > 1) {
        if (p->dtype == B200_BF16 && !p->out_f32) paged_attn_combine_kernel<__nv_bfloat16><<<p->n_tokens * units, 128, 0, s>>>(a.part, (__nv_bfloat16*)p->out, a.splits, p->vdim);
        else paged_attn_combine_kernel<float><<<p->n_tokens * units, 128, 0, s>>>(a.part, (float*)p->out, a.splits, p->vdim);
        count_launch();
    }
    return (int)cudaGetLastError();
}
