// Latent attention: the cache holds ONE normed low-rank row c_j per token and layer (no per-head keys or values).
// With k_j = W_uk c_j and v_j = W_uv c_j the key up-projection is folded into the query (qa = W_uk,h^T q_h) and the
// value up-projection is applied after the weighted sum, so attention runs on the cached rows themselves:
//   s_j = scale <qa_h, c_j>,  out_h = sum_j p_j c_j,  p = softmax over {s_j} and one sink logit per head that has no
//   row and no value (it only enlarges the denominator).
// Rows live in a page pool [n_pages, page_rows, rank] addressed through per-sequence page lists (page_pool.h), the
// same lists for every layer. Scores, softmax and the weighted sum are fp32 whatever the cache dtype.
// Designs that rotate one key part shared by all heads append it to the cached row ([latent | rotated part],
// latent_store_rot_kernel) and the head's rotated query part to the absorbed query: the score is still one dot product over
// the row, and of the weighted sum the caller uses the latent columns. A sliding window (window > 0: position p sees rows
// p - window < j <= p) bounds the walk from below; without a sink (NULL) the softmax is plain.
//
// Kernels:
//   latent_store_kernel        RMS norm (eps inside the root) of the down-projected row, times weight -> its page slot
//   latent_attn_kernel         one CTA per (token, head): the warps walk the visible rows round-robin, each row read
//                              coalesced by one warp; per-warp online softmax, merged with the sink at the end
//   latent_attn_tile_kernel    bf16 tensor-core form (mma.sync): one CTA per 32 (token, head) rows; half tiles of 32 cached
//                              rows arrive in two shared-memory buffers by cp.async and are the operand of both the
//                              scores and the weighted sum (prompt portions and decoded tokens alike; the default for
//                              bf16 caches); decode batches split long contexts over several CTAs
//   latent_attn_combine_kernel merges the shares of a split launch and the sink
#include <algorithm>

#include "b200_serve.h"
#include "common.cuh"
#include "launch_count.h"
#include "rotary.cuh"

namespace b200 {

constexpr int kMaxRankPerLane = 20;   // rank <= 640 (a latent of 512 with a rotated part of 64 or 128)

template <typename T>
__global__ void __launch_bounds__(128) latent_store_kernel(const float* __restrict__ raw, long long ld_raw,
                                                           const float* __restrict__ w, float eps, T* __restrict__ pool,
                                                           const int* __restrict__ pages, int max_pages, int page_rows,
                                                           const int* __restrict__ slot, const int* __restrict__ pos,
                                                           int rank) {
    __shared__ float red[4];
    const int t = blockIdx.x;
    const float* src = raw + (size_t)t * ld_raw;
    float q = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) q += src[i] * src[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
    if (threadIdx.x % 32 == 0) red[threadIdx.x / 32] = q;
    __syncthreads();
    const float tot = red[0] + red[1] + red[2] + red[3];
    const float r = 1.0f / sqrtf(tot / (float)rank + eps);
    const int p = pos[t];
    const size_t row = (size_t)pages[(size_t)slot[t] * max_pages + p / page_rows] * page_rows + p % page_rows;
    T* dst = pool + row * rank;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = DT<T>::from_f(src[i] * r * w[i]);
}

// row = [norm(raw[0:rank]) * w | rot(raw[rank:rank+extra])]
template <typename T>
__global__ void __launch_bounds__(128) latent_store_rot_kernel(const float* __restrict__ raw, long long ld_raw, const float* __restrict__ w,
                                                               float eps, T* __restrict__ pool, const int* __restrict__ pages, int max_pages,
                                                               int page_rows, const int* __restrict__ slot, const int* __restrict__ pos, int rank,
                                                               int extra, const float* __restrict__ cs, const float* __restrict__ sn, int layout) {
    __shared__ float red[4];
    const int t = blockIdx.x;
    const float* src = raw + (size_t)t * ld_raw;
    float q = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) q += src[i] * src[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
    if (threadIdx.x % 32 == 0) red[threadIdx.x / 32] = q;
    __syncthreads();
    const float tot = red[0] + red[1] + red[2] + red[3];
    const float r = 1.0f / sqrtf(tot / (float)rank + eps);
    const int p = pos[t];
    const size_t row = (size_t)pages[(size_t)slot[t] * max_pages + p / page_rows] * page_rows + p % page_rows;
    T* dst = pool + row * (rank + extra);
    for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = DT<T>::from_f(src[i] * r * w[i]);
    const int nf = extra / 2;
    for (int i = threadIdx.x; i < extra; i += blockDim.x)
        dst[rank + i] = DT<T>::from_f(rotary_component(src + rank, i, 2 * nf, layout, cs + (size_t)t * nf, sn + (size_t)t * nf));
}

template <typename T>
__global__ void __launch_bounds__(128) latent_attn_kernel(const float* __restrict__ qa, float* __restrict__ out,
                                                          const T* __restrict__ pool, const int* __restrict__ pages,
                                                          int max_pages, int page_rows, const int* __restrict__ slot,
                                                          const int* __restrict__ pos, const float* __restrict__ sink,
                                                          float scale, int heads, int rank, int window) {
    extern __shared__ float sm[];          // q[rank] | o[4][rank] | m[4] | l[4]
    float* q = sm;
    float* so = sm + rank;
    float* sml = so + 4 * rank;
    const int t = blockIdx.x, h = blockIdx.y;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const float* qsrc = qa + ((size_t)t * heads + h) * rank;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) q[i] = qsrc[i];
    __syncthreads();
    float qr[kMaxRankPerLane], o[kMaxRankPerLane];
#pragma unroll
    for (int i = 0; i < kMaxRankPerLane; ++i) {
        const int r = i * 32 + lane;
        qr[i] = r < rank ? q[r] : 0.f;
        o[i] = 0.f;
    }
    const int n_keys = pos[t] + 1;
    const int* list = pages + (size_t)slot[t] * max_pages;
    float m = -INFINITY, l = 0.f;
    const int j_lo = window > 0 ? max(0, n_keys - window) : 0;
    for (int j = j_lo + warp; j < n_keys; j += 4) {
        const T* c = pool + ((size_t)list[j / page_rows] * page_rows + j % page_rows) * rank;
        float cr[kMaxRankPerLane];
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < kMaxRankPerLane; ++i) {
            const int r = i * 32 + lane;
            cr[i] = (i * 32 < rank && r < rank) ? DT<T>::to_f(c[r]) : 0.f;
            d = fmaf(qr[i], cr[i], d);
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) d += __shfl_xor_sync(0xffffffffu, d, s);
        const float sc = d * scale;
        const float mn = fmaxf(m, sc);
        const float alpha = expf(m - mn), p = expf(sc - mn);
        l = l * alpha + p;
#pragma unroll
        for (int i = 0; i < kMaxRankPerLane; ++i) o[i] = o[i] * alpha + p * cr[i];
        m = mn;
    }
#pragma unroll
    for (int i = 0; i < kMaxRankPerLane; ++i) {
        const int r = i * 32 + lane;
        if (r < rank) so[warp * rank + r] = o[i];
    }
    if (lane == 0) { sml[warp] = m; sml[4 + warp] = l; }
    __syncthreads();
    const float sk = sink ? sink[h] : -INFINITY;   // no sink: nothing joins the denominator
    float M = sk;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sml[w]);
    float f[4], den = expf(sk - M);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        f[w] = expf(sml[w] - M);     // a warp without rows: exp(-inf) = 0
        den += sml[4 + w] * f[w];
    }
    const float inv = 1.0f / den;
    float* dst = out + ((size_t)t * heads + h) * rank;
    for (int r = threadIdx.x; r < rank; r += blockDim.x)
        dst[r] = (so[r] * f[0] + so[rank + r] * f[1] + so[2 * rank + r] * f[2] + so[3 * rank + r] * f[3]) * inv;
}


// ---- bf16 tensor-core form ---------------------------------------------------------------------------------------
// One CTA = 32 rows of (token, head) pairs: TQ consecutive tokens of the packed batch x HG heads (all heads share the
// cached rows, so a row tile staged once serves HG heads). 8 warps. Per half tile of 32 cached rows (two buffers: the
// next half arrives by cp.async while this one is used):
//   S = Q C^T   : warp w computes the 8 keys [8 (w & 3), +8) for all 32 rows over its half of the padded rank; the two
//                 partial scores go to smem and are added in the softmax
//   softmax     : warp w owns rows [4w, 4w+4): mask, running max / sum (fp32), P as bf16 to smem, rescale factors
//   O += P C    : warp w owns output columns [64w', ...) of all 32 rows; the SAME smem tile is the B operand, read
//                 transposed with ldmatrix.trans
// The sink enters as the initial state (m = sink, l = 1, O = 0): a virtual row with a zero value.
// Tokens of different sequences inside one CTA (entry borders, decode batches) are walked segment by segment.
constexpr int kTileRows = 32, kTileKeys = 64, kHalfKeys = 32, kTileWarps = 8, kMaxSplits = 16;

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x2_trans(uint32_t (&r)[2], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <int NT>   // n8 column tiles of the output per warp: padded rank <= 64 * NT
__global__ void __launch_bounds__(256, NT <= 8 ? 2 : 1) latent_attn_tile_kernel(const float* __restrict__ qa, float* __restrict__ out,
                                                               const __nv_bfloat16* __restrict__ pool, const int* __restrict__ pages,
                                                               int max_pages, int page_rows, const int* __restrict__ slot,
                                                               const int* __restrict__ pos, const float* __restrict__ sink, float scale,
                                                               int n_tokens, int heads, int rank, int HG, int TQ, int splits,
                                                               float* __restrict__ part, int window, int out_cols, int single) {
    // out_cols: the weighted sum is formed for the first out_cols columns of a row only (a caller that uses the latent part
    // of [latent | rotated part] rows). single: one half-tile buffer instead of two (rows wider than 512: two CTAs still
    // share an SM, and the other CTA's arithmetic covers this one's load)
    // splits > 1 (blockIdx.z): this CTA walks one share of the key tiles and leaves (m, l, unnormalised O) per row in
    // `part` [token, head, split, 2 + rank]; latent_attn_combine_kernel merges the shares and the sink
    using bf = __nv_bfloat16;
    extern __shared__ __align__(16) unsigned char smraw[];
    const int rpad = (rank + 15) & ~15, RS = rpad + 8;           // smem row stride in elements (16-byte multiple)
    bf* Qs = reinterpret_cast<bf*>(smraw);                        // [32][RS]
    bf* Ks = Qs + kTileRows * RS;                                 // [2][32][RS]: half tiles, one being filled while the other is used
    float* Ss = reinterpret_cast<float*>(Ks + (single ? kHalfKeys : kTileKeys) * RS);    // [2][32][36]: partial scores of the two halves of the rank
    bf* Ps = reinterpret_cast<bf*>(Ss);                           // [32][72]: a row's probabilities overwrite its own scores
    float* alpha_s = Ss + 2 * kTileRows * 36;                     // [32]
    float* linv_s = alpha_s + kTileRows;                          // [32]
    int* row_pos = reinterpret_cast<int*>(linv_s + kTileRows);    // [32]: position of the row's token, -1 = inactive

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, gid = lane / 4, tig = lane % 4;
    const int t0 = blockIdx.x * TQ, h0 = blockIdx.y * HG;
    const int ntok = min(TQ, n_tokens - t0);
    const int n8 = ((out_cols + 15) & ~15) / 8;                   // n8 tiles of the output
    const int ntw = (n8 + kTileWarps - 1) / kTileWarps;           // per warp (<= NT)
    const int tile0 = warp * ntw;

    for (int first = 0; first < ntok;) {
        const int sl = slot[t0 + first];
        int cnt = 1;
        while (first + cnt < ntok && slot[t0 + first + cnt] == sl) ++cnt;
        const int all_keys = pos[t0 + first + cnt - 1] + 1;
        // the first row of the segment sees the oldest key: whole tiles from there (a half tile stays inside its page)
        const int seg_lo = window > 0 ? max(0, pos[t0 + first] - window + 1) / kTileKeys * kTileKeys : 0;
        const int per = ((all_keys - seg_lo + kTileKeys - 1) / kTileKeys + splits - 1) / splits * kTileKeys;   // keys per share
        const int key_lo = seg_lo + blockIdx.z * per, n_keys = min(all_keys, key_lo + per);
        const int* list = pages + (size_t)sl * max_pages;
        __syncthreads();   // the previous segment's readers are done with the shared state
        if (threadIdx.x < kTileRows) {
            const int r = threadIdx.x, tl = r / HG, h = h0 + r % HG;
            row_pos[r] = (tl >= first && tl < first + cnt && tl < TQ && h < heads) ? pos[t0 + tl] : -1;
        }
        for (int i = threadIdx.x; i < kTileRows * rpad; i += blockDim.x) {
            const int r = i / rpad, c = i - r * rpad;
            const int tl = r / HG, h = h0 + r % HG;
            const bool on = tl >= first && tl < first + cnt && tl < TQ && h < heads && c < rank;
            Qs[r * RS + c] = __float2bfloat16_rn(on ? qa[((size_t)(t0 + tl) * heads + h) * rank + c] : 0.f);
        }
        // running state of the rows this warp owns in the softmax phase (uniform over the lanes)
        float m_run[4], l_run[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = warp * 4 + i, h = h0 + r % HG;
            const bool own_sink = splits == 1 && sink != nullptr;           // shares: the sink joins in the combine
            m_run[i] = !own_sink ? -1e30f : (h < heads ? sink[h] : 0.f);
            l_run[i] = own_sink ? 1.f : 0.f;
        }
        float o[2][NT][4];
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int b = 0; b < NT; ++b)
#pragma unroll
                for (int c = 0; c < 4; ++c) o[a][b][c] = 0.f;

        // half tiles of 32 cached rows, double-buffered: the rows of half i + 1 arrive (cp.async, 16 bytes each, zero-filled
        // beyond the context and in the padding columns) while half i is scored, normalised and accumulated
        const bool vec = (rank & 7) == 0;
        const int chunks = rpad / 8;
        auto load_half = [&](int k0, bf* dstbuf) {
            if (vec) {
                const bool one_page = page_rows % kHalfKeys == 0;   // a half tile never straddles two pages
                const size_t page_base = one_page ? (size_t)list[k0 / page_rows] * page_rows + k0 % page_rows : 0;
                for (int i = threadIdx.x; i < kHalfKeys * chunks; i += blockDim.x) {
                    const int kr = i / chunks, ch = i - kr * chunks;
                    const int j = k0 + kr;
                    const bool ok = j < n_keys && ch * 8 < rank;
                    const size_t row = !ok ? 0 : one_page ? page_base + kr : (size_t)list[j / page_rows] * page_rows + j % page_rows;
                    const bf* src = ok ? pool + row * rank + ch * 8 : pool;
                    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(dstbuf + kr * RS + ch * 8);
                    const int bytes = ok ? 16 : 0;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
                }
            } else {
                for (int i = threadIdx.x; i < kHalfKeys * rpad; i += blockDim.x) {
                    const int kr = i / rpad, c = i - kr * rpad;
                    const int j = k0 + kr;
                    bf v = __float2bfloat16_rn(0.f);
                    if (j < n_keys && c < rank) v = pool[((size_t)list[j / page_rows] * page_rows + j % page_rows) * rank + c];
                    dstbuf[kr * RS + c] = v;
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        // the rank is split between the warp groups 0-3 and 4-7 in the score phase (k steps of 16)
        const int ksplit = (rpad / 32) * 16;
        const int kbeg = warp < 4 ? 0 : ksplit, kend = warp < 4 ? ksplit : rpad;
        if (!single && key_lo < n_keys) load_half(key_lo, Ks);
        int buf = 0;
        for (int k0 = key_lo; k0 < n_keys; k0 += kHalfKeys, buf ^= single ? 0 : 1) {
            bf* Kb = Ks + buf * kHalfKeys * RS;
            if (single) {
                __syncthreads();   // the buffer, Ss and Ps are no longer read
                load_half(k0, Ks);
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();   // half k0 has landed for everybody; the other buffer, Ss and Ps are no longer read
            if (!single && k0 + kHalfKeys < n_keys) load_half(k0 + kHalfKeys, Ks + (buf ^ 1) * kHalfKeys * RS);
            {   // ---- partial scores: keys [8 (warp & 3), +8), rank columns [kbeg, kend)
                float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                const bf* krow = Kb + ((warp & 3) * 8 + gid) * RS + tig * 2;
                const bf* q0 = Qs + ((lane & 7) + ((lane >> 3) & 1) * 8) * RS + (lane >> 4) * 8;
                const bf* q1 = q0 + 16 * RS;
                for (int ks = kbeg; ks < kend; ks += 16) {
                    uint32_t a0[4], a1[4], b[2];
                    ldsm_x4(a0, q0 + ks);
                    ldsm_x4(a1, q1 + ks);
                    b[0] = *reinterpret_cast<const uint32_t*>(krow + ks);
                    b[1] = *reinterpret_cast<const uint32_t*>(krow + ks + 8);
                    mma_bf16_16816(s[0], a0, b);
                    mma_bf16_16816(s[1], a1, b);
                }
                float* base = Ss + (warp >> 2) * kTileRows * 36;
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    float* d0 = base + (mt * 16 + gid) * 36 + (warp & 3) * 8 + tig * 2;
                    d0[0] = s[mt][0]; d0[1] = s[mt][1];
                    d0[8 * 36] = s[mt][2]; d0[8 * 36 + 1] = s[mt][3];
                }
            }
            __syncthreads();
#pragma unroll
            for (int i = 0; i < 4; ++i) {   // ---- softmax of rows [4 warp, 4 warp + 4): one key per lane
                const int r = warp * 4 + i, rp = row_pos[r];
                const int ka = k0 + lane;
                const bool seen = ka <= rp && (window <= 0 || ka > rp - window);
                const float sa = seen ? (Ss[r * 36 + lane] + Ss[(kTileRows + r) * 36 + lane]) * scale : -INFINITY;
                float mx = sa;
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
                const float mn = fmaxf(m_run[i], mx);           // finite: m starts at the sink (or at -1e30 in a share)
                const float pa = seen ? expf(sa - mn) : 0.f;
                float sum = pa;
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
                const float al = expf(m_run[i] - mn);
                l_run[i] = l_run[i] * al + sum;
                m_run[i] = mn;
                Ps[r * 72 + lane] = __float2bfloat16_rn(pa);    // after every lane has read its scores (the shuffles above)
                if (lane == 0) alpha_s[r] = al;
            }
            __syncthreads();
            {   // ---- O = O * alpha + P C for this warp's output columns
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    const float a0 = alpha_s[mt * 16 + gid], a1 = alpha_s[mt * 16 + gid + 8];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) { o[mt][nt][0] *= a0; o[mt][nt][1] *= a0; o[mt][nt][2] *= a1; o[mt][nt][3] *= a1; }
                }
#pragma unroll
                for (int kk = 0; kk < kHalfKeys; kk += 16) {
                    uint32_t p0[4], p1[4];
                    ldsm_x4(p0, Ps + ((lane & 7) + ((lane >> 3) & 1) * 8) * 72 + kk + (lane >> 4) * 8);
                    ldsm_x4(p1, Ps + (16 + (lane & 7) + ((lane >> 3) & 1) * 8) * 72 + kk + (lane >> 4) * 8);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const int tile = tile0 + nt;
                        if (nt < ntw && tile < n8) {
                            uint32_t b[2];
                            ldsm_x2_trans(b, Kb + (kk + (lane & 15)) * RS + tile * 8);
                            mma_bf16_16816(o[0][nt], p0, b);
                            mma_bf16_16816(o[1][nt], p1, b);
                        }
                    }
                }
            }
        }
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = warp * 4 + i;
                linv_s[r] = splits > 1 ? 1.0f : 1.0f / l_run[i];
                if (splits > 1 && row_pos[r] >= 0) {
                    float* pr = part + (((size_t)(t0 + r / HG) * heads + h0 + r % HG) * splits + blockIdx.z) * (rank + 2);
                    pr[0] = m_run[i];
                    pr[1] = l_run[i];
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = mt * 16 + gid + half * 8;
                if (row_pos[r] < 0) continue;
                const int tl = r / HG, h = h0 + r % HG;
                float* dst = splits > 1 ? part + (((size_t)(t0 + tl) * heads + h) * splits + blockIdx.z) * (rank + 2) + 2
                                        : out + ((size_t)(t0 + tl) * heads + h) * rank;
                const float inv = linv_s[r];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const int tile = tile0 + nt;
                    if (nt < ntw && tile < n8) {
                        const int c = tile * 8 + tig * 2;
                        if (c < out_cols) dst[c] = o[mt][nt][half * 2] * inv;
                        if (c + 1 < out_cols) dst[c + 1] = o[mt][nt][half * 2 + 1] * inv;
                    }
                }
            }
        first += cnt;
    }
}

// merges the shares of a split launch: grid (token, head)
__global__ void __launch_bounds__(128) latent_attn_combine_kernel(const float* __restrict__ part, float* __restrict__ out,
                                                                  const float* __restrict__ sink, int heads, int rank, int splits, int out_cols) {
    const int t = blockIdx.x, h = blockIdx.y;
    const float* p = part + ((size_t)t * heads + h) * splits * (rank + 2);
    const float sk = sink ? sink[h] : -INFINITY;
    float M = sk;
    for (int z = 0; z < splits; ++z) M = fmaxf(M, p[(size_t)z * (rank + 2)]);
    float den = expf(sk - M);
    for (int z = 0; z < splits; ++z) den += p[(size_t)z * (rank + 2) + 1] * expf(p[(size_t)z * (rank + 2)] - M);
    const float inv = 1.0f / den;
    for (int c = threadIdx.x; c < out_cols; c += blockDim.x) {
        float acc = 0.f;
        for (int z = 0; z < splits; ++z) acc += p[(size_t)z * (rank + 2) + 2 + c] * expf(p[(size_t)z * (rank + 2)] - M);
        out[((size_t)t * heads + h) * rank + c] = acc * inv;
    }
}

static bool tile_attention_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("B200_LATENT_ATTN_SIMT");   // 1: the per-(token, head) kernel for bfloat16 caches too
        v = (e && e[0] == '1') ? 0 : 1;
    }
    return v == 1;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_latent_store(const float* raw, long long ld_raw, const float* w, float eps, void* pool, const int* pages,
                                 int max_pages, int page_rows, const int* slot, const int* pos, int n_tokens, int rank,
                                 int dtype, void* stream) {
    if (!raw || !w || !pool || !pages || !slot || !pos || n_tokens < 0 || rank < 1 || page_rows < 1) return B200_EINVAL;
    if (n_tokens == 0) return B200_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == B200_BF16)
        latent_store_kernel<__nv_bfloat16><<<n_tokens, 128, 0, s>>>(raw, ld_raw, w, eps, (__nv_bfloat16*)pool, pages, max_pages,
                                                                   page_rows, slot, pos, rank);
    else if (dtype == B200_F32)
        latent_store_kernel<float><<<n_tokens, 128, 0, s>>>(raw, ld_raw, w, eps, (float*)pool, pages, max_pages, page_rows, slot,
                                                           pos, rank);
    else
        return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}

extern "C" size_t b200_latent_attention_workspace_bytes(int n_tokens, int heads, int rank) {
    return (size_t)n_tokens * heads * kMaxSplits * (rank + 2) * sizeof(float);
}

extern "C" int b200_latent_store_rot(const float* raw, long long ld_raw, const float* w, float eps, void* pool, const int* pages,
                                     int max_pages, int page_rows, const int* slot, const int* pos, int n_tokens, int rank, int extra,
                                     const float* cos, const float* sin, int rot_layout, int dtype, void* stream) {
    if (!raw || !w || !pool || !pages || !slot || !pos || n_tokens < 0 || rank < 1 || extra < 0 || page_rows < 1) return B200_EINVAL;
    if (extra > 0 && (!cos || !sin || (rot_layout != B200_ROPE_HALF && rot_layout != B200_ROPE_INTERLEAVED))) return B200_EINVAL;
    if (n_tokens == 0) return B200_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == B200_BF16)
        latent_store_rot_kernel<__nv_bfloat16><<<n_tokens, 128, 0, s>>>(raw, ld_raw, w, eps, (__nv_bfloat16*)pool, pages, max_pages, page_rows,
                                                                       slot, pos, rank, extra, cos, sin, rot_layout);
    else if (dtype == B200_F32)
        latent_store_rot_kernel<float><<<n_tokens, 128, 0, s>>>(raw, ld_raw, w, eps, (float*)pool, pages, max_pages, page_rows, slot, pos, rank,
                                                               extra, cos, sin, rot_layout);
    else
        return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}

extern "C" int b200_latent_attention(const float* qa, float* out, const void* pool, const int* pages, int max_pages,
                                     int page_rows, const int* slot, const int* pos, const float* sink, float scale,
                                     int n_tokens, int heads, int rank, int dtype, int longest_entry, int longest_context,
                                     void* workspace, size_t workspace_bytes, void* stream) {
    if (!sink) return B200_EINVAL;
    b200_latent_attention_args a{qa, out, pool, pages, max_pages, page_rows, slot, pos, sink, scale, n_tokens, heads, rank, 0, dtype,
                                 longest_entry, longest_context, workspace, workspace_bytes, 0};
    return b200_latent_attention_ex(&a, stream);
}

extern "C" int b200_latent_attention_ex(const b200_latent_attention_args* ap, void* stream) {
    if (!ap) return B200_EINVAL;
    const float* qa = ap->qa; float* out = ap->out; const void* pool = ap->pool; const int* pages = ap->pages;
    const int max_pages = ap->max_pages, page_rows = ap->page_rows; const int* slot = ap->slot; const int* pos = ap->pos;
    const float* sink = ap->sink; const float scale = ap->scale;
    const int n_tokens = ap->n_tokens, heads = ap->heads, rank = ap->rank, window = ap->window, dtype = ap->dtype, longest_entry = ap->longest_entry;
    const int longest_context = window > 0 && ap->longest_context > 0 ? std::min(ap->longest_context, window + kTileKeys) : ap->longest_context;
    void* workspace = ap->workspace; const size_t workspace_bytes = ap->workspace_bytes;
    const int out_cols = ap->out_cols > 0 && ap->out_cols < rank ? ap->out_cols : rank;
    if (!qa || !out || !pool || !pages || !slot || !pos || n_tokens < 0 || heads < 1 || rank < 1 || window < 0) return B200_EINVAL;
    if (rank > 32 * kMaxRankPerLane || heads > 65535) return B200_EUNSUPPORTED;
    if (n_tokens == 0) return B200_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = ((size_t)5 * rank + 8) * sizeof(float);
    dim3 grid(n_tokens, heads);
    if (dtype == B200_BF16 && tile_attention_enabled()) {
        // tensor-core form: 32 rows of (token, head) per CTA
        // every entry a single token (a decode batch): one token per CTA, its heads the only rows
        const int HG = heads < kTileRows ? heads : kTileRows, TQ = longest_entry == 1 ? 1 : kTileRows / HG;
        const int rpad = (rank + 15) & ~15, RS = rpad + 8;
        const int single = rpad > 512;   // with one half-tile buffer two CTAs of such rows still fit an SM
        const size_t tsm = (size_t)(kTileRows + (single ? kHalfKeys : kTileKeys)) * RS * 2 + 2 * kTileRows * 36 * 4 + 3 * kTileRows * 4;
        const int ntw = ((((out_cols + 15) & ~15) / 8) + kTileWarps - 1) / kTileWarps;
        dim3 tg((n_tokens + TQ - 1) / TQ, (heads + HG - 1) / HG);
        // few CTAs over long contexts (decoding): shares of the key tiles on blockIdx.z, merged by the combine kernel
        int splits = 1;
        if (longest_context > 0 && workspace) {
            const int tiles = (longest_context + kTileKeys - 1) / kTileKeys;
            const int want = (2 * sm_count()) / (int)(tg.x * tg.y);
            splits = std::max(1, std::min({want, tiles / 2, kMaxSplits}));
            if (workspace_bytes < (size_t)n_tokens * heads * splits * (rank + 2) * sizeof(float)) splits = 1;
        }
        tg.z = splits;
        float* part = reinterpret_cast<float*>(workspace);
        // every instantiation has the same function type, so the lambda is ONE function: a mask per kernel, not one static
        auto go = [&](auto kern, int which) -> int {
            static unsigned long long done[5] = {0, 0, 0, 0, 0};
            if (tsm > 48 * 1024 && ensure_max_dynamic_smem((const void*)kern, 200 * 1024, done[which]) != cudaSuccess) return B200_EUNSUPPORTED;
            kern<<<tg, 256, tsm, s>>>(qa, out, (const __nv_bfloat16*)pool, pages, max_pages, page_rows, slot, pos, sink, scale, n_tokens,
                                      heads, rank, HG, TQ, splits, part, window, out_cols, single);
            count_launch();
            if (splits > 1) {
                latent_attn_combine_kernel<<<dim3(n_tokens, heads), 128, 0, s>>>(part, out, sink, heads, rank, splits, out_cols);
                count_launch();
            }
            return (int)cudaGetLastError();
        };
        if (ntw <= 1) return go(latent_attn_tile_kernel<1>, 0);
        if (ntw <= 2) return go(latent_attn_tile_kernel<2>, 1);
        if (ntw <= 4) return go(latent_attn_tile_kernel<4>, 2);
        if (ntw <= 8) return go(latent_attn_tile_kernel<8>, 3);
        return go(latent_attn_tile_kernel<10>, 4);
    }
    if (dtype == B200_BF16)
        latent_attn_kernel<__nv_bfloat16><<<grid, 128, smem, s>>>(qa, out, (const __nv_bfloat16*)pool, pages, max_pages, page_rows,
                                                                 slot, pos, sink, scale, heads, rank, window);
    else if (dtype == B200_F32)
        latent_attn_kernel<float><<<grid, 128, smem, s>>>(qa, out, (const float*)pool, pages, max_pages, page_rows, slot, pos,
                                                         sink, scale, heads, rank, window);
    else
        return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}
