// b200_gemm_grouped: C = A W^T (or A W) with the row bookkeeping that mixture-of-experts layers and per-head
// (strided) projections need, beside linear.cu's plain b200_linear:
//   * strided batches      : blockIdx.z = batch, A / W / C advance by element strides, rows have leading dimensions
//                            (a head's slice of a wider activation is addressed in place, no copies)
//   * groups               : blockIdx.z = group g owns rows [group_off[g], group_off[g+1]) of A and C and weight g
//                            (the experts of a routed layer; the offsets live on the DEVICE, no host sync)
//   * row gather           : A row r is a_rows[r] of the source (tokens sorted by expert are never materialised)
//   * epilogues            : none | acc * sigmoid(aux) (output gate) | silu(acc_gate) * acc_up (GLU: the W tile holds
//                            gate rows [0, N) and up rows [N, 2N) of the same features, the [M, 2N] intermediate is
//                            never stored)
// Element types: A and W float or bfloat16 (any mix), C float or bfloat16; accumulation is fp32 FMA in k order, so a
// row's result does not depend on which other rows share the launch. Two kernels behind the entry point:
//   gemm_grouped_mma_kernel  : bf16 operands (A converted on load), mma.sync m16n8k16, 64 or 128 x 64 x 64 tiles,
//                              ldmatrix fragments, 16-byte loads staged through registers one k tile ahead
//   gemm_grouped_simt_kernel : every combination, true fp32 products (the float32 serving mode)
#include <cuda_bf16.h>

#include "b200_serve.h"
#include "common.cuh"
#include "launch_count.h"

namespace b200 {

struct GG {
    const void* A; const void* W; void* C; const float* aux;
    const int* a_rows; const int* group_off;
    long long lda, ldw, ldc, ld_aux, sA, sW, sC, s_aux;
    int M, N, K, epi;
    float epi_param;
};

constexpr int GBM = 64, GBN = 64, GBK = 16;

template <typename TC>
__device__ __forceinline__ void gg_store(const GG& g, TC* C, long long row, int col, float v, float v2, long long aux_off) {
    if (g.epi == B200_GG_SIGMOID_MUL) v *= 1.f / (1.f + expf(-g.aux[aux_off + row * g.ld_aux + col]));
    else if (g.epi == B200_GG_GLU) v = v / (1.f + expf(-v)) * v2;
    else if (g.epi == B200_GG_GLU_GELU) v = gelu_tanh_f(v) * v2;
    else if (g.epi == B200_GG_GLU_CLAMP) v = glu_clamp_f(v, v2, g.epi_param);
    else if (g.epi == B200_GG_RELU2) { v = fmaxf(v, 0.f); v *= v; }
    else if (g.epi == B200_GG_BIAS_SOFTPLUS) {
        v += g.aux[aux_off + row * g.ld_aux + col];
        v = v > 20.f ? v : log1pf(expf(v));
    }
    C[row * g.ldc + col] = DT<TC>::from_f(v);
}

template <typename TA, typename TW, typename TC, bool TRANS_B, bool GLU>
__global__ void __launch_bounds__(256) gemm_grouped_simt_kernel(GG g) {
    __shared__ float As[GBK][GBM + 1];
    __shared__ float Bs[GLU ? 2 : 1][GBK][GBN + 1];
    const int z = blockIdx.z;
    long long row0 = 0;
    int M = g.M;
    const TA* A = (const TA*)g.A;
    const TW* W = (const TW*)g.W + (size_t)z * g.sW;
    TC* C = (TC*)g.C;
    long long aux_off = 0;
    if (g.group_off) {
        row0 = g.group_off[z];
        M = g.group_off[z + 1] - (int)row0;
    } else {
        A += (size_t)z * g.sA;
        C += (size_t)z * g.sC;
        aux_off = (long long)z * g.s_aux;
    }
    const int m0 = blockIdx.y * GBM, n0 = blockIdx.x * GBN;
    if (m0 >= M) return;
    const int N = g.N, K = g.K;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float acc[4][4], acc2[GLU ? 4 : 1][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) { acc[i][j] = 0.f; if (GLU) acc2[i][j] = 0.f; }
    // the source row of each of the tile's 64 rows (gather), resolved once
    __shared__ long long arow[GBM];
    if (threadIdx.x < GBM) {
        const int r = m0 + threadIdx.x;
        long long src = -1;
        if (r < M) src = g.a_rows ? (long long)g.a_rows[row0 + r] : row0 + r;
        arow[threadIdx.x] = src;
    }
    __syncthreads();
    for (int k0 = 0; k0 < K; k0 += GBK) {
        for (int i = threadIdx.x; i < GBM * GBK; i += 256) {
            const int r = i / GBK, kk = i - r * GBK;
            const int gk = k0 + kk;
            const long long src = arow[r];
            As[kk][r] = (src >= 0 && gk < K) ? DT<TA>::to_f(A[src * g.lda + gk]) : 0.f;
        }
        if (TRANS_B) {
            for (int i = threadIdx.x; i < GBN * GBK; i += 256) {
                const int c = i / GBK, kk = i - c * GBK;
                const int gn = n0 + c, gk = k0 + kk;
                const bool ok = gn < N && gk < K;
                Bs[0][kk][c] = ok ? DT<TW>::to_f(W[(long long)gn * g.ldw + gk]) : 0.f;
                if (GLU) Bs[GLU ? 1 : 0][kk][c] = ok ? DT<TW>::to_f(W[(long long)(gn + N) * g.ldw + gk]) : 0.f;
            }
        } else {
            for (int i = threadIdx.x; i < GBN * GBK; i += 256) {
                const int kk = i / GBN, c = i - kk * GBN;
                const int gn = n0 + c, gk = k0 + kk;
                Bs[0][kk][c] = (gn < N && gk < K) ? DT<TW>::to_f(W[(long long)gk * g.ldw + gn]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GBK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[0][kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
            if (GLU) {
#pragma unroll
                for (int j = 0; j < 4; ++j) b[j] = Bs[GLU ? 1 : 0][kk][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc2[GLU ? i : 0][j] = fmaf(a[i], b[j], acc2[GLU ? i : 0][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = m0 + ty * 4 + i;
        if (r >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = n0 + tx * 4 + j;
            if (c >= N) continue;
            gg_store<TC>(g, C, row0 + r, c, acc[i][j], GLU ? acc2[GLU ? i : 0][j] : 0.f, aux_off);
        }
    }
}

// ---- bf16 tensor-core tile: 64 x 64 x 32, 4 warps (2 x 2), each warp 32 x 32 = 2 m16 x 4 n8 fragments -----------
constexpr int MBK = 64, MPAD = 8;   // smem rows of 72 bf16 (144 B): ldmatrix rows fall into distinct 16-byte bank groups
constexpr int CPR = MBK / 8;        // 16-byte packets per tile row

__device__ __forceinline__ void gg_ldsm_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// eight consecutive elements as bf16 in one 16-byte packet (fp32 sources are rounded on the way)
template <typename T> __device__ __forceinline__ Pack16 load8_bf16(const T* p);
template <> __device__ __forceinline__ Pack16 load8_bf16<__nv_bfloat16>(const __nv_bfloat16* p) { return ld16(p); }
template <> __device__ __forceinline__ Pack16 load8_bf16<float>(const float* p) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    Pack16 v;
    __nv_bfloat162 h;
    h = __floats2bfloat162_rn(a.x, a.y); v.w[0] = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(a.z, a.w); v.w[1] = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(b.x, b.y); v.w[2] = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(b.z, b.w); v.w[3] = *reinterpret_cast<uint32_t*>(&h);
    return v;
}

// VEC: every row of A and W starts on a 16-byte boundary (32 for fp32 A) and K % 8 == 0: 16-byte global loads, the next
// k tile fetched into registers while the tensor cores work on the current one
// BM: rows per CTA, 64 (4 warps) or 128 (8 warps: the weight tile is read half as often, twice the MMAs per barrier)
template <typename TA, typename TC, bool TRANS_B, bool GLU, bool VEC = false, int BM = 64>
__global__ void __launch_bounds__(BM * 2) gemm_grouped_mma_kernel(GG g) {
    constexpr int NT = BM * 2;        // threads
    constexpr int NA = BM * CPR / NT;      // 16-byte packets of the A tile per thread
    constexpr int NB = GBN * CPR / NT;     // ... of the W tile
    using bf = __nv_bfloat16;
    __shared__ __align__(16) bf As[BM][MBK + MPAD];
    __shared__ __align__(16) bf Bs[GLU ? 2 : 1][GBN][MBK + MPAD];   // [n][k] (k contiguous) whatever W's layout
    __shared__ long long arow[BM];
    const int z = blockIdx.z;
    long long row0 = 0;
    int M = g.M;
    const TA* A = (const TA*)g.A;
    const bf* W = (const bf*)g.W + (size_t)z * g.sW;
    TC* C = (TC*)g.C;
    long long aux_off = 0;
    if (g.group_off) {
        row0 = g.group_off[z];
        M = g.group_off[z + 1] - (int)row0;
    } else {
        A += (size_t)z * g.sA;
        C += (size_t)z * g.sC;
        aux_off = (long long)z * g.s_aux;
    }
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * GBN;
    if (m0 >= M) return;
    const int N = g.N, K = g.K;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int wm = (warp / 2) * 32, wn = (warp % 2) * 32;
    const int gid = lane / 4, tig = lane % 4;
    float acc[2][4][4], acc2[GLU ? 2 : 1][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int k = 0; k < 4; ++k) { acc[i][j][k] = 0.f; if (GLU) acc2[i][j][k] = 0.f; }
    if (threadIdx.x < BM) {
        const int r = m0 + threadIdx.x;
        long long src = -1;
        if (r < M) src = g.a_rows ? (long long)g.a_rows[row0 + r] : row0 + r;
        arow[threadIdx.x] = src;
    }
    __syncthreads();
    // VEC: BM x MBK / 8 packets of 8 for A (NA per thread), GBN x MBK / 8 for the W tile (NB per thread)
    Pack16 ra[NA], rb[GLU ? 2 * NB : NB];
    auto fetch = [&](int k0) {
        Pack16 z; z.w[0] = z.w[1] = z.w[2] = z.w[3] = 0u;
#pragma unroll
        for (int i = 0; i < NA; ++i) {
            const int c = threadIdx.x + i * NT, r = c / CPR, gk = k0 + (c % CPR) * 8;
            const long long src = arow[r];
            ra[i] = (src >= 0 && gk < K) ? load8_bf16<TA>(A + src * g.lda + gk) : z;
        }
#pragma unroll
        for (int i = 0; i < NB; ++i) {
            const int c = threadIdx.x + i * NT;
            if (TRANS_B) {
                const int gn = n0 + c / CPR, gk = k0 + (c % CPR) * 8;
                const bool ok = gn < N && gk < K;
                rb[i] = ok ? ld16(W + (long long)gn * g.ldw + gk) : z;
                if (GLU) rb[GLU ? NB + i : 0] = ok ? ld16(W + (long long)(gn + N) * g.ldw + gk) : z;
            } else {   // W [K, N]: packets of 8 along n, transposed on the way into shared memory
                const int bk = k0 + (c >> 3), gn = n0 + (c & 7) * 8;
                rb[i] = (bk < K && gn < N) ? ld16(W + (long long)bk * g.ldw + gn) : z;
            }
        }
    };
    if (VEC) fetch(0);
    for (int k0 = 0; k0 < K; k0 += MBK) {
        if (VEC) {
#pragma unroll
            for (int i = 0; i < NA; ++i) {
                const int c = threadIdx.x + i * NT;
                st16(&As[c / CPR][(c % CPR) * 8], ra[i]);
            }
#pragma unroll
            for (int i = 0; i < NB; ++i) {
                const int c = threadIdx.x + i * NT;
                if (TRANS_B) {
                    st16(&Bs[0][c / CPR][(c % CPR) * 8], rb[i]);
                    if (GLU) st16(&Bs[GLU ? 1 : 0][c / CPR][(c % CPR) * 8], rb[GLU ? NB + i : 0]);
                } else {
                    const int bk = c >> 3, nc = (c & 7) * 8;
                    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&rb[i]);
#pragma unroll
                    for (int j = 0; j < 8; ++j) Bs[0][nc + j][bk] = e[j];
                }
            }
            __syncthreads();
            if (k0 + MBK < K) fetch(k0 + MBK);
        } else {
        for (int i = threadIdx.x; i < BM * MBK; i += NT) {
            const int r = i / MBK, kk = i - r * MBK;
            const int gk = k0 + kk;
            const long long src = arow[r];
            As[r][kk] = (src >= 0 && gk < K) ? __float2bfloat16_rn(DT<TA>::to_f(A[src * g.lda + gk])) : __float2bfloat16_rn(0.f);
        }
        if (TRANS_B) {
            for (int i = threadIdx.x; i < GBN * MBK; i += NT) {
                const int c = i / MBK, kk = i - c * MBK;
                const int gn = n0 + c, gk = k0 + kk;
                const bool ok = gn < N && gk < K;
                Bs[0][c][kk] = ok ? W[(long long)gn * g.ldw + gk] : __float2bfloat16_rn(0.f);
                if (GLU) Bs[GLU ? 1 : 0][c][kk] = ok ? W[(long long)(gn + N) * g.ldw + gk] : __float2bfloat16_rn(0.f);
            }
        } else {
            for (int i = threadIdx.x; i < GBN * MBK; i += NT) {
                const int kk = i / GBN, c = i - kk * GBN;
                const int gn = n0 + c, gk = k0 + kk;
                Bs[0][c][kk] = (gn < N && gk < K) ? W[(long long)gk * g.ldw + gn] : __float2bfloat16_rn(0.f);
            }
        }
        __syncthreads();
        }
#pragma unroll
        for (int ks = 0; ks < MBK; ks += 16) {
            // fragments by ldmatrix: one x4 per 16 x 16 block of A, one x4 per pair of n8 tiles of B
            uint32_t a[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i)
                gg_ldsm_x4(a[i], &As[wm + i * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][ks + (lane >> 4) * 8]);
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                uint32_t b4[4];
                gg_ldsm_x4(b4, &Bs[0][wn + j * 8 + (lane & 7) + ((lane >> 4) & 1) * 8][ks + ((lane >> 3) & 1) * 8]);
                const uint32_t b0[2] = {b4[0], b4[1]}, b1[2] = {b4[2], b4[3]};
                mma_bf16(acc[0][j], a[0], b0);
                mma_bf16(acc[1][j], a[1], b0);
                mma_bf16(acc[0][j + 1], a[0], b1);
                mma_bf16(acc[1][j + 1], a[1], b1);
                if (GLU) {
                    gg_ldsm_x4(b4, &Bs[GLU ? 1 : 0][wn + j * 8 + (lane & 7) + ((lane >> 4) & 1) * 8][ks + ((lane >> 3) & 1) * 8]);
                    const uint32_t u0[2] = {b4[0], b4[1]}, u1[2] = {b4[2], b4[3]};
                    mma_bf16(acc2[0][j], a[0], u0);
                    mma_bf16(acc2[GLU ? 1 : 0][j], a[1], u0);
                    mma_bf16(acc2[0][GLU ? j + 1 : 0], a[0], u1);
                    mma_bf16(acc2[GLU ? 1 : 0][GLU ? j + 1 : 0], a[1], u1);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int r = m0 + wm + i * 16 + gid + (k / 2) * 8;
                const int c = n0 + wn + j * 8 + tig * 2 + (k % 2);
                if (r < M && c < N)
                    gg_store<TC>(g, C, row0 + r, c, acc[i][j][k], GLU ? acc2[GLU ? i : 0][j][k] : 0.f, aux_off);
            }
}

template <typename TA, typename TW, typename TC>
static int gg_launch_simt(const GG& g, dim3 grid, bool trans_b, cudaStream_t s) {
    if (g.epi == B200_GG_GLU || g.epi == B200_GG_GLU_GELU || g.epi == B200_GG_GLU_CLAMP) {
        if (!trans_b) return B200_EUNSUPPORTED;
        gemm_grouped_simt_kernel<TA, TW, TC, true, true><<<grid, 256, 0, s>>>(g);
    } else if (trans_b)
        gemm_grouped_simt_kernel<TA, TW, TC, true, false><<<grid, 256, 0, s>>>(g);
    else
        gemm_grouped_simt_kernel<TA, TW, TC, false, false><<<grid, 256, 0, s>>>(g);
    return (int)cudaGetLastError();
}
template <typename TA, typename TC, bool TRANS_B, bool GLU>
static void gg_launch_mma_tile(const GG& g, dim3 grid, bool vec, bool tall, cudaStream_t s) {
    if (tall) {
        grid.y = (grid.y + 1) / 2;
        if (vec) gemm_grouped_mma_kernel<TA, TC, TRANS_B, GLU, true, 128><<<grid, 256, 0, s>>>(g);
        else gemm_grouped_mma_kernel<TA, TC, TRANS_B, GLU, false, 128><<<grid, 256, 0, s>>>(g);
    } else {
        if (vec) gemm_grouped_mma_kernel<TA, TC, TRANS_B, GLU, true, 64><<<grid, 128, 0, s>>>(g);
        else gemm_grouped_mma_kernel<TA, TC, TRANS_B, GLU, false, 64><<<grid, 128, 0, s>>>(g);
    }
}
template <typename TA, typename TC>
static int gg_launch_mma(const GG& g, dim3 grid, bool trans_b, cudaStream_t s) {
    auto al = [](const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; };
    const bool vec = g.K % 8 == 0 && g.lda % 8 == 0 && g.ldw % 8 == 0 && g.sA % 8 == 0 && g.sW % 8 == 0 &&
                     al(g.A, sizeof(TA) * 8) && al(g.W, 16) && (trans_b || g.N % 8 == 0);
    const bool tall = g.M > 64;   // the grid was sized for 64-row tiles (M is the row bound of a group)
    if (g.epi == B200_GG_GLU || g.epi == B200_GG_GLU_GELU || g.epi == B200_GG_GLU_CLAMP) {
        if (!trans_b) return B200_EUNSUPPORTED;
        gg_launch_mma_tile<TA, TC, true, true>(g, grid, vec, tall, s);
    } else if (trans_b)
        gg_launch_mma_tile<TA, TC, true, false>(g, grid, vec, tall, s);
    else
        gg_launch_mma_tile<TA, TC, false, false>(g, grid, vec, tall, s);
    return (int)cudaGetLastError();
}

int gemm_tcgen05_ex(const void* x, const void* W, void* y, int M, int N, int K, int in_bf16, int out_kind, int glu, void* workspace,
                    size_t workspace_bytes, cudaStream_t s, float glu_limit = 0.f);   // gemm_tcgen05.cu (glu: 0 none, 1 silu, 2 tanh-gelu, 3 no GLU but relu squared, 4 clamped)
size_t gemm_tcgen05_ex_workspace_bytes(int M, int N, int K);

static bool mma_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("B200_GG_SIMT");   // 1: bf16 operands on the SIMT kernel too (debugging aid)
        v = (e && e[0] == '1') ? 0 : 1;
    }
    return v == 1;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_gemm_grouped(const b200_gemm_grouped_args* p, void* stream) {
    if (!p || !p->A || !p->W || !p->C || p->N <= 0 || p->K <= 0 || p->M < 0 || p->batch < 1) return B200_EINVAL;
    if (p->M == 0) return B200_OK;
    if ((p->epi == B200_GG_SIGMOID_MUL || p->epi == B200_GG_BIAS_SOFTPLUS) && !p->aux) return B200_EINVAL;
    GG g;
    g.A = p->A; g.W = p->W; g.C = p->C; g.aux = p->aux; g.a_rows = p->a_rows; g.group_off = p->group_off;
    g.lda = p->lda; g.ldw = p->ldw; g.ldc = p->ldc; g.ld_aux = p->ld_aux;
    g.sA = p->stride_a; g.sW = p->stride_w; g.sC = p->stride_c; g.s_aux = p->stride_aux;
    g.M = p->M; g.N = p->N; g.K = p->K; g.epi = p->epi; g.epi_param = p->epi_param;
    if (p->epi == B200_GG_GLU_CLAMP && !(p->epi_param > 0.f)) return B200_EINVAL;
    // groups: M is the largest number of rows one group can own (the grid covers it; CTAs beyond a group's rows leave)
    dim3 grid((p->N + GBN - 1) / GBN, (p->M + GBM - 1) / GBM, p->batch);
    if (grid.y > 65535 || grid.z > 65535) return B200_EUNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const bool tb = p->trans_b != 0;
    using bf = __nv_bfloat16;
    const int ta = p->a_dtype, tw = p->w_dtype, tc = p->c_dtype;
    int rc = B200_EUNSUPPORTED;
    if (tw == B200_BF16 && mma_enabled()) {
        if (ta == B200_BF16 && tc == B200_F32) rc = gg_launch_mma<bf, float>(g, grid, tb, s);
        else if (ta == B200_BF16 && tc == B200_BF16) rc = gg_launch_mma<bf, bf>(g, grid, tb, s);
        else if (ta == B200_F32 && tc == B200_F32) rc = gg_launch_mma<float, float>(g, grid, tb, s);
        else if (ta == B200_F32 && tc == B200_BF16) rc = gg_launch_mma<float, bf>(g, grid, tb, s);
    } else if (tw == B200_BF16) {
        if (ta == B200_BF16 && tc == B200_F32) rc = gg_launch_simt<bf, bf, float>(g, grid, tb, s);
        else if (ta == B200_BF16 && tc == B200_BF16) rc = gg_launch_simt<bf, bf, bf>(g, grid, tb, s);
        else if (ta == B200_F32 && tc == B200_F32) rc = gg_launch_simt<float, bf, float>(g, grid, tb, s);
        else if (ta == B200_F32 && tc == B200_BF16) rc = gg_launch_simt<float, bf, bf>(g, grid, tb, s);
    } else if (tw == B200_F32 && ta == B200_F32 && tc == B200_F32) {
        rc = gg_launch_simt<float, float, float>(g, grid, tb, s);
    }
    if (rc == 0) count_launch();
    return rc;
}

extern "C" size_t b200_linear_ex_workspace_bytes(int n_tokens, int N, int K) {
    return n_tokens > 0 && N > 0 && K > 0 ? gemm_tcgen05_ex_workspace_bytes(n_tokens, N, K) : 0;
}

extern "C" int b200_linear_ex(const void* x, const void* W, void* y, int n_tokens, int N, int K, int in_dtype, int out_dtype, int epi,
                              void* workspace, size_t workspace_bytes, void* stream) {
    if (epi == B200_GG_GLU_CLAMP) return B200_EINVAL;   // needs its limit: b200_linear_ex2
    return b200_linear_ex2(x, W, y, n_tokens, N, K, in_dtype, out_dtype, epi, 0.f, workspace, workspace_bytes, stream);
}

extern "C" int b200_linear_ex2(const void* x, const void* W, void* y, int n_tokens, int N, int K, int in_dtype, int out_dtype, int epi,
                               float epi_param, void* workspace, size_t workspace_bytes, void* stream) {
    if (!x || !W || !y || n_tokens < 0 || N < 1 || K < 1 ||
        (epi != B200_GG_NONE && epi != B200_GG_GLU && epi != B200_GG_GLU_GELU && epi != B200_GG_RELU2 && epi != B200_GG_GLU_CLAMP))
        return B200_EINVAL;
    if (epi == B200_GG_GLU_CLAMP && !(epi_param > 0.f)) return B200_EINVAL;
    if (n_tokens == 0) return B200_OK;
    if (in_dtype == B200_BF16 && (out_dtype == B200_BF16 || out_dtype == B200_F32)) {
        const int glu = epi == B200_GG_GLU ? 1 : epi == B200_GG_GLU_GELU ? 2 : epi == B200_GG_RELU2 ? 3 : epi == B200_GG_GLU_CLAMP ? 4 : 0;
        const int rc = gemm_tcgen05_ex(x, W, y, n_tokens, N, K, 1, out_dtype == B200_BF16 ? 1 : 2, glu, workspace, workspace_bytes,
                                       (cudaStream_t)stream, epi_param);
        if (rc != B200_EUNSUPPORTED) return rc;
    }
    b200_gemm_grouped_args g{};
    g.A = x; g.W = W; g.C = y;
    g.lda = K; g.ldw = K; g.ldc = N;
    g.M = n_tokens; g.N = N; g.K = K; g.batch = 1; g.trans_b = 1; g.epi = epi; g.epi_param = epi_param;
    g.a_dtype = in_dtype; g.w_dtype = in_dtype; g.c_dtype = out_dtype;
    return b200_gemm_grouped(&g, stream);
}
