// Selective scan: a per-channel recurrence with a diagonal transition and input-dependent step sizes,
//   S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n,   y_c = sum_n S[c, n] C_n + D_c x_c,   out_c = y_c * silu(z_c),
// with dt = softplus(dt_raw + bias), the state S carried per sequence slot in fp32; and the short causal convolution
// with bias and silu in front of it (its last taps-1 inputs are carried per slot in a ring). Everything is fp32; only the
// GEMM operands these kernels hand on take the serving dtype.
//
//   conv_act_kernel          a thread per (token, channel): taps from this step's rows, the slot's ring or zeros.
//   selective_scan_kernel    a group of LP lanes owns one channel of one entry (a run of consecutive tokens of a
//                            sequence) and walks its tokens; a lane keeps up to 8 states in registers (eight consecutive
//                            ones behind 16-byte B / C loads when the state count fills the lanes, else state n of lane l
//                            is l + k LP behind predicated loads) and the channel's output is a shuffle sum over the group.
//                            Entries of 256 tokens or more are cut into chunks of 64 that run in parallel: chunk-local
//                            scans from zero, scan_carry_kernel over their summaries, then every chunk again from its
//                            true start state with outputs. bfloat16 serving takes exp(dt A) as exp2 of a pre-scaled A.
#include <cuda_bf16.h>

#include <algorithm>

#include "b200_serve.h"
#include "common.cuh"
#include "launch_count.h"

namespace b200 {

struct ConvAct {
    const float* u; long long ld_u; const float* w; const float* bias; int taps; const float* ring; float* ring_out;
    float* out32; void* out;
    const int* slot; const int* pos; const int* start;
    int channels;
};

template <typename T>
__global__ void __launch_bounds__(256) conv_act_kernel(const ConvAct a) {
    const int t = blockIdx.x, p = a.pos[t], b = a.slot[t], first = a.start[t], taps = a.taps, C = a.channels;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float y = a.bias ? a.bias[c] : 0.f;
        for (int j = 0; j < taps; ++j) {
            const int back = taps - 1 - j, src = p - back;
            if (src < 0) continue;
            const float uin = src >= first ? a.u[(size_t)(t - back) * a.ld_u + c]
                                           : a.ring[((size_t)b * (taps - 1) + src % (taps - 1)) * C + c];
            y = fmaf(a.w[(size_t)c * taps + j], uin, y);
        }
        // a one-token entry: nobody else reads this sequence's ring in this launch, and this thread has read its own places
        if (a.ring_out && taps > 1) a.ring_out[((size_t)b * (taps - 1) + p % (taps - 1)) * C + c] = a.u[(size_t)t * a.ld_u + c];
        y = y / (1.f + expf(-y));
        if (a.out32) a.out32[(size_t)t * C + c] = y;
        if (a.out) reinterpret_cast<T*>(a.out)[(size_t)t * C + c] = DT<T>::from_f(y);
    }
}

struct Scan {
    const float* x; const float* dt_raw; const float* dt_bias;
    const float* B; const float* C; long long ld_bc;
    const float* z; long long ld_z;
    const float* A; const float* D;
    float* state; void* out;
    const int* ent_row; const int* ent_len; const int* slot; const int* pos;
    int channels, n_state;
    // chunk form (entries of at least chunk_from tokens): chunk u covers tokens [chunk_first[u], + chunk) of entry chunk_ent[u]
    int chunk, chunk_from; const int* chunk_ent; const int* chunk_first; float* summary;
    int dt_ready;   // dt_raw holds the step sizes themselves
};

constexpr int kScanThreads = 128, kScanPerLane = 8, kScanGroup = 4;

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// MODE 0: the whole entry from the slot's state, which is left updated (decode steps, short portions; entries that take
//         the chunk form are skipped).
// MODE 1: one chunk from a zero state; leaves (sum of dt, local end state) per channel in `summary`, no outputs (the last
//         chunk of an entry has no successor and is skipped).
// MODE 2: one chunk from the state that the chunk scan left at its start (summary holds it), with outputs; the last
//         chunk of an entry stores the slot's state.
// FULL: every lane owns eight consecutive states (n_state == 8 LP) and the B / C rows allow 16-byte loads: no predicates on
// the state count, two vector loads per operand and token. Otherwise state n of lane l is l + k LP and every access is
// predicated.
template <typename T, int LP, int MODE, bool FULL>
__global__ void __launch_bounds__(kScanThreads) selective_scan_kernel(const Scan a) {
    constexpr int CPB = kScanThreads / LP;   // channels per CTA
    // bfloat16 serving: exp(dt A) as 2^(dt A log2 e) on the special-function unit (relative error about 2^-22); fp32
    // serving keeps the accurate exponential
    constexpr bool kFast = sizeof(T) == 2;
    const int lane = threadIdx.x % LP, c = blockIdx.x * CPB + threadIdx.x / LP, N = a.n_state, Cn = a.channels;
    const bool live = c < Cn;
    const int cc = live ? c : Cn - 1;        // lanes beyond the last channel walk along (shuffles need them) and store nothing
    int e, row0, len, first_pos, unit = 0;
    bool last_chunk = true;
    if (MODE == 0) {
        e = blockIdx.y;
        row0 = a.ent_row[e];
        len = a.ent_len[e];
        if (a.chunk > 0 && len >= a.chunk_from) return;
    } else {
        unit = blockIdx.y;
        e = a.chunk_ent[unit];
        if (e < 0) return;
        const int off = a.chunk_first[unit], elen = a.ent_len[e];
        row0 = a.ent_row[e] + off;
        len = min(a.chunk, elen - off);
        last_chunk = off + len >= elen;
        if (MODE == 1 && last_chunk) return;
    }
    first_pos = a.pos[row0];
    const int b = a.slot[row0];
    float S[kScanPerLane], Av[kScanPerLane];
    float* st = a.state + ((size_t)b * Cn + cc) * N;
    float* sm = MODE == 0 ? nullptr : a.summary + ((size_t)unit * Cn + cc) * (N + 1);
#pragma unroll
    for (int k = 0; k < kScanPerLane; ++k) {
        const int n = FULL ? lane * kScanPerLane + k : lane + k * LP;
        Av[k] = n < N ? a.A[(size_t)cc * N + n] * (kFast ? 1.4426950408889634f : 1.f) : 0.f;
        if (MODE == 0) S[k] = (n < N && first_pos > 0) ? st[n] : 0.f;
        else if (MODE == 1) S[k] = 0.f;
        else S[k] = n < N ? sm[1 + n] : 0.f;
    }
    const float dtb = a.dt_bias ? a.dt_bias[cc] : 0.f, Dc = a.D ? a.D[cc] : 0.f;
    float dt_sum = 0.f;
    // tokens in groups of kScanGroup: every operand of the group is loaded before the first update, so the walk pays one
    // round trip to memory per group and not one per token
    for (int i0 = 0; i0 < len; i0 += kScanGroup) {
        float dtr[kScanGroup], xv[kScanGroup], zv[kScanGroup], Bv[kScanGroup][kScanPerLane], Cv[kScanGroup][kScanPerLane];
#pragma unroll
        for (int j = 0; j < kScanGroup; ++j) {
            const bool in = i0 + j < len;
            const size_t t = (size_t)row0 + (in ? i0 + j : 0);
            dtr[j] = in ? __ldg(a.dt_raw + t * Cn + cc) : 0.f;
            xv[j] = in ? __ldg(a.x + t * Cn + cc) : 0.f;
            zv[j] = (MODE != 1 && in && lane == 0) ? __ldg(a.z + t * a.ld_z + cc) : 0.f;
            if (FULL) {
                const float4* bp = reinterpret_cast<const float4*>(a.B + t * a.ld_bc + lane * kScanPerLane);
                const float4* cp = reinterpret_cast<const float4*>(a.C + t * a.ld_bc + lane * kScanPerLane);
#pragma unroll
                for (int h = 0; h < kScanPerLane / 4; ++h) {
                    const float4 b4 = __ldg(bp + h), c4 = MODE != 1 ? __ldg(cp + h) : make_float4(0.f, 0.f, 0.f, 0.f);
                    Bv[j][4 * h] = b4.x; Bv[j][4 * h + 1] = b4.y; Bv[j][4 * h + 2] = b4.z; Bv[j][4 * h + 3] = b4.w;
                    Cv[j][4 * h] = c4.x; Cv[j][4 * h + 1] = c4.y; Cv[j][4 * h + 2] = c4.z; Cv[j][4 * h + 3] = c4.w;
                }
            } else {
#pragma unroll
                for (int k = 0; k < kScanPerLane; ++k) {
                    const int n = lane + k * LP;
                    Bv[j][k] = (in && n < N) ? __ldg(a.B + t * a.ld_bc + n) : 0.f;
                    Cv[j][k] = (MODE != 1 && in && n < N) ? __ldg(a.C + t * a.ld_bc + n) : 0.f;
                }
            }
        }
#pragma unroll
        for (int j = 0; j < kScanGroup; ++j) {
            if (i0 + j >= len) break;
            const float dt = a.dt_ready ? dtr[j] : softplus_f(dtr[j] + dtb), dx = dt * xv[j];
            float y = 0.f;
#pragma unroll
            for (int k = 0; k < kScanPerLane; ++k) {
                if (FULL || lane + k * LP < N) {
                    S[k] = fmaf(kFast ? exp2f(dt * Av[k]) : expf(dt * Av[k]), S[k], dx * Bv[j][k]);
                    if (MODE != 1) y = fmaf(S[k], Cv[j][k], y);
                }
            }
            if (MODE == 1) { dt_sum += dt; continue; }
#pragma unroll
            for (int o = LP / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
            if (lane == 0 && live)
                reinterpret_cast<T*>(a.out)[((size_t)row0 + i0 + j) * Cn + cc] = DT<T>::from_f((y + Dc * xv[j]) * (zv[j] / (1.f + expf(-zv[j]))));
        }
    }
    if (!live) return;
    if (MODE == 1) {
        if (lane == 0) sm[0] = dt_sum;
#pragma unroll
        for (int k = 0; k < kScanPerLane; ++k) {
            const int n = FULL ? lane * kScanPerLane + k : lane + k * LP;
            if (n < N) sm[1 + n] = S[k];
        }
    } else if (last_chunk) {
#pragma unroll
        for (int k = 0; k < kScanPerLane; ++k) {
            const int n = FULL ? lane * kScanPerLane + k : lane + k * LP;
            if (n < N) st[n] = S[k];
        }
    }
}

// Between MODE 1 and MODE 2: a thread per (entry, channel, state) walks the entry's chunks in order and replaces every
// chunk's local end state by the state at the chunk's START: S_start(k+1) = exp(A sum_dt(k)) S_start(k) + local_end(k).
__global__ void __launch_bounds__(256) scan_carry_kernel(const Scan a, const int* __restrict__ ent_chunk0, int n_entries) {
    const int N = a.n_state, Cn = a.channels;
    const size_t per = (size_t)Cn * N;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= per * n_entries) return;
    const int e = (int)(i / per), c = (int)((i % per) / N), n = (int)(i % N);
    const int u0 = ent_chunk0[e], u1 = ent_chunk0[e + 1];
    if (u0 == u1) return;
    const int row0 = a.ent_row[e];
    const float Av = a.A[(size_t)c * N + n];
    float S = a.pos[row0] > 0 ? a.state[((size_t)a.slot[row0] * Cn + c) * N + n] : 0.f;
    for (int g0 = u0; g0 < u1; g0 += 4) {   // the loads of four chunks in flight together
        float local[4], dts[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float* sm = a.summary + ((size_t)min(g0 + j, u1 - 1) * Cn + c) * (N + 1);
            local[j] = sm[1 + n];
            dts[j] = sm[0];
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (g0 + j >= u1) break;
            a.summary[((size_t)(g0 + j) * Cn + c) * (N + 1) + 1 + n] = S;
            S = fmaf(expf(Av * dts[j]), S, local[j]);
        }
    }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_conv_act(const b200_conv_act_args* p, void* stream) {
    if (!p || !p->u || !p->w || !p->slot || !p->pos || !p->start || p->taps < 1 || p->n_tokens < 0 || p->channels < 1 ||
        (p->taps > 1 && !p->conv_state) || (!p->out32 && !p->out))
        return B200_EINVAL;
    if (p->n_tokens == 0) return B200_OK;
    ConvAct a{p->u, p->ld_u, p->w, p->bias, p->taps, p->taps > 1 ? p->conv_state : p->u,
              p->update_state_inline ? const_cast<float*>(p->conv_state) : nullptr, p->out32, p->out, p->slot, p->pos, p->start, p->channels};
    const dim3 grid(p->n_tokens, std::min(64, (p->channels + 255) / 256));
    cudaStream_t s = (cudaStream_t)stream;
    if (p->out_dtype == B200_BF16) conv_act_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(a);
    else if (p->out_dtype == B200_F32) conv_act_kernel<float><<<grid, 256, 0, s>>>(a);
    else return B200_EINVAL;
    count_launch();
    return (int)cudaGetLastError();
}

namespace b200 {
constexpr int kScanChunk = 64;   // tokens per chunk of the chunk form
constexpr int kScanChunkFrom = 256;   // entries at least this long take it
static int scan_lanes(int n_state) {
    int lp = 1;
    while (lp < 32 && lp * kScanPerLane < n_state) lp *= 2;
    return lp;
}
template <typename T, int MODE, bool FULL>
static void scan_dispatch_lp(const Scan& a, int lp, dim3 grid, cudaStream_t s) {
    switch (lp) {
        case 1: selective_scan_kernel<T, 1, MODE, FULL><<<grid, kScanThreads, 0, s>>>(a); break;
        case 2: selective_scan_kernel<T, 2, MODE, FULL><<<grid, kScanThreads, 0, s>>>(a); break;
        case 4: selective_scan_kernel<T, 4, MODE, FULL><<<grid, kScanThreads, 0, s>>>(a); break;
        case 8: selective_scan_kernel<T, 8, MODE, FULL><<<grid, kScanThreads, 0, s>>>(a); break;
        case 16: selective_scan_kernel<T, 16, MODE, FULL><<<grid, kScanThreads, 0, s>>>(a); break;
        default: selective_scan_kernel<T, 32, MODE, FULL><<<grid, kScanThreads, 0, s>>>(a); break;
    }
}
template <typename T, int MODE>
static void scan_dispatch(const Scan& a, int lp, int units, cudaStream_t s) {
    const unsigned gx = (unsigned)((a.channels + kScanThreads / lp - 1) / (kScanThreads / lp));
    const dim3 grid(gx, units);
    const bool full = a.n_state == lp * kScanPerLane && a.ld_bc % 4 == 0 && (reinterpret_cast<uintptr_t>(a.B) & 15u) == 0 &&
                      (reinterpret_cast<uintptr_t>(a.C) & 15u) == 0;
    if (full) scan_dispatch_lp<T, MODE, true>(a, lp, grid, s);
    else scan_dispatch_lp<T, MODE, false>(a, lp, grid, s);
    count_launch();
}
}  // namespace b200

// Workspace of the chunk form: per chunk and channel (sum of dt, n_state states), then three int tables (chunk -> entry,
// chunk -> first token of the entry, entry -> first chunk).
static size_t scan_max_chunks(int n_tokens, int n_entries) { return (size_t)n_tokens / kScanChunk + (size_t)n_entries + 1; }
extern "C" size_t b200_selective_scan_workspace_bytes(int n_tokens, int n_entries, int channels, int n_state) {
    if (n_tokens < kScanChunkFrom || n_entries < 1 || channels < 1 || n_state < 1) return 0;
    const size_t chunks = scan_max_chunks(n_tokens, n_entries);
    return chunks * channels * (n_state + 1) * sizeof(float) + (2 * chunks + n_entries + 1) * sizeof(int);
}

namespace b200 {
// fills the chunk tables on the device from the entry lengths: one thread, the tables are tiny
__global__ void scan_tables_kernel(const int* __restrict__ ent_len, int n_entries, int chunk, int from, int* __restrict__ chunk_ent,
                                   int* __restrict__ chunk_first, int* __restrict__ ent_chunk0, int max_chunks) {
    if (threadIdx.x || blockIdx.x) return;
    int u = 0;
    for (int e = 0; e < n_entries; ++e) {
        ent_chunk0[e] = u;
        if (ent_len[e] < from) continue;
        for (int off = 0; off < ent_len[e] && u < max_chunks; off += chunk) {
            chunk_ent[u] = e;
            chunk_first[u] = off;
            ++u;
        }
    }
    ent_chunk0[n_entries] = u;
    for (; u < max_chunks; ++u) { chunk_ent[u] = -1; chunk_first[u] = 0; }
}
}  // namespace b200

extern "C" int b200_selective_scan(const b200_selective_scan_args* p, void* stream) {
    if (!p || !p->x || !p->dt_raw || !p->B || !p->C || !p->z || !p->A || !p->state || !p->out || !p->ent_row || !p->ent_len ||
        !p->slot || !p->pos || p->n_entries < 0 || p->n_tokens < 0 || p->channels < 1 || p->n_state < 1)
        return B200_EINVAL;
    if (p->n_state > 32 * kScanPerLane) return B200_EUNSUPPORTED;
    if (p->out_dtype != B200_BF16 && p->out_dtype != B200_F32) return B200_EINVAL;
    if (p->n_entries == 0 || p->n_tokens == 0) return B200_OK;
    if (p->n_entries > 65535) return B200_EUNSUPPORTED;
    Scan a{p->x, p->dt_raw, p->dt_bias, p->B, p->C, p->ld_bc, p->z, p->ld_z, p->A, p->D, p->state, p->out,
           p->ent_row, p->ent_len, p->slot, p->pos, p->channels, p->n_state, 0, 0, nullptr, nullptr, nullptr, p->dt_ready};
    const int lp = scan_lanes(p->n_state);
    cudaStream_t s = (cudaStream_t)stream;
    // long entries: chunk-local scans in parallel, a walk over the chunk summaries, then every chunk again from its true start
    const size_t need = b200_selective_scan_workspace_bytes(p->n_tokens, p->n_entries, p->channels, p->n_state);
    const size_t max_chunks = scan_max_chunks(p->n_tokens, p->n_entries);
    const bool chunked = p->longest_entry >= kScanChunkFrom && need > 0 && p->workspace && p->workspace_bytes >= need && max_chunks <= 65535;
    int* ent_chunk0 = nullptr;
    if (chunked) {
        a.chunk = kScanChunk;
        a.chunk_from = kScanChunkFrom;
        a.summary = reinterpret_cast<float*>(p->workspace);
        int* tables = reinterpret_cast<int*>(a.summary + max_chunks * p->channels * (p->n_state + 1));
        a.chunk_ent = tables;
        a.chunk_first = tables + max_chunks;
        ent_chunk0 = tables + 2 * max_chunks;
        scan_tables_kernel<<<1, 32, 0, s>>>(p->ent_len, p->n_entries, kScanChunk, kScanChunkFrom, tables, tables + max_chunks, ent_chunk0,
                                            (int)max_chunks);
        count_launch();
    }
    const bool bf = p->out_dtype == B200_BF16;
    if (bf) scan_dispatch<__nv_bfloat16, 0>(a, lp, p->n_entries, s);
    else scan_dispatch<float, 0>(a, lp, p->n_entries, s);
    if (chunked) {
        if (bf) scan_dispatch<__nv_bfloat16, 1>(a, lp, (int)max_chunks, s);
        else scan_dispatch<float, 1>(a, lp, (int)max_chunks, s);
        const size_t cells = (size_t)p->n_entries * p->channels * p->n_state;
        scan_carry_kernel<<<(unsigned)((cells + 255) / 256), 256, 0, s>>>(a, ent_chunk0, p->n_entries);
        count_launch();
        if (bf) scan_dispatch<__nv_bfloat16, 2>(a, lp, (int)max_chunks, s);
        else scan_dispatch<float, 2>(a, lp, (int)max_chunks, s);
    }
    return (int)cudaGetLastError();
}
