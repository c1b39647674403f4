// b200_gated_recurrence: an element-wise gated recurrence whose gate and candidate read only the current token,
//   S_t = (1 - z_t) S_(t-1) + z_t c_t,   z = sigmoid(.), c = u + 1/2 (u >= 0) | sigmoid(u) (u < 0),   out_t = S_t * silu(g_t)
// with one fp32 state per (sequence slot, channel). The recurrence is linear in S, S_t = a_t S_(t-1) + b_t with a = 1 - z and
// b = z c, so a run of tokens folds into one pair (A, B) = (prod a, its end state from zero) and long entries are cut into
// chunks of kGrChunk tokens:
//   gr_direct_kernel    entries of at most one chunk (decode batches, short portions): a thread per (entry, channel) walks
//                       its tokens from the carried state and leaves the new one
//   gr_summary_kernel   (A, B) of every chunk, a thread per (chunk, channel)
//   gr_carry_kernel     a thread per (entry, channel) folds the chunk pairs in order from the carried state: the start state
//                       of every chunk, and the entry's end state to the slot
//   gr_direct_kernel    again, per chunk, from the chunk's start state, writing the outputs
// Gate, candidate, state and output product are fp32; only the store takes the serving dtype. A slot that is used again
// needs no clearing: an entry that starts at position 0 starts from zero.
#include <cuda_bf16.h>

#include "b200_serve.h"
#include "common.cuh"
#include "launch_count.h"

namespace b200 {

constexpr int kGrChunk = 64, kGrThreads = 128;

struct GR {
    const float* pre; long long ld_pre; int z_off, u_off, g_off;
    const float* z_bias; const float* u_bias;
    float* state; void* out;
    const int* ent_row; const int* ent_len; const int* slot; const int* pos;
    int channels, chunks_per_entry;
    float* sumA; float* sumB; float* start;   // [chunk place, channel]
};
// Table place of chunk k of entry e: entries are packed back to back, so first row / chunk + e + k never collides and the
// table has at most tokens / chunk + entries + 1 places.
__device__ __forceinline__ size_t gr_place(const GR& a, int e, int k) { return (size_t)(a.ent_row[e] / kGrChunk + e + k); }

__device__ __forceinline__ float gr_sigmoid(float v) { return 1.f / (1.f + expf(-v)); }
// (a, b) of one token and channel
__device__ __forceinline__ void gr_coeffs(const GR& a, const float* row, int c, float zb, float ub, float& ka, float& kb) {
    const float z = gr_sigmoid(row[a.z_off + c] + zb);
    const float u = row[a.u_off + c] + ub;
    const float cand = u >= 0.f ? u + 0.5f : gr_sigmoid(u);
    ka = 1.f - z;
    kb = z * cand;
}

// grid (channel blocks, entries, chunks): CHUNKED false walks the whole entry (at most one chunk long) from the slot's state
template <typename T, bool CHUNKED>
__global__ void __launch_bounds__(kGrThreads) gr_direct_kernel(const GR a) {
    const int c = blockIdx.x * kGrThreads + threadIdx.x, e = blockIdx.y, k = blockIdx.z;
    const int len = a.ent_len[e], t0 = a.ent_row[e] + k * kGrChunk;
    if (c >= a.channels || k * kGrChunk >= len) return;
    const int n = min(kGrChunk, len - k * kGrChunk);
    const int b = a.slot[t0];
    float S;
    if (CHUNKED) S = a.start[gr_place(a, e, k) * a.channels + c];
    else S = a.pos[t0] > 0 ? a.state[(size_t)b * a.channels + c] : 0.f;
    const float zb = a.z_bias ? a.z_bias[c] : 0.f, ub = a.u_bias ? a.u_bias[c] : 0.f;
    T* out = reinterpret_cast<T*>(a.out);
    for (int i = 0; i < n; ++i) {
        const float* row = a.pre + (size_t)(t0 + i) * a.ld_pre;
        float ka, kb;
        gr_coeffs(a, row, c, zb, ub, ka, kb);
        S = fmaf(ka, S, kb);
        const float g = row[a.g_off + c];
        out[(size_t)(t0 + i) * a.channels + c] = DT<T>::from_f(S * (g * gr_sigmoid(g)));
    }
    if (!CHUNKED) a.state[(size_t)b * a.channels + c] = S;
}

__global__ void __launch_bounds__(kGrThreads) gr_summary_kernel(const GR a) {
    const int c = blockIdx.x * kGrThreads + threadIdx.x, e = blockIdx.y, k = blockIdx.z;
    const int len = a.ent_len[e], t0 = a.ent_row[e] + k * kGrChunk;
    if (c >= a.channels || k * kGrChunk >= len) return;
    const int n = min(kGrChunk, len - k * kGrChunk);
    const float zb = a.z_bias ? a.z_bias[c] : 0.f, ub = a.u_bias ? a.u_bias[c] : 0.f;
    float A = 1.f, B = 0.f;
    for (int i = 0; i < n; ++i) {
        float ka, kb;
        gr_coeffs(a, a.pre + (size_t)(t0 + i) * a.ld_pre, c, zb, ub, ka, kb);
        A *= ka;
        B = fmaf(ka, B, kb);
    }
    const size_t at = gr_place(a, e, k) * a.channels + c;
    a.sumA[at] = A;
    a.sumB[at] = B;
}

__global__ void __launch_bounds__(kGrThreads) gr_carry_kernel(const GR a) {
    const int c = blockIdx.x * kGrThreads + threadIdx.x, e = blockIdx.y;
    if (c >= a.channels) return;
    const int len = a.ent_len[e], t0 = a.ent_row[e], b = a.slot[t0];
    float S = a.pos[t0] > 0 ? a.state[(size_t)b * a.channels + c] : 0.f;
    const int chunks = (len + kGrChunk - 1) / kGrChunk;
    for (int k = 0; k < chunks; ++k) {
        const size_t at = gr_place(a, e, k) * a.channels + c;
        a.start[at] = S;
        S = fmaf(a.sumA[at], S, a.sumB[at]);
    }
    a.state[(size_t)b * a.channels + c] = S;
}

}  // namespace b200

using namespace b200;

extern "C" size_t b200_gated_recurrence_workspace_bytes(int n_tokens, int n_entries, int channels) {
    if (n_tokens < 1 || n_entries < 1 || channels < 1) return 0;
    const size_t places = (size_t)n_tokens / kGrChunk + n_entries + 1;
    return 3 * places * channels * sizeof(float);
}

extern "C" int b200_gated_recurrence(const b200_gated_recurrence_args* p, void* stream) {
    if (!p || !p->pre || !p->state || !p->out || !p->ent_row || !p->ent_len || !p->slot || !p->pos || p->n_entries < 0 || p->n_tokens < 0 ||
        p->channels < 1 || p->z_off < 0 || p->u_off < 0 || p->g_off < 0)
        return B200_EINVAL;
    if (p->out_dtype != B200_BF16 && p->out_dtype != B200_F32) return B200_EINVAL;
    if (p->n_tokens == 0 || p->n_entries == 0) return B200_OK;
    if (p->n_entries > 65535) return B200_EUNSUPPORTED;
    const int longest = p->longest_entry > 0 ? p->longest_entry : p->n_tokens;
    const int chunks = (longest + kGrChunk - 1) / kGrChunk;
    GR a{p->pre, p->ld_pre, p->z_off, p->u_off, p->g_off, p->z_bias, p->u_bias, p->state, p->out, p->ent_row, p->ent_len, p->slot, p->pos,
         p->channels, chunks, nullptr, nullptr, nullptr};
    cudaStream_t s = (cudaStream_t)stream;
    const unsigned cb = (unsigned)((p->channels + kGrThreads - 1) / kGrThreads);
    const bool bf = p->out_dtype == B200_BF16;
    if (chunks <= 1) {
        const dim3 grid(cb, p->n_entries, 1);
        if (bf) gr_direct_kernel<__nv_bfloat16, false><<<grid, kGrThreads, 0, s>>>(a);
        else gr_direct_kernel<float, false><<<grid, kGrThreads, 0, s>>>(a);
        count_launch();
        return (int)cudaGetLastError();
    }
    if (chunks > 65535) return B200_EUNSUPPORTED;
    const size_t table = ((size_t)p->n_tokens / kGrChunk + p->n_entries + 1) * p->channels;
    if (!p->workspace || p->workspace_bytes < 3 * table * sizeof(float)) return B200_EWORKSPACE;
    a.sumA = reinterpret_cast<float*>(p->workspace);
    a.sumB = a.sumA + table;
    a.start = a.sumB + table;
    const dim3 grid(cb, p->n_entries, chunks);
    gr_summary_kernel<<<grid, kGrThreads, 0, s>>>(a);
    gr_carry_kernel<<<dim3(cb, p->n_entries), kGrThreads, 0, s>>>(a);
    if (bf) gr_direct_kernel<__nv_bfloat16, true><<<grid, kGrThreads, 0, s>>>(a);
    else gr_direct_kernel<float, true><<<grid, kGrThreads, 0, s>>>(a);
    count_launch(3);
    return (int)cudaGetLastError();
}
