// Model family "Sakevik": a decoder whose norm sits on every sublayer's OUTPUT, x <- x + N1(mixer(x)), x <- x + N2(ff(x)),
// N y = y / rms(y) * w, so the sublayers read the residual stream itself. The embedding row is scaled and the row of a hashed
// (previous token, token) table is added (the previous token is carried per sequence slot). Three kinds of mixer that
// config.json orders freely:
//   "mingru"            an element-wise gated recurrence: gate z = sigmoid(W_z x + b), candidate from u = W_x x + b, one fp32
//                       state per channel carried per sequence; the state times silu(W_g x) goes through W_o.
//   "attention"         grouped heads with biases on q, k, v and the output projection; q and k take a per-head RMS norm
//                       (one weight shared by the heads) and rotate-half rotary positions on their first rot.dims
//                       dimensions; every VALUE is rotated by its own position over all vdim dimensions before it is
//                       cached, and a head's output is turned back by the query's position; a sliding window; the weight
//                       of a visible key is sigmoid(score + a number per head), not normalised over the keys; one sigmoid
//                       output gate per head.
//   "latent_attention"  the cache holds one normed latent row per token plus one rotated key part shared by all heads;
//                       keys and values are up-projections of the latent, so the key up-projection is folded into the
//                       query and the value up-projection follows the weighted sum; interleaved rotary pairs with the
//                       ramped frequency interpolation and its amplitude factor; a sliding window; softmax.
// Feed-forward: none, or the clamped gated unit g * sigmoid(1.702 g) * (u + 1) with g = min(gate, limit), u = clamp(up,
// +-limit). The logits are scaled by a constant.
//
// A step runs on the family-independent pieces of the library: StepRunner (stream, workspaces, graph replay of single-token
// steps, results to the host), SequenceBatch / PagePool for slots, pages and the per-token tables (among them the previous
// token), SlotState for the recurrent state, b200_embed_pair_hash, b200_linear_ex2 (tcgen05) and b200_gemm_grouped,
// b200_rope_angles_amp, b200_qk_prepare (biases, head norms, rotations of q, k and v, page stores), b200_paged_attention
// (window, sigmoid weights), b200_unrotate_gate, b200_latent_store_rot / b200_rotate_part / b200_latent_attention_ex,
// b200_gated_recurrence, b200_rmsnorm_residual in its output-norm form. The residual stream, all norms, rotary angles, scores
// and weights, gates, and the recurrence with everything that enters it after the projections are fp32 in both serving
// dtypes; in B200_BF16 the GEMM operands and the cache pages are bfloat16.
//
// Launch order of a layer (T tokens of all entries packed; h = x in the serving dtype):
//   mingru:  [z | u | g] = h W^T (one GEMM, fp32 out) -> recurrence (biases, gate, candidate, state, silu(g)) -> W_o
//   attention: [q | k | v | gate] = h W^T -> biases, head norms, rotations, page stores -> windowed sigmoid attention (fp32
//              out) -> turn back + head gates -> W_o (its bias joins in the norm kernel)
//   latent:  [q | latent | key part] = h W^T -> normed latent + rotated key part to the pages; per head q W_uk beside the
//            rotated query part -> windowed attention over the rows -> per head W_uv -> W_o
//   x += N1(y) with h = x out of the same kernel -> [gate ; up] GEMM with the clamped unit (fused epilogue, or split-K GEMM +
//   activation kernel for few rows) -> W_down -> x += N2(y), h = x.
#include <cuda_bf16.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "checkpoint_upload.h"
#include "common.cuh"
#include "launch_count.h"
#include "model_registry.h"
#include "safetensors.h"

namespace b200 {
namespace {

constexpr int kPageRows = 64;
constexpr int kStreamRows = 256;   // up to here b200_linear_ex2 streams weights through its M axis (split-K)
constexpr double kPi = 3.14159265358979323846;

struct SkFreq {
    std::vector<double> f;
    double amp = 1.0;
    double* dev = nullptr;
};
enum { kMixGru = 0, kMixAttn = 1, kMixLatent = 2 };

struct SkLayer {
    int kind = kMixGru;
    // mingru
    int channels = 0;
    float *z_b = nullptr, *u_b = nullptr;
    // attention / latent attention
    int heads = 0, kv_heads = 0, dim = 0, vdim = 0, rot_dims = 0, window = 0, table = -1, v_table = -1;
    int rank = 0, rot_dim = 0;                       // latent: cached latent width, rotated key part
    float scale = 1.f;
    float *q_norm = nullptr, *k_norm = nullptr, *head_bias = nullptr, *in_bias = nullptr, *o_bias = nullptr, *dkv_norm = nullptr;
    void *uk = nullptr, *uv = nullptr;
    // both
    int n_in = 0, n_mid = 0;                         // columns of the stacked input projection; inputs of W_o
    void *w_in = nullptr, *w_o = nullptr;
    float *n1 = nullptr, *n2 = nullptr;
    // feed-forward
    int ff = 0;
    float limit = 0.f;
    void *w_gu = nullptr, *w_down = nullptr;
    // cache and state
    void *k_pool = nullptr, *v_pool = nullptr;       // latent: k_pool holds the rows [latent | key part]
    SlotState state;
};

class Sakevik : public StepRunner {
public:
    ~Sakevik() override {
        if (stream_) cudaStreamSynchronize(stream_);
        cudaFree(scratch_);
    }
    const char* family() const override { return "Sakevik"; }
    int layer_count() const override { return (int)layers_.size(); }
    int load(const ModelDir& dir, const b200_model_options& opt, std::string& err);

private:
    int freq_table(SkFreq& fs, std::string& err);
    int ensure_scratch(int T, int W) override;
    int enqueue(int T, int W, int longest_entry, int longest_context, bool want_ids, std::string& err) override;
    size_t step_workspace_bytes(int T, int n_entries) const override {
        size_t need = 0;
        for (const SkLayer& L : layers_) {
            if (L.kind == kMixGru) need = std::max(need, b200_gated_recurrence_workspace_bytes(T, n_entries, L.channels));
            else if (L.kind == kMixAttn) need = std::max(need, b200_paged_attention_workspace_bytes(T, L.heads, L.vdim));
            else if ((long long)T * L.heads <= 8192)   // only batches of few rows split their contexts
                need = std::max(need, b200_latent_attention_workspace_bytes(T, L.heads, L.rank + L.rot_dim));
        }
        return need;
    }

    float eps_ = 1e-6f, embed_scale_ = 1.f, logit_scale_ = 1.f;
    int buckets_ = 0, mul_prev_ = 0, mul_cur_ = 0;
    std::vector<SkLayer> layers_;
    std::vector<SkFreq> freqs_;
    void *embed_ = nullptr, *pair_ = nullptr, *head_ = nullptr;
    float* fnw_ = nullptr;
    // scratch, grown to the largest step seen
    char* scratch_ = nullptr;
    int cap_T_ = 0, cap_W_ = 0;
    float *x_ = nullptr, *proj_ = nullptr, *y_ = nullptr, *attf_ = nullptr, *qa_ = nullptr, *oa_ = nullptr, *gu_ = nullptr, *cs_ = nullptr;
    void *h_ = nullptr, *q_ = nullptr, *mid_ = nullptr, *act_ = nullptr, *hf_ = nullptr;
    int max_in_ = 0, max_q_ = 0, max_attf_ = 0, max_mid_ = 0, max_qa_ = 0, max_ff_ = 0, freq_floats_ = 0;
    std::vector<int> freq_off_;
};

#define SK_TRY(call)                    \
    do {                                \
        const int rc_ = (call);         \
        if (rc_ != B200_OK) return rc_; \
    } while (0)

// equal (frequencies, amplitude) share one cos / sin table per step; returns the table's index in fs.dev's place
int Sakevik::freq_table(SkFreq& fs, std::string& err) {
    for (size_t k = 0; k < freqs_.size(); ++k)
        if (freqs_[k].f == fs.f && freqs_[k].amp == fs.amp) return (int)k;
    fs.dev = (double*)dalloc(std::max<size_t>(1, fs.f.size()) * sizeof(double));
    if (!fs.dev || cudaMemcpy(fs.dev, fs.f.data(), fs.f.size() * sizeof(double), cudaMemcpyHostToDevice) != cudaSuccess) { err = "out of device memory"; return -1; }
    freqs_.push_back(fs);
    return (int)freqs_.size() - 1;
}

// f_i = base^(-2i/span) for the first n pairs
static SkFreq plain_freqs(double base, int span, int n) {
    SkFreq fs;
    fs.f.resize(n);
    for (int i = 0; i < n; ++i) fs.f[i] = std::pow(base, -2.0 * i / span);
    return fs;
}

int Sakevik::load(const ModelDir& dir, const b200_model_options& opt, std::string& err) {
    const Json& c = dir.config;
    dtype_ = opt.dtype;
    if (dtype_ != B200_BF16 && dtype_ != B200_F32) { err = "dtype must be bfloat16 or float32"; return B200_EINVAL; }
    vocab_ = (int)c.integer("vocab", 0);
    D_ = (int)c.integer("width", 0);
    const Json* norm = c.get("norm");
    const Json* ls = c.get("layers");
    const Json* em = c.get("embedding");
    if (vocab_ < 1 || D_ < 1 || !norm || !norm->has("eps") || !ls || ls->kind != Json::Arr || ls->arr.empty()) {
        err = "config.json: vocab, width, norm.eps and layers are required";
        return B200_EINVAL;
    }
    eps_ = (float)norm->number("eps", 1e-6);
    logit_scale_ = (float)c.number("logit_scale", 1.0);
    const Json* bg = nullptr;
    if (em && !em->is_null()) {
        embed_scale_ = (float)em->number("scale", 1.0);
        bg = em->get("bigram");
        if (bg && bg->is_null()) bg = nullptr;
    }
    if (bg) {
        buckets_ = (int)bg->integer("buckets", 0);
        mul_prev_ = (int)bg->integer("mul_prev", 0);
        mul_cur_ = (int)bg->integer("mul_cur", 0);
        if (buckets_ < 1) { err = "embedding.bigram.buckets must be positive"; return B200_EINVAL; }
    }
    if (opt.max_tokens < 1 || opt.max_slots < 1) { err = "max_tokens and max_slots must be positive"; return B200_EINVAL; }
    // everything that can be refused from the configuration alone is refused before the first CUDA call
    const int n = (int)ls->arr.size();
    layers_.resize(n);
    for (int i = 0; i < n; ++i) {
        const Json& lj = ls->arr[i];
        SkLayer& L = layers_[i];
        const std::string type = lj.text("type"), where = "layer " + std::to_string(i) + ": ";
        const Json* mx = lj.get("mixer");
        if (!mx || mx->is_null()) { err = where + "no mixer"; return B200_EINVAL; }
        if (type == "mingru") {
            L.kind = kMixGru;
            L.channels = (int)mx->integer("width", 0);
            if (L.channels < 1) { err = where + "mingru needs width"; return B200_EINVAL; }
            L.n_in = 3 * L.channels;
            L.n_mid = L.channels;
        } else if (type == "attention" || type == "latent_attention") {
            const bool latent = type == "latent_attention";
            L.kind = latent ? kMixLatent : kMixAttn;
            L.heads = (int)mx->integer("heads", 0);
            L.dim = (int)mx->integer("dim", 0);
            L.vdim = (int)mx->integer("vdim", 0);
            if (L.heads < 1 || L.dim < 1 || L.vdim < 1 || !mx->has("scale")) { err = where + "attention needs heads, dim, vdim and scale"; return B200_EINVAL; }
            L.scale = (float)mx->number("scale", 1.0);
            const Json* mk = mx->get("mask");
            L.window = (mk && !mk->is_null()) ? (int)mk->integer("size", 0) : 0;
            if (L.window < 0) { err = where + "mask.size must be positive"; return B200_EINVAL; }
            const Json* r = mx->get("rot");
            const bool has_rot = r && !r->is_null();
            if (latent) {
                L.kv_heads = L.heads;
                L.rank = (int)mx->integer("kv_rank", 0);
                L.rot_dim = (int)mx->integer("rot_dim", 0);
                if (L.rank < 1 || L.rot_dim < 0 || (L.rot_dim & 1)) { err = where + "latent attention needs kv_rank and an even rot_dim"; return B200_EINVAL; }
                if (L.rot_dim > 0 && (!has_rot || (int)r->integer("dims", L.rot_dim) != L.rot_dim || !(r->number("base", 0.0) > 1.0))) {
                    err = where + "rot: dims must equal rot_dim, base above 1";
                    return B200_EINVAL;
                }
                if (L.rank + L.rot_dim > 640) { err = where + "cached rows wider than 640 are not supported by the latent attention kernels"; return B200_EUNSUPPORTED; }
                L.rot_dims = L.rot_dim;
                L.n_in = L.heads * (L.dim + L.rot_dim) + L.rank + L.rot_dim;
            } else {
                L.kv_heads = (int)mx->integer("kv_heads", L.heads);
                if (L.kv_heads < 1 || L.heads % L.kv_heads) { err = where + "heads must be a multiple of kv_heads"; return B200_EINVAL; }
                if (L.vdim > 256) { err = where + "vdim above 256 is not supported by the attention kernels"; return B200_EUNSUPPORTED; }
                L.rot_dims = has_rot ? (int)r->integer("dims", 0) : 0;
                if (L.rot_dims < 0 || (L.rot_dims & 1) || L.rot_dims > L.dim || (has_rot && !(r->number("base", 0.0) > 1.0))) {
                    err = where + "rot: dims must be even and at most dim, base above 1";
                    return B200_EINVAL;
                }
                L.n_in = L.heads * L.dim + L.kv_heads * L.dim + L.kv_heads * L.vdim + L.heads;
            }
            L.n_mid = L.heads * L.vdim;
        } else {
            err = where + "mixer type '" + type + "' is not part of this family";
            return B200_EUNSUPPORTED;
        }
        const Json* ml = lj.get("mlp");
        if (ml && !ml->is_null()) {
            if (ml->text("kind") != "dense") { err = where + "feed-forward kind '" + ml->text("kind") + "' is not part of this family"; return B200_EUNSUPPORTED; }
            L.ff = (int)ml->integer("ff", 0);
            L.limit = (float)ml->number("limit", 0.0);
            if (L.ff < 1 || !(L.limit > 0.f)) { err = where + "mlp needs ff and a positive limit"; return B200_EINVAL; }
        }
    }

    SK_TRY(init_runner(err));
    SafeTensorsFile st;
    if (!st.open(dir.path + "/model.safetensors", err)) return B200_EINVAL;
    // the design has no position limit of its own: a sequence can grow as long as the pool has pages
    const int n_pages = (opt.max_tokens + kPageRows - 1) / kPageRows;
    SK_TRY(seq_.init(opt.max_tokens, kPageRows, opt.max_slots, n_pages * kPageRows, err));

    const size_t E = esz();
    const long long D = D_;
    auto f32 = [&](const std::string& name, std::vector<long long> shape, float*& dst) -> int {
        size_t cnt = 1;
        for (long long d : shape) cnt *= (size_t)d;
        dst = (float*)dalloc(cnt * 4);
        if (!dst) { err = "out of device memory"; return B200_ENOMEM; }
        return upload_tensor(st, name, shape, true, dtype_, dst, err);
    };
    auto mat = [&](const std::string& name, long long rows, long long cols, void*& dst) -> int {
        dst = dalloc((size_t)rows * cols * E);
        if (!dst) { err = "out of device memory"; return B200_ENOMEM; }
        return upload_tensor(st, name, {rows, cols}, false, dtype_, dst, err);
    };
    // several checkpoint matrices that read the same input, stacked row-wise into one operand
    auto stacked = [&](const std::vector<std::pair<std::string, long long>>& parts, long long cols, void*& dst) -> int {
        long long rows = 0;
        for (auto& p : parts) rows += p.second;
        dst = dalloc((size_t)rows * cols * E);
        if (!dst) { err = "out of device memory"; return B200_ENOMEM; }
        long long at = 0;
        for (auto& p : parts) {
            SK_TRY(upload_tensor(st, p.first, {p.second, cols}, false, dtype_, (char*)dst + (size_t)at * cols * E, err));
            at += p.second;
        }
        return B200_OK;
    };
    // the biases of the stacked projection, fp32, zeros where a part has none
    auto stacked_bias = [&](const std::vector<std::pair<std::string, long long>>& parts, float*& dst) -> int {
        long long rows = 0;
        for (auto& p : parts) rows += p.second;
        std::vector<float> host((size_t)rows, 0.f);
        long long at = 0;
        for (auto& p : parts) {
            if (!p.first.empty()) {
                const SafeTensor* t = st.find(p.first);
                if (!t) { err = "tensor " + p.first + " is missing"; return B200_EINVAL; }
                if ((long long)t->elems() != p.second || (t->dtype != "BF16" && t->dtype != "F32")) { err = "tensor " + p.first + " does not have " + std::to_string(p.second) + " floating-point values"; return B200_EINVAL; }
                for (long long k = 0; k < p.second; ++k) host[(size_t)(at + k)] = st_value(*t, (size_t)k);
            }
            at += p.second;
        }
        dst = (float*)dalloc((size_t)rows * 4);
        if (!dst || cudaMemcpy(dst, host.data(), (size_t)rows * 4, cudaMemcpyHostToDevice) != cudaSuccess) { err = "out of device memory"; return B200_ENOMEM; }
        return B200_OK;
    };
    SK_TRY(mat("embed", vocab_, D, embed_));
    if (buckets_ > 0) SK_TRY(mat("bigram", buckets_ + 1ll, D, pair_));
    SK_TRY(mat("head", vocab_, D, head_));
    SK_TRY(f32("final.norm", {D}, fnw_));

    const size_t cache_rows = (size_t)seq_.pool.n_pages() * kPageRows;
    for (int i = 0; i < n; ++i) {
        const Json& lj = ls->arr[i];
        SkLayer& L = layers_[i];
        const std::string pre = "l" + std::to_string(i) + ".", mp = pre + "mix.", where = "layer " + std::to_string(i) + ": ";
        const Json& mx = *lj.get("mixer");
        SK_TRY(f32(pre + "norm1", {D}, L.n1));
        if (L.kind == kMixGru) {
            const long long C = L.channels;
            SK_TRY(stacked({{mp + "z", C}, {mp + "x", C}, {mp + "g", C}}, D, L.w_in));
            SK_TRY(f32(mp + "z.b", {C}, L.z_b));
            SK_TRY(f32(mp + "x.b", {C}, L.u_b));
            SK_TRY(mat(mp + "o", D, C, L.w_o));
            if (L.state.init(opt.max_slots, (size_t)C) != cudaSuccess) { err = "out of device memory (carried state)"; return B200_ENOMEM; }
        } else if (L.kind == kMixAttn) {
            const long long nq = (long long)L.heads * L.dim, nk = (long long)L.kv_heads * L.dim, nv = (long long)L.kv_heads * L.vdim;
            SK_TRY(stacked({{mp + "q", nq}, {mp + "k", nk}, {mp + "v", nv}, {mp + "g", L.heads}}, D, L.w_in));
            SK_TRY(stacked_bias({{mp + "q.b", nq}, {mp + "k.b", nk}, {mp + "v.b", nv}, {"", L.heads}}, L.in_bias));
            SK_TRY(f32(mp + "q.norm", {L.dim}, L.q_norm));
            SK_TRY(f32(mp + "k.norm", {L.dim}, L.k_norm));
            SK_TRY(f32(mp + "pb", {L.heads}, L.head_bias));
            SK_TRY(mat(mp + "o", D, L.n_mid, L.w_o));
            SK_TRY(f32(mp + "o.b", {D}, L.o_bias));
            const Json* r = mx.get("rot");
            const double base = (r && !r->is_null()) ? r->number("base", 10000.0) : 10000.0;
            if (L.rot_dims > 0) {
                SkFreq fs = plain_freqs(base, L.rot_dims, L.rot_dims / 2);
                if ((L.table = freq_table(fs, err)) < 0) return B200_ENOMEM;
            }
            {   // the values turn over all vdim dimensions, pair m by base^(-2m/vdim), whatever the keys do
                SkFreq fs = plain_freqs(base, L.vdim, L.vdim / 2);
                if ((L.v_table = freq_table(fs, err)) < 0) return B200_ENOMEM;
            }
            const size_t kb = cache_rows * nk * E, vb = cache_rows * nv * E;
            L.k_pool = dalloc(kb);
            L.v_pool = dalloc(vb);
            if (!L.k_pool || !L.v_pool) { err = "out of device memory (K / V pages)"; return B200_ENOMEM; }
            cudaMemset(L.k_pool, 0, kb);
            cudaMemset(L.v_pool, 0, vb);
            max_q_ = std::max(max_q_, (int)nq);
            max_attf_ = std::max(max_attf_, L.n_mid);
        } else {
            const long long nq = (long long)L.heads * (L.dim + L.rot_dim);
            SK_TRY(stacked({{mp + "q", nq}, {mp + "dkv", (long long)L.rank + L.rot_dim}}, D, L.w_in));
            SK_TRY(f32(mp + "dkv.norm", {L.rank}, L.dkv_norm));
            SK_TRY(mat(mp + "uk", (long long)L.heads * L.dim, L.rank, L.uk));
            SK_TRY(mat(mp + "uv", (long long)L.heads * L.vdim, L.rank, L.uv));
            SK_TRY(mat(mp + "o", D, L.n_mid, L.w_o));
            if (L.rot_dim > 0) {
                // ramped interpolation: f_i / factor and f_i blended by a ramp over the pair index between the indices whose
                // wavelengths make `fast` and `slow` turns within `original` positions; cos and sin times 0.1 ln(factor) + 1
                const Json* r = mx.get("rot");
                const double base = r->number("base", 10000.0);
                const int d = L.rot_dim;
                SkFreq fs = plain_freqs(base, d, d / 2);
                const Json* sc = r->get("scaling");
                if (sc && !sc->is_null()) {
                    const double factor = sc->number("factor", 1.0), orig = sc->number("original", 0.0), fast = sc->number("fast", 32.0),
                                 slow = sc->number("slow", 1.0);
                    if (!(factor > 0.0) || !(orig > 0.0) || !(fast > 0.0) || !(slow > 0.0)) { err = where + "rot.scaling needs positive factor, original, fast, slow"; return B200_EINVAL; }
                    auto index_of = [&](double turns) { return d * std::log(orig / (2.0 * kPi * turns)) / (2.0 * std::log(base)); };
                    const double lo = std::max(std::floor(index_of(fast)), 0.0), hi = std::min(std::ceil(index_of(slow)), (double)(d - 1));
                    for (int k = 0; k < d / 2; ++k) {
                        const double ramp = std::min(std::max((k - lo) / std::max(hi - lo, 0.001), 0.0), 1.0);
                        fs.f[k] = fs.f[k] / factor * ramp + fs.f[k] * (1.0 - ramp);
                    }
                    fs.amp = 0.1 * std::log(factor) + 1.0;
                }
                if ((L.table = freq_table(fs, err)) < 0) return B200_ENOMEM;
            }
            const size_t pb = cache_rows * (size_t)(L.rank + L.rot_dim) * E;
            L.k_pool = dalloc(pb);
            if (!L.k_pool) { err = "out of device memory (latent pages)"; return B200_ENOMEM; }
            cudaMemset(L.k_pool, 0, pb);
            max_qa_ = std::max(max_qa_, L.heads * (L.rank + L.rot_dim));
        }
        max_in_ = std::max(max_in_, L.n_in);
        max_mid_ = std::max(max_mid_, L.n_mid);
        if (L.ff > 0) {
            SK_TRY(f32(pre + "norm2", {D}, L.n2));
            SK_TRY(stacked({{pre + "mlp.gate", L.ff}, {pre + "mlp.up", L.ff}}, D, L.w_gu));
            SK_TRY(mat(pre + "mlp.down", D, L.ff, L.w_down));
            max_ff_ = std::max(max_ff_, L.ff);
        }
    }
    freq_off_.assign(freqs_.size(), 0);
    for (size_t k = 0; k < freqs_.size(); ++k) {
        freq_off_[k] = freq_floats_;
        freq_floats_ += 2 * (int)freqs_[k].f.size();   // cos and sin per token
    }
    if (cudaDeviceSynchronize() != cudaSuccess) { err = "weight upload failed"; return B200_EINVAL; }
    return B200_OK;
}

int Sakevik::ensure_scratch(int T, int W) {
    if (T <= cap_T_ && W <= cap_W_) return B200_OK;
    const int cT = std::max(T, cap_T_), cW = std::max(W, cap_W_);
    cudaStreamSynchronize(stream_);
    buffers_moved();
    cudaFree(scratch_);
    scratch_ = nullptr;
    cap_T_ = cap_W_ = 0;
    auto al = [](size_t b) { return (b + 255) & ~(size_t)255; };
    const size_t E = esz(), t = (size_t)cT;
    const size_t sizes[] = {
        al(t * D_ * 4),                                                    // x
        al(t * max_in_ * 4),                                               // proj
        al(t * D_ * 4),                                                    // y
        al(t * std::max(1, max_attf_) * 4),                                // attf
        al(t * std::max(1, max_qa_) * 4),                                  // qa
        al(t * std::max(1, max_qa_) * 4),                                  // oa
        al((size_t)std::min(cT, kStreamRows) * 2 * std::max(1, max_ff_) * 4),   // gu
        al((size_t)cW * vocab_ * 4),                                       // logits
        al(t * std::max(1, freq_floats_) * 4),                             // cos / sin tables
        al(t * D_ * E),                                                    // h
        al(t * std::max(1, max_q_) * E),                                   // q
        al(t * max_mid_ * E),                                              // mid
        al(t * std::max(1, max_ff_) * E),                                  // act
        al((size_t)cW * D_ * E),                                           // hf
        al((size_t)cW * 4),                                                // ids
    };
    size_t total = 0;
    for (size_t s : sizes) total += s;
    if (cudaMalloc(&scratch_, total) != cudaSuccess) return B200_ENOMEM;
    char* p = scratch_;
    int k = 0;
    auto take = [&](auto*& dst) { dst = reinterpret_cast<std::remove_reference_t<decltype(dst)>>(p); p += sizes[k++]; };
    take(x_); take(proj_); take(y_); take(attf_); take(qa_); take(oa_); take(gu_); take(logits_); take(cs_);
    take(h_); take(q_); take(mid_); take(act_); take(hf_); take(ids_dev_);
    cap_T_ = cT;
    cap_W_ = cW;
    return ensure_logits_host(cW);
}

// every launch of a step, in order, on stream_ (no synchronisation, no allocation: capturable into a graph)
int Sakevik::enqueue(int T, int W, int longest_entry, int longest_context, bool want_ids, std::string& err) {
    const int D = D_, dt = dtype_;
    const int* pages = seq_.pool.device();
    const int max_pages = seq_.pool.max_pages();
#define SK_OP(call)                                                             \
    do {                                                                        \
        const int rc_ = (call);                                                 \
        if (rc_ != B200_OK) { err = std::string(#call) + " failed (" + std::to_string(rc_) + ")"; return rc_; } \
    } while (0)
    // cos / sin of this step's positions, one table per frequency set: [T, n_freq] cos, then [T, n_freq] sin
    auto cos_of = [&](int table) { return cs_ + (size_t)T * freq_off_[table]; };
    auto sin_of = [&](int table) { return cs_ + (size_t)T * freq_off_[table] + (size_t)T * freqs_[table].f.size(); };
    for (size_t k = 0; k < freqs_.size(); ++k)
        if (!freqs_[k].f.empty())
            SK_OP(b200_rope_angles_amp(seq_.d_pos(), T, freqs_[k].dev, (int)freqs_[k].f.size(), freqs_[k].amp, cos_of((int)k), sin_of((int)k), stream_));
    SK_OP(b200_embed_pair_hash(seq_.d_ids(), seq_.d_prev(), embed_, embed_scale_, pair_, buckets_, mul_prev_, mul_cur_, x_, h_, T, D, dt, stream_));
    // x += N(y + bias); h = x in the serving dtype
    auto add_normed = [&](const float* nw, const float* y_bias) -> int {
        b200_rmsnorm_residual_args ra{};
        ra.x = x_; ra.y1 = y_; ra.y_bias = y_bias; ra.norm_addend = 1;
        ra.w = nw; ra.w_offset = 0.f; ra.eps = eps_; ra.out = h_; ra.out_dtype = dt;
        ra.n_rows = T; ra.width = D;
        return b200_rmsnorm_residual(&ra, stream_);
    };
    for (size_t li = 0; li < layers_.size(); ++li) {
        SkLayer& L = layers_[li];
        SK_OP(gemm(h_, L.w_in, proj_, B200_F32, T, L.n_in, D));
        if (L.kind == kMixGru) {
            b200_gated_recurrence_args ga{};
            ga.pre = proj_; ga.ld_pre = L.n_in; ga.z_off = 0; ga.u_off = L.channels; ga.g_off = 2 * L.channels;
            ga.z_bias = L.z_b; ga.u_bias = L.u_b;
            ga.state = L.state.data(); ga.out = mid_; ga.out_dtype = dt;
            ga.ent_row = seq_.d_ent_row(); ga.ent_len = seq_.d_ent_len(); ga.slot = seq_.d_slot(); ga.pos = seq_.d_pos();
            ga.n_entries = seq_.n_entries; ga.n_tokens = T; ga.channels = L.channels; ga.longest_entry = longest_entry;
            ga.workspace = attn_ws_; ga.workspace_bytes = attn_ws_bytes_;
            SK_OP(b200_gated_recurrence(&ga, stream_));
        } else if (L.kind == kMixAttn) {
            const int nq = L.heads * L.dim, nk = L.kv_heads * L.dim, nv = L.kv_heads * L.vdim;
            b200_qk_prepare_args qa{};
            qa.proj = proj_; qa.ld_proj = L.n_in; qa.bias = L.in_bias;
            qa.q_norm = L.q_norm; qa.k_norm = L.k_norm; qa.eps = eps_;
            if (L.rot_dims > 0) { qa.cos = cos_of(L.table); qa.sin = sin_of(L.table); }
            qa.rot_dims = L.rot_dims; qa.rot_layout = B200_ROPE_HALF;
            qa.q_out = q_; qa.k_pool = L.k_pool; qa.v_pool = L.v_pool;
            qa.pages = pages; qa.max_pages = max_pages; qa.page_rows = kPageRows;
            qa.slot = seq_.d_slot(); qa.pos = seq_.d_pos(); qa.start = seq_.d_start();
            qa.n_tokens = T; qa.heads = L.heads; qa.kv_heads = L.kv_heads; qa.dim = L.dim; qa.dtype = dt;
            qa.v_heads = L.kv_heads; qa.vdim = L.vdim; qa.v_off = nq + nk;
            if (L.vdim >= 2) { qa.v_cos = cos_of(L.v_table); qa.v_sin = sin_of(L.v_table); qa.v_rot_layout = B200_ROPE_HALF; }
            SK_OP(b200_qk_prepare(&qa, stream_));
            b200_paged_attention_args pa{};
            pa.q = q_; pa.out = attf_; pa.k_pool = L.k_pool; pa.v_pool = L.v_pool;
            pa.pages = pages; pa.max_pages = max_pages; pa.page_rows = kPageRows;
            pa.slot = seq_.d_slot(); pa.pos = seq_.d_pos();
            pa.n_tokens = T; pa.heads = L.heads; pa.kv_heads = L.kv_heads; pa.dim = L.dim; pa.vdim = L.vdim;
            pa.scale = L.scale; pa.dtype = dt; pa.longest_entry = longest_entry; pa.longest_context = longest_context;
            pa.workspace = attn_ws_; pa.workspace_bytes = attn_ws_bytes_;
            pa.out_f32 = 1; pa.window = L.window; pa.sigmoid_weights = 1; pa.head_bias = L.head_bias;
            SK_OP(b200_paged_attention(&pa, stream_));
            if (L.vdim >= 2)
                SK_OP(b200_unrotate_gate(attf_, cos_of(L.v_table), sin_of(L.v_table), B200_ROPE_HALF, proj_ + nq + nk + nv, L.n_in, mid_, T, L.heads,
                                         L.vdim, dt, stream_));
            else   // a one-dimensional value has no pair to turn: the gate alone
                SK_OP(b200_sigmoid_gate(attf_, proj_ + nq + nk + nv, L.n_in, mid_, T, L.heads, dt, stream_));
        } else {
            const int H = L.heads, R = L.rank, dr = L.rot_dim, row = R + dr, nq = H * (L.dim + dr);
            const float* cs = dr > 0 ? cos_of(L.table) : nullptr;
            const float* sn = dr > 0 ? sin_of(L.table) : nullptr;
            SK_OP(b200_latent_store_rot(proj_ + nq, L.n_in, L.dkv_norm, eps_, L.k_pool, pages, max_pages, kPageRows, seq_.d_slot(), seq_.d_pos(), T, R,
                                        dr, cs, sn, B200_ROPE_INTERLEAVED, dt, stream_));
            {   // qa[t, h, 0:R] = sum_d q[t, h, d] W_uk[h*dim + d, :]
                b200_gemm_grouped_args g{};
                g.A = proj_; g.lda = L.n_in; g.stride_a = L.dim + dr;
                g.W = L.uk; g.ldw = R; g.stride_w = (long long)L.dim * R; g.trans_b = 0;
                g.C = qa_; g.ldc = (long long)H * row; g.stride_c = row;
                g.M = T; g.N = R; g.K = L.dim; g.batch = H;
                g.a_dtype = B200_F32; g.w_dtype = dt; g.c_dtype = B200_F32;
                SK_OP(b200_gemm_grouped(&g, stream_));
            }
            if (dr > 0)   // qa[t, h, R:R+dr] = the head's rotated query part
                SK_OP(b200_rotate_part(proj_, L.n_in, L.dim, L.dim + dr, qa_, (long long)H * row, R, row, cs, sn, B200_ROPE_INTERLEAVED, T, H, dr, stream_));
            b200_latent_attention_args la{};
            la.qa = qa_; la.out = oa_; la.pool = L.k_pool; la.pages = pages; la.max_pages = max_pages; la.page_rows = kPageRows;
            la.slot = seq_.d_slot(); la.pos = seq_.d_pos(); la.sink = nullptr; la.scale = L.scale;
            la.n_tokens = T; la.heads = H; la.rank = row; la.window = L.window; la.dtype = dt;
            la.longest_entry = longest_entry; la.longest_context = longest_context;
            la.workspace = attn_ws_; la.workspace_bytes = attn_ws_bytes_;
            la.out_cols = R;   // the value up-projection reads the latent columns only
            SK_OP(b200_latent_attention_ex(&la, stream_));
            {   // mid[t, h, :] = W_uv,h oa[t, h, 0:R]
                b200_gemm_grouped_args g{};
                g.A = oa_; g.lda = (long long)H * row; g.stride_a = row;
                g.W = L.uv; g.ldw = R; g.stride_w = (long long)L.vdim * R; g.trans_b = 1;
                g.C = mid_; g.ldc = L.n_mid; g.stride_c = L.vdim;
                g.M = T; g.N = L.vdim; g.K = R; g.batch = H;
                g.a_dtype = B200_F32; g.w_dtype = dt; g.c_dtype = dt;
                SK_OP(b200_gemm_grouped(&g, stream_));
            }
        }
        SK_OP(gemm(mid_, L.w_o, y_, B200_F32, T, D, L.n_mid));
        SK_OP(add_normed(L.n1, L.o_bias));
        if (L.ff > 0) {
            if (dt == B200_BF16 && T <= kStreamRows) {   // few rows: the stacked [gate; up] streams once through the split-K GEMM
                SK_OP(gemm(h_, L.w_gu, gu_, B200_F32, T, 2 * L.ff, D));
                SK_OP(b200_glu_act_clamped(gu_, act_, T, L.ff, L.limit, dt, stream_));
            } else
                SK_OP(gemm(h_, L.w_gu, act_, dt, T, L.ff, D, B200_GG_GLU_CLAMP, L.limit));
            SK_OP(gemm(act_, L.w_down, y_, B200_F32, T, D, L.ff));
            SK_OP(add_normed(L.n2, nullptr));
        }
        keep_layer(li, x_, T);
    }
    if (W > 0) {
        b200_rmsnorm_residual_args fa{};
        fa.x = x_; fa.rows = seq_.d_want_rows(); fa.w = fnw_; fa.w_offset = 0.f; fa.eps = eps_; fa.out = hf_; fa.out_dtype = dt;
        fa.n_rows = W; fa.width = D;
        SK_OP(b200_rmsnorm_residual(&fa, stream_));
        SK_OP(gemm(hf_, head_, logits_, B200_F32, W, vocab_, D));
        if (logit_scale_ != 1.f) SK_OP(b200_scale(logits_, (size_t)W * vocab_, logit_scale_, stream_));
        if (want_ids) SK_OP(b200_argmax(logits_, ids_dev_, W, vocab_, B200_F32, stream_));
    }
    return B200_OK;
#undef SK_OP
}

Model* make_sakevik(const ModelDir& dir, const b200_model_options& opt, std::string& err) {
    Sakevik* m = new Sakevik();
    if (m->load(dir, opt, err) != B200_OK) {
        delete m;
        return nullptr;
    }
    return m;
}

FamilyRegistrar reg_sakevik("Sakevik", make_sakevik);

}  // namespace
}  // namespace b200
