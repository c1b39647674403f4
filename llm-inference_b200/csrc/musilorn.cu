// Model family "Musilorn": a decoder of sandwich-normed layers, x <- x + m * LN_b(sub(LN_a(x))) for a mixer and an
// optional dense GLU feed-forward (tanh-gelu), with two kinds of mixer that config.json orders freely:
//   "attention"  grouped query heads; a short causal convolution over time on the projected q and k; per-head RMS norm
//                with a weight shared by the heads; interleaved rotary positions with long-context frequency scaling;
//                the values ARE the convolved keys (no value projection); tanh-capped scores; softmax with one added
//                to its denominator; paged K / V cache.
//   "retention"  a fixed decay per head, rotate-half rotary positions, a carried state S <- decay S + k v^T per
//                sequence slot, unit-RMS outputs times a silu gate.
// A span of layers ("loop") runs several times with the same weights; every pass starts with x <- W_in [x; embedding],
// and every layer RUN (not every layer) owns its cache pages or state. The logits are tanh-capped.
//
// A step runs on the family-independent pieces of the library: StepRunner (stream, workspaces, graph replay of single-token
// steps, results to the host), SequenceBatch / PagePool for slots, pages and the per-token tables, SlotState for what is
// carried per slot, b200_layernorm_pair / b200_layernorm_residual,
// b200_linear_ex (tcgen05) and b200_gemm_grouped, b200_rope_angles, b200_qk_prepare, b200_paged_attention,
// b200_retention. The residual stream, all norms, the softmax, the recurrence and everything entering it are fp32 in
// both serving dtypes; in B200_BF16 the GEMM operands and the caches are bfloat16.
//
// Launch order of a layer run (T tokens of all entries packed):
//   [pass start: concat -> W_in GEMM -> LN]  ->  [q | k] or [q | k | v | g] = h W^T (one GEMM, fp32 out)
//   attention: qk_prepare (conv, norm, rotation, page stores) -> conv ring update -> paged attention -> W_o
//   retention: state walk -> unit RMS * silu(gate) -> W_o
//   x += m LN(y) fused with the next sublayer's input norm -> GLU GEMM (gelu epilogue) -> down GEMM -> the same again.
#include <cuda_bf16.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>

#include "checkpoint_upload.h"
#include "common.cuh"
#include "launch_count.h"
#include "model_registry.h"
#include "safetensors.h"

namespace b200 {
namespace {

constexpr int kPageRows = 64;
constexpr int kStreamRows = 256;   // up to here b200_linear_ex streams weights through its M axis (split-K)
constexpr double kPi = 3.14159265358979323846;

struct MuRot {
    int dims = 0, layout = B200_ROPE_HALF, table = -1;   // table: index of the step's cos / sin table
};
struct FreqSet {
    std::vector<double> f;
    double* dev = nullptr;
};

struct MuLayer {
    bool attention = true, has_mlp = false;
    int heads = 0, kv_heads = 0, dim = 0, vdim = 0, taps = 0, ff = 0;
    float scale = 1.f, softcap = 0.f;
    MuRot rot;
    int n_in = 0;   // rows of w_in
    float *n1w = nullptr, *n1b = nullptr, *n1bw = nullptr, *n1bb = nullptr, *n2w = nullptr, *n2b = nullptr, *n2bw = nullptr, *n2bb = nullptr;
    float *conv_w = nullptr, *q_norm = nullptr, *k_norm = nullptr, *decay = nullptr;
    void *w_in = nullptr, *o = nullptr, *w_gu = nullptr, *w_down = nullptr;
};

struct MuRun {
    int layer = 0;
    bool pass_start = false;
    void *k_pool = nullptr, *v_pool = nullptr;   // attention
    SlotState state;                             // attention: ring of conv inputs; retention: S
};

class Musilorn : public StepRunner {
public:
    ~Musilorn() override {
        if (stream_) cudaStreamSynchronize(stream_);
        cudaFree(scratch_);
    }
    const char* family() const override { return "Musilorn"; }
    int layer_count() const override { return (int)runs_.size(); }   // layer runs: what a step executes and captures

    int load(const ModelDir& dir, const b200_model_options& opt, std::string& err);

private:
    int parse_rot(const Json& mx, int dim, int layout, MuRot& rot, std::string& err);
    int ensure_scratch(int T, int W) override;
    int enqueue(int T, int W, int longest_entry, int longest_context, bool want_ids, std::string& err) override;
    size_t step_workspace_bytes(int T, int n_entries) const override {
        size_t need = 0;
        for (const MuLayer& L : layers_)
            need = std::max(need, L.attention ? b200_paged_attention_workspace_bytes(T, L.heads, L.vdim)
                                              : b200_retention_workspace_bytes(T, n_entries, L.heads, L.dim, L.vdim));
        return need;
    }

    float eps_ = 1e-5f, mult_ = 1.f, logit_cap_ = 0.f;
    std::vector<MuLayer> layers_;
    std::vector<MuRun> runs_;
    std::vector<FreqSet> freqs_;
    bool has_loop_ = false;
    void *embed_ = nullptr, *head_ = nullptr, *loop_in_ = nullptr;
    float *fnw_ = nullptr, *fnb_ = nullptr;
    // scratch, grown to the largest step seen
    char* scratch_ = nullptr;
    int cap_T_ = 0, cap_W_ = 0;
    float *gu_ = nullptr;   // [gate | up] of small batches before the activation
    float *x_ = nullptr, *x0_ = nullptr, *proj_ = nullptr, *y_ = nullptr, *ret_ = nullptr, *cs_ = nullptr;
    void *h1_ = nullptr, *h2_ = nullptr, *cat_ = nullptr, *q_ = nullptr, *att_ = nullptr, *act_ = nullptr, *hf_ = nullptr;
    int max_in_ = 0, max_q_ = 0, max_att_ = 0, max_ff_ = 0, freq_floats_ = 0;   // maxima over layers (scratch sizes)
    std::vector<int> freq_off_;   // first float of each frequency set's cos table in cs_ (per token: see step)
};

#define MU_TRY(call)                    \
    do {                                \
        const int rc_ = (call);         \
        if (rc_ != B200_OK) return rc_; \
    } while (0)

// Frequencies of a rotary block: f_i = base^(-2i/dims); with "scaling" {factor, low, high, original} wavelengths longer
// than original/low are stretched by factor, those shorter than original/high are kept, and the band between is blended
// linearly in original/wavelength. Equal sets share one cos / sin table per step.
int Musilorn::parse_rot(const Json& mx, int dim, int layout, MuRot& rot, std::string& err) {
    rot.layout = layout;
    const Json* r = mx.get("rot");
    if (!r || r->is_null()) { rot.dims = 0; return B200_OK; }
    rot.dims = (int)r->integer("dims", 0);
    const double base = r->number("base", 0.0);
    if (rot.dims < 0 || (rot.dims & 1) || rot.dims > dim || (rot.dims > 0 && !(base > 0.0))) { err = "rot: dims must be even and at most dim, base positive"; return B200_EINVAL; }
    if (rot.dims == 0) return B200_OK;
    std::vector<double> f(rot.dims / 2);
    for (int i = 0; i < rot.dims / 2; ++i) f[i] = std::pow(base, -2.0 * i / rot.dims);
    const Json* sc = r->get("scaling");
    if (sc && !sc->is_null()) {
        const double factor = sc->number("factor", 1.0), low = sc->number("low", 1.0), high = sc->number("high", 4.0),
                     orig = sc->number("original", 0.0);
        if (!(factor > 0.0) || !(orig > 0.0) || !(high > low)) { err = "rot.scaling needs factor, low < high and original"; return B200_EINVAL; }
        for (double& fi : f) {
            const double wl = 2.0 * kPi / fi;
            if (wl < orig / high) continue;
            if (wl > orig / low) fi = fi / factor;
            else {
                const double s = (orig / wl - low) / (high - low);
                fi = (1.0 - s) * fi / factor + s * fi;
            }
        }
    }
    for (size_t k = 0; k < freqs_.size(); ++k)
        if (freqs_[k].f == f) { rot.table = (int)k; return B200_OK; }
    FreqSet fs;
    fs.f = f;
    fs.dev = (double*)dalloc(f.size() * sizeof(double));
    if (!fs.dev || cudaMemcpy(fs.dev, f.data(), f.size() * sizeof(double), cudaMemcpyHostToDevice) != cudaSuccess) { err = "out of device memory"; return B200_ENOMEM; }
    rot.table = (int)freqs_.size();
    freqs_.push_back(fs);
    return B200_OK;
}

int Musilorn::load(const ModelDir& dir, const b200_model_options& opt, std::string& err) {
    const Json& c = dir.config;
    dtype_ = opt.dtype;
    if (dtype_ != B200_BF16 && dtype_ != B200_F32) { err = "dtype must be bfloat16 or float32"; return B200_EINVAL; }
    vocab_ = (int)c.integer("vocab", 0);
    D_ = (int)c.integer("width", 0);
    const Json* norm = c.get("norm");
    const Json* ls = c.get("layers");
    if (vocab_ < 1 || D_ < 1 || !norm || !norm->has("eps") || !ls || ls->kind != Json::Arr || ls->arr.empty() || !c.has("residual_mult")) {
        err = "config.json: vocab, width, norm.eps, residual_mult and layers are required";
        return B200_EINVAL;
    }
    eps_ = (float)norm->number("eps", 1e-5);
    mult_ = (float)c.number("residual_mult", 1.0);
    logit_cap_ = (float)c.number("logit_softcap", 0.0);
    if (opt.max_tokens < 1 || opt.max_slots < 1) { err = "max_tokens and max_slots must be positive"; return B200_EINVAL; }
    MU_TRY(init_runner(err));
    SafeTensorsFile st;
    if (!st.open(dir.path + "/model.safetensors", err)) return B200_EINVAL;
    // the design has no position limit of its own: a sequence can grow as long as the pool has pages
    const int n_pages = (opt.max_tokens + kPageRows - 1) / kPageRows;
    MU_TRY(seq_.init(opt.max_tokens, kPageRows, opt.max_slots, n_pages * kPageRows, err));

    const size_t E = esz();
    const long long D = D_;
    auto f32 = [&](const std::string& name, std::vector<long long> shape, float*& dst) -> int {
        size_t n = 1;
        for (long long d : shape) n *= (size_t)d;
        dst = (float*)dalloc(n * 4);
        if (!dst) { err = "out of device memory"; return B200_ENOMEM; }
        return upload_tensor(st, name, shape, true, dtype_, dst, err);
    };
    auto mat = [&](const std::string& name, long long rows, long long cols, void*& dst) -> int {
        dst = dalloc((size_t)rows * cols * E);
        if (!dst) { err = "out of device memory"; return B200_ENOMEM; }
        return upload_tensor(st, name, {rows, cols}, false, dtype_, dst, err);
    };
    // several checkpoint matrices that read the same input, stacked row-wise into one GEMM operand
    auto stacked = [&](const std::vector<std::pair<std::string, long long>>& parts, long long cols, void*& dst) -> int {
        long long rows = 0;
        for (auto& p : parts) rows += p.second;
        dst = dalloc((size_t)rows * cols * E);
        if (!dst) { err = "out of device memory"; return B200_ENOMEM; }
        long long at = 0;
        for (auto& p : parts) {
            MU_TRY(upload_tensor(st, p.first, {p.second, cols}, false, dtype_, (char*)dst + (size_t)at * cols * E, err));
            at += p.second;
        }
        return B200_OK;
    };
    MU_TRY(mat("embed", vocab_, D, embed_));
    MU_TRY(mat("head", vocab_, D, head_));
    MU_TRY(f32("final.norm", {D}, fnw_));
    MU_TRY(f32("final.norm.b", {D}, fnb_));

    layers_.resize(ls->arr.size());
    for (size_t i = 0; i < layers_.size(); ++i) {
        const Json& lj = ls->arr[i];
        MuLayer& L = layers_[i];
        const std::string pre = "l" + std::to_string(i) + ".", where = "layer " + std::to_string(i) + ": ";
        const std::string type = lj.text("type");
        const Json* mx = lj.get("mixer");
        if (!mx || mx->is_null()) { err = where + "no mixer"; return B200_EINVAL; }
        L.heads = (int)mx->integer("heads", 0);
        L.dim = (int)mx->integer("dim", 0);
        L.vdim = (int)mx->integer("vdim", 0);
        if (L.heads < 1 || L.dim < 1 || L.vdim < 1) { err = where + "mixer needs heads, dim, vdim"; return B200_EINVAL; }
        MU_TRY(f32(pre + "norm1", {D}, L.n1w));
        MU_TRY(f32(pre + "norm1.b", {D}, L.n1b));
        MU_TRY(f32(pre + "norm1b", {D}, L.n1bw));
        MU_TRY(f32(pre + "norm1b.b", {D}, L.n1bb));
        if (type == "attention") {
            L.attention = true;
            L.kv_heads = (int)mx->integer("kv_heads", L.heads);
            L.taps = (int)mx->integer("conv", 1);
            L.softcap = (float)mx->number("softcap", 0.0);
            if (!mx->has("scale")) { err = where + "attention needs scale"; return B200_EINVAL; }
            L.scale = (float)mx->number("scale", 1.0);
            if (L.kv_heads < 1 || L.heads % L.kv_heads) { err = where + "heads must be a multiple of kv_heads"; return B200_EINVAL; }
            if (L.vdim != L.dim) { err = where + "the values are the convolved keys, so vdim must equal dim"; return B200_EINVAL; }
            if (L.taps < 1) { err = where + "conv must be at least 1"; return B200_EINVAL; }
            if (L.vdim > 256) { err = where + "vdim above 256 is not supported by the attention kernels"; return B200_EUNSUPPORTED; }
            MU_TRY(parse_rot(*mx, L.dim, B200_ROPE_INTERLEAVED, L.rot, err));
            const long long nq = (long long)L.heads * L.dim, nk = (long long)L.kv_heads * L.dim;
            L.n_in = (int)(nq + nk);
            MU_TRY(stacked({{pre + "mix.q", nq}, {pre + "mix.k", nk}}, D, L.w_in));
            if (mx->has("conv")) {
                L.conv_w = (float*)dalloc((size_t)(nq + nk) * L.taps * 4);
                if (!L.conv_w) { err = "out of device memory"; return B200_ENOMEM; }
                MU_TRY(upload_tensor(st, pre + "mix.q.conv", {nq, L.taps}, true, dtype_, L.conv_w, err));
                MU_TRY(upload_tensor(st, pre + "mix.k.conv", {nk, L.taps}, true, dtype_, L.conv_w + (size_t)nq * L.taps, err));
            } else
                L.taps = 1;
            MU_TRY(f32(pre + "mix.q.norm", {L.dim}, L.q_norm));
            MU_TRY(f32(pre + "mix.k.norm", {L.dim}, L.k_norm));
            MU_TRY(mat(pre + "mix.o", D, (long long)L.heads * L.vdim, L.o));
            max_q_ = std::max(max_q_, (int)nq);
        } else if (type == "retention") {
            L.attention = false;
            if (L.dim > 256) { err = where + "dim above 256 is not supported by the retention kernel"; return B200_EUNSUPPORTED; }
            MU_TRY(parse_rot(*mx, L.dim, B200_ROPE_HALF, L.rot, err));
            const Json* dc = mx->get("decay");
            if (!dc || dc->kind != Json::Arr || (int)dc->arr.size() != L.heads) { err = where + "decay must list one value per head"; return B200_EINVAL; }
            std::vector<float> decay(L.heads);
            for (int h = 0; h < L.heads; ++h) decay[h] = (float)dc->arr[h].num;
            L.decay = (float*)dalloc((size_t)L.heads * 4);
            if (!L.decay || cudaMemcpy(L.decay, decay.data(), (size_t)L.heads * 4, cudaMemcpyHostToDevice) != cudaSuccess) { err = "out of device memory"; return B200_ENOMEM; }
            const long long nq = (long long)L.heads * L.dim, nv = (long long)L.heads * L.vdim;
            L.n_in = (int)(2 * nq + 2 * nv);
            MU_TRY(stacked({{pre + "mix.q", nq}, {pre + "mix.k", nq}, {pre + "mix.v", nv}, {pre + "mix.g", nv}}, D, L.w_in));
            MU_TRY(mat(pre + "mix.o", D, nv, L.o));
        } else {
            err = where + "mixer type '" + type + "' is not part of this family";
            return B200_EUNSUPPORTED;
        }
        max_in_ = std::max(max_in_, L.n_in);
        max_att_ = std::max(max_att_, L.heads * L.vdim);
        const Json* ml = lj.get("mlp");
        if (ml && !ml->is_null()) {
            const std::string kind = ml->text("kind");
            if (kind != "dense") { err = where + "feed-forward kind '" + kind + "' is not part of this family"; return B200_EUNSUPPORTED; }
            L.has_mlp = true;
            L.ff = (int)ml->integer("ff", 0);
            if (L.ff < 1) { err = where + "mlp.ff is required"; return B200_EINVAL; }
            MU_TRY(f32(pre + "norm2", {D}, L.n2w));
            MU_TRY(f32(pre + "norm2.b", {D}, L.n2b));
            MU_TRY(f32(pre + "norm2b", {D}, L.n2bw));
            MU_TRY(f32(pre + "norm2b.b", {D}, L.n2bb));
            MU_TRY(stacked({{pre + "mlp.gate", L.ff}, {pre + "mlp.up", L.ff}}, D, L.w_gu));
            MU_TRY(mat(pre + "mlp.down", D, L.ff, L.w_down));
            max_ff_ = std::max(max_ff_, L.ff);
        }
    }
    // the order in which layers run: before the span, the span `times` times, after it
    const int n = (int)layers_.size();
    std::vector<std::pair<int, bool>> order;
    const Json* lp = c.get("loop");
    if (lp && !lp->is_null()) {
        const int start = (int)lp->integer("start", 0), stop = (int)lp->integer("stop", 0), times = (int)lp->integer("times", 1);
        if (start < 0 || stop <= start || stop > n || times < 1) { err = "loop: need 0 <= start < stop <= layers and times >= 1"; return B200_EINVAL; }
        has_loop_ = true;
        MU_TRY(mat("loop.in", D, 2 * D, loop_in_));
        for (int i = 0; i < start; ++i) order.push_back({i, false});
        for (int k = 0; k < times; ++k)
            for (int i = start; i < stop; ++i) order.push_back({i, i == start});
        for (int i = stop; i < n; ++i) order.push_back({i, false});
    } else
        for (int i = 0; i < n; ++i) order.push_back({i, false});
    runs_.resize(order.size());
    const size_t cache_rows = (size_t)seq_.pool.n_pages() * kPageRows;
    for (size_t r = 0; r < runs_.size(); ++r) {
        MuRun& R = runs_[r];
        R.layer = order[r].first;
        R.pass_start = order[r].second;
        const MuLayer& L = layers_[R.layer];
        cudaError_t e = cudaSuccess;
        if (L.attention) {
            const size_t bytes = cache_rows * L.kv_heads * L.dim * E;
            R.k_pool = dalloc(bytes);
            R.v_pool = dalloc(bytes);
            if (!R.k_pool || !R.v_pool) { err = "out of device memory (K / V pages)"; return B200_ENOMEM; }
            cudaMemset(R.k_pool, 0, bytes);
            cudaMemset(R.v_pool, 0, bytes);
            if (L.taps > 1) e = R.state.init(opt.max_slots, (size_t)(L.taps - 1) * L.n_in);
        } else
            e = R.state.init(opt.max_slots, (size_t)L.heads * L.dim * L.vdim);
        if (e != cudaSuccess) { err = "out of device memory (carried state)"; return B200_ENOMEM; }
    }
    freq_off_.assign(freqs_.size(), 0);
    for (size_t k = 0; k < freqs_.size(); ++k) {
        freq_off_[k] = freq_floats_;
        freq_floats_ += 2 * (int)freqs_[k].f.size();   // cos and sin per token
    }
    if (cudaDeviceSynchronize() != cudaSuccess) { err = "weight upload failed"; return B200_EINVAL; }
    return B200_OK;
}

int Musilorn::ensure_scratch(int T, int W) {
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
        al(t * D_ * 4),                            // x
        al(t * D_ * 4),                            // x0
        al(t * max_in_ * 4),                       // proj
        al(t * D_ * 4),                            // y
        al(t * max_att_ * 4),                      // ret
        al((size_t)cW * vocab_ * 4),               // logits
        al(t * std::max(1, freq_floats_) * 4),     // cos / sin tables
        al(t * D_ * E),                            // h1
        al(t * D_ * E),                            // h2
        al(t * 2 * D_ * E),                        // cat
        al(t * std::max(1, max_q_) * E),           // q
        al(t * max_att_ * E),                      // att
        al(t * std::max(1, max_ff_) * E),          // act
        al((size_t)cW * D_ * E),                   // hf
        al((size_t)cW * 4),                        // ids
        al((size_t)std::min(cT, kStreamRows) * 2 * std::max(1, max_ff_) * 4),   // gu
    };
    size_t total = 0;
    for (size_t s : sizes) total += s;
    if (cudaMalloc(&scratch_, total) != cudaSuccess) return B200_ENOMEM;
    char* p = scratch_;
    int k = 0;
    auto take = [&](auto*& dst) { dst = reinterpret_cast<std::remove_reference_t<decltype(dst)>>(p); p += sizes[k++]; };
    take(x_); take(x0_); take(proj_); take(y_); take(ret_); take(logits_); take(cs_);
    take(h1_); take(h2_); take(cat_); take(q_); take(att_); take(act_); take(hf_); take(ids_dev_); take(gu_);
    cap_T_ = cT;
    cap_W_ = cW;
    return ensure_logits_host(cW);
}

// every launch of a step, in order, on stream_ (no synchronisation, no allocation: capturable into a graph)
int Musilorn::enqueue(int T, int W, int longest_entry, int longest_context, bool want_ids, std::string& err) {
    const int D = D_, dt = dtype_;
    const int* pages = seq_.pool.device();
    const int max_pages = seq_.pool.max_pages();
#define MU_OP(call)                                                             \
    do {                                                                        \
        const int rc_ = (call);                                                 \
        if (rc_ != B200_OK) { err = std::string(#call) + " failed (" + std::to_string(rc_) + ")"; return rc_; } \
    } while (0)
    // cos / sin of this step's positions, one table per frequency set: [T, n_freq] cos, then [T, n_freq] sin
    auto cos_of = [&](int table) { return cs_ + (size_t)T * freq_off_[table]; };
    auto sin_of = [&](int table) { return cs_ + (size_t)T * freq_off_[table] + (size_t)T * freqs_[table].f.size(); };
    for (size_t k = 0; k < freqs_.size(); ++k)
        MU_OP(b200_rope_angles(seq_.d_pos(), T, freqs_[k].dev, (int)freqs_[k].f.size(), cos_of((int)k), sin_of((int)k), stream_));
    MU_OP(b200_embed_positions(seq_.d_ids(), nullptr, embed_, nullptr, x_, T, D, dt, stream_));
    if (has_loop_) cudaMemcpyAsync(x0_, x_, (size_t)T * D * 4, cudaMemcpyDeviceToDevice, stream_);
    bool h1_ready = false;
    for (size_t r = 0; r < runs_.size(); ++r) {
        MuRun& R = runs_[r];
        const MuLayer& L = layers_[R.layer];
        if (R.pass_start) {
            MU_OP(b200_concat_cast(x_, x0_, cat_, T, D, dt, stream_));
            MU_OP(gemm(cat_, loop_in_, x_, B200_F32, T, D, 2 * D));
            h1_ready = false;
        }
        if (!h1_ready)
            MU_OP(b200_layernorm_pair(x_, nullptr, T, D, eps_, L.n1w, L.n1b, h1_, nullptr, nullptr, nullptr, dt, stream_));
        MU_OP(gemm(h1_, L.w_in, proj_, B200_F32, T, L.n_in, D));
        const int H = L.heads, natt = H * L.vdim;
        if (L.attention) {
            b200_qk_prepare_args qa{};
            qa.proj = proj_; qa.ld_proj = L.n_in;
            qa.conv_w = L.conv_w; qa.taps = L.taps; qa.conv_state = R.state.data();
            qa.q_norm = L.q_norm; qa.k_norm = L.k_norm; qa.eps = eps_;
            if (L.rot.dims > 0) { qa.cos = cos_of(L.rot.table); qa.sin = sin_of(L.rot.table); }
            qa.rot_dims = L.rot.dims; qa.rot_layout = L.rot.layout;
            qa.q_out = q_; qa.k_pool = R.k_pool; qa.v_pool = R.v_pool; qa.v_from_conv = 1;
            qa.pages = pages; qa.max_pages = max_pages; qa.page_rows = kPageRows;
            qa.slot = seq_.d_slot(); qa.pos = seq_.d_pos(); qa.start = seq_.d_start();
            qa.n_tokens = T; qa.heads = H; qa.kv_heads = L.kv_heads; qa.dim = L.dim; qa.dtype = dt;
            qa.update_state_inline = longest_entry == 1;
            MU_OP(b200_qk_prepare(&qa, stream_));
            if (L.conv_w && L.taps > 1 && longest_entry != 1)
                MU_OP(b200_conv_state_update(proj_, L.n_in, R.state.data(), seq_.d_slot(), seq_.d_pos(), seq_.d_end(), T, L.n_in, L.taps, stream_));
            b200_paged_attention_args pa{};
            pa.q = q_; pa.out = att_; pa.k_pool = R.k_pool; pa.v_pool = R.v_pool;
            pa.pages = pages; pa.max_pages = max_pages; pa.page_rows = kPageRows;
            pa.slot = seq_.d_slot(); pa.pos = seq_.d_pos();
            pa.n_tokens = T; pa.heads = H; pa.kv_heads = L.kv_heads; pa.dim = L.dim; pa.vdim = L.vdim;
            pa.scale = L.scale; pa.softcap = L.softcap; pa.denom_bias = 1.f;
            pa.dtype = dt; pa.longest_entry = longest_entry; pa.longest_context = longest_context;
            pa.workspace = attn_ws_; pa.workspace_bytes = attn_ws_bytes_;
            MU_OP(b200_paged_attention(&pa, stream_));
        } else {
            b200_retention_args ra{};
            ra.proj = proj_; ra.ld_proj = L.n_in;
            ra.q_off = 0; ra.k_off = H * L.dim; ra.v_off = 2 * H * L.dim;
            if (L.rot.dims > 0) { ra.cos = cos_of(L.rot.table); ra.sin = sin_of(L.rot.table); }
            ra.rot_dims = L.rot.dims; ra.rot_layout = L.rot.layout;
            ra.decay = L.decay; ra.k_scale = 1.0f / sqrtf((float)L.dim);
            ra.state = R.state.data(); ra.out = ret_;
            ra.ent_row = seq_.d_ent_row(); ra.ent_len = seq_.d_ent_len(); ra.slot = seq_.d_slot(); ra.pos = seq_.d_pos();
            ra.n_entries = seq_.n_entries; ra.n_tokens = T; ra.heads = H; ra.dim = L.dim; ra.vdim = L.vdim;
            ra.longest_entry = longest_entry;
            ra.workspace = attn_ws_; ra.workspace_bytes = attn_ws_bytes_;
            MU_OP(b200_retention(&ra, stream_));
            MU_OP(b200_unit_rms_gate(ret_, proj_ + 2 * H * L.dim + natt, L.n_in, att_, T, H, L.vdim, eps_, dt, stream_));
        }
        MU_OP(gemm(att_, L.o, y_, B200_F32, T, D, natt));
        // the norm that follows: this layer's feed-forward input, or the next run's mixer input (unless a pass starts there)
        const MuLayer* next = (r + 1 < runs_.size() && !runs_[r + 1].pass_start) ? &layers_[runs_[r + 1].layer] : nullptr;
        if (L.has_mlp) {
            MU_OP(b200_layernorm_residual(x_, y_, T, D, eps_, mult_, L.n1bw, L.n1bb, L.n2w, L.n2b, h2_, dt, stream_));
            if (dt == B200_BF16 && T <= kStreamRows) {   // few rows: the stacked [gate; up] streams once through the split-K GEMM
                MU_OP(gemm(h2_, L.w_gu, gu_, B200_F32, T, 2 * L.ff, D));
                MU_OP(b200_glu_act(gu_, act_, T, L.ff, B200_GG_GLU_GELU, dt, stream_));
            } else
                MU_OP(gemm(h2_, L.w_gu, act_, dt, T, L.ff, D, B200_GG_GLU_GELU));
            MU_OP(gemm(act_, L.w_down, y_, B200_F32, T, D, L.ff));
            MU_OP(b200_layernorm_residual(x_, y_, T, D, eps_, mult_, L.n2bw, L.n2bb, next ? next->n1w : nullptr, next ? next->n1b : nullptr,
                                          next ? h1_ : nullptr, dt, stream_));
        } else
            MU_OP(b200_layernorm_residual(x_, y_, T, D, eps_, mult_, L.n1bw, L.n1bb, next ? next->n1w : nullptr, next ? next->n1b : nullptr,
                                          next ? h1_ : nullptr, dt, stream_));
        h1_ready = next != nullptr;
        keep_layer(r, x_, T);
    }
    if (W > 0) {
        MU_OP(b200_layernorm_pair(x_, seq_.d_want_rows(), W, D, eps_, fnw_, fnb_, hf_, nullptr, nullptr, nullptr, dt, stream_));
        MU_OP(gemm(hf_, head_, logits_, B200_F32, W, vocab_, D));
        if (logit_cap_ > 0.f) MU_OP(b200_softcap(logits_, (size_t)W * vocab_, logit_cap_, stream_));
        if (want_ids) MU_OP(b200_argmax(logits_, ids_dev_, W, vocab_, B200_F32, stream_));
    }
    return B200_OK;
#undef MU_OP
}

Model* make_musilorn(const ModelDir& dir, const b200_model_options& opt, std::string& err) {
    Musilorn* m = new Musilorn();
    if (m->load(dir, opt, err) != B200_OK) {
        delete m;
        return nullptr;
    }
    return m;
}

FamilyRegistrar reg_musilorn("Musilorn", make_musilorn);

}  // namespace
}  // namespace b200
