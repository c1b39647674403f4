// Model family "Tomalix": a pre-norm decoder, x <- x + mixer(N1 x), x <- x + ff(N2 x), N x = x / rms(x) * (1 + w), with
// three kinds of mixer that config.json orders freely:
//   "attention"    differential attention: every query head holds two score maps [q1 | q2] against [k1 | k2] of its key
//                  head over the SAME values; o = a1 - lambda a2 with one lambda per layer, unit RMS per head, times
//                  (1 - diff); rotate-half rotary positions whose frequencies are divided by a factor.
//   "parallel"     two mixers read the same input and their outputs are added with two weights: an attention whose
//                  queries only see the keys of their own block of positions (blocks counted from position 0), with a
//                  sigmoid output gate; and a selective scan (short causal convolution + silu, input-dependent step
//                  sizes, a diagonal state per channel carried per sequence).
//   "attention_2"  plain grouped-query attention with the ramped frequency interpolation and its amplitude factor.
// Feed-forwards: none, dense (squared relu), or a routed mixture of such experts (top-k on the biased logits, softmax over
// the chosen). A span of layers ("loop") runs several times with the same weights; every pass adds a per-pass vector
// (and, from the second pass on, the embedding output) to x, and every layer RUN owns its cache pages and states. The
// logits are tanh-capped.
//
// A step runs on the family-independent pieces of the library: StepRunner (stream, workspaces, graph replay of single-token
// steps, results to the host), SequenceBatch / PagePool for slots, pages and the per-token tables, SlotState for what is
// carried per slot, b200_rmsnorm_residual, b200_linear_ex (tcgen05) and
// b200_gemm_grouped, b200_rope_angles_amp, b200_qk_prepare, b200_paged_attention (block mask, score maps),
// b200_diff_combine / b200_sigmoid_gate, b200_conv_act / b200_selective_scan, b200_moe_route_logits / b200_moe_dispatch.
// The residual stream, all norms, rotary angles, scores and softmax, the router, the scan and everything entering it
// after the projections are fp32 in both serving dtypes; in B200_BF16 the GEMM operands and the K / V pages are bfloat16.
//
// Launch order of a layer run (T tokens of all entries packed):
//   [pass start: x += x0 + step vector, N1]  ->  [q | k | v | (g) | (scan in)] = h W^T (one GEMM, fp32 out)
//   q / k rotation and page stores -> paged attention -> (map combination | gate) -> W_o
//   scan side: convolution + silu -> ring update -> [dt | B | C] GEMM -> dt GEMM -> scan (gated by silu(z)) -> W_o
//   x += (weighted) outputs fused with N2 -> up GEMM with squared relu (dense, or grouped by expert after routing) ->
//   down GEMM -> x += output (experts: weighted gather) fused with the next run's N1.
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
constexpr double kPi = 3.14159265358979323846;

struct TxFreq {
    std::vector<double> f;
    double amp = 1.0;
    double* dev = nullptr;
};

struct TxAttn {   // one attention (the whole mixer, or the left half of a parallel one)
    int heads = 0, kv_heads = 0, dim = 0, vdim = 0, maps = 1, chunk = 0, rot_dims = 0, table = -1;
    float scale = 1.f;
    int q_off = 0, k_off = 0, v_off = 0, g_off = -1;   // columns in the stacked input projection
    int nq() const { return heads * maps * dim; }
    int nk() const { return kv_heads * maps * dim; }
    int nv() const { return kv_heads * vdim; }
    int natt() const { return heads * vdim; }
};
struct TxScan {
    int inner = 0, state = 0, dt_rank = 0, taps = 1, in_off = 0;
    float *conv_w = nullptr, *conv_b = nullptr, *dt_b = nullptr, *A = nullptr, *Dv = nullptr;
    void *w_x = nullptr, *w_dt = nullptr, *w_o = nullptr;
};
enum { kMixDiff = 0, kMixParallel = 1, kMixPlain = 2 };
enum { kFfNone = 0, kFfDense = 1, kFfRouted = 2 };

struct TxLayer {
    int kind = kMixPlain, ff_kind = kFfNone;
    TxAttn at;
    TxScan sc;
    float left_scale = 1.f, right_scale = 1.f, lambda = 0.f, diff = 0.f;
    int n_in = 0, ff = 0, experts = 0, top = 0;
    float *n1 = nullptr, *n2 = nullptr, *router = nullptr, *router_b = nullptr;
    void *w_in = nullptr, *o = nullptr, *w_up = nullptr, *w_down = nullptr;
};

struct TxRun {
    int layer = 0, pass = -1;                     // pass >= 0: this run starts pass number `pass` of the span
    void *k_pool = nullptr, *v_pool = nullptr;
    SlotState ring, state;                        // parallel: the convolution's carried inputs, the scan state
};

class Tomalix : public StepRunner {
public:
    ~Tomalix() override {
        if (stream_) cudaStreamSynchronize(stream_);
        for (cudaStream_t s : side_) { cudaStreamSynchronize(s); cudaStreamDestroy(s); }
        for (cudaEvent_t e : joined_) cudaEventDestroy(e);
        if (forked_) cudaEventDestroy(forked_);
        if (group_off_host_) cudaFreeHost(group_off_host_);
        cudaFree(scratch_);
    }
    const char* family() const override { return "Tomalix"; }
    int layer_count() const override { return (int)runs_.size(); }   // layer runs: what a step executes and captures

    int load(const ModelDir& dir, const b200_model_options& opt, std::string& err);

private:
    int parse_attn(const Json& mx, const std::string& where, int maps, bool ramp_allowed, TxAttn& at, std::string& err);
    int ensure_scratch(int T, int W) override;
    int experts_on_side_streams(const TxLayer& L, int T, std::string& err);
    int enqueue(int T, int W, int longest_entry, int longest_context, bool want_ids, std::string& err) override;
    size_t step_workspace_bytes(int T, int n_entries) const override {
        size_t need = 0;
        for (const TxLayer& L : layers_) {
            need = std::max(need, b200_paged_attention_workspace_bytes(T, L.at.heads * L.at.maps, L.at.vdim));
            if (L.kind == kMixParallel) need = std::max(need, b200_selective_scan_workspace_bytes(T, n_entries, L.sc.inner, L.sc.state));
        }
        return need;
    }

    float eps_ = 1e-5f, logit_cap_ = 0.f;
    std::vector<TxLayer> layers_;
    std::vector<TxRun> runs_;
    std::vector<TxFreq> freqs_;
    bool has_loop_ = false;
    void *embed_ = nullptr, *head_ = nullptr;
    float *fnw_ = nullptr, *loop_step_ = nullptr;
    // scratch, grown to the largest step seen
    char* scratch_ = nullptr;
    int cap_T_ = 0, cap_W_ = 0;
    float *x_ = nullptr, *x0_ = nullptr, *proj_ = nullptr, *y_ = nullptr, *y2_ = nullptr, *attf_ = nullptr, *xc32_ = nullptr, *bc_ = nullptr,
          *dtr_ = nullptr, *eo_ = nullptr, *weight_ = nullptr, *cs_ = nullptr;
    void *h1_ = nullptr, *h2_ = nullptr, *q_ = nullptr, *att_ = nullptr, *xc_ = nullptr, *sy_ = nullptr, *act_ = nullptr, *hf_ = nullptr;
    int *chosen_ = nullptr, *group_off_ = nullptr, *src_row_ = nullptr, *dest_ = nullptr;
    // prompt steps: every expert's group as dense GEMMs of its own, spread over side streams
    void* gath_ = nullptr;
    int* group_off_host_ = nullptr;   // pinned
    std::vector<cudaStream_t> side_;
    std::vector<cudaEvent_t> joined_;
    cudaEvent_t forked_ = nullptr;
    // maxima over layers (scratch sizes)
    int max_in_ = 0, max_q_ = 0, max_attf_ = 0, max_att_ = 0, max_inner_ = 0, max_bc_ = 0, max_act_ = 0, max_top_ = 0, max_experts_ = 0,
        freq_floats_ = 0;
    std::vector<int> freq_off_;   // first float of each frequency set's cos table in cs_ (per token: see enqueue)
};

#define TX_TRY(call)                    \
    do {                                \
        const int rc_ = (call);         \
        if (rc_ != B200_OK) return rc_; \
    } while (0)

// Sizes, scale and rotary frequencies of one attention. f_i = base^(-2i/dims); "scaling" {factor} divides every f_i by
// factor; "scaling" {factor, original, fast, slow} (where the mixer has the ramped rule: ramp_allowed) blends f_i / factor
// and f_i with a ramp over the index i between the indices whose wavelengths make `fast` and `slow` turns within
// `original` positions, and multiplies cos and sin by 0.1 ln(factor) + 1. Equal (frequencies, amplitude) share one cos /
// sin table per step.
int Tomalix::parse_attn(const Json& mx, const std::string& where, int maps, bool ramp_allowed, TxAttn& at, std::string& err) {
    at.heads = (int)mx.integer("heads", 0);
    at.kv_heads = (int)mx.integer("kv_heads", at.heads);
    at.dim = (int)mx.integer("dim", 0);
    at.vdim = (int)mx.integer("vdim", 0);
    at.maps = maps;
    if (at.heads < 1 || at.kv_heads < 1 || at.dim < 1 || at.vdim < 1) { err = where + "attention needs heads, kv_heads, dim, vdim"; return B200_EINVAL; }
    if (at.heads % at.kv_heads) { err = where + "heads must be a multiple of kv_heads"; return B200_EINVAL; }
    if (at.vdim > 256) { err = where + "vdim above 256 is not supported by the attention kernels"; return B200_EUNSUPPORTED; }
    if (!mx.has("scale")) { err = where + "attention needs scale"; return B200_EINVAL; }
    at.scale = (float)mx.number("scale", 1.0);
    const Json* mk = mx.get("mask");
    at.chunk = (mk && !mk->is_null()) ? (int)mk->integer("size", 0) : 0;
    if (at.chunk < 0) { err = where + "mask.size must be positive"; return B200_EINVAL; }
    const Json* r = mx.get("rot");
    at.rot_dims = (r && !r->is_null()) ? (int)r->integer("dims", 0) : 0;
    if (at.rot_dims == 0) return B200_OK;
    const double base = r->number("base", 0.0);
    if (at.rot_dims < 0 || (at.rot_dims & 1) || at.rot_dims > at.dim || !(base > 1.0)) { err = where + "rot: dims must be even and at most dim, base above 1"; return B200_EINVAL; }
    const int d = at.rot_dims;
    TxFreq fs;
    fs.f.resize(d / 2);
    for (int i = 0; i < d / 2; ++i) fs.f[i] = std::pow(base, -2.0 * i / d);
    const Json* sc = r->get("scaling");
    if (sc && !sc->is_null()) {
        const double factor = sc->number("factor", 1.0);
        if (!(factor > 0.0)) { err = where + "rot.scaling.factor must be positive"; return B200_EINVAL; }
        if (ramp_allowed && sc->has("original")) {
            const double orig = sc->number("original", 0.0), fast = sc->number("fast", 32.0), slow = sc->number("slow", 1.0);
            if (!(orig > 0.0) || !(fast > 0.0) || !(slow > 0.0)) { err = where + "rot.scaling needs positive original, fast, slow"; return B200_EINVAL; }
            auto index_of = [&](double turns) { return d * std::log(orig / (2.0 * kPi * turns)) / (2.0 * std::log(base)); };
            const double lo = std::max(std::floor(index_of(fast)), 0.0), hi = std::min(std::ceil(index_of(slow)), (double)(d - 1));
            for (int i = 0; i < d / 2; ++i) {
                const double ramp = std::min(std::max((i - lo) / std::max(hi - lo, 0.001), 0.0), 1.0);
                fs.f[i] = fs.f[i] / factor * ramp + fs.f[i] * (1.0 - ramp);
            }
            fs.amp = 0.1 * std::log(factor) + 1.0;
        } else
            for (double& fi : fs.f) fi /= factor;
    }
    for (size_t k = 0; k < freqs_.size(); ++k)
        if (freqs_[k].f == fs.f && freqs_[k].amp == fs.amp) { at.table = (int)k; return B200_OK; }
    fs.dev = (double*)dalloc(fs.f.size() * sizeof(double));
    if (!fs.dev || cudaMemcpy(fs.dev, fs.f.data(), fs.f.size() * sizeof(double), cudaMemcpyHostToDevice) != cudaSuccess) { err = "out of device memory"; return B200_ENOMEM; }
    at.table = (int)freqs_.size();
    freqs_.push_back(fs);
    return B200_OK;
}

int Tomalix::load(const ModelDir& dir, const b200_model_options& opt, std::string& err) {
    const Json& c = dir.config;
    dtype_ = opt.dtype;
    if (dtype_ != B200_BF16 && dtype_ != B200_F32) { err = "dtype must be bfloat16 or float32"; return B200_EINVAL; }
    vocab_ = (int)c.integer("vocab", 0);
    D_ = (int)c.integer("width", 0);
    const Json* norm = c.get("norm");
    const Json* ls = c.get("layers");
    if (vocab_ < 1 || D_ < 1 || !norm || !norm->has("eps") || !ls || ls->kind != Json::Arr || ls->arr.empty()) {
        err = "config.json: vocab, width, norm.eps and layers are required";
        return B200_EINVAL;
    }
    eps_ = (float)norm->number("eps", 1e-5);
    logit_cap_ = (float)c.number("logit_softcap", 0.0);
    if (opt.max_tokens < 1 || opt.max_slots < 1) { err = "max_tokens and max_slots must be positive"; return B200_EINVAL; }
    // everything that can be refused from the configuration alone is refused before the first CUDA call
    for (size_t i = 0; i < ls->arr.size(); ++i) {
        const std::string type = ls->arr[i].text("type"), where = "layer " + std::to_string(i) + ": ";
        if (type != "attention" && type != "parallel" && type != "attention_2") { err = where + "mixer type '" + type + "' is not part of this family"; return B200_EUNSUPPORTED; }
        const Json* mx = ls->arr[i].get("mixer");
        if (!mx || mx->is_null()) { err = where + "no mixer"; return B200_EINVAL; }
        const Json* ml = ls->arr[i].get("mlp");
        if (ml && !ml->is_null()) {
            const std::string kind = ml->text("kind");
            if (kind != "dense" && kind != "moe") { err = where + "feed-forward kind '" + kind + "' is not part of this family"; return B200_EUNSUPPORTED; }
        }
    }
    const int n = (int)ls->arr.size();
    std::vector<std::pair<int, int>> order;   // (layer, pass number or -1)
    const Json* lp = c.get("loop");
    int loop_times = 0;
    if (lp && !lp->is_null()) {
        const int start = (int)lp->integer("start", 0), stop = (int)lp->integer("stop", 0), times = (int)lp->integer("times", 1);
        if (start < 0 || stop <= start || stop > n || times < 1) { err = "loop: need 0 <= start < stop <= layers and times >= 1"; return B200_EINVAL; }
        has_loop_ = true;
        loop_times = times;
        for (int i = 0; i < start; ++i) order.push_back({i, -1});
        for (int k = 0; k < times; ++k)
            for (int i = start; i < stop; ++i) order.push_back({i, i == start ? k : -1});
        for (int i = stop; i < n; ++i) order.push_back({i, -1});
    } else
        for (int i = 0; i < n; ++i) order.push_back({i, -1});

    TX_TRY(init_runner(err));
    SafeTensorsFile st;
    if (!st.open(dir.path + "/model.safetensors", err)) return B200_EINVAL;
    // the design has no position limit of its own: a sequence can grow as long as the pool has pages
    const int n_pages = (opt.max_tokens + kPageRows - 1) / kPageRows;
    TX_TRY(seq_.init(opt.max_tokens, kPageRows, opt.max_slots, n_pages * kPageRows, err));

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
    // several checkpoint matrices that read the same input (or the experts of one layer), stacked row-wise into one operand
    auto stacked = [&](const std::vector<std::pair<std::string, long long>>& parts, long long cols, void*& dst) -> int {
        long long rows = 0;
        for (auto& p : parts) rows += p.second;
        dst = dalloc((size_t)rows * cols * E);
        if (!dst) { err = "out of device memory"; return B200_ENOMEM; }
        long long at = 0;
        for (auto& p : parts) {
            TX_TRY(upload_tensor(st, p.first, {p.second, cols}, false, dtype_, (char*)dst + (size_t)at * cols * E, err));
            at += p.second;
        }
        return B200_OK;
    };
    // a small fp32 tensor read on the host
    auto host_vec = [&](const std::string& name, long long len, std::vector<double>& out) -> int {
        const SafeTensor* t = st.find(name);
        if (!t) { err = "tensor " + name + " is missing"; return B200_EINVAL; }
        if ((long long)t->elems() != len || (t->dtype != "BF16" && t->dtype != "F32")) { err = "tensor " + name + " does not have " + std::to_string(len) + " floating-point values"; return B200_EINVAL; }
        out.resize(len);
        for (long long i = 0; i < len; ++i) out[i] = st_value(*t, i);
        return B200_OK;
    };
    TX_TRY(mat("embed", vocab_, D, embed_));
    TX_TRY(mat("head", vocab_, D, head_));
    TX_TRY(f32("final.norm", {D}, fnw_));
    if (has_loop_) TX_TRY(f32("loop.step", {loop_times, D}, loop_step_));

    layers_.resize(n);
    for (int i = 0; i < n; ++i) {
        const Json& lj = ls->arr[i];
        TxLayer& L = layers_[i];
        const std::string pre = "l" + std::to_string(i) + ".", where = "layer " + std::to_string(i) + ": ";
        const std::string type = lj.text("type");
        const Json& mx = *lj.get("mixer");
        TX_TRY(f32(pre + "norm1", {D}, L.n1));
        std::vector<std::pair<std::string, long long>> parts;
        if (type == "parallel") {
            L.kind = kMixParallel;
            const Json* left = mx.get("left");
            const Json* right = mx.get("right");
            if (!left || left->is_null() || !right || right->is_null()) { err = where + "a parallel mixer needs left and right"; return B200_EINVAL; }
            L.left_scale = (float)mx.number("left_scale", 1.0);
            L.right_scale = (float)mx.number("right_scale", 1.0);
            TX_TRY(parse_attn(*left, where, 1, true, L.at, err));
            TxAttn& at = L.at;
            at.q_off = 0; at.k_off = at.nq(); at.v_off = at.k_off + at.nk(); at.g_off = at.v_off + at.nv();
            TxScan& sc = L.sc;
            sc.inner = (int)right->integer("inner", 0);
            sc.state = (int)right->integer("state", 0);
            sc.dt_rank = (int)right->integer("dt_rank", 0);
            sc.taps = (int)right->integer("conv", 1);
            if (sc.inner < 1 || sc.state < 1 || sc.dt_rank < 1 || sc.taps < 1) { err = where + "the scan needs inner, state, dt_rank, conv"; return B200_EINVAL; }
            if (sc.state > 256) { err = where + "state above 256 is not supported by the scan kernel"; return B200_EUNSUPPORTED; }
            sc.in_off = at.g_off + at.natt();
            L.n_in = sc.in_off + 2 * sc.inner;
            const std::string lp_ = pre + "mix.left.", rp = pre + "mix.right.";
            parts = {{lp_ + "q", at.nq()}, {lp_ + "k", at.nk()}, {lp_ + "v", at.nv()}, {lp_ + "g", at.natt()}, {rp + "in", 2ll * sc.inner}};
            TX_TRY(stacked(parts, D, L.w_in));
            TX_TRY(mat(lp_ + "o", D, at.natt(), L.o));
            TX_TRY(f32(rp + "conv", {sc.inner, sc.taps}, sc.conv_w));
            TX_TRY(f32(rp + "conv.b", {sc.inner}, sc.conv_b));
            TX_TRY(mat(rp + "x", sc.dt_rank + 2ll * sc.state, sc.inner, sc.w_x));
            TX_TRY(mat(rp + "dt", sc.inner, sc.dt_rank, sc.w_dt));
            TX_TRY(f32(rp + "dt.b", {sc.inner}, sc.dt_b));
            TX_TRY(f32(rp + "D", {sc.inner}, sc.Dv));
            {   // A = -exp(A_log), formed once in double
                std::vector<double> al;
                TX_TRY(host_vec(rp + "A_log", (long long)sc.inner * sc.state, al));
                const SafeTensor* t = st.find(rp + "A_log");
                if (t->shape != std::vector<long long>{sc.inner, sc.state}) { err = "tensor " + rp + "A_log has the wrong shape"; return B200_EINVAL; }
                std::vector<float> A(al.size());
                for (size_t k = 0; k < al.size(); ++k) A[k] = (float)-std::exp(al[k]);
                sc.A = (float*)dalloc(A.size() * 4);
                if (!sc.A || cudaMemcpy(sc.A, A.data(), A.size() * 4, cudaMemcpyHostToDevice) != cudaSuccess) { err = "out of device memory"; return B200_ENOMEM; }
            }
            TX_TRY(mat(rp + "o", D, sc.inner, sc.w_o));
            max_inner_ = std::max(max_inner_, sc.inner);
            max_bc_ = std::max(max_bc_, sc.dt_rank + 2 * sc.state);
        } else {
            const bool diff = type == "attention";
            L.kind = diff ? kMixDiff : kMixPlain;
            TX_TRY(parse_attn(mx, where, diff ? 2 : 1, !diff, L.at, err));
            TxAttn& at = L.at;
            at.q_off = 0; at.k_off = at.nq(); at.v_off = at.k_off + at.nk();
            L.n_in = at.v_off + at.nv();
            const std::string mp = pre + "mix.";
            parts = {{mp + "q", at.nq()}, {mp + "k", at.nk()}, {mp + "v", at.nv()}};
            TX_TRY(stacked(parts, D, L.w_in));
            TX_TRY(mat(mp + "o", D, at.natt(), L.o));
            if (diff) {
                L.diff = (float)mx.number("diff", 0.0);
                std::vector<double> q1, k1, q2, k2;
                TX_TRY(host_vec(mp + "lq1", at.dim, q1));
                TX_TRY(host_vec(mp + "lk1", at.dim, k1));
                TX_TRY(host_vec(mp + "lq2", at.dim, q2));
                TX_TRY(host_vec(mp + "lk2", at.dim, k2));
                double s1 = 0.0, s2 = 0.0;
                for (int k = 0; k < at.dim; ++k) { s1 += q1[k] * k1[k]; s2 += q2[k] * k2[k]; }
                L.lambda = (float)(std::exp(s1) - std::exp(s2) + (double)mx.number("diff", 0.0));
            }
        }
        max_in_ = std::max(max_in_, L.n_in);
        max_q_ = std::max(max_q_, L.at.nq());
        max_attf_ = std::max(max_attf_, L.at.heads * L.at.maps * L.at.vdim);
        max_att_ = std::max(max_att_, L.at.natt());
        const Json* ml = lj.get("mlp");
        if (ml && !ml->is_null()) {
            TX_TRY(f32(pre + "norm2", {D}, L.n2));
            if (ml->text("kind") == "dense") {
                L.ff_kind = kFfDense;
                L.ff = (int)ml->integer("ff", 0);
                if (L.ff < 1) { err = where + "mlp.ff is required"; return B200_EINVAL; }
                TX_TRY(mat(pre + "mlp.up", L.ff, D, L.w_up));
                TX_TRY(mat(pre + "mlp.down", D, L.ff, L.w_down));
                max_act_ = std::max(max_act_, L.ff);
            } else {
                L.ff_kind = kFfRouted;
                const Json* ex = ml->get("expert");
                const Json* ro = ml->get("router");
                L.ff = ex ? (int)ex->integer("ff", 0) : 0;
                L.experts = ro ? (int)ro->integer("experts", 0) : 0;
                L.top = ro ? (int)ro->integer("top", 0) : 0;
                if (L.ff < 1 || L.experts < 1 || L.top < 1 || L.top > L.experts) { err = where + "a routed feed-forward needs expert.ff, router.experts and 1 <= router.top <= experts"; return B200_EINVAL; }
                if (L.top > 16) { err = where + "more than 16 experts per token are not supported"; return B200_EUNSUPPORTED; }
                std::vector<std::pair<std::string, long long>> ups, downs;
                for (int e = 0; e < L.experts; ++e) {
                    ups.push_back({pre + "mlp.e" + std::to_string(e) + ".up", L.ff});
                    downs.push_back({pre + "mlp.e" + std::to_string(e) + ".down", D});
                }
                TX_TRY(stacked(ups, D, L.w_up));        // [experts, ff, D]
                TX_TRY(stacked(downs, L.ff, L.w_down)); // [experts, D, ff]
                TX_TRY(f32(pre + "mlp.router", {L.experts, D}, L.router));
                TX_TRY(f32(pre + "mlp.router.b", {L.experts}, L.router_b));
                max_act_ = std::max(max_act_, L.top * L.ff);
                max_top_ = std::max(max_top_, L.top);
                max_experts_ = std::max(max_experts_, L.experts);
            }
        }
    }
    runs_.resize(order.size());
    const size_t cache_rows = (size_t)seq_.pool.n_pages() * kPageRows;
    for (size_t r = 0; r < runs_.size(); ++r) {
        TxRun& R = runs_[r];
        R.layer = order[r].first;
        R.pass = order[r].second;
        const TxLayer& L = layers_[R.layer];
        const size_t kb = cache_rows * L.at.nk() * E, vb = cache_rows * L.at.nv() * E;
        R.k_pool = dalloc(kb);
        R.v_pool = dalloc(vb);
        if (!R.k_pool || !R.v_pool) { err = "out of device memory (K / V pages)"; return B200_ENOMEM; }
        cudaMemset(R.k_pool, 0, kb);
        cudaMemset(R.v_pool, 0, vb);
        if (L.kind == kMixParallel) {
            cudaError_t e = cudaSuccess;
            if (L.sc.taps > 1) e = R.ring.init(opt.max_slots, (size_t)(L.sc.taps - 1) * L.sc.inner);
            if (e == cudaSuccess) e = R.state.init(opt.max_slots, (size_t)L.sc.inner * L.sc.state);
            if (e != cudaSuccess) { err = "out of device memory (carried state)"; return B200_ENOMEM; }
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

int Tomalix::ensure_scratch(int T, int W) {
    if (T <= cap_T_ && W <= cap_W_) return B200_OK;
    const int cT = std::max(T, cap_T_), cW = std::max(W, cap_W_);
    cudaStreamSynchronize(stream_);
    buffers_moved();
    cudaFree(scratch_);
    scratch_ = nullptr;
    cap_T_ = cap_W_ = 0;
    auto al = [](size_t b) { return (b + 255) & ~(size_t)255; };
    const size_t E = esz(), t = (size_t)cT, top = (size_t)std::max(1, max_top_);
    const size_t sizes[] = {
        al(t * D_ * 4),                            // x
        al(t * D_ * 4),                            // x0
        al(t * max_in_ * 4),                       // proj
        al(t * D_ * 4),                            // y
        al(t * D_ * 4),                            // y2
        al(t * max_attf_ * 4),                     // attf
        al(t * std::max(1, max_inner_) * 4),       // xc32
        al(t * std::max(1, max_bc_) * 4),          // bc
        al(t * std::max(1, max_inner_) * 4),       // dtr
        al(t * top * D_ * 4),                      // eo
        al(t * top * 4),                           // weight
        al((size_t)cW * vocab_ * 4),               // logits
        al(t * std::max(1, freq_floats_) * 4),     // cos / sin tables
        al(t * D_ * E),                            // h1
        al(t * D_ * E),                            // h2
        al(t * std::max(1, max_q_) * E),           // q
        al(t * max_att_ * E),                      // att
        al(t * std::max(1, max_inner_) * E),       // xc
        al(t * std::max(1, max_inner_) * E),       // sy
        al(t * std::max(1, max_act_) * E),         // act
        al(t * top * D_ * E),                      // gath
        al((size_t)cW * D_ * E),                   // hf
        al(t * top * 4),                           // chosen
        al((size_t)(max_experts_ + 2) * 4),        // group_off
        al(t * top * 4),                           // src_row
        al(t * top * 4),                           // dest
        al((size_t)cW * 4),                        // ids
    };
    size_t total = 0;
    for (size_t s : sizes) total += s;
    if (cudaMalloc(&scratch_, total) != cudaSuccess) return B200_ENOMEM;
    char* p = scratch_;
    int k = 0;
    auto take = [&](auto*& dst) { dst = reinterpret_cast<std::remove_reference_t<decltype(dst)>>(p); p += sizes[k++]; };
    take(x_); take(x0_); take(proj_); take(y_); take(y2_); take(attf_); take(xc32_); take(bc_); take(dtr_); take(eo_); take(weight_);
    take(logits_); take(cs_);
    take(h1_); take(h2_); take(q_); take(att_); take(xc_); take(sy_); take(act_); take(gath_); take(hf_);
    take(chosen_); take(group_off_); take(src_row_); take(dest_); take(ids_dev_);
    cap_T_ = cT;
    cap_W_ = cW;
    return ensure_logits_host(cW);
}

// Routed experts of a prompt step. With hundreds of rows per expert the groups are dense GEMMs in their own right: the
// group sizes come to the host (one small copy and a synchronisation: a prompt step is not captured into a graph), the
// sorted rows are gathered side by side, and every expert's up (squared relu) and down products run on the tcgen05 GEMM,
// spread over side streams so that products of a few dozen tiles each fill the GPU together. Single-token steps and
// small prompts stay on the grouped kernel, which needs no host round trip.
constexpr int kExpertStreamsFrom = 1024, kExpertStreams = 4;
int Tomalix::experts_on_side_streams(const TxLayer& L, int T, std::string& err) {
    const int D = D_, dt = dtype_, E = L.experts;
    const size_t ez = esz();
    if (side_.empty()) {
        if (cudaEventCreateWithFlags(&forked_, cudaEventDisableTiming) != cudaSuccess) { err = "cudaEventCreate"; return B200_EINVAL; }
        for (int k = 0; k < kExpertStreams; ++k) {
            cudaStream_t s = nullptr;
            cudaEvent_t e = nullptr;
            if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess || cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) { err = "cudaStreamCreate"; return B200_EINVAL; }
            side_.push_back(s);
            joined_.push_back(e);
        }
    }
    if (!group_off_host_ && cudaMallocHost(&group_off_host_, (size_t)(max_experts_ + 2) * sizeof(int)) != cudaSuccess) { err = "cudaMallocHost"; return B200_ENOMEM; }
    cudaMemcpyAsync(group_off_host_, group_off_, (size_t)(E + 1) * sizeof(int), cudaMemcpyDeviceToHost, stream_);
    int rc = b200_gather_rows(h2_, src_row_, gath_, T * L.top, D, dt, stream_);
    if (rc != B200_OK) { err = "b200_gather_rows failed"; return rc; }
    cudaEventRecord(forked_, stream_);
    if (cudaStreamSynchronize(stream_) != cudaSuccess) { err = "step: synchronisation before the expert products failed"; return B200_EINVAL; }
    for (cudaStream_t s : side_) cudaStreamWaitEvent(s, forked_, 0);
    int used = 0;
    for (int e = 0; e < E; ++e) {
        const int off = group_off_host_[e], n = group_off_host_[e + 1] - off;
        if (n <= 0) continue;
        cudaStream_t s = side_[used++ % kExpertStreams];
        // no split-K workspace: the products of different streams run at the same time and must not share one
        rc = b200_linear_ex((const char*)gath_ + (size_t)off * D * ez, (const char*)L.w_up + (size_t)e * L.ff * D * ez,
                            (char*)act_ + (size_t)off * L.ff * ez, n, L.ff, D, dt, dt, B200_GG_RELU2, nullptr, 0, s);
        if (rc == B200_OK)
            rc = b200_linear_ex((const char*)act_ + (size_t)off * L.ff * ez, (const char*)L.w_down + (size_t)e * D * L.ff * ez,
                                eo_ + (size_t)off * D, n, D, L.ff, dt, B200_F32, B200_GG_NONE, nullptr, 0, s);
        if (rc != B200_OK) { err = "expert product failed (" + std::to_string(rc) + ")"; break; }
    }
    for (int k = 0; k < kExpertStreams; ++k) {   // joined even after a failure: nothing of this step stays in flight behind stream_
        cudaEventRecord(joined_[k], side_[k]);
        cudaStreamWaitEvent(stream_, joined_[k], 0);
    }
    return rc;
}

// every launch of a step, in order, on stream_ (no synchronisation, no allocation: capturable into a graph)
int Tomalix::enqueue(int T, int W, int longest_entry, int longest_context, bool want_ids, std::string& err) {
    const int D = D_, dt = dtype_;
    const int* pages = seq_.pool.device();
    const int max_pages = seq_.pool.max_pages();
#define TX_OP(call)                                                             \
    do {                                                                        \
        const int rc_ = (call);                                                 \
        if (rc_ != B200_OK) { err = std::string(#call) + " failed (" + std::to_string(rc_) + ")"; return rc_; } \
    } while (0)
    // cos / sin of this step's positions, one table per frequency set: [T, n_freq] cos, then [T, n_freq] sin
    auto cos_of = [&](int table) { return cs_ + (size_t)T * freq_off_[table]; };
    auto sin_of = [&](int table) { return cs_ + (size_t)T * freq_off_[table] + (size_t)T * freqs_[table].f.size(); };
    for (size_t k = 0; k < freqs_.size(); ++k)
        TX_OP(b200_rope_angles_amp(seq_.d_pos(), T, freqs_[k].dev, (int)freqs_[k].f.size(), freqs_[k].amp, cos_of((int)k), sin_of((int)k), stream_));
    TX_OP(b200_embed_positions(seq_.d_ids(), nullptr, embed_, nullptr, x_, T, D, dt, stream_));
    if (has_loop_) cudaMemcpyAsync(x0_, x_, (size_t)T * D * 4, cudaMemcpyDeviceToDevice, stream_);
    // the residual update of a sublayer boundary, fused with the norm that reads x next (nw NULL: nobody does yet)
    auto boundary = [&](const float* y1, float s1, const float* y2, float s2, bool experts, int top, const float* bcast, const float* nw,
                        void* out) -> int {
        b200_rmsnorm_residual_args ra{};
        ra.x = x_; ra.y1 = y1; ra.s1 = s1; ra.y2 = y2; ra.s2 = s2;
        if (experts) { ra.expert_out = eo_; ra.dest = dest_; ra.weight = weight_; ra.top = top; }
        ra.bcast = bcast;
        ra.w = nw; ra.w_offset = 1.f; ra.eps = eps_; ra.out = out; ra.out_dtype = dt;
        ra.n_rows = T; ra.width = D;
        return b200_rmsnorm_residual(&ra, stream_);
    };
    bool h1_ready = false;
    for (size_t r = 0; r < runs_.size(); ++r) {
        TxRun& R = runs_[r];
        const TxLayer& L = layers_[R.layer];
        const TxAttn& at = L.at;
        if (R.pass >= 0) {   // a pass of the span starts: x += embedding output (not the first pass) + the pass's vector
            TX_OP(boundary(R.pass > 0 ? x0_ : nullptr, 1.f, nullptr, 0.f, false, 0, loop_step_ + (size_t)R.pass * D, L.n1, h1_));
            h1_ready = true;
        }
        if (!h1_ready) TX_OP(boundary(nullptr, 0.f, nullptr, 0.f, false, 0, nullptr, L.n1, h1_));
        TX_OP(gemm(h1_, L.w_in, proj_, B200_F32, T, L.n_in, D));
        // ---- attention: rotation and page stores, scores / softmax / values, head post-processing, W_o
        {
            b200_qk_prepare_args qa{};
            qa.proj = proj_; qa.ld_proj = L.n_in;
            if (at.rot_dims > 0) { qa.cos = cos_of(at.table); qa.sin = sin_of(at.table); }
            qa.rot_dims = at.rot_dims; qa.rot_layout = B200_ROPE_HALF;
            qa.q_out = q_; qa.k_pool = R.k_pool; qa.v_pool = R.v_pool;
            qa.pages = pages; qa.max_pages = max_pages; qa.page_rows = kPageRows;
            qa.slot = seq_.d_slot(); qa.pos = seq_.d_pos(); qa.start = seq_.d_start();
            qa.n_tokens = T; qa.heads = at.heads * at.maps; qa.kv_heads = at.kv_heads * at.maps; qa.dim = at.dim; qa.dtype = dt;
            qa.v_heads = at.kv_heads; qa.vdim = at.vdim; qa.v_off = at.v_off;
            TX_OP(b200_qk_prepare(&qa, stream_));
            const bool post = L.kind != kMixPlain;   // maps are combined, or the heads gated, in fp32
            b200_paged_attention_args pa{};
            pa.q = q_; pa.out = post ? (void*)attf_ : att_; pa.k_pool = R.k_pool; pa.v_pool = R.v_pool;
            pa.pages = pages; pa.max_pages = max_pages; pa.page_rows = kPageRows;
            pa.slot = seq_.d_slot(); pa.pos = seq_.d_pos();
            pa.n_tokens = T; pa.heads = at.heads; pa.kv_heads = at.kv_heads; pa.dim = at.dim; pa.vdim = at.vdim;
            pa.scale = at.scale; pa.softcap = 0.f; pa.denom_bias = 0.f;
            pa.dtype = dt; pa.longest_entry = longest_entry; pa.longest_context = longest_context;
            pa.workspace = attn_ws_; pa.workspace_bytes = attn_ws_bytes_;
            pa.chunk = at.chunk; pa.maps = at.maps; pa.out_f32 = post;
            TX_OP(b200_paged_attention(&pa, stream_));
            if (L.kind == kMixDiff)
                TX_OP(b200_diff_combine(attf_, L.lambda, eps_, 1.f - L.diff, att_, T, at.heads, at.vdim, dt, stream_));
            else if (L.kind == kMixParallel)
                TX_OP(b200_sigmoid_gate(attf_, proj_ + at.g_off, L.n_in, att_, T, at.natt(), dt, stream_));
            TX_OP(gemm(att_, L.o, y_, B200_F32, T, D, at.natt()));
        }
        // ---- the scan beside it
        if (L.kind == kMixParallel) {
            const TxScan& sc = L.sc;
            const float* u = proj_ + sc.in_off;
            b200_conv_act_args ca{};
            ca.u = u; ca.ld_u = L.n_in; ca.w = sc.conv_w; ca.bias = sc.conv_b; ca.taps = sc.taps; ca.conv_state = R.ring.data();
            ca.out32 = xc32_; ca.out = xc_; ca.out_dtype = dt;
            ca.slot = seq_.d_slot(); ca.pos = seq_.d_pos(); ca.start = seq_.d_start();
            ca.n_tokens = T; ca.channels = sc.inner; ca.update_state_inline = longest_entry == 1;
            TX_OP(b200_conv_act(&ca, stream_));
            if (sc.taps > 1 && longest_entry != 1)
                TX_OP(b200_conv_state_update(u, L.n_in, R.ring.data(), seq_.d_slot(), seq_.d_pos(), seq_.d_end(), T, sc.inner, sc.taps, stream_));
            const int nbc = sc.dt_rank + 2 * sc.state;
            TX_OP(gemm(xc_, sc.w_x, bc_, B200_F32, T, nbc, sc.inner));
            {   // dt = softplus(bc[:, 0:dt_rank] W_dt^T + bias): the fp32 columns are the operand as they are (leading dimension nbc)
                b200_gemm_grouped_args g{};
                g.A = bc_; g.lda = nbc; g.W = sc.w_dt; g.ldw = sc.dt_rank; g.trans_b = 1;
                g.epi = B200_GG_BIAS_SOFTPLUS; g.aux = sc.dt_b; g.ld_aux = 0;   // the step sizes leave the GEMM finished
                g.C = dtr_; g.ldc = sc.inner;
                g.M = T; g.N = sc.inner; g.K = sc.dt_rank; g.batch = 1;
                g.a_dtype = B200_F32; g.w_dtype = dt; g.c_dtype = B200_F32;
                TX_OP(b200_gemm_grouped(&g, stream_));
            }
            b200_selective_scan_args sa{};
            sa.x = xc32_; sa.dt_raw = dtr_; sa.dt_ready = 1;
            sa.B = bc_ + sc.dt_rank; sa.C = bc_ + sc.dt_rank + sc.state; sa.ld_bc = nbc;
            sa.z = u + sc.inner; sa.ld_z = L.n_in;
            sa.A = sc.A; sa.D = sc.Dv;
            sa.state = R.state.data(); sa.out = sy_; sa.out_dtype = dt;
            sa.ent_row = seq_.d_ent_row(); sa.ent_len = seq_.d_ent_len(); sa.slot = seq_.d_slot(); sa.pos = seq_.d_pos();
            sa.n_entries = seq_.n_entries; sa.n_tokens = T; sa.channels = sc.inner; sa.n_state = sc.state; sa.longest_entry = longest_entry;
            sa.workspace = attn_ws_; sa.workspace_bytes = attn_ws_bytes_;
            TX_OP(b200_selective_scan(&sa, stream_));
            TX_OP(gemm(sy_, sc.w_o, y2_, B200_F32, T, D, sc.inner));
        }
        // the norm that follows the layer: the next run's mixer input, unless a pass starts there (it adds to x first)
        const TxLayer* next = (r + 1 < runs_.size() && runs_[r + 1].pass < 0) ? &layers_[runs_[r + 1].layer] : nullptr;
        const bool par = L.kind == kMixParallel;
        const float s1 = par ? L.left_scale : 1.f, s2 = par ? L.right_scale : 0.f;
        if (L.ff_kind == kFfNone) {
            TX_OP(boundary(y_, s1, par ? y2_ : nullptr, s2, false, 0, nullptr, next ? next->n1 : nullptr, h1_));
        } else {
            TX_OP(boundary(y_, s1, par ? y2_ : nullptr, s2, false, 0, nullptr, L.n2, h2_));
            if (L.ff_kind == kFfDense) {
                TX_OP(gemm(h2_, L.w_up, act_, dt, T, L.ff, D, B200_GG_RELU2));
                TX_OP(gemm(act_, L.w_down, y_, B200_F32, T, D, L.ff));
                TX_OP(boundary(y_, 1.f, nullptr, 0.f, false, 0, nullptr, next ? next->n1 : nullptr, h1_));
            } else {
                TX_OP(b200_moe_route_logits(h2_, dt, L.router, L.router_b, T, D, L.experts, L.top, chosen_, weight_, stream_));
                TX_OP(b200_moe_dispatch(chosen_, T, L.top, L.experts, group_off_, src_row_, dest_, stream_));
                if (dt == B200_BF16 && !capturing_ && T >= kExpertStreamsFrom && D % 8 == 0 && L.ff % 8 == 0) {
                    const int rc_ = experts_on_side_streams(L, T, err);
                    if (rc_ != B200_OK) return rc_;
                    TX_OP(boundary(nullptr, 0.f, nullptr, 0.f, true, L.top, nullptr, next ? next->n1 : nullptr, h1_));
                    h1_ready = next != nullptr;
                    keep_layer(r, x_, T);
                    continue;
                }
                b200_gemm_grouped_args g{};
                g.A = h2_; g.lda = D; g.a_rows = src_row_; g.group_off = group_off_;
                g.W = L.w_up; g.ldw = D; g.stride_w = (long long)L.ff * D; g.trans_b = 1; g.epi = B200_GG_RELU2;
                g.C = act_; g.ldc = L.ff;
                g.M = T; g.N = L.ff; g.K = D; g.batch = L.experts;   // an expert owns at most one row per token
                g.a_dtype = dt; g.w_dtype = dt; g.c_dtype = dt;
                TX_OP(b200_gemm_grouped(&g, stream_));
                b200_gemm_grouped_args d{};
                d.A = act_; d.lda = L.ff; d.group_off = group_off_;
                d.W = L.w_down; d.ldw = L.ff; d.stride_w = (long long)D * L.ff; d.trans_b = 1;
                d.C = eo_; d.ldc = D;
                d.M = T; d.N = D; d.K = L.ff; d.batch = L.experts;
                d.a_dtype = dt; d.w_dtype = dt; d.c_dtype = B200_F32;
                TX_OP(b200_gemm_grouped(&d, stream_));
                TX_OP(boundary(nullptr, 0.f, nullptr, 0.f, true, L.top, nullptr, next ? next->n1 : nullptr, h1_));
            }
        }
        h1_ready = next != nullptr;
        keep_layer(r, x_, T);
    }
    if (W > 0) {
        b200_rmsnorm_residual_args fa{};
        fa.x = x_; fa.rows = seq_.d_want_rows(); fa.w = fnw_; fa.w_offset = 1.f; fa.eps = eps_; fa.out = hf_; fa.out_dtype = dt;
        fa.n_rows = W; fa.width = D;
        TX_OP(b200_rmsnorm_residual(&fa, stream_));
        TX_OP(gemm(hf_, head_, logits_, B200_F32, W, vocab_, D));
        if (logit_cap_ > 0.f) TX_OP(b200_softcap(logits_, (size_t)W * vocab_, logit_cap_, stream_));
        if (want_ids) TX_OP(b200_argmax(logits_, ids_dev_, W, vocab_, B200_F32, stream_));
    }
    return B200_OK;
#undef TX_OP
}

Model* make_tomalix(const ModelDir& dir, const b200_model_options& opt, std::string& err) {
    Tomalix* m = new Tomalix();
    if (m->load(dir, opt, err) != B200_OK) {
        delete m;
        return nullptr;
    }
    return m;
}

FamilyRegistrar reg_tomalix("Tomalix", make_tomalix);

}  // namespace
}  // namespace b200
