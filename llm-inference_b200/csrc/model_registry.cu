// Registry of model families, the shared sequence / page bookkeeping, the continuous-batching scheduler with greedy
// sampling, trace sessions, and the b200_model_* C ABI (include/b200_serve.h).
#include "model_registry.h"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <map>

#include "common.cuh"
#include "launch_count.h"

namespace b200 {

static thread_local std::string g_serve_err;
static int serve_fail(const std::string& m, int code = B200_EINVAL) {
    g_serve_err = m;
    return code;
}

struct Family {
    std::string name;
    ModelFactory factory;
};
static std::vector<Family>& families() {
    static std::vector<Family> f;   // constructed on first use: registrars run during static initialisation
    return f;
}
FamilyRegistrar::FamilyRegistrar(const char* architecture, ModelFactory factory) { families().push_back({architecture, factory}); }

// ------------------------------------------------------------------------------------------
// SequenceBatch
// ------------------------------------------------------------------------------------------
SequenceBatch::~SequenceBatch() {
    if (host_) cudaFreeHost(host_);
    if (dev_) cudaFree(dev_);
    if (copied_) cudaEventDestroy(copied_);
}

int SequenceBatch::init(int max_tokens, int page_rows, int slots, int max_pos, std::string& err) {
    if (max_tokens < 1 || page_rows < 1 || slots < 1 || max_pos < 1) { err = "sequence cache: bad sizes"; return B200_EINVAL; }
    n_slots = slots;
    max_positions = max_pos;
    const int n_pages = (max_tokens + page_rows - 1) / page_rows;
    const int per_slot = (max_pos + page_rows - 1) / page_rows;
    const cudaError_t e = pool.init(n_pages, page_rows, slots, per_slot);
    if (e != cudaSuccess) { err = std::string("page pool: ") + cudaGetErrorString(e); return (int)e; }
    length.assign(slots, 0);
    last_id.assign(slots, -1);
    if (cudaEventCreateWithFlags(&copied_, cudaEventDisableTiming) != cudaSuccess) { err = "cudaEventCreate"; return B200_EINVAL; }
    return B200_OK;
}

int SequenceBatch::ensure_capacity(int tokens) {
    if (tokens <= cap_) return B200_OK;
    int cap = std::max(256, cap_);
    while (cap < tokens) cap *= 2;
    if (copied_) cudaEventSynchronize(copied_);
    cudaDeviceSynchronize();   // kernels in flight may still read the old tables
    if (host_) cudaFreeHost(host_);
    if (dev_) cudaFree(dev_);
    host_ = nullptr; dev_ = nullptr; cap_ = 0;
    if (cudaMallocHost(&host_, (size_t)kTables * cap * sizeof(int)) != cudaSuccess) return B200_ENOMEM;
    if (cudaMalloc(&dev_, (size_t)kTables * cap * sizeof(int)) != cudaSuccess) return B200_ENOMEM;
    cap_ = cap;
    return B200_OK;
}

int SequenceBatch::begin_step(const std::vector<StepEntry>& entries, cudaStream_t stream, std::string& err) {
    int total = 0, wants = 0;
    std::vector<int> grow(n_slots, 0);
    for (const StepEntry& en : entries) {
        if (en.slot < 0 || en.slot >= n_slots) { err = "step: slot out of range"; return B200_EINVAL; }
        if (en.n_tokens < 1 || !en.tokens) { err = "step: an entry brings no tokens"; return B200_EINVAL; }
        if (grow[en.slot]) { err = "step: a slot appears twice"; return B200_EINVAL; }
        if (length[en.slot] + en.n_tokens > max_positions) { err = "step: sequence longer than the model's positions"; return B200_EINVAL; }
        for (int k = 0; k < en.n_want; ++k)
            if (en.want[k] < 0 || en.want[k] >= en.n_tokens) { err = "step: wanted place outside the entry"; return B200_EINVAL; }
        grow[en.slot] = en.n_tokens;
        total += en.n_tokens;
        wants += en.n_want;
    }
    // pages: check the whole step before taking any
    int missing = 0;
    for (int b = 0; b < n_slots; ++b)
        if (grow[b]) missing += pool.missing(b, length[b] + grow[b]);
    if (missing > pool.free_count()) {
        err = "step: page pool exhausted (" + std::to_string(pool.n_pages()) + " pages of " + std::to_string(pool.page_rows()) + " rows, " +
              std::to_string(pool.free_count()) + " free, " + std::to_string(missing) + " needed)";
        return B200_ENOMEM;
    }
    int rc = ensure_capacity(std::max(total, wants));
    if (rc != B200_OK) { err = "step: no memory for the batch tables"; return rc; }
    for (int b = 0; b < n_slots; ++b)
        if (grow[b]) pool.ensure(b, length[b] + grow[b]);
    if (copied_) cudaEventSynchronize(copied_);
    int* ids = host_;
    int* slot = host_ + cap_;
    int* pos = host_ + 2 * (size_t)cap_;
    int* rows = host_ + 3 * (size_t)cap_;
    int* start = host_ + 4 * (size_t)cap_;
    int* end = host_ + 5 * (size_t)cap_;
    int* ent_row = host_ + 6 * (size_t)cap_;
    int* ent_len = host_ + 7 * (size_t)cap_;
    int* prev = host_ + 8 * (size_t)cap_;
    int t = 0, w = 0, ne = 0;
    for (const StepEntry& en : entries) {
        for (int k = 0; k < en.n_want; ++k) rows[w++] = t + en.want[k];
        ent_row[ne] = t;
        ent_len[ne++] = en.n_tokens;
        for (int i = 0; i < en.n_tokens; ++i, ++t) {
            ids[t] = en.tokens[i];
            slot[t] = en.slot;
            pos[t] = length[en.slot] + i;
            start[t] = length[en.slot];
            end[t] = length[en.slot] + en.n_tokens;
            prev[t] = i > 0 ? en.tokens[i - 1] : length[en.slot] > 0 ? last_id[en.slot] : -1;
        }
        last_id[en.slot] = en.tokens[en.n_tokens - 1];
        length[en.slot] += en.n_tokens;
    }
    n_tokens = total;
    n_entries = ne;
    n_want = wants;
    cudaError_t e = cudaMemcpyAsync(dev_, host_, (size_t)kTables * cap_ * sizeof(int), cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaEventRecord(copied_, stream);
    if (e == cudaSuccess && pool.dirty()) e = pool.upload(stream);
    if (e != cudaSuccess) { err = std::string("step: upload: ") + cudaGetErrorString(e); return (int)e; }
    return B200_OK;
}

int SequenceBatch::release(int slot) {
    if (slot < 0 || slot >= n_slots) return B200_EINVAL;
    pool.release(slot);
    length[slot] = 0;
    last_id[slot] = -1;
    return B200_OK;
}

// ------------------------------------------------------------------------------------------
// StepRunner
// ------------------------------------------------------------------------------------------
StepRunner::~StepRunner() {
    if (stream_) cudaStreamSynchronize(stream_);
    drop_graphs();
    for (void* p : owned_) cudaFree(p);
    cudaFree(ws_);
    cudaFree(attn_ws_);
    cudaFree(capture_);
    if (logits_host_) cudaFreeHost(logits_host_);
    if (stream_) cudaStreamDestroy(stream_);
}

int StepRunner::init_runner(std::string& err) {
    if (cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking) != cudaSuccess) { err = "no CUDA device: this library has no CPU path"; return B200_EINVAL; }
    const char* e = getenv("B200_NO_GRAPH");
    graphs_enabled_ = !(e && e[0] == '1');
    return B200_OK;
}

void* StepRunner::dalloc(size_t bytes) {
    void* p = nullptr;
    if (cudaMalloc(&p, bytes ? bytes : 16) != cudaSuccess) return nullptr;
    owned_.push_back(p);
    return p;
}

void StepRunner::drop_graphs() {
    for (auto& kv : graphs_) cudaGraphExecDestroy(kv.second.exec);
    graphs_.clear();
}

int StepRunner::slot_pages(int slot, int* out, int max_n) const {
    const int n = std::min(max_n, seq_.pool.owned(slot));
    for (int i = 0; i < n; ++i) out[i] = seq_.pool.list(slot)[i];
    return n;
}

int StepRunner::release(int slot) {
    cudaStreamSynchronize(stream_);   // pages and state change owner only behind the work that reads them
    return seq_.release(slot);
}

int StepRunner::captured_layers(float* out, size_t max_floats) {
    const size_t n = (size_t)layer_count() * captured_tokens_ * D_;
    if (!capture_ || n == 0) return 0;
    if (n > max_floats) return B200_EWORKSPACE;
    cudaStreamSynchronize(stream_);
    if (cudaMemcpy(out, capture_, n * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess) return B200_EINVAL;
    return captured_tokens_;
}

void StepRunner::keep_layer(size_t run, const float* x, int T) {
    if (capture_on_) cudaMemcpyAsync(capture_ + run * (size_t)T * D_, x, (size_t)T * D_ * 4, cudaMemcpyDeviceToDevice, stream_);
}

int StepRunner::ensure_logits_host(int W) {
    const size_t lf = (size_t)W * vocab_;
    if (lf <= logits_host_floats_) return B200_OK;
    if (logits_host_) cudaFreeHost(logits_host_);
    logits_host_ = nullptr;
    logits_host_floats_ = 0;
    if (cudaMallocHost(&logits_host_, lf * 4) != cudaSuccess) return B200_ENOMEM;
    logits_host_floats_ = lf;
    return B200_OK;
}

int StepRunner::gemm(const void* A, const void* W, void* C, int c_dt, int M, int N, int K, int epi, float epi_param) {
    const size_t need = b200_linear_ex_workspace_bytes(M, N, K);
    if (need > ws_bytes_ && !capturing_) {
        cudaStreamSynchronize(stream_);
        ++buffers_epoch_;
        cudaFree(ws_);
        ws_ = nullptr;
        ws_bytes_ = 0;
        if (cudaMalloc(&ws_, need) == cudaSuccess) ws_bytes_ = need;   // without it the call runs with a single split
    }
    return b200_linear_ex2(A, W, C, M, N, K, dtype_, c_dt, epi, epi_param, ws_, ws_bytes_, stream_);
}

int StepRunner::step(const std::vector<StepEntry>& entries, float* logits_out, int* ids_out, std::string& err) {
    if (entries.empty()) return B200_OK;
    const uint64_t launches0 = b200_launch_count();
    int rc = seq_.begin_step(entries, stream_, err);
    if (rc != B200_OK) return rc;
    const int T = seq_.n_tokens, W = seq_.n_want, D = D_;
    if (ensure_scratch(T, std::max(W, 1)) != B200_OK) { err = "step: out of device memory for the scratch buffers"; return B200_ENOMEM; }
    int longest_entry = 0, longest_context = 0;
    for (const StepEntry& en : entries) {
        longest_entry = std::max(longest_entry, en.n_tokens);
        longest_context = std::max(longest_context, seq_.length[en.slot]);
    }
    {   // room for the shares of split contexts (batches of few rows) and for the chunk states of long recurrent entries
        const size_t need = step_workspace_bytes(T, seq_.n_entries);
        if (need > attn_ws_bytes_) {
            cudaStreamSynchronize(stream_);
            ++buffers_epoch_;
            cudaFree(attn_ws_);
            attn_ws_ = nullptr;
            attn_ws_bytes_ = 0;
            if (cudaMalloc(&attn_ws_, need) == cudaSuccess) attn_ws_bytes_ = need;
        }
    }
    if (capture_on_) {
        const size_t need = (size_t)layer_count() * T * D;
        if (capture_cap_ < need) {
            cudaStreamSynchronize(stream_);
            cudaFree(capture_);
            capture_ = nullptr;
            capture_cap_ = 0;
            if (cudaMalloc(&capture_, need * 4) != cudaSuccess) { err = "step: no memory to keep the layers"; return B200_ENOMEM; }
            capture_cap_ = need;
        }
        captured_tokens_ = T;
    }
    // Batches of single tokens repeat their shape step after step: the second time a shape is seen its launch sequence is
    // captured into a CUDA graph, from then on the step is one graph launch (the per-step tables are read through fixed
    // pointers that begin_step refreshes). Anything that moves a buffer drops the graphs.
    const bool want_ids = ids_out != nullptr;
    if (buffers_epoch_ != graph_epoch_ || seq_.d_ids() != graph_tables_) {   // a buffer was reallocated (even to the same address:
        drop_graphs();                                                         // the carving inside it changed)
        graph_epoch_ = buffers_epoch_;
        graph_tables_ = seq_.d_ids();
    }
    const bool graph_ok = graphs_enabled_ && longest_entry == 1 && !capture_on_ && T <= 4096 && W <= 4096;
    const int ctx_bucket = longest_context > 256 ? std::min(16, (longest_context + 127) / 128) : 0;
    const uint64_t key = (uint64_t)T | ((uint64_t)W << 16) | ((uint64_t)ctx_bucket << 32) | ((uint64_t)want_ids << 40);
    rc = B200_OK;
    auto it = graph_ok ? graphs_.find(key) : graphs_.end();
    if (it != graphs_.end()) {
        if (cudaGraphLaunch(it->second.exec, stream_) != cudaSuccess) { err = "step: graph launch failed"; return B200_EINVAL; }
        count_launch(it->second.launches);
    } else if (graph_ok && ++graph_seen_[key] >= 2) {
        const uint64_t before = b200_launch_count();
        capturing_ = true;
        cudaGraph_t g = nullptr;
        if (cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
            rc = enqueue(T, W, longest_entry, longest_context, want_ids, err);
            const cudaError_t ce = cudaStreamEndCapture(stream_, &g);
            capturing_ = false;
            cudaGraphExec_t exec = nullptr;
            if (rc == B200_OK && ce == cudaSuccess && g && cudaGraphInstantiate(&exec, g, 0) == cudaSuccess) {
                graphs_[key] = {exec, (int)(b200_launch_count() - before)};
                if (cudaGraphLaunch(exec, stream_) != cudaSuccess) { err = "step: graph launch failed"; return B200_EINVAL; }
            } else {   // not capturable here: run the launches directly, and do not try again
                cudaGetLastError();
                graphs_enabled_ = false;
                rc = enqueue(T, W, longest_entry, longest_context, want_ids, err);
            }
            if (g) cudaGraphDestroy(g);
        } else {
            capturing_ = false;
            cudaGetLastError();
            graphs_enabled_ = false;
            rc = enqueue(T, W, longest_entry, longest_context, want_ids, err);
        }
    } else
        rc = enqueue(T, W, longest_entry, longest_context, want_ids, err);
    if (rc != B200_OK) return rc;
    if (W > 0) {
        if (logits_out) cudaMemcpyAsync(logits_host_, logits_, (size_t)W * vocab_ * 4, cudaMemcpyDeviceToHost, stream_);
        if (ids_out) cudaMemcpyAsync(ids_out, ids_dev_, (size_t)W * 4, cudaMemcpyDeviceToHost, stream_);
    }
    const cudaError_t e = cudaStreamSynchronize(stream_);
    if (e != cudaSuccess) { err = std::string("step: ") + cudaGetErrorString(e); return (int)e; }
    if (W > 0 && logits_out) memcpy(logits_out, logits_host_, (size_t)W * vocab_ * 4);
    launches_ = (int)(b200_launch_count() - launches0);
    return B200_OK;
}

// ------------------------------------------------------------------------------------------
// scheduler: continuous batching with greedy sampling
// ------------------------------------------------------------------------------------------
int generate_greedy(Model& m, int n_requests, const int* prompt_ids, const int* lens, int max_new, int eos_id, int chunk,
                    int* out_ids, int* n_generated, std::string& err) {
    const int PR = m.page_rows(), n_slots = m.n_slots(), n_pages = m.pages_total();
    struct Live { int req, slot, fed, made, last, pages; };
    std::vector<size_t> start(n_requests + 1, 0);
    for (int r = 0; r < n_requests; ++r) {
        if (lens[r] < 1) { err = "generate: empty prompt"; return B200_EINVAL; }
        if (lens[r] + max_new - 1 > m.max_positions()) { err = "generate: prompt + new tokens exceed the model's positions"; return B200_EINVAL; }
        if ((lens[r] + max_new - 1 + PR - 1) / PR > n_pages) { err = "generate: a request does not fit the page pool"; return B200_ENOMEM; }
        start[r + 1] = start[r] + lens[r];
    }
    for (size_t i = 0; i < (size_t)n_requests * max_new; ++i) out_ids[i] = eos_id;
    if (n_generated) std::fill(n_generated, n_generated + n_requests, 0);
    std::deque<int> waiting;
    for (int r = 0; r < n_requests; ++r) waiting.push_back(r);
    std::vector<Live> live;
    std::vector<char> slot_used(n_slots, 0);
    for (int b = 0; b < n_slots; ++b) slot_used[b] = m.slot_length(b) > 0;   // slots the caller holds stay untouched
    int reserved = 0;   // pages promised to the live requests over their whole life
    for (int b = 0; b < n_slots; ++b) reserved += m.slot_page_count(b);
    int steps = 0;
    std::vector<StepEntry> entries;
    std::vector<int> want_last, ids, dec_tok;
    while (!waiting.empty() || !live.empty()) {
        // admission, first come first served: a slot and pages for the request's whole life
        while (!waiting.empty()) {
            const int r = waiting.front();
            const int need = (lens[r] + max_new - 1 + PR - 1) / PR;
            int slot = -1;
            for (int b = 0; b < n_slots; ++b)
                if (!slot_used[b]) { slot = b; break; }
            if (slot < 0 || reserved + need > n_pages) break;
            slot_used[slot] = 1;
            reserved += need;
            live.push_back({r, slot, 0, 0, 0, need});
            waiting.pop_front();
        }
        if (live.empty()) { err = "generate: nothing can be admitted (slots or pages held elsewhere)"; return B200_ENOMEM; }
        entries.clear();
        want_last.assign(live.size(), 0);
        dec_tok.resize(live.size());
        for (size_t i = 0; i < live.size(); ++i) {
            Live& L = live[i];
            StepEntry en{};
            en.slot = L.slot;
            if (L.fed < lens[L.req]) {   // a portion of the prompt
                const int left = lens[L.req] - L.fed;
                en.n_tokens = chunk > 0 ? std::min(chunk, left) : left;
                en.tokens = prompt_ids + start[L.req] + L.fed;
                if (en.n_tokens == left) { want_last[i] = en.n_tokens - 1; en.n_want = 1; en.want = &want_last[i]; }
            } else {                     // one decoded token
                dec_tok[i] = L.last;
                en.n_tokens = 1;
                en.tokens = &dec_tok[i];
                en.n_want = 1;
                en.want = &want_last[i];
            }
            entries.push_back(en);
        }
        int n_want = 0;
        for (auto& en : entries) n_want += en.n_want;
        ids.assign(std::max(1, n_want), 0);
        const int rc = m.step(entries, nullptr, n_want ? ids.data() : nullptr, err);
        if (rc != B200_OK) return rc > 0 ? -1000 - rc : rc;
        ++steps;
        int w = 0;
        std::vector<Live> next;
        for (size_t i = 0; i < live.size(); ++i) {
            Live L = live[i];
            L.fed += (L.fed < lens[L.req]) ? entries[i].n_tokens : 0;
            bool done = false;
            if (entries[i].n_want) {
                const int id = ids[w++];
                // as the framework's LLaMA loop: the first token is emitted unconditionally, a later eos_id ends the
                // sequence without being emitted
                if (L.made > 0 && eos_id >= 0 && id == eos_id) done = true;
                else {
                    out_ids[(size_t)L.req * max_new + L.made++] = id;
                    L.last = id;
                    if (L.made >= max_new) done = true;
                }
            }
            if (done) {
                if (n_generated) n_generated[L.req] = L.made;
                m.release(L.slot);
                slot_used[L.slot] = 0;
                reserved -= L.pages;
            } else
                next.push_back(L);
        }
        live.swap(next);
    }
    return steps;
}

}  // namespace b200

using namespace b200;

struct b200_model {
    Model* impl;
};
struct b200_session {
    b200_model* m;
    std::map<std::string, int> slot_of;
    std::vector<char> used;
};

extern "C" const char* b200_serve_last_error(void) { return g_serve_err.c_str(); }

extern "C" const char* b200_model_families(void) {
    static std::string s;
    s.clear();
    for (auto& f : families()) s += (s.empty() ? "" : ",") + f.name;
    return s.c_str();
}

extern "C" b200_model* b200_model_open(const char* dir, const b200_model_options* opt) {
    if (!dir || !opt) { serve_fail("model_open: null argument"); return nullptr; }
    ModelDir md;
    md.path = dir;
    const std::string cpath = md.path + "/config.json";
    FILE* f = fopen(cpath.c_str(), "rb");
    if (!f) { serve_fail("model_open: cannot read " + cpath); return nullptr; }
    std::string text;
    char buf[4096];
    size_t n;
    while ((n = fread(buf, 1, sizeof buf, f)) > 0) text.append(buf, n);
    fclose(f);
    std::string err;
    if (!JsonParser::parse(text.data(), text.size(), md.config, err)) { serve_fail(cpath + ": " + err); return nullptr; }
    const std::string arch = md.config.text("architecture");
    for (auto& fam : families()) {
        if (fam.name != arch) continue;
        Model* impl = fam.factory(md, *opt, err);
        if (!impl) { serve_fail(arch + ": " + err); return nullptr; }
        return new b200_model{impl};
    }
    serve_fail("model_open: no family registered for architecture '" + arch + "' (have: " + b200_model_families() + ")", B200_EUNSUPPORTED);
    return nullptr;
}

extern "C" void b200_model_close(b200_model* m) {
    if (!m) return;
    delete m->impl;
    delete m;
}
extern "C" const char* b200_model_family(const b200_model* m) { return m ? m->impl->family() : ""; }
extern "C" int b200_model_vocab(const b200_model* m) { return m ? m->impl->vocab() : 0; }
extern "C" int b200_model_width(const b200_model* m) { return m ? m->impl->width() : 0; }
extern "C" int b200_model_layer_count(const b200_model* m) { return m ? m->impl->layer_count() : 0; }
extern "C" int b200_model_max_positions(const b200_model* m) { return m ? m->impl->max_positions() : 0; }
extern "C" int b200_model_page_rows(const b200_model* m) { return m ? m->impl->page_rows() : 0; }
extern "C" int b200_model_pages_total(const b200_model* m) { return m ? m->impl->pages_total() : 0; }
extern "C" int b200_model_pages_free(const b200_model* m) { return m ? m->impl->pages_free() : 0; }
extern "C" int b200_model_slot_length(const b200_model* m, int slot) {
    if (!m || slot < 0 || slot >= m->impl->n_slots()) return B200_EINVAL;
    return m->impl->slot_length(slot);
}
extern "C" int b200_model_slot_pages(const b200_model* m, int slot, int* out, int max_n) {
    if (!m || !out || slot < 0 || slot >= m->impl->n_slots()) return B200_EINVAL;
    return m->impl->slot_pages(slot, out, max_n);
}

extern "C" int b200_model_step(b200_model* m, int n_entries, const int* slots, const int* n_tokens, const int* tokens,
                               const int* n_want, const int* want, float* logits_out, int* ids_out) {
    if (!m || n_entries < 0 || (n_entries && (!slots || !n_tokens || !tokens))) return serve_fail("model_step: null argument");
    std::vector<StepEntry> entries(n_entries);
    size_t t = 0, w = 0;
    for (int i = 0; i < n_entries; ++i) {
        entries[i].slot = slots[i];
        entries[i].n_tokens = n_tokens[i];
        entries[i].tokens = tokens + t;
        entries[i].n_want = n_want ? n_want[i] : 0;
        entries[i].want = want ? want + w : nullptr;
        if (entries[i].n_want && !want) return serve_fail("model_step: n_want without want");
        t += n_tokens[i] > 0 ? n_tokens[i] : 0;
        w += entries[i].n_want;
    }
    std::string err;
    const int rc = m->impl->step(entries, logits_out, ids_out, err);
    if (rc != B200_OK) g_serve_err = err;
    return rc;
}
extern "C" int b200_model_release(b200_model* m, int slot) { return m ? m->impl->release(slot) : B200_EINVAL; }
extern "C" int b200_model_capture_layers(b200_model* m, int on) { return m ? m->impl->capture_layers(on) : B200_EINVAL; }
extern "C" int b200_model_captured_layers(b200_model* m, float* out, size_t max_floats) {
    return m ? m->impl->captured_layers(out, max_floats) : B200_EINVAL;
}
extern "C" int b200_model_step_launches(const b200_model* m) { return m ? m->impl->step_launches() : 0; }

extern "C" int b200_model_generate(b200_model* m, int n_requests, const int* prompt_ids, const int* lens, int max_new, int eos_id,
                                   int chunk, int* out_ids, int* n_generated) {
    if (!m || n_requests < 1 || !prompt_ids || !lens || max_new < 1 || !out_ids) return serve_fail("model_generate: bad argument");
    std::string err;
    const int rc = generate_greedy(*m->impl, n_requests, prompt_ids, lens, max_new, eos_id, chunk, out_ids, n_generated, err);
    if (rc < 0) g_serve_err = err;
    return rc;
}

extern "C" b200_session* b200_session_create(b200_model* m) {
    if (!m) return nullptr;
    b200_session* s = new b200_session{m, {}, {}};
    s->used.assign(m->impl->n_slots(), 0);
    return s;
}
extern "C" void b200_session_destroy(b200_session* s) { delete s; }
extern "C" int b200_session_slot(b200_session* s, const char* id) {
    if (!s || !id) return B200_EINVAL;
    auto it = s->slot_of.find(id);
    if (it != s->slot_of.end()) return it->second;
    for (size_t b = 0; b < s->used.size(); ++b)
        if (!s->used[b]) {
            s->used[b] = 1;
            s->slot_of[id] = (int)b;
            return (int)b;
        }
    return serve_fail(std::string("session: no free sequence slot for request ") + id, B200_ENOMEM);
}
extern "C" int b200_session_end(b200_session* s, const char* id) {
    if (!s || !id) return B200_EINVAL;
    auto it = s->slot_of.find(id);
    if (it == s->slot_of.end()) return serve_fail(std::string("session: unknown request ") + id);
    const int b = it->second;
    s->slot_of.erase(it);
    s->used[b] = 0;
    return s->m->impl->release(b);
}
