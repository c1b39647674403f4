// Model families behind b200_serve.h: the interface a family implements, the registry that maps config.json's
// "architecture" to a factory, and the batch bookkeeping every family shares (sequence slots, their lengths, the page
// pool of their cache, the per-token slot / position / row tables of a step).
#pragma once
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "b200_serve.h"
#include "json_min.h"
#include "page_pool.h"

namespace b200 {

struct StepEntry {
    int slot;
    int n_tokens;
    const int* tokens;
    int n_want;
    const int* want;   // indices into this entry's tokens
};

struct ModelDir {
    std::string path;
    Json config;
};

// Sequence slots over one PagePool, plus the device tables of a step: for token t of the packed batch its id, slot and
// position, and for every wanted place its row in the batch; for layers that carry state from token to token also the
// position at which the token's sequence starts in this step and its length after it (what is older than the step comes
// from carried state), and per entry its first batch row and its token count; for embeddings that read a pair of tokens,
// the id of the token before it in its sequence (-1 for a sequence's first token; the last id of every slot is kept from
// step to step). Filled on the host (pinned), uploaded with one copy.
class SequenceBatch {
public:
    ~SequenceBatch();
    // page_rows rows per page; the pool holds ceil(max_tokens / page_rows) pages (each sequence rounds up to whole pages)
    int init(int max_tokens, int page_rows, int n_slots, int max_positions, std::string& err);
    // Validates the entries, takes pages, advances the slots' lengths and uploads the tables on `stream`.
    // On failure nothing has changed (B200_ENOMEM: the pool cannot hold the step).
    int begin_step(const std::vector<StepEntry>& entries, cudaStream_t stream, std::string& err);
    int release(int slot);

    PagePool pool;
    int n_slots = 0, max_positions = 0;
    std::vector<int> length;      // tokens cached per slot
    std::vector<int> last_id;     // the slot's newest token (what the next step's first token follows)
    // the step prepared by begin_step
    int n_tokens = 0, n_want = 0;
    const int* d_ids() const { return dev_; }
    const int* d_slot() const { return dev_ + cap_; }
    const int* d_pos() const { return dev_ + 2 * (size_t)cap_; }
    const int* d_want_rows() const { return dev_ + 3 * (size_t)cap_; }
    const int* d_start() const { return dev_ + 4 * (size_t)cap_; }     // per token: position of its entry's first token
    const int* d_end() const { return dev_ + 5 * (size_t)cap_; }       // per token: its sequence's length after the step
    const int* d_ent_row() const { return dev_ + 6 * (size_t)cap_; }   // per entry: first row in the batch
    const int* d_ent_len() const { return dev_ + 7 * (size_t)cap_; }   // per entry: tokens
    const int* d_prev() const { return dev_ + 8 * (size_t)cap_; }      // per token: id of the token before it, -1 at position 0
    int n_entries = 0;

private:
    int ensure_capacity(int tokens);
    static constexpr int kTables = 9;
    int* host_ = nullptr;   // pinned [kTables, cap]
    int* dev_ = nullptr;
    int cap_ = 0;
    cudaEvent_t copied_ = nullptr;   // the upload out of host_ has run (host_ may be rewritten)
};

// State that a layer carries from token to token for each sequence slot (a recurrent state, the last inputs of a short
// convolution): one fp32 block per slot, addressed by the slot index that SequenceBatch hands out. Nothing is cleared
// when a slot changes owner: kernels start from zero whenever a sequence starts at position 0.
class SlotState {
public:
    SlotState() = default;
    SlotState(const SlotState&) = delete;
    SlotState& operator=(const SlotState&) = delete;
    SlotState(SlotState&& o) noexcept : dev_(o.dev_), per_slot_(o.per_slot_) { o.dev_ = nullptr; }
    ~SlotState() { if (dev_) cudaFree(dev_); }
    cudaError_t init(int n_slots, size_t floats_per_slot) {
        per_slot_ = floats_per_slot;
        const size_t bytes = std::max<size_t>(16, (size_t)n_slots * floats_per_slot * sizeof(float));
        cudaError_t e = cudaMalloc(&dev_, bytes);
        if (e == cudaSuccess) e = cudaMemset(dev_, 0, bytes);
        return e;
    }
    float* data() const { return dev_; }
    size_t floats_per_slot() const { return per_slot_; }

private:
    float* dev_ = nullptr;
    size_t per_slot_ = 0;
};

class Model {
public:
    virtual ~Model() {}
    virtual const char* family() const = 0;
    virtual int vocab() const = 0;
    virtual int width() const = 0;
    virtual int layer_count() const = 0;
    // sequence slots and the page pool behind the cache
    virtual int n_slots() const = 0;
    virtual int max_positions() const = 0;
    virtual int page_rows() const = 0;
    virtual int pages_total() const = 0;
    virtual int pages_free() const = 0;
    virtual int slot_length(int slot) const = 0;
    virtual int slot_page_count(int slot) const = 0;
    virtual int slot_pages(int slot, int* out, int max_n) const = 0;
    // entries as ONE batch; logits_out host fp32 [sum n_want, vocab] and ids_out host [sum n_want] may be NULL
    virtual int step(const std::vector<StepEntry>& entries, float* logits_out, int* ids_out, std::string& err) = 0;
    virtual int release(int slot) = 0;
    virtual int capture_layers(int) { return B200_EUNSUPPORTED; }
    virtual int captured_layers(float*, size_t) { return B200_EUNSUPPORTED; }
    virtual int step_launches() const { return 0; }
};

// What the families that serve config.json + model.safetensors checkpoints share around their launch sequence: the
// stream, the sequence batch behind the Model interface, the workspaces that grow with the largest step seen, the copy of
// the residual stream after every layer run, CUDA-graph replay of repeated single-token steps, and the way logits and
// greedy picks reach the host. A family supplies enqueue() (every launch of a step, in order, on stream_: no
// synchronisation, no allocation, so that it can be captured), ensure_scratch() (its own buffers, among them logits_ and
// ids_dev_) and step_workspace_bytes() (what its attention / recurrence kernels want as shared workspace).
class StepRunner : public Model {
public:
    ~StepRunner() override;
    int vocab() const override { return vocab_; }
    int width() const override { return D_; }
    int n_slots() const override { return seq_.n_slots; }
    int max_positions() const override { return seq_.max_positions; }
    int page_rows() const override { return seq_.pool.page_rows(); }
    int pages_total() const override { return seq_.pool.n_pages(); }
    int pages_free() const override { return seq_.pool.free_count(); }
    int slot_length(int slot) const override { return seq_.length[slot]; }
    int slot_page_count(int slot) const override { return seq_.pool.owned(slot); }
    int slot_pages(int slot, int* out, int max_n) const override;
    int step_launches() const override { return launches_; }
    int step(const std::vector<StepEntry>& entries, float* logits_out, int* ids_out, std::string& err) override;
    int release(int slot) override;
    int capture_layers(int on) override { capture_on_ = on != 0; return B200_OK; }
    int captured_layers(float* out, size_t max_floats) override;

protected:
    virtual int enqueue(int T, int W, int longest_entry, int longest_context, bool want_ids, std::string& err) = 0;
    virtual int ensure_scratch(int T, int W) = 0;
    virtual size_t step_workspace_bytes(int T, int n_entries) const = 0;
    // stream_ and the graph switch (B200_NO_GRAPH=1: every step as plain launches)
    int init_runner(std::string& err);
    size_t esz() const { return dtype_ == B200_BF16 ? 2 : 4; }
    void* dalloc(size_t bytes);   // device memory owned until the model closes
    // y[M, N] = A[M, K] W[N, K]^T, contiguous; A and W of the serving dtype: the tcgen05 GEMM when it fits, else the grouped one
    int gemm(const void* A, const void* W, void* C, int c_dt, int M, int N, int K, int epi = B200_GG_NONE, float epi_param = 0.f);
    // the host buffer of the logits follows the largest number of wanted places (called from ensure_scratch)
    int ensure_logits_host(int W);
    void buffers_moved() { ++buffers_epoch_; }   // a buffer that captured launches point into was reallocated
    void keep_layer(size_t run, const float* x, int T);   // inside enqueue, after a layer run

    int dtype_ = B200_BF16, vocab_ = 0, D_ = 0;
    SequenceBatch seq_;
    cudaStream_t stream_ = nullptr;
    void* ws_ = nullptr;        // split-K partials of the weight-streaming GEMM
    size_t ws_bytes_ = 0;
    void* attn_ws_ = nullptr;   // shares of split attention contexts / chunk summaries of a recurrence
    size_t attn_ws_bytes_ = 0;
    float* logits_ = nullptr;   // device, inside the family's scratch
    int* ids_dev_ = nullptr;
    bool capture_on_ = false, capturing_ = false;

private:
    void drop_graphs();
    std::vector<void*> owned_;
    float* logits_host_ = nullptr;
    size_t logits_host_floats_ = 0;
    struct StepGraph { cudaGraphExec_t exec; int launches; };
    std::map<uint64_t, StepGraph> graphs_;
    std::map<uint64_t, int> graph_seen_;
    uint64_t buffers_epoch_ = 0, graph_epoch_ = 0;
    const int* graph_tables_ = nullptr;   // the per-step tables the graphs read
    bool graphs_enabled_ = true;
    float* capture_ = nullptr;
    size_t capture_cap_ = 0;
    int captured_tokens_ = 0, launches_ = 0;
};

using ModelFactory = Model* (*)(const ModelDir& dir, const b200_model_options& opt, std::string& err);
// static registration: one FamilyRegistrar object per family, in the family's own translation unit
struct FamilyRegistrar {
    FamilyRegistrar(const char* architecture, ModelFactory factory);
};

// Continuous-batching greedy generation over any Model (b200_model_generate)
int generate_greedy(Model& m, int n_requests, const int* prompt_ids, const int* lens, int max_new, int eos_id, int chunk,
                    int* out_ids, int* n_generated, std::string& err);

}  // namespace b200
