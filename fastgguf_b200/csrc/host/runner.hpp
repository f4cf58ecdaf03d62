// Sampling state, the generation loop, and the graph-replayed decode path that serving uses.
//
// The loop for one sequence in the reference (fastgguf.c:5284-5309): run the prompt, then repeat { sample; if
// the token is a stop token, end WITHOUT emitting, feeding or recording it (:5296); emit; if the context is
// full, end (:5300); run the token }.  max_tokens <= 0 means until a stop token or a full context (:5294).
// Here a batch starts together: one step with all prompts (logits at each prompt's last token), then one token
// per live sequence a step; a sequence that finishes leaves the step list and its slot goes back when the batch
// ends, so the next batch uses it again.
//
// Plain path: run_batch over an abstract backend (acquire / release / step / sample / room) - one step and one
// device->host read of the sampled tokens per step; a fake backend tests the decisions without a GPU.
// Graph path: the decode step of a batch - the model's layers, the sampler and the feedback of the sampled
// tokens into the next step's inputs - is recorded once per batch-size bucket as a CUDA graph over fixed
// buffers and replayed.  Tokens and positions stay on the device; the host only reserves pages (its
// bookkeeping is deterministic), uploads page-table entries when a sequence crosses a page, replays, and reads
// the sampled tokens one step late to decide about stop tokens.  A sequence that drew a stop token is therefore
// fed for one more step; that step's output for it is dropped.  Rows of finished sequences and padding rows
// point at the reserved page 0 and at the spare state row, so they change nothing that is read.
#pragma once
#include <deque>
#include <list>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "model.hpp"

namespace fg {

struct SamplingParams {
    float temp = 1.0f;
    int top_k = 64;
    float top_p = 0.95f;
    float repeat_penalty = 1.0f;
    int repeat_last_n = 64;
    uint64_t seed = 0;
    void validate() const;
    bool greedy() const { return temp <= 0.0f; }
    bool penalizes() const { return repeat_penalty > 0.0f && repeat_penalty != 1.0f && repeat_last_n > 0; }
};

// 0 means "from the clock"; the state of xorshift64* must never be zero (fastgguf.c:5232-5233).
uint64_t resolve_seed(uint64_t seed);
// Generator state of request `index` of a call seeded with `seed` (already resolved): the first request starts
// from the seed itself, as the reference's single conversation does; request i > 0 from a mix of (seed, i).
uint64_t request_seed(uint64_t seed, uint64_t index);

struct Completion {
    int prompt_len = 0;
    std::vector<int> tokens;
    int finish_reason = 0;            // 1 = stop, 2 = length
};

std::vector<std::pair<int, int>> plan_batches(int n_requests, int batch_size);

// What the loop needs from whoever runs the model.
class LoopBackend {
public:
    virtual ~LoopBackend() = default;
    virtual int acquire(int request_index, const int *prompt, int prompt_len) = 0;
    virtual void release(int slot) = 0;
    // one step: sequence i in slots[i] brings n_tok[i] tokens; logits are wanted at each sequence's last token
    virtual void step(const std::vector<int> &slots, const std::vector<int> &n_tok, const std::vector<int> &tokens) = 0;
    virtual std::vector<int> sample(const std::vector<int> &slots) = 0;
    virtual int room(int slot) = 0;
};

using TokenCallback = void (*)(void *user, int request_index, int token);

std::vector<Completion> run_batch(LoopBackend &backend, const std::vector<std::vector<int>> &prompts, int first_index,
                                  int max_tokens, const std::vector<int> &stop_ids, TokenCallback on_token, void *user);

// The graph path's host loop over an abstract batch: tokens are seen one step late.
class LateSession {
public:
    virtual ~LateSession() = default;
    virtual const std::vector<int> &first() const = 0;          // the tokens sampled from the prompts
    virtual int advance(const std::vector<int> &live) = 0;      // one decode step; a handle for its tokens
    virtual const int *wait(int handle) = 0;                    // the sampled tokens of all rows of that step
};
std::vector<Completion> run_batch_late(LateSession &session, const std::vector<int> &prompt_lens, int first_index, int max_tokens,
                                       const std::vector<int> &stop_ids, int max_seq_len, TokenCallback on_token, void *user);

class Engine;

// Device state of a sampler for n_slots sequences (one row per cache slot, plus a spare row that padded rows of a
// fixed-shape step use): an xorshift64* generator (fastgguf.c:3334-3339) and the ring of recent tokens for the
// repeat penalty per sequence, so that what a sequence draws does not depend on its batch-mates.
class Sampler {
public:
    Sampler(const SamplingParams &p, int n_slots, const std::vector<int> &stop_ids, cudaStream_t stream);
    // give a sequence its generator state and the tail of its prompt as history
    void begin(int row, uint64_t state, const int *prompt, int prompt_len);
    // one token per row of logits ([B, V] f32, modified in place by the repeat penalty); rows[b] (device) = state row
    void sample(float *logits, int B, int V, int ldl, const int *rows_dev, int *out_dev, cudaStream_t s);
    SamplingParams params;
    int spare_row;

private:
    int n_rows_, hist_cap_;
    bool use_hist_;
    cudaStream_t stream_;
    DeviceBuffer rng_, hist_, hist_count_, stop_, scratch_;
    int n_stop_ = 0;
};

// Fixed buffers and the recorded decode step for `width` rows.
class DecodeGraph {
public:
    DecodeGraph(Engine &e, Sampler &sampler, int width);
    ~DecodeGraph();
    void replay();
    int width, table_width;
    long long launches_per_step = 0;
    // device views
    int *tokens, *positions, *row_seq, *cu_rows, *rows, *want, *active, *next_tokens, *spare_cell;
    std::vector<int *> tables;
    // pinned host memory, a few regions in turn, each guarded by an event: the sampled tokens of a step on their
    // way to the host, and the page-table entries of a step on their way to the device (copies from pageable
    // memory would make the host wait for the stream at every step)
    struct Region { int *tokens = nullptr; int *upload = nullptr; cudaEvent_t done = nullptr; };
    std::vector<Region> regions;
    int next_region = 0;
    size_t upload_cap = 0;

private:
    void run(cudaStream_t s, bool recording);
    Engine &engine_;
    Sampler &sampler_;
    Arena arena_;
    DeviceBuffer ints_;
    Batch batch_;
    cudaGraph_t graph_ = nullptr;
    cudaGraphExec_t exec_ = nullptr;
};

// Sampler state and recorded graphs for one set of sampling options (kept, so that a second call with the same
// options replays the graphs of the first).  The seed is NOT part of the key: it only enters through begin().
class SamplingBackend : public LoopBackend {
public:
    SamplingBackend(Engine &e, const SamplingParams &p, const std::vector<int> &stop_ids);
    int acquire(int request_index, const int *prompt, int prompt_len) override;
    void release(int slot) override;
    void step(const std::vector<int> &slots, const std::vector<int> &n_tok, const std::vector<int> &tokens) override;
    std::vector<int> sample(const std::vector<int> &slots) override;
    int room(int slot) override;
    DecodeGraph &graph(int width);

    Engine &engine;
    Sampler sampler;
    uint64_t seed = 0;
    std::vector<int> stop_ids;
    Tensor last_logits;
    std::map<int, std::unique_ptr<DecodeGraph>> graphs;
};

// One batch on the graph path: the prompt step, then advance(live) once per decode step.
class DecodeSession : public LateSession {
public:
    DecodeSession(SamplingBackend &backend, const std::vector<std::vector<int>> &prompts, int first_index);
    ~DecodeSession() override;
    const std::vector<int> &first() const override { return first_tokens; }
    // One decode step for the sequences `live` (indices into the batch).  Returns the index of the pinned host
    // buffer that receives the sampled tokens of all rows; wait(index) blocks until they are there.
    int advance(const std::vector<int> &live) override;
    const int *wait(int index) override;
    void close();
    std::vector<int> slots;
    std::vector<int> first_tokens;
    DecodeGraph *graph = nullptr;

private:
    SamplingBackend &backend_;
    int n_;
    std::vector<int> widths_;                    // page-table entries of each row already uploaded (-1: retired)
};

struct EngineOptions {
    int dtype = FG_BF16, max_batch = 64, max_seq_len = 0, device = 0;
    int64_t max_tokens = 8192;
    bool use_graphs = true, verbose = false;
    cudaStream_t stream = nullptr;
};

// A loaded model with its cache: what every program drives.
class Engine {
public:
    Engine(const ModelSpec &spec, const EngineOptions &opts, const TensorSource *source, bool seed_random, uint64_t seed);
    ~Engine();
    std::vector<Completion> generate(const std::vector<std::vector<int>> &prompts, const SamplingParams &params, int max_tokens,
                                     const std::vector<int> &stop_ids, int batch_size, int use_graphs, TokenCallback on_token, void *user);
    SamplingBackend &backend(const SamplingParams &params, const std::vector<int> &stop_ids);
    std::vector<Completion> run_batch_graphs(SamplingBackend &b, const std::vector<std::vector<int>> &prompts, int first_index,
                                             int max_tokens, const std::vector<int> &stop_ids, TokenCallback on_token, void *user);
    void check_device(const char *where);            // synchronises, then raises if a bounded wait ran out

    EngineOptions opts;
    std::unique_ptr<DecoderModel> model;
    cudaStream_t stream = nullptr, capture_stream = nullptr;
    bool own_stream = false;
    struct Stats { long long steps = 0, h2d_bytes = 0, d2h_bytes = 0, launches_per_step = 0, graphs = 0; } stats;
    size_t backend_count() const { return backends_.size(); }        // sets of sampling options kept with their graphs

private:
    std::list<std::pair<std::string, std::unique_ptr<SamplingBackend>>> backends_;   // most recently used first
};

static const int kBuckets[] = {1, 2, 4, 8, 16, 32, 64, 128, 256};
int bucket_for(int n);

}  // namespace fg
