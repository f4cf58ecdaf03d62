// DecoderModel: parts assembled from a model spec, the weights, the cache, and the ONE step function.
//
// `step` takes a batch of sequences, each with its next tokens (all prompts of a batch of unequal lengths in
// one step, then one token each - or any other cut), runs exactly those tokens as one batch from the cache
// that earlier steps left, and returns float32 logits at the wanted places.  Generation, trace replay, the
// benchmark and the tests all call this function; there is no second forward pass.
//
// Reference: forward (one token, fastgguf.c:4648-4907) and forward_chunk / forward_batch (a prompt in chunks of
// 64 with logits for its last token only, :4943-5143), both for one sequence at an explicit position; model_load
// (:4180-4573) builds what the constructor, load_weights and make_cache build here.  Order of work per layer as
// there: norm, q/k/v, rotary, cache write, attention, output projection + residual, norm, gate/up, SiLU-mul,
// down + residual; then the final norm and the head on the wanted rows only (:5113-5117).
#pragma once
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "cache.hpp"
#include "parts.hpp"
#include "safetensors.hpp"

namespace fg {

struct PartSpec {
    std::string kind;
    Json params = Json::object();
    std::map<std::string, std::string> tensors;      // local name -> checkpoint name
};
struct LayerSpec {
    std::string block;
    PartSpec mixer, feed_forward, mixer_norm, feed_forward_norm;
};
struct RunSpec {
    int layer = 0;
    int cache_from = -1;                             // an EARLIER schedule entry whose cache this run reads
};
struct ModelSpec {
    int64_t hidden_size = 0, vocab_size = 0, max_positions = 0;
    PartSpec embedding, final_norm, head;
    std::vector<LayerSpec> layers;
    std::vector<RunSpec> schedule;
    std::vector<int> stop_token_ids;
    std::vector<std::string> ignored_tensors;        // regular expressions of tensors that may be present unused
    static ModelSpec from_json(const Json &j);       // validates the schedule
};

struct ExpectedTensor {
    std::vector<int64_t> shape;
    bool is_int = false;
    int init = 0;
    float std = 0.02f;
};

class TensorSource;
// Checks a source against the parts' declarations - ONE error lists missing, unexpected and wrongly shaped tensors -
// and returns the dtype each tensor takes on the device under the dtype policy.
std::map<std::string, int> check_source(const TensorSource &source, const std::map<std::string, ExpectedTensor> &expected,
                                        const std::vector<std::string> &ignored_tensors, int engine_dtype);

// One entry of a step: a slot, its next tokens, the places among them whose logits are wanted.
struct StepEntry {
    int slot = 0;
    const int *tokens = nullptr;
    int n_tokens = 0;
    std::vector<int> want;
};

class DecoderModel {
public:
    DecoderModel(const ModelSpec &spec, int dtype, int device, cudaStream_t stream);
    ~DecoderModel();
    DecoderModel(const DecoderModel &) = delete;

    // checkpoint name -> what the parts declare
    const std::map<std::string, ExpectedTensor> &expected_tensors() const { return expected_; }
    // Checks the source against the parts' declarations - ONE error lists missing, unexpected and wrongly shaped
    // tensors - then brings every tensor to the device under the dtype policy and hands it to its parts.
    // seed_random: no source; values from the seeded generator.
    void load_weights(const TensorSource *source, bool seed_random, uint64_t seed);
    int64_t weight_bytes() const { return weight_bytes_; }

    // max_tokens: the most tokens live sequences hold at any time, each rounded up to a page
    void make_cache(int64_t max_tokens, int n_slots, int max_seq_len, int page_size, bool verbose);
    int acquire_slot();
    void release_slot(int slot);

    // Runs the step; float32 logits [wanted, vocab] on the device (undefined tensor if none wanted), valid until
    // the next step.  Validation comes before any launch; on error nothing has changed.
    Tensor step(const std::vector<StepEntry> &entries);
    // The layers over a prepared batch (pages reserved, integers on the device), activations from rt.arena.
    Tensor forward(Runtime &rt, const Batch &batch);
    // ONE schedule entry's block on rows given by the caller (x: [rows, hidden] float32 on the host, updated in place),
    // through the real cache: pages are reserved and committed as in a step.  For tests of a part alone.
    void block_forward(int entry, const std::vector<std::pair<int, int>> &steps, float *x_host);

    ModelSpec spec;
    Runtime runtime;                                 // the step path's runtime (its arena is reset per step)
    std::unique_ptr<PagedKVCache> cache;
    std::unique_ptr<StatePool> state;
    std::vector<LayerIO> io;                         // per schedule entry
    Json describe() const;

private:
    Part *build(int role, const PartSpec &ps);
    Part *nested(int role, const Json &nested_spec);
    void bind(Part *part, const PartSpec &ps);
    void build_batch(const std::vector<StepEntry> &entries, Batch &batch);

    std::vector<std::unique_ptr<Part>> owned_;
    std::map<std::string, Part *> shared_;           // nested parts by (role, kind, params)
    struct Bound { Part *part; std::map<std::string, std::string> names; };
    std::vector<Bound> bound_;
    Embedding *embedding_ = nullptr;
    Head *head_ = nullptr;
    Norm *final_norm_ = nullptr;
    std::vector<std::unique_ptr<Block>> blocks_;     // per layer
    std::vector<Mixer *> mixers_;                    // per layer
    std::map<std::string, ExpectedTensor> expected_;
    int64_t weight_bytes_ = 0;
    Arena step_arena_;
    // pinned staging for the integers of a step: a few buffers in turn, each guarded by an event
    struct Staging { int *host = nullptr; size_t cap = 0; cudaEvent_t done = nullptr; };
    std::vector<Staging> staging_;
    size_t next_staging_ = 0;
};

}  // namespace fg
