// See model.hpp.
#include "model.hpp"

#include <cstdlib>

#include <algorithm>
#include <cstring>
#include <regex>
#include <set>

namespace fg {

// ------------------------------------------------------------------------------------ spec
static PartSpec part_spec_from_json(const Json &j, const char *what) {
    if (!j.is_object() || !j.get("kind").is_string()) fail(FG_E_CONFIG, format("model spec: '%s' must be {\"kind\": ..., \"params\": ..., \"tensors\": ...}", what));
    PartSpec p;
    p.kind = j.get("kind").as_string();
    if (j.get("params").is_object()) p.params = j.get("params");
    const Json &t = j.get("tensors");
    if (t.is_object())
        for (auto &m : t.members()) {
            if (!m.second.is_string()) fail(FG_E_CONFIG, format("model spec: tensor name of '%s.%s' must be a string", what, m.first.c_str()));
            p.tensors[m.first] = m.second.as_string();
        }
    return p;
}

ModelSpec ModelSpec::from_json(const Json &j) {
    if (!j.is_object()) fail(FG_E_CONFIG, "model spec: must be a JSON object");
    ModelSpec s;
    s.hidden_size = param_int(j, "hidden_size", "model spec");
    s.vocab_size = param_int(j, "vocab_size", "model spec");
    s.max_positions = param_int(j, "max_positions", "model spec");
    if (s.hidden_size <= 0 || s.vocab_size <= 0 || s.max_positions <= 0) fail(FG_E_CONFIG, "model spec: sizes must be positive");
    s.embedding = part_spec_from_json(j.get("embedding"), "embedding");
    s.final_norm = part_spec_from_json(j.get("final_norm"), "final_norm");
    s.head = part_spec_from_json(j.get("head"), "head");
    if (!j.get("layers").is_array() || !j.get("schedule").is_array()) fail(FG_E_CONFIG, "model spec: 'layers' and 'schedule' must be lists");
    for (auto &l : j.get("layers").items()) {
        LayerSpec ls;
        if (!l.is_object() || !l.get("block").is_string()) fail(FG_E_CONFIG, "model spec: a layer needs a 'block' kind");
        ls.block = l.get("block").as_string();
        ls.mixer = part_spec_from_json(l.get("mixer"), "mixer");
        ls.feed_forward = part_spec_from_json(l.get("feed_forward"), "feed_forward");
        ls.mixer_norm = part_spec_from_json(l.get("mixer_norm"), "mixer_norm");
        ls.feed_forward_norm = part_spec_from_json(l.get("feed_forward_norm"), "feed_forward_norm");
        s.layers.push_back(std::move(ls));
    }
    for (auto &r : j.get("schedule").items()) {
        RunSpec rs;
        if (r.is_int()) rs.layer = (int)r.as_int();
        else if (r.is_object() && r.get("layer").is_int()) {
            rs.layer = (int)r.get("layer").as_int();
            if (r.get("cache_from").is_int()) rs.cache_from = (int)r.get("cache_from").as_int();
        } else fail(FG_E_CONFIG, "model spec: a schedule entry is {\"layer\": i, \"cache_from\": j or null}");
        s.schedule.push_back(rs);
    }
    for (size_t i = 0; i < s.schedule.size(); i++) {
        const RunSpec &run = s.schedule[i];
        if (run.layer < 0 || run.layer >= (int)s.layers.size())
            fail(FG_E_CONFIG, format("schedule[%zu] names layer %d, but there are %zu layers", i, run.layer, s.layers.size()));
        if (run.cache_from >= 0) {
            if (run.cache_from >= (int)i) fail(FG_E_CONFIG, format("schedule[%zu].cache_from must name an earlier entry, got %d", i, run.cache_from));
            if (s.schedule[(size_t)run.cache_from].cache_from >= 0)
                fail(FG_E_CONFIG, format("schedule[%zu].cache_from names entry %d, which owns no cache", i, run.cache_from));
        }
    }
    if (j.get("stop_token_ids").is_array())
        for (auto &t : j.get("stop_token_ids").items())
            if (t.is_int()) s.stop_token_ids.push_back((int)t.as_int());
    if (j.get("ignored_tensors").is_array())
        for (auto &t : j.get("ignored_tensors").items())
            if (t.is_string()) s.ignored_tensors.push_back(t.as_string());
    return s;
}

// ------------------------------------------------------------------------------------ building
DecoderModel::DecoderModel(const ModelSpec &spec_, int dtype, int device, cudaStream_t stream) : spec(spec_) {
    if (dtype != FG_BF16 && dtype != FG_F32) fail(FG_E_USAGE, "the engine runs in bfloat16 or float32");
    runtime.dtype = dtype;
    runtime.device = device;
    runtime.stream = stream;
    runtime.arena = &step_arena_;
    int n_sm = 0;
    FG_CUDA(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, device));
    runtime.n_sm = n_sm;
    // FASTGGUF_PLAIN_KERNELS=1: the any-size FMA kernels everywhere - the same results up to rounding, slower; a safety
    // switch in the manner of the reference's FASTGGUF_BATCH=0 (fastgguf.c:5126-5127).  Read when an engine is made.
    const char *plain = getenv("FASTGGUF_PLAIN_KERNELS");
    runtime.plain_kernels = plain && plain[0] == '1';
    embedding_ = dynamic_cast<Embedding *>(build(FG_ROLE_EMBEDDING, spec.embedding));
    for (auto &layer : spec.layers) {
        Mixer *mixer = dynamic_cast<Mixer *>(build(FG_ROLE_MIXER, layer.mixer));
        FeedForward *ffn = dynamic_cast<FeedForward *>(build(FG_ROLE_FEED_FORWARD, layer.feed_forward));
        Norm *n1 = dynamic_cast<Norm *>(build(FG_ROLE_NORM, layer.mixer_norm));
        Norm *n2 = dynamic_cast<Norm *>(build(FG_ROLE_NORM, layer.feed_forward_norm));
        std::unique_ptr<Block> b = build_block(layer.block, runtime);
        b->mixer = mixer; b->feed_forward = ffn; b->mixer_norm = n1; b->feed_forward_norm = n2;
        blocks_.push_back(std::move(b));
        mixers_.push_back(mixer);
    }
    final_norm_ = dynamic_cast<Norm *>(build(FG_ROLE_NORM, spec.final_norm));
    head_ = dynamic_cast<Head *>(build(FG_ROLE_HEAD, spec.head));
    if (!embedding_ || !final_norm_ || !head_) fail(FG_E_INTERNAL, "a part was registered under the wrong role");
    // checkpoint name -> declaration, over every part
    for (auto &b : bound_) {
        for (auto &d : b.part->tensor_decls()) {
            auto it = b.names.find(d.name);
            if (it == b.names.end())
                fail(FG_E_CONFIG, "a part declares tensor '" + d.name + "' but the architecture gives no checkpoint name for it");
            ExpectedTensor e{d.shape, d.is_int, d.init, d.std};
            auto have = expected_.find(it->second);
            if (have != expected_.end()) {
                if (have->second.shape != d.shape)
                    fail(FG_E_CONFIG, "tensor '" + it->second + "' is used with shapes " + shape_text(have->second.shape) + " and " + shape_text(d.shape));
            } else expected_[it->second] = e;
        }
    }
    staging_.resize(4);
}

DecoderModel::~DecoderModel() {
    for (auto &s : staging_) {
        if (s.host) cudaFreeHost(s.host);
        if (s.done) cudaEventDestroy(s.done);
    }
}

Part *DecoderModel::nested(int role, const Json &ns) {
    if (!ns.is_object() || !ns.get("kind").is_string()) fail(FG_E_CONFIG, "a nested part must be {\"kind\": ..., \"params\": ...}");
    std::string key = std::to_string(role) + ":" + ns.get("kind").as_string() + ":" + ns.get("params").dump();
    auto it = shared_.find(key);
    if (it != shared_.end()) return it->second;
    PartSpec ps;
    ps.kind = ns.get("kind").as_string();
    if (ns.get("params").is_object()) ps.params = ns.get("params");
    Part *p = build(role, ps);
    shared_[key] = p;
    return p;
}

Part *DecoderModel::build(int role, const PartSpec &ps) {
    BuildContext ctx;
    ctx.nested = [this](int r, const Json &n) { return nested(r, n); };
    std::unique_ptr<Part> part = build_part(role, ps.kind, runtime, ps.params, ctx);
    Part *raw = part.get();
    owned_.push_back(std::move(part));
    bound_.push_back({raw, ps.tensors});
    return raw;
}

// ------------------------------------------------------------------------------------ weights
// dtype policy: in the bfloat16 engine, float tensors stored in 16 bits become bfloat16; a tensor stored in 32
// bits stays float32 (the plain contraction kernel takes mixed operands); integer tables become int32.  In the
// float32 engine every float tensor is widened to float32, which is exact for bfloat16 and float16 sources.
static int target_dtype(int stored, bool is_int, int engine_dtype) {
    if (is_int) return FG_I32;
    if (engine_dtype == FG_F32 || stored == FG_F32) return FG_F32;
    return FG_BF16;
}

static std::string join(const std::vector<std::string> &v, const char *sep) {
    std::string s;
    for (size_t i = 0; i < v.size(); i++) s += (i ? sep : "") + v[i];
    return s;
}

// Everything that is wrong, in ONE error (the reference prints "missing tensor: NAME" per tensor and fails after the
// loop, fastgguf.c:4154-4164, :4387; shapes that do not fit are errors, :4309-4314).  Returns the dtype each
// expected tensor takes on the device.
std::map<std::string, int> check_source(const TensorSource &source, const std::map<std::string, ExpectedTensor> &expected,
                                        const std::vector<std::string> &ignored_tensors, int engine_dtype) {
    std::vector<std::string> names = source.names(), missing, unexpected, wrong;
    std::set<std::string> have(names.begin(), names.end());
    std::vector<std::regex> ignore;
    for (auto &p : ignored_tensors) ignore.emplace_back(p);
    for (auto &kv : expected)
        if (!have.count(kv.first)) missing.push_back(kv.first);
    for (auto &n : have) {
        if (expected.count(n)) continue;
        bool ignored = false;
        for (auto &r : ignore) ignored = ignored || std::regex_match(n, r);
        if (!ignored) unexpected.push_back(n);
    }
    std::map<std::string, int> target;
    for (auto &kv : expected) {
        const TensorInfo *t = source.find(kv.first);
        if (!t) continue;
        if (t->shape != kv.second.shape)
            wrong.push_back(kv.first + " is " + shape_text(t->shape) + ", the configuration needs " + shape_text(kv.second.shape));
        else if (kv.second.is_int && dtype_is_float(t->dtype))
            wrong.push_back(kv.first + " is " + dtype_long_name(t->dtype) + ", an integer table is needed");
        else if (!kv.second.is_int && !dtype_is_float(t->dtype))
            wrong.push_back(kv.first + " is " + dtype_long_name(t->dtype) + ", a float tensor is needed");
        else target[kv.first] = target_dtype(t->dtype, kv.second.is_int, engine_dtype);
    }
    if (!missing.empty() || !unexpected.empty() || !wrong.empty()) {
        std::string msg = source.where() + ": the weights do not fit the configuration";
        if (!missing.empty()) msg += format("\n  missing tensors (%zu): ", missing.size()) + join(missing, ", ");
        if (!unexpected.empty()) msg += format("\n  unexpected tensors (%zu): ", unexpected.size()) + join(unexpected, ", ");
        if (!wrong.empty()) msg += format("\n  wrong shapes or types (%zu): ", wrong.size()) + join(wrong, "; ");
        fail(FG_E_WEIGHTS, msg);
    }
    return target;
}

void DecoderModel::load_weights(const TensorSource *source, bool seed_random, uint64_t seed) {
    cudaStream_t s = runtime.stream;
    if (!seed_random) check_source(*source, expected_, spec.ignored_tensors, runtime.dtype);
    std::map<std::string, Weight> store;
    weight_bytes_ = 0;
    DeviceBuffer raw;                                  // staging for tensors that need a conversion
    for (auto &kv : expected_) {
        const ExpectedTensor &e = kv.second;
        int64_t rows = 1, cols = 1;
        if (e.shape.size() == 1) cols = e.shape[0];
        else if (e.shape.size() >= 2) {
            cols = e.shape.back();
            for (size_t i = 0; i + 1 < e.shape.size(); i++) rows *= e.shape[i];
        }
        Weight w;
        if (seed_random) {
            int dt = target_dtype(runtime.dtype, e.is_int, runtime.dtype);
            w = make_weight(rows, cols, dt, kv.first.c_str());
            dev_fill_random(w.t.data, dt, rows * cols, seed, name_hash64(kv.first), e.init, e.std, s);
        } else {
            const TensorInfo *t = source->find(kv.first);
            int dt = target_dtype(t->dtype, e.is_int, runtime.dtype);
            w = make_weight(rows, cols, dt, kv.first.c_str());
            if (t->nbytes() > 0) {
                if (dt == t->dtype) {
                    FG_CUDA(cudaMemcpyAsync(w.t.data, t->data, (size_t)t->nbytes(), cudaMemcpyHostToDevice, s));
                } else {
                    if (raw.bytes() < (size_t)t->nbytes()) {
                        FG_CUDA(cudaStreamSynchronize(s));
                        raw = DeviceBuffer((size_t)t->nbytes(), "weight staging");
                    }
                    FG_CUDA(cudaMemcpyAsync(raw.get(), t->data, (size_t)t->nbytes(), cudaMemcpyHostToDevice, s));
                    dev_convert(raw.get(), t->dtype, w.t.data, dt, rows * cols, s);
                }
            }
        }
        weight_bytes_ += (int64_t)w.buffer->bytes();
        store[kv.first] = std::move(w);
    }
    FG_CUDA(cudaStreamSynchronize(s));
    int64_t fused_bytes = 0;
    (void)fused_bytes;
    for (auto &b : bound_) {
        std::map<std::string, Weight> mine;
        for (auto &d : b.part->tensor_decls()) mine[d.name] = store.at(b.names.at(d.name));
        b.part->load(mine, runtime);
    }
    FG_CUDA(cudaStreamSynchronize(s));
    // `store` goes away here: tensors that parts replaced by fused matrices are freed, the others live on in their parts
}

// ------------------------------------------------------------------------------------ cache
void DecoderModel::make_cache(int64_t max_tokens, int n_slots, int max_seq_len, int page_size, bool verbose) {
    if (max_tokens <= 0 || n_slots <= 0 || page_size <= 0) fail(FG_E_USAGE, "max_tokens, max_batch and the page size must be positive");
    int64_t limit = spec.max_positions;
    int64_t rounded = (max_tokens + page_size - 1) / page_size * page_size;
    int64_t msl = std::min(limit, std::min<int64_t>(max_seq_len > 0 ? max_seq_len : limit, rounded));
    std::map<int, CacheRequest> cache_req;
    std::map<int, int64_t> state_req;
    for (size_t i = 0; i < spec.schedule.size(); i++) {
        Mixer *m = mixers_[(size_t)spec.schedule[i].layer];
        CacheRequest r;
        bool wants = m->cache_request(&r);
        if (spec.schedule[i].cache_from < 0 && wants) cache_req[(int)i] = r;
        if (spec.schedule[i].cache_from >= 0) {
            // a borrowed cache must be of the shape the borrower reads
            Mixer *owner = mixers_[(size_t)spec.schedule[(size_t)spec.schedule[i].cache_from].layer];
            CacheRequest ro;
            if (!wants || !owner->cache_request(&ro) || !(ro == r))
                fail(FG_E_CONFIG, format("schedule[%zu] reads the cache of entry %d, whose mixer keeps different keys and values", i,
                                         spec.schedule[i].cache_from));
        }
        if (m->state_bytes() > 0) state_req[(int)i] = m->state_bytes();
    }
    cache = std::make_unique<PagedKVCache>(cache_req, max_tokens, (int)msl, n_slots, page_size);
    if (verbose) {
        // the reference prints kv_mem at load (fastgguf.c:4561-4565)
        fprintf(stderr, "[cache] slots=%d pages=%d page=%d max_seq_len=%d bytes/token=%lld bytes=%lld (%.1f MiB) dtype=%s\n", n_slots,
                cache->groups.empty() ? 0 : cache->groups[0].n_pages - 1, page_size, (int)msl, (long long)cache->bytes_per_token(runtime.dtype),
                (long long)cache->pool_bytes(runtime.dtype), cache->pool_bytes(runtime.dtype) / 1048576.0, dtype_long_name(runtime.dtype));
    }
    cache->allocate(runtime.dtype);
    state = std::make_unique<StatePool>(state_req, n_slots, true);
    io.clear();
    for (size_t i = 0; i < spec.schedule.size(); i++) {
        const RunSpec &run = spec.schedule[i];
        int owner = run.cache_from < 0 ? (int)i : run.cache_from;
        LayerIO l;
        l.write_cache = run.cache_from < 0;
        l.state = state->of((int)i);
        l.state_bytes = state->bytes_of((int)i);
        l.n_slots = n_slots;
        l.page_size = page_size;
        l.cache_dtype = runtime.dtype;
        auto it = cache->group_of_entry.find(owner);
        if (it != cache->group_of_entry.end()) {
            CacheGroup &g = cache->groups[(size_t)it->second];
            l.group = it->second;
            l.k_pool = g.k_pools[owner];
            l.v_pool = g.v_pools[owner];
            l.n_pages = g.n_pages;
            l.n_kv_heads = g.request.n_kv_heads;
            l.head_dim = g.request.head_dim;
        }
        io.push_back(l);
    }
    for (Mixer *m : mixers_) m->prepare(runtime, (int)msl);
}

int DecoderModel::acquire_slot() {
    if (!cache) fail(FG_E_USAGE, "the engine has no cache yet");
    int s = cache->acquire();
    state->reset(s, runtime.stream);
    return s;
}

void DecoderModel::release_slot(int s) { cache->release(s); }

// ------------------------------------------------------------------------------------ the step
// The integers of a step travel to the device in ONE copy from pinned memory; the views below are slices of it.
void DecoderModel::build_batch(const std::vector<StepEntry> &entries, Batch &b) {
    const int n_seq = (int)entries.size();
    const int page = cache->page_size;
    const int n_groups = (int)cache->groups.size();
    int M = 0, n_want = 0, max_new = 0, max_len = 0;
    bool single = true;
    b.host_cu_rows.assign(1, 0);
    b.host_seq_start.clear();
    b.host_slots.clear();
    for (auto &e : entries) {
        int start = cache->length(e.slot);
        b.host_seq_start.push_back(start);
        b.host_slots.push_back(e.slot);
        M += e.n_tokens;
        b.host_cu_rows.push_back(M);
        n_want += (int)e.want.size();
        max_new = std::max(max_new, e.n_tokens);
        max_len = std::max(max_len, start + e.n_tokens);
        single = single && e.n_tokens == 1;
    }
    const int width = (max_len + page - 1) / page;
    auto pad = [](size_t n) { return (n + 3) / 4 * 4; };
    size_t sizes[7] = {(size_t)M, (size_t)M, (size_t)M, (size_t)n_seq + 1, (size_t)n_seq, (size_t)n_seq, (size_t)n_want};
    size_t offs[8], total = 0;
    for (int i = 0; i < 7; i++) { offs[i] = total; total += pad(sizes[i]); }
    offs[7] = total;
    size_t table_ints = pad((size_t)n_seq * width);
    total += table_ints * n_groups;
    total = std::max<size_t>(total, 4);
    Staging &st = staging_[next_staging_];
    next_staging_ = (next_staging_ + 1) % staging_.size();
    if (st.done) FG_CUDA(cudaEventSynchronize(st.done));           // its last copy has left the buffer
    else FG_CUDA(cudaEventCreateWithFlags(&st.done, cudaEventDisableTiming));
    if (st.cap < total) {
        if (st.host) FG_CUDA(cudaFreeHost(st.host));
        st.host = nullptr;
        st.cap = std::max(total, (size_t)4096);
        FG_CUDA(cudaMallocHost((void **)&st.host, st.cap * sizeof(int)));
    }
    int *h = st.host;
    int row = 0;
    bool want_all = n_want == M;
    int wi = 0;
    for (int s = 0; s < n_seq; s++) {
        const StepEntry &e = entries[(size_t)s];
        int start = b.host_seq_start[(size_t)s];
        for (int i = 0; i < e.n_tokens; i++, row++) {
            h[offs[0] + row] = e.tokens[i];
            h[offs[1] + row] = start + i;
            h[offs[2] + row] = s;
        }
        h[offs[3] + s] = b.host_cu_rows[(size_t)s];
        h[offs[4] + s] = start;
        h[offs[5] + s] = e.slot;
        for (int w : e.want) {
            int flat = b.host_cu_rows[(size_t)s] + w;
            want_all = want_all && flat == wi;
            h[offs[6] + wi++] = flat;
        }
    }
    h[offs[3] + n_seq] = M;
    for (int gi = 0; gi < n_groups; gi++)
        for (int s = 0; s < n_seq; s++) cache->block_table(gi, entries[(size_t)s].slot, width, h + offs[7] + gi * table_ints + (size_t)s * width);
    int *dev = (int *)runtime.arena->alloc(total * sizeof(int));
    FG_CUDA(cudaMemcpyAsync(dev, h, total * sizeof(int), cudaMemcpyHostToDevice, runtime.stream));
    FG_CUDA(cudaEventRecord(st.done, runtime.stream));
    b.n_seq = n_seq; b.n_rows = M; b.n_want = n_want; b.max_new = max_new; b.max_len = max_len;
    b.single_token = single; b.want_all = want_all && n_want > 0;
    b.tokens = dev + offs[0]; b.positions = dev + offs[1]; b.row_seq = dev + offs[2]; b.cu_rows = dev + offs[3];
    b.seq_start = dev + offs[4]; b.slots = dev + offs[5]; b.want_rows = n_want ? dev + offs[6] : nullptr;
    b.block_tables.clear();
    for (int gi = 0; gi < n_groups; gi++) b.block_tables.push_back(dev + offs[7] + gi * table_ints);
    b.table_width = width;
}

Tensor DecoderModel::step(const std::vector<StepEntry> &entries) {
    if (!cache) fail(FG_E_USAGE, "the engine has no cache yet");
    if (entries.empty()) fail(FG_E_TOKEN, "a step needs at least one sequence");
    std::vector<std::pair<int, int>> steps;
    for (auto &e : entries) {
        if (e.n_tokens <= 0) fail(FG_E_TOKEN, format("slot %d: a step must bring at least one token", e.slot));
        for (int i = 0; i < e.n_tokens; i++)
            if (e.tokens[i] < 0 || e.tokens[i] >= spec.vocab_size)
                fail(FG_E_TOKEN, format("slot %d: token id %d lies outside the vocabulary [0, %lld)", e.slot, e.tokens[i], (long long)spec.vocab_size));
        for (int w : e.want)
            if (w < 0 || w >= e.n_tokens)
                fail(FG_E_TOKEN, format("slot %d: wanted place %d is not among its %d tokens", e.slot, w, e.n_tokens));
        steps.emplace_back(e.slot, e.n_tokens);
    }
    cache->reserve(steps);                       // all or nothing; throws before any launch
    runtime.arena = &step_arena_;
    runtime.recording = false;
    step_arena_.reset();
    Batch batch;
    build_batch(entries, batch);
    Tensor logits = forward(runtime, batch);
    cache->commit(steps);
    return logits;
}

Tensor DecoderModel::forward(Runtime &rt, const Batch &batch) {
    const bool bf16 = rt.dtype == FG_BF16;
    const size_t n = spec.schedule.size();
    auto block_at = [&](size_t i) { return blocks_[(size_t)spec.schedule[i].layer].get(); };
    // the norm a block starts with, if whoever writes the residual stream may start it
    auto entry_norm = [&](Block *b) -> Norm * {
        return (bf16 && b->mixer->supports_deferred_norm() && b->mixer_norm->deferrable()) ? b->mixer_norm : nullptr;
    };
    // the final norm can be started by the last block when the head takes every row as it is
    Norm *head_norm = (batch.want_all && bf16 && final_norm_->deferrable() && head_->supports_deferred_norm()) ? final_norm_ : nullptr;
    Tensor x = rt.arena->matrix(batch.n_rows, spec.hidden_size, FG_F32);      // the float32 residual stream
    Norm *first = n ? entry_norm(block_at(0)) : nullptr;
    DeferredNorm pending = embedding_->forward(rt, batch, x, first);
    for (size_t i = 0; i < n; i++) {
        Norm *next = i + 1 < n ? entry_norm(block_at(i + 1)) : head_norm;
        rt.arena->begin_layer((int)i);                 // this entry's temporaries reuse the memory of entry i - 2
        pending = block_at(i)->forward(rt, x, batch, io[i], pending, next);
    }
    rt.arena->end_layers();
    if (!batch.want_rows) return Tensor();
    if (head_norm && pending.defined() && n) return head_->forward(rt, Tensor(), &pending);
    return head_->forward(rt, final_norm_->forward(rt, x, batch.want_rows, batch.n_want), nullptr);
}

void DecoderModel::block_forward(int entry, const std::vector<std::pair<int, int>> &steps, float *x_host) {
    if (!cache) fail(FG_E_USAGE, "the engine has no cache yet");
    if (entry < 0 || entry >= (int)spec.schedule.size()) fail(FG_E_USAGE, format("schedule entry %d does not exist", entry));
    std::vector<StepEntry> entries;
    std::vector<std::vector<int>> zeros;
    int M = 0;
    for (auto &st : steps) {
        zeros.emplace_back((size_t)std::max(0, st.second), 0);
        M += st.second;
    }
    for (size_t i = 0; i < steps.size(); i++) {
        StepEntry e;
        e.slot = steps[i].first;
        e.tokens = zeros[i].data();
        e.n_tokens = steps[i].second;
        entries.push_back(e);
    }
    cache->reserve(steps);
    runtime.arena = &step_arena_;
    runtime.recording = false;
    step_arena_.reset();
    Batch batch;
    build_batch(entries, batch);
    Tensor x = runtime.arena->matrix(M, spec.hidden_size, FG_F32);
    size_t bytes = (size_t)M * (size_t)spec.hidden_size * 4;
    FG_CUDA(cudaMemcpyAsync(x.data, x_host, bytes, cudaMemcpyHostToDevice, runtime.stream));
    blocks_[(size_t)spec.schedule[(size_t)entry].layer]->forward(runtime, x, batch, io[(size_t)entry], DeferredNorm(), nullptr);
    FG_CUDA(cudaMemcpyAsync(x_host, x.data, bytes, cudaMemcpyDeviceToHost, runtime.stream));
    FG_CUDA(cudaStreamSynchronize(runtime.stream));
    cache->commit(steps);
}

Json DecoderModel::describe() const {
    Json j = Json::object();
    j.set("vocab_size", (long long)spec.vocab_size);
    j.set("hidden_size", (long long)spec.hidden_size);
    j.set("layers", (long long)spec.layers.size());
    j.set("schedule", (long long)spec.schedule.size());
    j.set("dtype", dtype_long_name(runtime.dtype));
    j.set("tensors", (long long)expected_.size());
    j.set("weight_bytes", (long long)weight_bytes_);
    Json stops = Json::array();
    for (int t : spec.stop_token_ids) stops.push(Json(t));
    j.set("stop_token_ids", stops);
    if (cache) {
        j.set("max_seq_len", cache->max_seq_len);
        j.set("page_size", cache->page_size);
        j.set("slots", cache->n_slots);
        j.set("pages", cache->groups.empty() ? 0 : cache->groups[0].n_pages - 1);
        j.set("bytes_per_token", (long long)cache->bytes_per_token(runtime.dtype));
        j.set("cache_bytes", (long long)cache->pool_bytes(runtime.dtype));
        j.set("state_bytes", (long long)(state ? state->total_bytes() : 0));
        j.set("groups", cache->info().get("groups"));
    }
    return j;
}

}  // namespace fg
