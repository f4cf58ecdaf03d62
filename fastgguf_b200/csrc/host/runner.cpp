// See runner.hpp.
#include "runner.hpp"

#include <algorithm>
#include <chrono>
#include <cstring>
#include <ctime>
#include <set>

namespace fg {

// ------------------------------------------------------------------------------------ sampling parameters
void SamplingParams::validate() const {
    if (top_k > 1024) fail(FG_E_USAGE, format("top_k %d exceeds 1024, the most the sampler takes (0 turns top-k off)", top_k));
    if (repeat_last_n < 0) fail(FG_E_USAGE, "repeat_last_n cannot be negative");
}

uint64_t resolve_seed(uint64_t seed) {
    if (seed == 0) {
        uint64_t now = (uint64_t)time(nullptr);
        uint64_t ticks = (uint64_t)std::chrono::duration_cast<std::chrono::microseconds>(
                             std::chrono::steady_clock::now().time_since_epoch()).count();
        seed = (now * 0x9E3779B97F4A7C15ull) ^ ticks;
    }
    return seed ? seed : 0x9E3779B97F4A7C15ull;
}

uint64_t request_seed(uint64_t seed, uint64_t index) {
    if (index == 0) return seed;
    uint64_t z = seed + index * 0x9E3779B97F4A7C15ull;           // splitmix64 finaliser
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return z ? z : 0x9E3779B97F4A7C15ull;
}

std::vector<std::pair<int, int>> plan_batches(int n_requests, int batch_size) {
    if (batch_size <= 0) fail(FG_E_USAGE, "batch_size must be positive");
    std::vector<std::pair<int, int>> out;
    for (int b = 0; b < n_requests; b += batch_size) out.emplace_back(b, std::min(n_requests, b + batch_size));
    return out;
}

int bucket_for(int n) {
    for (int b : kBuckets)
        if (n <= b) return b;
    fail(FG_E_USAGE, format("a batch of %d sequences exceeds the largest fixed-shape step (256)", n));
}

// ------------------------------------------------------------------------------------ the loop's decisions
std::vector<Completion> run_batch(LoopBackend &backend, const std::vector<std::vector<int>> &prompts, int first_index, int max_tokens,
                                  const std::vector<int> &stop_ids, TokenCallback on_token, void *user) {
    std::set<int> stop(stop_ids.begin(), stop_ids.end());
    for (auto &p : prompts)
        if (p.empty()) fail(FG_E_TOKEN, "a prompt needs at least one token");
    std::vector<int> slots;
    std::vector<Completion> done(prompts.size());
    struct Release {
        LoopBackend &b;
        std::vector<int> &slots;
        ~Release() {
            for (int s : slots) {
                try { b.release(s); } catch (...) {}
            }
        }
    } release{backend, slots};
    for (size_t i = 0; i < prompts.size(); i++) {
        slots.push_back(backend.acquire(first_index + (int)i, prompts[i].data(), (int)prompts[i].size()));
        done[i].prompt_len = (int)prompts[i].size();
    }
    std::vector<int> live;
    for (size_t i = 0; i < prompts.size(); i++) live.push_back((int)i);
    {
        std::vector<int> sl, nt, toks;
        for (int i : live) {
            sl.push_back(slots[(size_t)i]);
            nt.push_back((int)prompts[(size_t)i].size());
            toks.insert(toks.end(), prompts[(size_t)i].begin(), prompts[(size_t)i].end());
        }
        backend.step(sl, nt, toks);
    }
    while (!live.empty()) {
        std::vector<int> sl;
        for (int i : live) sl.push_back(slots[(size_t)i]);
        std::vector<int> tokens = backend.sample(sl);
        std::vector<int> next;
        for (size_t k = 0; k < live.size(); k++) {
            int i = live[k], tok = tokens[k];
            Completion &c = done[(size_t)i];
            if (stop.count(tok)) {                    // not emitted, not fed, not recorded
                c.finish_reason = 1;
                continue;
            }
            c.tokens.push_back(tok);
            if (on_token) on_token(user, first_index + i, tok);
            if ((max_tokens > 0 && (int)c.tokens.size() >= max_tokens) || backend.room(slots[(size_t)i]) <= 0) {
                c.finish_reason = 2;
                continue;
            }
            next.push_back(i);
        }
        live = next;
        if (!live.empty()) {
            std::vector<int> sl2, nt, toks;
            for (int i : live) {
                sl2.push_back(slots[(size_t)i]);
                nt.push_back(1);
                toks.push_back(done[(size_t)i].tokens.back());
            }
            backend.step(sl2, nt, toks);
        }
    }
    return done;
}

// ------------------------------------------------------------------------------------ sampler state
Sampler::Sampler(const SamplingParams &p, int n_slots, const std::vector<int> &stop_ids, cudaStream_t stream)
    : params(p), spare_row(n_slots), n_rows_(n_slots + 1), hist_cap_(std::max(1, p.repeat_last_n)), use_hist_(p.penalizes()),
      stream_(stream) {
    p.validate();
    std::vector<uint64_t> init((size_t)n_rows_, 0x9E3779B97F4A7C15ull);
    rng_ = DeviceBuffer((size_t)n_rows_ * 8, "sampler state");
    FG_CUDA(cudaMemcpy(rng_.get(), init.data(), init.size() * 8, cudaMemcpyHostToDevice));
    if (use_hist_) {
        hist_ = DeviceBuffer((size_t)n_rows_ * hist_cap_ * 4, "sampler history");
        hist_count_ = DeviceBuffer((size_t)n_rows_ * 4, "sampler history");
        FG_CUDA(cudaMemset(hist_.get(), 0, hist_.bytes()));
        FG_CUDA(cudaMemset(hist_count_.get(), 0, hist_count_.bytes()));
    }
    n_stop_ = (int)stop_ids.size();
    if (n_stop_) {
        stop_ = DeviceBuffer((size_t)n_stop_ * 4, "stop ids");
        FG_CUDA(cudaMemcpy(stop_.get(), stop_ids.data(), (size_t)n_stop_ * 4, cudaMemcpyHostToDevice));
    }
    // 4096 words a batch row: the candidates of the two-stage top-k, or (greedy) the two words in which the blocks
    // of a row meet.  Owned by this sampler, so samplers of other engines or streams share nothing with it.
    scratch_ = DeviceBuffer((size_t)bucket_for(std::max(1, n_slots)) * 4096 * 8, "sampler scratch");
    FG_CUDA(cudaMemset(scratch_.get(), 0, scratch_.bytes()));
}

void Sampler::begin(int row, uint64_t state, const int *prompt, int prompt_len) {
    if (row < 0 || row >= n_rows_) fail(FG_E_CACHE, format("sampler row %d does not exist", row));
    FG_CUDA(cudaMemcpyAsync((uint64_t *)rng_.get() + row, &state, 8, cudaMemcpyHostToDevice, stream_));
    if (use_hist_) {
        int n = std::min(prompt_len, hist_cap_);
        FG_CUDA(cudaMemcpyAsync((int *)hist_count_.get() + row, &n, 4, cudaMemcpyHostToDevice, stream_));
        if (n > 0)
            FG_CUDA(cudaMemcpyAsync((int *)hist_.get() + (size_t)row * hist_cap_, prompt + (prompt_len - n), (size_t)n * 4,
                                    cudaMemcpyHostToDevice, stream_));
    }
    // a batch starts: whatever an unfinished launch may have left in the meeting words is gone
    FG_CUDA(cudaMemsetAsync(scratch_.get(), 0, scratch_.bytes(), stream_));
}

void Sampler::sample(float *logits, int B, int V, int ldl, const int *rows_dev, int *out_dev, cudaStream_t s) {
    const SamplingParams &p = params;
    if ((size_t)B * 4096 * 8 > scratch_.bytes()) fail(FG_E_USAGE, format("a step of %d rows exceeds the sampler's scratch", B));
    FG_LAUNCH("core", fg_sample, logits, B, V, ldl, p.temp, p.top_k, p.top_p, p.repeat_penalty, p.repeat_last_n, rows_dev,
              (unsigned long long *)rng_.get(), (int *)hist_.get(), use_hist_ ? hist_cap_ : 0, (int *)hist_count_.get(),
              (const int *)stop_.get(), n_stop_, out_dev, (unsigned long long *)scratch_.get(), s);
}

// ------------------------------------------------------------------------------------ recorded decode step
DecodeGraph::DecodeGraph(Engine &e, Sampler &sampler, int width_) : width(width_), engine_(e), sampler_(sampler), arena_((size_t)16 << 20) {
    DecoderModel &model = *e.model;
    PagedKVCache &cache = *model.cache;
    table_width = (cache.max_seq_len + cache.page_size - 1) / cache.page_size;
    const int B = width, n_groups = (int)cache.groups.size();
    auto pad = [](size_t n) { return (n + 3) / 4 * 4; };
    std::vector<size_t> sizes = {(size_t)B, (size_t)B, (size_t)B, (size_t)B + 1, (size_t)B, (size_t)B, (size_t)B, (size_t)B, 4};
    for (int g = 0; g < n_groups; g++) sizes.push_back((size_t)B * table_width);
    std::vector<size_t> offs;
    size_t total = 0;
    for (size_t sz : sizes) { offs.push_back(total); total += pad(sz); }
    ints_ = DeviceBuffer(total * 4, "decode graph buffers");
    FG_CUDA(cudaMemset(ints_.get(), 0, total * 4));
    int *base = (int *)ints_.get();
    tokens = base + offs[0]; positions = base + offs[1]; row_seq = base + offs[2]; cu_rows = base + offs[3];
    rows = base + offs[4]; want = base + offs[5]; active = base + offs[6]; next_tokens = base + offs[7];
    spare_cell = base + offs[8];
    for (int g = 0; g < n_groups; g++) tables.push_back(base + offs[9 + (size_t)g]);
    std::vector<int> ar((size_t)B + 1), spare((size_t)B, sampler.spare_row);
    for (int i = 0; i <= B; i++) ar[(size_t)i] = i;
    FG_CUDA(cudaMemcpy(row_seq, ar.data(), (size_t)B * 4, cudaMemcpyHostToDevice));
    FG_CUDA(cudaMemcpy(cu_rows, ar.data(), ((size_t)B + 1) * 4, cudaMemcpyHostToDevice));
    FG_CUDA(cudaMemcpy(want, ar.data(), (size_t)B * 4, cudaMemcpyHostToDevice));
    FG_CUDA(cudaMemcpy(rows, spare.data(), (size_t)B * 4, cudaMemcpyHostToDevice));
    FG_CUDA(cudaMemcpy(spare_cell, spare.data(), 4, cudaMemcpyHostToDevice));
    upload_cap = std::max<size_t>(16, (size_t)B * table_width * (size_t)std::max(1, n_groups));
    regions.resize(4);
    for (auto &r : regions) {
        FG_CUDA(cudaMallocHost((void **)&r.tokens, (size_t)B * 4));
        FG_CUDA(cudaMallocHost((void **)&r.upload, upload_cap * 4));
        FG_CUDA(cudaEventCreateWithFlags(&r.done, cudaEventDisableTiming));
    }
    batch_.n_seq = B; batch_.n_rows = B; batch_.n_want = B; batch_.max_new = 1; batch_.max_len = cache.max_seq_len;
    batch_.single_token = true; batch_.want_all = true;
    batch_.tokens = tokens; batch_.positions = positions; batch_.row_seq = row_seq; batch_.cu_rows = cu_rows;
    batch_.seq_start = positions; batch_.slots = rows; batch_.want_rows = want;
    for (int *t : tables) batch_.block_tables.push_back(t);
    batch_.table_width = table_width;
    // host_* stay empty: a part may rely on the device arrays only (see fastgguf_parts.h)

    // warm-up outside the recording: loads modules, sets kernel attributes, sizes the arena
    FG_CUDA(cudaStreamSynchronize(e.stream));
    long long before = launch_count();
    run(e.stream, false);
    launches_per_step = launch_count() - before;
    FG_CUDA(cudaStreamSynchronize(e.stream));
    FG_CUDA(cudaMemset(tokens, 0, (size_t)B * 4));
    FG_CUDA(cudaMemset(positions, 0, (size_t)B * 4));
    arena_.reset();                                  // one block for what the warm-up needed
    arena_.forbid_growth(true);
    FG_CUDA(cudaStreamBeginCapture(e.capture_stream, cudaStreamCaptureModeRelaxed));
    try {
        run(e.capture_stream, true);
    } catch (...) {
        cudaGraph_t g = nullptr;
        cudaStreamEndCapture(e.capture_stream, &g);
        if (g) cudaGraphDestroy(g);
        throw;
    }
    FG_CUDA(cudaStreamEndCapture(e.capture_stream, &graph_));
    FG_CUDA(cudaGraphInstantiate(&exec_, graph_, 0));
    e.stats.graphs++;
}

DecodeGraph::~DecodeGraph() {
    for (auto &r : regions) {
        if (r.done) { cudaEventSynchronize(r.done); cudaEventDestroy(r.done); }
        if (r.tokens) cudaFreeHost(r.tokens);
        if (r.upload) cudaFreeHost(r.upload);
    }
    if (exec_) cudaGraphExecDestroy(exec_);
    if (graph_) cudaGraphDestroy(graph_);
}

// The recorded step: layers, sampler, and LAST the feedback of the sampled tokens into the next step's inputs.
// decode_advance must stay the last launch: it is the only kernel of the step that writes positions and tokens,
// and the fused decode attention reads them before waiting for its predecessor (see common.cuh).
void DecodeGraph::run(cudaStream_t s, bool recording) {
    Runtime rt = engine_.model->runtime;
    rt.stream = s;
    rt.arena = &arena_;
    rt.recording = recording;
    arena_.reset();
    Tensor logits = engine_.model->forward(rt, batch_);
    sampler_.sample(logits.ptr<float>(), width, (int)logits.cols, (int)logits.ld, rows, next_tokens, s);
    FG_LAUNCH("core", fg_decode_advance, tokens, positions, next_tokens, active, width, s);
}

void DecodeGraph::replay() { FG_CUDA(cudaGraphLaunch(exec_, engine_.stream)); }

// ------------------------------------------------------------------------------------ backend of the loop
SamplingBackend::SamplingBackend(Engine &e, const SamplingParams &p, const std::vector<int> &stops)
    : engine(e), sampler(p, e.model->cache->n_slots, stops, e.stream), stop_ids(stops) {}

int SamplingBackend::acquire(int request_index, const int *prompt, int prompt_len) {
    int slot = engine.model->acquire_slot();
    try {
        sampler.begin(slot, request_seed(seed, (uint64_t)request_index), prompt, prompt_len);
    } catch (...) {
        engine.model->release_slot(slot);
        throw;
    }
    return slot;
}

void SamplingBackend::release(int slot) { engine.model->release_slot(slot); }

int SamplingBackend::room(int slot) { return engine.model->cache->max_seq_len - engine.model->cache->length(slot); }

void SamplingBackend::step(const std::vector<int> &slots, const std::vector<int> &n_tok, const std::vector<int> &tokens) {
    std::vector<StepEntry> entries;
    size_t at = 0;
    for (size_t i = 0; i < slots.size(); i++) {
        StepEntry e;
        e.slot = slots[i];
        e.tokens = tokens.data() + at;
        e.n_tokens = n_tok[i];
        e.want = {n_tok[i] - 1};
        at += (size_t)n_tok[i];
        entries.push_back(std::move(e));
    }
    engine.stats.steps++;
    engine.stats.h2d_bytes += 4 * (long long)tokens.size();
    last_logits = engine.model->step(entries);
}

std::vector<int> SamplingBackend::sample(const std::vector<int> &slots) {
    const int n = (int)slots.size();
    if (!last_logits.defined() || last_logits.rows != n) fail(FG_E_INTERNAL, "sample: no logits of the last step for these sequences");
    Arena *arena = engine.model->runtime.arena;            // the step's arena: valid until the next step
    int *rows = (int *)arena->alloc((size_t)n * 4), *out = (int *)arena->alloc((size_t)n * 4);
    FG_CUDA(cudaMemcpyAsync(rows, slots.data(), (size_t)n * 4, cudaMemcpyHostToDevice, engine.stream));
    sampler.sample(last_logits.ptr<float>(), n, (int)last_logits.cols, (int)last_logits.ld, rows, out, engine.stream);
    std::vector<int> host((size_t)n);
    FG_CUDA(cudaMemcpyAsync(host.data(), out, (size_t)n * 4, cudaMemcpyDeviceToHost, engine.stream));
    FG_CUDA(cudaStreamSynchronize(engine.stream));
    engine.stats.d2h_bytes += 4LL * n;
    raise_on_device_error("decode step");
    return host;
}

DecodeGraph &SamplingBackend::graph(int width) {
    auto it = graphs.find(width);
    if (it == graphs.end()) it = graphs.emplace(width, std::make_unique<DecodeGraph>(engine, sampler, width)).first;
    return *it->second;
}

// ------------------------------------------------------------------------------------ one batch on the graph path
DecodeSession::DecodeSession(SamplingBackend &backend, const std::vector<std::vector<int>> &prompts, int first_index)
    : backend_(backend), n_((int)prompts.size()) {
    Engine &eng = backend.engine;
    for (auto &p : prompts)
        if (p.empty()) fail(FG_E_TOKEN, "a prompt needs at least one token");
    graph = &backend.graph(bucket_for(n_));        // recorded before slots are taken: its warm-up uses page 0
    DecodeGraph &g = *graph;
    cudaStream_t s = eng.stream;
    try {
        for (int i = 0; i < n_; i++) slots.push_back(backend.acquire(first_index + i, prompts[(size_t)i].data(), (int)prompts[(size_t)i].size()));
        std::vector<int> nt, toks;
        for (auto &p : prompts) {
            nt.push_back((int)p.size());
            toks.insert(toks.end(), p.begin(), p.end());
        }
        backend.step(slots, nt, toks);
        const Tensor &logits = backend.last_logits;
        const int B = g.width;
        std::vector<int> rows_h((size_t)B, backend.sampler.spare_row), pos_h((size_t)B, 0), act_h((size_t)B, 0);
        for (int i = 0; i < n_; i++) {
            rows_h[(size_t)i] = slots[(size_t)i];
            pos_h[(size_t)i] = (int)prompts[(size_t)i].size();
            act_h[(size_t)i] = 1;
        }
        FG_CUDA(cudaMemsetAsync(g.tokens, 0, (size_t)B * 4, s));
        for (int *t : g.tables) FG_CUDA(cudaMemsetAsync(t, 0, (size_t)B * g.table_width * 4, s));
        FG_CUDA(cudaMemcpyAsync(g.rows, rows_h.data(), (size_t)B * 4, cudaMemcpyHostToDevice, s));
        FG_CUDA(cudaMemcpyAsync(g.positions, pos_h.data(), (size_t)B * 4, cudaMemcpyHostToDevice, s));
        FG_CUDA(cudaMemcpyAsync(g.active, act_h.data(), (size_t)B * 4, cudaMemcpyHostToDevice, s));
        // the first tokens: sampled from the prompt step's logits straight into the graph's input
        backend.sampler.sample(logits.ptr<float>(), n_, (int)logits.cols, (int)logits.ld, g.rows, g.tokens, s);
        first_tokens.resize((size_t)n_);
        FG_CUDA(cudaMemcpyAsync(first_tokens.data(), g.tokens, (size_t)n_ * 4, cudaMemcpyDeviceToHost, s));
        FG_CUDA(cudaStreamSynchronize(s));
        widths_.assign((size_t)n_, 0);
        raise_on_device_error("prompt step");
        eng.stats.d2h_bytes += 4LL * n_;
    } catch (...) {
        close();
        throw;
    }
}

DecodeSession::~DecodeSession() { close(); }

void DecodeSession::close() {
    for (int s : slots) {
        try { backend_.release(s); } catch (...) {}
    }
    slots.clear();
}

int DecodeSession::advance(const std::vector<int> &live) {
    Engine &eng = backend_.engine;
    PagedKVCache &cache = *eng.model->cache;
    DecodeGraph &g = *graph;
    cudaStream_t s = eng.stream;
    std::vector<std::pair<int, int>> steps;
    std::vector<char> is_live((size_t)n_, 0);
    for (int i : live) {
        if (i < 0 || i >= n_) fail(FG_E_USAGE, format("sequence %d is not in this batch of %d", i, n_));
        steps.emplace_back(slots[(size_t)i], 1);
        is_live[(size_t)i] = 1;
    }
    cache.reserve(steps);
    for (int i = 0; i < n_; i++) {
        if (!is_live[(size_t)i] && widths_[(size_t)i] >= 0) {        // finished: page 0, spare state row, position 0
            for (int *t : g.tables) FG_CUDA(cudaMemsetAsync(t + (size_t)i * g.table_width, 0, (size_t)g.table_width * 4, s));
            FG_CUDA(cudaMemsetAsync(g.active + i, 0, 4, s));
            FG_CUDA(cudaMemsetAsync(g.positions + i, 0, 4, s));
            FG_CUDA(cudaMemcpyAsync(g.rows + i, g.spare_cell, 4, cudaMemcpyDeviceToDevice, s));
            widths_[(size_t)i] = -1;
        }
    }
    const int idx = g.next_region;
    g.next_region = (g.next_region + 1) % (int)g.regions.size();
    DecodeGraph::Region &region = g.regions[(size_t)idx];
    FG_CUDA(cudaEventSynchronize(region.done));                      // its copies of four steps ago have left it
    size_t used = 0;
    std::vector<int> row((size_t)g.table_width);
    for (int i : live) {                                             // upload page-table entries the step will touch
        if (widths_[(size_t)i] < 0) fail(FG_E_USAGE, format("sequence %d has left this batch", i));
        int need = (cache.length(slots[(size_t)i]) + 1 + cache.page_size - 1) / cache.page_size;
        if (need > widths_[(size_t)i]) {
            int have = widths_[(size_t)i];
            for (size_t gi = 0; gi < g.tables.size(); gi++) {
                cache.block_table((int)gi, slots[(size_t)i], need, row.data());
                size_t n = (size_t)(need - have);
                if (used + n > g.upload_cap) fail(FG_E_INTERNAL, "the page-table upload region is too small");
                memcpy(region.upload + used, row.data() + have, n * 4);
                FG_CUDA(cudaMemcpyAsync(g.tables[gi] + (size_t)i * g.table_width + have, region.upload + used, n * 4,
                                        cudaMemcpyHostToDevice, s));
                used += n;
                eng.stats.h2d_bytes += 4LL * (long long)n;
            }
            widths_[(size_t)i] = need;
        }
    }
    g.replay();
    cache.commit(steps);
    eng.stats.steps++;
    FG_CUDA(cudaMemcpyAsync(region.tokens, g.next_tokens, (size_t)g.width * 4, cudaMemcpyDeviceToHost, s));
    FG_CUDA(cudaEventRecord(region.done, s));
    eng.stats.d2h_bytes += 4LL * g.width;
    return idx;
}

const int *DecodeSession::wait(int index) {
    DecodeGraph::Region &region = graph->regions.at((size_t)index);
    FG_CUDA(cudaEventSynchronize(region.done));
    return region.tokens;
}

// ------------------------------------------------------------------------------------ engine
Engine::Engine(const ModelSpec &spec, const EngineOptions &o, const TensorSource *source, bool seed_random, uint64_t seed) : opts(o) {
    int n_dev = 0;
    cudaError_t e = cudaGetDeviceCount(&n_dev);
    if (e != cudaSuccess || n_dev <= 0) {
        cudaGetLastError();
        fail(FG_E_DEVICE, "fastgguf_b200 runs on a CUDA device (sm_100a); no GPU is visible and there is no CPU path");
    }
    if (o.device < 0 || o.device >= n_dev) fail(FG_E_DEVICE, format("CUDA device %d does not exist (%d visible)", o.device, n_dev));
    FG_CUDA(cudaSetDevice(o.device));
    if (o.stream) stream = o.stream;
    else {
        FG_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
        own_stream = true;
    }
    FG_CUDA(cudaStreamCreateWithFlags(&capture_stream, cudaStreamNonBlocking));
    model = std::make_unique<DecoderModel>(spec, o.dtype, o.device, stream);
    model->load_weights(source, seed_random, seed);
    model->make_cache(o.max_tokens, o.max_batch, o.max_seq_len, 64, o.verbose);
}

Engine::~Engine() {
    cudaStreamSynchronize(stream);
    backends_.clear();
    model.reset();
    if (capture_stream) cudaStreamDestroy(capture_stream);
    if (own_stream && stream) cudaStreamDestroy(stream);
}

void Engine::check_device(const char *where) {
    FG_CUDA(cudaStreamSynchronize(stream));
    raise_on_device_error(where);
}

SamplingBackend &Engine::backend(const SamplingParams &p, const std::vector<int> &stop_ids) {
    p.validate();
    std::string key = format("%a/%d/%a/%a/%d/", p.temp, p.top_k, p.top_p, p.repeat_penalty, p.repeat_last_n);
    for (int t : stop_ids) key += std::to_string(t) + ",";
    for (auto it = backends_.begin(); it != backends_.end(); ++it) {
        if (it->first == key) {
            backends_.splice(backends_.begin(), backends_, it);      // most recently used first
            return *backends_.front().second;
        }
    }
    // a few sets of options are kept; the oldest goes with its recorded graphs and their activation memory
    const size_t kMaxBackends = 4;
    while (backends_.size() >= kMaxBackends) {
        FG_CUDA(cudaStreamSynchronize(stream));
        backends_.pop_back();
    }
    backends_.emplace_front(key, std::make_unique<SamplingBackend>(*this, p, stop_ids));
    return *backends_.front().second;
}

std::vector<Completion> Engine::generate(const std::vector<std::vector<int>> &prompts, const SamplingParams &params, int max_tokens,
                                         const std::vector<int> &stop_ids, int batch_size, int use_graphs, TokenCallback on_token,
                                         void *user) {
    SamplingBackend &b = backend(params, stop_ids);
    b.seed = resolve_seed(params.seed);
    if (batch_size <= 0) batch_size = opts.max_batch;
    if (batch_size > opts.max_batch) fail(FG_E_USAGE, format("batch_size %d exceeds the engine's %d sequence slots", batch_size, opts.max_batch));
    bool graphs = (use_graphs < 0 ? opts.use_graphs : use_graphs != 0) && !profile_on();
    std::vector<Completion> out;
    for (auto &rng : plan_batches((int)prompts.size(), batch_size)) {
        std::vector<std::vector<int>> part(prompts.begin() + rng.first, prompts.begin() + rng.second);
        std::vector<Completion> done = (graphs && (int)part.size() <= 256)
                                           ? run_batch_graphs(b, part, rng.first, max_tokens, stop_ids, on_token, user)
                                           : run_batch(b, part, rng.first, max_tokens, stop_ids, on_token, user);
        for (auto &c : done) out.push_back(std::move(c));
    }
    return out;
}

std::vector<Completion> Engine::run_batch_graphs(SamplingBackend &b, const std::vector<std::vector<int>> &prompts, int first_index,
                                                 int max_tokens, const std::vector<int> &stop_ids, TokenCallback on_token, void *user) {
    DecodeSession session(b, prompts, first_index);
    std::vector<int> lens;
    for (auto &p : prompts) lens.push_back((int)p.size());
    std::vector<Completion> done = run_batch_late(session, lens, first_index, max_tokens, stop_ids, model->cache->max_seq_len, on_token, user);
    check_device("batch");
    stats.launches_per_step = session.graph->launches_per_step;
    return done;
}

std::vector<Completion> run_batch_late(LateSession &session, const std::vector<int> &prompt_lens, int first_index, int max_tokens,
                                       const std::vector<int> &stop_ids, int max_seq_len, TokenCallback on_token, void *user) {
    std::set<int> stop(stop_ids.begin(), stop_ids.end());
    const int n = (int)prompt_lens.size();
    std::vector<Completion> done((size_t)n);
    for (int i = 0; i < n; i++) done[(size_t)i].prompt_len = prompt_lens[(size_t)i];
    // sample k is produced by step k (k = 0: the prompt step); the host sees it one step late
    struct Pending { std::vector<int> who; int handle; };
    std::deque<Pending> pending;
    {
        std::vector<int> all;
        for (int i = 0; i < n; i++) all.push_back(i);
        pending.push_back({all, -1});
    }
    std::vector<char> known_done((size_t)n, 0);          // decided from tokens the host has seen
    auto settle = [&](bool block) {
        while (!pending.empty() && (block || pending.size() > 1 || pending.front().handle < 0)) {
            Pending p = std::move(pending.front());
            pending.pop_front();
            const int *toks = p.handle >= 0 ? session.wait(p.handle) : session.first().data();
            for (int i : p.who) {
                if (known_done[(size_t)i]) continue;
                int tok = toks[i];
                Completion &c = done[(size_t)i];
                if (stop.count(tok)) {                    // not emitted, not fed on purpose, not recorded
                    c.finish_reason = 1;
                    known_done[(size_t)i] = 1;
                    continue;
                }
                c.tokens.push_back(tok);
                if (on_token) on_token(user, first_index + i, tok);
                if ((max_tokens > 0 && (int)c.tokens.size() >= max_tokens) ||
                    prompt_lens[(size_t)i] + (int)c.tokens.size() - 1 >= max_seq_len) {
                    c.finish_reason = 2;
                    known_done[(size_t)i] = 1;
                }
            }
        }
    };
    int step_no = 0;
    while (true) {
        settle(false);
        step_no++;
        // a sequence takes decode step s when it is not known to have ended, when sample s - 1 cannot have been
        // its last by length, and when the cache has room for the token
        std::vector<int> live;
        for (int i = 0; i < n; i++)
            if (!known_done[(size_t)i] && (max_tokens <= 0 || step_no < max_tokens) && prompt_lens[(size_t)i] + step_no <= max_seq_len)
                live.push_back(i);
        if (live.empty()) break;
        int handle = session.advance(live);
        pending.push_back({live, handle});
    }
    settle(true);
    return done;
}

}  // namespace fg
