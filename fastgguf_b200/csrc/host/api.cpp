// The exported C functions of fastgguf_engine.h and fastgguf_parts.h: argument checks, then the host classes;
// every exception becomes a status code and a message kept for fg_last_error().
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <sys/stat.h>

#include "../fastgguf_engine.h"
#include "../fastgguf_parts.h"
#include "cache.hpp"
#include "config.hpp"
#include "model.hpp"
#include "runner.hpp"
#include "safetensors.hpp"

using namespace fg;

struct fg_config { std::unique_ptr<ModelConfig> cfg; };
struct fg_engine { std::unique_ptr<Engine> engine; };
struct fg_cache { std::unique_ptr<PagedKVCache> cache; };
struct fg_result { std::vector<Completion> done; };
struct fg_session { fg_engine *owner; std::unique_ptr<DecodeSession> session; };

static thread_local std::string g_last_error;

template <typename F>
static int guarded(F &&f) {
    try {
        f();
        return FG_OK;
    } catch (const Error &e) {
        g_last_error = e.what();
        return e.code;
    } catch (const JsonError &e) {
        g_last_error = std::string("not valid JSON (") + e.what() + ")";
        return FG_E_USAGE;
    } catch (const std::bad_alloc &) {
        g_last_error = "out of host memory";
        return FG_E_INTERNAL;
    } catch (const std::exception &e) {
        g_last_error = e.what();
        return FG_E_INTERNAL;
    }
}

#define NEED(p) \
    if (!(p)) fail(FG_E_USAGE, std::string(__func__) + ": argument '" #p "' is null")

static char *dup_string(const std::string &s) {
    char *p = (char *)malloc(s.size() + 1);
    if (!p) throw std::bad_alloc();
    memcpy(p, s.c_str(), s.size() + 1);
    return p;
}

extern "C" {

const char *fg_last_error(void) { return g_last_error.c_str(); }
void fg_free(void *p) { free(p); }

// ---------------------------------------------------------------- configuration
int fg_config_from_json(const char *json_text, fg_config **out) {
    return guarded([&] {
        NEED(json_text); NEED(out);
        Json d;
        try {
            d = Json::parse(json_text);
        } catch (const JsonError &e) {
            fail(FG_E_CONFIG, std::string("config.json: not valid JSON (") + e.what() + ")");
        }
        *out = new fg_config{config_from_json(d)};
    });
}

int fg_config_from_dir(const char *model_dir, fg_config **out) {
    return guarded([&] {
        NEED(model_dir); NEED(out);
        *out = new fg_config{config_from_dir(model_dir)};
    });
}

void fg_config_destroy(fg_config *cfg) { delete cfg; }

int fg_config_to_json(const fg_config *cfg, char **json_out) {
    return guarded([&] { NEED(cfg); NEED(json_out); *json_out = dup_string(cfg->cfg->to_json().dump(2)); });
}
int fg_config_describe(const fg_config *cfg, char **json_out) {
    return guarded([&] {
        NEED(cfg); NEED(json_out);
        Json d = cfg->cfg->describe();
        d.set("architecture", cfg->cfg->architecture());
        *json_out = dup_string(d.dump());
    });
}
int fg_config_spec(const fg_config *cfg, char **spec_json_out) {
    return guarded([&] { NEED(cfg); NEED(spec_json_out); *spec_json_out = dup_string(cfg->cfg->spec().dump()); });
}
int fg_registered_architectures(char **json_out) {
    return guarded([&] {
        NEED(json_out);
        Json a = Json::array();
        for (auto &n : registered_architectures()) a.push(n);
        *json_out = dup_string(a.dump());
    });
}

// An architecture from outside: its configuration is the JSON text itself; the caller's function builds the spec.
class ExternalConfig : public ModelConfig {
public:
    ExternalConfig(std::string name, Json d, fg_spec_builder f, void *user) : name_(std::move(name)), d_(std::move(d)), f_(f), user_(user) {
        spec_ = build();                       // refuses a bad configuration when it is read, not at the first step
    }
    const std::string &architecture() const override { return name_; }
    Json to_json() const override { return d_; }
    Json describe() const override { return d_; }
    Json spec() const override { return spec_; }

private:
    Json build() const {
        char err[512] = {0};
        char *text = f_(d_.dump().c_str(), err, sizeof err, user_);
        if (!text) fail(FG_E_CONFIG, "config.json: " + std::string(err[0] ? err : "the architecture refused it"));
        std::string s(text);
        free(text);
        Json j = Json::parse(s);
        ModelSpec::from_json(j);               // validates
        return j;
    }
    std::string name_;
    Json d_, spec_;
    fg_spec_builder f_;
    void *user_;
};

int fg_register_architecture(const char *name, fg_spec_builder to_spec, void *user) {
    return guarded([&] {
        NEED(name); NEED(to_spec);
        std::string n = name;
        if (n == "LlamaForCausalLM") fail(FG_E_USAGE, "architecture 'LlamaForCausalLM' is built in and cannot be replaced");
        register_architecture(n, [n, to_spec, user](const Json &d) -> std::unique_ptr<ModelConfig> {
            return std::make_unique<ExternalConfig>(n, d, to_spec, user);
        });
    });
}

int fg_register_part(int role, const char *kind, const fg_part_vtable *vt) {
    return guarded([&] { NEED(kind); NEED(vt); register_external_part(role, kind, *vt); });
}

// ---------------------------------------------------------------- weights
// Checkpoint name -> declaration of every tensor the model's parts declare.  Parts are built without a device
// for this: a declaration depends on the parameters alone.
static std::map<std::string, ExpectedTensor> declared_tensors(const ModelSpec &spec, int dtype);

struct RandomFill { uint64_t seed; const std::map<std::string, ExpectedTensor> *decl; };
static void random_fill(const TensorInfo &t, void *dst, void *ctx) {
    RandomFill *r = (RandomFill *)ctx;
    const ExpectedTensor &e = r->decl->at(t.name);
    fill_random_host(dst, t.dtype, t.numel(), r->seed, name_hash64(t.name), e.init, e.std);
}

int fg_write_random_model(const fg_config *cfg, uint64_t seed, const char *out_dir, int dtype) {
    return guarded([&] {
        NEED(cfg); NEED(out_dir);
        if (dtype != FG_F32 && dtype != FG_BF16) fail(FG_E_USAGE, "a random model folder is written as float32 or bfloat16");
        ModelSpec spec = ModelSpec::from_json(cfg->cfg->spec());
        auto decl = declared_tensors(spec, dtype);
        std::string dir = out_dir;
        mkdir(dir.c_str(), 0777);
        struct stat st;
        if (stat(dir.c_str(), &st) != 0 || !S_ISDIR(st.st_mode)) fail(FG_E_WEIGHTS, dir + ": cannot create the folder");
        Json c = cfg->cfg->to_json();
        c.set("torch_dtype", dtype_long_name(dtype));
        FILE *f = fopen((dir + "/config.json").c_str(), "w");
        if (!f) fail(FG_E_WEIGHTS, dir + "/config.json: cannot write");
        std::string text = c.dump(2);
        fwrite(text.data(), 1, text.size(), f);
        fclose(f);
        std::vector<TensorInfo> tensors;
        for (auto &kv : decl) {
            TensorInfo t;
            t.name = kv.first;
            t.dtype = kv.second.is_int ? FG_I32 : dtype;
            t.shape = kv.second.shape;
            tensors.push_back(std::move(t));
        }
        Json meta = Json::object();
        meta.set("format", "pt");
        meta.set("seed", std::to_string(seed));
        RandomFill rf{seed, &decl};
        write_safetensors(dir + "/model.safetensors", tensors, meta, random_fill, &rf);
    });
}

static Json expected_json(const std::map<std::string, ExpectedTensor> &m);

int fg_spec_tensors(const char *spec_json, char **json_out) {
    return guarded([&] {
        NEED(spec_json); NEED(json_out);
        ModelSpec spec = ModelSpec::from_json(Json::parse(spec_json));
        *json_out = dup_string(expected_json(declared_tensors(spec, FG_BF16)).dump());
    });
}

static std::vector<TensorInfo> host_tensors(const fg_host_tensor *tensors, int n);

int fg_check_weights(const char *spec_json, const char *model_dir, const fg_host_tensor *tensors, int n_tensors, int dtype,
                     char **json_out) {
    return guarded([&] {
        NEED(spec_json); NEED(json_out);
        if (dtype != FG_F32 && dtype != FG_BF16) fail(FG_E_USAGE, "the engine runs in bfloat16 or float32");
        ModelSpec spec = ModelSpec::from_json(Json::parse(spec_json));
        auto decl = declared_tensors(spec, dtype);
        std::map<std::string, int> target;
        if (model_dir) {
            FolderSource src(model_dir);
            target = check_source(src, decl, spec.ignored_tensors, dtype);
        } else {
            MemorySource src(host_tensors(tensors, n_tensors));
            target = check_source(src, decl, spec.ignored_tensors, dtype);
        }
        Json o = Json::object();
        for (auto &kv : target) o.set(kv.first, dtype_long_name(kv.second));
        *json_out = dup_string(o.dump());
    });
}

int fg_folder_tensors(const char *model_dir, char **json_out) {
    return guarded([&] {
        NEED(model_dir); NEED(json_out);
        FolderSource src(model_dir);
        Json a = Json::array();
        for (auto &n : src.names()) {
            const TensorInfo *t = src.find(n);
            Json o = Json::object();
            o.set("name", n);
            o.set("dtype", dtype_long_name(t->dtype));
            Json shape = Json::array();
            for (auto s : t->shape) shape.push(Json((long long)s));
            o.set("shape", shape);
            a.push(o);
        }
        *json_out = dup_string(a.dump());
    });
}

// ---------------------------------------------------------------- engine
void fg_engine_default_options(fg_engine_options *o) {
    if (!o) return;
    memset(o, 0, sizeof *o);
    o->dtype = FG_BF16;
    o->max_batch = 64;
    o->max_tokens = 8192;
    o->use_graphs = 1;
}

static EngineOptions options_from(const fg_engine_options *opts) {
    fg_engine_options d;
    fg_engine_default_options(&d);
    if (opts) d = *opts;
    EngineOptions o;
    if (d.dtype != FG_BF16 && d.dtype != FG_F32) fail(FG_E_USAGE, "the engine runs in bfloat16 (FG_BF16) or float32 (FG_F32)");
    o.dtype = d.dtype;
    o.max_batch = d.max_batch;
    o.max_tokens = d.max_tokens;
    o.max_seq_len = d.max_seq_len;
    o.device = d.device;
    o.use_graphs = d.use_graphs != 0;
    o.verbose = d.verbose != 0;
    o.stream = (cudaStream_t)d.stream;
    return o;
}

static std::vector<TensorInfo> host_tensors(const fg_host_tensor *tensors, int n) {
    std::vector<TensorInfo> out;
    for (int i = 0; i < n; i++) {
        const fg_host_tensor &h = tensors[i];
        if (!h.name) fail(FG_E_USAGE, format("tensor %d has no name", i));
        if (dtype_size(h.dtype) == 0) fail(FG_E_WEIGHTS, format("tensor '%s': unsupported type %d", h.name, h.dtype));
        if (h.ndim < 0 || h.ndim > 4) fail(FG_E_WEIGHTS, format("tensor '%s' has %d dimensions (at most 4)", h.name, h.ndim));
        TensorInfo t;
        t.name = h.name;
        t.dtype = h.dtype;
        for (int k = 0; k < h.ndim; k++) t.shape.push_back(h.shape[k]);
        t.data = h.data;
        if (t.numel() > 0 && !h.data) fail(FG_E_USAGE, format("tensor '%s' has no data", h.name));
        out.push_back(std::move(t));
    }
    return out;
}

int fg_engine_create(const fg_config *cfg, const char *model_dir, const fg_engine_options *opts, fg_engine **out) {
    return guarded([&] {
        NEED(cfg); NEED(model_dir); NEED(out);
        EngineOptions o = options_from(opts);
        ModelSpec spec = ModelSpec::from_json(cfg->cfg->spec());
        FolderSource src(model_dir);
        *out = new fg_engine{std::make_unique<Engine>(spec, o, &src, false, 0)};
    });
}

int fg_engine_create_from_tensors(const fg_config *cfg, const fg_host_tensor *tensors, int n_tensors, const fg_engine_options *opts,
                                  fg_engine **out) {
    return guarded([&] {
        NEED(cfg); NEED(out);
        if (n_tensors > 0) NEED(tensors);
        EngineOptions o = options_from(opts);
        ModelSpec spec = ModelSpec::from_json(cfg->cfg->spec());
        MemorySource src(host_tensors(tensors, n_tensors));
        *out = new fg_engine{std::make_unique<Engine>(spec, o, &src, false, 0)};
    });
}

int fg_engine_create_random(const fg_config *cfg, uint64_t seed, const fg_engine_options *opts, fg_engine **out) {
    return guarded([&] {
        NEED(cfg); NEED(out);
        EngineOptions o = options_from(opts);
        ModelSpec spec = ModelSpec::from_json(cfg->cfg->spec());
        *out = new fg_engine{std::make_unique<Engine>(spec, o, nullptr, true, seed)};
    });
}

int fg_engine_create_from_spec(const char *spec_json, const fg_host_tensor *tensors, int n_tensors, const fg_engine_options *opts,
                               fg_engine **out) {
    return guarded([&] {
        NEED(spec_json); NEED(out);
        if (n_tensors > 0) NEED(tensors);
        EngineOptions o = options_from(opts);
        ModelSpec spec = ModelSpec::from_json(Json::parse(spec_json));
        MemorySource src(host_tensors(tensors, n_tensors));
        *out = new fg_engine{std::make_unique<Engine>(spec, o, &src, false, 0)};
    });
}

void fg_engine_destroy(fg_engine *e) { delete e; }

int fg_engine_info(const fg_engine *e, char **json_out) {
    return guarded([&] { NEED(e); NEED(json_out); *json_out = dup_string(e->engine->model->describe().dump()); });
}

static Json expected_json(const std::map<std::string, ExpectedTensor> &m) {
    Json o = Json::object();
    for (auto &kv : m) {
        Json t = Json::object();
        Json shape = Json::array();
        for (auto s : kv.second.shape) shape.push(Json((long long)s));
        t.set("shape", shape);
        t.set("kind", kv.second.is_int ? "int" : "float");
        t.set("init", kv.second.init == 1 ? "one_plus_normal" : "normal");
        t.set("std", (double)kv.second.std);
        o.set(kv.first, t);
    }
    return o;
}

int fg_engine_expected_tensors(const fg_engine *e, char **json_out) {
    return guarded([&] { NEED(e); NEED(json_out); *json_out = dup_string(expected_json(e->engine->model->expected_tensors()).dump()); });
}

void *fg_engine_stream(const fg_engine *e) { return e ? (void *)e->engine->stream : nullptr; }

int fg_slot_acquire(fg_engine *e, int *slot_out) {
    return guarded([&] { NEED(e); NEED(slot_out); *slot_out = e->engine->model->acquire_slot(); });
}
int fg_slot_release(fg_engine *e, int slot) {
    return guarded([&] { NEED(e); e->engine->model->release_slot(slot); });
}
int fg_slot_length(const fg_engine *e, int slot, int *length_out) {
    return guarded([&] { NEED(e); NEED(length_out); *length_out = e->engine->model->cache->length(slot); });
}
int fg_engine_cache_check(const fg_engine *e) {
    return guarded([&] { NEED(e); e->engine->model->cache->check(); });
}
int fg_engine_free_pages(const fg_engine *e, int group, int *out) {
    return guarded([&] { NEED(e); NEED(out); *out = e->engine->model->cache->free_pages(group); });
}

int fg_step(fg_engine *e, int n_seq, const int *slots, const int *n_tok, const int *tokens, int n_want, const int *want_rows,
            float *logits_out) {
    return guarded([&] {
        NEED(e);
        if (n_seq <= 0) fail(FG_E_TOKEN, "a step needs at least one sequence");
        NEED(slots); NEED(n_tok); NEED(tokens);
        if (n_want < 0) fail(FG_E_USAGE, "n_want cannot be negative");
        if (n_want > 0) { NEED(want_rows); NEED(logits_out); }
        Engine &eng = *e->engine;
        std::vector<StepEntry> entries((size_t)n_seq);
        std::vector<long long> cu((size_t)n_seq + 1, 0);
        for (int s = 0; s < n_seq; s++) {
            if (n_tok[s] <= 0) fail(FG_E_TOKEN, format("slot %d: a step must bring at least one token", slots[s]));
            cu[(size_t)s + 1] = cu[(size_t)s] + n_tok[s];
            entries[(size_t)s].slot = slots[s];
            entries[(size_t)s].tokens = tokens + cu[(size_t)s];
            entries[(size_t)s].n_tokens = n_tok[s];
        }
        // Wanted rows are flat indices into the token list.  The step returns them sequence by sequence, each
        // sequence's in the order given; that is the caller's order whenever want_rows does not jump back to an
        // earlier sequence, and otherwise the rows are put into the caller's order while copying out.
        std::vector<int> seq_of((size_t)n_want);
        bool grouped = true;
        for (int w = 0; w < n_want; w++) {
            long long r = want_rows[w];
            if (r < 0 || r >= cu[(size_t)n_seq]) fail(FG_E_TOKEN, format("wanted row %lld is not among the step's %lld tokens", r, cu[(size_t)n_seq]));
            int q = (int)(std::upper_bound(cu.begin(), cu.end(), r) - cu.begin()) - 1;
            seq_of[(size_t)w] = q;
            grouped = grouped && (w == 0 || q >= seq_of[(size_t)w - 1]);
            entries[(size_t)q].want.push_back((int)(r - cu[(size_t)q]));
        }
        Tensor logits = eng.model->step(entries);
        eng.stats.steps++;
        eng.stats.h2d_bytes += 4 * cu[(size_t)n_seq];
        if (n_want > 0) {
            const size_t row_bytes = (size_t)logits.cols * sizeof(float);
            if (grouped) {
                FG_CUDA(cudaMemcpy2DAsync(logits_out, row_bytes, logits.data, (size_t)logits.ld * 4, row_bytes, (size_t)n_want,
                                          cudaMemcpyDefault, eng.stream));
            } else {
                int out_row = 0;
                for (int q = 0; q < n_seq; q++)
                    for (int w = 0; w < n_want; w++) {
                        if (seq_of[(size_t)w] != q) continue;
                        FG_CUDA(cudaMemcpyAsync((char *)logits_out + (size_t)w * row_bytes, (char *)logits.data + (size_t)out_row * logits.ld * 4,
                                                row_bytes, cudaMemcpyDefault, eng.stream));
                        out_row++;
                    }
            }
            eng.stats.d2h_bytes += (long long)row_bytes * n_want;
        }
        FG_CUDA(cudaStreamSynchronize(eng.stream));
        raise_on_device_error("step");
    });
}

int fg_engine_check_device(fg_engine *e) {
    return guarded([&] { NEED(e); e->engine->check_device("engine"); });
}

// ---------------------------------------------------------------- sampling and generation
void fg_sampling_default(fg_sampling *s) {
    if (!s) return;
    s->temp = 1.0f; s->top_k = 64; s->top_p = 0.95f; s->repeat_penalty = 1.0f; s->repeat_last_n = 64; s->seed = 0;
}

static SamplingParams params_from(const fg_sampling *s) {
    fg_sampling d;
    fg_sampling_default(&d);
    if (s) d = *s;
    SamplingParams p;
    p.temp = d.temp; p.top_k = d.top_k; p.top_p = d.top_p; p.repeat_penalty = d.repeat_penalty;
    p.repeat_last_n = d.repeat_last_n; p.seed = d.seed;
    p.validate();
    return p;
}

static std::vector<int> int_list(const int *p, int n, const char *what) {
    if (n < 0) fail(FG_E_USAGE, std::string(what) + ": a count cannot be negative");
    if (n > 0 && !p) fail(FG_E_USAGE, std::string(what) + ": the list is null");
    return std::vector<int>(p, p + n);
}

int fg_engine_sampler_begin(fg_engine *e, const fg_sampling *s, const int *stop_ids, int n_stop, int slot, uint64_t state, const int *prompt,
                     int prompt_len) {
    return guarded([&] {
        NEED(e);
        SamplingBackend &b = e->engine->backend(params_from(s), int_list(stop_ids, n_stop, "stop_ids"));
        e->engine->model->cache->length(slot);             // the slot must be held
        b.sampler.begin(slot, state ? state : 0x9E3779B97F4A7C15ull, prompt, prompt ? prompt_len : 0);
    });
}

int fg_engine_sample(fg_engine *e, const fg_sampling *s, const int *stop_ids, int n_stop, float *logits, int n, const int *slots, int *tokens_out) {
    return guarded([&] {
        NEED(e); NEED(logits); NEED(slots); NEED(tokens_out);
        if (n <= 0) fail(FG_E_USAGE, "fg_sample needs at least one row");
        Engine &eng = *e->engine;
        SamplingBackend &b = eng.backend(params_from(s), int_list(stop_ids, n_stop, "stop_ids"));
        for (int i = 0; i < n; i++) eng.model->cache->length(slots[i]);
        DeviceBuffer buf((size_t)n * 8, "sampled tokens");
        int *rows = (int *)buf.get(), *out = rows + n;
        FG_CUDA(cudaMemcpyAsync(rows, slots, (size_t)n * 4, cudaMemcpyHostToDevice, eng.stream));
        int V = (int)eng.model->spec.vocab_size;
        b.sampler.sample(logits, n, V, V, rows, out, eng.stream);
        FG_CUDA(cudaMemcpyAsync(tokens_out, out, (size_t)n * 4, cudaMemcpyDeviceToHost, eng.stream));
        FG_CUDA(cudaStreamSynchronize(eng.stream));
    });
}

static std::vector<std::vector<int>> prompts_from(int n_prompts, const int *tokens, const int64_t *offsets) {
    if (n_prompts < 0) fail(FG_E_USAGE, "the number of prompts cannot be negative");
    std::vector<std::vector<int>> prompts;
    for (int i = 0; i < n_prompts; i++) {
        if (offsets[i + 1] < offsets[i]) fail(FG_E_USAGE, "prompt offsets must not decrease");
        prompts.emplace_back(tokens + offsets[i], tokens + offsets[i + 1]);
    }
    return prompts;
}

int fg_generate(fg_engine *e, int n_prompts, const int *prompt_tokens, const int64_t *offsets, const fg_sampling *sampling, int max_tokens,
                const int *stop_ids, int n_stop, int batch_size, int use_graphs, fg_token_callback on_token, void *user, fg_result **out) {
    return guarded([&] {
        NEED(e); NEED(out);
        if (n_prompts > 0) { NEED(prompt_tokens); NEED(offsets); }
        auto prompts = prompts_from(n_prompts, prompt_tokens, offsets);
        auto done = e->engine->generate(prompts, params_from(sampling), max_tokens, int_list(stop_ids, n_stop, "stop_ids"), batch_size,
                                        use_graphs, on_token, user);
        *out = new fg_result{std::move(done)};
    });
}

int fg_result_count(const fg_result *r) { return r ? (int)r->done.size() : 0; }

int fg_result_get(const fg_result *r, int i, const int **tokens, int *n_tokens, int *finish_reason) {
    return guarded([&] {
        NEED(r);
        if (i < 0 || i >= (int)r->done.size()) fail(FG_E_USAGE, format("result %d does not exist (there are %zu)", i, r->done.size()));
        const Completion &c = r->done[(size_t)i];
        if (tokens) *tokens = c.tokens.data();
        if (n_tokens) *n_tokens = (int)c.tokens.size();
        if (finish_reason) *finish_reason = c.finish_reason;
    });
}

void fg_result_destroy(fg_result *r) { delete r; }

int fg_engine_stats(const fg_engine *e, char **json_out) {
    return guarded([&] {
        NEED(e); NEED(json_out);
        const Engine::Stats &s = e->engine->stats;
        Json j = Json::object();
        j.set("steps", s.steps);
        j.set("h2d_bytes", s.h2d_bytes);
        j.set("d2h_bytes", s.d2h_bytes);
        j.set("launches_per_step", s.launches_per_step);
        j.set("graphs", s.graphs);
        j.set("backends", (long long)e->engine->backend_count());
        j.set("launches", launch_count());
        *json_out = dup_string(j.dump());
    });
}

int fg_engine_profile(fg_engine *e, int on) {
    return guarded([&] {
        NEED(e);
        profile_enable(on != 0, e->engine->stream);
    });
}

int fg_engine_profile_report(fg_engine *e, char **json_out) {
    return guarded([&] {
        NEED(e); NEED(json_out);
        *json_out = dup_string(profile_report_json());
    });
}

int fg_session_begin(fg_engine *e, int n_prompts, const int *prompt_tokens, const int64_t *offsets, const fg_sampling *sampling,
                     const int *stop_ids, int n_stop, fg_session **out) {
    return guarded([&] {
        NEED(e); NEED(out); NEED(prompt_tokens); NEED(offsets);
        auto prompts = prompts_from(n_prompts, prompt_tokens, offsets);
        if (prompts.empty()) fail(FG_E_USAGE, "a batch needs at least one prompt");
        if (profile_on()) fail(FG_E_USAGE, "a session replays recorded graphs, whose kernels cannot be timed one by one: profile through generate");
        SamplingParams p = params_from(sampling);
        SamplingBackend &b = e->engine->backend(p, int_list(stop_ids, n_stop, "stop_ids"));
        b.seed = resolve_seed(p.seed);
        *out = new fg_session{e, std::make_unique<DecodeSession>(b, prompts, 0)};
    });
}

int fg_session_advance(fg_session *s, const int *live, int n_live) {
    return guarded([&] {
        NEED(s);
        s->session->advance(int_list(live, n_live, "live"));
    });
}

int fg_session_slots(const fg_session *s, int *slots_out) {
    return guarded([&] {
        NEED(s); NEED(slots_out);
        for (size_t i = 0; i < s->session->slots.size(); i++) slots_out[i] = s->session->slots[i];
    });
}

int fg_session_launches_per_step(const fg_session *s) { return s ? (int)s->session->graph->launches_per_step : 0; }

void fg_session_close(fg_session *s) {
    if (!s) return;
    try {
        cudaStreamSynchronize(s->owner->engine->stream);
        s->session->close();
    } catch (...) {
    }
    delete s;
}

// ---------------------------------------------------------------- the loop over callbacks
class CallbackBackend : public LoopBackend {
public:
    explicit CallbackBackend(const fg_loop_backend *b) : b_(*b) {}
    void check(int code, const char *what) {
        if (code != 0) fail(code > 0 && code <= FG_E_INTERNAL ? code : FG_E_INTERNAL, format("the backend's %s returned status %d", what, code));
    }
    int acquire(int request_index, const int *prompt, int prompt_len) override {
        int slot = -1;
        check(b_.acquire(b_.user, request_index, prompt, prompt_len, &slot), "acquire");
        return slot;
    }
    void release(int slot) override { check(b_.release(b_.user, slot), "release"); }
    void step(const std::vector<int> &slots, const std::vector<int> &n_tok, const std::vector<int> &tokens) override {
        check(b_.step(b_.user, (int)slots.size(), slots.data(), n_tok.data(), tokens.data()), "step");
    }
    std::vector<int> sample(const std::vector<int> &slots) override {
        std::vector<int> out(slots.size());
        check(b_.sample(b_.user, (int)slots.size(), slots.data(), out.data()), "sample");
        return out;
    }
    int room(int slot) override {
        int r = 0;
        check(b_.room(b_.user, slot, &r), "room");
        return r;
    }

private:
    fg_loop_backend b_;
};

int fg_run_batch(const fg_loop_backend *b, int n_prompts, const int *prompt_tokens, const int64_t *offsets, int first_index, int max_tokens,
                 const int *stop_ids, int n_stop, fg_token_callback on_token, void *user, fg_result **out) {
    return guarded([&] {
        NEED(b); NEED(out);
        if (!b->acquire || !b->release || !b->step || !b->sample || !b->room) fail(FG_E_USAGE, "the backend lacks a function");
        if (n_prompts > 0) { NEED(prompt_tokens); NEED(offsets); }
        CallbackBackend backend(b);
        auto done = run_batch(backend, prompts_from(n_prompts, prompt_tokens, offsets), first_index, max_tokens,
                              int_list(stop_ids, n_stop, "stop_ids"), on_token, user);
        *out = new fg_result{std::move(done)};
    });
}

class CallbackSession : public LateSession {
public:
    CallbackSession(const fg_late_backend *b, int n) : b_(*b), n_(n), first_((size_t)n, 0) {
        int code = b_.begin(b_.user, n, first_.data());
        if (code != 0) fail(FG_E_INTERNAL, format("the backend's begin returned status %d", code));
    }
    ~CallbackSession() override {
        if (b_.close) b_.close(b_.user);
    }
    const std::vector<int> &first() const override { return first_; }
    int advance(const std::vector<int> &live) override {
        steps_.emplace_back((size_t)n_, 0);
        int code = b_.advance(b_.user, (int)live.size(), live.data(), steps_.back().data());
        if (code != 0) fail(FG_E_INTERNAL, format("the backend's advance returned status %d", code));
        return (int)steps_.size() - 1;
    }
    const int *wait(int handle) override { return steps_.at((size_t)handle).data(); }

private:
    fg_late_backend b_;
    int n_;
    std::vector<int> first_;
    std::vector<std::vector<int>> steps_;
};

int fg_run_batch_late(const fg_late_backend *b, int n_prompts, const int *prompt_tokens, const int64_t *offsets, int first_index,
                      int max_tokens, const int *stop_ids, int n_stop, int max_seq_len, fg_token_callback on_token, void *user,
                      fg_result **out) {
    return guarded([&] {
        NEED(b); NEED(out); NEED(offsets);
        if (!b->begin || !b->advance) fail(FG_E_USAGE, "the backend lacks a function");
        (void)prompt_tokens;
        std::vector<int> lens;
        for (int i = 0; i < n_prompts; i++) lens.push_back((int)(offsets[i + 1] - offsets[i]));
        CallbackSession session(b, n_prompts);
        auto done = run_batch_late(session, lens, first_index, max_tokens, int_list(stop_ids, n_stop, "stop_ids"), max_seq_len, on_token, user);
        *out = new fg_result{std::move(done)};
    });
}

int fg_seed_resolve(uint64_t seed, uint64_t *out) {
    return guarded([&] { NEED(out); *out = resolve_seed(seed); });
}
int fg_seed_of_request(uint64_t resolved_seed, uint64_t index, uint64_t *out) {
    return guarded([&] { NEED(out); *out = request_seed(resolved_seed, index); });
}

int fg_plan_batches(int n_requests, int batch_size, char **json_out) {
    return guarded([&] {
        NEED(json_out);
        Json a = Json::array();
        for (auto &r : plan_batches(n_requests, batch_size)) {
            Json p = Json::array();
            p.push(Json(r.first));
            p.push(Json(r.second));
            a.push(p);
        }
        *json_out = dup_string(a.dump());
    });
}

// ---------------------------------------------------------------- parts alone
static std::vector<std::pair<int, int>> steps_from(int n, const int *slots, const int *n_new);
static void need_device() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        fail(FG_E_DEVICE, "fastgguf_b200 runs on a CUDA device (sm_100a); no GPU is visible and there is no CPU path");
    }
}

int fg_part_run(int role, const char *kind, const char *params_json, int dtype, const fg_host_tensor *tensors, int n_tensors,
                const int *tokens, const float *x, float *residual, float *out, int M, int cols_in, int cols_out) {
    return guarded([&] {
        NEED(kind); NEED(params_json);
        if (dtype != FG_F32 && dtype != FG_BF16) fail(FG_E_USAGE, "the engine runs in bfloat16 or float32");
        if (M <= 0) fail(FG_E_USAGE, "a part needs at least one row");
        need_device();
        Arena arena;
        Runtime rt;
        rt.dtype = dtype;
        rt.arena = &arena;
        FG_CUDA(cudaGetDevice(&rt.device));
        FG_CUDA(cudaDeviceGetAttribute(&rt.n_sm, cudaDevAttrMultiProcessorCount, rt.device));
        BuildContext ctx;
        ctx.nested = [](int, const Json &) -> Part * { fail(FG_E_USAGE, "fg_part_run: parts with nested parts need an engine"); };
        std::unique_ptr<Part> part = build_part(role, kind, rt, Json::parse(params_json), ctx);
        // the part's tensors under the dtype policy
        MemorySource src(host_tensors(tensors, n_tensors));
        std::map<std::string, Weight> mine;
        for (auto &d : part->tensor_decls()) {
            const TensorInfo *t = src.find(d.name);
            if (!t) fail(FG_E_WEIGHTS, "the part's tensor '" + d.name + "' was not given");
            if (t->shape != d.shape) fail(FG_E_WEIGHTS, d.name + " is " + shape_text(t->shape) + ", the part needs " + shape_text(d.shape));
            int dt = d.is_int ? FG_I32 : (dtype == FG_F32 || t->dtype == FG_F32) ? FG_F32 : FG_BF16;
            int64_t cols = d.shape.empty() ? 1 : d.shape.back(), rows = t->numel() / std::max<int64_t>(1, cols);
            Weight w = make_weight(rows, cols, dt, d.name.c_str());
            DeviceBuffer raw((size_t)t->nbytes(), "tensor staging");
            FG_CUDA(cudaMemcpy(raw.get(), t->data, (size_t)t->nbytes(), cudaMemcpyHostToDevice));
            dev_convert(raw.get(), t->dtype, w.t.data, dt, t->numel(), nullptr);
            FG_CUDA(cudaDeviceSynchronize());
            mine[d.name] = w;
        }
        part->load(mine, rt);
        auto upload = [&](const float *host, int64_t rows, int64_t cols, int dt) {
            Tensor f = arena.matrix(rows, cols, FG_F32);
            FG_CUDA(cudaMemcpy(f.data, host, (size_t)rows * cols * 4, cudaMemcpyHostToDevice));
            if (dt == FG_F32) return f;
            Tensor t = arena.matrix(rows, cols, dt);
            dev_convert(f.data, FG_F32, t.data, dt, rows * cols, nullptr);
            return t;
        };
        auto download = [&](const Tensor &t, float *host) {
            Tensor f = t;
            if (t.dtype != FG_F32) {
                f = arena.matrix(t.rows, t.cols, FG_F32);
                for (int64_t r = 0; r < t.rows; r++)
                    dev_convert((char *)t.data + r * t.ld * elem_size(t.dtype), t.dtype, (char *)f.data + r * f.ld * 4, FG_F32, t.cols, nullptr);
            }
            FG_CUDA(cudaMemcpy2D(host, (size_t)t.cols * 4, f.data, (size_t)f.ld * 4, (size_t)t.cols * 4, (size_t)t.rows, cudaMemcpyDeviceToHost));
        };
        Batch batch;
        batch.n_seq = 1; batch.n_rows = M; batch.max_new = M; batch.max_len = M; batch.single_token = M == 1;
        if (role == FG_ROLE_NORM) {
            NEED(x); NEED(out);
            Tensor xin = upload(x, M, cols_in, FG_F32);
            download(dynamic_cast<Norm &>(*part).forward(rt, xin, nullptr, 0), out);
        } else if (role == FG_ROLE_FEED_FORWARD) {
            NEED(x); NEED(residual);
            Tensor xn = upload(x, M, cols_in, dtype), res = upload(residual, M, cols_in, FG_F32);
            dynamic_cast<FeedForward &>(*part).forward(rt, xn, nullptr, batch, res, nullptr);
            download(res, residual);
        } else if (role == FG_ROLE_HEAD) {
            NEED(x); NEED(out);
            Tensor xn = upload(x, M, cols_in, dtype);
            download(dynamic_cast<Head &>(*part).forward(rt, xn, nullptr), out);
        } else if (role == FG_ROLE_EMBEDDING) {
            NEED(tokens); NEED(out);
            int *tok = (int *)arena.alloc((size_t)M * 4);
            FG_CUDA(cudaMemcpy(tok, tokens, (size_t)M * 4, cudaMemcpyHostToDevice));
            batch.tokens = tok;
            Tensor xo = arena.matrix(M, cols_out, FG_F32);
            dynamic_cast<Embedding &>(*part).forward(rt, batch, xo, nullptr);
            download(xo, out);
        } else {
            fail(FG_E_USAGE, std::string("fg_part_run cannot run a ") + role_name(role) + " alone");
        }
        FG_CUDA(cudaDeviceSynchronize());
        raise_on_device_error("part");
    });
}

int fg_position_tables(const char *kind, const char *params_json, int max_positions, float *cos_out, float *sin_out, int *perm_out) {
    return guarded([&] {
        NEED(kind); NEED(params_json); NEED(cos_out); NEED(sin_out);
        if (max_positions <= 0) fail(FG_E_USAGE, "max_positions must be positive");
        need_device();
        Arena arena;
        Runtime rt;
        rt.arena = &arena;
        BuildContext ctx;
        std::unique_ptr<Part> part = build_part(FG_ROLE_POSITION, kind, rt, Json::parse(params_json), ctx);
        PositionEncoding &pe = dynamic_cast<PositionEncoding &>(*part);
        pe.prepare(rt, max_positions);
        size_t bytes = (size_t)max_positions * (pe.head_dim() / 2) * 4;
        FG_CUDA(cudaMemcpy(cos_out, pe.cos_table(), bytes, cudaMemcpyDeviceToHost));
        FG_CUDA(cudaMemcpy(sin_out, pe.sin_table(), bytes, cudaMemcpyDeviceToHost));
        if (perm_out)
            for (int i = 0; i < pe.head_dim(); i++) perm_out[i] = pe.permutation().empty() ? i : pe.permutation()[(size_t)i];
    });
}

int fg_engine_block_forward(fg_engine *e, int schedule_entry, int n_seq, const int *slots, const int *n_tok, float *x) {
    return guarded([&] {
        NEED(e); NEED(slots); NEED(n_tok); NEED(x);
        e->engine->model->block_forward(schedule_entry, steps_from(n_seq, slots, n_tok), x);
        raise_on_device_error("block");
    });
}

// ---------------------------------------------------------------- cache bookkeeping alone
int fg_cache_create(const char *requests_json, int64_t max_tokens, int max_seq_len, int n_slots, int page_size, fg_cache **out) {
    return guarded([&] {
        NEED(requests_json); NEED(out);
        auto req = cache_requests_from_json(Json::parse(requests_json));
        *out = new fg_cache{std::make_unique<PagedKVCache>(req, max_tokens, max_seq_len, n_slots, page_size)};
    });
}
void fg_cache_destroy(fg_cache *c) { delete c; }
int fg_cache_acquire(fg_cache *c, int *slot_out) {
    return guarded([&] { NEED(c); NEED(slot_out); *slot_out = c->cache->acquire(); });
}
int fg_cache_release(fg_cache *c, int slot) {
    return guarded([&] { NEED(c); c->cache->release(slot); });
}
int fg_cache_length(const fg_cache *c, int slot, int *out) {
    return guarded([&] { NEED(c); NEED(out); *out = c->cache->length(slot); });
}
static std::vector<std::pair<int, int>> steps_from(int n, const int *slots, const int *n_new) {
    std::vector<std::pair<int, int>> steps;
    for (int i = 0; i < n; i++) steps.emplace_back(slots[i], n_new[i]);
    return steps;
}
int fg_cache_reserve(fg_cache *c, int n, const int *slots, const int *n_new) {
    return guarded([&] { NEED(c); NEED(slots); NEED(n_new); c->cache->reserve(steps_from(n, slots, n_new)); });
}
int fg_cache_commit(fg_cache *c, int n, const int *slots, const int *n_new) {
    return guarded([&] { NEED(c); NEED(slots); NEED(n_new); c->cache->commit(steps_from(n, slots, n_new)); });
}
int fg_cache_pages_needed(const fg_cache *c, int slot, int n_new, int *per_group_out) {
    return guarded([&] {
        NEED(c); NEED(per_group_out);
        auto v = c->cache->pages_needed(slot, n_new);
        for (size_t i = 0; i < v.size(); i++) per_group_out[i] = v[i];
    });
}
int fg_cache_free_pages(const fg_cache *c, int group, int *out) {
    return guarded([&] { NEED(c); NEED(out); *out = c->cache->free_pages(group); });
}
int fg_cache_block_table(const fg_cache *c, int group, int slot, int width, int *out) {
    return guarded([&] { NEED(c); NEED(out); c->cache->block_table(group, slot, width, out); });
}
int fg_cache_check(const fg_cache *c) {
    return guarded([&] { NEED(c); c->cache->check(); });
}
int fg_cache_info(const fg_cache *c, char **json_out) {
    return guarded([&] { NEED(c); NEED(json_out); *json_out = dup_string(c->cache->info().dump()); });
}
int fg_cache_bytes(const char *requests_json, int64_t max_tokens, int page_size, int dtype, char **json_out) {
    return guarded([&] {
        NEED(requests_json); NEED(json_out);
        if (dtype != FG_F32 && dtype != FG_BF16) fail(FG_E_USAGE, "the cache is kept in bfloat16 or float32");
        PagedKVCache cache(cache_requests_from_json(Json::parse(requests_json)), max_tokens, 1 << 30, 1, page_size);
        Json j = Json::object();
        j.set("bytes_per_token", (long long)cache.bytes_per_token(dtype));
        j.set("pages", cache.groups.empty() ? 0 : cache.groups[0].n_pages - 1);
        j.set("bytes", (long long)cache.pool_bytes(dtype));
        *json_out = dup_string(j.dump());
    });
}

}  // extern "C"

// Declarations of a spec's tensors without a device: parts are built (their constructors only read parameters),
// asked for their declarations, and dropped.
static std::map<std::string, ExpectedTensor> declared_tensors(const ModelSpec &spec, int dtype) {
    Runtime rt;
    rt.dtype = dtype;
    std::vector<std::unique_ptr<Part>> owned;
    std::map<std::string, Part *> shared;
    std::map<std::string, ExpectedTensor> out;
    BuildContext ctx;
    std::function<Part *(int, const PartSpec &)> build = [&](int role, const PartSpec &ps) -> Part * {
        owned.push_back(build_part(role, ps.kind, rt, ps.params, ctx));
        Part *p = owned.back().get();
        for (auto &d : p->tensor_decls()) {
            auto it = ps.tensors.find(d.name);
            if (it == ps.tensors.end()) fail(FG_E_CONFIG, "a part declares tensor '" + d.name + "' but the architecture gives no checkpoint name for it");
            out.emplace(it->second, ExpectedTensor{d.shape, d.is_int, d.init, d.std});
        }
        return p;
    };
    ctx.nested = [&](int role, const Json &ns) -> Part * {
        std::string key = std::to_string(role) + ":" + ns.get("kind").as_string() + ":" + ns.get("params").dump();
        auto it = shared.find(key);
        if (it != shared.end()) return it->second;
        PartSpec ps;
        ps.kind = ns.get("kind").as_string();
        if (ns.get("params").is_object()) ps.params = ns.get("params");
        Part *p = build(role, ps);
        shared[key] = p;
        return p;
    };
    build(FG_ROLE_EMBEDDING, spec.embedding);
    for (auto &l : spec.layers) {
        build(FG_ROLE_MIXER, l.mixer);
        build(FG_ROLE_FEED_FORWARD, l.feed_forward);
        build(FG_ROLE_NORM, l.mixer_norm);
        build(FG_ROLE_NORM, l.feed_forward_norm);
    }
    build(FG_ROLE_NORM, spec.final_norm);
    build(FG_ROLE_HEAD, spec.head);
    return out;
}
