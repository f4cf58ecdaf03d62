/* The engine's C interface (libfg_engine.so): configuration, weights, cache, the ONE step function,
 * sampling and the generation loop, for C and C++ programs and, through ctypes, for the Python package.
 *
 * The reference engine is callable C: model_load(m, g, n_ctx) (fastgguf.c:4180), forward(m, token, pos)
 * (:4648), forward_batch(m, tokens, n, pos0) (:5128), sample_next (:4008) and the loop of cmd_chat
 * (:5284-5309).  This header is their counterpart for a model folder (config.json + safetensors), many
 * sequences at once and a paged cache on one B200.
 *
 * Conventions
 *   - Every function returns FG_OK (0) or an FG_E_* status; fg_last_error() gives the message of the
 *     calling thread's last failure.  On failure nothing of the engine's state has changed unless said.
 *   - Strings handed out through `char **` are owned by the caller and freed with fg_free().
 *   - dtype codes: FG_F32 0, FG_BF16 1 (the engine's compute dtype), plus FG_F16 2, FG_I32 3, FG_I64 4 for
 *     tensors given by the caller.
 *   - The host code needs no GPU for configuration, weight checking, cache bookkeeping and the loop's
 *     decisions; anything that computes needs one and fails with FG_E_DEVICE otherwise (there is no CPU path).
 */
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FG_OK 0
#define FG_E_USAGE 1        /* a bad argument: null pointer, unknown option, wrong count */
#define FG_E_CONFIG 2       /* config.json missing, malformed, or describing an impossible model */
#define FG_E_WEIGHTS 3      /* missing / unexpected / wrongly shaped tensors, or a broken safetensors file */
#define FG_E_CACHE 4        /* slot misuse: unknown, not held, held twice in a step */
#define FG_E_CAPACITY 5     /* no free slot, no free pages, or a sequence past the cache's longest length */
#define FG_E_TOKEN 6        /* a token id outside the vocabulary, an empty step, a wanted place out of range */
#define FG_E_DEVICE 7       /* no GPU, a CUDA call failed, a kernel library is missing, out of device memory */
#define FG_E_KERNEL 8       /* a launcher refused its sizes, or a bounded device-side wait ran out */
#define FG_E_INTERNAL 9

#ifndef FG_F32
#define FG_F32 0
#define FG_BF16 1
#endif
#define FG_F16 2
#define FG_I32 3
#define FG_I64 4

typedef struct fg_config fg_config;   /* a typed configuration of a registered architecture */
typedef struct fg_engine fg_engine;   /* a loaded model with its cache */
typedef struct fg_cache fg_cache;     /* cache bookkeeping alone (what fg_engine holds inside) */
typedef struct fg_result fg_result;   /* what fg_generate returns */

const char *fg_last_error(void);
void fg_free(void *p);

/* ---------------------------------------------------------------- configuration and registry */
/* The model class is chosen by "architectures"[0]; an unknown name is an error that lists the known ones. */
int fg_config_from_json(const char *json_text, fg_config **out);
/* Reads DIR/config.json and adds the eos_token_id values of DIR/generation_config.json, if present. */
int fg_config_from_dir(const char *model_dir, fg_config **out);
void fg_config_destroy(fg_config *cfg);
/* The config.json form (what fg_config_from_json reads back). */
int fg_config_to_json(const fg_config *cfg, char **json_out);
/* Every field plus derived sizes (q_dim, kv_dim, group_size, parameters, kv_bytes_per_token per dtype,
 * parameter_bytes per dtype, and "defaulted": the keys the file did not give). */
int fg_config_describe(const fg_config *cfg, char **json_out);
/* The model as data: parts, layers, execution order, checkpoint tensor names (a JSON object). */
int fg_config_spec(const fg_config *cfg, char **spec_json_out);
/* A JSON list of registered architecture names. */
int fg_registered_architectures(char **json_out);

/* Another architecture: `to_spec` turns the text of a config.json into the JSON of a model spec (both
 * described in fastgguf_parts.h).  Returns a malloc'ed string, or NULL after writing a message to err. */
typedef char *(*fg_spec_builder)(const char *config_json, char *err, size_t err_cap, void *user);
int fg_register_architecture(const char *name, fg_spec_builder to_spec, void *user);

/* ---------------------------------------------------------------- weights */
/* Writes DIR/config.json and DIR/model.safetensors: weights ~ N(0, 0.02), norm weights 1 + N(0, 0.01),
 * from a counter-based generator (the same values on the host and on the device). dtype: FG_F32 / FG_BF16. */
int fg_write_random_model(const fg_config *cfg, uint64_t seed, const char *out_dir, int dtype);
/* Checkpoint name -> {"shape", "kind": "float" | "int", "init", "std"} of every tensor the parts of a model spec
 * declare (no device needed). */
int fg_spec_tensors(const char *spec_json, char **json_out);
/* The tensor table of a model folder: [{"name", "dtype", "shape"}], sorted by name. */
int fg_folder_tensors(const char *model_dir, char **json_out);

/* defined below */
struct fg_host_tensor;
/* Checks weights against a model spec without a device: model_dir, or (model_dir NULL) the given tensors.
 * FG_E_WEIGHTS with ONE message that lists missing, unexpected and wrongly shaped tensors; else json_out is
 * checkpoint name -> the dtype the tensor takes in an engine of `dtype` ("float32", "bfloat16", "int32"). */
int fg_check_weights(const char *spec_json, const char *model_dir, const struct fg_host_tensor *tensors, int n_tensors,
                     int dtype, char **json_out);

typedef struct fg_host_tensor {
    const char *name;
    int dtype;               /* FG_F32, FG_BF16, FG_F16, FG_I32, FG_I64 */
    int ndim;
    int64_t shape[4];
    const void *data;        /* host memory, contiguous */
} fg_host_tensor;

/* ---------------------------------------------------------------- engine */
typedef struct fg_engine_options {
    int dtype;               /* FG_BF16 (serving) or FG_F32 (true 32-bit path) */
    int max_batch;           /* sequence slots; also the largest batch of fg_generate */
    int64_t max_tokens;      /* most tokens live sequences hold at any time, each rounded up to a page of 64 */
    int max_seq_len;         /* longest sequence; 0 = the model's max_position_embeddings */
    int device;              /* CUDA device ordinal */
    int use_graphs;          /* 1: the decode step of fg_generate is a CUDA graph per batch-size bucket */
    int verbose;             /* 1: print the [cache] line to stderr at creation */
    void *stream;            /* a cudaStream_t to work on; NULL = a stream of the engine's own */
} fg_engine_options;
void fg_engine_default_options(fg_engine_options *opts);

/* Where the weights come from: a model folder, given host tensors, or the seeded generator. */
int fg_engine_create(const fg_config *cfg, const char *model_dir, const fg_engine_options *opts, fg_engine **out);
int fg_engine_create_from_tensors(const fg_config *cfg, const fg_host_tensor *tensors, int n_tensors,
                                  const fg_engine_options *opts, fg_engine **out);
int fg_engine_create_random(const fg_config *cfg, uint64_t seed, const fg_engine_options *opts, fg_engine **out);
/* The same from a model spec (JSON) instead of a registered architecture's configuration. */
int fg_engine_create_from_spec(const char *spec_json, const fg_host_tensor *tensors, int n_tensors,
                               const fg_engine_options *opts, fg_engine **out);
void fg_engine_destroy(fg_engine *e);

/* {"vocab_size", "hidden_size", "layers", "schedule", "max_seq_len", "page_size", "slots", "pages",
 *  "bytes_per_token", "cache_bytes", "weight_bytes", "tensors", "stop_token_ids", "groups": [...]} */
int fg_engine_info(const fg_engine *e, char **json_out);
/* Checkpoint name -> shape / kind / initialisation of every tensor the model's parts declare (JSON). */
int fg_engine_expected_tensors(const fg_engine *e, char **json_out);
void *fg_engine_stream(const fg_engine *e);

int fg_slot_acquire(fg_engine *e, int *slot_out);
int fg_slot_release(fg_engine *e, int slot);
int fg_slot_length(const fg_engine *e, int slot, int *length_out);
/* Raises FG_E_CACHE if a page or a slot is lost, held twice or freed twice. */
int fg_engine_cache_check(const fg_engine *e);
int fg_engine_free_pages(const fg_engine *e, int group, int *out);

/* The ONE step function.  Sequence s (in slot slots[s]) brings n_tok[s] >= 1 next tokens, laid out one
 * sequence after another in `tokens`; want_rows are flat indices into `tokens` whose logits are wanted.
 * logits_out receives [n_want, vocab] float32 and may be host or device memory (NULL if n_want == 0).
 * All prompts of a batch in one call, then one token each - or any other cut.  Validation (slots held and
 * distinct, token ids in range, capacity, wanted rows in range) comes before any launch. */
int fg_step(fg_engine *e, int n_seq, const int *slots, const int *n_tok, const int *tokens, int n_want,
            const int *want_rows, float *logits_out);
/* Raises FG_E_KERNEL if a bounded device-side wait ran out since the last call (synchronises the stream). */
int fg_engine_check_device(fg_engine *e);

/* ---------------------------------------------------------------- sampling and generation */
/* The reference's chat options with their defaults (fastgguf.c:6957-6982). */
typedef struct fg_sampling {
    float temp;              /* 1.0; <= 0 = greedy */
    int top_k;               /* 64; 0 = off; at most 1024 */
    float top_p;             /* 0.95 */
    float repeat_penalty;    /* 1.0 = off */
    int repeat_last_n;       /* 64 */
    uint64_t seed;           /* 0 = from the clock */
} fg_sampling;
void fg_sampling_default(fg_sampling *s);

/* One token per row of `logits` ([n, vocab] float32 on the DEVICE, modified in place by the repeat penalty);
 * slots[i] names the sequence whose generator and history row i uses.  tokens_out: host memory.
 * A slot's generator is (re)seeded by fg_engine_sampler_begin. */
int fg_engine_sampler_begin(fg_engine *e, const fg_sampling *s, const int *stop_ids, int n_stop, int slot,
                     uint64_t state, const int *prompt, int prompt_len);
int fg_engine_sample(fg_engine *e, const fg_sampling *s, const int *stop_ids, int n_stop, float *logits, int n,
              const int *slots, int *tokens_out);

typedef void (*fg_token_callback)(void *user, int request_index, int token);

/* Generate for n_prompts prompts (prompt i = prompt_tokens[offsets[i] .. offsets[i + 1])), batch_size at a
 * time (0 = the engine's max_batch), one batch after another.  max_tokens <= 0: until a stop token or a
 * full context.  A drawn stop token ends its sequence and is neither emitted, fed nor recorded. */
int fg_generate(fg_engine *e, int n_prompts, const int *prompt_tokens, const int64_t *offsets,
                const fg_sampling *sampling, int max_tokens, const int *stop_ids, int n_stop, int batch_size,
                int use_graphs /* -1 = the engine's option */, fg_token_callback on_token, void *user,
                fg_result **out);
int fg_result_count(const fg_result *r);
/* finish_reason: 1 = "stop" (a stop token was drawn), 2 = "length" (max_tokens or a full context). */
int fg_result_get(const fg_result *r, int i, const int **tokens, int *n_tokens, int *finish_reason);
void fg_result_destroy(fg_result *r);
/* {"steps", "h2d_bytes", "d2h_bytes", "launches_per_step", "graphs"} accumulated over fg_generate calls. */
int fg_engine_stats(const fg_engine *e, char **json_out);
/* Per-launcher device times.  While on, every kernel launcher call of this engine is bracketed by two events (kernels
 * then run one after another, without the overlap of dependent launches) and fg_generate runs its decode steps
 * eagerly; fg_session_begin is refused.  The report is a JSON list [{"name", "calls", "ms"}], longest first, of
 * everything launched since profiling was switched on or last reported.  One engine at a time. */
int fg_engine_profile(fg_engine *e, int on);
int fg_engine_profile_report(fg_engine *e, char **json_out);

/* A batch on the graph path, step by step (what the benchmark times): begin runs the prompts and samples
 * the first tokens; each advance runs one decode step for the sequences `live` (indices into the batch). */
typedef struct fg_session fg_session;
int fg_session_begin(fg_engine *e, int n_prompts, const int *prompt_tokens, const int64_t *offsets,
                     const fg_sampling *sampling, const int *stop_ids, int n_stop, fg_session **out);
int fg_session_advance(fg_session *s, const int *live, int n_live);
int fg_session_slots(const fg_session *s, int *slots_out);
int fg_session_launches_per_step(const fg_session *s);
void fg_session_close(fg_session *s);

/* ---------------------------------------------------------------- the generation loop over an abstract backend */
/* The loop's decisions alone, over callbacks (a fake backend tests them without a GPU).  Each callback
 * returns 0 or an FG_E_* status, which ends the loop. */
typedef struct fg_loop_backend {
    void *user;
    int (*acquire)(void *user, int request_index, const int *prompt, int prompt_len, int *slot_out);
    int (*release)(void *user, int slot);
    /* run the step; keep the logits of the wanted rows for `sample` */
    int (*step)(void *user, int n_seq, const int *slots, const int *n_tok, const int *tokens);
    int (*sample)(void *user, int n_seq, const int *slots, int *tokens_out);
    int (*room)(void *user, int slot, int *room_out);
} fg_loop_backend;
int fg_run_batch(const fg_loop_backend *b, int n_prompts, const int *prompt_tokens, const int64_t *offsets,
                 int first_index, int max_tokens, const int *stop_ids, int n_stop, fg_token_callback on_token,
                 void *user, fg_result **out);
/* The graph path's decisions alone: tokens of a decode step reach the host one step late.  begin fills the
 * tokens sampled from the prompts; advance runs one step for `live` and fills the tokens of all n rows. */
typedef struct fg_late_backend {
    void *user;
    int (*begin)(void *user, int n, int *first_tokens_out);
    int (*advance)(void *user, int n_live, const int *live, int *tokens_out);
    int (*close)(void *user);
} fg_late_backend;
int fg_run_batch_late(const fg_late_backend *b, int n_prompts, const int *prompt_tokens, const int64_t *offsets,
                      int first_index, int max_tokens, const int *stop_ids, int n_stop, int max_seq_len,
                      fg_token_callback on_token, void *user, fg_result **out);
/* The generator state a call seeded with `seed` starts from (0 = from the clock; never zero), and the state
 * of its request `index`. */
int fg_seed_resolve(uint64_t seed, uint64_t *out);
int fg_seed_of_request(uint64_t resolved_seed, uint64_t index, uint64_t *out);
/* [[first, last + 1], ...] of the batches that serve n_requests in order, batch_size at a time. */
int fg_plan_batches(int n_requests, int batch_size, char **json_out);

/* ---------------------------------------------------------------- parts alone (for tests of one part) */
/* Builds ONE part of `role` / `kind` from its parameters and the given tensors, runs it once and returns float32
 * results on the host.  norm: x [M, cols_in] -> out [M, cols_in].  feed_forward: xn = x (converted to the engine
 * dtype), adds into residual [M, cols_in].  head: xn = x -> out [M, cols_out].  embedding: tokens [M] -> out
 * [M, cols_out].  Mixers need a cache: see fg_engine_block_forward. */
int fg_part_run(int role, const char *kind, const char *params_json, int dtype, const fg_host_tensor *tensors,
                int n_tensors, const int *tokens, const float *x, float *residual, float *out, int M, int cols_in,
                int cols_out);
/* cos / sin [max_positions, head_dim / 2] and the row permutation [head_dim] of a position encoding. */
int fg_position_tables(const char *kind, const char *params_json, int max_positions, float *cos_out, float *sin_out,
                       int *perm_out);
/* ONE schedule entry's block on rows of the caller: sequence s (slot slots[s]) brings n_tok[s] rows of
 * x [sum n_tok, hidden] (float32, host, updated in place); pages are reserved and committed as in a step. */
int fg_engine_block_forward(fg_engine *e, int schedule_entry, int n_seq, const int *slots, const int *n_tok, float *x);

/* ---------------------------------------------------------------- cache bookkeeping alone (no device memory) */
/* requests_json: [{"entry": 0, "n_kv_heads": 2, "head_dim": 16, "window": null}, ...] */
int fg_cache_create(const char *requests_json, int64_t max_tokens, int max_seq_len, int n_slots, int page_size,
                    fg_cache **out);
void fg_cache_destroy(fg_cache *c);
int fg_cache_acquire(fg_cache *c, int *slot_out);
int fg_cache_release(fg_cache *c, int slot);
int fg_cache_length(const fg_cache *c, int slot, int *out);
int fg_cache_reserve(fg_cache *c, int n, const int *slots, const int *n_new);   /* all or nothing */
int fg_cache_commit(fg_cache *c, int n, const int *slots, const int *n_new);
int fg_cache_pages_needed(const fg_cache *c, int slot, int n_new, int *per_group_out);
int fg_cache_free_pages(const fg_cache *c, int group, int *out);
int fg_cache_block_table(const fg_cache *c, int group, int slot, int width, int *out);
int fg_cache_check(const fg_cache *c);
int fg_cache_info(const fg_cache *c, char **json_out);   /* groups, entries, pages, live slots */
/* Bytes the pools of a cache would take: {"bytes_per_token", "pages", "bytes"}; no allocation. */
int fg_cache_bytes(const char *requests_json, int64_t max_tokens, int page_size, int dtype, char **json_out);

#ifdef __cplusplus
}
#endif
