// The parts a decoder layer is put together from, their interfaces and their registries.
//
// Roles: norm, position encoding, mixer (attention here), feed-forward, the block that arranges them,
// embedding and head.  A part is built from {"kind", "params", "tensors"} of the model spec: its kind is
// looked up in the registry of its role, and its sizes and constants arrive as parameters.  No part knows
// which model it is in; kinds the library does not have are registered from outside through the C
// interface of fastgguf_parts.h (an ExternalPart wraps the caller's table of functions).
//
// The reference expresses the same choices as flags and optional per-layer tensors on one struct
// (fastgguf.c:4064-4100) inside one fixed loop over layers (:4674).
#pragma once
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "cache.hpp"
#include "device.hpp"
#include "json.hpp"

namespace fg {

struct Runtime {
    int dtype = FG_BF16;              // activation / weight dtype: FG_BF16 (serving) or FG_F32 (true 32-bit path)
    int device = 0;
    int n_sm = 148;
    cudaStream_t stream = nullptr;
    Arena *arena = nullptr;           // activations of the step being run
    bool recording = false;           // the step is being recorded into a CUDA graph
    bool plain_kernels = false;       // the safety switch: the any-size FMA kernels everywhere, bfloat16 included
};

struct TensorDecl {
    std::string name;                 // the part's local name
    std::vector<int64_t> shape;
    bool is_int = false;
    int init = 0;                     // random weights: 0 = N(0, std), 1 = 1 + N(0, std)
    float std = 0.02f;
};

// A tensor on the device together with the allocation that holds it (shared: a tied head and the
// embedding are one allocation; a fused matrix replaces the tensors it was made from).
struct Weight {
    std::shared_ptr<DeviceBuffer> buffer;
    Tensor t;
};
Weight make_weight(int64_t rows, int64_t cols, int dtype, const char *what);
// rows of several matrices one after another, converted to `dtype`
Weight concat_rows(const std::vector<Weight> &parts, int dtype, cudaStream_t s);
// out row r = in row rows[r]
Weight gather_rows(const Weight &w, const std::vector<int64_t> &rows, cudaStream_t s);

// The device-side description of one step: which rows belong to which sequence, at which position, with
// which pages.  Rows are laid out sequence after sequence.
struct Batch {
    int n_seq = 0, n_rows = 0, n_want = 0, max_new = 1, max_len = 1;
    bool single_token = true;         // every sequence brings exactly one token (a decode step)
    bool want_all = false;            // the wanted rows are all rows, in order
    const int *tokens = nullptr, *positions = nullptr, *row_seq = nullptr, *cu_rows = nullptr;
    const int *seq_start = nullptr, *slots = nullptr, *want_rows = nullptr;
    std::vector<const int *> block_tables;       // per cache group: [n_seq, table_width] (device)
    int table_width = 0;
    std::vector<int> host_cu_rows, host_seq_start, host_slots;   // empty while a graph records
    fg_batch_view view(cudaStream_t s) const;
};

// What one schedule entry owns or borrows: cache pools and state rows.
struct LayerIO {
    int group = -1;
    void *k_pool = nullptr, *v_pool = nullptr;
    int n_pages = 0, page_size = 64, n_kv_heads = 0, head_dim = 0, cache_dtype = FG_BF16;
    bool write_cache = true;          // false: the cache belongs to an earlier entry
    void *state = nullptr;
    int64_t state_bytes = 0;
    int n_slots = 0;
    fg_layer_io view() const;
};

// An RMSNorm whose 1/rms has not been applied yet: xw = bf16(x * weight) and partial sums of squares of
// each row of x (ss[t, m], t < tiles).  A tensor-core contraction takes xw as its input and applies
// 1/sqrt(sum / size + eps) per row in its epilogue; materialize() gives the normalised rows to anything else.
struct DeferredNorm {
    Tensor xw;
    float *ss = nullptr;
    int tiles = 0, size = 0;
    float eps = 0.f;
    Tensor x;
    const float *weight = nullptr;
    bool defined() const { return xw.defined(); }
    Tensor materialize(Runtime &rt) const;
};

class Part {
public:
    virtual ~Part() = default;
    virtual std::vector<TensorDecl> tensor_decls() const { return {}; }
    virtual void load(const std::map<std::string, Weight> &tensors, Runtime &rt) { (void)tensors; (void)rt; }
};

class Norm : public Part {
public:
    // x: [M, E] f32 residual stream; returns [R, E] in the activation dtype; rows (device) picks rows
    virtual Tensor forward(Runtime &rt, const Tensor &x, const int *rows, int n_rows) = 0;
    // a norm of the form x * rsqrt(mean(x^2) + eps) * w may be started by the contraction before it
    virtual bool deferrable() const { return false; }
    virtual const float *weight() const { return nullptr; }
    virtual float eps() const { return 0.f; }
    virtual int size() const { return 0; }
};

class PositionEncoding : public Part {
public:
    // builds cos / sin [max_positions, head_dim / 2] f32 on the device, for pairs (j, j + head_dim / 2)
    virtual void prepare(Runtime &rt, int max_positions) = 0;
    virtual const float *cos_table() const = 0;
    virtual const float *sin_table() const = 0;
    virtual int head_dim() const = 0;
    // perm[i]: the stored row of a head that becomes row i (empty = identity)
    virtual const std::vector<int> &permutation() const = 0;
};

class Mixer : public Part {
public:
    virtual bool cache_request(CacheRequest *out) const { (void)out; return false; }
    virtual int64_t state_bytes() const { return 0; }
    virtual bool supports_deferred_norm() const { return false; }
    // adds its output into residual ([M, E] f32).  xn: normalised rows, or (deferred) a started norm;
    // emit_norm: start this norm from the updated residual and return it (only with supports_deferred_norm)
    virtual DeferredNorm forward(Runtime &rt, const Tensor &xn, const DeferredNorm *deferred, const Batch &batch,
                                 const LayerIO &io, Tensor &residual, Norm *emit_norm) = 0;
    // called once when the cache exists (tables for the longest sequence)
    virtual void prepare(Runtime &rt, int max_positions) { (void)rt; (void)max_positions; }
};

class FeedForward : public Part {
public:
    virtual bool supports_deferred_norm() const { return false; }
    virtual DeferredNorm forward(Runtime &rt, const Tensor &xn, const DeferredNorm *deferred, const Batch &batch,
                                 Tensor &residual, Norm *emit_norm) = 0;
};

// An arrangement of a mixer, a feed-forward and their norms around the residual stream.
class Block {
public:
    virtual ~Block() = default;
    Mixer *mixer = nullptr;
    FeedForward *feed_forward = nullptr;
    Norm *mixer_norm = nullptr, *feed_forward_norm = nullptr;
    // Runs the block on x in place.  pending: the mixer's norm already started by whoever produced x;
    // next_norm: the norm that will read x after this block, to be started by the block's last projection.
    // Returns the started next_norm (or an undefined DeferredNorm).
    virtual DeferredNorm forward(Runtime &rt, Tensor &x, const Batch &batch, const LayerIO &io, const DeferredNorm &pending,
                                 Norm *next_norm) = 0;
};

class Embedding : public Part {
public:
    // fills x [M, E] f32; with emit_norm (deferrable) may also start that norm
    virtual DeferredNorm forward(Runtime &rt, const Batch &batch, Tensor &x, Norm *emit_norm) = 0;
};

class Head : public Part {
public:
    virtual bool supports_deferred_norm() const { return false; }
    // float32 logits [rows, vocab] of normalised rows
    virtual Tensor forward(Runtime &rt, const Tensor &xn, const DeferredNorm *deferred) = 0;
};

// ---- registries, one per role
struct BuildContext;                               // resolves nested parts (shared position encodings)
using PartFactory = std::function<std::unique_ptr<Part>(Runtime &, const Json &params, BuildContext &)>;
using BlockFactory = std::function<std::unique_ptr<Block>(Runtime &)>;

struct BuildContext {
    // the shared instance of a nested part {"kind", "params"} of `role`
    std::function<Part *(int role, const Json &nested)> nested;
};

void register_part_factory(int role, const std::string &kind, PartFactory f);
void register_block_factory(const std::string &kind, BlockFactory f);
std::unique_ptr<Part> build_part(int role, const std::string &kind, Runtime &rt, const Json &params, BuildContext &ctx);
std::unique_ptr<Block> build_block(const std::string &kind, Runtime &rt);
const char *role_name(int role);
void register_external_part(int role, const std::string &kind, const fg_part_vtable &vt);

// parameter access with the messages of a spec error
long long param_int(const Json &params, const char *key, const char *part);
long long param_int(const Json &params, const char *key, long long dflt, const char *part);
double param_float(const Json &params, const char *key, const char *part);
double param_float(const Json &params, const char *key, double dflt, const char *part);

// ---- a weight matrix [out, in] and the choice of contraction kernel for it
// y = W x with no bias, W row-major [out, in] as in the checkpoint and as the reference keeps it
// (fastgguf.c:2582-2585).  The reference picks a kernel by tensor type and batch size inside
// matvec / matmul (:2575-2622, :3004-3093); here the choice is by dtype, row count and alignment:
// float32 operands, or sizes the fast kernels refuse -> the plain FMA kernel; bfloat16 with few rows
// (decode) -> the weight-streaming tensor-core kernel; bfloat16 with many rows -> the tiled tcgen05 kernel.
class Linear {
public:
    Linear() = default;
    explicit Linear(Weight w);
    Linear rows(int64_t begin, int64_t end) const;       // shares storage
    bool defined() const { return w_.t.defined(); }
    int64_t out_features() const { return w_.t.rows; }
    int64_t in_features() const { return w_.t.cols; }
    const Weight &weight() const { return w_; }
    // out[m, n] (+)= sum_k a[m, k] W[n, k].  `out` undefined: allocated in the arena as out_dtype.
    // accumulate adds into a float32 out.  deferred: a is deferred->xw.  emit_norm (needs accumulate): the
    // next norm started from the updated out when the tensor-core kernel ran (undefined when the plain one did).
    Tensor forward(Runtime &rt, const Tensor &a, const DeferredNorm *deferred, Tensor out, int out_dtype, bool accumulate,
                   Norm *emit_norm, DeferredNorm *emitted) const;
    // silu(a gate^T) * (a up^T) as bf16 [M, F] from rows interleaved in blocks of 64; false if refused
    bool forward_silu(Runtime &rt, const Tensor &a, const DeferredNorm *deferred, Tensor *out) const;

private:
    Weight w_;
    bool fast_ = false;
};

// Rotary encoding of q (and k), cache append (when the entry owns its cache) and attention of a step's
// rows; picks kernels by dtype, sizes and step shape.  qkv: [M, H*hd (+ 2*KV*hd)].
Tensor rope_attention(Runtime &rt, const Tensor &qkv, const Batch &batch, const LayerIO &io, const float *cos_t,
                      const float *sin_t, int n_heads, int n_kv_heads, int head_dim, float scale, int window);
int decode_splits(int n_sm, int n_seq, int n_heads, int n_kv_heads, int table_width, int head_dim);

// llama3 frequency divisors per rotary pair (all ones without scaling)
std::vector<double> rotary_divisors(int rotary_dim, double theta, const Json &scaling);

}  // namespace fg
