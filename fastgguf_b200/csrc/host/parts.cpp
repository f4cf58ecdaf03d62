// See parts.hpp.  Built-in kinds: rmsnorm, rope, gqa_attention, swiglu, prenorm, embedding, lm_head; and
// the adapter that runs a part registered from outside through fastgguf_parts.h.
#include "parts.hpp"

#include <cmath>
#include <cstring>
#include <mutex>

namespace fg {

static const int EPI_BF16 = 0, EPI_F32 = 1, EPI_ADD_F32 = 2, EPI_SILU_MUL = 3;
static const int KERNEL_BAD_SIZE = 10002;

const char *role_name(int role) {
    static const char *n[] = {"norm", "position", "mixer", "feed_forward", "block", "embedding", "head"};
    return role >= 0 && role <= 6 ? n[role] : "?";
}

// ------------------------------------------------------------------------------------ parameters
static const Json &need(const Json &params, const char *key, const char *part) {
    const Json *v = params.find(key);
    if (!v || v->is_null()) fail(FG_E_CONFIG, format("%s: parameter '%s' is missing", part, key));
    return *v;
}
long long param_int(const Json &params, const char *key, const char *part) {
    const Json &v = need(params, key, part);
    if (!v.is_int() && !(v.is_number() && v.as_double() == std::floor(v.as_double())))
        fail(FG_E_CONFIG, format("%s: parameter '%s' must be an integer, got %s", part, key, v.dump().c_str()));
    return v.is_int() ? v.as_int() : (long long)v.as_double();
}
long long param_int(const Json &params, const char *key, long long dflt, const char *part) {
    const Json *v = params.find(key);
    return (!v || v->is_null()) ? dflt : param_int(params, key, part);
}
double param_float(const Json &params, const char *key, const char *part) {
    const Json &v = need(params, key, part);
    if (!v.is_number() || v.is_bool()) fail(FG_E_CONFIG, format("%s: parameter '%s' must be a number, got %s", part, key, v.dump().c_str()));
    return v.as_double();
}
double param_float(const Json &params, const char *key, double dflt, const char *part) {
    const Json *v = params.find(key);
    return (!v || v->is_null()) ? dflt : param_float(params, key, part);
}

// ------------------------------------------------------------------------------------ views
fg_batch_view Batch::view(cudaStream_t s) const {
    fg_batch_view v = {};
    v.n_seq = n_seq; v.n_rows = n_rows; v.n_want = n_want; v.max_new = max_new; v.max_len = max_len;
    v.single_token = single_token; v.want_all = want_all;
    v.tokens = tokens; v.positions = positions; v.row_seq = row_seq; v.cu_rows = cu_rows;
    v.seq_start = seq_start; v.slots = slots; v.want_rows = want_rows;
    v.n_groups = (int)block_tables.size();
    v.block_tables = block_tables.empty() ? nullptr : block_tables.data();
    v.table_width = table_width;
    v.host_cu_rows = host_cu_rows.empty() ? nullptr : host_cu_rows.data();
    v.host_seq_start = host_seq_start.empty() ? nullptr : host_seq_start.data();
    v.host_slots = host_slots.empty() ? nullptr : host_slots.data();
    v.stream = s;
    return v;
}

fg_layer_io LayerIO::view() const {
    fg_layer_io v = {};
    v.group = group; v.k_pool = k_pool; v.v_pool = v_pool; v.n_pages = n_pages; v.page_size = page_size;
    v.n_kv_heads = n_kv_heads; v.head_dim = head_dim; v.cache_dtype = cache_dtype; v.write_cache = write_cache;
    v.state = state; v.state_bytes = state_bytes; v.n_slots = n_slots;
    return v;
}

// ------------------------------------------------------------------------------------ weights
Weight make_weight(int64_t rows, int64_t cols, int dtype, const char *what) {
    Weight w;
    w.buffer = std::make_shared<DeviceBuffer>((size_t)rows * (size_t)cols * elem_size(dtype), what);
    w.t.data = w.buffer->get();
    w.t.dtype = dtype;
    w.t.rows = rows;
    w.t.cols = cols;
    w.t.ld = cols;
    return w;
}

Weight concat_rows(const std::vector<Weight> &parts, int dtype, cudaStream_t s) {
    int64_t rows = 0, cols = parts.at(0).t.cols;
    for (auto &p : parts) {
        if (p.t.cols != cols || p.t.ld != p.t.cols) fail(FG_E_INTERNAL, "concat_rows: parts must be contiguous and equally wide");
        rows += p.t.rows;
    }
    Weight out = make_weight(rows, cols, dtype, "a fused weight matrix");
    int64_t at = 0;
    for (auto &p : parts) {
        dev_convert(p.t.data, p.t.dtype, (char *)out.t.data + at * cols * elem_size(dtype), dtype, p.t.numel(), s);
        at += p.t.rows;
    }
    return out;
}

Weight gather_rows(const Weight &w, const std::vector<int64_t> &rows, cudaStream_t s) {
    if (w.t.ld != w.t.cols) fail(FG_E_INTERNAL, "gather_rows: the matrix must be contiguous");
    Weight out = make_weight((int64_t)rows.size(), w.t.cols, w.t.dtype, "a permuted weight matrix");
    dev_gather_rows(w.t.data, out.t.data, rows, w.t.cols, w.t.dtype, s);
    return out;
}

static const Weight &tensor_of(const std::map<std::string, Weight> &tensors, const char *name) {
    auto it = tensors.find(name);
    if (it == tensors.end()) fail(FG_E_INTERNAL, format("a part was not given its tensor '%s'", name));
    return it->second;
}

// ------------------------------------------------------------------------------------ deferred norm
Tensor DeferredNorm::materialize(Runtime &rt) const {
    Tensor out = rt.arena->matrix(x.rows, x.cols, FG_BF16);
    FG_LAUNCH("core", fg_rmsnorm, x.ptr<float>(), weight, nullptr, out.data, FG_BF16, (int)x.rows, (int)x.cols, eps, rt.stream);
    return out;
}

// ------------------------------------------------------------------------------------ Linear
Linear::Linear(Weight w) : w_(std::move(w)) {
    const Tensor &t = w_.t;
    fast_ = t.dtype == FG_BF16 && t.cols % 8 == 0 && t.ld % 8 == 0 && ((uintptr_t)t.data % 16) == 0;
}

Linear Linear::rows(int64_t begin, int64_t end) const {
    Weight w = w_;
    w.t = w_.t.row_range(begin, end);
    return Linear(w);
}

Tensor Linear::forward(Runtime &rt, const Tensor &a_in, const DeferredNorm *deferred, Tensor out, int out_dtype, bool accumulate,
                       Norm *emit_norm, DeferredNorm *emitted) const {
    if (emitted) *emitted = DeferredNorm();
    const Tensor &W = w_.t;
    Tensor a = deferred ? deferred->xw : a_in;
    const int64_t M = a.rows, K = a.cols, N = W.rows;
    if (K != W.cols) fail(FG_E_INTERNAL, format("contraction: the input is [%lld, %lld] but the weight is [%lld, %lld]", (long long)M, (long long)K, (long long)N, (long long)W.cols));
    if (accumulate && (!out.defined() || out.dtype != FG_F32))
        fail(FG_E_INTERNAL, "contraction: the residual sum is 32-bit; accumulate needs a float32 output");
    if (!out.defined()) out = rt.arena->matrix(M, N, out_dtype);
    if (out.rows != M || out.cols != N) fail(FG_E_INTERNAL, "contraction: the output has the wrong shape");
    if (M == 0) return out;
    if (fast_ && !rt.plain_kernels && a.dtype == FG_BF16 && (out.dtype == FG_BF16 || out.dtype == FG_F32)) {
        int epi = accumulate ? EPI_ADD_F32 : out.dtype == FG_BF16 ? EPI_BF16 : EPI_F32;
        const float *ss_in = nullptr;
        int ss_tiles = 0, ss_size = 1;
        float ss_eps = 0.f;
        if (deferred) { ss_in = deferred->ss; ss_tiles = deferred->tiles; ss_size = deferred->size; ss_eps = deferred->eps; }
        Tensor xw_out;
        float *ss_out = nullptr;
        const float *norm_w = nullptr;
        bool emit = emit_norm && emitted && accumulate && emit_norm->deferrable() && emit_norm->size() == N;
        if (emit) {
            norm_w = emit_norm->weight();
            xw_out = rt.arena->matrix(M, N, FG_BF16);
            int max_tiles = FG_KERNEL("tc", fg_gemm_tc_max_ss_tiles)((int)N);
            ss_out = (float *)rt.arena->alloc((size_t)max_tiles * (size_t)M * sizeof(float));
        }
        int tiles_out = 0;
        count_launch();
        ProfileScope scope("fg_gemm_tc", profile_on() ? format("%lld x %lld, %lld rows%s", (long long)N, (long long)K, (long long)M, accumulate ? ", residual add" : "").c_str() : nullptr);
        // scratch memory for a split along K (a prompt of a few hundred rows through a projection of few output tiles)
        const long long ws_bytes = FG_KERNEL("tc", fg_gemm_tc_workspace_bytes)((int)M, (int)N, (int)K, epi);
        void *ws = ws_bytes > 0 ? rt.arena->alloc((size_t)ws_bytes) : nullptr;
        int code = FG_KERNEL("tc", fg_gemm_tc_ws)(a.data, (int)a.ld, W.data, (int)W.ld, out.data, (int)out.ld, epi, (int)M, (int)N,
                                                  (int)K, 0, ss_in, ss_tiles, ss_size, ss_eps, norm_w, xw_out.data, ss_out,
                                                  &tiles_out, ws, ws_bytes, rt.stream);
        if (code != KERNEL_BAD_SIZE) {
            check_kernel(code, "fg_gemm_tc");
            if (emit) {
                emitted->xw = xw_out; emitted->ss = ss_out; emitted->tiles = tiles_out; emitted->size = (int)N;
                emitted->eps = emit_norm->eps(); emitted->x = out; emitted->weight = norm_w;
            }
            return out;
        }
    }
    if (deferred) a = deferred->materialize(rt);
    FG_LAUNCH("core", fg_gemm_generic, a.data, a.dtype, (int)a.ld, W.data, W.dtype, (int)W.ld, out.data, out.dtype, (int)out.ld,
              accumulate ? 1 : 0, (int)M, (int)N, (int)K, rt.stream);
    return out;
}

bool Linear::forward_silu(Runtime &rt, const Tensor &a_in, const DeferredNorm *deferred, Tensor *out) const {
    const Tensor &W = w_.t;
    Tensor a = deferred ? deferred->xw : a_in;
    if (!fast_ || rt.plain_kernels || a.dtype != FG_BF16 || W.rows % 128) return false;
    const int64_t M = a.rows, F = W.rows / 2;
    Tensor t = rt.arena->matrix(M, F, FG_BF16);
    if (M == 0) { *out = t; return true; }
    const float *ss_in = nullptr;
    int ss_tiles = 0, ss_size = 1, tiles_out = 0;
    float ss_eps = 0.f;
    if (deferred) { ss_in = deferred->ss; ss_tiles = deferred->tiles; ss_size = deferred->size; ss_eps = deferred->eps; }
    count_launch();
    ProfileScope scope("fg_gemm_tc", profile_on() ? format("%lld x %lld, %lld rows, silu", (long long)W.rows, (long long)a.cols, (long long)M).c_str() : nullptr);
    int code = FG_KERNEL("tc", fg_gemm_tc)(a.data, (int)a.ld, W.data, (int)W.ld, t.data, (int)t.ld, EPI_SILU_MUL, (int)M,
                                           (int)W.rows, (int)a.cols, 0, ss_in, ss_tiles, ss_size, ss_eps, nullptr, nullptr,
                                           nullptr, &tiles_out, rt.stream);
    if (code == KERNEL_BAD_SIZE) return false;
    check_kernel(code, "fg_gemm_tc (silu)");
    *out = t;
    return true;
}

// ------------------------------------------------------------------------------------ attention ops
// How many CTAs share one sequence's pages in a decode step: about one and a half CTAs per SM in all, and
// never more than fit on the GPU at once - three per SM at head size 64, one at 128 (each warp holds a K and
// a V page in shared memory).  What does not fit runs as a second wave whose page loads start late; measured
// at batch 8 with 8 KV heads and head size 64, 4 splits (256 CTAs) beat both 2 and 8, and at head size 128
// two splits beat four.  Up to 8 splits (a power of two) are merged inside a thread-block cluster; only
// contexts beyond 16K positions take more splits and the scratch-memory path.
int decode_splits(int n_sm, int n_seq, int n_heads, int n_kv_heads, int table_width, int head_dim) {
    int ctas = n_seq * n_kv_heads * ((n_heads / n_kv_heads + 15) / 16);
    int want = head_dim <= 64 ? (3 * n_sm / 2 + ctas - 1) / ctas : n_sm / ctas;
    want = std::max(1, std::min(want, table_width));
    if (want > 8 && table_width > 256) return want;
    int s = 1;
    while (s < want && s < 8) s *= 2;
    return s;
}

static bool fast_attention_ok(const Runtime &rt, const Tensor &q, const LayerIO &io, int head_dim) {
    return !rt.plain_kernels && q.dtype == FG_BF16 && io.cache_dtype == FG_BF16 && (head_dim == 64 || head_dim == 128) && io.page_size == 64 &&
           q.ld % 2 == 0 && ((uintptr_t)q.data % 4) == 0;
}

static Tensor attention(Runtime &rt, const Tensor &q, const Batch &b, const LayerIO &io, int H, int KV, int hd, float scale,
                        int window) {
    const int *table = b.block_tables.at((size_t)io.group);
    Tensor out = rt.arena->matrix(q.rows, (int64_t)H * hd, q.dtype);
    if (fast_attention_ok(rt, q, io, hd)) {
        if (b.single_token) {
            int n_splits = decode_splits(rt.n_sm, b.n_seq, H, KV, b.table_width, hd);
            float *part_o = nullptr, *part_ml = nullptr;
            if (n_splits != 1 && n_splits != 2 && n_splits != 4 && n_splits != 8) {      // very long contexts
                part_o = (float *)rt.arena->alloc((size_t)b.n_seq * H * n_splits * hd * sizeof(float));
                part_ml = (float *)rt.arena->alloc((size_t)b.n_seq * H * n_splits * 2 * sizeof(float));
            }
            FG_LAUNCH("attn", fg_attention_decode, q.data, (int)q.ld, out.data, (int)out.ld, b.positions, table, b.table_width,
                      io.k_pool, io.v_pool, b.n_seq, H, KV, hd, io.page_size, scale, window, n_splits, part_o, part_ml, rt.stream);
            return out;
        }
        // Many new tokens: 128-row tiles on the tcgen05 tensor cores.  A few rows (a sequence fed in short
        // pieces) waste less of the mma.sync kernel's 64-row tile.
        bool tc = b.max_new * (H / KV) >= 64 && q.ld % 8 == 0 && ((uintptr_t)q.data % 16) == 0;
        if (tc)
            FG_LAUNCH("attn", fg_attention_prefill_tc, q.data, (int)q.ld, out.data, (int)out.ld, b.cu_rows, b.seq_start, table,
                      b.table_width, io.k_pool, io.v_pool, io.n_pages, b.n_seq, b.max_new, H, KV, hd, io.page_size, scale, window,
                      rt.stream);
        else
            FG_LAUNCH("attn", fg_attention_prefill, q.data, (int)q.ld, out.data, (int)out.ld, b.cu_rows, b.seq_start, table,
                      b.table_width, io.k_pool, io.v_pool, b.n_seq, b.max_new, H, KV, hd, io.page_size, scale, window, rt.stream);
        return out;
    }
    if (q.dtype != io.cache_dtype) fail(FG_E_INTERNAL, "attention: q and the cache must share a dtype");
    if (hd > 256) fail(FG_E_KERNEL, format("attention: head_dim %d exceeds 256, the largest the any-size kernel takes", hd));
    FG_LAUNCH("core", fg_attention_generic, q.data, (int)q.ld, out.data, (int)out.ld, q.dtype, b.positions, b.row_seq, table,
              b.table_width, io.k_pool, io.v_pool, (int)q.rows, H, KV, hd, io.page_size, scale, window, rt.stream);
    return out;
}

Tensor rope_attention(Runtime &rt, const Tensor &qkv, const Batch &b, const LayerIO &io, const float *cos_t, const float *sin_t,
                      int H, int KV, int hd, float scale, int window) {
    if (io.group < 0 || !io.k_pool) fail(FG_E_INTERNAL, "attention: the schedule entry has no cache");
    const int *table = b.block_tables.at((size_t)io.group);
    // A decode step in bfloat16 with head size 64 / 128 on the entry's own cache runs as ONE kernel.  It reads
    // positions, the page table and its own pages before waiting for the kernel in front of it; see common.cuh
    // for why that is allowed here and only here.
    if (io.write_cache && b.single_token && fast_attention_ok(rt, qkv, io, hd) && qkv.ld % 8 == 0 && ((uintptr_t)qkv.data % 16) == 0) {
        int n_splits = decode_splits(rt.n_sm, b.n_seq, H, KV, b.table_width, hd);
        if (n_splits == 1 || n_splits == 2 || n_splits == 4 || n_splits == 8) {
            Tensor out = rt.arena->matrix(qkv.rows, (int64_t)H * hd, FG_BF16);
            FG_LAUNCH("attn", fg_attention_decode_fused, qkv.data, (int)qkv.ld, out.data, (int)out.ld, b.positions, table,
                      b.table_width, io.k_pool, io.v_pool, cos_t, sin_t, b.n_seq, H, KV, hd, io.page_size, scale, window, n_splits,
                      rt.stream);
            return out;
        }
    }
    FG_LAUNCH("core", fg_rope_append, qkv.data, qkv.dtype, (int)qkv.ld, b.positions, b.row_seq, table, b.table_width,
              io.write_cache ? io.k_pool : nullptr, io.write_cache ? io.v_pool : nullptr, cos_t, sin_t, (int)qkv.rows, H, KV, hd,
              io.page_size, io.write_cache ? 1 : 0, rt.stream);
    return attention(rt, qkv, b, io, H, KV, hd, scale, window);
}

// ------------------------------------------------------------------------------------ RMSNorm
// y = x * (1 / sqrt(mean(x^2) + eps)) * w; the weight multiplies directly (no +1), in the order x * inv * w
// (rmsnorm_w, fastgguf.c:3100-3105).  Statistics are 32-bit here (the reference sums in double).
class RMSNorm : public Norm {
public:
    RMSNorm(const Json &p) : size_((int)param_int(p, "size", "rmsnorm")), eps_((float)param_float(p, "eps", "rmsnorm")) {
        if (size_ <= 0 || !(eps_ > 0.f)) fail(FG_E_CONFIG, "rmsnorm: size and eps must be positive");
    }
    std::vector<TensorDecl> tensor_decls() const override { return {{"weight", {size_}, false, 1, 0.01f}}; }
    void load(const std::map<std::string, Weight> &tensors, Runtime &rt) override {
        const Weight &w = tensor_of(tensors, "weight");
        // widening bf16 -> f32 is exact; the kernels read the weight as f32
        if (w.t.dtype == FG_F32) w_ = w;
        else w_ = concat_rows({w}, FG_F32, rt.stream);
    }
    Tensor forward(Runtime &rt, const Tensor &x, const int *rows, int n_rows) override {
        int R = rows ? n_rows : (int)x.rows;
        Tensor out = rt.arena->matrix(R, x.cols, rt.dtype);
        if (R > 0)
            FG_LAUNCH("core", fg_rmsnorm, x.ptr<float>(), w_.t.ptr<float>(), rows, out.data, rt.dtype, R, (int)x.cols, eps_, rt.stream);
        return out;
    }
    bool deferrable() const override { return true; }
    const float *weight() const override { return w_.t.ptr<float>(); }
    float eps() const override { return eps_; }
    int size() const override { return size_; }

private:
    int size_;
    float eps_;
    Weight w_;
};

// ------------------------------------------------------------------------------------ rotary encoding
// apply_rope (fastgguf.c:3123-3145): for pair j of a head, angle = pos / theta^(2j / n_rot), divided by
// freq_factors[j] when the model file carries such a vector (:3131), computed in double and rounded to float
// (:3130-3133); the pair is rotated by (a, b) <- (a cos - b sin, a sin + b cos) (:3140-3141).  Pair members
// are (j, j + n_rot/2) ("halves", the row order of model folders; the neox branch of :3138-3139) or adjacent
// (2j, 2j + 1) (the reference's own Llama layout).  The kernels rotate pairs (j, j + head_dim/2) of a head, so
// any other pairing, and a rotary dimension smaller than the head, is brought to that form by permuting the
// rows of the q and k projections once at load (scores do not change under a common permutation of q and k)
// and by identity entries (cos 1, sin 0) for the dimensions that are not rotated.
//
// The llama3 divisors are what GGUF files store as rope_freqs.weight (fastgguf.c:4278); the reference has no
// code that computes them.  With base frequency f_j = theta^(-2j/n_rot) and wavelength l_j = 2 pi / f_j:
//     l_j < orig / high_freq_factor   -> divisor 1                   (high frequencies: untouched)
//     l_j > orig / low_freq_factor    -> divisor factor              (low frequencies: slowed)
//     else  s = (orig / l_j - low) / (high - low);  divisor = 1 / ((1 - s) / factor + s)
std::vector<double> rotary_divisors(int rotary_dim, double theta, const Json &scaling) {
    int half = rotary_dim / 2;
    std::vector<double> div((size_t)half, 1.0);
    if (!scaling.is_object()) return div;
    const Json &kind = scaling.get("rope_type");
    if (kind.is_null() || (kind.is_string() && kind.as_string() == "default")) return div;
    if (!kind.is_string() || kind.as_string() != "llama3")
        fail(FG_E_CONFIG, "rotary scaling " + kind.dump() + " is not known (known: default, llama3)");
    double factor = param_float(scaling, "factor", "rope scaling"), low = param_float(scaling, "low_freq_factor", "rope scaling");
    double high = param_float(scaling, "high_freq_factor", "rope scaling");
    double orig = param_float(scaling, "original_max_position_embeddings", "rope scaling");
    const double two_pi = 2.0 * 3.14159265358979323846;
    for (int j = 0; j < half; j++) {
        double freq = std::pow(theta, -2.0 * j / rotary_dim);
        double wavelen = two_pi / freq;
        if (wavelen < orig / high) div[(size_t)j] = 1.0;
        else if (wavelen > orig / low) div[(size_t)j] = factor;
        else {
            double smooth = (orig / wavelen - low) / (high - low);
            div[(size_t)j] = 1.0 / ((1.0 - smooth) / factor + smooth);
        }
    }
    return div;
}

class RotaryEncoding : public PositionEncoding {
public:
    RotaryEncoding(const Json &p) {
        hd_ = (int)param_int(p, "head_dim", "rope");
        theta_ = param_float(p, "theta", "rope");
        n_rot_ = (int)param_int(p, "rotary_dim", hd_, "rope");
        scaling_ = p.get("scaling");
        std::string layout = p.get("layout").is_string() ? p.get("layout").as_string() : "halves";
        if (hd_ <= 0 || hd_ % 2) fail(FG_E_CONFIG, format("rope: head_dim must be even and positive, got %d", hd_));
        if (n_rot_ <= 0 || n_rot_ % 2 || n_rot_ > hd_)
            fail(FG_E_CONFIG, format("rope: rotary_dim must be even, positive and at most head_dim, got %d", n_rot_));
        if (layout != "halves" && layout != "adjacent")
            fail(FG_E_CONFIG, "rope: layout '" + layout + "' is not known (known: halves, adjacent)");
        if (!(theta_ > 0)) fail(FG_E_CONFIG, "rope: theta must be positive");
        rotary_divisors(n_rot_, theta_, scaling_);           // refuses unknown scaling kinds at build time
        adjacent_ = layout == "adjacent";
        if (adjacent_ || n_rot_ != hd_) {
            // canonical row i < hd/2 pairs with i + hd/2; first the rotated pairs, then the untouched dimensions
            perm_.assign((size_t)hd_, 0);
            int half = hd_ / 2, rh = n_rot_ / 2, rest = (hd_ - n_rot_) / 2;
            for (int j = 0; j < rh; j++) {
                perm_[(size_t)j] = adjacent_ ? 2 * j : j;
                perm_[(size_t)(half + j)] = adjacent_ ? 2 * j + 1 : j + rh;
            }
            for (int t = 0; t < rest; t++) {
                perm_[(size_t)(rh + t)] = n_rot_ + t;
                perm_[(size_t)(half + rh + t)] = n_rot_ + rest + t;
            }
        }
    }
    void prepare(Runtime &rt, int max_positions) override {
        if (cos_.buffer && max_positions_ >= max_positions) return;
        int half = hd_ / 2, rh = n_rot_ / 2;
        std::vector<double> div = rotary_divisors(n_rot_, theta_, scaling_);
        std::vector<double> inv((size_t)rh);
        for (int j = 0; j < rh; j++) inv[(size_t)j] = std::pow(theta_, -2.0 * j / n_rot_) / div[(size_t)j];
        std::vector<float> c((size_t)max_positions * half), s((size_t)max_positions * half);
        for (int pos = 0; pos < max_positions; pos++) {
            for (int j = 0; j < half; j++) {
                double ang = j < rh ? (double)pos * inv[(size_t)j] : 0.0;
                c[(size_t)pos * half + j] = (float)std::cos(ang);
                s[(size_t)pos * half + j] = (float)std::sin(ang);
            }
        }
        cos_ = make_weight(max_positions, half, FG_F32, "rotary tables");
        sin_ = make_weight(max_positions, half, FG_F32, "rotary tables");
        FG_CUDA(cudaMemcpyAsync(cos_.t.data, c.data(), c.size() * 4, cudaMemcpyHostToDevice, rt.stream));
        FG_CUDA(cudaMemcpyAsync(sin_.t.data, s.data(), s.size() * 4, cudaMemcpyHostToDevice, rt.stream));
        FG_CUDA(cudaStreamSynchronize(rt.stream));
        max_positions_ = max_positions;
    }
    const float *cos_table() const override { return cos_.t.ptr<float>(); }
    const float *sin_table() const override { return sin_.t.ptr<float>(); }
    int head_dim() const override { return hd_; }
    const std::vector<int> &permutation() const override { return perm_; }

private:
    int hd_ = 0, n_rot_ = 0, max_positions_ = 0;
    double theta_ = 0;
    bool adjacent_ = false;
    Json scaling_;
    std::vector<int> perm_;
    Weight cos_, sin_;
};

// no position encoding: identity tables (cos 1, sin 0), so that the same kernels append keys and values
class NoPosition : public PositionEncoding {
public:
    explicit NoPosition(int hd) : hd_(hd) {}
    void prepare(Runtime &rt, int max_positions) override {
        if (cos_.buffer && max_positions_ >= max_positions) return;
        int half = hd_ / 2;
        std::vector<float> c((size_t)max_positions * half, 1.0f);
        cos_ = make_weight(max_positions, half, FG_F32, "identity rotation tables");
        sin_ = make_weight(max_positions, half, FG_F32, "identity rotation tables");
        FG_CUDA(cudaMemcpyAsync(cos_.t.data, c.data(), c.size() * 4, cudaMemcpyHostToDevice, rt.stream));
        FG_CUDA(cudaMemsetAsync(sin_.t.data, 0, c.size() * 4, rt.stream));
        FG_CUDA(cudaStreamSynchronize(rt.stream));
        max_positions_ = max_positions;
    }
    const float *cos_table() const override { return cos_.t.ptr<float>(); }
    const float *sin_table() const override { return sin_.t.ptr<float>(); }
    int head_dim() const override { return hd_; }
    const std::vector<int> &permutation() const override { return perm_; }

private:
    int hd_, max_positions_ = 0;
    std::vector<int> perm_;
    Weight cos_, sin_;
};

// ------------------------------------------------------------------------------------ attention mixer
// GQAAttention(hidden_size, n_heads, n_kv_heads, head_dim, position, scale, window).  Reference, per token
// (fastgguf.c): q, k, v projections in one fused pass (:4692-4696), rotary encoding of q and k (:4702, :4718),
// K stored after rotation and V raw at the token's position (:4720, :4738-4739), scale = 1/sqrt(head_dim)
// (:4744), each query head h attends with KV head h / (H / KV) (:4781) to positions [start, pos] (:4754-4758),
// softmax and value sum (attn_rows :3273-3326), output projection added onto the un-normalized input
// (:4860-4862).  A run that borrows the cache of an earlier entry computes only q and attends to the owner's
// keys and values (the reference's shared-KV layers, :4745-4751).
class GQAAttention : public Mixer {
public:
    GQAAttention(const Json &p, BuildContext &ctx) {
        const char *me = "gqa_attention";
        E_ = (int)param_int(p, "hidden_size", me);
        H_ = (int)param_int(p, "n_heads", me);
        KV_ = (int)param_int(p, "n_kv_heads", me);
        hd_ = (int)param_int(p, "head_dim", me);
        if (E_ <= 0 || H_ <= 0 || KV_ <= 0 || hd_ <= 0) fail(FG_E_CONFIG, "gqa_attention: sizes must be positive");
        if (H_ % KV_) fail(FG_E_CONFIG, format("gqa_attention: %d heads are not a multiple of %d KV heads", H_, KV_));
        if (hd_ % 2) fail(FG_E_CONFIG, format("gqa_attention: head_dim must be even, got %d", hd_));
        scale_ = (float)param_float(p, "scale", 1.0 / std::sqrt((double)hd_), me);
        window_ = (int)param_int(p, "window", 0, me);
        if (window_ < 0) fail(FG_E_CONFIG, "gqa_attention: window cannot be negative");
        const Json &pos = p.get("position");
        if (pos.is_null()) {
            own_position_ = std::make_unique<NoPosition>(hd_);
            position_ = own_position_.get();
        } else {
            position_ = dynamic_cast<PositionEncoding *>(ctx.nested(FG_ROLE_POSITION, pos));
            if (!position_) fail(FG_E_CONFIG, "gqa_attention: 'position' is not a position encoding");
            if (position_->head_dim() != hd_)
                fail(FG_E_CONFIG, format("gqa_attention: the position encoding is built for head_dim %d, the mixer has %d",
                                         position_->head_dim(), hd_));
        }
    }
    std::vector<TensorDecl> tensor_decls() const override {
        int64_t Q = (int64_t)H_ * hd_, D = (int64_t)KV_ * hd_;
        return {{"q_proj.weight", {Q, E_}}, {"k_proj.weight", {D, E_}}, {"v_proj.weight", {D, E_}}, {"o_proj.weight", {E_, Q}}};
    }
    bool cache_request(CacheRequest *out) const override {
        out->n_kv_heads = KV_; out->head_dim = hd_; out->window = window_;
        return true;
    }
    bool supports_deferred_norm() const override { return true; }
    void load(const std::map<std::string, Weight> &tensors, Runtime &rt) override {
        Weight q = tensor_of(tensors, "q_proj.weight"), k = tensor_of(tensors, "k_proj.weight");
        const Weight &v = tensor_of(tensors, "v_proj.weight");
        const std::vector<int> &perm = position_->permutation();
        if (!perm.empty()) {
            auto head_rows = [&](int heads) {
                std::vector<int64_t> rows;
                for (int h = 0; h < heads; h++)
                    for (int i = 0; i < hd_; i++) rows.push_back((int64_t)h * hd_ + perm[(size_t)i]);
                return rows;
            };
            q = gather_rows(q, head_rows(H_), rt.stream);
            k = gather_rows(k, head_rows(KV_), rt.stream);
        }
        int dt = (q.t.dtype == k.t.dtype && k.t.dtype == v.t.dtype) ? q.t.dtype : FG_F32;
        qkv_ = Linear(concat_rows({q, k, v}, dt, rt.stream));
        q_only_ = qkv_.rows(0, (int64_t)H_ * hd_);
        o_ = Linear(tensor_of(tensors, "o_proj.weight"));
    }
    void prepare(Runtime &rt, int max_positions) override { position_->prepare(rt, max_positions); }
    DeferredNorm forward(Runtime &rt, const Tensor &xn, const DeferredNorm *deferred, const Batch &batch, const LayerIO &io,
                         Tensor &residual, Norm *emit_norm) override {
        const Linear &proj = io.write_cache ? qkv_ : q_only_;
        Tensor qkv = proj.forward(rt, xn, deferred, Tensor(), rt.dtype, false, nullptr, nullptr);
        Tensor attn = rope_attention(rt, qkv, batch, io, position_->cos_table(), position_->sin_table(), H_, KV_, hd_, scale_, window_);
        DeferredNorm started;
        o_.forward(rt, attn, nullptr, residual, FG_F32, true, emit_norm, &started);
        return started;
    }

private:
    int E_, H_, KV_, hd_, window_;
    float scale_;
    PositionEncoding *position_ = nullptr;
    std::unique_ptr<PositionEncoding> own_position_;
    Linear qkv_, q_only_, o_;
};

// ------------------------------------------------------------------------------------ SwiGLU
// down( silu(gate x) * (up x) ): gate and up in one fused pass (fastgguf.c:4870-4872), silu(z) = z / (1 + exp(-z))
// (:3118) times up (:4876), down projection added onto the layer's input (:4877-4880).
class SwiGLU : public FeedForward {
public:
    SwiGLU(const Json &p) : E_((int)param_int(p, "hidden_size", "swiglu")), F_((int)param_int(p, "d_ff", "swiglu")) {
        if (E_ <= 0 || F_ <= 0) fail(FG_E_CONFIG, "swiglu: sizes must be positive");
    }
    std::vector<TensorDecl> tensor_decls() const override {
        return {{"gate_proj.weight", {F_, E_}}, {"up_proj.weight", {F_, E_}}, {"down_proj.weight", {E_, F_}}};
    }
    bool supports_deferred_norm() const override { return true; }
    void load(const std::map<std::string, Weight> &tensors, Runtime &rt) override {
        const Weight &g = tensor_of(tensors, "gate_proj.weight"), &u = tensor_of(tensors, "up_proj.weight");
        int dt = g.t.dtype == u.t.dtype ? g.t.dtype : FG_F32;
        Weight both = concat_rows({g, u}, dt, rt.stream);
        if (dt == FG_BF16 && F_ % 64 == 0 && E_ % 8 == 0 && !rt.plain_kernels) {
            // gate, up and SiLU-mul in one tensor-core kernel: rows interleaved in blocks of 64
            std::vector<int64_t> rows;
            for (int64_t blk = 0; blk < F_ / 64; blk++) {
                for (int64_t i = 0; i < 64; i++) rows.push_back(blk * 64 + i);
                for (int64_t i = 0; i < 64; i++) rows.push_back(F_ + blk * 64 + i);
            }
            fused_ = Linear(gather_rows(both, rows, rt.stream));
        } else {
            gate_up_ = Linear(both);
        }
        down_ = Linear(tensor_of(tensors, "down_proj.weight"));
    }
    DeferredNorm forward(Runtime &rt, const Tensor &xn, const DeferredNorm *deferred, const Batch &, Tensor &residual,
                         Norm *emit_norm) override {
        Tensor t;
        bool done = fused_.defined() && fused_.forward_silu(rt, xn, deferred, &t);
        if (!done) {
            if (fused_.defined()) fail(FG_E_KERNEL, "the fused gate/up kernel refused a shape it was planned for");
            Tensor gu = gate_up_.forward(rt, xn, deferred, Tensor(), rt.dtype, false, nullptr, nullptr);
            t = rt.arena->matrix(gu.rows, F_, gu.dtype);
            if (gu.rows > 0) FG_LAUNCH("core", fg_silu_mul, gu.data, t.data, gu.dtype, (int)gu.rows, F_, rt.stream);
        }
        DeferredNorm started;
        down_.forward(rt, t, nullptr, residual, FG_F32, true, emit_norm, &started);
        return started;
    }

private:
    int E_, F_;
    Linear fused_, gate_up_, down_;
};

// ------------------------------------------------------------------------------------ pre-norm block
// x += mixer(norm1(x)); x += feed_forward(norm2(x)): the norm stands before attention (fastgguf.c:4686-4687) and
// before the feed-forward (:4865-4866); both residual sums add the projection onto the un-normalized input
// (:4862, :4880).  The residual stream x is float32 and is updated in place by the parts' output projections.
// In bfloat16 a norm may be STARTED by the contraction that writes the residual stream and FINISHED by the one
// that reads the normalised rows; parts that do not take part get plain normalised tensors.
class PreNormBlock : public Block {
public:
    DeferredNorm forward(Runtime &rt, Tensor &x, const Batch &batch, const LayerIO &io, const DeferredNorm &pending,
                         Norm *next_norm) override {
        bool bf16 = rt.dtype == FG_BF16;
        bool mixer_defers = bf16 && mixer->supports_deferred_norm(), ffn_defers = bf16 && feed_forward->supports_deferred_norm();
        DeferredNorm started;
        if (mixer_defers) {
            Norm *emit = (ffn_defers && feed_forward_norm->deferrable()) ? feed_forward_norm : nullptr;
            if (pending.defined()) started = mixer->forward(rt, Tensor(), &pending, batch, io, x, emit);
            else started = mixer->forward(rt, mixer_norm->forward(rt, x, nullptr, 0), nullptr, batch, io, x, emit);
        } else {
            mixer->forward(rt, mixer_norm->forward(rt, x, nullptr, 0), nullptr, batch, io, x, nullptr);
        }
        if (ffn_defers) {
            if (started.defined()) return feed_forward->forward(rt, Tensor(), &started, batch, x, next_norm);
            return feed_forward->forward(rt, feed_forward_norm->forward(rt, x, nullptr, 0), nullptr, batch, x, next_norm);
        }
        feed_forward->forward(rt, feed_forward_norm->forward(rt, x, nullptr, 0), nullptr, batch, x, nullptr);
        return DeferredNorm();
    }
};

// ------------------------------------------------------------------------------------ embedding and head
// read_embedding copies row `token` of token_embd into the residual stream, times embd_scale, which is 1 for
// Llama (fastgguf.c:4576-4581, :4652, :4219); the head is output.weight or, when that tensor is absent, the
// embedding table again (:4269-4270); logits are float (:4900).  Here tied-ness comes from the spec (both parts
// name the same checkpoint tensor), and a tied head shares the embedding's storage.
class TokenEmbedding : public Embedding {
public:
    TokenEmbedding(const Json &p)
        : V_(param_int(p, "vocab_size", "embedding")), E_(param_int(p, "hidden_size", "embedding")),
          scale_((float)param_float(p, "scale", 1.0, "embedding")) {
        if (V_ <= 0 || E_ <= 0) fail(FG_E_CONFIG, "embedding: sizes must be positive");
    }
    std::vector<TensorDecl> tensor_decls() const override { return {{"weight", {V_, E_}}}; }
    void load(const std::map<std::string, Weight> &tensors, Runtime &) override { w_ = tensor_of(tensors, "weight"); }
    DeferredNorm forward(Runtime &rt, const Batch &batch, Tensor &x, Norm *emit_norm) override {
        DeferredNorm started;
        int M = batch.n_rows;
        if (M == 0) return started;
        if (emit_norm && emit_norm->deferrable() && emit_norm->size() == E_ && rt.dtype == FG_BF16 && scale_ == 1.0f) {
            Tensor xw = rt.arena->matrix(M, E_, FG_BF16);
            float *ss = (float *)rt.arena->alloc((size_t)M * sizeof(float));
            FG_LAUNCH("core", fg_embed_gather_norm, w_.t.data, w_.t.dtype, batch.tokens, x.ptr<float>(), emit_norm->weight(), xw.data,
                      ss, M, (int)E_, rt.stream);
            started.xw = xw; started.ss = ss; started.tiles = 1; started.size = (int)E_; started.eps = emit_norm->eps();
            started.x = x; started.weight = emit_norm->weight();
            return started;
        }
        FG_LAUNCH("core", fg_embed_gather, w_.t.data, w_.t.dtype, batch.tokens, x.ptr<float>(), M, (int)E_, rt.stream);
        if (scale_ != 1.0f) dev_scale_f32(x.ptr<float>(), (int64_t)M * E_, scale_, rt.stream);
        return started;
    }

private:
    int64_t V_, E_;
    float scale_;
    Weight w_;
};

class LMHead : public Head {
public:
    LMHead(const Json &p) : V_(param_int(p, "vocab_size", "lm_head")), E_(param_int(p, "hidden_size", "lm_head")) {
        if (V_ <= 0 || E_ <= 0) fail(FG_E_CONFIG, "lm_head: sizes must be positive");
    }
    std::vector<TensorDecl> tensor_decls() const override { return {{"weight", {V_, E_}}}; }
    void load(const std::map<std::string, Weight> &tensors, Runtime &) override { linear_ = Linear(tensor_of(tensors, "weight")); }
    bool supports_deferred_norm() const override { return true; }
    Tensor forward(Runtime &rt, const Tensor &xn, const DeferredNorm *deferred) override {
        return linear_.forward(rt, xn, deferred, Tensor(), FG_F32, false, nullptr, nullptr);
    }

private:
    int64_t V_, E_;
    Linear linear_;
};

// ------------------------------------------------------------------------------------ parts from outside
static void *arena_alloc_cb(void *ctx, size_t bytes) {
    try {
        return ((Arena *)ctx)->alloc(bytes);
    } catch (...) {
        return nullptr;
    }
}

struct ExternalCore {
    fg_part_vtable vt;
    std::string kind;
    int role;
    void *self = nullptr;
    ExternalCore(const fg_part_vtable &v, std::string k, int r, const Json &params, int dtype) : vt(v), kind(std::move(k)), role(r) {
        if (!vt.create) fail(FG_E_CONFIG, "part '" + kind + "' has no create function");
        char err[512] = {0};
        self = vt.create(params.dump().c_str(), dtype, vt.user, err, sizeof err);
        if (!self) fail(FG_E_CONFIG, std::string(role_name(role)) + " '" + kind + "': " + (err[0] ? err : "refused its parameters"));
    }
    ~ExternalCore() {
        if (self && vt.destroy) vt.destroy(self);
    }
    std::vector<TensorDecl> decls() const {
        std::vector<TensorDecl> out;
        int n = vt.n_tensors ? vt.n_tensors(self) : 0;
        for (int i = 0; i < n; i++) {
            fg_tensor_decl d = {};
            if (!vt.tensor_decl || vt.tensor_decl(self, i, &d) != 0) fail(FG_E_CONFIG, "part '" + kind + "' could not describe its tensors");
            TensorDecl t;
            d.name[sizeof d.name - 1] = 0;
            t.name = d.name;
            for (int k = 0; k < d.ndim && k < 4; k++) t.shape.push_back(d.shape[k]);
            t.is_int = d.is_int != 0;
            t.init = d.init;
            t.std = d.std;
            out.push_back(t);
        }
        return out;
    }
    void load(const std::map<std::string, Weight> &tensors) {
        auto ds = decls();
        for (size_t i = 0; i < ds.size(); i++) {
            const Weight &w = tensor_of(tensors, ds[i].name.c_str());
            held.push_back(w);                                  // the part may keep the pointer
            fg_dev_tensor v = w.t.view();
            v.ndim = (int)ds[i].shape.size();
            for (size_t k = 0; k < ds[i].shape.size(); k++) v.shape[k] = ds[i].shape[k];
            if (vt.load && vt.load(self, (int)i, &v) != 0) fail(FG_E_WEIGHTS, "part '" + kind + "' refused tensor '" + ds[i].name + "'");
        }
    }
    void call(fg_part_call &c, Runtime &rt) {
        c.role = role;
        c.alloc = arena_alloc_cb;
        c.alloc_ctx = rt.arena;
        c.stream = rt.stream;
        if (!vt.forward) fail(FG_E_CONFIG, "part '" + kind + "' has no forward function");
        count_launch();
        int code = vt.forward(self, &c);
        if (code != 0) fail(code > 0 && code <= FG_E_INTERNAL ? code : FG_E_KERNEL, format("%s '%s' failed with status %d", role_name(role), kind.c_str(), code));
    }
    std::vector<Weight> held;
};

class ExternalNorm : public Norm {
public:
    ExternalNorm(const fg_part_vtable &v, const std::string &k, const Json &p, int dtype) : core(v, k, FG_ROLE_NORM, p, dtype) {}
    std::vector<TensorDecl> tensor_decls() const override { return core.decls(); }
    void load(const std::map<std::string, Weight> &t, Runtime &) override { core.load(t); }
    Tensor forward(Runtime &rt, const Tensor &x, const int *rows, int n_rows) override {
        int R = rows ? n_rows : (int)x.rows;
        Tensor out = rt.arena->matrix(R, x.cols, rt.dtype);
        fg_part_call c = {};
        c.x = x.view(); c.out = out.view(); c.rows = rows; c.n_rows = R;
        core.call(c, rt);
        return out;
    }
    ExternalCore core;
};

class ExternalPosition : public PositionEncoding {
public:
    ExternalPosition(const fg_part_vtable &v, const std::string &k, const Json &p, int dtype) : core(v, k, FG_ROLE_POSITION, p, dtype) {
        hd_ = (int)param_int(p, "head_dim", k.c_str());
        if (hd_ <= 0 || hd_ % 2) fail(FG_E_CONFIG, "position '" + k + "': head_dim must be even and positive");
        if (!core.vt.position_tables) fail(FG_E_CONFIG, "position '" + k + "' has no position_tables function");
        std::vector<float> c(hd_ / 2), s(hd_ / 2);
        tables(1, c, s);                                        // the permutation is known at build time
    }
    void tables(int max_positions, std::vector<float> &c, std::vector<float> &s) {
        int half = hd_ / 2;
        c.assign((size_t)max_positions * half, 1.f);
        s.assign((size_t)max_positions * half, 0.f);
        std::vector<int> perm((size_t)hd_);
        for (int i = 0; i < hd_; i++) perm[(size_t)i] = i;
        if (core.vt.position_tables(core.self, max_positions, hd_, c.data(), s.data(), perm.data()) != 0)
            fail(FG_E_CONFIG, "position '" + core.kind + "' could not build its tables");
        std::vector<char> seen((size_t)hd_, 0);
        bool identity = true;
        for (int i = 0; i < hd_; i++) {
            int p = perm[(size_t)i];
            if (p < 0 || p >= hd_ || seen[(size_t)p]) fail(FG_E_CONFIG, "position '" + core.kind + "': its row permutation is no permutation");
            seen[(size_t)p] = 1;
            identity = identity && p == i;
        }
        perm_ = identity ? std::vector<int>() : perm;
    }
    void prepare(Runtime &rt, int max_positions) override {
        if (cos_.buffer && max_positions_ >= max_positions) return;
        std::vector<float> c, s;
        tables(max_positions, c, s);
        cos_ = make_weight(max_positions, hd_ / 2, FG_F32, "position tables");
        sin_ = make_weight(max_positions, hd_ / 2, FG_F32, "position tables");
        FG_CUDA(cudaMemcpyAsync(cos_.t.data, c.data(), c.size() * 4, cudaMemcpyHostToDevice, rt.stream));
        FG_CUDA(cudaMemcpyAsync(sin_.t.data, s.data(), s.size() * 4, cudaMemcpyHostToDevice, rt.stream));
        FG_CUDA(cudaStreamSynchronize(rt.stream));
        max_positions_ = max_positions;
    }
    const float *cos_table() const override { return cos_.t.ptr<float>(); }
    const float *sin_table() const override { return sin_.t.ptr<float>(); }
    int head_dim() const override { return hd_; }
    const std::vector<int> &permutation() const override { return perm_; }
    ExternalCore core;

private:
    int hd_ = 0, max_positions_ = 0;
    std::vector<int> perm_;
    Weight cos_, sin_;
};

class ExternalMixer : public Mixer {
public:
    ExternalMixer(const fg_part_vtable &v, const std::string &k, const Json &p, int dtype) : core(v, k, FG_ROLE_MIXER, p, dtype) {}
    std::vector<TensorDecl> tensor_decls() const override { return core.decls(); }
    void load(const std::map<std::string, Weight> &t, Runtime &) override { core.load(t); }
    bool cache_request(CacheRequest *out) const override {
        if (!core.vt.cache_request) return false;
        int kv = 0, hd = 0, w = 0;
        if (!core.vt.cache_request(core.self, &kv, &hd, &w)) return false;
        out->n_kv_heads = kv; out->head_dim = hd; out->window = w;
        return true;
    }
    int64_t state_bytes() const override { return core.vt.state_bytes ? core.vt.state_bytes(core.self) : 0; }
    DeferredNorm forward(Runtime &rt, const Tensor &xn, const DeferredNorm *, const Batch &batch, const LayerIO &io, Tensor &residual,
                         Norm *) override {
        fg_batch_view bv = batch.view(rt.stream);
        fg_layer_io iv = io.view();
        fg_part_call c = {};
        c.batch = &bv; c.io = &iv; c.xn = xn.view(); c.residual = residual.view();
        core.call(c, rt);
        return DeferredNorm();
    }
    ExternalCore core;
};

class ExternalFeedForward : public FeedForward {
public:
    ExternalFeedForward(const fg_part_vtable &v, const std::string &k, const Json &p, int dtype) : core(v, k, FG_ROLE_FEED_FORWARD, p, dtype) {}
    std::vector<TensorDecl> tensor_decls() const override { return core.decls(); }
    void load(const std::map<std::string, Weight> &t, Runtime &) override { core.load(t); }
    DeferredNorm forward(Runtime &rt, const Tensor &xn, const DeferredNorm *, const Batch &batch, Tensor &residual, Norm *) override {
        fg_batch_view bv = batch.view(rt.stream);
        fg_part_call c = {};
        c.batch = &bv; c.xn = xn.view(); c.residual = residual.view();
        core.call(c, rt);
        return DeferredNorm();
    }
    ExternalCore core;
};

class ExternalEmbedding : public Embedding {
public:
    ExternalEmbedding(const fg_part_vtable &v, const std::string &k, const Json &p, int dtype) : core(v, k, FG_ROLE_EMBEDDING, p, dtype) {}
    std::vector<TensorDecl> tensor_decls() const override { return core.decls(); }
    void load(const std::map<std::string, Weight> &t, Runtime &) override { core.load(t); }
    DeferredNorm forward(Runtime &rt, const Batch &batch, Tensor &x, Norm *) override {
        fg_batch_view bv = batch.view(rt.stream);
        fg_part_call c = {};
        c.batch = &bv; c.x = x.view();
        core.call(c, rt);
        return DeferredNorm();
    }
    ExternalCore core;
};

class ExternalHead : public Head {
public:
    ExternalHead(const fg_part_vtable &v, const std::string &k, const Json &p, int dtype) : core(v, k, FG_ROLE_HEAD, p, dtype) {
        V_ = param_int(p, "vocab_size", k.c_str());
    }
    std::vector<TensorDecl> tensor_decls() const override { return core.decls(); }
    void load(const std::map<std::string, Weight> &t, Runtime &) override { core.load(t); }
    Tensor forward(Runtime &rt, const Tensor &xn, const DeferredNorm *) override {
        Tensor out = rt.arena->matrix(xn.rows, V_, FG_F32);
        fg_part_call c = {};
        c.xn = xn.view(); c.out = out.view();
        core.call(c, rt);
        return out;
    }
    ExternalCore core;

private:
    int64_t V_;
};

// A block arrangement from outside runs the engine's parts through fg_block_ops.
struct BlockCallContext {
    Runtime *rt;
    Block *block;
    const Batch *batch;
    const LayerIO *io;
    Tensor *x;
    std::string error;
};

static int block_op_guard(const fg_part_call *call, const std::function<void(BlockCallContext &)> &f) {
    BlockCallContext *ctx = (BlockCallContext *)call->engine_ctx;
    try {
        f(*ctx);
        return 0;
    } catch (const Error &e) {
        ctx->error = e.what();
        return e.code;
    } catch (const std::exception &e) {
        ctx->error = e.what();
        return FG_E_INTERNAL;
    }
}
static Tensor tensor_from_view(const fg_dev_tensor &v) {
    Tensor t;
    t.data = v.data; t.dtype = v.dtype; t.rows = v.shape[0]; t.cols = v.shape[1]; t.ld = v.ld;
    return t;
}
static int block_op_norm(const fg_part_call *call, int which, fg_dev_tensor *xn_out) {
    return block_op_guard(call, [&](BlockCallContext &c) {
        Norm *n = which == 0 ? c.block->mixer_norm : c.block->feed_forward_norm;
        *xn_out = n->forward(*c.rt, *c.x, nullptr, 0).view();
    });
}
static int block_op_mixer(const fg_part_call *call, const fg_dev_tensor *xn) {
    return block_op_guard(call, [&](BlockCallContext &c) {
        c.block->mixer->forward(*c.rt, tensor_from_view(*xn), nullptr, *c.batch, *c.io, *c.x, nullptr);
    });
}
static int block_op_ffn(const fg_part_call *call, const fg_dev_tensor *xn) {
    return block_op_guard(call, [&](BlockCallContext &c) {
        c.block->feed_forward->forward(*c.rt, tensor_from_view(*xn), nullptr, *c.batch, *c.x, nullptr);
    });
}
static const fg_block_ops kBlockOps = {block_op_norm, block_op_mixer, block_op_ffn};

class ExternalBlock : public Block {
public:
    ExternalBlock(const fg_part_vtable &v, const std::string &k, int dtype) : core(v, k, FG_ROLE_BLOCK, Json::object(), dtype) {}
    DeferredNorm forward(Runtime &rt, Tensor &x, const Batch &batch, const LayerIO &io, const DeferredNorm &, Norm *) override {
        BlockCallContext ctx{&rt, this, &batch, &io, &x, ""};
        fg_batch_view bv = batch.view(rt.stream);
        fg_layer_io iv = io.view();
        fg_part_call c = {};
        c.batch = &bv; c.io = &iv; c.residual = x.view(); c.x = x.view();
        c.block_ops = &kBlockOps; c.engine_ctx = &ctx;
        try {
            core.call(c, rt);
        } catch (const Error &e) {
            if (!ctx.error.empty()) fail(e.code, ctx.error);
            throw;
        }
        return DeferredNorm();
    }
    ExternalCore core;
};

// ------------------------------------------------------------------------------------ registries
static std::mutex g_parts_mutex;
static std::map<std::string, PartFactory> &factories(int role) {
    static std::map<std::string, PartFactory> r[7];
    static bool init = false;
    if (!init) {
        init = true;
        r[FG_ROLE_NORM]["rmsnorm"] = [](Runtime &, const Json &p, BuildContext &) { return std::make_unique<RMSNorm>(p); };
        r[FG_ROLE_POSITION]["rope"] = [](Runtime &, const Json &p, BuildContext &) { return std::make_unique<RotaryEncoding>(p); };
        r[FG_ROLE_MIXER]["gqa_attention"] = [](Runtime &, const Json &p, BuildContext &c) { return std::make_unique<GQAAttention>(p, c); };
        r[FG_ROLE_FEED_FORWARD]["swiglu"] = [](Runtime &, const Json &p, BuildContext &) { return std::make_unique<SwiGLU>(p); };
        r[FG_ROLE_EMBEDDING]["embedding"] = [](Runtime &, const Json &p, BuildContext &) { return std::make_unique<TokenEmbedding>(p); };
        r[FG_ROLE_HEAD]["lm_head"] = [](Runtime &, const Json &p, BuildContext &) { return std::make_unique<LMHead>(p); };
    }
    if (role < 0 || role > 6) fail(FG_E_USAGE, format("role %d does not exist", role));
    return r[role];
}
static std::map<std::string, BlockFactory> &block_factories() {
    static std::map<std::string, BlockFactory> r = {{"prenorm", [](Runtime &) { return std::make_unique<PreNormBlock>(); }}};
    return r;
}

void register_part_factory(int role, const std::string &kind, PartFactory f) {
    std::lock_guard<std::mutex> lock(g_parts_mutex);
    factories(role)[kind] = std::move(f);
}
void register_block_factory(const std::string &kind, BlockFactory f) {
    std::lock_guard<std::mutex> lock(g_parts_mutex);
    block_factories()[kind] = std::move(f);
}

template <typename M>
static std::string known_kinds(const M &m) {
    std::string s;
    for (auto &kv : m) s += (s.empty() ? "" : ", ") + kv.first;
    return s.empty() ? "none" : s;
}

std::unique_ptr<Part> build_part(int role, const std::string &kind, Runtime &rt, const Json &params, BuildContext &ctx) {
    PartFactory f;
    {
        std::lock_guard<std::mutex> lock(g_parts_mutex);
        auto &m = factories(role);
        auto it = m.find(kind);
        if (it == m.end())
            fail(FG_E_CONFIG, format("no %s of kind '%s' is registered (registered: %s)", role_name(role), kind.c_str(), known_kinds(m).c_str()));
        f = it->second;
    }
    return f(rt, params.is_object() ? params : Json::object(), ctx);
}

std::unique_ptr<Block> build_block(const std::string &kind, Runtime &rt) {
    BlockFactory f;
    {
        std::lock_guard<std::mutex> lock(g_parts_mutex);
        auto &m = block_factories();
        auto it = m.find(kind);
        if (it == m.end())
            fail(FG_E_CONFIG, format("no block of kind '%s' is registered (registered: %s)", kind.c_str(), known_kinds(m).c_str()));
        f = it->second;
    }
    return f(rt);
}

void register_external_part(int role, const std::string &kind, const fg_part_vtable &vt) {
    static const char *builtin[] = {"rmsnorm", "rope", "gqa_attention", "swiglu", "prenorm", "embedding", "lm_head"};
    for (auto b : builtin)
        if (kind == b) fail(FG_E_USAGE, "kind '" + kind + "' is built in and cannot be replaced");
    if (kind.empty()) fail(FG_E_USAGE, "a part kind needs a name");
    fg_part_vtable v = vt;
    switch (role) {
    case FG_ROLE_NORM:
        register_part_factory(role, kind, [v, kind](Runtime &rt, const Json &p, BuildContext &) { return std::make_unique<ExternalNorm>(v, kind, p, rt.dtype); });
        break;
    case FG_ROLE_POSITION:
        register_part_factory(role, kind, [v, kind](Runtime &rt, const Json &p, BuildContext &) { return std::make_unique<ExternalPosition>(v, kind, p, rt.dtype); });
        break;
    case FG_ROLE_MIXER:
        register_part_factory(role, kind, [v, kind](Runtime &rt, const Json &p, BuildContext &) { return std::make_unique<ExternalMixer>(v, kind, p, rt.dtype); });
        break;
    case FG_ROLE_FEED_FORWARD:
        register_part_factory(role, kind, [v, kind](Runtime &rt, const Json &p, BuildContext &) { return std::make_unique<ExternalFeedForward>(v, kind, p, rt.dtype); });
        break;
    case FG_ROLE_EMBEDDING:
        register_part_factory(role, kind, [v, kind](Runtime &rt, const Json &p, BuildContext &) { return std::make_unique<ExternalEmbedding>(v, kind, p, rt.dtype); });
        break;
    case FG_ROLE_HEAD:
        register_part_factory(role, kind, [v, kind](Runtime &rt, const Json &p, BuildContext &) { return std::make_unique<ExternalHead>(v, kind, p, rt.dtype); });
        break;
    case FG_ROLE_BLOCK:
        register_block_factory(kind, [v, kind](Runtime &rt) { return std::make_unique<ExternalBlock>(v, kind, rt.dtype); });
        break;
    default:
        fail(FG_E_USAGE, format("role %d does not exist", role));
    }
}

}  // namespace fg
