// See config.hpp.  LlamaConfig reads the keys of a Llama model folder's config.json; the registry maps
// "architectures"[0] to the reader of its typed configuration.
#include "config.hpp"

#include <sys/stat.h>

#include <algorithm>
#include <cmath>
#include <fstream>
#include <mutex>
#include <sstream>

namespace fg {

std::string read_text_file(const std::string &path, bool *exists) {
    std::ifstream f(path, std::ios::binary);
    if (exists) *exists = (bool)f;
    if (!f) return std::string();
    std::stringstream ss;
    ss << f.rdbuf();
    return ss.str();
}

std::string json_repr(const Json &v) {
    if (v.is_string()) return "'" + v.as_string() + "'";
    if (v.is_bool()) return v.as_bool() ? "True" : "False";
    return v.dump();
}

// ------------------------------------------------------------------------------------ typed access
static const Json *present(const Json &d, const std::string &key) {
    const Json *v = d.find(key);
    return (v && !v->is_null()) ? v : nullptr;
}

[[noreturn]] static void missing(const std::string &key, const char *where) {
    fail(FG_E_CONFIG, format("%s: required key '%s' is missing", where, key.c_str()));
}

static long long int_of(const Json &v, const std::string &key, const char *where) {
    if (v.is_bool()) fail(FG_E_CONFIG, format("%s: key '%s' must be an integer, got %s", where, key.c_str(), json_repr(v).c_str()));
    if (v.is_int()) return v.as_int();
    if (v.is_number() && v.as_double() == std::floor(v.as_double()) && std::fabs(v.as_double()) < 9e15)
        return (long long)v.as_double();
    fail(FG_E_CONFIG, format("%s: key '%s' must be int, got %s (%s)", where, key.c_str(), v.type_name(), json_repr(v).c_str()));
}

static double float_of(const Json &v, const std::string &key, const char *where) {
    if (v.is_number() && !v.is_bool()) return v.as_double();
    fail(FG_E_CONFIG, format("%s: key '%s' must be float, got %s (%s)", where, key.c_str(), v.type_name(), json_repr(v).c_str()));
}

long long take_int(const Json &d, const std::string &key, const char *where) {
    const Json *v = present(d, key);
    if (!v) missing(key, where);
    return int_of(*v, key, where);
}
long long take_int(const Json &d, const std::string &key, long long dflt, const char *where) {
    const Json *v = present(d, key);
    return v ? int_of(*v, key, where) : dflt;
}
double take_float(const Json &d, const std::string &key, const char *where) {
    const Json *v = present(d, key);
    if (!v) missing(key, where);
    return float_of(*v, key, where);
}
double take_float(const Json &d, const std::string &key, double dflt, const char *where) {
    const Json *v = present(d, key);
    return v ? float_of(*v, key, where) : dflt;
}
bool take_bool(const Json &d, const std::string &key, bool dflt, const char *where) {
    const Json *v = present(d, key);
    if (!v) return dflt;
    if (!v->is_bool())
        fail(FG_E_CONFIG, format("%s: key '%s' must be bool, got %s (%s)", where, key.c_str(), v->type_name(), json_repr(*v).c_str()));
    return v->as_bool();
}
std::string take_string(const Json &d, const std::string &key, const std::string &dflt, const char *where) {
    const Json *v = present(d, key);
    if (!v) return dflt;
    if (!v->is_string())
        fail(FG_E_CONFIG, format("%s: key '%s' must be str, got %s (%s)", where, key.c_str(), v->type_name(), json_repr(*v).c_str()));
    return v->as_string();
}

// ------------------------------------------------------------------------------------ files
Json read_config_json(const std::string &model_dir) {
    std::string path = model_dir + "/config.json";
    bool exists = false;
    std::string text = read_text_file(path, &exists);
    if (!exists) fail(FG_E_CONFIG, path + ": no such file");
    Json d;
    try {
        d = Json::parse(text);
    } catch (const JsonError &e) {
        fail(FG_E_CONFIG, path + ": not valid JSON (" + e.what() + ")");
    }
    if (!d.is_object()) fail(FG_E_CONFIG, path + ": top level must be an object");
    return d;
}

static bool plain_int(const Json &v) { return v.is_int() && !v.is_bool(); }

// Stop tokens a model folder names beside config.json: generation_config.json may list further
// eos_token_id values (instruction-tuned checkpoints end a turn with tokens config.json does not name).
// The union, config.json's first, replaces d["eos_token_id"].  (The reference takes its stop set from
// the model file's metadata plus named control tokens, fastgguf.c:3644-3652.)
Json merge_generation_config(const std::string &model_dir, const Json &d) {
    std::string path = model_dir + "/generation_config.json";
    bool exists = false;
    std::string text = read_text_file(path, &exists);
    if (!exists) return d;
    Json g;
    try {
        g = Json::parse(text);
    } catch (const JsonError &e) {
        fail(FG_E_CONFIG, path + ": not valid JSON (" + e.what() + ")");
    }
    const Json *more = g.is_object() ? present(g, "eos_token_id") : nullptr;
    if (!more) return d;
    std::vector<long long> extra;
    bool ok = true;
    if (plain_int(*more)) extra.push_back(more->as_int());
    else if (more->is_array()) {
        for (auto &t : more->items()) {
            if (!plain_int(t)) { ok = false; break; }
            extra.push_back(t.as_int());
        }
    } else ok = false;
    if (!ok)
        fail(FG_E_CONFIG, path + ": 'eos_token_id' must be an integer or a list of integers, got " + json_repr(*more));
    std::vector<long long> have;
    const Json *own = present(d, "eos_token_id");
    if (own) {
        if (plain_int(*own)) have.push_back(own->as_int());
        else if (own->is_array()) {
            for (auto &t : own->items()) {
                if (!plain_int(t)) return d;        // config.json's own value is wrong: its reader says so
                have.push_back(t.as_int());
            }
        } else return d;
    }
    for (long long t : extra)
        if (std::find(have.begin(), have.end(), t) == have.end()) have.push_back(t);
    Json out = d;
    if (have.size() == 1) out.set("eos_token_id", Json(have[0]));
    else {
        Json a = Json::array();
        for (long long t : have) a.push(Json(t));
        out.set("eos_token_id", a);
    }
    return out;
}

// ------------------------------------------------------------------------------------ registry
static std::mutex g_registry_mutex;
static std::map<std::string, ConfigReader> &registry() {
    static std::map<std::string, ConfigReader> r = {{"LlamaForCausalLM", &LlamaConfig::from_json}};
    return r;
}

void register_architecture(const std::string &name, ConfigReader reader) {
    std::lock_guard<std::mutex> lock(g_registry_mutex);
    registry()[name] = std::move(reader);
}

std::vector<std::string> registered_architectures() {
    std::lock_guard<std::mutex> lock(g_registry_mutex);
    std::vector<std::string> names;
    for (auto &kv : registry()) names.push_back(kv.first);
    return names;
}

std::unique_ptr<ModelConfig> config_from_json(const Json &d) {
    const Json &archs = d.get("architectures");
    if (!d.is_object() || !archs.is_array() || archs.size() == 0 || !archs[0].is_string())
        fail(FG_E_CONFIG, "config.json: 'architectures' must be a non-empty list of names");
    ConfigReader reader;
    {
        std::lock_guard<std::mutex> lock(g_registry_mutex);
        auto it = registry().find(archs[0].as_string());
        if (it != registry().end()) reader = it->second;
    }
    if (!reader) {
        std::string known;
        for (auto &n : registered_architectures()) known += (known.empty() ? "" : ", ") + n;
        fail(FG_E_CONFIG, "architecture '" + archs[0].as_string() + "' is not registered (registered: " +
                              (known.empty() ? "none" : known) + ")");
    }
    return reader(d);
}

std::unique_ptr<ModelConfig> config_from_dir(const std::string &model_dir) {
    return config_from_json(merge_generation_config(model_dir, read_config_json(model_dir)));
}

// ------------------------------------------------------------------------------------ Llama
Json RopeScaling::to_json() const {
    if (rope_type == "default") return Json();
    Json j = Json::object();
    j.set("rope_type", rope_type);
    j.set("factor", factor);
    j.set("low_freq_factor", low_freq_factor);
    j.set("high_freq_factor", high_freq_factor);
    j.set("original_max_position_embeddings", original_max_position_embeddings);
    return j;
}

static RopeScaling read_rope_scaling(const Json *d) {
    RopeScaling rs;
    if (!d || d->is_null()) return rs;
    if (!d->is_object()) fail(FG_E_CONFIG, "config.json: 'rope_scaling' must be an object or null");
    const Json *kind = present(*d, "rope_type");
    if (!kind) kind = present(*d, "type");
    if (!kind || (kind->is_string() && kind->as_string() == "default")) return rs;
    if (!kind->is_string() || kind->as_string() != "llama3")
        fail(FG_E_CONFIG, "config.json: rope_scaling.rope_type " + json_repr(*kind) + " is not supported (known: default, llama3)");
    const char *w = "config.json rope_scaling";
    rs.rope_type = "llama3";
    rs.factor = take_float(*d, "factor", w);
    rs.low_freq_factor = take_float(*d, "low_freq_factor", w);
    rs.high_freq_factor = take_float(*d, "high_freq_factor", w);
    rs.original_max_position_embeddings = take_int(*d, "original_max_position_embeddings", w);
    return rs;
}

static const std::string kLlamaName = "LlamaForCausalLM";
const std::string &LlamaConfig::architecture() const { return kLlamaName; }

std::unique_ptr<ModelConfig> LlamaConfig::from_json(const Json &d) {
    auto cfg = std::make_unique<LlamaConfig>();
    LlamaConfig &c = *cfg;
    auto note_default = [&](const char *key) {
        if (!present(d, key)) c.defaulted.push_back(key);
    };
    long long H = take_int(d, "num_attention_heads");
    long long E = take_int(d, "hidden_size");
    // newer config files nest the rotary parameters under "rope_parameters"
    const Json *rp = present(d, "rope_parameters");
    if (rp && !rp->is_object()) rp = nullptr;
    const Json &theta_src = (rp && rp->has("rope_theta")) ? *rp : d;
    const Json *scaling_src = present(d, "rope_scaling");
    if (!scaling_src && rp) {
        const Json *t = present(*rp, "rope_type");
        if (t && !(t->is_string() && t->as_string() == "default")) scaling_src = rp;
    }
    if (const Json *eos = present(d, "eos_token_id")) {
        bool ok = true;
        if (plain_int(*eos)) c.eos_token_ids.push_back(eos->as_int());
        else if (eos->is_array()) {
            for (auto &t : eos->items()) {
                if (!plain_int(t)) { ok = false; break; }
                c.eos_token_ids.push_back(t.as_int());
            }
        } else ok = false;
        if (!ok)
            fail(FG_E_CONFIG, "config.json: 'eos_token_id' must be an integer or a list of integers, got " + json_repr(*eos));
    }
    if (take_bool(d, "attention_bias", false))
        fail(FG_E_CONFIG, "config.json: attention_bias=true is not supported (the Llama path has no biases)");
    if (take_bool(d, "mlp_bias", false))
        fail(FG_E_CONFIG, "config.json: mlp_bias=true is not supported (the Llama path has no biases)");
    if (H <= 0) fail(FG_E_CONFIG, format("config.json: num_attention_heads must be positive, got %lld", H));
    c.hidden_size = E;
    c.num_hidden_layers = take_int(d, "num_hidden_layers");
    c.num_attention_heads = H;
    // absent: as many KV heads as heads (plain multi-head attention)
    note_default("num_key_value_heads");
    c.num_key_value_heads = take_int(d, "num_key_value_heads", H);
    // absent: hidden_size / heads, the reference's fallback (fastgguf.c:4283)
    note_default("head_dim");
    c.head_dim = take_int(d, "head_dim", E / H);
    c.intermediate_size = take_int(d, "intermediate_size");
    c.vocab_size = take_int(d, "vocab_size");
    // the reference's defaults for absent keys (fastgguf.c:4228, 4224)
    note_default("rms_norm_eps");
    c.rms_norm_eps = take_float(d, "rms_norm_eps", 1e-6);
    if (!present(theta_src, "rope_theta")) c.defaulted.push_back("rope_theta");
    c.rope_theta = take_float(theta_src, "rope_theta", 10000.0);
    c.rope_scaling = read_rope_scaling(scaling_src);
    c.max_position_embeddings = take_int(d, "max_position_embeddings");
    note_default("tie_word_embeddings");
    c.tie_word_embeddings = take_bool(d, "tie_word_embeddings", false);
    if (!present(d, "torch_dtype") && !present(d, "dtype")) c.defaulted.push_back("torch_dtype");
    c.torch_dtype = take_string(d, "torch_dtype", take_string(d, "dtype", "bfloat16"));
    if (const Json *bos = present(d, "bos_token_id")) {
        c.has_bos = true;
        c.bos_token_id = int_of(*bos, "bos_token_id", "config.json");
    }
    note_default("hidden_act");
    c.hidden_act = take_string(d, "hidden_act", "silu");
    c.validate();
    return cfg;
}

void LlamaConfig::validate() const {
    struct { const char *name; long long v; } sizes[] = {
        {"hidden_size", hidden_size}, {"num_hidden_layers", num_hidden_layers},
        {"num_attention_heads", num_attention_heads}, {"num_key_value_heads", num_key_value_heads},
        {"head_dim", head_dim}, {"intermediate_size", intermediate_size}, {"vocab_size", vocab_size},
        {"max_position_embeddings", max_position_embeddings}};
    for (auto &s : sizes)
        if (s.v <= 0) fail(FG_E_CONFIG, format("config.json: %s must be positive, got %lld", s.name, s.v));
    if (num_attention_heads % num_key_value_heads != 0)
        fail(FG_E_CONFIG, format("config.json: num_attention_heads (%lld) must be a multiple of num_key_value_heads (%lld)",
                                 num_attention_heads, num_key_value_heads));
    if (head_dim % 2 != 0) fail(FG_E_CONFIG, format("config.json: head_dim must be even for rotary pairs, got %lld", head_dim));
    if (!(rms_norm_eps > 0.0)) fail(FG_E_CONFIG, format("config.json: rms_norm_eps must be positive, got %g", rms_norm_eps));
    if (!(rope_theta > 0.0)) fail(FG_E_CONFIG, format("config.json: rope_theta must be positive, got %g", rope_theta));
    if (hidden_act != "silu")
        fail(FG_E_CONFIG, "config.json: hidden_act '" + hidden_act + "' is not supported (known: silu)");
    if (rope_scaling.rope_type == "llama3") {
        if (rope_scaling.factor <= 0 || rope_scaling.original_max_position_embeddings <= 0)
            fail(FG_E_CONFIG, "config.json: rope_scaling needs positive factor and original_max_position_embeddings");
        if (rope_scaling.high_freq_factor <= rope_scaling.low_freq_factor)
            fail(FG_E_CONFIG, "config.json: rope_scaling.high_freq_factor must exceed low_freq_factor");
    }
    for (long long t : eos_token_ids)
        if (t < 0 || t >= vocab_size)
            fail(FG_E_CONFIG, format("config.json: eos_token_id %lld lies outside the vocabulary [0, %lld)", t, vocab_size));
}

long long LlamaConfig::parameter_count() const {
    long long E = hidden_size, F = intermediate_size, V = vocab_size;
    long long per_layer = E * (q_dim() + 2 * kv_dim()) + q_dim() * E + 3 * E * F + 2 * E;
    long long head = tie_word_embeddings ? 0 : V * E;
    return num_hidden_layers * per_layer + V * E + E + head;
}

Json LlamaConfig::to_json() const {
    Json d = Json::object();
    Json archs = Json::array();
    archs.push(kLlamaName);
    d.set("architectures", archs);
    d.set("model_type", "llama");
    d.set("hidden_size", hidden_size);
    d.set("num_hidden_layers", num_hidden_layers);
    d.set("num_attention_heads", num_attention_heads);
    d.set("num_key_value_heads", num_key_value_heads);
    d.set("head_dim", head_dim);
    d.set("intermediate_size", intermediate_size);
    d.set("vocab_size", vocab_size);
    d.set("rms_norm_eps", rms_norm_eps);
    d.set("rope_theta", rope_theta);
    d.set("rope_scaling", rope_scaling.to_json());
    d.set("max_position_embeddings", max_position_embeddings);
    d.set("tie_word_embeddings", tie_word_embeddings);
    d.set("torch_dtype", torch_dtype);
    d.set("hidden_act", hidden_act);
    d.set("attention_bias", false);
    d.set("mlp_bias", false);
    if (has_bos) d.set("bos_token_id", bos_token_id);
    if (eos_token_ids.size() == 1) d.set("eos_token_id", eos_token_ids[0]);
    else if (!eos_token_ids.empty()) {
        Json a = Json::array();
        for (long long t : eos_token_ids) a.push(Json(t));
        d.set("eos_token_id", a);
    }
    return d;
}

Json LlamaConfig::describe() const {
    Json d = Json::object();
    d.set("hidden_size", hidden_size);
    d.set("num_hidden_layers", num_hidden_layers);
    d.set("num_attention_heads", num_attention_heads);
    d.set("num_key_value_heads", num_key_value_heads);
    d.set("head_dim", head_dim);
    d.set("intermediate_size", intermediate_size);
    d.set("vocab_size", vocab_size);
    d.set("rms_norm_eps", rms_norm_eps);
    d.set("rope_theta", rope_theta);
    Json rs = Json::object();
    rs.set("rope_type", rope_scaling.rope_type);
    rs.set("factor", rope_scaling.factor);
    rs.set("low_freq_factor", rope_scaling.low_freq_factor);
    rs.set("high_freq_factor", rope_scaling.high_freq_factor);
    rs.set("original_max_position_embeddings", rope_scaling.original_max_position_embeddings);
    d.set("rope_scaling", rs);
    d.set("max_position_embeddings", max_position_embeddings);
    d.set("tie_word_embeddings", tie_word_embeddings);
    d.set("torch_dtype", torch_dtype);
    d.set("bos_token_id", has_bos ? Json(bos_token_id) : Json());
    Json eos = Json::array();
    for (long long t : eos_token_ids) eos.push(Json(t));
    d.set("eos_token_ids", eos);
    d.set("hidden_act", hidden_act);
    // derived sizes
    d.set("q_dim", q_dim());
    d.set("kv_dim", kv_dim());
    d.set("group_size", num_attention_heads / num_key_value_heads);
    d.set("parameters", parameter_count());
    // memory: keys and values of one token over all layers, and the parameters, per engine dtype
    // (the reference prints kv_mem at load: fastgguf.c:4561-4565)
    Json kvb = Json::object(), pb = Json::object();
    kvb.set("bfloat16", 2 * num_hidden_layers * kv_dim() * 2);
    kvb.set("float32", 2 * num_hidden_layers * kv_dim() * 4);
    pb.set("bfloat16", parameter_count() * 2);
    pb.set("float32", parameter_count() * 4);
    d.set("kv_bytes_per_token", kvb);
    d.set("parameter_bytes", pb);
    Json df = Json::array();
    for (auto &k : defaulted) df.push(k);
    d.set("defaulted", df);
    return d;
}

// The dense Llama decoder as data: every layer is a pre-norm block of grouped-query attention with rotary
// encoding and a SwiGLU feed-forward; the schedule runs the layers once, in order, each with a cache of its
// own.  Tensor names are those of a model folder's safetensors; the reference's GGUF names for the same
// tensors are token_embd, output, output_norm, blk.N.attn_norm, blk.N.attn_{q,k,v,output}, blk.N.ffn_norm,
// blk.N.ffn_{gate,up,down} (fastgguf.c:4266-4278, :4292-4365).  The head is the embedding table again when
// tie_word_embeddings is set (the reference decides by the absence of output.weight, :4269-4270).
static Json part(const char *kind, Json params, Json tensors = Json::object()) {
    Json p = Json::object();
    p.set("kind", kind);
    p.set("params", std::move(params));
    p.set("tensors", std::move(tensors));
    return p;
}

Json LlamaConfig::spec() const {
    long long E = hidden_size;
    Json rope_params = Json::object();
    rope_params.set("head_dim", head_dim);
    rope_params.set("theta", rope_theta);
    rope_params.set("scaling", rope_scaling.to_json());
    Json rope = part("rope", rope_params);
    auto norm = [&](const std::string &name) {
        Json p = Json::object();
        p.set("size", E);
        p.set("eps", rms_norm_eps);
        Json t = Json::object();
        t.set("weight", name);
        return part("rmsnorm", p, t);
    };
    Json layers = Json::array(), schedule = Json::array();
    for (long long i = 0; i < num_hidden_layers; i++) {
        std::string p = format("model.layers.%lld.", i);
        Json ap = Json::object();
        ap.set("hidden_size", E);
        ap.set("n_heads", num_attention_heads);
        ap.set("n_kv_heads", num_key_value_heads);
        ap.set("head_dim", head_dim);
        ap.set("position", rope);
        Json at = Json::object();
        for (const char *n : {"q", "k", "v", "o"})
            at.set(std::string(n) + "_proj.weight", p + "self_attn." + n + "_proj.weight");
        Json fp = Json::object();
        fp.set("hidden_size", E);
        fp.set("d_ff", intermediate_size);
        Json ft = Json::object();
        for (const char *n : {"gate", "up", "down"})
            ft.set(std::string(n) + "_proj.weight", p + "mlp." + n + "_proj.weight");
        Json layer = Json::object();
        layer.set("block", "prenorm");
        layer.set("mixer", part("gqa_attention", ap, at));
        layer.set("feed_forward", part("swiglu", fp, ft));
        layer.set("mixer_norm", norm(p + "input_layernorm.weight"));
        layer.set("feed_forward_norm", norm(p + "post_attention_layernorm.weight"));
        layers.push(layer);
        Json run = Json::object();
        run.set("layer", i);
        run.set("cache_from", Json());
        schedule.push(run);
    }
    Json ep = Json::object();
    ep.set("vocab_size", vocab_size);
    ep.set("hidden_size", E);
    Json et = Json::object();
    et.set("weight", "model.embed_tokens.weight");
    Json ht = Json::object();
    ht.set("weight", tie_word_embeddings ? "model.embed_tokens.weight" : "lm_head.weight");
    Json stops = Json::array();
    for (long long t : eos_token_ids) stops.push(Json(t));
    // tensors some checkpoints carry that the model does not use
    Json ignored = Json::array();
    ignored.push("model\\.layers\\.\\d+\\.self_attn\\.rotary_emb\\.inv_freq");
    if (tie_word_embeddings) ignored.push("lm_head\\.weight");
    Json s = Json::object();
    s.set("hidden_size", E);
    s.set("vocab_size", vocab_size);
    s.set("max_positions", max_position_embeddings);
    s.set("embedding", part("embedding", ep, et));
    s.set("layers", layers);
    s.set("schedule", schedule);
    s.set("final_norm", norm("model.norm.weight"));
    s.set("head", part("lm_head", ep, ht));
    s.set("stop_token_ids", stops);
    s.set("ignored_tensors", ignored);
    return s;
}

}  // namespace fg
