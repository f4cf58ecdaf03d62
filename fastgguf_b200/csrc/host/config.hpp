// Typed model configuration, read from the architecture's own config.json keys, and the one
// registry from an architecture's name to its model.
//
// The reference reads the same numbers from GGUF metadata through kv_num(g, key, default)
// (fastgguf.c:448-454) with an architecture prefix (:4189), fails with "bad config" on nonsense
// (:4215-4218), and picks its code path by strcmp on general.architecture, carrying on with the
// Llama path for unknown names (:4191-4198).  Here an unknown name is an error that lists what is
// registered, and every size or constant config.json gives lives in the typed object only.
#pragma once
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "errors.hpp"
#include "json.hpp"

namespace fg {

// A configuration of some architecture.  `spec()` is the model as data (see fastgguf_parts.h).
class ModelConfig {
public:
    virtual ~ModelConfig() = default;
    virtual const std::string &architecture() const = 0;
    virtual Json to_json() const = 0;        // the config.json form
    virtual Json describe() const = 0;       // every field plus derived sizes
    virtual Json spec() const = 0;
};

struct RopeScaling {
    std::string rope_type = "default";       // "default" (none) or "llama3"
    double factor = 1.0, low_freq_factor = 1.0, high_freq_factor = 1.0;
    long long original_max_position_embeddings = 0;
    Json to_json() const;                    // null for "default"
};

// The dense Llama decoder's config.json (keys and the reference's defaults for absent ones:
// rms_norm_eps 1e-6 fastgguf.c:4228, rope_theta 10000 :4224, head_dim = hidden / heads :4281-4283).
class LlamaConfig : public ModelConfig {
public:
    long long hidden_size = 0, num_hidden_layers = 0, num_attention_heads = 0, num_key_value_heads = 0;
    long long head_dim = 0, intermediate_size = 0, vocab_size = 0, max_position_embeddings = 0;
    double rms_norm_eps = 0.0, rope_theta = 0.0;
    RopeScaling rope_scaling;
    bool tie_word_embeddings = false;
    std::string torch_dtype = "bfloat16", hidden_act = "silu";
    bool has_bos = false;
    long long bos_token_id = 0;
    std::vector<long long> eos_token_ids;
    std::vector<std::string> defaulted;      // keys the file did not give

    static std::unique_ptr<ModelConfig> from_json(const Json &d);
    void validate() const;
    long long q_dim() const { return num_attention_heads * head_dim; }
    long long kv_dim() const { return num_key_value_heads * head_dim; }
    long long parameter_count() const;

    const std::string &architecture() const override;
    Json to_json() const override;
    Json describe() const override;
    Json spec() const override;
};

using ConfigReader = std::function<std::unique_ptr<ModelConfig>(const Json &)>;

void register_architecture(const std::string &name, ConfigReader reader);
std::vector<std::string> registered_architectures();
std::unique_ptr<ModelConfig> config_from_json(const Json &d);
std::unique_ptr<ModelConfig> config_from_dir(const std::string &model_dir);
Json read_config_json(const std::string &model_dir);
Json merge_generation_config(const std::string &model_dir, const Json &d);

// typed key access with the messages of a configuration error
long long take_int(const Json &d, const std::string &key, const char *where = "config.json");
long long take_int(const Json &d, const std::string &key, long long dflt, const char *where = "config.json");
double take_float(const Json &d, const std::string &key, const char *where = "config.json");
double take_float(const Json &d, const std::string &key, double dflt, const char *where = "config.json");
bool take_bool(const Json &d, const std::string &key, bool dflt, const char *where = "config.json");
std::string take_string(const Json &d, const std::string &key, const std::string &dflt, const char *where = "config.json");
std::string json_repr(const Json &v);        // how a value is quoted in an error message

std::string read_text_file(const std::string &path, bool *exists = nullptr);

}  // namespace fg
