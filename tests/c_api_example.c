/* A C program on the engine's C interface: a tiny random Llama, a batch of three prompts, eight greedy tokens each.
 * Built and run by tests/test_c_api.py; prints one line of token ids per prompt.
 *
 *     cc c_api_example.c -I fastgguf_b200/csrc -L fastgguf_b200/csrc/_build -lfg_engine -o example
 */
#include <stdio.h>

#include "fastgguf_engine.h"

static const char *CONFIG =
    "{\"architectures\": [\"LlamaForCausalLM\"], \"hidden_size\": 64, \"num_hidden_layers\": 2, \"num_attention_heads\": 4,"
    " \"num_key_value_heads\": 2, \"head_dim\": 16, \"intermediate_size\": 192, \"vocab_size\": 256, \"rms_norm_eps\": 1e-5,"
    " \"rope_theta\": 10000.0, \"max_position_embeddings\": 512, \"tie_word_embeddings\": true, \"eos_token_id\": 2}";

#define CHECK(call)                                                            \
    do {                                                                       \
        int rc_ = (call);                                                      \
        if (rc_ != FG_OK) {                                                    \
            fprintf(stderr, "%s: status %d: %s\n", #call, rc_, fg_last_error()); \
            return 1;                                                          \
        }                                                                      \
    } while (0)

int main(int argc, char **argv) {
    fg_config *cfg = NULL;
    fg_engine *engine = NULL;
    fg_result *result = NULL;
    fg_engine_options opts;
    fg_sampling sampling;
    const int prompts[] = {5, 17, 3, 9, 200, 1, 1, 4, 77};
    const int64_t offsets[] = {0, 3, 4, 9};
    int i, k;

    CHECK(fg_config_from_json(CONFIG, &cfg));
    fg_engine_default_options(&opts);
    opts.dtype = (argc > 1 && argv[1][0] == 'b') ? 1 /* FG_BF16 */ : 0 /* FG_F32 */;
    opts.max_batch = 4;
    opts.max_tokens = 1024;
    CHECK(fg_engine_create_random(cfg, 7, &opts, &engine));
    fg_sampling_default(&sampling);
    sampling.temp = 0.0f;                               /* greedy */
    CHECK(fg_generate(engine, 3, prompts, offsets, &sampling, 8, NULL, 0, 0, -1, NULL, NULL, &result));
    for (i = 0; i < fg_result_count(result); i++) {
        const int *tokens;
        int n, why;
        CHECK(fg_result_get(result, i, &tokens, &n, &why));
        for (k = 0; k < n; k++) printf("%d%s", tokens[k], k + 1 < n ? " " : "");
        printf("\n");
    }
    /* a status code, not a crash: a slot that nobody holds */
    if (fg_slot_release(engine, 3) != FG_E_CACHE) return 2;
    fg_result_destroy(result);
    fg_engine_destroy(engine);
    fg_config_destroy(cfg);
    return 0;
}
