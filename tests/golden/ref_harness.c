// Calls the reference engine's own model code on a GGUF file and dumps logits.
// Built by make_golden.py as:  gcc -O2 -I<reference dir> ref_harness.c -lm -ldl
// The reference is one translation unit with static functions; defining FG_VARIANT renames its
// entry points (fastgguf.c:48-59) so that it can be included and its forward() called directly.
#define FG_VARIANT golden
#include "fastgguf.c"

int main(int argc, char **argv) {
    if (argc < 4) { fprintf(stderr, "usage: harness model.gguf out.f32 tok tok ...\n"); return 1; }
    fp16_init();
    gguf_t g;
    if (gguf_open(&g, argv[1]) != 0) return 2;
    model_t *m = (model_t *)calloc(1, sizeof(model_t));
    if (model_load(m, &g, 128) != 0) return 2;
    FILE *f = fopen(argv[2], "wb");
    for (int i = 3; i < argc; i++) {
        float *lg = forward(m, atoi(argv[i]), i - 3);      // one token at a time, position i - 3
        if (!lg) return 3;
        fwrite(lg, sizeof(float), m->n_vocab, f);
    }
    fclose(f);
    // the same tokens through the prompt path (chunks) must give the same last row
    return 0;
}
