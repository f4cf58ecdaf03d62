/* Adding parts to the engine from outside: the model spec (JSON) and the C interface a new kind of
 * norm, position encoding, mixer, feed-forward, block arrangement, embedding or head has to offer.
 *
 * The reference chooses between such variants with flags and optional per-layer tensors on one struct
 * (is_swa[], kv_donor[], act_gelu, rope_neox, embd_scale, final_softcap: fastgguf.c:4064-4100, :4191-4229).
 * Here a layer names the KIND of each of its parts, kinds are looked up in one registry per role, and a
 * kind the library does not have is registered with fg_register_part - no file of the library changes.
 *
 * The model spec
 *   {"hidden_size": E, "vocab_size": V, "max_positions": N,
 *    "embedding":  PART, "final_norm": PART, "head": PART,
 *    "layers":   [{"block": "prenorm", "mixer": PART, "feed_forward": PART, "mixer_norm": PART,
 *                  "feed_forward_norm": PART}, ...],
 *    "schedule": [{"layer": 0, "cache_from": null}, ...],      the order in which layers run: an entry may
 *                                                               name a layer twice (a cache of its own each
 *                                                               time) or read an EARLIER entry's cache
 *    "stop_token_ids": [...], "ignored_tensors": ["regex", ...]}
 *   PART = {"kind": "rmsnorm", "params": {...}, "tensors": {"local name": "checkpoint name"}}
 *   A parameter whose value is itself {"kind": ..., "params": ...} is a nested part (the position encoding
 *   of an attention mixer); nested parts with equal kind and parameters are built once and shared.
 *
 * Built-in kinds
 *   norm          "rmsnorm"        {size, eps}
 *   position      "rope"           {head_dim, theta, scaling: null | {rope_type: "llama3", ...},
 *                                   rotary_dim: head_dim, layout: "halves" | "adjacent"}
 *   mixer         "gqa_attention"  {hidden_size, n_heads, n_kv_heads, head_dim, position: PART | null,
 *                                   scale: null = 1/sqrt(head_dim), window: null}
 *   feed_forward  "swiglu"         {hidden_size, d_ff}
 *   block         "prenorm"        x += mixer(norm1(x)); x += feed_forward(norm2(x))
 *   embedding     "embedding"      {vocab_size, hidden_size, scale: 1.0}
 *   head          "lm_head"        {vocab_size, hidden_size}
 *
 * What a part may rely on in fg_batch_view: every device array, and the host integers n_seq, n_rows,
 * n_want, max_new, max_len, single_token, want_all, table_width.  The three host_* arrays are NULL when the
 * step is being recorded into a CUDA graph (the decode step of the generation loop): a part that needs
 * per-sequence bounds then reads cu_rows / seq_start / slots on the device.  Under graph replay rows of
 * finished or padded sequences name the slot `n_slots` (a spare row that every state array has) and page 0
 * of every cache group, so whatever a part writes for them lands where nothing reads.
 * A part launches its work on call->stream and takes scratch memory from call->alloc (valid until the step
 * ends; the same addresses at every replay of a recorded step).  It must not allocate, free or synchronise.
 */
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FG_ROLE_NORM 0
#define FG_ROLE_POSITION 1
#define FG_ROLE_MIXER 2
#define FG_ROLE_FEED_FORWARD 3
#define FG_ROLE_BLOCK 4
#define FG_ROLE_EMBEDDING 5
#define FG_ROLE_HEAD 6

typedef struct fg_tensor_decl {
    char name[96];           /* the part's local tensor name */
    int ndim;
    int64_t shape[4];
    int is_int;              /* 0: a float tensor (follows the engine's dtype policy); 1: an int32 table */
    int init;                /* random weights: 0 = N(0, std), 1 = 1 + N(0, std) */
    float std;
} fg_tensor_decl;

typedef struct fg_dev_tensor {
    void *data;              /* device memory */
    int dtype;               /* FG_F32 0, FG_BF16 1, FG_I32 3 */
    int ndim;
    int64_t shape[4];
    int64_t ld;              /* elements between rows of a 2-d tensor */
} fg_dev_tensor;

typedef struct fg_batch_view {
    int n_seq, n_rows, n_want, max_new, max_len, single_token, want_all;
    const int *tokens;       /* [n_rows] token ids */
    const int *positions;    /* [n_rows] position of each row in its sequence */
    const int *row_seq;      /* [n_rows] index of the row's sequence within the step */
    const int *cu_rows;      /* [n_seq + 1] first row of each sequence */
    const int *seq_start;    /* [n_seq] length of each sequence before the step */
    const int *slots;        /* [n_seq] cache / state slot of each sequence */
    const int *want_rows;    /* [n_want] rows whose logits are wanted, or NULL */
    int n_groups;
    const int *const *block_tables;   /* per cache group: [n_seq, table_width] page ids (device) */
    int table_width;
    const int *host_cu_rows, *host_seq_start, *host_slots;   /* host copies; NULL while a graph records */
    void *stream;
} fg_batch_view;

typedef struct fg_layer_io {
    int group;               /* cache group of this entry (index into block_tables), -1 = none */
    void *k_pool, *v_pool;   /* [n_pages, n_kv_heads, page_size, head_dim] in the engine's dtype, or NULL */
    int n_pages, page_size, n_kv_heads, head_dim, cache_dtype;
    int write_cache;         /* 0: the pools belong to an earlier entry; read only */
    void *state;             /* [n_slots + 1, state_bytes] fixed-size state of this entry, or NULL */
    int64_t state_bytes;
    int n_slots;
} fg_layer_io;

struct fg_part_call;
typedef struct fg_block_ops {       /* what a block arrangement may ask the engine to run (ctx = call) */
    /* which: 0 = the mixer's norm, 1 = the feed-forward's norm; returns normalised rows [M, E] */
    int (*norm)(const struct fg_part_call *call, int which, fg_dev_tensor *xn_out);
    int (*mixer)(const struct fg_part_call *call, const fg_dev_tensor *xn);          /* adds into call->residual */
    int (*feed_forward)(const struct fg_part_call *call, const fg_dev_tensor *xn);   /* adds into call->residual */
} fg_block_ops;

typedef struct fg_part_call {
    int role;
    const fg_batch_view *batch;
    const fg_layer_io *io;          /* mixer and block: the entry's cache pools and state */
    fg_dev_tensor x;                /* norm: the residual stream in, f32 [M, E]; embedding: f32 [M, E] to fill */
    fg_dev_tensor xn;               /* mixer, feed_forward, head: normalised rows in the activation dtype */
    fg_dev_tensor out;              /* norm: [R, E] in the activation dtype; head: f32 [R, V] */
    fg_dev_tensor residual;         /* mixer, feed_forward, block: f32 [M, E]; ADD the part's output into it */
    const int *rows;                /* norm: device indices of the R rows to normalise, or NULL for all */
    int n_rows;
    void *(*alloc)(void *alloc_ctx, size_t bytes);   /* 256-byte aligned device scratch for this step */
    void *alloc_ctx;
    const fg_block_ops *block_ops;  /* block only */
    void *engine_ctx;               /* block only: opaque */
    void *stream;
} fg_part_call;

typedef struct fg_part_vtable {
    /* A new instance from the part's parameters (JSON text).  dtype: the engine's activation dtype.
     * NULL with a message in err refuses the parameters. */
    void *(*create)(const char *params_json, int dtype, void *user, char *err, size_t err_cap);
    void (*destroy)(void *self);
    int (*n_tensors)(void *self);
    int (*tensor_decl)(void *self, int i, fg_tensor_decl *out);
    /* Tensor i on the device (engine dtype policy applied); it lives as long as the engine. */
    int (*load)(void *self, int i, const fg_dev_tensor *t);
    /* mixer: 1 and the three numbers if it keeps keys and values per position (window 0 = all of them) */
    int (*cache_request)(void *self, int *n_kv_heads, int *head_dim, int *window);
    /* mixer: bytes of fixed-size state per sequence (zeroed when a sequence takes its slot); 0 = none */
    int64_t (*state_bytes)(void *self);
    /* position: fill cos/sin [max_positions, head_dim / 2] (host, float32) for pairs (j, j + head_dim / 2), and
     * perm [head_dim]: perm[i] = the row of a head (as stored) that becomes row i, so that the stored pairs
     * land on (j, j + head_dim / 2); the identity for the halves layout. */
    int (*position_tables)(void *self, int max_positions, int head_dim, float *cos_out, float *sin_out, int *perm);
    /* every other role: run on call->stream; 0 or an FG_E_* status */
    int (*forward)(void *self, const fg_part_call *call);
    void *user;
} fg_part_vtable;

/* Unused entries may be NULL.  The table is copied; `kind` must not clash with a built-in kind. */
int fg_register_part(int role, const char *kind, const fg_part_vtable *vt);

#ifdef __cplusplus
}
#endif
