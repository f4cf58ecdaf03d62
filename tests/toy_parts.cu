// Toy parts for the tests, built into a shared library of their own and registered through the C interface of
// fastgguf_parts.h - no file of the framework changes.  They are no model of anyone's:
//   toy_running_mean   mixer with fixed-size state of its own (no keys, no values): out_t = W * mean(xn_0 .. xn_t)
//   toy_routed         feed-forward with routing: two experts, each row goes to the one its router scores higher
//   toy_half_rotary    position encoding: rotates the first `rot` pairs of a head with scaled positions
//   toy_scaled_embed   embedding: table row times a constant
//   toy_parallel       block arrangement: x += mixer(norm1(x)) + feed_forward(norm2(x)), both norms of the SAME x
// Every kernel reads the step's shape from the DEVICE arrays of the batch view, so the parts also run inside a
// recorded decode step, where padded rows name the spare state row and page 0.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "fastgguf_parts.h"

#define FG_F32 0
#define FG_BF16 1

static double json_number(const char *json, const char *key, double dflt) {
    char pat[128];
    snprintf(pat, sizeof pat, "\"%s\"", key);
    const char *p = strstr(json, pat);
    if (!p) return dflt;
    p = strchr(p + strlen(pat), ':');
    return p ? strtod(p + 1, nullptr) : dflt;
}

__device__ __forceinline__ float load_elem(const void *p, int dtype, long long i) {
    return dtype == FG_F32 ? ((const float *)p)[i] : __bfloat162float(((const __nv_bfloat16 *)p)[i]);
}

static void decl(fg_tensor_decl *d, const char *name, long long rows, long long cols) {
    memset(d, 0, sizeof *d);
    snprintf(d->name, sizeof d->name, "%s", name);
    d->ndim = 2;
    d->shape[0] = rows;
    d->shape[1] = cols;
    d->std = 0.02f;
}

// ------------------------------------------------------------------------------------ running-mean mixer
struct RunningMean {
    int E;
    fg_dev_tensor w;
};

static void *rm_create(const char *params, int, void *, char *err, size_t cap) {
    int E = (int)json_number(params, "hidden_size", 0);
    if (E <= 0 || E > 1024) { snprintf(err, cap, "hidden_size must lie in 1..1024"); return nullptr; }
    RunningMean *m = new RunningMean();
    m->E = E;
    return m;
}
static void rm_destroy(void *self) { delete (RunningMean *)self; }
static int rm_n_tensors(void *) { return 1; }
static int rm_tensor_decl(void *self, int, fg_tensor_decl *d) {
    decl(d, "mix.weight", ((RunningMean *)self)->E, ((RunningMean *)self)->E);
    return 0;
}
static int rm_load(void *self, int, const fg_dev_tensor *t) { ((RunningMean *)self)->w = *t; return 0; }
static int64_t rm_state_bytes(void *self) { return (int64_t)(((RunningMean *)self)->E + 1) * 4; }

// one block per sequence, E threads; the sequence's rows in order; state row = [running sum (E), count]
__global__ void running_mean_kernel(const void *xn, int xn_dtype, long long ldx, float *residual, long long ldr, const void *w,
                                    int w_dtype, long long ldw, const int *cu_rows, const int *slots, float *state, int E) {
    extern __shared__ float mean[];
    const int s = blockIdx.x, j = threadIdx.x;
    float *st = state + (long long)slots[s] * (E + 1);
    float sum = st[j], count = st[E];
    for (int row = cu_rows[s]; row < cu_rows[s + 1]; row++) {
        sum += load_elem(xn, xn_dtype, row * ldx + j);
        count += 1.0f;
        __syncthreads();
        mean[j] = sum / count;
        __syncthreads();
        float acc = 0.f;
        for (int k = 0; k < E; k++) acc += load_elem(w, w_dtype, j * ldw + k) * mean[k];
        residual[row * ldr + j] += acc;
    }
    __syncthreads();
    st[j] = sum;
    if (j == 0) st[E] = count;
}

static int rm_forward(void *self, const fg_part_call *c) {
    RunningMean *m = (RunningMean *)self;
    if (!c->io->state || c->io->state_bytes < (long long)(m->E + 1) * 4) return 9;
    running_mean_kernel<<<c->batch->n_seq, m->E, m->E * sizeof(float), (cudaStream_t)c->stream>>>(
        c->xn.data, c->xn.dtype, c->xn.ld, (float *)c->residual.data, c->residual.ld, m->w.data, m->w.dtype, m->w.ld,
        c->batch->cu_rows, c->batch->slots, (float *)c->io->state, m->E);
    return cudaGetLastError() == cudaSuccess ? 0 : 7;
}

// ------------------------------------------------------------------------------------ routed feed-forward
struct Routed {
    int E, F;
    fg_dev_tensor t[5];          // router, up 0, down 0, up 1, down 1
};
static void *rt_create(const char *params, int, void *, char *err, size_t cap) {
    Routed *r = new Routed();
    r->E = (int)json_number(params, "hidden_size", 0);
    r->F = (int)json_number(params, "d_ff", 0);
    if (r->E <= 0 || r->F <= 0 || r->E + r->F > 8000) { snprintf(err, cap, "bad sizes"); delete r; return nullptr; }
    return r;
}
static void rt_destroy(void *self) { delete (Routed *)self; }
static int rt_n_tensors(void *) { return 5; }
static int rt_tensor_decl(void *self, int i, fg_tensor_decl *d) {
    Routed *r = (Routed *)self;
    static const char *names[] = {"router.weight", "experts.0.up", "experts.0.down", "experts.1.up", "experts.1.down"};
    if (i == 0) decl(d, names[0], 2, r->E);
    else if (i % 2 == 1) decl(d, names[i], r->F, r->E);
    else decl(d, names[i], r->E, r->F);
    return 0;
}
static int rt_load(void *self, int i, const fg_dev_tensor *t) { ((Routed *)self)->t[i] = *t; return 0; }

// one block per row; router logits in float32, first maximum wins
__global__ void routed_kernel(const void *xn, int xn_dtype, long long ldx, float *residual, long long ldr, fg_dev_tensor router,
                              fg_dev_tensor up0, fg_dev_tensor down0, fg_dev_tensor up1, fg_dev_tensor down1, int E, int F) {
    extern __shared__ float sh[];
    float *x = sh, *h = sh + E;
    __shared__ int pick;
    const int row = blockIdx.x;
    for (int k = threadIdx.x; k < E; k += blockDim.x) x[k] = load_elem(xn, xn_dtype, row * ldx + k);
    __syncthreads();
    if (threadIdx.x == 0) {
        float l0 = 0.f, l1 = 0.f;
        for (int k = 0; k < E; k++) {
            l0 += load_elem(router.data, router.dtype, k) * x[k];
            l1 += load_elem(router.data, router.dtype, router.ld + k) * x[k];
        }
        pick = l1 > l0 ? 1 : 0;
    }
    __syncthreads();
    const fg_dev_tensor &up = pick ? up1 : up0, &down = pick ? down1 : down0;
    for (int f = threadIdx.x; f < F; f += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < E; k++) acc += load_elem(up.data, up.dtype, f * up.ld + k) * x[k];
        h[f] = fmaxf(acc, 0.f);
    }
    __syncthreads();
    for (int j = threadIdx.x; j < E; j += blockDim.x) {
        float acc = 0.f;
        for (int f = 0; f < F; f++) acc += load_elem(down.data, down.dtype, j * down.ld + f) * h[f];
        residual[row * ldr + j] += acc;
    }
}

static int rt_forward(void *self, const fg_part_call *c) {
    Routed *r = (Routed *)self;
    int M = (int)c->xn.shape[0];
    if (M <= 0) return 0;
    routed_kernel<<<M, 128, (r->E + r->F) * sizeof(float), (cudaStream_t)c->stream>>>(
        c->xn.data, c->xn.dtype, c->xn.ld, (float *)c->residual.data, c->residual.ld, r->t[0], r->t[1], r->t[2], r->t[3], r->t[4],
        r->E, r->F);
    return cudaGetLastError() == cudaSuccess ? 0 : 7;
}

// ------------------------------------------------------------------------------------ half-rotary position encoding
struct HalfRotary {
    int hd, rot;
    double theta, scale;
};
static void *hr_create(const char *params, int, void *, char *err, size_t cap) {
    HalfRotary *h = new HalfRotary();
    h->hd = (int)json_number(params, "head_dim", 0);
    h->rot = (int)json_number(params, "rot", 0);
    h->theta = json_number(params, "theta", 10000.0);
    h->scale = json_number(params, "scale", 1.0);
    if (h->hd <= 0 || h->rot < 0 || h->rot > h->hd / 2) { snprintf(err, cap, "rot must lie in 0..head_dim/2"); delete h; return nullptr; }
    return h;
}
static void hr_destroy(void *self) { delete (HalfRotary *)self; }
// pairs (j, j + head_dim/2) as the engine's kernels rotate them; the first `rot` pairs turn, the others stay (cos 1, sin 0)
static int hr_tables(void *self, int max_positions, int head_dim, float *cos_out, float *sin_out, int *) {
    HalfRotary *h = (HalfRotary *)self;
    if (head_dim != h->hd) return 2;
    int half = head_dim / 2;
    for (int pos = 0; pos < max_positions; pos++)
        for (int j = 0; j < half; j++) {
            double ang = j < h->rot ? pos * h->scale * pow(h->theta, -2.0 * j / head_dim) : 0.0;
            cos_out[(size_t)pos * half + j] = (float)cos(ang);
            sin_out[(size_t)pos * half + j] = (float)sin(ang);
        }
    return 0;
}

// ------------------------------------------------------------------------------------ scaled embedding
struct ScaledEmbed {
    int V, E;
    float scale;
    fg_dev_tensor w;
};
static void *se_create(const char *params, int, void *, char *err, size_t cap) {
    ScaledEmbed *e = new ScaledEmbed();
    e->V = (int)json_number(params, "vocab_size", 0);
    e->E = (int)json_number(params, "hidden_size", 0);
    e->scale = (float)json_number(params, "scale", 1.0);
    if (e->V <= 0 || e->E <= 0) { snprintf(err, cap, "bad sizes"); delete e; return nullptr; }
    return e;
}
static void se_destroy(void *self) { delete (ScaledEmbed *)self; }
static int se_n_tensors(void *) { return 1; }
static int se_tensor_decl(void *self, int, fg_tensor_decl *d) {
    decl(d, "weight", ((ScaledEmbed *)self)->V, ((ScaledEmbed *)self)->E);
    return 0;
}
static int se_load(void *self, int, const fg_dev_tensor *t) { ((ScaledEmbed *)self)->w = *t; return 0; }
__global__ void scaled_embed_kernel(const int *tokens, fg_dev_tensor w, float *x, long long ldx, int E, float scale) {
    const int row = blockIdx.x, tok = tokens[row];
    for (int k = threadIdx.x; k < E; k += blockDim.x) x[row * ldx + k] = load_elem(w.data, w.dtype, tok * w.ld + k) * scale;
}
static int se_forward(void *self, const fg_part_call *c) {
    ScaledEmbed *e = (ScaledEmbed *)self;
    int M = c->batch->n_rows;
    if (M <= 0) return 0;
    scaled_embed_kernel<<<M, 64, 0, (cudaStream_t)c->stream>>>(c->batch->tokens, e->w, (float *)c->x.data, c->x.ld, e->E, e->scale);
    return cudaGetLastError() == cudaSuccess ? 0 : 7;
}

// ------------------------------------------------------------------------------------ parallel block
static void *pb_create(const char *, int, void *, char *, size_t) { return new int(0); }
static void pb_destroy(void *self) { delete (int *)self; }
static int pb_forward(void *, const fg_part_call *c) {
    fg_dev_tensor a, b;
    int e = c->block_ops->norm(c, 0, &a);          // both norms read the block's input ...
    if (e) return e;
    e = c->block_ops->norm(c, 1, &b);
    if (e) return e;
    e = c->block_ops->mixer(c, &a);                // ... before either part adds into it
    if (e) return e;
    return c->block_ops->feed_forward(c, &b);
}

extern "C" {
const fg_part_vtable *toy_running_mean_vtable(void) {
    static fg_part_vtable vt = {};
    vt.create = rm_create; vt.destroy = rm_destroy; vt.n_tensors = rm_n_tensors; vt.tensor_decl = rm_tensor_decl;
    vt.load = rm_load; vt.state_bytes = rm_state_bytes; vt.forward = rm_forward;
    return &vt;
}
const fg_part_vtable *toy_routed_vtable(void) {
    static fg_part_vtable vt = {};
    vt.create = rt_create; vt.destroy = rt_destroy; vt.n_tensors = rt_n_tensors; vt.tensor_decl = rt_tensor_decl;
    vt.load = rt_load; vt.forward = rt_forward;
    return &vt;
}
const fg_part_vtable *toy_half_rotary_vtable(void) {
    static fg_part_vtable vt = {};
    vt.create = hr_create; vt.destroy = hr_destroy; vt.position_tables = hr_tables;
    return &vt;
}
const fg_part_vtable *toy_scaled_embed_vtable(void) {
    static fg_part_vtable vt = {};
    vt.create = se_create; vt.destroy = se_destroy; vt.n_tensors = se_n_tensors; vt.tensor_decl = se_tensor_decl;
    vt.load = se_load; vt.forward = se_forward;
    return &vt;
}
const fg_part_vtable *toy_parallel_vtable(void) {
    static fg_part_vtable vt = {};
    vt.create = pb_create; vt.destroy = pb_destroy; vt.forward = pb_forward;
    return &vt;
}
}
