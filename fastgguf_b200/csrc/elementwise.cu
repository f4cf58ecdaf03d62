// Row-wise kernels of the decoder: embedding gather, RMSNorm, rotary encoding with cache
// append, SiLU-multiply.  Each takes both storage dtypes (f32, bf16) and computes in f32.
//
// Reference formulas (file fastgguf.c of the reference engine):
//   embedding  read_embedding            :4576-4581   x = Emb[token, :]
//   RMSNorm    rmsnorm_w                 :3100-3105   y = x * (1/sqrt(mean(x^2) + eps)) * w
//   RoPE       apply_rope                :3123-3145   (a, b) <- (a cos - b sin, a sin + b cos)
//   cache      forward                   :4720, 4738-4739   K stored after RoPE, V raw
//   SiLU-mul   silu_f, forward           :3118, 4876  t = g / (1 + exp(-g)) * u
#include "common.cuh"

// ------------------------------------------------------------------ embedding gather
template <typename TW>
__global__ void embed_gather_kernel(const TW *__restrict__ table, const int *__restrict__ tokens,
                                    float *__restrict__ x, int E) {
    pdl_launch_dependents();
    pdl_wait();
    int m = blockIdx.x;
    const TW *row = table + (size_t)tokens[m] * E;
    float *out = x + (size_t)m * E;
    for (int i = threadIdx.x; i < E; i += blockDim.x) out[i] = to_f32<TW>(row[i]);
}

extern "C" int fg_embed_gather(const void *table, int table_dtype, const int *tokens, float *x,
                               int M, int E, cudaStream_t stream) {
    if (M <= 0) return 0;
    int threads = E >= 1024 ? 256 : 128;
    if (table_dtype == FG_F32)
        return fg_launch(embed_gather_kernel<float>, dim3(M), dim3(threads), 0, stream, (const float *)table, tokens, x, E);
    else if (table_dtype == FG_BF16)
        return fg_launch(embed_gather_kernel<bf16>, dim3(M), dim3(threads), 0, stream, (const bf16 *)table, tokens, x, E);
    else return FG_ERR_BAD_DTYPE;
    return FG_LAUNCH_CHECK();
}

// The same gather that also starts a deferred RMSNorm: xw = bf16(x * norm_w) and the row's sum of squares
// (one "tile"), for a contraction that applies 1/rms in its epilogue.
template <typename TW>
__global__ void embed_gather_norm_kernel(const TW *__restrict__ table, const int *__restrict__ tokens,
                                         float *__restrict__ x, const float *__restrict__ norm_w,
                                         bf16 *__restrict__ xw, float *__restrict__ ss, int E) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    int m = blockIdx.x;
    const TW *row = table + (size_t)tokens[m] * E;
    float acc = 0.f;
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        float v = to_f32<TW>(row[i]);
        x[(size_t)m * E + i] = v;
        xw[(size_t)m * E + i] = __float2bfloat16_rn(v * norm_w[i]);
        acc += v * v;
    }
    acc = block_sum(acc, scratch);
    if (threadIdx.x == 0) ss[m] = acc;
}

extern "C" int fg_embed_gather_norm(const void *table, int table_dtype, const int *tokens, float *x,
                                    const float *norm_w, void *xw, float *ss, int M, int E, cudaStream_t stream) {
    if (M <= 0) return 0;
    int threads = E >= 1024 ? 256 : 128;
    if (table_dtype == FG_F32)
        return fg_launch(embed_gather_norm_kernel<float>, dim3(M), dim3(threads), 0, stream, (const float *)table, tokens, x,
                         norm_w, (bf16 *)xw, ss, E);
    if (table_dtype == FG_BF16)
        return fg_launch(embed_gather_norm_kernel<bf16>, dim3(M), dim3(threads), 0, stream, (const bf16 *)table, tokens, x,
                         norm_w, (bf16 *)xw, ss, E);
    return FG_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------ RMSNorm
// One block per output row.  `rows` (optional) names the input row of each output row, so the
// final norm runs only on the rows whose logits are wanted.  Statistics in f32 with a fixed
// reduction order: a row's result does not depend on what else is in the batch.
template <typename TO> __device__ __forceinline__ void store4(TO *dst, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float *dst, float a, float b, float c, float d) {
    *(float4 *)dst = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<bf16>(bf16 *dst, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    *(uint2 *)dst = make_uint2(*(uint32_t *)&lo, *(uint32_t *)&hi);
}

// VEC: rows are read and written four elements at a time (E % 4 == 0, 16-byte aligned rows)
template <typename TO, bool VEC>
__global__ void rmsnorm_kernel(const float *__restrict__ x, const float *__restrict__ w,
                               const int *__restrict__ rows, TO *__restrict__ out, int E, float eps) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    int r = blockIdx.x;
    const float *xi = x + (size_t)(rows ? rows[r] : r) * E;
    TO *o = out + (size_t)r * E;
    float ss = 0.f;
    if (VEC) {
        const float4 *x4 = (const float4 *)xi;
        for (int i = threadIdx.x; i < E / 4; i += blockDim.x) {
            float4 v = x4[i];
            ss += v.x * v.x; ss += v.y * v.y; ss += v.z * v.z; ss += v.w * v.w;
        }
    } else {
        for (int i = threadIdx.x; i < E; i += blockDim.x) { float v = xi[i]; ss += v * v; }
    }
    ss = block_sum(ss, scratch);
    float inv = 1.0f / sqrtf(ss / (float)E + eps);
    if (VEC) {
        const float4 *x4 = (const float4 *)xi, *w4 = (const float4 *)w;
        for (int i = threadIdx.x; i < E / 4; i += blockDim.x) {
            float4 v = x4[i], g = w4[i];
            store4<TO>(o + 4 * i, v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w);
        }
    } else {
        for (int i = threadIdx.x; i < E; i += blockDim.x) o[i] = from_f32<TO>(xi[i] * inv * w[i]);
    }
}

extern "C" int fg_rmsnorm(const float *x, const float *w, const int *rows, void *out, int out_dtype,
                          int R, int E, float eps, cudaStream_t stream) {
    if (R <= 0) return 0;
    bool vec = E % 4 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)out & 15) == 0;
    int per = vec ? E / 4 : E;
    int threads = per >= 1024 ? 256 : (per >= 256 ? 128 : 64);
    if (out_dtype == FG_F32) {
        if (vec) return fg_launch(rmsnorm_kernel<float, true>, dim3(R), dim3(threads), 0, stream, x, w, rows, (float *)out, E, eps);
        return fg_launch(rmsnorm_kernel<float, false>, dim3(R), dim3(threads), 0, stream, x, w, rows, (float *)out, E, eps);
    } else if (out_dtype == FG_BF16) {
        if (vec) return fg_launch(rmsnorm_kernel<bf16, true>, dim3(R), dim3(threads), 0, stream, x, w, rows, (bf16 *)out, E, eps);
        return fg_launch(rmsnorm_kernel<bf16, false>, dim3(R), dim3(threads), 0, stream, x, w, rows, (bf16 *)out, E, eps);
    }
    return FG_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------ RoPE + cache append
// qkv: [M, ld] rows of (q heads | k heads | v heads).  q is rotated in place; k is rotated and
// written, v copied, into the sequence's page at the row's position.  Pairs are (j, j + hd/2).
// cos/sin: [max_pos, hd/2] f32, built on the host in double.  Page pools: [n_pages, KV, P, hd].
template <typename T>
__global__ void rope_append_kernel(T *__restrict__ qkv, int ld, const int *__restrict__ positions,
                                   const int *__restrict__ row_seq, const int *__restrict__ block_table,
                                   int table_width, T *__restrict__ k_pool, T *__restrict__ v_pool,
                                   const float *__restrict__ cos_t, const float *__restrict__ sin_t,
                                   int H, int KV, int hd, int page_size, int write_kv) {
    pdl_launch_dependents();
    pdl_wait();
    int m = blockIdx.x;
    int pos = positions[m];
    int half = hd >> 1;
    T *row = qkv + (size_t)m * ld;
    const float *cs = cos_t + (size_t)pos * half, *sn = sin_t + (size_t)pos * half;
    // q heads
    for (int i = threadIdx.x; i < H * half; i += blockDim.x) {
        int h = i / half, j = i - h * half;
        T *p = row + h * hd;
        float a = to_f32<T>(p[j]), b = to_f32<T>(p[j + half]);
        float c = cs[j], s = sn[j];
        p[j] = from_f32<T>(a * c - b * s);
        p[j + half] = from_f32<T>(a * s + b * c);
    }
    if (!write_kv) return;
    int page = block_table[(size_t)row_seq[m] * table_width + pos / page_size];
    int off = pos % page_size;
    const T *krow = row + H * hd, *vrow = krow + KV * hd;
    for (int i = threadIdx.x; i < KV * half; i += blockDim.x) {
        int h = i / half, j = i - h * half;
        const T *p = krow + h * hd;
        float a = to_f32<T>(p[j]), b = to_f32<T>(p[j + half]);
        float c = cs[j], s = sn[j];
        T *dst = k_pool + (((size_t)page * KV + h) * page_size + off) * hd;
        dst[j] = from_f32<T>(a * c - b * s);
        dst[j + half] = from_f32<T>(a * s + b * c);
    }
    for (int i = threadIdx.x; i < KV * hd; i += blockDim.x) {
        int h = i / hd, d = i - h * hd;
        v_pool[(((size_t)page * KV + h) * page_size + off) * hd + d] = vrow[i];
    }
}

// bf16 rows with head sizes that are multiples of 16: eight pairs (two 16-byte loads) a thread
__global__ void rope_append_vec_kernel(bf16 *__restrict__ qkv, int ld, const int *__restrict__ positions,
                                       const int *__restrict__ row_seq, const int *__restrict__ block_table,
                                       int table_width, bf16 *__restrict__ k_pool, bf16 *__restrict__ v_pool,
                                       const float *__restrict__ cos_t, const float *__restrict__ sin_t,
                                       int H, int KV, int hd, int page_size, int write_kv) {
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x, pos = positions[m], half = hd >> 1, cph = half >> 3;   // chunks of 8 pairs per head
    bf16 *row = qkv + (size_t)m * ld;
    const float *cs = cos_t + (size_t)pos * half, *sn = sin_t + (size_t)pos * half;
    size_t kv_base = 0;
    if (write_kv) {
        int page = block_table[(size_t)row_seq[m] * table_width + pos / page_size];
        kv_base = ((size_t)page * KV * page_size + pos % page_size) * hd;              // + h * page_size * hd
    }
    const int n_rot = (H + (write_kv ? KV : 0)) * cph;
    for (int i = threadIdx.x; i < n_rot; i += blockDim.x) {
        int h = i / cph, j0 = (i - h * cph) * 8;
        const bf16 *src = row + (size_t)h * hd;                                         // k heads follow the q heads
        uint4 lo = *(const uint4 *)(src + j0), hi = *(const uint4 *)(src + j0 + half);
        float4 c0 = *(const float4 *)(cs + j0), c1 = *(const float4 *)(cs + j0 + 4);
        float4 s0 = *(const float4 *)(sn + j0), s1 = *(const float4 *)(sn + j0 + 4);
        const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        const __nv_bfloat162 *lp = (const __nv_bfloat162 *)&lo, *hp = (const __nv_bfloat162 *)&hi;
        uint4 olo, ohi;
        __nv_bfloat162 *ol = (__nv_bfloat162 *)&olo, *oh = (__nv_bfloat162 *)&ohi;
#pragma unroll
        for (int e = 0; e < 4; e++) {
            float2 a = __bfloat1622float2(lp[e]), b = __bfloat1622float2(hp[e]);
            ol[e] = __floats2bfloat162_rn(a.x * c[2 * e] - b.x * sv[2 * e], a.y * c[2 * e + 1] - b.y * sv[2 * e + 1]);
            oh[e] = __floats2bfloat162_rn(a.x * sv[2 * e] + b.x * c[2 * e], a.y * sv[2 * e + 1] + b.y * c[2 * e + 1]);
        }
        bf16 *dst = h < H ? row + (size_t)h * hd : k_pool + kv_base + (size_t)(h - H) * page_size * hd;
        *(uint4 *)(dst + j0) = olo;
        *(uint4 *)(dst + j0 + half) = ohi;
    }
    if (!write_kv) return;
    const bf16 *vrow = row + (size_t)(H + KV) * hd;
    for (int i = threadIdx.x; i < KV * (hd >> 3); i += blockDim.x) {
        int h = i / (hd >> 3), d0 = (i - h * (hd >> 3)) * 8;
        *(uint4 *)(v_pool + kv_base + (size_t)h * page_size * hd + d0) = *(const uint4 *)(vrow + (size_t)h * hd + d0);
    }
}

extern "C" int fg_rope_append(void *qkv, int dtype, int ld, const int *positions, const int *row_seq,
                              const int *block_table, int table_width, void *k_pool, void *v_pool,
                              const float *cos_t, const float *sin_t, int M, int H, int KV, int hd,
                              int page_size, int write_kv, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (hd % 2) return FG_ERR_BAD_SIZE;
    int work = H * hd / 2;
    int threads = work >= 1024 ? 256 : (work >= 128 ? 128 : 64);
    if (dtype == FG_BF16 && hd % 16 == 0 && ld % 8 == 0 && ((uintptr_t)qkv & 15) == 0 &&
        (!write_kv || ((((uintptr_t)k_pool | (uintptr_t)v_pool) & 15) == 0))) {
        int items = (H + KV) * (hd / 16);
        return fg_launch(rope_append_vec_kernel, dim3(M), dim3(items >= 256 ? 256 : (items >= 128 ? 128 : 64)), 0, stream,
                         (bf16 *)qkv, ld, positions, row_seq, block_table, table_width, (bf16 *)k_pool, (bf16 *)v_pool,
                         cos_t, sin_t, H, KV, hd, page_size, write_kv);
    }
    if (dtype == FG_F32)
        return fg_launch(rope_append_kernel<float>, dim3(M), dim3(threads), 0, stream, (float *)qkv, ld, positions, row_seq, block_table,
            table_width, (float *)k_pool, (float *)v_pool, cos_t, sin_t, H, KV, hd, page_size, write_kv);
    else if (dtype == FG_BF16)
        return fg_launch(rope_append_kernel<bf16>, dim3(M), dim3(threads), 0, stream, (bf16 *)qkv, ld, positions, row_seq, block_table,
            table_width, (bf16 *)k_pool, (bf16 *)v_pool, cos_t, sin_t, H, KV, hd, page_size, write_kv);
    else return FG_ERR_BAD_DTYPE;
    return FG_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ SiLU(g) * u
// gu: [M, 2F] rows of (gate | up); out: [M, F].
template <typename T>
__global__ void silu_mul_kernel(const T *__restrict__ gu, T *__restrict__ out, size_t total, int F) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        size_t m = i / F;
        int f = (int)(i - m * F);
        float g = to_f32<T>(gu[m * 2 * F + f]), u = to_f32<T>(gu[m * 2 * F + F + f]);
        out[i] = from_f32<T>(g / (1.0f + expf(-g)) * u);
    }
}

extern "C" int fg_silu_mul(const void *gu, void *out, int dtype, int M, int F, cudaStream_t stream) {
    size_t total = (size_t)M * F;
    if (total == 0) return 0;
    int threads = 256;
    size_t want = (total + threads - 1) / threads;
    int blocks = (int)(want > 148 * 16 ? 148 * 16 : want);
    if (dtype == FG_F32)
        return fg_launch(silu_mul_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float *)gu, (float *)out, total, F);
    else if (dtype == FG_BF16)
        return fg_launch(silu_mul_kernel<bf16>, dim3(blocks), dim3(threads), 0, stream, (const bf16 *)gu, (bf16 *)out, total, F);
    else return FG_ERR_BAD_DTYPE;
    return FG_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ decode feedback
// After a decode step of a fixed-shape (graph-replayed) batch: the sampled token of every row
// becomes its next input, and live rows move on by one position.
__global__ void decode_advance_kernel(int *__restrict__ tokens, int *__restrict__ positions,
                                      const int *__restrict__ next_tokens, const int *__restrict__ active, int B) {
    pdl_launch_dependents();
    pdl_wait();
    int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    tokens[b] = next_tokens[b];
    if (active[b]) positions[b] += 1;
}

extern "C" int fg_decode_advance(int *tokens, int *positions, const int *next_tokens, const int *active, int B,
                                 cudaStream_t stream) {
    if (B <= 0) return 0;
    return fg_launch(decode_advance_kernel, dim3((B + 127) / 128), dim3(128), 0, stream, tokens, positions, next_tokens, active, B);
}
