// Attention over the paged cache for any head size and any dtype: the true 32-bit path and
// the any-size fallback.  One block per (token row, query head).
//
// Reference formulas (fastgguf.c): scores s_p = scale * (q . K[p]) for p in [lo, pos]
// (:3246, :3317), the mask is the loop range (:4782, :5030-5035), softmax with max
// subtraction (:3147-3156), o = sum_p w_p V[p] (:3320-3323); query head h uses KV head
// h / (H / KV) (:4781).  A window of w keeps only the last w positions (:4754-4758).
//
// Keys are visited in chunks of CHUNK positions counted from lo, with a running maximum and
// sum in f32 (online softmax).  The order depends only on the row's own position, so a row's
// result is the same whatever else is in the batch and however the tokens were cut into steps.
#include "common.cuh"

#define ATT_THREADS 128
#define CHUNK 1024

template <typename T>
__global__ void __launch_bounds__(ATT_THREADS)
attention_generic_kernel(const T *__restrict__ q, int ldq, T *__restrict__ out, int ldo,
                         const int *__restrict__ positions, const int *__restrict__ row_seq,
                         const int *__restrict__ block_table, int table_width,
                         const T *__restrict__ k_pool, const T *__restrict__ v_pool,
                         int H, int KV, int hd, int page_size, float scale, int window) {
    extern __shared__ float smem[];
    float *qs = smem;                 // [hd]
    float *sc = smem + hd;            // [CHUNK]
    __shared__ float scratch[32];
    int m = blockIdx.x, h = blockIdx.y;
    int kvh = h / (H / KV);
    int pos = positions[m];
    int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int *bt = block_table + (size_t)row_seq[m] * table_width;
    const T *qrow = q + (size_t)m * ldq + (size_t)h * hd;
    for (int d = threadIdx.x; d < hd; d += ATT_THREADS) qs[d] = to_f32<T>(qrow[d]);
    __syncthreads();

    float m_run = -INFINITY, l_run = 0.f;
    float acc0 = 0.f, acc1 = 0.f;     // output dims threadIdx.x and threadIdx.x + 128 (hd <= 256)
    for (int c0 = lo; c0 <= pos; c0 += CHUNK) {
        int n = min(CHUNK, pos - c0 + 1);
        float cmax = -INFINITY;
        for (int i = threadIdx.x; i < n; i += ATT_THREADS) {
            int p = c0 + i;
            const T *kr = k_pool + (((size_t)bt[p / page_size] * KV + kvh) * page_size + p % page_size) * hd;
            float s = 0.f;
            for (int d = 0; d < hd; d++) s = fmaf(qs[d], to_f32<T>(kr[d]), s);
            s *= scale;
            sc[i] = s;
            cmax = fmaxf(cmax, s);
        }
        cmax = block_max(cmax, scratch);
        float m_new = fmaxf(m_run, cmax);
        float csum = 0.f;
        for (int i = threadIdx.x; i < n; i += ATT_THREADS) {
            float e = expf(sc[i] - m_new);
            sc[i] = e;
            csum += e;
        }
        csum = block_sum(csum, scratch);   // its barriers also publish sc[] to every thread
        float corr = expf(m_run - m_new);  // 0 on the first chunk (m_run = -inf)
        l_run = l_run * corr + csum;
        acc0 *= corr; acc1 *= corr;
        int d0 = threadIdx.x, d1 = threadIdx.x + ATT_THREADS;
        if (d0 < hd) {
            for (int i = 0; i < n; i++) {
                int p = c0 + i;
                const T *vr = v_pool + (((size_t)bt[p / page_size] * KV + kvh) * page_size + p % page_size) * hd;
                float w = sc[i];
                acc0 = fmaf(w, to_f32<T>(vr[d0]), acc0);
                if (d1 < hd) acc1 = fmaf(w, to_f32<T>(vr[d1]), acc1);
            }
        }
        m_run = m_new;
        __syncthreads();                   // sc[] is rewritten by the next chunk
    }
    T *orow = out + (size_t)m * ldo + (size_t)h * hd;
    float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
    if (threadIdx.x < hd) orow[threadIdx.x] = from_f32<T>(acc0 * inv);
    if (threadIdx.x + ATT_THREADS < hd) orow[threadIdx.x + ATT_THREADS] = from_f32<T>(acc1 * inv);
}

extern "C" int fg_attention_generic(const void *q, int ldq, void *out, int ldo, int dtype,
                                    const int *positions, const int *row_seq, const int *block_table,
                                    int table_width, const void *k_pool, const void *v_pool,
                                    int M, int H, int KV, int hd, int page_size, float scale, int window,
                                    cudaStream_t stream) {
    if (M <= 0) return 0;
    if (hd > 2 * ATT_THREADS || hd <= 0 || H % KV != 0 || H > 65535) return FG_ERR_BAD_SIZE;
    dim3 grid(M, H);
    size_t smem = (size_t)(hd + CHUNK) * sizeof(float);
    if (dtype == FG_F32)
        attention_generic_kernel<float><<<grid, ATT_THREADS, smem, stream>>>((const float *)q, ldq, (float *)out, ldo,
            positions, row_seq, block_table, table_width, (const float *)k_pool, (const float *)v_pool,
            H, KV, hd, page_size, scale, window);
    else if (dtype == FG_BF16)
        attention_generic_kernel<bf16><<<grid, ATT_THREADS, smem, stream>>>((const bf16 *)q, ldq, (bf16 *)out, ldo,
            positions, row_seq, block_table, table_width, (const bf16 *)k_pool, (const bf16 *)v_pool,
            H, KV, hd, page_size, scale, window);
    else return FG_ERR_BAD_DTYPE;
    return FG_LAUNCH_CHECK();
}
