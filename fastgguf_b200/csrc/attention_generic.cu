// Attention over the paged cache for any head size and any dtype: the true 32-bit path and
// the any-size fallback.  One block per (token row, query head).
//
// Reference formulas (fastgguf.c): scores s_p = scale * (q . K[p]) for p in [lo, pos]
// (:3246, :3317), the mask is the loop range (:4782, :5030-5035), softmax with max
// subtraction (:3147-3156), o = sum_p w_p V[p] (:3320-3323); query head h uses KV head
// h / (H / KV) (:4781).  A window of w keeps only the last w positions (:4754-4758).
//
// Keys are visited in chunks of CHUNK positions counted from lo, with a running maximum and
// sum in f32 (online softmax).  Within a chunk a thread scores whole keys; for the weighted sum of
// values the chunk's keys are dealt to the warps in equal runs, every lane owns output dimensions
// (lane, lane + 32, ...), and the warps' partial sums are added in warp order.  All of that depends
// only on the row's own position, so a row's result is the same whatever else is in the batch and
// however the tokens were cut into steps.
#include "common.cuh"

#define ATT_THREADS 256
#define ATT_WARPS (ATT_THREADS / 32)
#define MAX_DPL 8                     // output dimensions a lane owns at most: head sizes up to 256
#define CHUNK 1024

template <typename T, int DPL>          // DPL: output dimensions a lane owns (32 * DPL >= head size)
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

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float *part = sc + CHUNK;         // [ATT_WARPS][hd] partial value sums of a chunk
    float m_run = -INFINITY, l_run = 0.f;
    float acc[DPL];               // warp 0 keeps the running output: dims lane + 32 j
#pragma unroll
    for (int j = 0; j < DPL; j++) acc[j] = 0.f;
    for (int c0 = lo; c0 <= pos; c0 += CHUNK) {
        int n = min(CHUNK, pos - c0 + 1);
        float cmax = -INFINITY;
        for (int i = threadIdx.x; i < n; i += ATT_THREADS) {
            int p = c0 + i;
            const T *kr = k_pool + (((size_t)bt[p / page_size] * KV + kvh) * page_size + p % page_size) * hd;
            float s = 0.f;
            if (sizeof(T) == 4 && (hd & 3) == 0) {
                // 16-byte loads along the key's row (rows of a pool start 16-byte aligned when hd is a multiple of 4)
                for (int d = 0; d < hd; d += 4) {
                    const float4 kv4 = *(const float4 *)((const float *)kr + d);
                    s = fmaf(qs[d], kv4.x, s);
                    s = fmaf(qs[d + 1], kv4.y, s);
                    s = fmaf(qs[d + 2], kv4.z, s);
                    s = fmaf(qs[d + 3], kv4.w, s);
                }
            } else {
                for (int d = 0; d < hd; d++) s = fmaf(qs[d], to_f32<T>(kr[d]), s);
            }
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
        // values: warp w takes keys [w * run, (w + 1) * run) of the chunk, page by page, eight rows in flight
        const int run = (n + ATT_WARPS - 1) / ATT_WARPS;
        const int i_end = min(n, (warp + 1) * run);
        float pv[DPL];
#pragma unroll
        for (int j = 0; j < DPL; j++) pv[j] = 0.f;
        for (int i = warp * run; i < i_end;) {
            const int p = c0 + i, off = p % page_size;
            const int cnt = min(page_size - off, i_end - i);
            const T *vr = v_pool + (((size_t)bt[p / page_size] * KV + kvh) * page_size + off) * hd;
            for (int u0 = 0; u0 < cnt; u0 += 8) {
                float v[8][DPL];
#pragma unroll
                for (int u = 0; u < 8; u++)
#pragma unroll
                    for (int j = 0; j < DPL; j++) {
                        const int d = lane + 32 * j;
                        v[u][j] = (u0 + u < cnt && d < hd) ? to_f32<T>(vr[(size_t)(u0 + u) * hd + d]) : 0.f;
                    }
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    if (u0 + u >= cnt) break;
                    const float w = sc[i + u0 + u];
#pragma unroll
                    for (int j = 0; j < DPL; j++) pv[j] = fmaf(w, v[u][j], pv[j]);
                }
            }
            i += cnt;
        }
#pragma unroll
        for (int j = 0; j < DPL; j++)
            if (lane + 32 * j < hd) part[warp * hd + lane + 32 * j] = pv[j];
        __syncthreads();
        if (warp == 0) {
#pragma unroll
            for (int j = 0; j < DPL; j++) {
                const int d = lane + 32 * j;
                if (d >= hd) break;
                float t = 0.f;
                for (int w = 0; w < ATT_WARPS; w++) t += part[w * hd + d];      // warp order
                acc[j] = acc[j] * corr + t;
            }
        }
        m_run = m_new;
        __syncthreads();                   // sc[] and part[] are rewritten by the next chunk
    }
    if (warp == 0) {
        T *orow = out + (size_t)m * ldo + (size_t)h * hd;
        const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
#pragma unroll
        for (int j = 0; j < DPL; j++)
            if (lane + 32 * j < hd) orow[lane + 32 * j] = from_f32<T>(acc[j] * inv);
    }
}

extern "C" int fg_attention_generic(const void *q, int ldq, void *out, int ldo, int dtype,
                                    const int *positions, const int *row_seq, const int *block_table,
                                    int table_width, const void *k_pool, const void *v_pool,
                                    int M, int H, int KV, int hd, int page_size, float scale, int window,
                                    cudaStream_t stream) {
    if (M <= 0) return 0;
    if (hd > 32 * MAX_DPL || hd <= 0 || H % KV != 0 || H > 65535) return FG_ERR_BAD_SIZE;
    dim3 grid(M, H);
    size_t smem = (size_t)(hd + CHUNK + ATT_WARPS * hd) * sizeof(float);
#define ATT_LAUNCH(T, DPL) attention_generic_kernel<T, DPL><<<grid, ATT_THREADS, smem, stream>>>((const T *)q, ldq, (T *)out, ldo, \
        positions, row_seq, block_table, table_width, (const T *)k_pool, (const T *)v_pool, H, KV, hd, page_size, scale, window)
#define ATT_BY_SIZE(T) do { if (hd <= 64) ATT_LAUNCH(T, 2); else if (hd <= 128) ATT_LAUNCH(T, 4); else ATT_LAUNCH(T, 8); } while (0)
    if (dtype == FG_F32) ATT_BY_SIZE(float);
    else if (dtype == FG_BF16) ATT_BY_SIZE(bf16);
    else return FG_ERR_BAD_DTYPE;
#undef ATT_BY_SIZE
#undef ATT_LAUNCH
    return FG_LAUNCH_CHECK();
}
