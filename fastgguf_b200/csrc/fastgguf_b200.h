/* The C interface of the kernel libraries (libfg_core.so, libfg_tc.so, libfg_attn.so).
 *
 * Every function launches on `stream` and returns 0, a cudaError_t, or one of the FG_ERR_* codes
 * below; none allocates device memory.  Pointers are device pointers unless said otherwise.
 * dtype codes: FG_F32 = 0, FG_BF16 = 1.  Page pools are [pages, kv_heads, page, head_dim]; block
 * tables are [sequences, table_width] int32 page ids.  The Python package calls these through ctypes
 * (fastgguf_b200/ops); the formulas each one follows are cited in its .cu file.
 */
#pragma once
#include <cuda_runtime.h>

#define FG_F32 0
#define FG_BF16 1
#define FG_ERR_BAD_DTYPE 10001
#define FG_ERR_BAD_SIZE 10002
#define FG_ERR_PIPELINE 10003      /* a bounded device-side wait ran out */
#define FG_ERR_TENSORMAP 10004

#ifdef __cplusplus
extern "C" {
#endif

/* ---- libfg_core: row-wise kernels, plain contraction, any-size attention, sampling */
int fg_embed_gather(const void *table, int table_dtype, const int *tokens, float *x, int M, int E, cudaStream_t stream);
int fg_embed_gather_norm(const void *table, int table_dtype, const int *tokens, float *x, const float *norm_w,
                         void *xw, float *ss, int M, int E, cudaStream_t stream);
int fg_rmsnorm(const float *x, const float *w, const int *rows, void *out, int out_dtype, int R, int E, float eps,
               cudaStream_t stream);
int fg_rope_append(void *qkv, int dtype, int ld, const int *positions, const int *row_seq, const int *block_table,
                   int table_width, void *k_pool, void *v_pool, const float *cos_t, const float *sin_t, int M, int H,
                   int KV, int hd, int page_size, int write_kv, cudaStream_t stream);
int fg_silu_mul(const void *gu, void *out, int dtype, int M, int F, cudaStream_t stream);
int fg_decode_advance(int *tokens, int *positions, const int *next_tokens, const int *active, int B, cudaStream_t stream);
int fg_gemm_generic(const void *A, int a_dtype, int lda, const void *W, int w_dtype, int ldw, void *C, int out_dtype,
                    int ldc, int accumulate, int M, int N, int K, cudaStream_t stream);
int fg_attention_generic(const void *q, int ldq, void *out, int ldo, int dtype, const int *positions,
                         const int *row_seq, const int *block_table, int table_width, const void *k_pool,
                         const void *v_pool, int M, int H, int KV, int hd, int page_size, float scale, int window,
                         cudaStream_t stream);
int fg_sample(float *logits, int B, int V, int ldl, float temp, int top_k, float top_p, float repeat_penalty,
              int repeat_last_n, const int *seq_slot, unsigned long long *rng, int *hist, int hist_cap,
              int *hist_count, const int *stop_ids, int n_stop, int *out_tokens,
              unsigned long long *scratch /* [B, 4096] or null */, cudaStream_t stream);
int fg_argmax(const float *logits, int B, int V, int ldl, int *out, cudaStream_t stream);

/* ---- libfg_tc: bf16 contraction on tcgen05 / TMA / tensor memory */
int fg_gemm_tc(const void *X, int ldx, const void *W, int ldw, void *out, int ldc, int epi, int M, int N, int K,
               int force_splits, const float *ss_in, int ss_tiles, int ss_size, float ss_eps, const float *norm_w,
               void *xw_out, float *ss_out, int *ss_tiles_out /* host */, cudaStream_t stream);
/* the same with device memory the call may use: with fg_gemm_tc_workspace_bytes(M, N, K, epi) of it (0: none needed) a
   prefill contraction of few output tiles is split along K over all SMs and summed, in order, by a second kernel */
int fg_gemm_tc_ws(const void *X, int ldx, const void *W, int ldw, void *out, int ldc, int epi, int M, int N, int K,
                  int force_splits, const float *ss_in, int ss_tiles, int ss_size, float ss_eps, const float *norm_w,
                  void *xw_out, float *ss_out, int *ss_tiles_out /* host */, void *workspace, long long workspace_bytes,
                  cudaStream_t stream);
long long fg_gemm_tc_workspace_bytes(int M, int N, int K, int epi);
int fg_gemm_tc_max_ss_tiles(int N);
int fg_gemm_tc_error(void);
/* tests only: shorten the bounded waits and make the decode kernel's pipeline stall, see gemm_tc.cu */
int fg_gemm_tc_test_hook(long long wait_limit_cycles, int skip_copy);

/* ---- libfg_attn: bf16 tensor-core attention over the paged cache (head sizes 64 and 128, pages of 64) */
int fg_attention_decode(const void *q, int ldq, void *out, int ldo, const int *positions, const int *block_table,
                        int table_width, const void *k_pool, const void *v_pool, int B, int H, int KV, int hd,
                        int page_size, float scale, int window, int n_splits, float *part_o, float *part_ml,
                        cudaStream_t stream);
int fg_attention_decode_fused(const void *qkv, int ldq, void *out, int ldo, const int *positions,
                              const int *block_table, int table_width, void *k_pool, void *v_pool, const float *cos_t,
                              const float *sin_t, int B, int H, int KV, int hd, int page_size, float scale, int window,
                              int n_splits, cudaStream_t stream);
int fg_attention_prefill(const void *q, int ldq, void *out, int ldo, const int *cu_rows, const int *seq_start,
                         const int *block_table, int table_width, const void *k_pool, const void *v_pool, int n_seq,
                         int max_new, int H, int KV, int hd, int page_size, float scale, int window, cudaStream_t stream);
int fg_attention_prefill_tc(const void *q, int ldq, void *out, int ldo, const int *cu_rows, const int *seq_start,
                            const int *block_table, int table_width, const void *k_pool, const void *v_pool,
                            int n_pages, int n_seq, int max_new, int H, int KV, int hd, int page_size, float scale,
                            int window, cudaStream_t stream);
int fg_attention_prefill_tc_error(void);
int fg_attention_prefill_tc_variant(int bits);   /* bit 0 / 1: two score tiles at head size 64 / 128; negative: by shape */
int fg_attention_prefill_tc_test_hook(long long wait_limit_cycles, int skip_copy);   /* tests only */
/* fg_attention_decode_noalloc: see fastgguf_noalloc.h */

#ifdef __cplusplus
}
#endif
