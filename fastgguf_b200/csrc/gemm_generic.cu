// Plain tiled contraction C[m, n] = sum_k A[m, k] * W[n, k] on the FMA units, f32 accumulation.
//
// This is the true 32-bit path of every projection (no tensor cores, no TF32, no reduced
// precision anywhere) and the any-size fallback of the bf16 path.  Each output element is
// summed over k in increasing order by one thread, so a row's result does not depend on how
// many other rows are in the batch.
//
// Reference role: matvec / matmul with F32, BF16 weights (fastgguf.c:2575-2622, 3004-3093,
// dot_f32v :1618-1643); W is [out, in] row-major exactly as there (tensor_rows :4166).
#include "common.cuh"

#define TM 64
#define TN 64
#define TK 16

template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
gemm_generic_kernel(const TA *__restrict__ A, int lda, const TW *__restrict__ W, int ldw,
                    void *__restrict__ C, int ldc, int out_dtype, int accumulate, int M, int N, int K) {
    __shared__ float As[TK][TM + 1];
    __shared__ float Ws[TK][TN + 1];
    int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // tx: n direction, ty: m direction
    int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += TK) {
        // 64 rows x 16 k = 1024 elements per tile, 4 per thread; consecutive threads read along k
        for (int e = threadIdx.x; e < TM * TK; e += 256) {
            int r = e >> 4, kk = e & 15;
            int gm = m0 + r, gk = k0 + kk;
            As[kk][r] = (gm < M && gk < K) ? to_f32<TA>(A[(size_t)gm * lda + gk]) : 0.f;
            int gn = n0 + r;
            Ws[kk][r] = (gn < N && gk < K) ? to_f32<TW>(W[(size_t)gn * ldw + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; kk++) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[kk][ty + 16 * i];
#pragma unroll
            for (int j = 0; j < 4; j++) w[j] = Ws[kk][tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int gm = m0 + ty + 16 * i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int gn = n0 + tx + 16 * j;
            if (gn >= N) continue;
            size_t idx = (size_t)gm * ldc + gn;
            float v = acc[i][j];
            if (accumulate) v += ((float *)C)[idx];   // residual sum in f32, in place
            store_as(C, out_dtype, idx, v);
        }
    }
}

// a_dtype / w_dtype / out_dtype: FG_F32 or FG_BF16.  accumulate=1 needs out_dtype == FG_F32.
extern "C" int fg_gemm_generic(const void *A, int a_dtype, int lda, const void *W, int w_dtype, int ldw,
                               void *C, int out_dtype, int ldc, int accumulate, int M, int N, int K,
                               cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (accumulate && out_dtype != FG_F32) return FG_ERR_BAD_DTYPE;
    dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
    if (grid.y > 65535) return FG_ERR_BAD_SIZE;
#define LAUNCH(TA, TW) gemm_generic_kernel<TA, TW><<<grid, 256, 0, stream>>>( \
        (const TA *)A, lda, (const TW *)W, ldw, C, ldc, out_dtype, accumulate, M, N, K)
    if (a_dtype == FG_F32 && w_dtype == FG_F32) LAUNCH(float, float);
    else if (a_dtype == FG_BF16 && w_dtype == FG_BF16) LAUNCH(bf16, bf16);
    else if (a_dtype == FG_BF16 && w_dtype == FG_F32) LAUNCH(bf16, float);
    else if (a_dtype == FG_F32 && w_dtype == FG_BF16) LAUNCH(float, bf16);
    else return FG_ERR_BAD_DTYPE;
#undef LAUNCH
    return FG_LAUNCH_CHECK();
}
