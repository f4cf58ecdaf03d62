// Plain tiled contraction C[m, n] = sum_k A[m, k] * W[n, k] on the FMA units, f32 accumulation.
//
// This is the true 32-bit path of every projection (no tensor cores, no TF32, no reduced
// precision anywhere) and the any-size fallback of the bf16 path.  Three kernels by row count: a
// weight-streaming one for up to 16 rows (a decode step), 64 x 64 tiles up to 64 rows, 128 x 128
// tiles beyond.  In each the order of additions for an output depends on K alone, so a row's result
// does not depend on how many other rows are in the batch; between the kernels the order differs
// (rounding only).
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

template <typename T> __device__ __forceinline__ float4 load4(const T *p);
template <> __device__ __forceinline__ float4 load4<float>(const float *p) { return *(const float4 *)p; }
template <> __device__ __forceinline__ float4 load4<bf16>(const bf16 *p) {
    uint2 u = *(const uint2 *)p;
    __nv_bfloat162 lo = *(__nv_bfloat162 *)&u.x, hi = *(__nv_bfloat162 *)&u.y;
    return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}

// ---------------------------------------------------------------------------- many rows: 128 x 128 tiles, 8 x 8 a thread
// The same sums in the same order (k increasing, one fused multiply-add at a time) with more reuse: a thread
// keeps an 8 x 8 block of outputs in registers and reads two 16-byte vectors of each operand per k from shared
// memory.  VEC: rows of both operands allow 16-byte (f32) / 8-byte (bf16) loads along k.
#define T2 128
#define T2K 16

template <typename T, bool VEC>
__device__ __forceinline__ float4 load4_guarded(const T *base, size_t ld, int row, int rows, int k, int K) {
    if (row >= rows) return make_float4(0.f, 0.f, 0.f, 0.f);
    const T *p = base + (size_t)row * ld + k;
    if (VEC && k + 3 < K) return load4<T>(p);
    float4 v;
    v.x = k < K ? to_f32<T>(p[0]) : 0.f;
    v.y = k + 1 < K ? to_f32<T>(p[1]) : 0.f;
    v.z = k + 2 < K ? to_f32<T>(p[2]) : 0.f;
    v.w = k + 3 < K ? to_f32<T>(p[3]) : 0.f;
    return v;
}

template <typename TA, typename TW, bool VEC>
__global__ void __launch_bounds__(256)
gemm_tile128_kernel(const TA *__restrict__ A, int lda, const TW *__restrict__ W, int ldw, void *__restrict__ C, int ldc,
                    int out_dtype, int accumulate, int M, int N, int K) {
    __shared__ __align__(16) float As[T2K][T2 + 4];
    __shared__ __align__(16) float Ws[T2K][T2 + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * T2, n0 = blockIdx.x * T2;
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += T2K) {
        // 128 rows x 16 k of each operand: 512 vectors of four, two per thread
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int idx = threadIdx.x + i * 256, row = idx >> 2, kq = (idx & 3) * 4;
            float4 a = load4_guarded<TA, VEC>(A, lda, m0 + row, M, k0 + kq, K);
            float4 w = load4_guarded<TW, VEC>(W, ldw, n0 + row, N, k0 + kq, K);
            As[kq][row] = a.x; As[kq + 1][row] = a.y; As[kq + 2][row] = a.z; As[kq + 3][row] = a.w;
            Ws[kq][row] = w.x; Ws[kq + 1][row] = w.y; Ws[kq + 2][row] = w.z; Ws[kq + 3][row] = w.w;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < T2K; kk++) {
            const float4 a0 = *(const float4 *)&As[kk][ty * 4], a1 = *(const float4 *)&As[kk][ty * 4 + 64];
            const float4 w0 = *(const float4 *)&Ws[kk][tx * 4], w1 = *(const float4 *)&Ws[kk][tx * 4 + 64];
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int gm = m0 + ty * 4 + (i & 3) + (i >> 2) * 64;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int gn = n0 + tx * 4 + (j & 3) + (j >> 2) * 64;
            if (gn >= N) continue;
            size_t idx = (size_t)gm * ldc + gn;
            float v = acc[i][j];
            if (accumulate) v += ((float *)C)[idx];
            store_as(C, out_dtype, idx, v);
        }
    }
}

// ---------------------------------------------------------------------------- few rows: stream the weights once
// With at most 16 rows (a decode step) the contraction is bound by reading W.  A warp owns a few weight
// rows and streams them with 16-byte loads, lanes side by side along k; the activations of the step sit in shared
// memory, a chunk of k at a time, and every value read from there is used for all of the warp's weight rows.  Each
// lane sums its own k positions in increasing order, then the lanes are added in a fixed tree: the order of
// additions for an output (m, n) depends on K alone, not on how many rows the step has or which they are.
#define GEMV_WARPS 8

// RPW weight rows a warp (4 where there are many rows to go round, 1 where the grid would otherwise be too small to
// fill the GPU), U vectors of each row in flight per lane before the arithmetic starts.
template <int MB, int RPW, int U, typename TA, typename TW>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
gemv_rows_kernel(const TA *__restrict__ A, int lda, const TW *__restrict__ W, int ldw, void *__restrict__ C, int ldc,
                 int out_dtype, int accumulate, int M, int N, int K) {
    constexpr int KC = MB <= 4 ? 2048 : MB == 8 ? 1024 : 512;       // 32 KB of activations at a time
    __shared__ __align__(16) float As[MB][KC];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = (blockIdx.x * GEMV_WARPS + warp) * RPW;
    float acc[RPW][MB];
#pragma unroll
    for (int r = 0; r < RPW; r++)
#pragma unroll
        for (int m = 0; m < MB; m++) acc[r][m] = 0.f;
    for (int kc0 = 0; kc0 < K; kc0 += KC) {
        const int kc = min(KC, K - kc0);
        __syncthreads();
        for (int e = threadIdx.x; e < MB * KC; e += GEMV_WARPS * 32) {
            int m = e / KC, k = e % KC;
            As[m][k] = (m < M && k < kc) ? to_f32<TA>(A[(size_t)m * lda + kc0 + k]) : 0.f;
        }
        __syncthreads();
        for (int kb = lane * 4; kb < kc; kb += 128 * U) {
            float4 w[U][RPW];
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int r = 0; r < RPW; r++) {
                    const int k = kb + 128 * u;
                    w[u][r] = (n0 + r < N && k < kc) ? load4<TW>(W + (size_t)(n0 + r) * ldw + kc0 + k) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int k = kb + 128 * u;
                if (k >= kc) break;                       // the products below would all be zero: same sums either way
#pragma unroll
                for (int m = 0; m < MB; m++) {
                    const float4 a = *(const float4 *)&As[m][k];
#pragma unroll
                    for (int r = 0; r < RPW; r++) {
                        float v = acc[r][m];
                        v = fmaf(a.x, w[u][r].x, v);
                        v = fmaf(a.y, w[u][r].y, v);
                        v = fmaf(a.z, w[u][r].z, v);
                        v = fmaf(a.w, w[u][r].w, v);
                        acc[r][m] = v;
                    }
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < RPW; r++)
#pragma unroll
        for (int m = 0; m < MB; m++) {
            float v = acc[r][m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && m < M && n0 + r < N) {
                size_t idx = (size_t)m * ldc + n0 + r;
                if (accumulate) v += ((float *)C)[idx];
                store_as(C, out_dtype, idx, v);
            }
        }
}

// The same for matrices of few rows (the projections of a layer): a block owns R weight rows and its warps split
// the reduction length among them, each reading its part of the activations straight from global memory; the warps'
// partial sums are added in warp order.  More, smaller blocks than above, and no stop-and-go between chunks.
template <int MB, int R, typename TA, typename TW>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
gemv_splitk_kernel(const TA *__restrict__ A, int lda, const TW *__restrict__ W, int ldw, void *__restrict__ C, int ldc,
                   int out_dtype, int accumulate, int M, int N, int K) {
    __shared__ float part[GEMV_WARPS][R][MB];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * R;
    const int slice = ((K + 127) / 128 + GEMV_WARPS - 1) / GEMV_WARPS * 128;     // a multiple of the warp's stride
    const int k_end = min(K, (warp + 1) * slice);
    float acc[R][MB];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int m = 0; m < MB; m++) acc[r][m] = 0.f;
#pragma unroll 2
    for (int k = warp * slice + lane * 4; k < k_end; k += 128) {
        float4 w[R], a[MB];
#pragma unroll
        for (int r = 0; r < R; r++)
            w[r] = n0 + r < N ? load4<TW>(W + (size_t)(n0 + r) * ldw + k) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int m = 0; m < MB; m++) a[m] = m < M ? load4<TA>(A + (size_t)m * lda + k) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int m = 0; m < MB; m++)
#pragma unroll
            for (int r = 0; r < R; r++) {
                float v = acc[r][m];
                v = fmaf(a[m].x, w[r].x, v);
                v = fmaf(a[m].y, w[r].y, v);
                v = fmaf(a[m].z, w[r].z, v);
                v = fmaf(a[m].w, w[r].w, v);
                acc[r][m] = v;
            }
    }
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int m = 0; m < MB; m++) {
            float v = acc[r][m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) part[warp][r][m] = v;
        }
    __syncthreads();
    for (int e = threadIdx.x; e < R * MB; e += GEMV_WARPS * 32) {
        const int r = e / MB, m = e % MB;
        if (m >= M || n0 + r >= N) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < GEMV_WARPS; w++) v += part[w][r][m];       // warp order
        size_t idx = (size_t)m * ldc + n0 + r;
        if (accumulate) v += ((float *)C)[idx];
        store_as(C, out_dtype, idx, v);
    }
}

template <typename TA, typename TW>
static void launch_gemv(const void *A, int lda, const void *W, int ldw, void *C, int ldc, int out_dtype, int accumulate, int M,
                        int N, int K, cudaStream_t stream) {
    const bool many = N >= 16384;         // enough weight rows for four a warp to fill the GPU
    const int a_bytes = sizeof(TA);
    // the block-split kernel reads the activations with vector loads too
    const bool split = !many && lda % 4 == 0 && ((uintptr_t)A % (4 * a_bytes)) == 0;
    const int rows_per_block = many ? GEMV_WARPS * 4 : split ? (M <= 8 ? 4 : 2) : GEMV_WARPS;
    dim3 grid((N + rows_per_block - 1) / rows_per_block);
#define GEMV_ARGS (const TA *)A, lda, (const TW *)W, ldw, C, ldc, out_dtype, accumulate, M, N, K
#define GEMV(MB) do { \
        if (many) gemv_rows_kernel<MB, 4, 2, TA, TW><<<grid, GEMV_WARPS * 32, 0, stream>>>(GEMV_ARGS); \
        else if (split) gemv_splitk_kernel<MB, (MB <= 8 ? 4 : 2), TA, TW><<<grid, GEMV_WARPS * 32, 0, stream>>>(GEMV_ARGS); \
        else gemv_rows_kernel<MB, 1, 8, TA, TW><<<grid, GEMV_WARPS * 32, 0, stream>>>(GEMV_ARGS); } while (0)
    if (M <= 1) GEMV(1);
    else if (M <= 2) GEMV(2);
    else if (M <= 4) GEMV(4);
    else if (M <= 8) GEMV(8);
    else GEMV(16);
#undef GEMV
#undef GEMV_ARGS
}

// a_dtype / w_dtype / out_dtype: FG_F32 or FG_BF16.  accumulate=1 needs out_dtype == FG_F32.
extern "C" int fg_gemm_generic(const void *A, int a_dtype, int lda, const void *W, int w_dtype, int ldw,
                               void *C, int out_dtype, int ldc, int accumulate, int M, int N, int K,
                               cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (accumulate && out_dtype != FG_F32) return FG_ERR_BAD_DTYPE;
    // few rows and weight rows that 16-byte (f32) / 8-byte (bf16) loads can walk: the weight-streaming kernel
    const int w_bytes = w_dtype == FG_F32 ? 4 : 2;
    if (M <= 16 && K % 4 == 0 && ldw % 4 == 0 && ((uintptr_t)W % (4 * w_bytes)) == 0) {
        if (a_dtype == FG_F32 && w_dtype == FG_F32) launch_gemv<float, float>(A, lda, W, ldw, C, ldc, out_dtype, accumulate, M, N, K, stream);
        else if (a_dtype == FG_BF16 && w_dtype == FG_BF16) launch_gemv<bf16, bf16>(A, lda, W, ldw, C, ldc, out_dtype, accumulate, M, N, K, stream);
        else if (a_dtype == FG_BF16 && w_dtype == FG_F32) launch_gemv<bf16, float>(A, lda, W, ldw, C, ldc, out_dtype, accumulate, M, N, K, stream);
        else if (a_dtype == FG_F32 && w_dtype == FG_BF16) launch_gemv<float, bf16>(A, lda, W, ldw, C, ldc, out_dtype, accumulate, M, N, K, stream);
        else return FG_ERR_BAD_DTYPE;
        return FG_LAUNCH_CHECK();
    }
    if (M > 64) {
        dim3 g2((N + T2 - 1) / T2, (M + T2 - 1) / T2);
        if (g2.y > 65535) return FG_ERR_BAD_SIZE;
        const int a_bytes = a_dtype == FG_F32 ? 4 : 2;
        const bool vec = K % 4 == 0 && lda % 4 == 0 && ldw % 4 == 0 && ((uintptr_t)A % (4 * a_bytes)) == 0 &&
                         ((uintptr_t)W % (4 * w_bytes)) == 0;
#define LAUNCH2(TA, TW) do { \
        if (vec) gemm_tile128_kernel<TA, TW, true><<<g2, 256, 0, stream>>>((const TA *)A, lda, (const TW *)W, ldw, C, ldc, out_dtype, accumulate, M, N, K); \
        else gemm_tile128_kernel<TA, TW, false><<<g2, 256, 0, stream>>>((const TA *)A, lda, (const TW *)W, ldw, C, ldc, out_dtype, accumulate, M, N, K); } while (0)
        if (a_dtype == FG_F32 && w_dtype == FG_F32) LAUNCH2(float, float);
        else if (a_dtype == FG_BF16 && w_dtype == FG_BF16) LAUNCH2(bf16, bf16);
        else if (a_dtype == FG_BF16 && w_dtype == FG_F32) LAUNCH2(bf16, float);
        else if (a_dtype == FG_F32 && w_dtype == FG_BF16) LAUNCH2(float, bf16);
        else return FG_ERR_BAD_DTYPE;
#undef LAUNCH2
        return FG_LAUNCH_CHECK();
    }
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
