// bfloat16 contraction on the 5th-generation tensor cores (tcgen05), operands staged by TMA,
// accumulators in tensor memory.  C[m, n] = sum_k X[m, k] * W[n, k], f32 accumulation.
//
// Role in the reference: matvec / matvec_multi / matmul (fastgguf.c:2575-2622, :2552-2573,
// :3004-3093) - every projection of the decoder, for one token or a batch of prompt tokens.
//
// Shape of the kernel ("swap-AB"): the WEIGHT rows are the 128-row M operand of the MMA and the
// token rows are its N operand (16..256), so the same kernel streams weights for a decode step of
// 1..64 tokens and tiles a prefill of thousands.  One CTA computes a 128 (features) x BN (tokens)
// tile; blockIdx.z splits K when there are too few tiles to fill the GPU (decode), the last CTA
// of a tile then sums the partial tiles in split order (deterministic) and runs the epilogue.
//
//   warp 0      TMA producer   (one lane): K-blocks of 64 into a ring of smem stages, 128B swizzle
//   warp 1      MMA issuer     (one lane): tcgen05.mma 128 x BN x 16, commit frees the stage
//   warps 2-5   epilogue: tcgen05.ld of the f32 tile, then one of
//               store bf16 | store f32 | add into f32 (residual) | silu(gate) * up -> bf16
//
// The silu epilogue runs two accumulators: the gate rows and the up rows of the same features
// are two A tiles against one B tile, so gate and up of a feature meet in one thread.
//
// Every wait on an mbarrier is bounded; when it runs out the kernel raises an error flag, waits
// (bounded) for its own copies in flight, frees its tensor memory and returns.
#include <cuda.h>
#include "common.cuh"

#define FG_ERR_PIPELINE 10003
#define FG_ERR_TENSORMAP 10004

#define BM 128          // weight rows per tile (MMA M)
#define BK 64           // K elements per stage: 64 bf16 = one 128-byte swizzle row
#define UMMA_K 16
#define GEMM_THREADS 192
#define WAIT_LIMIT_CYCLES 2000000000ll

enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_ADD_F32 = 2, EPI_SILU_MUL = 3 };

__device__ int g_gemm_error = 0;      // 0, or (code << 8 | role) of the first wait that ran out

// ---------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// bounded wait: false when the limit ran out
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    long long t0 = clock64();
    for (;;) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) return false;
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows at 128 B, 8-row groups at 1024 B
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);          // start address
    d |= (uint64_t)1 << 16;                           // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;                 // stride byte offset: 8 rows * 128 B
    d |= (uint64_t)1 << 46;                           // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                           // swizzle mode: 128 B
    return d;
}
// instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M x N
__device__ __forceinline__ uint32_t make_idesc(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void raise_error(int role) { atomicCAS(&g_gemm_error, 0, (FG_ERR_PIPELINE << 8) | role); }

struct GemmArgs {
    void *out;            // [M, ldc] bf16 or f32 by epilogue
    float *ws;            // split-K partial tiles [splits, M, N] f32
    int *counters;        // split-K arrival counters, one per tile, zero between launches
    int M, N, K;          // tokens, output features, reduction
    int ldc;
    int up_row_offset;    // EPI_SILU_MUL: first row of the up projection inside W (= F)
    int kb_per_split;     // K-blocks of 64 per split
};

template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, GemmArgs a) {
    constexpr bool DUAL = EPI == EPI_SILU_MUL;
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
    constexpr int STAGE_BYTES = (DUAL ? 2 : 1) * A_BYTES + B_BYTES;
    constexpr int TMEM_NEED = (DUAL ? 2 : 1) * BN;
    constexpr int TMEM_COLS = TMEM_NEED <= 32 ? 32 : TMEM_NEED <= 64 ? 64 : TMEM_NEED <= 128 ? 128 : TMEM_NEED <= 256 ? 256 : 512;

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);   // swizzle atoms need 1 KB alignment
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 1];
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BM, m0 = blockIdx.y * BN;
    const int total_kb = (a.K + BK - 1) / BK;
    const int kb0 = blockIdx.z * a.kb_per_split;
    const int nkb = min(a.kb_per_split, total_kb - kb0);
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]), tfull = smem_u32(&bars[2 * STAGES]);
    const uint32_t smem0 = smem_u32(smem);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(tfull, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            bool ok = true;
            int issued = 0;
            for (int kb = 0; kb < nkb && ok; kb++) {
                int s = kb % STAGES;
                uint32_t ph = (kb / STAGES) & 1;
                ok = mbar_wait(empty0 + 8 * s, ph ^ 1);
                if (!ok) { raise_error(1); break; }
                uint32_t dst = smem0 + s * STAGE_BYTES, bar = full0 + 8 * s;
                mbar_expect_tx(bar, STAGE_BYTES);
                int kx = (kb0 + kb) * BK;
                tma_load_2d(dst, &tmW, kx, n0, bar);
                if (DUAL) tma_load_2d(dst + A_BYTES, &tmW, kx, a.up_row_offset + n0, bar);
                tma_load_2d(dst + (DUAL ? 2 : 1) * A_BYTES, &tmX, kx, m0, bar);
                issued = kb + 1;
            }
            // copies still in flight must land before the CTA may exit
            for (int kb = max(0, issued - STAGES); kb < issued; kb++)
                mbar_wait(full0 + 8 * (kb % STAGES), (kb / STAGES) & 1);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = make_idesc(BM, BN);
            for (int kb = 0; kb < nkb; kb++) {
                int s = kb % STAGES;
                if (!mbar_wait(full0 + 8 * s, (kb / STAGES) & 1)) { raise_error(2); break; }
                tc_fence_after();
                uint32_t sa = smem0 + s * STAGE_BYTES;
                uint64_t adesc = make_smem_desc(sa), bdesc = make_smem_desc(sa + (DUAL ? 2 : 1) * A_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; k++) {
                    uint32_t acc = (kb | k) != 0;
                    uint64_t koff = (uint64_t)((k * UMMA_K * 2) >> 4);     // advance inside the swizzle row
                    tc_mma_bf16(tmem_base, adesc + koff, bdesc + koff, idesc, acc);
                    if (DUAL) tc_mma_bf16(tmem_base + BN, make_smem_desc(sa + A_BYTES) + koff, bdesc + koff, idesc, acc);
                }
                tc_commit(empty0 + 8 * s);        // arrives when these MMAs have read the stage
            }
            tc_commit(tfull);                     // arrives when every MMA above is complete
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int lg = warp & 3;                  // the TMEM lane group this warp may read
        const int n = n0 + lg * 32 + lane;        // output feature of this thread
        const bool n_ok = n < a.N;
        bool ok = nkb > 0 ? mbar_wait(tfull, 0) : true;
        if (!ok) raise_error(3);
        tc_fence_after();
        const uint32_t trow = tmem_base + ((uint32_t)(lg * 32) << 16);
        const int splits = gridDim.z;
        bool last = true;
        if (splits > 1) {
            // partial tile -> workspace; the CTA that arrives last sums all splits in order
            if (ok) {
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    uint32_t r[16];
                    tc_ld16(trow + c0, r);
                    tc_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        int m = m0 + c0 + j;
                        if (n_ok && m < a.M)
                            a.ws[((size_t)blockIdx.z * a.M + m) * a.N + n] = nkb > 0 ? __uint_as_float(r[j]) : 0.f;
                    }
                }
            }
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (threadIdx.x == 64) {
                int tile = blockIdx.y * gridDim.x + blockIdx.x;
                int old = atomicAdd(&a.counters[tile], 1);
                s_flag = old == splits - 1;
                if (old == splits - 1) a.counters[tile] = 0;      // ready for the next launch
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            last = s_flag != 0;
            if (last) __threadfence();
        }
        if (last && ok) {
            for (int c0 = 0; c0 < BN; c0 += 16) {
                float v[16], u[16];
                if (splits > 1) {
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        int m = m0 + c0 + j;
                        float s = 0.f;
                        if (n_ok && m < a.M)
                            for (int z = 0; z < splits; z++) s += __ldcg(&a.ws[((size_t)z * a.M + m) * a.N + n]);
                        v[j] = s;
                    }
                } else {
                    uint32_t r[16];
                    tc_ld16(trow + c0, r);
                    if (DUAL) {
                        uint32_t r2[16];
                        tc_ld16(trow + BN + c0, r2);
                        tc_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; j++) u[j] = __uint_as_float(r2[j]);
                    } else tc_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; j++) v[j] = nkb > 0 ? __uint_as_float(r[j]) : 0.f;
                }
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    int m = m0 + c0 + j;
                    if (!n_ok || m >= a.M) continue;
                    size_t idx = (size_t)m * a.ldc + n;
                    if (EPI == EPI_BF16) ((bf16 *)a.out)[idx] = __float2bfloat16_rn(v[j]);
                    else if (EPI == EPI_F32) ((float *)a.out)[idx] = v[j];
                    else if (EPI == EPI_ADD_F32) ((float *)a.out)[idx] += v[j];
                    else {
                        float g = v[j];
                        ((bf16 *)a.out)[idx] = __float2bfloat16_rn(g / (1.0f + expf(-g)) * u[j]);
                    }
                }
            }
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// a [rows, K] bf16 matrix with row stride ld (elements), boxes of box_rows x 64, 128-byte swizzle
static int make_map(CUtensorMap *map, const void *base, int rows, int K, int ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return FG_ERR_TENSORMAP;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void *)base, dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : FG_ERR_TENSORMAP;
}

template <int BN, int STAGES, int EPI>
static int launch(const CUtensorMap &tmW, const CUtensorMap &tmX, const GemmArgs &a, int splits, cudaStream_t stream) {
    constexpr int stage = ((EPI == EPI_SILU_MUL ? 2 : 1) * BM + BN) * BK * 2;
    constexpr int smem = STAGES * stage + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid((a.N + BM - 1) / BM, (a.M + BN - 1) / BN, splits);
    gemm_tc_kernel<BN, STAGES, EPI><<<grid, GEMM_THREADS, smem, stream>>>(tmW, tmX, a);
    return FG_LAUNCH_CHECK();
}

template <int EPI>
static int dispatch_bn(int bn, const CUtensorMap &tmW, const CUtensorMap &tmX, const GemmArgs &a, int splits, cudaStream_t st) {
    constexpr bool D = EPI == EPI_SILU_MUL;
    switch (bn) {
    case 16: return launch<16, D ? 5 : 8, EPI>(tmW, tmX, a, splits, st);
    case 32: return launch<32, D ? 5 : 8, EPI>(tmW, tmX, a, splits, st);
    case 64: return launch<64, D ? 5 : 8, EPI>(tmW, tmX, a, splits, st);
    case 128: return launch<128, D ? 4 : 6, EPI>(tmW, tmX, a, splits, st);
    case 256: return launch<256, D ? 3 : 4, EPI>(tmW, tmX, a, splits, st);
    }
    return FG_ERR_BAD_SIZE;
}

// Largest workspace (floats) and counter count any call may need: callers allocate once.
extern "C" long long fg_gemm_tc_workspace_floats(void) { return 8ll * 64 * 8192; }
extern "C" int fg_gemm_tc_counter_count(void) { return 4096; }

// X: [M, K] bf16 (row stride ldx), W: [N, K] bf16 (row stride ldw); epi as the enum above.
// EPI_SILU_MUL: W holds gate rows [0, N) and up rows [up_row_offset, up_row_offset + N); out is [M, N] bf16.
// Returns FG_ERR_BAD_SIZE for shapes TMA cannot describe (K % 8, unaligned bases): the caller
// then uses the plain kernel.
extern "C" int fg_gemm_tc(const void *X, int ldx, const void *W, int ldw, void *out, int ldc, int epi,
                          int M, int N, int K, int w_rows_total, int up_row_offset, float *ws, int *counters,
                          int force_splits, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return FG_ERR_BAD_SIZE;
    int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    int total_kb = (K + BK - 1) / BK;
    int tiles = ((N + BM - 1) / BM) * ((M + bn - 1) / bn);
    int splits = 1;
    if (epi != EPI_SILU_MUL && ws && counters && tiles <= 74 && tiles <= fg_gemm_tc_counter_count()) {
        splits = (148 + tiles - 1) / tiles;
        if (splits > 8) splits = 8;
        if (splits > total_kb / 2) splits = total_kb / 2 > 0 ? total_kb / 2 : 1;
        if ((long long)splits * M * N > fg_gemm_tc_workspace_floats()) splits = 1;
    }
    if (force_splits > 0 && epi != EPI_SILU_MUL && ws && counters && force_splits <= total_kb &&
        (long long)force_splits * M * N <= fg_gemm_tc_workspace_floats() && tiles <= fg_gemm_tc_counter_count())
        splits = force_splits;
    int kb_per_split = (total_kb + splits - 1) / splits;
    splits = (total_kb + kb_per_split - 1) / kb_per_split;      // no empty split
    CUtensorMap tmW, tmX;
    int e = make_map(&tmW, W, w_rows_total, K, ldw, BM);
    if (e) return e;
    e = make_map(&tmX, X, M, K, ldx, bn);
    if (e) return e;
    GemmArgs a{out, ws, counters, M, N, K, ldc, up_row_offset, kb_per_split};
    switch (epi) {
    case EPI_BF16: return dispatch_bn<EPI_BF16>(bn, tmW, tmX, a, splits, stream);
    case EPI_F32: return dispatch_bn<EPI_F32>(bn, tmW, tmX, a, splits, stream);
    case EPI_ADD_F32: return dispatch_bn<EPI_ADD_F32>(bn, tmW, tmX, a, splits, stream);
    case EPI_SILU_MUL: return dispatch_bn<EPI_SILU_MUL>(bn, tmW, tmX, a, splits, stream);
    }
    return FG_ERR_BAD_DTYPE;
}

// The error flag of the pipelines: 0, or FG_ERR_PIPELINE << 8 | role.  Reading clears it.
extern "C" int fg_gemm_tc_error(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
    return v;
}
