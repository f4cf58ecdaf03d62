// bfloat16 contraction on the 5th-generation tensor cores (tcgen05), operands staged by TMA,
// accumulators in tensor memory.  C[m, n] = sum_k X[m, k] * W[n, k], f32 accumulation.
//
// Role in the reference: matvec / matvec_multi / matmul (fastgguf.c:2575-2622, :2552-2573,
// :3004-3093) - every projection of the decoder, for one token or a batch of prompt tokens.
//
// Two kernels share the building blocks of this file:
//   gemm_tc_decode_kernel (up to 64 tokens): the 128 rows of the MMA's M side are weight rows, its N side the
//     token rows (BN = 16/32/64).  The kernel streams the weights once; when there are too few tiles to fill
//     the GPU, a thread-block cluster of 2/4/8 CTAs splits K: every CTA pushes the columns of its partial
//     tile into the shared memory of the CTA that owns them (st.shared::cluster), one cluster barrier makes
//     the pushes visible, and the owner sums them in rank order (deterministic) from its own shared memory -
//     no scratch in global memory, no remote loads.
//   gemm_tc_prefill_kernel: 128 token rows x BN = 128/192/256 weight rows per tile, persistent CTAs, two
//     accumulators in tensor memory.
//   gemm_tc_prefill_pair_kernel: the same for 256 token rows x 256 weight rows on a pair of CTAs
//     (tcgen05.mma.cta_group::2): each SM loads half of the weight rows of a tile.
//
//   warp 0      TMA producer (the warp walks the ring, one elected lane issues): K-blocks of 64 into a ring
//               of smem stages, 128B swizzle.
//               The weight tiles of the first stages are fetched BEFORE the wait on the preceding
//               kernel (weights are never written), so weight traffic overlaps that kernel's tail.
//   warp 1      MMA issuer (the same way): tcgen05.mma 128 x BN x 16; its commit frees the stage.
//   warps 2-5   epilogue: tcgen05.ld of the f32 tile, then one of
//               store bf16 | store f32 | add into f32 (residual) | silu(gate) * up -> bf16
//               (the decode kernel has eight epilogue warps, 2-9: two per lane group of tensor memory)
//
// The silu epilogue expects the gate and up matrices interleaved in blocks of 64 rows
// (g0..g63, u0..u63, g64..g127, ...): a 128-row weight tile then holds gate and up of the same
// 64 features.
//
// Every wait on an mbarrier is bounded; when it runs out the kernel raises an error flag, waits
// (bounded) for its own copies in flight, frees its tensor memory and returns.
#include <cuda.h>
#include "common.cuh"

#define FG_ERR_PIPELINE 10003
#define FG_ERR_TENSORMAP 10004

#define BM 128          // P rows per tile (MMA M)
#define BK 64           // K elements per stage: 64 bf16 = one 128-byte swizzle row
#define UMMA_K 16
#define GEMM_THREADS 192
// decode kernel: producer, issuer and four epilogue warps at 16 token columns, eight at 32 and 64
#define DEC_EPI_WARPS(BN) ((BN) >= 32 ? 8 : 4)
#define DEC_THREADS(BN) (64 + 32 * DEC_EPI_WARPS(BN))
#define WAIT_LIMIT_CYCLES 2000000000ll
#define WAIT_SHORT_CYCLES 1000000ll

enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_ADD_F32 = 2, EPI_SILU_MUL = 3 };

__device__ int g_gemm_error = 0;      // 0, or (code << 8 | role) of the first wait that ran out
// How long a wait may last, in SM cycles (about a second).  A variable, so that a test can make a wait run out within a
// millisecond (fg_gemm_tc_test_hook); it is read only by waits that have already lasted WAIT_SHORT_CYCLES.
__device__ long long g_gemm_wait_limit = WAIT_LIMIT_CYCLES;

// ---------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// bounded wait: false when the limit ran out
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// The clock is read only once the first try has failed: the waiting warp is often the one that issues the MMAs
// or the copies, where every instruction of the loop is on the critical path.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try(bar, parity)) return true;
        const long long waited = clock64() - t0;
        if (waited > WAIT_SHORT_CYCLES) {
            // once a wait has run out somewhere, every later wait gives up after a short time: a broken pipeline
            // costs milliseconds for the kernels that follow, not a second per wait
            if (*(volatile int *)&g_gemm_error != 0) return false;
            if (waited > *(volatile long long *)&g_gemm_wait_limit) return false;
        }
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// the same with an L2 eviction policy: weights of a decode step are read once, and marking them evict-first keeps
// them from pushing everything else (activations, the cache, norm weights, the kernels' own code) out of L2
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar, uint64_t policy) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar), "l"(policy) : "memory");
}
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
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
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int j = 0; j < 16; j++) v[j] = __uint_as_float(r[j]);
}

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

// all threads of all CTAs of the cluster; release/acquire so that shared-memory writes are seen remotely
__device__ __forceinline__ void cluster_sync() {
    __syncwarp();                                 // lanes that skipped a single-lane role rejoin first
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// write a float to the same shared-memory offset in the CTA of rank `rank` of this cluster
__device__ __forceinline__ void st_dsmem_f32(uint32_t local_addr, int rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
// Write a float to the same shared-memory offset in the CTA of rank `rank`, and count its four bytes on that CTA's
// mbarrier `local_bar` (same offset there): the receiver waits for BYTES on a barrier of its own instead of for the
// whole cluster at a cluster barrier, and a sender has nothing to wait for.
// Two or four consecutive floats into the shared memory of CTA `rank` of the cluster, counted as bytes on that CTA's
// mbarrier: one packet on the SM-to-SM network instead of two or four (the network moves packets, not bytes: at 64
// token columns the exchange of single floats took 7.8 us of a 14 us launch).
__device__ __forceinline__ void st_async_f32x4(uint32_t local_addr, uint32_t local_bar, int rank, const float *v) {
    uint32_t remote, remote_bar;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_bar) : "r"(local_bar), "r"(rank));
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
                 ::"r"(remote), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
                   "r"(__float_as_uint(v[3])), "r"(remote_bar) : "memory");
}
__device__ __forceinline__ void st_async_f32x2(uint32_t local_addr, uint32_t local_bar, int rank, const float *v) {
    uint32_t remote, remote_bar;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_bar) : "r"(local_bar), "r"(rank));
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.b32 [%0], {%1, %2}, [%3];"
                 ::"r"(remote), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(remote_bar) : "memory");
}
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// silu(g) * u in f32 with the fast exponential and division (2 ulp each): the result is rounded to bfloat16
// (8 bits of mantissa) right after, and the precise forms made the epilogue of a 64-token tile several us long
__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

static int g_test_skip_copy = 0;      // host side of fg_gemm_tc_test_hook

struct GemmArgs {
    void *out;            // [M, ldc] bf16 or f32 by epilogue
    int M, N, K;          // tokens, weight rows (2F for the silu epilogue), reduction
    int ldc;
    int kb_per_split;     // K-blocks of 64 per split
    int vec_ok;           // rows of `out` allow 16-byte accesses
    // input side of a deferred RMSNorm: X holds x * w, and 1/rms(x) of each token row is applied to
    // the accumulators here; ss_in[t * M + m] are partial sums of squares of row m (null: none)
    const float *ss_in;
    int ss_tiles, ss_size;
    float ss_eps;
    // output side (residual-add epilogue only): besides out = out + acc, write the next norm's
    // input xw = bf16(out * norm_w) and the partial sums of squares of out, one per tile of features
    const float *norm_w;  // [N], or null
    bf16 *xw_out;         // [M, N]
    float *ss_out;        // [tiles, M]
    int epi, stages;      // decode kernel: epilogue and ring depth are run-time values
    int test_skip_copy;   // tests only: the decode kernel's producer omits the activation copy of its first stage
    int splits;           // prefill kernel: > 1 = partial products of `kb_per_split` K-blocks each into out[split][M][ldc]
};

__device__ __forceinline__ float inv_rms(const GemmArgs &a, int m) {
    float s = 0.f;
    for (int t = 0; t < a.ss_tiles; t++) s += a.ss_in[(size_t)t * a.M + m];     // tile order: deterministic
    return 1.0f / sqrtf(s / (float)a.ss_size + a.ss_eps);
}

// Epilogue of a token-major tile: thread = token row p0 + prow, columns = weight rows q0 .. q0 + BN.
// `qt` is the index of the tile along the features (row of ss_out it writes).
template <int BN, int EPI>
__device__ __forceinline__ void epilogue_token_major(const GemmArgs &a, uint32_t trow, int p0, int q0, int qt, int prow,
                                                     size_t out_row0 = 0) {
    // thread = token row, columns = weight rows (features): runs of 16 consecutive outputs
    const int m = p0 + prow;
    const bool m_ok = m < a.M;
    const float iv = (a.ss_in && m_ok) ? inv_rms(a, m) : 1.0f;
    if (EPI == EPI_SILU_MUL) {
        const int F = a.N >> 1;
        for (int blk = 0; blk < BN / 128; blk++) {
            for (int c0 = 0; c0 < 64; c0 += 16) {
                float g[16], u[16];
                tc_ld16(trow + blk * 128 + c0, g);
                tc_ld16(trow + blk * 128 + 64 + c0, u);
                const int f0 = ((q0 + blk * 128) >> 1) + c0;
                if (!m_ok || f0 >= F) continue;
                bf16 *dst = (bf16 *)a.out + (size_t)m * a.ldc + f0;
                if (a.vec_ok && f0 + 16 <= F) {
                    uint32_t w[8];
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        __nv_bfloat162 t = __floats2bfloat162_rn(silu_mul(g[2 * j] * iv, u[2 * j] * iv),
                                                                 silu_mul(g[2 * j + 1] * iv, u[2 * j + 1] * iv));
                        w[j] = *(uint32_t *)&t;
                    }
                    ((uint4 *)dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
                    ((uint4 *)dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j++)
                        if (f0 + j < F) dst[j] = __float2bfloat16_rn(silu_mul(g[j] * iv, u[j] * iv));
                }
            }
        }
    } else {
        float sq = 0.f;
        for (int c0 = 0; c0 < BN; c0 += 16) {
            float v[16];
            tc_ld16(trow + c0, v);
            const int n0 = q0 + c0;
            if (!m_ok || n0 >= a.N) continue;
#pragma unroll
            for (int j = 0; j < 16; j++) v[j] *= iv;
            const size_t idx = (out_row0 + (size_t)m) * a.ldc + n0;       // (out_row0: the split's block of a partial product)
            const bool full = a.vec_ok && n0 + 16 <= a.N;
            if (EPI == EPI_BF16) {
                bf16 *dst = (bf16 *)a.out + idx;
                if (full) {
                    uint32_t w[8];
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        __nv_bfloat162 t = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                        w[j] = *(uint32_t *)&t;
                    }
                    ((uint4 *)dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
                    ((uint4 *)dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j++) if (n0 + j < a.N) dst[j] = __float2bfloat16_rn(v[j]);
                }
            } else {
                float *dst = (float *)a.out + idx;
                if (full) {
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        if (EPI == EPI_ADD_F32) {
                            float4 o = ((float4 *)dst)[j];
                            v[4 * j] += o.x; v[4 * j + 1] += o.y; v[4 * j + 2] += o.z; v[4 * j + 3] += o.w;
                        }
                        ((float4 *)dst)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j++)
                        if (n0 + j < a.N) { if (EPI == EPI_ADD_F32) v[j] += dst[j]; dst[j] = v[j]; }
                }
                if (EPI == EPI_ADD_F32 && a.norm_w) {
                    // the next norm's input, and this thread's share of its row's sum of squares
                    bf16 *xw = a.xw_out + (size_t)m * a.N + n0;
                    if (full && (a.N & 7) == 0) {
                        uint32_t w[8];
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            float4 g = ((const float4 *)(a.norm_w + n0))[j];
                            __nv_bfloat162 t0 = __floats2bfloat162_rn(v[4 * j] * g.x, v[4 * j + 1] * g.y);
                            __nv_bfloat162 t1 = __floats2bfloat162_rn(v[4 * j + 2] * g.z, v[4 * j + 3] * g.w);
                            w[2 * j] = *(uint32_t *)&t0; w[2 * j + 1] = *(uint32_t *)&t1;
                        }
                        ((uint4 *)xw)[0] = make_uint4(w[0], w[1], w[2], w[3]);
                        ((uint4 *)xw)[1] = make_uint4(w[4], w[5], w[6], w[7]);
#pragma unroll
                        for (int j = 0; j < 16; j++) sq += v[j] * v[j];
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; j++)
                            if (n0 + j < a.N) { xw[j] = __float2bfloat16_rn(v[j] * a.norm_w[n0 + j]); sq += v[j] * v[j]; }
                    }
                }
            }
        }
        if (EPI == EPI_ADD_F32 && a.norm_w && m_ok) a.ss_out[(size_t)qt * a.M + m] = sq;
    }
}

#define EPI_STAGE_BYTES 6144      // per epilogue warp: a 32 x 32 f32 tile and a 32 x 32 bf16 tile

__device__ __forceinline__ void tc_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]);
}

// Residual-add epilogue of a token-major tile for whole, aligned rows (N % 32 == 0, 16-byte aligned rows).
// In tensor memory a thread owns one token row, and if it also did the global accesses every warp instruction
// would touch 32 different lines, 16 bytes each - the load/store unit then bounds the epilogue (18 us for a
// 128 x 256 tile, against 11 us of MMAs).  Here a warp passes each 32-column chunk through a tile of its own in
// shared memory, so that the global loads and stores are four whole 128-byte lines per instruction:
//   residual: global -> (coalesced) -> tile;   thread = row: tile + accumulator -> new residual, x * w, sum of squares
//   -> tile;   tile -> (coalesced) -> global.   16-byte chunks are swizzled by row, all accesses are conflict-free.
template <int BN>
__device__ __forceinline__ void epilogue_add_coalesced(const GemmArgs &a, uint32_t trow, int p0, int q0, int ss_index, int lg,
                                                       int lane, uint8_t *stage, int c_begin = 0, int c_end = BN / 32) {
    float *T = (float *)stage;                    // [32][32] f32
    uint8_t *X = stage + 4096;                    // [32][32] bf16
    const int m_base = p0 + lg * 32, m_own = m_base + lane;
    const float iv = (a.ss_in && m_own < a.M) ? inv_rms(a, m_own) : 1.0f;
    float sq = 0.f;
    // The residual values of a chunk are requested one chunk ahead, the norm weights of a chunk at its start (behind
    // the stores into the tile the compiler would not move them, and each would wait for L2 on its own).
    float4 rl[8], g[8], rl_next[8];
    auto request = [&](int c, float4 (&r)[8]) {
        const int n0 = q0 + c * 32;
#pragma unroll
        for (int pass = 0; pass < 8; pass++) {
            const int row = pass * 4 + (lane >> 3), ch = lane & 7, m = m_base + row;
            r[pass] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (m < a.M && n0 < a.N) r[pass] = __ldcg((const float4 *)((const float *)a.out + (size_t)m * a.ldc + n0) + ch);
        }
    };
    request(c_begin, rl);
#pragma unroll 1
    for (int c = c_begin; c < c_end; c++) {                // the chunks of 32 columns this warp takes
        const int n0 = q0 + c * 32;
        if (n0 >= a.N) break;
#pragma unroll
        for (int ch = 0; ch < 8; ch++)
            g[ch] = a.norm_w ? __ldg((const float4 *)(a.norm_w + n0) + ch) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (c + 1 < c_end) request(c + 1, rl_next);
#pragma unroll
        for (int pass = 0; pass < 8; pass++) {
            const int row = pass * 4 + (lane >> 3), ch = lane & 7;
            *(float4 *)(T + row * 32 + ((ch ^ (row & 7)) << 2)) = rl[pass];
        }
        __syncwarp();
        float v[32];
        tc_ld32(trow + c * 32, v);
        uint32_t xb[16];
#pragma unroll
        for (int ch = 0; ch < 8; ch++) {
            float4 *tp = (float4 *)(T + lane * 32 + ((ch ^ (lane & 7)) << 2));
            const float4 r = *tp;
            const float4 o = make_float4(v[4 * ch] * iv + r.x, v[4 * ch + 1] * iv + r.y, v[4 * ch + 2] * iv + r.z, v[4 * ch + 3] * iv + r.w);
            *tp = o;
            if (a.norm_w) {
                __nv_bfloat162 t0 = __floats2bfloat162_rn(o.x * g[ch].x, o.y * g[ch].y), t1 = __floats2bfloat162_rn(o.z * g[ch].z, o.w * g[ch].w);
                xb[2 * ch] = *(uint32_t *)&t0; xb[2 * ch + 1] = *(uint32_t *)&t1;
                sq += o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w;
            }
        }
        if (a.norm_w) {
#pragma unroll
            for (int ch = 0; ch < 4; ch++)
                *(uint4 *)(X + lane * 64 + ((ch ^ ((lane >> 1) & 3)) << 4)) = make_uint4(xb[4 * ch], xb[4 * ch + 1], xb[4 * ch + 2], xb[4 * ch + 3]);
        }
        __syncwarp();
#pragma unroll
        for (int pass = 0; pass < 8; pass++) {
            const int row = pass * 4 + (lane >> 3), ch = lane & 7, m = m_base + row;
            const float4 t = *(const float4 *)(T + row * 32 + ((ch ^ (row & 7)) << 2));
            if (m < a.M) ((float4 *)((float *)a.out + (size_t)m * a.ldc + n0))[ch] = t;
        }
        if (a.norm_w) {
#pragma unroll
            for (int pass = 0; pass < 4; pass++) {
                const int row = pass * 8 + (lane >> 2), ch = lane & 3, m = m_base + row;
                const uint4 t = *(const uint4 *)(X + row * 64 + ((ch ^ ((row >> 1) & 3)) << 4));
                if (m < a.M) ((uint4 *)(a.xw_out + (size_t)m * a.N + n0))[ch] = t;
            }
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; i++) rl[i] = rl_next[i];
    }
    if (a.norm_w && m_own < a.M) a.ss_out[(size_t)ss_index * a.M + m_own] = sq;
}

// ---------------------------------------------------------------------------- decode: weights stream once
// One kernel for every projection of a decode step: the epilogue, the number of K splits and the depth of the
// ring are run-time values.  A decode step alternates between four or five projections per layer, each launch
// runs its code once, and code that has left the SM's instruction cache is fetched again at hundreds of cycles
// a line: one small kernel that every projection shares stays resident, a family of specialised ones does not.
// For the same reason the once-per-launch epilogue code is written as rolled loops.
#define MAX_STAGES 9

template <int BN>
__global__ void __launch_bounds__(DEC_THREADS(BN), 1)
gemm_tc_decode_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, GemmArgs a) {
    constexpr int W_BYTES = BM * BK * 2, X_BYTES = BN * BK * 2;
    constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
    constexpr int TMEM_COLS = BN <= 32 ? 32 : BN;
    constexpr int RES_AHEAD = 8;                  // residual values of the split-K sum fetched during the main loop
    constexpr int EW = DEC_EPI_WARPS(BN), ET = 32 * EW;           // epilogue warps and threads
    auto epi_sync = [] { asm volatile("bar.sync 1, %0;" ::"n"(ET) : "memory"); };

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);   // swizzle atoms need 1 KB alignment
    __shared__ __align__(8) uint64_t bars[2 * MAX_STAGES + 2];
    __shared__ uint32_t tmem_base_s;
    __shared__ float inv_s[BN];                   // 1/rms of the token columns (deferred norm), else 1
    __shared__ float inv_part[256];               // partial sums on the way to inv_s

    const int warp = warp_index(), lane = threadIdx.x & 31;      // uniform: the role branches below are not divergent
    const int stages = a.stages, epi = a.epi, S = gridDim.z;
    const bool split = S > 1;
    // grid (token block, weight tile, K split): the CTAs next to each other share a weight tile, which the second
    // one finds in L2
    const int p0 = blockIdx.y * BM, q0 = blockIdx.x * BN;      // first weight row (feature) and first token of the tile
    const int total_kb = (a.K + BK - 1) / BK;
    const int kb0 = blockIdx.z * a.kb_per_split;
    const int nkb = min(a.kb_per_split, total_kb - kb0);
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[MAX_STAGES]), tfull = smem_u32(&bars[2 * MAX_STAGES]);
    const uint32_t inbox = smem_u32(&bars[2 * MAX_STAGES + 1]);
    const uint32_t smem0 = smem_u32(smem);
    // split-K: partial columns arrive here from the whole cluster, [rank][group of VW columns][128 rows][VW] f32 with
    // VW = 4 (2 when a CTA owns only two columns), so that a lane sends the VW columns of its row as one packet and
    // the lanes of a warp fill consecutive 16 (8) bytes; a region of its own, since a faster CTA pushes while this one
    // is still in its main loop.  Every CTA of the cluster (this one included) sends BM * VW floats for each of this
    // CTA's column groups whose first column holds a token; `inbox` counts the bytes.
    float *recv = (float *)(smem + stages * STAGE_BYTES);
    const int vw_log = (BN / S) >= 4 ? 2 : 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(tfull, 1);
        mbar_init(inbox, 1);
        if (split) {
            const int per0 = BN / S, vw = 1 << vw_log;
            const int mine = max(0, min(per0 >> vw_log, (a.M - q0 - (int)blockIdx.z * per0 + vw - 1) >> vw_log));   // my groups with a token
            mbar_expect_tx(inbox, (uint32_t)(S * mine * BM * vw * 4));
        }
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
    // the barriers above are initialised: tell the cluster (matched by the wait before the first push, which thereby
    // also knows that every CTA of the cluster runs and that its inbox counts)
    if (split) cluster_arrive_release();
    const uint32_t tmem_base = tmem_base_s;
    pdl_launch_dependents();
    if (threadIdx.x == 32) {                      // descriptors into the cache before their first use
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmW) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmX) : "memory");
    }
    float res_pre[RES_AHEAD], nw_pre[4] = {0.f, 0.f, 0.f, 0.f};

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        // The whole warp walks the ring and waits; one elected lane issues the copies.
        const int pre = min(stages, nkb);
        const uint64_t stream_once = l2_evict_first_policy();
        if (elect_one()) {
            for (int kb = 0; kb < pre; kb++) {                 // weights of the first stages: no dependency
                mbar_expect_tx(full0 + 8 * kb, STAGE_BYTES);
                tma_load_2d_hint(smem0 + kb * STAGE_BYTES, &tmW, (kb0 + kb) * BK, p0, full0 + 8 * kb, stream_once);
            }
        }
        __syncwarp();
        pdl_wait();                                            // activations come from the kernel before
        if (elect_one()) {
            // (a test may ask for stage 0 to stay incomplete: its barrier then never fires and every wait runs out)
            for (int kb = a.test_skip_copy ? 1 : 0; kb < pre; kb++)
                tma_load_2d(smem0 + kb * STAGE_BYTES + W_BYTES, &tmX, (kb0 + kb) * BK, q0, full0 + 8 * kb);
        }
        __syncwarp();
        int s = 0, ph = 1;                                     // ring position of K-block `kb`, parity of its empty barrier
        bool ok = true;
        for (int kb = pre; kb < nkb; kb++) {
            ok = __all_sync(0xffffffffu, mbar_wait(empty0 + 8 * s, ph ^ 1));
            if (!ok) { raise_error(1); break; }
            if (elect_one()) {
                const uint32_t dst = smem0 + s * STAGE_BYTES, bar = full0 + 8 * s;
                mbar_expect_tx(bar, STAGE_BYTES);
                tma_load_2d_hint(dst, &tmW, (kb0 + kb) * BK, p0, bar, stream_once);
                tma_load_2d(dst + W_BYTES, &tmX, (kb0 + kb) * BK, q0, bar);
            }
            __syncwarp();
            if (++s == stages) { s = 0; ph ^= 1; }
        }
        // copies still in flight must land before the CTA may exit: the last pass over the ring
        if (!ok || nkb <= stages) { for (int j = 0; j < min(stages, nkb); j++) mbar_wait(full0 + 8 * j, 0); }
        else {
            // K-block kb sits in stage kb % stages with parity (kb / stages) & 1; wait for the last `stages` of them
            for (int kb = nkb - stages; kb < nkb; kb++) mbar_wait(full0 + 8 * (kb % stages), (kb / stages) & 1);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // The whole warp walks the ring and waits; one elected lane issues.  The descriptor of a stage is the
        // first stage's plus the stage's offset (the address field counts 16-byte units and shared memory is
        // far below its 14 bits).
        const uint32_t idesc = make_idesc(BM, BN);
        const uint64_t wdesc0 = make_smem_desc(smem0), xdesc0 = make_smem_desc(smem0 + W_BYTES);
        int s = 0, ph = 0;
        for (int kb = 0; kb < nkb; kb++) {
            if (!__all_sync(0xffffffffu, mbar_wait(full0 + 8 * s, ph))) { raise_error(2); break; }
            tc_fence_after();
            const uint64_t soff = (uint64_t)(s * (STAGE_BYTES >> 4));
            const uint64_t wdesc = wdesc0 + soff, xdesc = xdesc0 + soff;
            if (elect_one()) {
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; k++) {
                    const uint64_t koff = (uint64_t)((k * UMMA_K * 2) >> 4);     // advance inside the swizzle row
                    tc_mma_bf16(tmem_base, wdesc + koff, xdesc + koff, idesc, (kb | k) != 0);
                }
                tc_commit(empty0 + 8 * s);        // arrives when these MMAs have read the stage
            }
            __syncwarp();
            if (++s == stages) { s = 0; ph ^= 1; }
        }
        if (elect_one()) tc_commit(tfull);        // arrives when every MMA above is complete
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int lg = warp & 3;                  // the TMEM lane group this warp may read
        const int prow = lg * 32 + lane;          // row of the tile this thread owns
        // At 32 and 64 columns two warps share each lane group of tensor memory (warps 2..5 and 6..9) and take alternate
        // runs of 16 columns: with one epilogue warp a scheduler every instruction's latency is exposed, and at 64
        // columns the once-per-launch epilogue was two thirds of a split contraction's time (o: 8.3 -> 7.3 us a layer;
        // at 16 columns the larger CTA cost 1 % of the step instead).
        const int half = EW == 8 ? (warp - 2) >> 2 : 0, et = half * 128 + prow;
        const bool emit = epi == EPI_ADD_F32 && a.norm_w != nullptr;
        // the next norm's weights of the features this thread finishes (lane + 32 i): weights, so they are fetched
        // before the wait on the preceding kernel (a miss in L2 behind the weight tiles in flight takes microseconds)
        if (emit) {
#pragma unroll
            for (int i = 0; i < 4; i++)
                if (p0 + lane + 32 * i < a.N)
                    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(nw_pre[i]) : "l"(a.norm_w + p0 + lane + 32 * i));
        }
        pdl_wait();
        // 1/rms of the token columns of this tile, while the main loop runs
        // (ET / BN threads per column, each striding over the tiles, and their sums added in thread order)
        {
            constexpr int P = ET / BN;
            const int c = et % BN, pp = et / BN;
            const bool live = a.ss_in && q0 + c < a.M;
            float s = 0.f;
            if (live)
                for (int tt = pp; tt < a.ss_tiles; tt += P) s += __ldcg(a.ss_in + (size_t)tt * a.M + q0 + c);
            inv_part[pp * BN + c] = s;
            epi_sync();
            if (et < BN) {
                float tot = 0.f;
#pragma unroll
                for (int p = 0; p < P; p++) tot += inv_part[p * BN + et];
                inv_s[et] = live ? 1.0f / sqrtf(tot / (float)a.ss_size + a.ss_eps) : 1.0f;
            }
        }
        epi_sync();
        if (split && epi == EPI_ADD_F32) {
            // the residual values this thread adds to after the main loop: columns w and w + EW of this CTA's share
            const int per = BN / S, c_begin = blockIdx.z * per, w = warp - 2;
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int cl = w + EW * j, m = q0 + c_begin + cl, nn = p0 + lane + 32 * i;
                    res_pre[4 * j + i] = (cl < per && nn < a.N && m < a.M) ? __ldcg((const float *)a.out + (size_t)m * a.ldc + nn) : 0.f;
                }
        }
        // one lane of each warp polls the barrier, the others wait for it at the shuffle
        int ok_i = 1;
        if (lane == 0 && nkb > 0) ok_i = mbar_wait(tfull, 0) ? 1 : 0;
        const bool ok = __shfl_sync(0xffffffffu, ok_i, 0) != 0;
        if (!ok) raise_error(3);
        tc_fence_after();
        const uint32_t trow = tmem_base + ((uint32_t)(lg * 32) << 16);
        const bool have = ok && nkb > 0;          // the accumulator holds this CTA's part of the sum
        if (epi == EPI_SILU_MUL && !split) {
            // rows 0..63 of the tile are gate, 64..127 up of the same 64 features: both halves go to
            // shared memory as [token][feature], then all 128 threads share the activations
            float *exg = (float *)smem;           // [BN][64]; the stages are idle once tfull has fired
            float *exu = exg + BN * 64;
            const int ncol = min(BN, a.M - q0);
            if (ok) {
                float *ex = prow < 64 ? exg : exu;
#pragma unroll 1
                for (int c0 = 16 * half; c0 < ncol; c0 += 4 * EW) {
                    float v[16];
                    tc_ld16(trow + c0, v);
#pragma unroll
                    for (int j = 0; j < 16; j++) ex[(c0 + j) * 64 + (prow & 63)] = v[j];
                }
            }
            epi_sync();
            const int fl = prow & 63, f = (p0 >> 1) + fl;
            if (ok && f < (a.N >> 1)) {
#pragma unroll 1
                for (int c = et >> 6; c < ncol; c += EW / 2) {      // 64 threads a token
                    const float iv = inv_s[c];
                    ((bf16 *)a.out)[(size_t)(q0 + c) * a.ldc + f] =
                        __float2bfloat16_rn(silu_mul(exg[c * 64 + fl] * iv, exu[c * 64 + fl] * iv));
                }
            }
        } else {
            // partial tile -> the owners of its columns: CTA r of the cluster sums columns [r * per, (r + 1) * per).
            // Without a split the CTA is its own owner and the tile passes through its (now idle) ring instead.
            const int per = BN / S, per_log = __ffs(per) - 1;       // BN and S are powers of two
            if (split) cluster_wait();            // every CTA of the cluster has started (arrived at its top)
            const uint32_t recv0 = smem_u32(recv);
            const int groups = per >> vw_log;     // column groups an owner receives from each rank
#pragma unroll 1
            for (int c0 = 16 * half; c0 < BN; c0 += 4 * EW) {
                float v[16];
                if (have) tc_ld16(trow + c0, v);
                else {
#pragma unroll
                    for (int j = 0; j < 16; j++) v[j] = 0.f;
                }
                if (!split) {
#pragma unroll
                    for (int j = 0; j < 16; j++)
                        if (q0 + c0 + j < a.M) ((float *)smem)[(c0 + j) * BM + prow] = v[j];      // a column without a token is never read
                } else if (vw_log == 2) {
#pragma unroll
                    for (int j = 0; j < 16; j += 4) {
                        const int c = c0 + j, r = c >> per_log, cg = (c & (per - 1)) >> 2;
                        if (q0 + c >= a.M) continue;
                        st_async_f32x4(recv0 + ((((int)blockIdx.z * groups + cg) * BM + prow) << 4), inbox, r, v + j);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j += 2) {
                        const int c = c0 + j, r = c >> per_log, cg = (c & (per - 1)) >> 1;
                        if (q0 + c >= a.M) continue;
                        st_async_f32x2(recv0 + ((((int)blockIdx.z * groups + cg) * BM + prow) << 3), inbox, r, v + j);
                    }
                }
            }
        }
        tc_fence_before();
    }
    if (epi != EPI_SILU_MUL || split) {
        // ---- after the barrier this CTA's shared memory holds, for its columns, the partial sums of every CTA of
        // the cluster; they are added in rank order and the epilogue runs on the totals
        if (split) {
            // every partial sum for this CTA's columns has landed when the inbox has counted its bytes; nobody waits
            // for the cluster (the producer and issuer warps only close the barrier phase that opened at the top)
            if (warp < 2) { __syncwarp(); cluster_wait(); }
            else if (!mbar_wait(inbox, 0)) raise_error(5);
        } else if (warp >= 2) epi_sync();
        if (warp >= 2) {
            // A warp takes whole columns (tokens) here: its lanes cover the 128 features in four steps, so the sum of
            // squares of a column needs one warp reduction and no exchange between warps, and it comes before the
            // column's stores (a shuffle queues behind the warp's earlier stores in the memory pipeline).
            const int w = warp - 2;
            const int per = BN / S, c_begin = blockIdx.z * per;
            const bool emit = epi == EPI_ADD_F32 && a.norm_w != nullptr;
            const float *part = split ? recv : (const float *)smem;
#pragma unroll 1
            for (int cl = w; cl < per; cl += EW) {
                const int m = q0 + c_begin + cl;
                if (m >= a.M) break;                                               // tokens fill the columns from 0
                // a short rolled loop over the ranks, the four features' loads in flight together
                float v[4] = {0.f, 0.f, 0.f, 0.f};
                const float *pc = split ? part + ((((cl >> vw_log) * BM + lane) << vw_log) + (cl & ((1 << vw_log) - 1))) : part + cl * BM + lane;
                const int zstride = split ? ((per >> vw_log) * BM) << vw_log : 0, istride = split ? 32 << vw_log : 32;
#pragma unroll 1
                for (int z = 0; z < S; z++, pc += zstride) {                       // rank order
#pragma unroll
                    for (int i = 0; i < 4; i++) v[i] += pc[i * istride];
                }
                const float iv = inv_s[c_begin + cl];
                if (epi == EPI_SILU_MUL) {
                    // features lane and lane + 32 of the tile's 64: gate in rows 0..63 (v[0], v[1]), up in 64..127
#pragma unroll
                    for (int i = 0; i < 2; i++) {
                        const int f = (p0 >> 1) + lane + 32 * i;
                        if (f < (a.N >> 1))
                            ((bf16 *)a.out)[(size_t)m * a.ldc + f] = __float2bfloat16_rn(silu_mul(v[i] * iv, v[i + 2] * iv));
                    }
                    continue;
                }
                float sq = 0.f;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int n = p0 + lane + 32 * i;
                    v[i] *= iv;
                    if (epi == EPI_ADD_F32 && n < a.N) {
                        v[i] += (split && cl < 2 * EW) ? (cl < EW ? res_pre[i] : res_pre[4 + i]) : ((const float *)a.out)[(size_t)m * a.ldc + n];
                        sq += v[i] * v[i];
                    }
                }
                if (emit) sq = warp_sum(sq);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int n = p0 + lane + 32 * i;
                    if (n >= a.N) continue;
                    const size_t idx = (size_t)m * a.ldc + n;
                    if (epi == EPI_BF16) ((bf16 *)a.out)[idx] = __float2bfloat16_rn(v[i]);
                    else {
                        ((float *)a.out)[idx] = v[i];
                        if (emit) a.xw_out[(size_t)m * a.N + n] = __float2bfloat16_rn(v[i] * nw_pre[i]);
                    }
                }
                if (emit && lane == 0) a.ss_out[(size_t)blockIdx.y * a.M + m] = sq;
            }
        }
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------- prefill: persistent tiles
// Token-major tiles (P = 128 token rows, Q = BN weight rows) for many rows.  One CTA per SM walks
// the tiles with a stride of the grid; two accumulators in tensor memory alternate, so the
// epilogue of a tile (tcgen05.ld, conversion, stores) runs while the MMAs of the next tile fill the
// other accumulator.  Consecutive CTAs take tiles of the same weight rows, so those stay in L2.
template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_prefill_kernel(const __grid_constant__ CUtensorMap tmP, const __grid_constant__ CUtensorMap tmQ, GemmArgs a,
                       int n_pt, int n_tiles) {
    constexpr int P_BYTES = BM * BK * 2, Q_BYTES = BN * BK * 2;
    constexpr int STAGE_BYTES = P_BYTES + Q_BYTES;
    constexpr int TMEM_COLS = BN <= 128 ? 256 : 512;   // two accumulators of BN columns; allocations are powers of two

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 4];
    __shared__ uint32_t tmem_base_s;

    const int warp = warp_index(), lane = threadIdx.x & 31;
    const int nkb = (a.K + BK - 1) / BK;
    // Split along K (a.splits > 1, plain f32 epilogue only): the tile index also counts the split, slowest, and split z
    // writes the product over its K-blocks into block z of the output; gemm_splitk_finish_kernel adds the blocks.
    const int per_split = a.splits > 1 ? n_tiles / a.splits : n_tiles;
    auto kb_range = [&](int tile, int &kb_begin, int &kb_end) {
        if (a.splits > 1) { kb_begin = (tile / per_split) * a.kb_per_split; kb_end = min(nkb, kb_begin + a.kb_per_split); }
        else { kb_begin = 0; kb_end = nkb; }
    };
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
    const uint32_t tfull0 = smem_u32(&bars[2 * STAGES]), tempty0 = smem_u32(&bars[2 * STAGES + 2]);
    const uint32_t smem0 = smem_u32(smem);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int i = 0; i < 2; i++) { mbar_init(tfull0 + 8 * i, 1); mbar_init(tempty0 + 8 * i, 4); }   // 4 epilogue warps
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
    pdl_launch_dependents();
    if (threadIdx.x == 32) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmP) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmQ) : "memory");
    }

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        // the whole warp walks the tiles and the ring and waits; one elected lane issues the copies
        pdl_wait();
        int s = 0, ph = 0, issued = 0;                 // ring position, pass over the ring (parity), stages filled so far
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
            const int t2 = tile % per_split, p0 = (t2 % n_pt) * BM, q0 = (t2 / n_pt) * BN;
            int kb_begin, kb_end;
            kb_range(tile, kb_begin, kb_end);
            for (int kb = kb_begin; kb < kb_end; kb++) {
                ok = __all_sync(0xffffffffu, mbar_wait(empty0 + 8 * s, ph ^ 1));
                if (!ok) { raise_error(1); break; }
                if (elect_one()) {
                    const uint32_t dst = smem0 + s * STAGE_BYTES, bar = full0 + 8 * s;
                    mbar_expect_tx(bar, STAGE_BYTES);
                    tma_load_2d(dst, &tmP, kb * BK, p0, bar);
                    tma_load_2d(dst + P_BYTES, &tmQ, kb * BK, q0, bar);
                }
                __syncwarp();
                issued++;
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
        }
        for (int j = max(0, issued - STAGES); j < issued; j++)      // copies in flight land before the CTA exits
            mbar_wait(full0 + 8 * (j % STAGES), (j / STAGES) & 1);
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // the whole warp walks the tiles and the ring and waits; one elected lane issues
        const uint32_t idesc = make_idesc(BM, BN);
        const uint64_t pdesc0 = make_smem_desc(smem0), qdesc0 = make_smem_desc(smem0 + P_BYTES);
        int s = 0, ph = 0, i = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, i++) {
            const int acc = i & 1;
            // the epilogue must have emptied this accumulator (its use before the last one)
            if (!__all_sync(0xffffffffu, mbar_wait(tempty0 + 8 * acc, ((i >> 1) & 1) ^ 1))) { raise_error(4); break; }
            tc_fence_after();
            int kb_begin, kb_end;
            kb_range(tile, kb_begin, kb_end);
            for (int kb = kb_begin; kb < kb_end; kb++) {
                ok = __all_sync(0xffffffffu, mbar_wait(full0 + 8 * s, ph));
                if (!ok) { raise_error(2); break; }
                tc_fence_after();
                const uint64_t soff = (uint64_t)(s * (STAGE_BYTES >> 4));      // the address field counts 16-byte units
                const uint64_t pdesc = pdesc0 + soff, qdesc = qdesc0 + soff;
                if (elect_one()) {
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++) {
                        const uint64_t koff = (uint64_t)((k * UMMA_K * 2) >> 4);
                        tc_mma_bf16(tmem_base + acc * BN, pdesc + koff, qdesc + koff, idesc, ((kb - kb_begin) | k) != 0);
                    }
                    tc_commit(empty0 + 8 * s);
                }
                __syncwarp();
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
            if (elect_one()) tc_commit(tfull0 + 8 * acc);      // also after an error: the epilogue is not left waiting
            __syncwarp();
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        pdl_wait();
        const int lg = warp & 3, prow = lg * 32 + lane;
        int i = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, i++) {
            const int acc = i & 1;
            const int t2 = tile % per_split, pt = t2 % n_pt, qt = t2 / n_pt;
            if (!mbar_wait(tfull0 + 8 * acc, (i >> 1) & 1)) { raise_error(3); break; }
            tc_fence_after();
            const uint32_t trow = tmem_base + ((uint32_t)(lg * 32) << 16) + acc * BN;
            if (EPI == EPI_ADD_F32 && a.vec_ok && (a.N & 31) == 0)
                epilogue_add_coalesced<BN>(a, trow, pt * BM, qt * BN, qt, lg, lane, smem + STAGES * STAGE_BYTES + lg * EPI_STAGE_BYTES);
            else
                epilogue_token_major<BN, EPI>(a, trow, pt * BM, qt * BN, qt, prow, (size_t)(tile / per_split) * (size_t)a.M);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tempty0 + 8 * acc) : "memory");
        }
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// Second half of a prefill contraction split along K: out = epilogue(sum over the splits of ws[split][M][N]), the
// splits added in their order.  A warp takes one token row and 128 features (lane + 32 i), so that the sum of squares
// of the started norm is one warp reduction; ss_out is indexed by 128-feature tile like the decode kernel's.
template <int EPI>
__global__ void __launch_bounds__(256)
gemm_splitk_finish_kernel(GemmArgs a, const float *__restrict__ ws, int S) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, m = blockIdx.y * 8 + (threadIdx.x >> 5), qt = blockIdx.x, q0 = qt * 128;
    if (m >= a.M) return;
    // everything this warp reads is asked for at once: the partial sums of squares of the row (a lane each), the
    // residual values and norm weights of its features, then the partial products
    float ss_mine[2] = {0.f, 0.f};
    if (a.ss_in) {
#pragma unroll
        for (int h = 0; h < 2; h++)
            if (lane + 32 * h < a.ss_tiles) ss_mine[h] = __ldcg(a.ss_in + (size_t)(lane + 32 * h) * a.M + m);
    }
    float res[4] = {0.f, 0.f, 0.f, 0.f}, nw[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int n = q0 + lane + 32 * i;
        if (n >= a.N) continue;
        if (EPI == EPI_ADD_F32) res[i] = ((const float *)a.out)[(size_t)m * a.ldc + n];
        if (EPI == EPI_ADD_F32 && a.norm_w) nw[i] = a.norm_w[n];
    }
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    const float *p = ws + (size_t)m * a.N + q0 + lane;
    const size_t zstride = (size_t)a.M * a.N;
#pragma unroll 1
    for (int z = 0; z < S; z++, p += zstride) {
#pragma unroll
        for (int i = 0; i < 4; i++)
            if (q0 + lane + 32 * i < a.N) v[i] += __ldcg(p + 32 * i);
    }
    float iv = 1.0f;
    if (a.ss_in) {
        // the sum in tile order, as inv_rms adds it (up to 64 tiles; more fall back to its loop)
        if (a.ss_tiles <= 64) {
            float s = 0.f;
            for (int t = 0; t < a.ss_tiles; t++) s += __shfl_sync(0xffffffffu, t < 32 ? ss_mine[0] : ss_mine[1], t & 31);
            iv = 1.0f / sqrtf(s / (float)a.ss_size + a.ss_eps);
        } else iv = inv_rms(a, m);
    }
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int n = q0 + lane + 32 * i;
        if (n >= a.N) continue;
        const size_t idx = (size_t)m * a.ldc + n;
        float x = v[i] * iv;
        if (EPI == EPI_BF16) { ((bf16 *)a.out)[idx] = __float2bfloat16_rn(x); continue; }
        if (EPI == EPI_ADD_F32) x += res[i];
        ((float *)a.out)[idx] = x;
        if (EPI == EPI_ADD_F32 && a.norm_w) {
            a.xw_out[(size_t)m * a.N + n] = __float2bfloat16_rn(x * nw[i]);
            sq += x * x;
        }
    }
    if (EPI == EPI_ADD_F32 && a.norm_w) {
        sq = warp_sum(sq);
        if (lane == 0) a.ss_out[(size_t)qt * a.M + m] = sq;
    }
}

// ---------------------------------------------------------------------------- prefill: pairs of CTAs on 256-row tiles
// Two CTAs of a cluster (a pair of SMs) share a tile of 256 token rows x BN weight rows: each loads its own 128
// token rows and HALF of the weight rows, and the pair's leader issues tcgen05.mma.cta_group::2, which reads both
// CTAs' shared memory and writes each CTA's 128 accumulator rows into that CTA's tensor memory.  Per K-block an
// SM then receives 16 + BN/4 KB instead of 16 + BN/2 KB for the same MMA time: the main loop of the 128-row kernel
// is bound by the L2-to-SM path, not by the tensor pipe.
//   every copy of both CTAs completes on the LEADER's full barrier (cp.async.bulk.tensor .cta_group::2); the
//   leader's commit frees the stage in both CTAs and hands the accumulator to both epilogues
//   (tcgen05.commit .multicast::cluster); both epilogues release the accumulator on the leader's barrier.
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local_addr, int rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    return remote;
}
// a copy whose completion is counted on a barrier given by its cluster address (the pair leader's)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t cluster_bar) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, bool accumulate) {
    const uint32_t acc = accumulate ? 1u : 0u, z = 0u;
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc), "r"(z) : "memory");
}
// arrives on the barrier at this address in BOTH CTAs of the pair once the MMAs issued so far are complete
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(both) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// The residual-add epilogue is exposed whole when a launch is one round of tiles (o and down at 2,048 rows), and with
// one epilogue warp a scheduler every instruction's latency shows: that variant runs eight epilogue warps, two per
// lane group of tensor memory, each half of the tile's columns (and writes two partial sums of squares a tile).
#define PAIR_EPI_WARPS(EPI) ((EPI) == EPI_ADD_F32 ? 8 : 4)
#define PAIR_THREADS(EPI) (64 + 32 * PAIR_EPI_WARPS(EPI))
template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(PAIR_THREADS(EPI), 1)
gemm_tc_prefill_pair_kernel(const __grid_constant__ CUtensorMap tmP, const __grid_constant__ CUtensorMap tmQ, GemmArgs a,
                            int n_pt, int n_tiles) {
    constexpr int P_BYTES = BM * BK * 2, Q_BYTES = (BN / 2) * BK * 2;      // this CTA's share of a stage
    constexpr int STAGE_BYTES = P_BYTES + Q_BYTES;
    constexpr int TMEM_COLS = BN <= 128 ? 256 : 512;

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 4];
    __shared__ uint32_t tmem_base_s;

    const int warp = warp_index(), lane = threadIdx.x & 31;
    const int rank = (int)(blockIdx.x & 1);            // 0: the pair's leader (issues the MMAs), 1: its peer
    const int pair = (int)(blockIdx.x >> 1), n_pairs = (int)(gridDim.x >> 1);
    const int nkb = (a.K + BK - 1) / BK;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
    const uint32_t tfull0 = smem_u32(&bars[2 * STAGES]), tempty0 = smem_u32(&bars[2 * STAGES + 2]);
    const uint32_t smem0 = smem_u32(smem);
    const uint32_t lead_full0 = mapa_u32(full0, 0), lead_tempty0 = mapa_u32(tempty0, 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int i = 0; i < 2; i++) { mbar_init(tfull0 + 8 * i, 1); mbar_init(tempty0 + 8 * i, 2 * PAIR_EPI_WARPS(EPI)); }   // epilogue warps x 2 CTAs
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();                                    // the partner's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    pdl_launch_dependents();
    if (threadIdx.x == 32) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmP) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmQ) : "memory");
    }

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        pdl_wait();
        int s = 0, ph = 0;
        bool ok = true;
        for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
            const int p0 = (tile % n_pt) * (2 * BM) + rank * BM, q0 = (tile / n_pt) * BN + rank * (BN / 2);
            for (int kb = 0; kb < nkb; kb++) {
                ok = __all_sync(0xffffffffu, mbar_wait(empty0 + 8 * s, ph ^ 1));
                if (!ok) { raise_error(1); break; }
                if (elect_one()) {
                    const uint32_t dst = smem0 + s * STAGE_BYTES, bar = lead_full0 + 8 * s;
                    if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);     // both CTAs' copies of the stage
                    tma_load_2d_pair(dst, &tmP, kb * BK, p0, bar);
                    tma_load_2d_pair(dst + P_BYTES, &tmQ, kb * BK, q0, bar);
                }
                __syncwarp();
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
        }
        // the copies of both CTAs have landed once the leader has seen every stage full; the cluster barrier at the
        // end of the kernel comes after that
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (the leader only)
        if (rank == 0) {
            const uint32_t idesc = make_idesc(2 * BM, BN);
            const uint64_t pdesc0 = make_smem_desc(smem0), qdesc0 = make_smem_desc(smem0 + P_BYTES);
            int s = 0, ph = 0, i = 0;
            bool ok = true;
            for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, i++) {
                const int acc = i & 1;
                if (!__all_sync(0xffffffffu, mbar_wait(tempty0 + 8 * acc, ((i >> 1) & 1) ^ 1))) { raise_error(4); break; }
                tc_fence_after();
                for (int kb = 0; kb < nkb; kb++) {
                    ok = __all_sync(0xffffffffu, mbar_wait(full0 + 8 * s, ph));
                    if (!ok) { raise_error(2); break; }
                    tc_fence_after();
                    const uint64_t soff = (uint64_t)(s * (STAGE_BYTES >> 4));
                    const uint64_t pdesc = pdesc0 + soff, qdesc = qdesc0 + soff;
                    if (elect_one()) {
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; k++) {
                            const uint64_t koff = (uint64_t)((k * UMMA_K * 2) >> 4);
                            tc_mma_bf16_pair(tmem_base + acc * BN, pdesc + koff, qdesc + koff, idesc, (kb | k) != 0);
                        }
                        tc_commit_pair(empty0 + 8 * s);              // frees the stage in both CTAs
                    }
                    __syncwarp();
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
                if (elect_one()) tc_commit_pair(tfull0 + 8 * acc);   // both epilogues; also after an error
                __syncwarp();
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2.., both CTAs): this CTA's 128 rows
        pdl_wait();
        constexpr int EW = PAIR_EPI_WARPS(EPI);
        const int lg = warp & 3, prow = lg * 32 + lane, half = EW == 8 ? (warp - 2) >> 2 : 0;
        int i = 0;
        for (int tile = pair; tile < n_tiles; tile += n_pairs, i++) {
            const int acc = i & 1;
            const int pt = tile % n_pt, qt = tile / n_pt;
            const int p0 = pt * (2 * BM) + rank * BM;
            if (!mbar_wait(tfull0 + 8 * acc, (i >> 1) & 1)) { raise_error(3); break; }
            tc_fence_after();
            const uint32_t trow = tmem_base + ((uint32_t)(lg * 32) << 16) + acc * BN;
            if (EPI == EPI_ADD_F32 && a.vec_ok && (a.N & 31) == 0)
                epilogue_add_coalesced<BN>(a, trow, p0, qt * BN, qt * (EW / 4) + half, lg, lane,
                                           smem + STAGES * STAGE_BYTES + (half * 4 + lg) * EPI_STAGE_BYTES, half * (BN / 64), EW == 8 ? (half + 1) * (BN / 64) : BN / 32);
            else if (half == 0)
                epilogue_token_major<BN, EPI>(a, trow, p0, qt * BN, qt * (EW / 4), prow);
            else if (EPI == EPI_ADD_F32 && a.norm_w && p0 + prow < a.M)
                a.ss_out[(size_t)(qt * 2 + 1) * a.M + p0 + prow] = 0.f;      // the second partial sum of a tile the row-wise path leaves empty
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(lead_tempty0 + 8 * acc);      // the leader's barrier counts both CTAs' warps
        }
    }
    // Neither CTA leaves, or frees tensor memory, while the other may still read its shared memory (the leader's
    // MMAs), wait for its copies (they complete on the leader's barriers) or arrive on its barriers.
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
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

static int sm_count();
template <int BN>
static int launch_decode(const CUtensorMap &tmW, const CUtensorMap &tmX, GemmArgs a, dim3 grid, cudaStream_t stream) {
    // two CTAs share an SM: ring and (split-K) receive buffer together stay under half its shared memory ...
    const bool split = grid.z > 1;
    constexpr int stage_bytes = (BM + BN) * BK * 2;
    a.stages = BN == 16 ? (split ? 5 : 6) : BN == 32 ? (split ? 4 : 5) : (split ? 3 : 4);
    // a launch of one CTA an SM at most that streams a whole matrix (gate/up): a deeper ring, alone on its SM
    // (measured: 3 % of the step at batch 64, under 1 % at batch 8)
    if (!split && (int)(grid.x * grid.y) <= sm_count()) a.stages = BN == 16 ? 9 : BN == 32 ? 8 : 6;
    if (a.stages > a.kb_per_split) a.stages = a.kb_per_split;      // a short K loop needs no deeper ring: room for other CTAs
    // without a split the epilogue passes the f32 tile (BN x 128) through the idle ring: the ring is at least that large
    int ring = a.stages * stage_bytes;
    if (!split && ring < BN * BM * 4) ring = BN * BM * 4;
    const int smem = ring + 1024 + (split ? BN * BM * 4 : 0);
    constexpr int smem_max = MAX_STAGES * stage_bytes + 1024;
    static FgPerDevice configured;
    if (fg_needs_setup(configured)) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_decode_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max);
        if (e != cudaSuccess) return (int)e;
    }
    return fg_launch_cluster(gemm_tc_decode_kernel<BN>, grid, dim3(DEC_THREADS(BN)), (size_t)smem, stream, (int)grid.z, tmW, tmX, a);
}

template <int BN, int STAGES, int EPI>
static int launch_prefill(const CUtensorMap &tmP, const CUtensorMap &tmQ, const GemmArgs &a, cudaStream_t stream) {
    constexpr int smem = STAGES * (BM + BN) * BK * 2 + 1024 + (EPI == EPI_ADD_F32 ? 4 * EPI_STAGE_BYTES : 0);
    static FgPerDevice configured;
    static int n_sm = 0;
    if (fg_needs_setup(configured)) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_prefill_kernel<BN, STAGES, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0) n_sm = 148;
    }
    int n_pt = (a.M + BM - 1) / BM, n_tiles = n_pt * ((a.N + BN - 1) / BN) * (a.splits > 1 ? a.splits : 1);
    dim3 grid(n_tiles < n_sm ? n_tiles : n_sm);
    return fg_launch(gemm_tc_prefill_kernel<BN, STAGES, EPI>, grid, dim3(GEMM_THREADS), (size_t)smem, stream, tmP, tmQ, a,
                     n_pt, n_tiles);
}

static int sm_count();
template <int BN, int STAGES, int EPI>
static int launch_prefill_pair(const CUtensorMap &tmP, const CUtensorMap &tmQ, const GemmArgs &a, cudaStream_t stream) {
    constexpr int smem = STAGES * (BM + BN / 2) * BK * 2 + 1024 + (EPI == EPI_ADD_F32 ? PAIR_EPI_WARPS(EPI) * EPI_STAGE_BYTES : 0);
    static FgPerDevice configured;
    static int n_sm = 0;
    if (fg_needs_setup(configured)) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_prefill_pair_kernel<BN, STAGES, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        n_sm = sm_count();
    }
    int n_pt = (a.M + 2 * BM - 1) / (2 * BM), n_tiles = n_pt * ((a.N + BN - 1) / BN);
    int pairs = n_sm / 2;
    // the CTAs of a pair are neighbours along x
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (n_tiles < pairs ? n_tiles : pairs), 1, 1); cfg.blockDim = dim3(PAIR_THREADS(EPI));
    cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (fg_pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        n++;
    }
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = 2; attr[n].val.clusterDim.y = 1; attr[n].val.clusterDim.z = 1;
    n++;
    cfg.attrs = attr; cfg.numAttrs = n;
    return (int)cudaLaunchKernelEx(&cfg, gemm_tc_prefill_pair_kernel<BN, STAGES, EPI>, tmP, tmQ, a, n_pt, n_tiles);
}

template <int EPI>
static int dispatch(bool swap, int bn, const CUtensorMap &tmP, const CUtensorMap &tmQ, const GemmArgs &a, dim3 grid, cudaStream_t st) {
    if (swap) {
        GemmArgs d = a;
        d.epi = EPI;
        switch (bn) {
        case 16: return launch_decode<16>(tmP, tmQ, d, grid, st);
        case 32: return launch_decode<32>(tmP, tmQ, d, grid, st);
        case 64: return launch_decode<64>(tmP, tmQ, d, grid, st);
        }
    } else {
        switch (bn) {
        case -256: return launch_prefill_pair<256, EPI == EPI_ADD_F32 ? 5 : 6, EPI>(tmP, tmQ, a, st);      // (room for eight epilogue tiles)
        case -192: if (EPI != EPI_SILU_MUL) return launch_prefill_pair<192, 6, EPI == EPI_SILU_MUL ? EPI_BF16 : EPI>(tmP, tmQ, a, st); break;
        case 128: return launch_prefill<128, 6, EPI>(tmP, tmQ, a, st);
        case 192: if (EPI != EPI_SILU_MUL) return launch_prefill<192, 5, EPI == EPI_SILU_MUL ? EPI_BF16 : EPI>(tmP, tmQ, a, st); break;
        case 256: return launch_prefill<256, 4, EPI>(tmP, tmQ, a, st);
        }
    }
    return FG_ERR_BAD_SIZE;
}

// Upper bound of the tiles along N that the residual-add epilogue writes sums of squares for.
extern "C" int fg_gemm_tc_max_ss_tiles(int N) {
    // 128-wide tiles, or two partial sums for each 192-wide tile of a pair of CTAs
    const int narrow = (N + BM - 1) / BM, halves = 2 * ((N + 191) / 192);
    return narrow > halves ? narrow : halves;
}

// X: [M, K] bf16 (row stride ldx), W: [N, K] bf16 (row stride ldw); epi as the enum above.
// ss_in (optional): X holds rows x * w of a deferred RMSNorm; ss_in[t * M + m], t < ss_tiles, are partial
// sums of squares of row m over ss_size elements, and 1/sqrt(sum / ss_size + ss_eps) scales row m's results.
// norm_w (optional, residual-add epilogue): also write xw_out[M, N] = bf16(out * norm_w) and the partial
// sums of squares ss_out[tile, M]; *ss_tiles_out receives the number of tiles.
// EPI_SILU_MUL: W is [N = 2F, K] with gate and up interleaved in blocks of 64 rows; out is [M, F] bf16.
// Returns FG_ERR_BAD_SIZE for shapes TMA cannot describe (K % 8, unaligned bases): the caller
// then uses the plain kernel.
// streaming multiprocessors of the current device (148 on a B200)
static int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

// How a prefill contraction with few output tiles is split along K: 128 x 128 tiles, as many splits as bring the CTAs
// towards one an SM, each at least 8 K-blocks long.  0: no split (the decode kernel's range, enough tiles, short K).
static int prefill_splits(int M, int N, int K, int epi, int *kb_per_split) {
    static int off = -1;                           // FASTGGUF_SPLITK=0: never (the prefill kernels as they were without it)
    if (off < 0) { const char *e = getenv("FASTGGUF_SPLITK"); off = (e && e[0] == '0') ? 1 : 0; }
    if (off || M <= 128 || epi == EPI_SILU_MUL) return 0;
    const int total_kb = (K + BK - 1) / BK, sms = sm_count();
    const long long tiles = (long long)((M + BM - 1) / BM) * ((N + 127) / 128);
    if (tiles * 2 > sms || total_kb < 16) return 0;
    int S = (int)(sms / tiles);
    if (S > 8) S = 8;
    if (S > total_kb / 8) S = total_kb / 8;
    // what the split saves (K-blocks off each CTA's walk) against what the second kernel costs (about 5 us, 20 K-blocks)
    if (S < 2 || (long long)total_kb * (S - 1) < 24ll * S) return 0;
    const int kbs = (total_kb + S - 1) / S;
    *kb_per_split = kbs;
    return (total_kb + kbs - 1) / kbs;             // no empty split
}

// Bytes of workspace with which fg_gemm_tc_ws splits this contraction along K (0: it does not split it).
extern "C" long long fg_gemm_tc_workspace_bytes(int M, int N, int K, int epi) {
    int kbs = 0;
    const int S = prefill_splits(M, N, K, epi, &kbs);
    return S ? (long long)S * M * N * 4 : 0;
}

extern "C" int fg_gemm_tc_ws(const void *X, int ldx, const void *W, int ldw, void *out, int ldc, int epi,
                             int M, int N, int K, int force_splits, const float *ss_in, int ss_tiles, int ss_size,
                             float ss_eps, const float *norm_w, void *xw_out, float *ss_out, int *ss_tiles_out,
                             void *workspace, long long workspace_bytes, cudaStream_t stream);

extern "C" int fg_gemm_tc(const void *X, int ldx, const void *W, int ldw, void *out, int ldc, int epi,
                          int M, int N, int K, int force_splits, const float *ss_in, int ss_tiles, int ss_size,
                          float ss_eps, const float *norm_w, void *xw_out, float *ss_out, int *ss_tiles_out,
                          cudaStream_t stream) {
    return fg_gemm_tc_ws(X, ldx, W, ldw, out, ldc, epi, M, N, K, force_splits, ss_in, ss_tiles, ss_size, ss_eps, norm_w, xw_out,
                         ss_out, ss_tiles_out, nullptr, 0, stream);
}

// As fg_gemm_tc, with `workspace_bytes` of 16-byte aligned device memory that the call may use (and the kernels it
// launches, until they have run): with at least fg_gemm_tc_workspace_bytes(M, N, K, epi) of it, a prefill contraction
// of few output tiles (o and down at a few hundred rows: 32 CTAs walking all of K) runs as partial products over
// slices of K on all SMs and a second kernel that adds them in order and applies the epilogue.
extern "C" int fg_gemm_tc_ws(const void *X, int ldx, const void *W, int ldw, void *out, int ldc, int epi,
                             int M, int N, int K, int force_splits, const float *ss_in, int ss_tiles, int ss_size,
                             float ss_eps, const float *norm_w, void *xw_out, float *ss_out, int *ss_tiles_out,
                             void *workspace, long long workspace_bytes, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return FG_ERR_BAD_SIZE;
    if (epi == EPI_SILU_MUL && N % 128) return FG_ERR_BAD_SIZE;
    // Up to 128 rows the weights stream through the decode kernel, in blocks of 64 tokens whose CTAs run side by side
    // and share each weight tile through L2; beyond that the prefill kernel is faster (measured: 56.6 against 45.5 k tok/s
    // at 96 rows, 65.8 against 74.0 k at 200).
    if (norm_w && (epi != EPI_ADD_F32 || !xw_out || !ss_out)) return FG_ERR_BAD_DTYPE;
    if (workspace && force_splits == 0 && ((uintptr_t)workspace & 15) == 0 && N % 4 == 0) {
        int kbs = 0;
        const int S = prefill_splits(M, N, K, epi, &kbs);
        if (S && (long long)S * M * N * 4 <= workspace_bytes) {
            CUtensorMap tmP, tmQ;
            int e = make_map(&tmP, X, M, K, ldx, BM);
            if (e) return e;
            e = make_map(&tmQ, W, N, K, ldw, 128);
            if (e) return e;
            GemmArgs part{workspace, M, N, K, N, kbs, 1, nullptr, 0, 1, 0.f, nullptr, nullptr, nullptr, EPI_F32, 0, g_test_skip_copy, S};
            e = launch_prefill<128, 6, EPI_F32>(tmP, tmQ, part, stream);
            if (e) return e;
            const int esz = (epi == EPI_F32 || epi == EPI_ADD_F32) ? 4 : 2;
            const int vec = ((uintptr_t)out % 16 == 0) && ((size_t)ldc * esz % 16 == 0);
            if (ss_tiles_out) *ss_tiles_out = (N + 127) / 128;
            GemmArgs fin{out, M, N, K, ldc, kbs, vec, ss_in, ss_tiles, ss_size, ss_eps, norm_w, (bf16 *)xw_out, ss_out, epi, 0, 0, S};
            dim3 grid((N + 127) / 128, (M + 7) / 8);
            const float *ws = (const float *)workspace;
            // The second kernel starts in plain stream order, when the partial products are complete.  Launched as a
            // dependent it sat resident on every SM while they ran, its own successor (a contraction with tensor
            // memory and nearly all of an SM's shared memory) started beside them too, and one prompt step in a few
            // hundred then never finished; with the successor held back until this kernel runs, none did.
            switch (epi) {
            case EPI_BF16: return fg_launch_in_order(gemm_splitk_finish_kernel<EPI_BF16>, grid, dim3(256), 0, stream, fin, ws, S);
            case EPI_F32: return fg_launch_in_order(gemm_splitk_finish_kernel<EPI_F32>, grid, dim3(256), 0, stream, fin, ws, S);
            case EPI_ADD_F32: return fg_launch_in_order(gemm_splitk_finish_kernel<EPI_ADD_F32>, grid, dim3(256), 0, stream, fin, ws, S);
            }
            return FG_ERR_BAD_DTYPE;
        }
    }
    const bool swap = M <= 128;
    const int total_kb = (K + BK - 1) / BK;
    int bn, splits = 1;
    dim3 grid;
    if (swap) {
        bn = M <= 16 ? 16 : M <= 32 ? 32 : 64;
        int tiles = (N + BM - 1) / BM, blocks = (M + bn - 1) / bn;
        // too few tiles to fill the SMs: a cluster of 2, 4 or 8 CTAs shares each tile along K
        while (splits < 8 && tiles * blocks * splits < sm_count() * 4 / 5 && total_kb >= 4 * splits) splits *= 2;
        if (force_splits == 1 || force_splits == 2 || force_splits == 4 || force_splits == 8)
            if (force_splits <= total_kb) splits = force_splits;
        grid = dim3(blocks, tiles, 1);
    } else {
        // tile width: rounds of tiles over the persistent CTAs (one an SM) times the width (a 128-wide tile costs a tenth
        // more per column); 192 is there for feature counts like 3072 that quantise badly at 128 and 256
        int pt = (M + BM - 1) / BM;
        long long t256 = (long long)pt * ((N + 255) / 256), t192 = (long long)pt * ((N + 191) / 192), t128 = (long long)pt * ((N + 127) / 128);
        const int sms = sm_count();
        double c256 = (double)((t256 + sms - 1) / sms), c192 = 0.75 * (double)((t192 + sms - 1) / sms), c128 = 0.55 * (double)((t128 + sms - 1) / sms);
        bn = (N <= 128 || c128 < c256) ? 128 : 256;
        if (epi != EPI_SILU_MUL && N > 128 && c192 < (bn == 128 ? c128 : c256)) bn = 192;
        grid = dim3(pt, (N + bn - 1) / bn, 1);
        // 256-wide tiles: a pair of CTAs on 256 x 256 (half the weight rows per SM and K-block) where that takes no more
        // rounds than single CTAs on 128 x 256.  FASTGGUF_PAIR=0 keeps the single-CTA kernel.
        static int pair_on = -1;
        if (pair_on < 0) { const char *e = getenv("FASTGGUF_PAIR"); pair_on = !(e && e[0] == '0'); }
        bool pair = false;
        if (pair_on && bn >= 192 && M > 128 && sms >= 2) {
            const long long tp = (long long)((M + 255) / 256) * ((N + bn - 1) / bn);
            const long long rounds_pair = (tp + sms / 2 - 1) / (sms / 2), rounds_one = ((bn == 256 ? t256 : t192) + sms - 1) / sms;
            pair = rounds_pair <= rounds_one;
        }
        if (force_splits == -2 && sms >= 2) { pair = true; if (bn < 192) bn = 256; }      // tests: the pair kernel at any size
        if (force_splits == -4 && sms >= 2 && epi != EPI_SILU_MUL) { pair = true; bn = 192; }      // tests: ... on 256 x 192 tiles
        if (pair) { grid = dim3((M + 255) / 256, (N + bn - 1) / bn, 1); bn = -bn; }
    }
    int kb_per_split = (total_kb + splits - 1) / splits;       // a split may be empty: it adds zeros
    grid.z = splits;
    CUtensorMap tmP, tmQ;
    int e = swap ? make_map(&tmP, W, N, K, ldw, BM) : make_map(&tmP, X, M, K, ldx, BM);
    if (e) return e;
    e = swap ? make_map(&tmQ, X, M, K, ldx, bn) : make_map(&tmQ, W, N, K, ldw, bn < 0 ? -bn / 2 : bn);
    if (e) return e;
    int esz = (epi == EPI_F32 || epi == EPI_ADD_F32) ? 4 : 2;
    int vec_ok = ((uintptr_t)out % 16 == 0) && ((size_t)ldc * esz % 16 == 0);
    if (ss_tiles_out) *ss_tiles_out = (int)grid.y * (bn < 0 && epi == EPI_ADD_F32 ? 2 : 1);
    GemmArgs a{out, M, N, K, ldc, kb_per_split, vec_ok, ss_in, ss_tiles, ss_size, ss_eps, norm_w, (bf16 *)xw_out, ss_out, epi, 0,
               g_test_skip_copy};
    switch (epi) {
    case EPI_BF16: return dispatch<EPI_BF16>(swap, bn, tmP, tmQ, a, grid, stream);
    case EPI_F32: return dispatch<EPI_F32>(swap, bn, tmP, tmQ, a, grid, stream);
    case EPI_ADD_F32: return dispatch<EPI_ADD_F32>(swap, bn, tmP, tmQ, a, grid, stream);
    case EPI_SILU_MUL: return dispatch<EPI_SILU_MUL>(swap, bn, tmP, tmQ, a, grid, stream);
    }
    return FG_ERR_BAD_DTYPE;
}

// For the test of the bounded waits: wait_limit_cycles > 0 sets how long a wait may last (0 restores the default of
// about a second; values below half a millisecond act as half a millisecond), and skip_copy != 0 makes the decode
// kernel's producer leave the first stage of every launch incomplete, so that its waits run out: the kernel then
// raises the error flag, frees its tensor memory and returns.  Never set outside a test.
extern "C" int fg_gemm_tc_test_hook(long long wait_limit_cycles, int skip_copy) {
    long long v = wait_limit_cycles > 0 ? wait_limit_cycles : WAIT_LIMIT_CYCLES;
    g_test_skip_copy = skip_copy ? 1 : 0;
    return (int)cudaMemcpyToSymbol(g_gemm_wait_limit, &v, sizeof v);
}

// The error flag of the pipelines: 0, or FG_ERR_PIPELINE << 8 | role.  Reading clears it.
extern "C" int fg_gemm_tc_error(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
    return v;
}
