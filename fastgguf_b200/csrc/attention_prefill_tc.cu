// Prefill attention over the paged bf16 cache on the 5th-generation tensor cores (tcgen05):
// S = Q K^T and O = P V run as 128-row MMAs with accumulators in tensor memory, K/V pages arrive
// by TMA, and the softmax works one thread per row straight out of tensor memory.
//
// Reference role and formulas: as attention_prefill.cu (fastgguf.c:5022-5039, :3273-3326).
//
// Grid (kv head x head chunk, query tile, sequence): CTAs are dispatched x first, so the tiles that see the most
// keys (the late ones, y = 0) all start before any light one and the tail of the kernel is short.  A CTA owns 128 rows = TQ consecutive new
// tokens x Gc query heads of one KV head (Gc = min(G, 16), row r = token r / Gc, head r % Gc) and
// walks the sequence's pages so that two CTAs fit on an SM and the softmax of one runs under the MMAs of the other.
// Three forms (template parameters; fg_attention_prefill_tc says which runs when):
//   one score tile     two pages (128 keys) an iteration at head size 64, one (64 keys) at 128; S, softmax and P V of an
//                      iteration follow one another
//   PIPE               one page an iteration, TWO score tiles in tensor memory and two P tiles in shared memory: S of
//                      iteration j + 1 is computed during the softmax of iteration j, P V of iteration j during the
//                      softmax of j + 1 (the form that runs by default)
//   PIPE + PP          head size 64: two sets of softmax warps (2-5 and 6-9) take the iterations in turn, each with its
//                      own score tile, P tile, O accumulator, running maximum and sum; the two partial results of a row
//                      are combined at the end (long prompts)
//
//   warp 0             TMA (one elected lane issues): the K tile and the V tile of an iteration (128B
//                      swizzle); the next K tile is fetched as soon as S has consumed the current one,
//                      the next V tile after P V
//   warp 1             MMA (one elected lane issues): S = Q K^T (128 x KEYS x HD), then, once P is in shared memory,
//                      O += P V (128 x HD x KEYS) into the same tensor-memory accumulator, iteration after
//                      iteration; V is the MN-major operand (its rows are keys)
//   warps 2-5          thread = row: read S from tensor memory, scale, mask, running max and sum in
//                      f32 (base-2 exponent), write P as bf16 into swizzled shared memory.  Probabilities are
//                      taken relative to a base that may lag the row's true maximum (see below); only when a
//                      row's base has to move does its warp rescale its rows of O in tensor memory
//                      (tcgen05.ld / st), after the MMAs before have finished.  At the end the row is read
//                      once, divided by the sum and stored.
//
// Every mbarrier wait is bounded (error flag, tensor memory freed, copies in flight awaited).
#include <cuda.h>
#include <climits>
#include "common.cuh"

#define FG_ERR_PIPELINE 10003
#define FG_ERR_TENSORMAP 10004
#define PAGE 64
#define ROWS 128
#define ATT_THREADS(PP) ((PP) ? 320 : 192)      // producer warp, issuer warp, four softmax warps (eight: PP)
#define WAIT_LIMIT_CYCLES 2000000000ll
#define WAIT_SHORT_CYCLES 1000000ll
#define LOG2E 1.4426950408889634f

__device__ int g_attn_error = 0;
// how long a wait may last, in SM cycles; a variable so that a test can shorten it (fg_attention_prefill_tc_test_hook)
__device__ long long g_attn_wait_limit = WAIT_LIMIT_CYCLES;
static int g_test_skip_copy = 0;
static int g_variant = -2;             // -2: not read yet; -1: chosen by shape; else bit 0 / bit 1 = two score tiles at head size 64 / 128

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    long long t0 = clock64();
    for (;;) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        const long long waited = clock64() - t0;
        if (waited > WAIT_SHORT_CYCLES) {
            // once a wait has run out somewhere, every later wait gives up after a short time: a broken pipeline
            // costs milliseconds for the kernels that follow, not a second per wait
            if (*(volatile int *)&g_attn_error != 0) return false;
            if (waited > *(volatile long long *)&g_attn_wait_limit) return false;
        }
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
// the same load without the wait: the registers hold the values only after tc_ld_wait()
__device__ __forceinline__ void tc_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_st32(uint32_t taddr, const float (&v)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                 "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                 ::"r"(taddr),
                   "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
                   "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
                   "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
                   "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
                   "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
                   "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
                   "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
                   "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
                 : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// K-major operand tile (rows of 128 B, 8-row groups 1024 B apart), 128-byte swizzle
__device__ __forceinline__ uint64_t desc_k_major(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major operand tile: rows of 128 B hold 64 consecutive N elements of one k; groups of 8 k are
// 1024 B apart (stride offset); blocks of 64 N elements are `mn_block_bytes` apart (leading offset)
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t saddr, uint32_t mn_block_bytes) {
    return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)((mn_block_bytes >> 4) & 0x3FFF) << 16) |
           ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// instruction descriptor: bf16 x bf16 -> f32, M x N; b_mn_major: B's rows are k (keys)
__device__ __forceinline__ uint32_t make_idesc(int M, int N, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) |
           ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void raise_error(int role) { atomicCAS(&g_attn_error, 0, (FG_ERR_PIPELINE << 8) | role); }

// One 32-key chunk of a row's scores: p = 2^(v * scale - base) as bf16 pairs into w, their sum added to `acc`, the
// largest raw score kept in `mx_raw` (the scale is positive, so the largest scaled score is mx_raw * scale).
// MASKED: keys outside [lo, hi] count as -infinity.
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
template <bool MASKED>
__device__ __forceinline__ void softmax_chunk(const float (&v)[32], int key, int lo, int hi, float scale, float neg_base,
                                              float &mx_raw, float &acc, uint32_t (&w)[16]) {
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
        float a = v[i], b = v[i + 1];
        if (MASKED) {
            if (key + i < lo || key + i > hi) a = -INFINITY;
            if (key + i + 1 < lo || key + i + 1 > hi) b = -INFINITY;
        }
        mx_raw = max3(mx_raw, a, b);
        const float p0 = ex2(fmaf(a, scale, neg_base)), p1 = ex2(fmaf(b, scale, neg_base));
        acc += p0 + p1;
        __nv_bfloat162 t = __floats2bfloat162_rn(p0, p1);
        w[i >> 1] = *(uint32_t *)&t;
    }
}

// PIPE: 64 keys an iteration with TWO score tiles in tensor memory and two P tiles in shared memory, so that S of
// iteration j + 1 is computed while the softmax of iteration j runs and P V of iteration j while the softmax of j + 1
// runs: the iterations of a CTA no longer add S + softmax + P V, and the heaviest tile of a long sequence (which bounds
// the kernel) takes about the time of its softmaxes.
// PP (with PIPE, head size 64): two sets of four softmax warps take the iterations in turn - set 0 the even ones with
// score tile, P tile and O accumulator 0, set 1 the odd ones with those of index 1 - each with a running maximum and sum
// of its own, so that nothing orders the softmax of one iteration behind the one before it; the two partial results
// of a row (O, maximum, sum) are combined at the end.  Four softmax streams an SM instead of two keep the exponential
// unit busier.
template <int HD, bool PIPE, bool PP>
__global__ void __launch_bounds__(ATT_THREADS(PP), 2)              // two CTAs share an SM and overlap
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                       const bf16 *__restrict__ q, int ldq, bf16 *__restrict__ out, int ldo,
                       const int *__restrict__ cu_rows, const int *__restrict__ seq_start,
                       const int *__restrict__ block_table, int table_width, int KV, int G, float scale_log2, int window,
                       int test_skip_copy) {
    constexpr int CH = HD / 64;                        // 64-wide chunks of the head dimension
    constexpr int KEYS = PIPE ? 64 : (HD > 64 ? 64 : 128), NPG = KEYS / PAGE;      // keys and pages per iteration
    constexpr int NS = PIPE ? 2 : 1;                   // score tiles in tensor memory, P tiles in shared memory
    constexpr int Q_BYTES = ROWS * HD * 2, KV_TILE = KEYS * HD * 2, P_TILE = ROWS * KEYS * 2;
    constexpr uint32_t TMEM_COLS = 256;                // S tiles: columns 0..NS*KEYS-1, O: the HD columns after them (PP: twice)
    constexpr uint32_t O_COL = NS * KEYS;
    static_assert(!PP || (PIPE && O_COL + 2 * HD <= TMEM_COLS), "two accumulators need two score tiles and head size 64");

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t bars[10];
    __shared__ float x_ml[2][ROWS][2];                 // PP: a set's final maximum and sum of each row
    __shared__ uint32_t tmem_base_s;

    const int warp = warp_index(), lane = threadIdx.x & 31;
    const int Gc = G < 16 ? G : 16, TQ = ROWS / Gc, chunks = (G + Gc - 1) / Gc;
    const int kvh = blockIdx.x / chunks, g0 = (blockIdx.x % chunks) * Gc;
    const int b = blockIdx.z;
    const uint32_t qs = smem_u32(smem), kt = qs + Q_BYTES, vt = kt + KV_TILE, ps = vt + KV_TILE;
    const uint32_t k_full = smem_u32(&bars[0]), k_empty = smem_u32(&bars[1]);
    const uint32_t v_full = smem_u32(&bars[2]), v_empty = smem_u32(&bars[3]);
    const uint32_t s_full = smem_u32(&bars[4]), p_full = smem_u32(&bars[6]), o_full = smem_u32(&bars[8]);     // s_full, p_full: one per tile
    // iteration j uses score / P tile j % NS, for the (j / NS)-th time
    auto tile_of = [](int j) { return PIPE ? (j & 1) : 0; };
    auto use_parity = [](int j) { return (uint32_t)(PIPE ? (j >> 1) & 1 : j & 1); };

    if (threadIdx.x == 0) {
        mbar_init(k_full, 1); mbar_init(k_empty, 1); mbar_init(v_full, 1); mbar_init(v_empty, 1);
        mbar_init(s_full, 1); mbar_init(s_full + 8, 1); mbar_init(p_full, ROWS); mbar_init(p_full + 8, ROWS); mbar_init(o_full, 1); mbar_init(o_full + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    pdl_launch_dependents();
    pdl_wait();                                        // q and the cache come from the kernels before
    const int row0 = cu_rows[b], n_tok = cu_rows[b + 1] - row0, start = seq_start[b];
    const int q0 = (gridDim.y - 1 - blockIdx.y) * TQ;  // late tiles see the most keys: start them first
    const bool active = q0 < n_tok;                    // a CTA past the sequence's tokens only sets up and leaves
    const int tq = active ? min(TQ, n_tok - q0) : 0;
    const int tile_hi = start + q0 + tq - 1;
    const int tile_lo = (window > 0 && start + q0 - window + 1 > 0) ? start + q0 - window + 1 : 0;
    const int p_begin = tile_lo / PAGE, p_end = tile_hi / PAGE + 1;
    const int n_iter = active ? (p_end - p_begin + NPG - 1) / NPG : 0;
    const int *bt = block_table + (size_t)b * table_width;

    // ---- Q tile -> shared memory, swizzled like a TMA tile (rows past the valid ones are zero)
    int t_row = 0, g_row = 0, hi = -1, lo = 0;
    bool valid = false;
    if (warp >= 2) {
        const int r = (warp & 3) * 32 + lane;
        t_row = r / Gc; g_row = g0 + r % Gc;
        valid = t_row < tq && g_row < G;
        // A row past the tile's tokens or heads has a zero query and is never stored.  It sees every key, so that it
        // neither asks for the masked loop nor, with a maximum that stays at minus infinity, for the second pass in
        // every iteration of its warp (group sizes that do not divide 128 leave such rows in every tile).
        hi = valid ? start + q0 + t_row : INT_MAX;
        lo = !valid ? INT_MIN : (window > 0 && hi - window + 1 > 0) ? hi - window + 1 : 0;
        const bf16 *src = q + (size_t)(row0 + q0 + t_row) * ldq + (size_t)(kvh * G + g_row) * HD;
#pragma unroll
        for (int c = (warp < 6 ? 0 : HD / 8); c < HD / 8; c++) {       // (PP: the first set brings the tile)
            uint4 v = valid ? *(const uint4 *)(src + c * 8) : make_uint4(0, 0, 0, 0);
            uint32_t dst = qs + (c >> 3) * (ROWS * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        // the whole warp walks the pages and waits; one elected lane issues the copies
        // order: K(0), then for every iteration K(j + 1) before V(j) - K(j + 1) may go as soon as S(j) has read the K
        // tile, V(j) only when P V of iteration j - 1 has read the V tile, which is later
        int k_issued = 0, v_issued = 0;
        auto page_rows = [&](int j, int (&y)[NPG]) {
            for (int h = 0; h < NPG; h++)
                y[h] = (bt[min(p_begin + NPG * j + h, p_end - 1)] * KV + kvh) * PAGE;   // a page past the end is masked anyway
        };
        auto load_k = [&](int j) {
            int y[NPG];
            page_rows(j, y);
            if (!__all_sync(0xffffffffu, mbar_wait(k_empty, (j & 1) ^ 1))) { raise_error(1); return false; }
            if (elect_one()) {
                mbar_expect_tx(k_full, KV_TILE);
                // (a test may ask for the first K tile to stay incomplete: its barrier never fires and every wait runs out)
                if (!(test_skip_copy && j == 0))
                    for (int h = 0; h < NPG; h++)
                        for (int c = 0; c < CH; c++) tma_load_2d(kt + c * (KEYS * 128) + h * (PAGE * 128), &tmK, c * 64, y[h], k_full);
            }
            __syncwarp();
            k_issued = j + 1;
            return true;
        };
        bool ok = n_iter > 0 && load_k(0);
        for (int j = 0; j < n_iter && ok; j++) {
            if (j + 1 < n_iter && !load_k(j + 1)) break;
            int y[NPG];
            page_rows(j, y);
            if (!__all_sync(0xffffffffu, mbar_wait(v_empty, (j & 1) ^ 1))) { raise_error(1); break; }
            if (elect_one()) {
                mbar_expect_tx(v_full, KV_TILE);
                for (int h = 0; h < NPG; h++)
                    for (int c = 0; c < CH; c++) tma_load_2d(vt + c * (KEYS * 128) + h * (PAGE * 128), &tmV, c * 64, y[h], v_full);
            }
            __syncwarp();
            v_issued = j + 1;
        }
        if (k_issued) mbar_wait(k_full, (k_issued - 1) & 1);      // copies in flight land before the CTA exits
        if (v_issued) mbar_wait(v_full, (v_issued - 1) & 1);
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // the whole warp walks the iterations and waits; one elected lane issues
        if (n_iter > 0) {
            const uint32_t idesc_s = make_idesc(ROWS, KEYS, 0), idesc_o = make_idesc(ROWS, HD, 1);
            auto issue_s = [&](int j) {
                if (!__all_sync(0xffffffffu, mbar_wait(k_full, j & 1))) { raise_error(2); return false; }
                tc_fence_after();
                if (elect_one()) {
#pragma unroll
                    for (int ks = 0; ks < HD / 16; ks++) {
                        // 64-wide chunk ks / 4 of the head dimension (ROWS rows of Q, KEYS rows of K), 32 B inside its swizzle row
                        const uint32_t qoff = (ks >> 2) * (ROWS * 128) + (ks & 3) * 32, koff = (ks >> 2) * (KEYS * 128) + (ks & 3) * 32;
                        tc_mma_bf16(tmem_base + tile_of(j) * KEYS, desc_k_major(qs + qoff), desc_k_major(kt + koff), idesc_s, ks != 0);
                    }
                    tc_commit(s_full + 8 * tile_of(j));
                    tc_commit(k_empty);              // the K tile is free once S is complete
                }
                __syncwarp();
                return true;
            };
            bool ok = issue_s(0);
            if (PIPE && ok && n_iter > 1) ok = issue_s(1);         // the second score tile is free from the start
            for (int j = 0; j < n_iter && ok; j++) {
                if (!__all_sync(0xffffffffu, mbar_wait(p_full + 8 * tile_of(j), use_parity(j)))) { raise_error(3); break; }
                if (!__all_sync(0xffffffffu, mbar_wait(v_full, j & 1))) { raise_error(2); break; }
                tc_fence_after();
                if (elect_one()) {
#pragma unroll
                    for (int ks = 0; ks < KEYS / 16; ks++) {
                        // A = P: 64-key chunk ks / 4, 32 B inside its swizzle row; B = V: 16 keys = two 8-key groups
                        uint64_t adesc = desc_k_major(ps + tile_of(j) * P_TILE + (ks >> 2) * (ROWS * 128) + (ks & 3) * 32);
                        uint64_t bdesc = desc_mn_major(vt + ks * 2048, KEYS * 128);
                        // O accumulates over the iterations (PP: over those of the iteration's set, in that set's columns)
                        if (PP) tc_mma_bf16(tmem_base + O_COL + (j & 1) * HD, adesc, bdesc, idesc_o, ((j >> 1) | ks) != 0);
                        else tc_mma_bf16(tmem_base + O_COL, adesc, bdesc, idesc_o, (j | ks) != 0);
                    }
                    tc_commit(PP ? o_full + 8 * (j & 1) : o_full);
                    tc_commit(v_empty);
                }
                __syncwarp();
                // the score tile that iteration j + NS will fill is free: every row has read S(j) (p_full above)
                if (j + NS < n_iter) ok = issue_s(j + NS);
            }
        }
    } else {
        // ------------------------------------------------------------ softmax, one thread per row (PP: and set)
        const int lg = warp & 3, r = lg * 32 + lane, set = PP ? (warp - 2) >> 2 : 0;
        const int step = PP ? 2 : 1;                    // this thread's iterations: set, set + step, ...
        const uint32_t trow = tmem_base + ((uint32_t)(lg * 32) << 16);
        const uint32_t ocol = O_COL + set * HD, my_o_full = o_full + 8 * set;
        // the wait for the P V of this thread's previous iteration names a phase by its parity: PP counts the set's own
        auto o_parity = [&](int j_prev) { return (uint32_t)((PP ? j_prev >> 1 : j_prev) & 1); };
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        int j_last = -1;
        for (int j = set; j < n_iter; j += step) {
            const int key0 = (p_begin + NPG * j) * PAGE;
            const bool masked = key0 + KEYS - 1 > hi || key0 < lo;
            if (!mbar_wait(s_full + 8 * tile_of(j), use_parity(j))) { raise_error(4); ok = false; break; }
            tc_fence_after();
            const uint32_t srow = trow + tile_of(j) * KEYS, pj = ps + tile_of(j) * P_TILE;
            // One pass when the running base is still good: probabilities relative to m, which may lag the
            // true maximum by up to 2^8 (harmless in f32 / bf16, and the same factor is in l and in O).  A row
            // whose new scores exceed that makes its warp redo the tile in two passes with the true maximum.
            float corr = 1.f, sum = 0.f;
            bool redo = !__all_sync(0xffffffffu, m != -INFINITY);
            // a warp whose 32 rows all see every key of this tile runs the loops without the mask's compares
            const bool any_masked = __any_sync(0xffffffffu, masked);
            // probabilities of the tile relative to `base`, written to the P tile; the largest RAW score in mx
            auto pass = [&](float base, float &mx_raw, float &acc) {
                const float neg_base = -base;
                auto chunk = [&](int c, const float (&v)[32]) {
                    uint32_t w[16];
                    if (any_masked) softmax_chunk<true>(v, key0 + c * 32, masked ? lo : INT_MIN, masked ? hi : INT_MAX, scale_log2, neg_base, mx_raw, acc, w);
                    else softmax_chunk<false>(v, 0, 0, 0, scale_log2, neg_base, mx_raw, acc, w);
                    // 32 keys = four 16-byte chunks of this row, in the 64-key chunk c / 2
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        int cc = (c & 1) * 4 + k;
                        uint32_t dst = pj + (c >> 1) * (ROWS * 128) + r * 128 + ((cc ^ (r & 7)) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                     ::"r"(dst), "r"(w[4 * k]), "r"(w[4 * k + 1]), "r"(w[4 * k + 2]), "r"(w[4 * k + 3]) : "memory");
                    }
                };
                if (PIPE && !PP) {
                    // The scores of the second 32 keys are on their way from tensor memory while the first 32 are worked
                    // on: 4 to 6 % off prompts of 4,096 tokens and more at head size 64 (32,768 tokens: 6.53 -> 6.14 ms),
                    // nothing at 128.  With one score tile (four chunks an iteration) it gains nothing.  (PP: 320 threads
                    // and two CTAs an SM leave no registers for it.)
                    uint32_t raw[2][32];
                    tc_ld32_issue(srow, raw[0]);
#pragma unroll
                    for (int c = 0; c < KEYS / 32; c++) {
                        tc_ld_wait();
                        float v[32];
#pragma unroll
                        for (int i = 0; i < 32; i++) v[i] = __uint_as_float(raw[c & 1][i]);
                        if (c + 1 < KEYS / 32) tc_ld32_issue(srow + (c + 1) * 32, raw[(c + 1) & 1]);
                        chunk(c, v);
                    }
                } else {
#pragma unroll 1
                    for (int c = 0; c < KEYS / 32; c++) {
                        float v[32];
                        tc_ld32(srow + c * 32, v);
                        chunk(c, v);
                    }
                }
            };
            if (!redo) {
                float mx_raw = -INFINITY;
                pass(m, mx_raw, sum);
                redo = __any_sync(0xffffffffu, mx_raw * scale_log2 > m + 8.0f);
            }
            float m_keep = m;
            if (redo) {
                float mx_raw = -INFINITY;
#pragma unroll 1
                for (int c = 0; c < KEYS / 32; c++) {
                    float v[32];
                    tc_ld32(srow + c * 32, v);
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        int key = key0 + c * 32 + i;
                        float x = v[i];
                        if (masked && (key < lo || key > hi)) x = -INFINITY;
                        mx_raw = fmaxf(mx_raw, x);
                    }
                }
                const float m_new = fmaxf(m, mx_raw * scale_log2);            // the scale is positive
                corr = m == -INFINITY ? 1.f : ex2(m - m_new);                 // m_new >= m; nothing seen yet: keep zeros
                const float base = m_new == -INFINITY ? 0.f : m_new;
                sum = 0.f;
                float unused = -INFINITY;
                pass(base, unused, sum);
                m_keep = m_new;
            }
            l = l * corr + sum;
            m = m_keep;
            // With two score tiles a row could run two P V ahead of what it has seen complete, and a wait names a phase
            // by its parity only: every row watches every P V (PP: of its set) finish, in order (the one before this
            // iteration's is long done when the softmax of this iteration ends, so this costs nothing).
            if (PIPE && j_last >= 0 && !mbar_wait(my_o_full, o_parity(j_last))) { raise_error(5); ok = false; break; }
            if (j_last >= 0 && __any_sync(0xffffffffu, corr != 1.f)) {
                // a base moved: the rows of O so far are rescaled in tensor memory, once the MMAs before this
                // iteration have finished (the next P V is not issued before every row has arrived below)
                if (!PIPE && !mbar_wait(my_o_full, o_parity(j_last))) { raise_error(5); ok = false; break; }
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < HD / 32; c++) {
                    float v[32];
                    tc_ld32(trow + ocol + c * 32, v);
#pragma unroll
                    for (int i = 0; i < 32; i++) v[i] *= corr;
                    tc_st32(trow + ocol + c * 32, v);
                }
            }
            tc_fence_before();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(p_full + 8 * tile_of(j));
            j_last = j;
        }
        if (ok && j_last >= 0 && !mbar_wait(my_o_full, o_parity(j_last))) { raise_error(5); ok = false; }
        float w_own = 1.f, w_other = 0.f;
        const int n_other = PP ? (n_iter + set) / 2 : 0;               // iterations of the other set: (n + 1) / 2 even ones, n / 2 odd ones
        if (PP) {
            // The other set's last P V: complete or one behind when this set's is (the MMAs run in iteration order), so
            // the parity names the right phase.  Then the two sets exchange each row's maximum and sum.
            if (ok && n_other > 0 && !mbar_wait(o_full + 8 * (set ^ 1), (uint32_t)((n_other - 1) & 1))) { raise_error(5); ok = false; }
            x_ml[set][r][0] = m; x_ml[set][r][1] = l;
            asm volatile("bar.sync %0, 64;" ::"r"(1 + lg) : "memory");       // the two warps of these 32 rows
            const float m2 = x_ml[set ^ 1][r][0], l2 = x_ml[set ^ 1][r][1], mm = fmaxf(m, m2);
            w_own = m == -INFINITY ? 0.f : ex2(m - mm);
            w_other = m2 == -INFINITY ? 0.f : ex2(m2 - mm);
            l = l * w_own + l2 * w_other;
        }
        tc_fence_after();
        if (n_iter > 0 && __all_sync(0xffffffffu, ok)) {           // the tensor-memory loads are warp-wide: every lane takes part
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            bf16 *dst = out + (size_t)(row0 + q0 + t_row) * ldo + (size_t)(kvh * G + g_row) * HD;
            // (PP: each set stores half of the row's columns, from both accumulators)
#pragma unroll 1
            for (int c = PP ? set * (HD / 64) : 0; c < (PP ? (set + 1) * (HD / 64) : HD / 32); c++) {
                float v[32];
                if (!PP) tc_ld32(trow + O_COL + c * 32, v);
                else {
                    float a[32], b2[32];
                    tc_ld32(trow + O_COL + set * HD + c * 32, a);              // this set's accumulator (set 0 always has one)
                    const bool have_own = set == 0 || n_iter > 1, have_other = n_other > 0;
                    if (have_other) tc_ld32(trow + O_COL + (set ^ 1) * HD + c * 32, b2);
#pragma unroll
                    for (int i = 0; i < 32; i++) v[i] = (have_own ? a[i] * w_own : 0.f) + (have_other ? b2[i] * w_other : 0.f);
                }
                if (!valid) continue;
#pragma unroll
                for (int k8 = 0; k8 < 4; k8++) {
                    uint32_t w[4];
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        __nv_bfloat162 t = __floats2bfloat162_rn(v[k8 * 8 + 2 * k] * inv, v[k8 * 8 + 2 * k + 1] * inv);
                        w[k] = *(uint32_t *)&t;
                    }
                    *(uint4 *)(dst + c * 32 + k8 * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
        }
    }
    tc_fence_before();
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

// a page pool [pages * KV * 64 rows, hd] bf16 in boxes of 64 rows x 64 elements, 128-byte swizzle
static int pool_map(CUtensorMap *map, const void *pool, long long rows, int hd) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return FG_ERR_TENSORMAP;
    cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
    cuuint32_t box[2] = {64, PAGE};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void *)pool, dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : FG_ERR_TENSORMAP;
}

template <int HD, bool PIPE, bool PP>
static int launch_tc(const CUtensorMap &tmK, const CUtensorMap &tmV, const void *q, int ldq, void *out, int ldo,
                     const int *cu_rows, const int *seq_start, const int *block_table, int table_width, int n_seq,
                     int max_new, int H, int KV, float scale, int window, cudaStream_t stream) {
    constexpr int KEYS = PIPE ? 64 : (HD > 64 ? 64 : 128);
    constexpr int smem = ROWS * HD * 2 + 2 * KEYS * HD * 2 + (PIPE ? 2 : 1) * ROWS * KEYS * 2 + 1024;
    // the attributes belong to the function on ONE device: set them once on every device that launches
    static bool configured[64] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FG_ERR_BAD_SIZE;
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD, PIPE, PP>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        cudaFuncSetAttribute(attn_prefill_tc_kernel<HD, PIPE, PP>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        configured[dev] = true;
    }
    int G = H / KV, Gc = G < 16 ? G : 16, TQ = ROWS / Gc;
    dim3 grid(KV * ((G + Gc - 1) / Gc), (max_new + TQ - 1) / TQ, n_seq);
    return fg_launch(attn_prefill_tc_kernel<HD, PIPE, PP>, grid, dim3(ATT_THREADS(PP)), (size_t)smem, stream, tmK, tmV, (const bf16 *)q, ldq,
                     (bf16 *)out, ldo, cu_rows, seq_start, block_table, table_width, KV, G, scale * LOG2E, window, g_test_skip_copy);
}

// Arguments as fg_attention_prefill, plus the number of pages in the pools.  Takes HD 64 and 128.
extern "C" int fg_attention_prefill_tc(const void *q, int ldq, void *out, int ldo, const int *cu_rows,
                                       const int *seq_start, const int *block_table, int table_width,
                                       const void *k_pool, const void *v_pool, int n_pages, int n_seq, int max_new,
                                       int H, int KV, int hd, int page_size, float scale, int window,
                                       cudaStream_t stream) {
    if (n_seq <= 0 || max_new <= 0) return 0;
    if (page_size != PAGE || H % KV || n_seq > 65535 || ldq % 8 || ldo % 8 || ((uintptr_t)q & 15) || ((uintptr_t)out & 15) ||
        ((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15) || (hd != 64 && hd != 128))
        return FG_ERR_BAD_SIZE;
    CUtensorMap tmK, tmV;
    long long rows = (long long)n_pages * KV * PAGE;
    int e = pool_map(&tmK, k_pool, rows, hd);
    if (e) return e;
    e = pool_map(&tmV, v_pool, rows, hd);
    if (e) return e;
    // Which form runs.  Two score tiles (S of iteration j + 1 under the softmax of iteration j, P V of iteration j under
    // the softmax of j + 1): always - at head size 128 it took a fifth off the kernel (3B shapes, 2,048 tokens: 81 -> 62
    // us a layer); at head size 64, 64 keys an iteration instead of 128, 38 against 43 us on one prompt of 2,048 tokens,
    // 6.16 against 6.68 ms at 32,768, 283 against 312 us on eight prompts of 2,048.  Two sets of softmax warps at head
    // size 64: from 3,072 rows of new tokens on (3,000 tokens: 70 against 73 us; 32,768: 5.78 against 6.16 ms; one
    // prompt of 2,048: 39.5 against 38.2).  FASTGGUF_ATTN_PIPE or fg_attention_prefill_tc_variant override (bit 0 / 1:
    // two score tiles at head size 64 / 128; bit 2: two softmax sets; negative: this rule); the tests run every form.
    if (g_variant == -2) { const char *e = getenv("FASTGGUF_ATTN_PIPE"); g_variant = e ? atoi(e) : -1; }
    const bool pipe = g_variant >= 0 ? ((g_variant >> (hd == 64 ? 0 : 1)) & 1) != 0 : true;
    const bool pp = hd == 64 && pipe && (g_variant >= 0 ? (g_variant & 4) != 0 : (long long)n_seq * max_new >= 3072);
#define TC_RUN(HD, PIPE, PP) launch_tc<HD, PIPE, PP>(tmK, tmV, q, ldq, out, ldo, cu_rows, seq_start, block_table, table_width, \
                                                     n_seq, max_new, H, KV, scale, window, stream)
    if (hd == 64) return pipe ? (pp ? TC_RUN(64, true, true) : TC_RUN(64, true, false)) : TC_RUN(64, false, false);
    return pipe ? TC_RUN(128, true, false) : TC_RUN(128, false, false);
#undef TC_RUN
}

// For the test of the bounded waits: wait_limit_cycles > 0 sets how long a wait may last (0 restores the default of
// about a second; values below half a millisecond act as half a millisecond), and skip_copy != 0 makes the producer
// leave the first K tile of every CTA incomplete, so that the waits run out: the kernel then raises the error flag,
// frees its tensor memory and returns.  Never set outside a test.
extern "C" int fg_attention_prefill_tc_test_hook(long long wait_limit_cycles, int skip_copy) {
    long long v = wait_limit_cycles > 0 ? wait_limit_cycles : WAIT_LIMIT_CYCLES;
    g_test_skip_copy = skip_copy ? 1 : 0;
    return (int)cudaMemcpyToSymbol(g_attn_wait_limit, &v, sizeof v);
}

// Which variant runs: see fg_attention_prefill_tc.  Negative: chosen by head size and step shape (the default).
extern "C" int fg_attention_prefill_tc_variant(int bits) {
    g_variant = bits < 0 ? -1 : (bits & 7);
    return 0;
}

extern "C" int fg_attention_prefill_tc_error(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_attn_error, &zero, sizeof(int));
    return v;
}
