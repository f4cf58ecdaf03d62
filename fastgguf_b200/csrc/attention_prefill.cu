// Prefill attention over the paged bf16 cache on the tensor cores: every sequence of the step
// brings one or more new tokens whose keys and values are already in the cache.
//
// Reference role: attn_rows for a prompt chunk (fastgguf.c:5022-5039): rows are (token, head of
// the group) pairs of one KV head, each attending to [start, its own position]; the whole chunk's
// K/V are in the cache, so causality inside the chunk is the per-row upper bound (:5030-5035).
//
// Grid (query tile, kv head x head chunk, sequence).  A CTA owns 16 rows a warp (128 rows with
// eight warps for head size 64, 64 rows with four warps for head size 128) = TQ consecutive new
// tokens x Gc query heads of one KV head (Gc = min(G, 16)), and walks the sequence's pages from
// the first page any row may see to the page of its last row.  All
// warps share each K/V page in shared memory (two stages, cp.async), so the query heads of a
// group reuse every load.  Scores, running max and sum are f32 (online softmax); P is rounded to
// bf16 for the PV product.  A row's keys are always visited in ascending page order, so its
// result does not depend on the other rows of the step.
#include "attention_mma.cuh"

template <int HD, int PF_WARPS>
__device__ __forceinline__ void load_page_cta(uint32_t sdst, const bf16 *src, int tid) {
    constexpr int CPR = HD / 8;
#pragma unroll
    for (int i = tid; i < PAGE * CPR; i += PF_WARPS * 32) {
        int r = i / CPR, c = i % CPR;
        cp_async16(sdst + r * (HD * 2) + ((c ^ (r & 7)) << 4), src + (size_t)r * HD + c * 8);
    }
}

template <int HD, int PF_WARPS>
__global__ void __launch_bounds__(PF_WARPS * 32, PF_WARPS == 8 ? 2 : 1)
attn_prefill_kernel(const bf16 *__restrict__ q, int ldq, bf16 *__restrict__ out, int ldo,
                    const int *__restrict__ cu_rows, const int *__restrict__ seq_start,
                    const int *__restrict__ block_table, int table_width,
                    const bf16 *__restrict__ k_pool, const bf16 *__restrict__ v_pool,
                    int KV, int G, float scale, int window) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int TILE_BYTES = PAGE * HD * 2;
    constexpr int PF_ROWS = PF_WARPS * 16;
    const int warp = warp_index(), lane = threadIdx.x & 31, tid = threadIdx.x;
    const int Gc = G < 16 ? G : 16;
    const int TQ = PF_ROWS / Gc;                       // new tokens per CTA tile
    const int chunks = (G + Gc - 1) / Gc;
    const int kvh = blockIdx.y / chunks, g0 = (blockIdx.y % chunks) * Gc;
    const int b = blockIdx.z;
    pdl_launch_dependents();
    pdl_wait();
    const int row0 = cu_rows[b], n_tok = cu_rows[b + 1] - row0, start = seq_start[b];
    const int q0 = (gridDim.x - 1 - blockIdx.x) * TQ;   // late tiles see the most keys: start them first
    if (q0 >= n_tok) return;
    const int tq = min(TQ, n_tok - q0);                // valid tokens in this tile
    const int *bt = block_table + (size_t)b * table_width;

    // rows of this thread: r = warp*16 + lane/4 (+8); token t = r / Gc, head g0 + r % Gc
    int t_[2], g_[2], hi[2], lo[2];
    bool valid[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        int r = warp * 16 + (lane >> 2) + 8 * i;
        t_[i] = r / Gc; g_[i] = g0 + r % Gc;
        valid[i] = t_[i] < tq && g_[i] < G;
        hi[i] = valid[i] ? start + q0 + t_[i] : -1;    // the row's own position; -1 masks everything
        lo[i] = (window > 0 && hi[i] - window + 1 > 0) ? hi[i] - window + 1 : 0;
    }
    // page range of the whole tile, and of this warp (to skip pages no row of the warp can see)
    const int tile_hi = start + q0 + tq - 1;
    const int tile_lo = (window > 0 && start + q0 - window + 1 > 0) ? start + q0 - window + 1 : 0;
    const int p_begin = tile_lo / PAGE, p_end = tile_hi / PAGE + 1;
    int warp_hi = max(hi[0], hi[1]), warp_min_hi = min(hi[0], hi[1]), warp_max_lo = max(lo[0], lo[1]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        warp_hi = max(warp_hi, __shfl_xor_sync(0xffffffffu, warp_hi, o));
        warp_min_hi = min(warp_min_hi, __shfl_xor_sync(0xffffffffu, warp_min_hi, o));   // -1 with an invalid row: always mask
        warp_max_lo = max(warp_max_lo, __shfl_xor_sync(0xffffffffu, warp_max_lo, o));
    }

    uint32_t qf[HD / 16][4];
    {
        const int c = (lane & 3) * 2;
#pragma unroll
        for (int kk = 0; kk < HD / 16; kk++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                int i = e & 1, k = kk * 16 + c + (e >> 1) * 8;
                qf[kk][e] = valid[i]
                    ? *(const uint32_t *)(q + (size_t)(row0 + q0 + t_[i]) * ldq + (size_t)(kvh * G + g_[i]) * HD + k) : 0u;
            }
    }
    float o[HD / 8][4];
#pragma unroll
    for (int d = 0; d < HD / 8; d++) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    const uint32_t s0 = smem_addr(smem);
    auto kaddr = [&](int st) { return s0 + st * 2 * TILE_BYTES; };
    auto vaddr = [&](int st) { return s0 + st * 2 * TILE_BYTES + TILE_BYTES; };
    {
        size_t base = ((size_t)bt[p_begin] * KV + kvh) * PAGE * HD;
        load_page_cta<HD, PF_WARPS>(kaddr(0), k_pool + base, tid);
        load_page_cta<HD, PF_WARPS>(vaddr(0), v_pool + base, tid);
        cp_async_commit();
    }
    for (int p = p_begin; p < p_end; p++) {
        const int st = (p - p_begin) & 1;
        if (p + 1 < p_end) {
            size_t base = ((size_t)bt[p + 1] * KV + kvh) * PAGE * HD;
            load_page_cta<HD, PF_WARPS>(kaddr(st ^ 1), k_pool + base, tid);
            load_page_cta<HD, PF_WARPS>(vaddr(st ^ 1), v_pool + base, tid);
        }
        cp_async_commit();
        cp_async_wait<1>();                    // page p has landed (p + 1 may be in flight)
        __syncthreads();
        if (p * PAGE <= warp_hi) {             // some row of this warp sees a key of the page
            float s[8][4];
#pragma unroll
            for (int j = 0; j < 8; j++) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
            qk_page<HD>(s, qf, kaddr(st), lane);
            // only pages that hold a row's own position (or a window's edge) need the mask
            if (p * PAGE + PAGE - 1 <= warp_min_hi && p * PAGE >= warp_max_lo)
                softmax_update<HD / 8, false>(s, o, m, l, scale * LOG2E, p * PAGE, lo, hi, lane);
            else
                softmax_update<HD / 8, true>(s, o, m, l, scale * LOG2E, p * PAGE, lo, hi, lane);
            pv_page<HD>(o, s, vaddr(st), lane);
        }
        __syncthreads();                       // the stage is overwritten by the load after next
    }
    cp_async_wait<0>();
    const int c = (lane & 3) * 2;
#pragma unroll
    for (int i = 0; i < 2; i++) {
        if (!valid[i]) continue;
        float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
        bf16 *orow = out + (size_t)(row0 + q0 + t_[i]) * ldo + (size_t)(kvh * G + g_[i]) * HD;
#pragma unroll
        for (int d = 0; d < HD / 8; d++)
            *(uint32_t *)(orow + d * 8 + c) = pack_bf16(o[d][2 * i] * inv, o[d][2 * i + 1] * inv);
    }
}

template <int HD, int PF_WARPS>
static int launch_prefill(const void *q, int ldq, void *out, int ldo, const int *cu_rows, const int *seq_start,
                          const int *block_table, int table_width, const void *k_pool, const void *v_pool,
                          int n_seq, int max_new, int H, int KV, float scale, int window, cudaStream_t stream) {
    constexpr int smem = 2 * 2 * PAGE * HD * 2;
    static FgPerDevice configured;
    if (fg_needs_setup(configured)) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<HD, PF_WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
    }
    int G = H / KV, Gc = G < 16 ? G : 16, TQ = PF_WARPS * 16 / Gc;
    dim3 grid((max_new + TQ - 1) / TQ, KV * ((G + Gc - 1) / Gc), n_seq);
    return fg_launch(attn_prefill_kernel<HD, PF_WARPS>, grid, dim3(PF_WARPS * 32), (size_t)smem, stream, (const bf16 *)q, ldq, (bf16 *)out, ldo, cu_rows,
        seq_start, block_table, table_width, (const bf16 *)k_pool, (const bf16 *)v_pool, KV, G, scale, window);
}

// q: [rows, ldq] bf16 rows of all sequences one after another (cu_rows[b] = first row of sequence b,
// seq_start[b] = its length before the step); pools [pages, KV, 64, HD] bf16; out [rows, ldo] bf16.
// max_new: most rows any sequence brings.  Takes HD 64 and 128 and pages of 64.
extern "C" int fg_attention_prefill(const void *q, int ldq, void *out, int ldo, const int *cu_rows,
                                    const int *seq_start, const int *block_table, int table_width,
                                    const void *k_pool, const void *v_pool, int n_seq, int max_new, int H, int KV,
                                    int hd, int page_size, float scale, int window, cudaStream_t stream) {
    if (n_seq <= 0 || max_new <= 0) return 0;
    if (page_size != PAGE || H % KV || n_seq > 65535 || ldq % 2 || ldo % 2 || ((uintptr_t)q & 3) || ((uintptr_t)out & 3))
        return FG_ERR_BAD_SIZE;
    if (hd == 64) return launch_prefill<64, 8>(q, ldq, out, ldo, cu_rows, seq_start, block_table, table_width, k_pool, v_pool, n_seq, max_new, H, KV, scale, window, stream);
    if (hd == 128) return launch_prefill<128, 4>(q, ldq, out, ldo, cu_rows, seq_start, block_table, table_width, k_pool, v_pool, n_seq, max_new, H, KV, scale, window, stream);
    return FG_ERR_BAD_SIZE;
}
