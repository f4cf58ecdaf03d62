// Decode attention over the paged bf16 cache on the tensor cores: one new token per sequence.
//
// Reference role: attn_rows for one token (fastgguf.c:4769-4786, :3273-3326): the query heads
// of one KV head share every K/V load (the reference's "up to 4 query rows sharing one KV head",
// :3268-3272).  Formulas as in attention_generic.cu.
//
// Grid (split, kv head x head chunk, sequence).  The pages of a sequence are divided evenly
// among `n_splits` CTAs, so one long sequence fills the GPU as well as many short ones; inside a
// CTA four warps take pages round-robin, each with K and V buffers of its own (one K and one V
// load always in flight), and merge their running (max, sum, O) through shared memory.  With
// n_splits > 1 the CTAs of a sequence and KV head either form a thread-block cluster (2, 4 or 8
// splits) and merge their partial (O, max, sum) through distributed shared memory, or (more
// splits, very long contexts) write them to scratch memory for a second kernel to merge.
//
// The merge inside a cluster: CTA r owns the slice [r * HD / S, (r + 1) * HD / S) of the head dimension.  Every
// warp that read pages pushes its running (max, sum) to all CTAs and the slices of its O to their owners
// (st.shared::cluster), one cluster barrier makes the pushes visible, and each owner combines the up to 4 S
// partial results of its slice in (split, warp) order from its own shared memory and writes the output.
#include "attention_mma.cuh"

#define DEC_WARPS 4

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// two floats to the same shared-memory offset in the CTA of rank `rank` of this cluster (p 8-byte aligned)
__device__ __forceinline__ void st_dsmem2(const float *p, int rank, float a, float b) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_addr(p)), "r"(rank));
    asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(remote), "f"(a), "f"(b) : "memory");
}
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// What the fused variant (FUSE) also does, so that no separate RoPE kernel runs in a decode step:
// q arrives unrotated, with the new token's k and v behind it in the same row (the output of the
// fused q/k/v projection); q is rotated in registers, and the warp that reads the sequence's last
// page puts the rotated k and the v of the new token into its shared-memory copy of that page
// (and, in one CTA per KV head, into the cache).  Pages hold only older tokens otherwise, so every
// page load starts BEFORE the wait on the preceding kernel.
struct RopeArgs {
    const float *cos_t, *sin_t;      // [positions, HD / 2]
    bf16 *k_pool, *v_pool;           // the cache, writable
    int q_heads;                     // H: k starts at q + H * HD, v at q + (H + KV) * HD
};

template <int HD, bool CLUSTER, bool FUSE>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_decode_kernel(const bf16 *__restrict__ q, int ldq, const int *__restrict__ positions,
                   const int *__restrict__ block_table, int table_width,
                   const bf16 *__restrict__ k_pool, const bf16 *__restrict__ v_pool,
                   int KV, int G, float scale, int window, int n_splits,
                   float *__restrict__ part_o, float *__restrict__ part_ml,
                   bf16 *__restrict__ out, int ldo, RopeArgs rope) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int TILE_BYTES = PAGE * HD * 2;
    const int warp = warp_index(), lane = threadIdx.x & 31;
    const int chunks = (G + 15) / 16;
    const int kvh = blockIdx.y / chunks, g0 = (blockIdx.y % chunks) * 16;
    const int rows = min(16, G - g0);
    const int b = blockIdx.z, split = blockIdx.x;
    if (CLUSTER && n_splits > 1) cluster_arrive_relaxed();       // matched before the first push: every CTA runs
    pdl_launch_dependents();
    if (!FUSE) pdl_wait();
    // Read before the wait (fused form): positions, the page table and this entry's own pages.  Allowed only
    // because nothing launched since the stream's last full barrier writes them (see common.cuh): positions
    // and tables change by the step's opening copy or by decode_advance, the last kernel of a step, and this
    // pool is appended to by this kernel alone.  A caller that reorders that must launch without the overlap.
    const int pos = positions[b];
    const int lo_key = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int first_page = lo_key / PAGE, n_pages = pos / PAGE - first_page + 1;
    const int per = (n_pages + n_splits - 1) / n_splits;
    const int p_begin = first_page + split * per, p_end = min(first_page + n_pages, p_begin + per);
    const int *bt = block_table + (size_t)b * table_width;

    uint8_t *kbuf = smem + (size_t)warp * 2 * TILE_BYTES, *vbuf = kbuf + TILE_BYTES;
    const uint32_t ks = smem_addr(kbuf), vs = smem_addr(vbuf);

    float o[HD / 8][4];
#pragma unroll
    for (int d = 0; d < HD / 8; d++) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const int lo[2] = {lo_key, lo_key}, hi[2] = {pos, pos};

    int p = p_begin + warp;
    if (p < p_end) {
        size_t base = ((size_t)bt[p] * KV + kvh) * PAGE * HD;
        load_page_warp<HD>(ks, k_pool + base, lane);
        cp_async_commit();
        load_page_warp<HD>(vs, v_pool + base, lane);
        cp_async_commit();
    }
    if (FUSE) pdl_wait();                      // q, k, v of the new token come from the kernel before
    // the warp that will read the sequence's last page fetches the new token's k and v now, with q
    const int p_new = pos / PAGE;
    const bool mine = FUSE && p_new >= p_begin && p_new < p_end && ((p_new - p_begin) & (DEC_WARPS - 1)) == warp;
    uint4 knew_lo = make_uint4(0, 0, 0, 0), knew_hi = knew_lo, vnew = knew_lo;
    if (mine) {
        const bf16 *ksrc = q + (size_t)b * ldq + (size_t)(rope.q_heads + kvh) * HD;
        const bf16 *vsrc = q + (size_t)b * ldq + (size_t)(rope.q_heads + KV + kvh) * HD;
        if (lane < HD / 16) { knew_lo = *(const uint4 *)(ksrc + lane * 8); knew_hi = *(const uint4 *)(ksrc + HD / 2 + lane * 8); }
        if (lane < HD / 8) vnew = *(const uint4 *)(vsrc + lane * 8);
    }
    // Q fragments of rows g0 .. g0+15 of this KV head's group (rows past the group are zero)
    uint32_t qf[HD / 16][4];
    {
        const int r0 = lane >> 2, c = (lane & 3) * 2;
        const bf16 *qrow = q + (size_t)b * ldq + (size_t)(kvh * G + g0) * HD;
#pragma unroll
        for (int kk = 0; kk < HD / 16; kk++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                int r = r0 + (e & 1) * 8, k = kk * 16 + c + (e >> 1) * 8;
                qf[kk][e] = r < rows ? *(const uint32_t *)(qrow + (size_t)r * HD + k) : 0u;
            }
        }
        if (FUSE) {
            // rotate: dims (j, j + HD/2) are the same registers of k-steps kk and kk + HD/32
            const float *cs = rope.cos_t + (size_t)pos * (HD / 2), *sn = rope.sin_t + (size_t)pos * (HD / 2);
#pragma unroll
            for (int kk = 0; kk < HD / 32; kk++) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    int j = kk * 16 + c + (e >> 1) * 8;
                    float2 lo2 = __bfloat1622float2(*(__nv_bfloat162 *)&qf[kk][e]);
                    float2 hi2 = __bfloat1622float2(*(__nv_bfloat162 *)&qf[kk + HD / 32][e]);
                    float c0 = cs[j], c1 = cs[j + 1], s0 = sn[j], s1 = sn[j + 1];
                    qf[kk][e] = pack_bf16(lo2.x * c0 - hi2.x * s0, lo2.y * c1 - hi2.y * s1);
                    qf[kk + HD / 32][e] = pack_bf16(lo2.x * s0 + hi2.x * c0, lo2.y * s1 + hi2.y * c1);
                }
            }
        }
    }
    for (; p < p_end; p += DEC_WARPS) {
        const int pn = p + DEC_WARPS;
        const size_t nbase = pn < p_end ? ((size_t)bt[pn] * KV + kvh) * PAGE * HD : 0;
        cp_async_wait<1>();                    // K of this page has landed (V may still be in flight)
        __syncwarp();
        const bool newest = FUSE && p == pos / PAGE;      // this page holds the new token's row
        if (newest) {
            // rotated k of the new token -> row pos % 64 of the K tile (and the cache, once per KV head)
            const int off = pos % PAGE;
            const bool to_cache = blockIdx.y % chunks == 0;
            const float *cs = rope.cos_t + (size_t)pos * (HD / 2), *sn = rope.sin_t + (size_t)pos * (HD / 2);
            if (lane < HD / 16) {
                const int j0 = lane * 8;
                uint4 lo4 = knew_lo, hi4 = knew_hi;
                const __nv_bfloat162 *lp = (const __nv_bfloat162 *)&lo4, *hp = (const __nv_bfloat162 *)&hi4;
                uint4 olo, ohi;
                uint32_t *ol = (uint32_t *)&olo, *oh = (uint32_t *)&ohi;
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    float2 a = __bfloat1622float2(lp[e]), bb = __bfloat1622float2(hp[e]);
                    float c0 = cs[j0 + 2 * e], c1 = cs[j0 + 2 * e + 1], s0 = sn[j0 + 2 * e], s1 = sn[j0 + 2 * e + 1];
                    ol[e] = pack_bf16(a.x * c0 - bb.x * s0, a.y * c1 - bb.y * s1);
                    oh[e] = pack_bf16(a.x * s0 + bb.x * c0, a.y * s1 + bb.y * c1);
                }
                const int clo = lane, chi = lane + HD / 16;
                *(uint4 *)(kbuf + off * (HD * 2) + ((clo ^ (off & 7)) << 4)) = olo;
                *(uint4 *)(kbuf + off * (HD * 2) + ((chi ^ (off & 7)) << 4)) = ohi;
                if (to_cache) {
                    bf16 *dst = rope.k_pool + (((size_t)bt[p] * KV + kvh) * PAGE + off) * HD;
                    *(uint4 *)(dst + j0) = olo;
                    *(uint4 *)(dst + HD / 2 + j0) = ohi;
                }
            }
            __syncwarp();
        }
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; j++) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
        qk_page<HD>(s, qf, ks, lane);
        __syncwarp();
        if (pn < p_end) load_page_warp<HD>(ks, k_pool + nbase, lane);
        cp_async_commit();                     // (possibly empty) group: keeps the wait counts uniform
        if (p * PAGE + PAGE - 1 <= pos && p * PAGE >= lo_key)
            softmax_update<HD / 8, false>(s, o, m, l, scale * LOG2E, p * PAGE, lo, hi, lane);
        else
            softmax_update<HD / 8, true>(s, o, m, l, scale * LOG2E, p * PAGE, lo, hi, lane);
        cp_async_wait<1>();                    // V of this page has landed
        __syncwarp();
        if (newest) {
            const int off = pos % PAGE;
            if (lane < HD / 8) {
                uint4 v4 = vnew;
                *(uint4 *)(vbuf + off * (HD * 2) + ((lane ^ (off & 7)) << 4)) = v4;
                if (blockIdx.y % chunks == 0)
                    *(uint4 *)(rope.v_pool + (((size_t)bt[p] * KV + kvh) * PAGE + off) * HD + lane * 8) = v4;
            }
            __syncwarp();
        }
        pv_page<HD>(o, s, vs, lane);
        __syncwarp();
        if (pn < p_end) load_page_warp<HD>(vs, v_pool + nbase, lane);
        cp_async_commit();
    }
    cp_async_wait<0>();
    if (CLUSTER) {
        // ---- every warp's partial result goes to the owners of its slices; see the head of this file
        const int S = n_splits, dsl = HD / S, dsl_log = __ffs(dsl) - 1;          // HD and S are powers of two
        float *recv_o = (float *)(smem + (size_t)DEC_WARPS * 2 * TILE_BYTES);     // [4 S][rows][dsl]
        float *recv_ml = recv_o + DEC_WARPS * rows * HD;                           // [4 S][16][2]
        if (S > 1) cluster_wait();                                                // the phase opened at the top
        if (p_begin + warp < p_end) {                                             // this warp read at least one page
            const int slot = split * DEC_WARPS + warp, r0 = lane >> 2, c = (lane & 3) * 2;
#pragma unroll
            for (int d = 0; d < HD / 8; d++) {
                const int col = d * 8 + c, owner = col >> dsl_log, cc = col & (dsl - 1);
                if (r0 < rows) st_dsmem2(&recv_o[(slot * rows + r0) * dsl + cc], owner, o[d][0], o[d][1]);
                if (r0 + 8 < rows) st_dsmem2(&recv_o[(slot * rows + r0 + 8) * dsl + cc], owner, o[d][2], o[d][3]);
            }
            if ((lane & 3) == 0) {
                for (int z = 0; z < S; z++) {
                    if (r0 < rows) st_dsmem2(&recv_ml[(slot * 16 + r0) * 2], z, m[0], l[0]);
                    if (r0 + 8 < rows) st_dsmem2(&recv_ml[(slot * 16 + r0 + 8) * 2], z, m[1], l[1]);
                }
            }
        }
        if (S > 1) cluster_sync_all(); else __syncthreads();
        // this CTA's slice: columns [split * dsl, (split + 1) * dsl) of every row, over the warps that had pages
        for (int e = threadIdx.x; e < rows * dsl; e += DEC_WARPS * 32) {
            const int r = e >> dsl_log, cc = e & (dsl - 1);
            // the four warps of a split at a time, their loads in flight together; a warp without pages counts as -inf
            float M = -INFINITY;
#pragma unroll 1
            for (int z = 0; z < S; z++) {
                const int have = min(first_page + n_pages, first_page + (z + 1) * per) - (first_page + z * per);
                float mw[DEC_WARPS];
#pragma unroll
                for (int w = 0; w < DEC_WARPS; w++) mw[w] = w < have ? recv_ml[((z * DEC_WARPS + w) * 16 + r) * 2] : -INFINITY;
#pragma unroll
                for (int w = 0; w < DEC_WARPS; w++) M = fmaxf(M, mw[w]);
            }
            float O = 0.f, L = 0.f;
#pragma unroll 1
            for (int z = 0; z < S; z++) {
                const int have = min(first_page + n_pages, first_page + (z + 1) * per) - (first_page + z * per);
                float mw[DEC_WARPS], lw[DEC_WARPS], ow[DEC_WARPS];
#pragma unroll
                for (int w = 0; w < DEC_WARPS; w++) {
                    const int sl = z * DEC_WARPS + w;
                    const bool in = w < have;
                    mw[w] = in ? recv_ml[(sl * 16 + r) * 2] : -INFINITY;
                    lw[w] = in ? recv_ml[(sl * 16 + r) * 2 + 1] : 0.f;
                    ow[w] = in ? recv_o[(sl * rows + r) * dsl + cc] : 0.f;
                }
#pragma unroll
                for (int w = 0; w < DEC_WARPS; w++) {                              // (split, warp) order
                    const float wgt = mw[w] == -INFINITY ? 0.f : ex2(mw[w] - M);
                    O += wgt * ow[w];
                    L += wgt * lw[w];
                }
            }
            out[(size_t)b * ldo + (size_t)(kvh * G + g0 + r) * HD + split * dsl + cc] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
        }
        return;
    }
    __syncthreads();

    // ---- scratch path: merge the four warps, each leaves (m, l) and O[16][HD] in its own buffer
    float *wo = (float *)kbuf;                 // 16 * HD floats <= TILE_BYTES
    float *wml = (float *)vbuf;                // 16 * 2 floats
    {
        const int r0 = lane >> 2, c = (lane & 3) * 2;
#pragma unroll
        for (int d = 0; d < HD / 8; d++) {
            wo[r0 * HD + d * 8 + c] = o[d][0];       wo[r0 * HD + d * 8 + c + 1] = o[d][1];
            wo[(r0 + 8) * HD + d * 8 + c] = o[d][2]; wo[(r0 + 8) * HD + d * 8 + c + 1] = o[d][3];
        }
        if ((lane & 3) == 0) {
            wml[r0 * 2] = m[0]; wml[r0 * 2 + 1] = l[0];
            wml[(r0 + 8) * 2] = m[1]; wml[(r0 + 8) * 2 + 1] = l[1];
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < rows * HD; i += DEC_WARPS * 32) {
        int r = i / HD, d = i % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; w++) M = fmaxf(M, ((float *)(smem + (size_t)w * 2 * TILE_BYTES + TILE_BYTES))[r * 2]);
        float O = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; w++) {
            const float *pml = (const float *)(smem + (size_t)w * 2 * TILE_BYTES + TILE_BYTES);
            const float *po = (const float *)(smem + (size_t)w * 2 * TILE_BYTES);
            float mw = pml[r * 2];
            float wgt = mw == -INFINITY ? 0.f : ex2(mw - M);
            O += wgt * po[r * HD + d];
            L += wgt * pml[r * 2 + 1];
        }
        int h = kvh * G + g0 + r;
        if (n_splits == 1) {
            out[(size_t)b * ldo + (size_t)h * HD + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
        } else {
            size_t prow = ((size_t)b * KV * G + h) * n_splits + split;
            part_o[prow * HD + d] = O;
            if (d == 0) { part_ml[prow * 2] = M; part_ml[prow * 2 + 1] = L; }
        }
    }
}

// merge the splits of one (sequence, head) in split order
template <int HD>
__global__ void attn_decode_merge_kernel(const float *__restrict__ part_o, const float *__restrict__ part_ml,
                                         int n_splits, int H, bf16 *__restrict__ out, int ldo) {
    const int b = blockIdx.y, h = blockIdx.x, d = threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const size_t prow0 = ((size_t)b * H + h) * n_splits;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; s++) M = fmaxf(M, part_ml[(prow0 + s) * 2]);
    float O = 0.f, L = 0.f;
    for (int s = 0; s < n_splits; s++) {
        float ms = part_ml[(prow0 + s) * 2];
        float wgt = ms == -INFINITY ? 0.f : ex2(ms - M);
        O += wgt * part_o[(prow0 + s) * HD + d];
        L += wgt * part_ml[(prow0 + s) * 2 + 1];
    }
    out[(size_t)b * ldo + (size_t)h * HD + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
}

template <int HD, bool CLUSTER, bool FUSE = false>
static int launch_decode_kernel(dim3 grid, int cluster_x, cudaStream_t stream, const void *q, int ldq, void *out, int ldo,
                                const int *positions, const int *block_table, int table_width, const void *k_pool,
                                const void *v_pool, int KV, int G, float scale, int window, int n_splits,
                                float *part_o, float *part_ml, RopeArgs rope = RopeArgs{}) {
    // behind the page buffers: the cluster merge receives 4 S partial slices [rows][HD / S] and (max, sum) pairs
    constexpr int smem_max = DEC_WARPS * 2 * PAGE * HD * 2 + (CLUSTER ? DEC_WARPS * 16 * HD * 4 + DEC_WARPS * 8 * 16 * 2 * 4 : 0);
    const int rows_cap = G < 16 ? G : 16;
    const int smem = DEC_WARPS * 2 * PAGE * HD * 2 + (CLUSTER ? DEC_WARPS * rows_cap * HD * 4 + DEC_WARPS * n_splits * 16 * 2 * 4 : 0);
    // the attribute belongs to the function on ONE device: set it once on every device that launches
    static bool configured[64] = {false};
    int dev = 0;
    cudaError_t ed = cudaGetDevice(&dev);
    if (ed != cudaSuccess) return (int)ed;
    if (dev < 0 || dev >= 64) return FG_ERR_BAD_SIZE;
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<HD, CLUSTER, FUSE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(DEC_WARPS * 32); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (fg_pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        n++;
    }
    if (cluster_x > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster_x; attr[n].val.clusterDim.y = 1; attr[n].val.clusterDim.z = 1;
        n++;
    }
    cfg.attrs = attr; cfg.numAttrs = n;
    return (int)cudaLaunchKernelEx(&cfg, attn_decode_kernel<HD, CLUSTER, FUSE>, (const bf16 *)q, ldq, positions, block_table,
                                   table_width, (const bf16 *)k_pool, (const bf16 *)v_pool, KV, G, scale, window, n_splits,
                                   part_o, part_ml, (bf16 *)out, ldo, rope);
}

template <int HD>
static int launch_decode(const void *q, int ldq, void *out, int ldo, const int *positions, const int *block_table,
                         int table_width, const void *k_pool, const void *v_pool, int B, int H, int KV, float scale,
                         int window, int n_splits, float *part_o, float *part_ml, cudaStream_t stream) {
    int G = H / KV;
    dim3 grid(n_splits, KV * ((G + 15) / 16), B);
    // 2, 4 or 8 splits without scratch memory: merged inside a cluster
    bool cluster = !part_o && (n_splits == 2 || n_splits == 4 || n_splits == 8);
    if (n_splits == 1 || cluster)
        return launch_decode_kernel<HD, true>(grid, cluster ? n_splits : 1, stream, q, ldq, out, ldo, positions, block_table,
                                              table_width, k_pool, v_pool, KV, G, scale, window, n_splits, nullptr, nullptr);
    int e = launch_decode_kernel<HD, false>(grid, 1, stream, q, ldq, out, ldo, positions, block_table, table_width, k_pool,
                                            v_pool, KV, G, scale, window, n_splits, part_o, part_ml);
    if (e) return e;
    return fg_launch(attn_decode_merge_kernel<HD>, dim3(H, B), dim3(HD), 0, stream, (const float *)part_o,
                     (const float *)part_ml, n_splits, H, (bf16 *)out, ldo);
}

// q: [B, ldq] bf16, one row per sequence, heads first in the row; positions[b] is the position of
// that row (its key and value are already in the cache); pools [pages, KV, 64, HD] bf16.
// part_o: [B, H, n_splits, HD] f32 and part_ml: [B, H, n_splits, 2] f32 scratch for the two-kernel
// path; pass null pointers with n_splits 1, 2, 4 or 8 for the path that needs no scratch.
// Takes HD 64 and 128 and pages of 64; anything else returns FG_ERR_BAD_SIZE.
extern "C" int fg_attention_decode(const void *q, int ldq, void *out, int ldo, const int *positions,
                                   const int *block_table, int table_width, const void *k_pool, const void *v_pool,
                                   int B, int H, int KV, int hd, int page_size, float scale, int window,
                                   int n_splits, float *part_o, float *part_ml, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (KV <= 0 || H <= 0) return FG_ERR_BAD_SIZE;
    if (page_size != PAGE || H % KV || n_splits < 1 || B > 65535 || ldq % 2 || ((uintptr_t)q & 3)) return FG_ERR_BAD_SIZE;
    if ((part_o == nullptr) != (part_ml == nullptr)) return FG_ERR_BAD_SIZE;
    if (!part_o && n_splits != 1 && n_splits != 2 && n_splits != 4 && n_splits != 8) return FG_ERR_BAD_SIZE;
    if (hd == 64) return launch_decode<64>(q, ldq, out, ldo, positions, block_table, table_width, k_pool, v_pool, B, H, KV, scale, window, n_splits, part_o, part_ml, stream);
    if (hd == 128) return launch_decode<128>(q, ldq, out, ldo, positions, block_table, table_width, k_pool, v_pool, B, H, KV, scale, window, n_splits, part_o, part_ml, stream);
    return FG_ERR_BAD_SIZE;
}

// The fused decode step of an attention layer: RoPE of q and of the new k, cache append of k and v, and
// attention, in one kernel.  qkv: [B, ldq] rows of (q heads | k heads | v heads) straight from the
// projection; cos/sin: [positions, hd / 2] f32; n_splits 1, 2, 4 or 8 (merged inside a cluster).
extern "C" int fg_attention_decode_fused(const void *qkv, int ldq, void *out, int ldo, const int *positions,
                                         const int *block_table, int table_width, void *k_pool, void *v_pool,
                                         const float *cos_t, const float *sin_t, int B, int H, int KV, int hd,
                                         int page_size, float scale, int window, int n_splits, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (KV <= 0 || H <= 0) return FG_ERR_BAD_SIZE;
    if (page_size != PAGE || H % KV || B > 65535 || ldq % 8 || ((uintptr_t)qkv & 15) || ((uintptr_t)k_pool & 15) ||
        ((uintptr_t)v_pool & 15) || (n_splits != 1 && n_splits != 2 && n_splits != 4 && n_splits != 8))
        return FG_ERR_BAD_SIZE;
    int G = H / KV;
    dim3 grid(n_splits, KV * ((G + 15) / 16), B);
    RopeArgs rope{cos_t, sin_t, (bf16 *)k_pool, (bf16 *)v_pool, H};
    if (hd == 64)
        return launch_decode_kernel<64, true, true>(grid, n_splits, stream, qkv, ldq, out, ldo, positions, block_table,
                                                    table_width, k_pool, v_pool, KV, G, scale, window, n_splits, nullptr,
                                                    nullptr, rope);
    if (hd == 128)
        return launch_decode_kernel<128, true, true>(grid, n_splits, stream, qkv, ldq, out, ldo, positions, block_table,
                                                     table_width, k_pool, v_pool, KV, G, scale, window, n_splits, nullptr,
                                                     nullptr, rope);
    return FG_ERR_BAD_SIZE;
}

// ---------------------------------------------------------------------------- no allocation
// See fastgguf_noalloc.h.  The scratch of the two-kernel path lives in this array, which is part
// of the library image: every GPU that loads the library holds it until the process exits.
#include "fastgguf_noalloc.h"

static __device__ __align__(256) float g_noalloc_scratch[FG_NOALLOC_SCRATCH_FLOATS];

// In host code the name of a __device__ array is only a handle; the address the kernels need comes
// from cudaGetSymbolAddress, asked once per device with that device current.
static int noalloc_scratch_address(float **ptr) {
    static float *per_device[64] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return FG_ERR_BAD_SIZE;
    if (!per_device[dev]) {
        float *p = nullptr;
        e = cudaGetSymbolAddress((void **)&p, g_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        per_device[dev] = p;
    }
    *ptr = per_device[dev];
    return 0;
}

extern "C" int fg_attention_decode_noalloc(const void *q, int ldq, void *out, int ldo, const int *positions,
                                           const int *block_table, int table_width, const void *k_pool,
                                           const void *v_pool, int B, int H, int KV, int hd, int page_size, float scale,
                                           int window, int n_splits, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (n_splits < 1 || H <= 0 || KV <= 0 || hd <= 0) return FG_ERR_BAD_SIZE;
    long long rows = (long long)B * H * n_splits;
    // with one split the kernel writes the output itself and never touches the array
    if (n_splits > 1 && rows * (hd + 2) > FG_NOALLOC_SCRATCH_FLOATS) return FG_ERR_NOALLOC_TOO_LARGE;
    float *scratch = nullptr;
    int e = noalloc_scratch_address(&scratch);
    if (e) return e;
    // partial outputs first, then the (max, sum) pairs; each call writes every element it later reads
    float *part_o = scratch, *part_ml = scratch + rows * hd;
    if (page_size != PAGE || H % KV || B > 65535 || ldq % 2 || ((uintptr_t)q & 3)) return FG_ERR_BAD_SIZE;
    int G = H / KV;
    dim3 grid(n_splits, KV * ((G + 15) / 16), B);
#define NOALLOC_RUN(HD) do { \
        e = launch_decode_kernel<HD, false>(grid, 1, stream, q, ldq, out, ldo, positions, block_table, table_width, \
                                            k_pool, v_pool, KV, G, scale, window, n_splits, part_o, part_ml); \
        if (e || n_splits == 1) return e;      /* one split writes the output itself */ \
        return fg_launch(attn_decode_merge_kernel<HD>, dim3(H, B), dim3(HD), 0, stream, (const float *)part_o, \
                         (const float *)part_ml, n_splits, H, (bf16 *)out, ldo); } while (0)
    if (hd == 64) NOALLOC_RUN(64);
    if (hd == 128) NOALLOC_RUN(128);
#undef NOALLOC_RUN
    return FG_ERR_BAD_SIZE;
}
