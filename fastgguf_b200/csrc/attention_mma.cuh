// Building blocks of the bf16 tensor-core attention kernels: asynchronous page loads into
// swizzled shared memory, ldmatrix fragment loads, and the m16n8k16 MMA.
//
// A cache page is [64 positions][HD] bf16 for one KV head.  In shared memory its rows keep
// their HD*2-byte pitch and the 16-byte chunk c of row r lands at chunk (c ^ (r & 7)), so that
// the eight rows an ldmatrix reads fall into different banks.
#pragma once
#include "common.cuh"

#define PAGE 64

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(uint32_t *)&v;
}

// One warp copies a page tile [PAGE][HD] bf16 from global memory into its shared buffer.
template <int HD>
__device__ __forceinline__ void load_page_warp(uint32_t sdst, const bf16 *src, int lane) {
    constexpr int CPR = HD / 8;                       // 16-byte chunks per row
#pragma unroll
    for (int i = lane; i < PAGE * CPR; i += 32) {
        int r = i / CPR, c = i % CPR;
        cp_async16(sdst + r * (HD * 2) + ((c ^ (r & 7)) << 4), src + (size_t)r * HD + c * 8);
    }
}

// S[16 x 64] += Q[16 x HD] K^T for one page: s[j] is the n-tile of keys 8j..8j+7.
template <int HD>
__device__ __forceinline__ void qk_page(float (&s)[8][4], const uint32_t (&qf)[HD / 16][4], uint32_t ks, int lane) {
    const int mi = lane >> 3, r = lane & 7;
#pragma unroll
    for (int kk = 0; kk < HD / 16; kk++) {
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
            int row = jj * 16 + (mi >> 1) * 8 + r, c = kk * 2 + (mi & 1);
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(ks + row * (HD * 2) + ((c ^ (row & 7)) << 4), b0, b1, b2, b3);
            mma_bf16(s[2 * jj], qf[kk], b0, b1);
            mma_bf16(s[2 * jj + 1], qf[kk], b2, b3);
        }
    }
}

// O[16 x HD] += P[16 x 64] V for one page; P comes from the S accumulators rounded to bf16.
template <int HD>
__device__ __forceinline__ void pv_page(float (&o)[HD / 8][4], const float (&s)[8][4], uint32_t vs, int lane) {
    const int mi = lane >> 3, r = lane & 7;
#pragma unroll
    for (int ks = 0; ks < 4; ks++) {
        uint32_t a[4] = {pack_bf16(s[2 * ks][0], s[2 * ks][1]), pack_bf16(s[2 * ks][2], s[2 * ks][3]),
                         pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]), pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3])};
#pragma unroll
        for (int dd = 0; dd < HD / 16; dd++) {
            int row = ks * 16 + (mi & 1) * 8 + r, c = dd * 2 + (mi >> 1);
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(vs + row * (HD * 2) + ((c ^ (row & 7)) << 4), b0, b1, b2, b3);
            mma_bf16(o[2 * dd], a, b0, b1);
            mma_bf16(o[2 * dd + 1], a, b2, b3);
        }
    }
}

// 2^x on the special-function unit (2 ulp); exponents are kept in the base-2 domain so that one
// multiply-add and one ex2 make a probability.  ex2(-inf) = 0.
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
#define LOG2E 1.4426950408889634f

// Online-softmax update of one 16 x 64 score tile held by a warp.  Thread t owns rows t/4 and
// t/4 + 8 (index 0 / 1 below) and key columns 8j + 2(t%4) + {0, 1} of every n-tile j.
// `scale_log2` = scale * log2(e): running maxima `m` live in the base-2 domain.
// MASK: `key0` is the position of the tile's first key and keys outside [lo[i], hi[i]] are
// masked; without MASK every key of the tile is visible to every row (no compares).
// On return s holds the probabilities 2^(score - m_new) and o, l are rescaled.
template <int NO, bool MASK>
__device__ __forceinline__ void softmax_update(float (&s)[8][4], float (&o)[NO][4], float (&m)[2], float (&l)[2],
                                               float scale_log2, int key0, const int (&lo)[2], const int (&hi)[2], int lane) {
    const int c0 = key0 + 2 * (lane & 3);
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
            int i = e >> 1, key = c0 + 8 * j + (e & 1);
            float v = s[j][e] * scale_log2;
            if (MASK) v = (key >= lo[i] && key <= hi[i]) ? v : -INFINITY;
            s[j][e] = v;
            mx[i] = fmaxf(mx[i], v);
        }
#pragma unroll
    for (int i = 0; i < 2; i++) {
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
    }
    float corr[2], mn[2], sum[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 2; i++) {
        mn[i] = fmaxf(m[i], mx[i]);
        corr[i] = mn[i] == -INFINITY ? 1.f : ex2(m[i] - mn[i]);     // nothing seen yet: keep zeros
        if (mn[i] == -INFINITY) mn[i] = 0.f;                        // every key masked: 2^(-inf - 0) = 0 below
    }
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
            int i = e >> 1;
            float p = ex2(s[j][e] - mn[i]);
            s[j][e] = p;
            sum[i] += p;
        }
#pragma unroll
    for (int i = 0; i < 2; i++) {
        sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 1);
        sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 2);
        l[i] = l[i] * corr[i] + sum[i];
        m[i] = fmaxf(m[i], mx[i]);
    }
#pragma unroll
    for (int d = 0; d < NO; d++) {
        o[d][0] *= corr[0]; o[d][1] *= corr[0];
        o[d][2] *= corr[1]; o[d][3] *= corr[1];
    }
}
