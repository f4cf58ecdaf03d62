// Next-token selection on the device, one block per sequence.
//
// Order of operations, as the reference's sample_next (fastgguf.c:4008-4056):
//   repeat penalty (logit > 0 ? / p : * p, once per distinct token of the last n, stop tokens
//   exempt; :4010-4021) -> greedy argmax if temp <= 0, first maximum wins (:4022, :3328-3332)
//   -> candidates: the top_k largest sorted descending, earlier index first on ties
//   (:3989-4005), or with top_k <= 0 everything above max - 20*temp (:4026-4035)
//   -> p_i = expf((v_i - max) / temp), summed in candidate order (:4036-4037)
//   -> top-p: shortest prefix whose sum reaches top_p * total (:4039-4047)
//   -> r = uniform * tot, walk the prefix subtracting until r < 0 (:4049-4055).
// Random numbers: xorshift64* with 24-bit uniforms (:3334-3339, :3979-3981); the state of
// each sequence lives in device memory, so a sequence's stream does not depend on its batch.
//
// With top_k in [1, 1024] the candidate order and every float operation follow the reference,
// so the same logits give the same token.  With top_k <= 0 the candidates are walked in index
// order instead of sorted order (same distribution, other token for the same draw) and top-p
// is applied through a probability threshold.
#include "common.cuh"

#define SAMPLE_THREADS 1024
#define MAX_TOP_K 1024

__device__ __forceinline__ uint32_t float_key(float v) {
    uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);      // larger float <=> larger key
}
__device__ __forceinline__ float key_float(uint32_t k) {
    uint32_t b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
    return __uint_as_float(b);
}

__device__ __forceinline__ uint64_t xorshift64star(uint64_t *s) {
    uint64_t x = *s;
    x ^= x >> 12; x ^= x << 25; x ^= x >> 27;
    *s = x;
    return x * 0x2545F4914F6CDD1DULL;
}

// block-wide argmax, lowest index on ties; result valid in every thread
__device__ int block_argmax(const float *row, int V, float *out_max) {
    __shared__ float s_v[32];
    __shared__ int s_i[32];
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        float v = row[i];
        if (v > bv) { bv = v; bi = i; }           // strict: the earliest index of a thread wins
    }
    if (bi == 0x7fffffff) { bi = threadIdx.x < V ? threadIdx.x : 0; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) { s_v[w] = bv; s_i[w] = bi; }
    __syncthreads();
    bv = s_v[0]; bi = s_i[0];
    for (int i = 1; i < nw; i++)
        if (s_v[i] > bv || (s_v[i] == bv && s_i[i] < bi)) { bv = s_v[i]; bi = s_i[i]; }
    if (out_max) *out_max = bv;
    return bi;
}

// exclusive prefix count of a per-thread flag over the block, in thread order; total in *total
__device__ int block_excl_count(int flag, int *total) {
    __shared__ int s_w[32];
    unsigned ball = __ballot_sync(0xffffffffu, flag);
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    int within = __popc(ball & ((1u << lane) - 1));
    __syncthreads();
    if (lane == 0) s_w[w] = __popc(ball);
    __syncthreads();
    int before = 0, tot = 0;
    for (int i = 0; i < nw; i++) { int c = s_w[i]; if (i < w) before += c; tot += c; }
    *total = tot;
    return before + within;
}

struct SampleParams {
    float temp, top_p, repeat_penalty;
    int top_k, repeat_last_n;
};

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(float *__restrict__ logits, int V, int ldl, SampleParams sp,
              const int *__restrict__ seq_slot,          // [B] row of rng / history of each sequence
              unsigned long long *__restrict__ rng,      // [n_slots]
              int *__restrict__ hist, int hist_cap,      // [n_slots, hist_cap] ring of recent tokens
              int *__restrict__ hist_count,              // [n_slots] tokens ever recorded
              const int *__restrict__ stop_ids, int n_stop,
              int *__restrict__ out_tokens) {
    __shared__ unsigned long long cand[MAX_TOP_K];       // (key << 32) | (~index)
    __shared__ int s_hist[256];
    __shared__ int s_misc[4];
    float *row = logits + (size_t)blockIdx.x * ldl;
    int slot = seq_slot[blockIdx.x];
    int *h = hist ? hist + (size_t)slot * hist_cap : nullptr;
    int tid = threadIdx.x;

    // ---- repeat penalty, in place, once per distinct recent token
    if (h && sp.repeat_penalty > 0.f && sp.repeat_penalty != 1.0f && sp.repeat_last_n > 0) {
        int have = min(hist_count[slot], min(hist_cap, sp.repeat_last_n));
        for (int i = tid; i < have; i += blockDim.x) {
            int id = h[i];
            bool skip = id < 0 || id >= V;
            for (int s = 0; s < n_stop && !skip; s++) skip = stop_ids[s] == id;
            for (int j = 0; j < i && !skip; j++) skip = h[j] == id;
            if (!skip) {
                float v = row[id];
                row[id] = v > 0.f ? v / sp.repeat_penalty : v * sp.repeat_penalty;
            }
        }
        __syncthreads();
    }

    float mx;
    int best = block_argmax(row, V, &mx);
    int chosen = best;

    if (sp.temp > 0.f && sp.top_k > 0) {
        // ---- k-th largest key by radix select, 8 bits a pass
        int k = min(min(sp.top_k, MAX_TOP_K), V);
        uint32_t prefix = 0, mask = 0;
        int need = k;                                    // rank still wanted among keys matching prefix
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tid < 256) s_hist[tid] = 0;
            __syncthreads();
            for (int i = tid; i < V; i += blockDim.x) {
                uint32_t key = float_key(row[i]);
                if ((key & mask) == prefix) atomicAdd(&s_hist[(key >> shift) & 255], 1);
            }
            __syncthreads();
            if (tid == 0) {
                int cum = 0, b = 255;
                for (; b > 0; b--) { if (cum + s_hist[b] >= need) break; cum += s_hist[b]; }
                s_misc[0] = b; s_misc[1] = need - cum;
            }
            __syncthreads();
            prefix |= (uint32_t)s_misc[0] << shift;
            mask |= 255u << shift;
            need = s_misc[1];
            __syncthreads();
        }
        uint32_t kth = prefix;                           // key of the k-th largest; `need` ties of it are taken
        // ---- collect: every key above kth, and the first `need` equal to it in index order
        if (tid == 0) s_misc[2] = 0;
        __syncthreads();
        int taken_eq = 0;
        for (int c0 = 0; c0 < V; c0 += blockDim.x) {
            int i = c0 + tid;
            uint32_t key = i < V ? float_key(row[i]) : 0u;
            int gt = i < V && key > kth, eq = i < V && key == kth;
            int tot_eq;
            int rank_eq = block_excl_count(eq, &tot_eq);
            bool take = gt || (eq && taken_eq + rank_eq < need);
            if (take) {
                int slot_c = atomicAdd(&s_misc[2], 1);
                cand[slot_c] = ((unsigned long long)key << 32) | (uint32_t)(~(uint32_t)i);
            }
            taken_eq += tot_eq;
        }
        __syncthreads();
        int n = s_misc[2];                               // == k
        for (int i = n + tid; i < MAX_TOP_K; i += blockDim.x) cand[i] = 0ull;
        __syncthreads();
        // ---- bitonic sort, descending: value first, then lower index first
        for (int size = 2; size <= MAX_TOP_K; size <<= 1) {
            for (int stride = size >> 1; stride > 0; stride >>= 1) {
                int i = tid, j = i ^ stride;
                if (j > i) {
                    unsigned long long a = cand[i], b = cand[j];
                    bool desc = (i & size) == 0;
                    if (desc ? a < b : a > b) { cand[i] = b; cand[j] = a; }
                }
                __syncthreads();
            }
        }
        // ---- probabilities, top-p and the draw, sequentially in candidate order like the reference
        if (tid == 0) {
            float top = key_float((uint32_t)(cand[0] >> 32));
            float sum = 0.f;
            for (int i = 0; i < n; i++) sum += expf((key_float((uint32_t)(cand[i] >> 32)) - top) / sp.temp);
            int keep = n;
            if (sp.top_p > 0.f && sp.top_p < 1.0f) {
                float cum = 0.f, lim = sp.top_p * sum;
                for (int i = 0; i < n; i++) {
                    cum += expf((key_float((uint32_t)(cand[i] >> 32)) - top) / sp.temp);
                    if (cum >= lim) { keep = i + 1; break; }
                }
            }
            float tot = 0.f;
            for (int i = 0; i < keep; i++) tot += expf((key_float((uint32_t)(cand[i] >> 32)) - top) / sp.temp);
            uint64_t st = rng[slot];
            float r = (float)(xorshift64star(&st) >> 40) / 16777216.0f * tot;
            rng[slot] = st;
            int pick = keep - 1;
            for (int i = 0; i < keep; i++) {
                r -= expf((key_float((uint32_t)(cand[i] >> 32)) - top) / sp.temp);
                if (r < 0.f) { pick = i; break; }
            }
            s_misc[3] = (int)(~(uint32_t)(cand[pick] & 0xffffffffull));
        }
        __syncthreads();
        chosen = s_misc[3];
    } else if (sp.temp > 0.f) {
        // ---- no top-k: everything above max - 20*temp, walked in index order
        __shared__ float s_part[SAMPLE_THREADS];
        __shared__ float s_scr[32];
        float cut = mx - 20.0f * sp.temp;
        // optional top-p: largest threshold key t such that the mass of keys >= t reaches top_p * sum
        int per = (V + blockDim.x - 1) / blockDim.x;       // contiguous span of indices per thread
        int i0 = tid * per, i1 = min(V, i0 + per);
        float part = 0.f;
        for (int i = i0; i < i1; i++) { float v = row[i]; if (v > cut) part += expf((v - mx) / sp.temp); }
        float sum = block_sum(part, s_scr);
        uint32_t thr_key = 0;                               // keep keys >= thr_key
        if (sp.top_p > 0.f && sp.top_p < 1.0f) {
            // binary search on the 32-bit key for the largest t with mass(key >= t) >= top_p * sum
            float lim = sp.top_p * sum;
            uint32_t lo_k = 0, hi_k = float_key(mx);        // mass(>= lo_k) = sum >= lim always
            while (lo_k < hi_k) {
                uint32_t mid = lo_k + (uint32_t)(((unsigned long long)hi_k - lo_k + 1) >> 1);
                float pm = 0.f;
                for (int i = i0; i < i1; i++) {
                    float v = row[i];
                    if (v > cut && float_key(v) >= mid) pm += expf((v - mx) / sp.temp);
                }
                float mass = block_sum(pm, s_scr);
                if (mass >= lim) lo_k = mid; else hi_k = mid - 1;
            }
            thr_key = lo_k;
            part = 0.f;
            for (int i = i0; i < i1; i++) {
                float v = row[i];
                if (v > cut && float_key(v) >= thr_key) part += expf((v - mx) / sp.temp);
            }
        }
        s_part[tid] = part;
        __syncthreads();
        if (tid == 0) {
            float tot = 0.f;
            for (int t = 0; t < (int)blockDim.x; t++) tot += s_part[t];
            uint64_t st = rng[slot];
            float r = (float)(xorshift64star(&st) >> 40) / 16777216.0f * tot;
            rng[slot] = st;
            int t = 0;
            for (; t < (int)blockDim.x - 1; t++) { if (r < s_part[t]) break; r -= s_part[t]; }
            int lo_i = t * per, hi_i = min(V, lo_i + per);
            int pick = -1, last = best;
            for (int i = lo_i; i < hi_i; i++) {
                float v = row[i];
                if (v > cut && float_key(v) >= thr_key) {
                    last = i;
                    r -= expf((v - mx) / sp.temp);
                    if (r < 0.f) { pick = i; break; }
                }
            }
            s_misc[3] = pick >= 0 ? pick : last;
        }
        __syncthreads();
        chosen = s_misc[3];
    }

    if (tid == 0) {
        out_tokens[blockIdx.x] = chosen;
        if (h) {
            // keep the ring in age order: slide when full (hist_cap is small)
            int c = hist_count[slot];
            if (c < hist_cap) h[c] = chosen;
            else { for (int i = 1; i < hist_cap; i++) h[i - 1] = h[i]; h[hist_cap - 1] = chosen; }
            hist_count[slot] = c + 1;
        }
    }
}

// ---- top-k sampling in two stages (k <= 128): the vocabulary of a row is split over segments of at most 4,096 entries; a block per segment hands over its K best (K = 64 or 128 >= k) as 64-bit words (value key, then lower index first), sorted;
// one block per row then finds the K best of those and draws exactly as the single-block kernel does.  The k best
// of the row are among the K best of each segment, and the words order them totally, so the result is the
// single-block kernel's.
#define TOPK_SEG 4096                  // most vocabulary entries a stage-1 block takes
#define TOPK_CAND 4096                 // most candidates per row after stage 1 (the caller's scratch holds as many words a row)
#define TOPK_MAX_K 128

__global__ void __launch_bounds__(64)
penalty_kernel(float *__restrict__ logits, int V, int ldl, float penalty, int last_n, const int *__restrict__ seq_slot,
               const int *__restrict__ hist, int hist_cap, const int *__restrict__ hist_count,
               const int *__restrict__ stop_ids, int n_stop) {
    pdl_launch_dependents();
    pdl_wait();
    float *row = logits + (size_t)blockIdx.x * ldl;
    int slot = seq_slot[blockIdx.x];
    const int *h = hist + (size_t)slot * hist_cap;
    int have = min(hist_count[slot], min(hist_cap, last_n));
    for (int i = threadIdx.x; i < have; i += blockDim.x) {
        int id = h[i];
        bool skip = id < 0 || id >= V;
        for (int s = 0; s < n_stop && !skip; s++) skip = stop_ids[s] == id;
        for (int j = 0; j < i && !skip; j++) skip = h[j] == id;
        if (!skip) {
            float v = row[id];
            row[id] = v > 0.f ? v / penalty : v * penalty;
        }
    }
}

// The K largest of the words that the 256 threads of a block hold in registers (PT each; value key, then lower
// index first; all words are distinct; 0 = empty, the smallest), written to out[0 .. K) in descending order, zeros
// after the last.  The K-th largest of the threads' own maxima is a lower bound of the K-th largest of all (K
// entries are at least that large), so only what reaches it - K entries and a few more, PT * K at the very most -
// is ranked by counting, and a word's rank is its place in the output.  (A radix select over the keys with a
// histogram in shared memory took 29 us at a vocabulary of 128,256 - logits share their exponent bits, so its first
// passes are thousands of atomic adds on two or three words - and a bitonic sort of the segment 90 us; sorting the
// 2,048 candidates of the second stage to use the first 64 took 31 us.)
#define TOPK_KEEP (TOPK_MAX_K * 16)
struct TopkScratch {
    unsigned long long best[256];
    unsigned long long keep[TOPK_KEEP];
    unsigned long long bound;
    int n_keep;
};
template <int PT>
__device__ __forceinline__ void block_topk_ranked(const unsigned long long (&w)[PT], int K, TopkScratch &sc, unsigned long long *out) {
    static_assert(PT <= 16, "the kept list holds 16 K words");
    const int tid = threadIdx.x;
    unsigned long long mine = 0ull;
#pragma unroll
    for (int j = 0; j < PT; j++) mine = w[j] > mine ? w[j] : mine;
    sc.best[tid] = mine;
    if (tid == 0) { sc.bound = 1ull; sc.n_keep = 0; }    // fewer than K threads with an entry: every entry is kept
    for (int i = tid; i < K; i += 256) out[i] = 0ull;
    __syncthreads();
    {
        int above = 0;
        for (int t = 0; t < 256; t++) above += sc.best[t] > mine;
        if (above == K - 1 && mine != 0ull) sc.bound = mine;
    }
    __syncthreads();
    const unsigned long long lb = sc.bound;
#pragma unroll
    for (int j = 0; j < PT; j++)
        if (w[j] >= lb) sc.keep[atomicAdd(&sc.n_keep, 1)] = w[j];
    __syncthreads();
    const int c = sc.n_keep;
    for (int i = tid; i < c; i += 256) {
        const unsigned long long x = sc.keep[i];
        int above = 0;
        for (int t = 0; t < c; t++) above += sc.keep[t] > x;
        if (above < K) out[above] = x;
    }
}

// Stage 1: the K best words of a segment of at most TOPK_SEG entries.
__global__ void __launch_bounds__(256)
topk_stage1_kernel(const float *__restrict__ logits, int V, int ldl, int K, int n_blocks,
                   unsigned long long *__restrict__ cand) {        // [B, n_blocks * K], zero where unused
    __shared__ TopkScratch sc;
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y, tid = threadIdx.x;
    const float *row = logits + (size_t)b * ldl;
    const int per = (V + n_blocks - 1) / n_blocks;
    const int i0 = blockIdx.x * per, n = max(0, min(V, i0 + per) - i0);
    unsigned long long w[TOPK_SEG / 256];
#pragma unroll
    for (int j = 0; j < TOPK_SEG / 256; j++) {
        const int i = tid + 256 * j;
        w[j] = i < n ? (((unsigned long long)float_key(row[i0 + i]) << 32) | (uint32_t)(~(uint32_t)(i0 + i))) : 0ull;
    }
    block_topk_ranked(w, K, sc, cand + ((size_t)b * n_blocks + blockIdx.x) * K);
}

// m chunks of K words in shared memory, each sorted descending (m and K powers of two) -> the K largest of all,
// sorted descending, in w[0 .. K): chunk p takes max(A[i], B[K - 1 - i]) with its partner chunk p + m / 2, which
// leaves the K largest of both as a bitonic sequence, and log2 K merge steps sort it again; the number of chunks
// halves every round.  The time does not depend on the values.
__device__ void topk_merge_desc(unsigned long long *w, int m, int K) {
    const int k_log = __ffs(K) - 1;
    for (; m > 1; m >>= 1) {
        const int half = m >> 1;
        for (int e = threadIdx.x; e < half * K; e += blockDim.x) {
            const int p = e >> k_log, i = e & (K - 1);
            const unsigned long long b = w[(p + half) * K + (K - 1 - i)];
            if (b > w[e]) w[e] = b;
        }
        __syncthreads();
        for (int s_log = k_log - 1; s_log >= 0; s_log--) {
            for (int e = threadIdx.x; e < (half * K >> 1); e += blockDim.x) {
                const int i = ((e >> s_log) << (s_log + 1)) + (e & ((1 << s_log) - 1)), j = i + (1 << s_log);
                const unsigned long long x = w[i], y = w[j];
                if (x < y) { w[i] = y; w[j] = x; }
            }
            __syncthreads();
        }
    }
}

// Stage 2, one block per row: the K best of the segments' sorted candidates by merging, and the draw.  (Sorting all
// candidates to use the first 64 took 31 us.)
__global__ void __launch_bounds__(256)
topk_stage2_kernel(const unsigned long long *__restrict__ cand_in, int n_chunks, int K, int k, SampleParams sp,
                   const int *__restrict__ seq_slot, unsigned long long *__restrict__ rng,
                   int *__restrict__ hist, int hist_cap, int *__restrict__ hist_count, int *__restrict__ out_tokens) {
    __shared__ unsigned long long cand[TOPK_CAND];
    __shared__ float wgt[TOPK_MAX_K];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x, tid = threadIdx.x, slot = seq_slot[b];
    int m = 1;
    while (m < n_chunks) m <<= 1;                         // chunks beyond the segments are empty
    for (int i = tid; i < m * K; i += blockDim.x) cand[i] = i < n_chunks * K ? cand_in[(size_t)b * n_chunks * K + i] : 0ull;
    __syncthreads();
    topk_merge_desc(cand, m, K);
    // the weights exp((v - top) / temp) of the k best, one thread each (0 beyond them: adding it changes no sum); the
    // sums below add them in index order, as the serial sampler does (the same floats in the same order: the same token)
    if (tid < TOPK_MAX_K)
        wgt[tid] = (tid < k && tid < K && cand[tid] != 0ull)
                       ? expf((key_float((uint32_t)(cand[tid] >> 32)) - key_float((uint32_t)(cand[0] >> 32))) / sp.temp) : 0.f;
    __syncthreads();
    const int n = __syncthreads_count(tid < k && tid < K && cand[tid] != 0ull);      // the candidates fill the front
    if (tid == 0) {
        // (weights are read eight at a time, ahead of the additions that wait for one another)
        float sum = 0.f;
#pragma unroll 16
        for (int i = 0; i < TOPK_MAX_K; i++) sum += wgt[i];
        int keep = n;
        float tot = sum;
        if (sp.top_p > 0.f && sp.top_p < 1.0f) {
            float cum = 0.f;
            const float lim = sp.top_p * sum;
            bool found = false;
            for (int i0 = 0; i0 < n && !found; i0 += 8) {
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; j++) v[j] = wgt[i0 + j];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    if (found || i0 + j >= n) continue;
                    cum += v[j];
                    if (cum >= lim) { keep = i0 + j + 1; found = true; }
                }
            }
            tot = cum;                                 // the same floats added in the same order as a sum over the kept ones
        }
        uint64_t st = rng[slot];
        float r = (float)(xorshift64star(&st) >> 40) / 16777216.0f * tot;
        rng[slot] = st;
        int pick = keep - 1;
        bool found = false;
        for (int i0 = 0; i0 < keep && !found; i0 += 8) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; j++) v[j] = wgt[i0 + j];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                if (found || i0 + j >= keep) continue;
                r -= v[j];
                if (r < 0.f) { pick = i0 + j; found = true; }
            }
        }
        int chosen = (int)(~(uint32_t)(cand[pick] & 0xffffffffull));
        out_tokens[b] = chosen;
        if (hist) {
            int *h = hist + (size_t)slot * hist_cap;
            int c = hist_count[slot];
            if (c < hist_cap) h[c] = chosen;
            else { for (int i = 1; i < hist_cap; i++) h[i - 1] = h[i]; h[hist_cap - 1] = chosen; }
            hist_count[slot] = c + 1;
        }
    }
}

// ---- greedy without a repeat penalty: the vocabulary of each row is split over GREEDY_BLOCKS blocks;
// each folds its best (value, lowest index) into one 64-bit word per row with atomicMax, and the
// block that arrives last writes the token and clears the word for the next call.  The words (best,
// arrivals) are the first two of the caller's scratch row when `scratch` is given - a sampler that
// owns its scratch shares nothing with other samplers and can clear it when a batch starts - and
// otherwise live in device memory of this library, which every caller without scratch shares: such
// calls must follow one another on ONE stream, and a launch that never finished leaves its row's
// count behind.
#define GREEDY_BLOCKS 32
#define GREEDY_MAX_ROWS 1024
__device__ unsigned long long g_greedy_best[GREEDY_MAX_ROWS];
__device__ int g_greedy_count[GREEDY_MAX_ROWS];

__global__ void __launch_bounds__(256)
greedy_kernel(const float *__restrict__ logits, int V, int ldl, const int *__restrict__ seq_slot,
              int *__restrict__ hist, int hist_cap, int *__restrict__ hist_count, int *__restrict__ out_tokens,
              unsigned long long *__restrict__ scratch, int scratch_stride) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ unsigned long long s_best[8];
    const int b = blockIdx.y;
    unsigned long long *word = scratch ? scratch + (size_t)b * scratch_stride : &g_greedy_best[b];
    int *count = scratch ? (int *)(scratch + (size_t)b * scratch_stride + 1) : &g_greedy_count[b];
    const float *row = logits + (size_t)b * ldl;
    const int per = (V + GREEDY_BLOCKS - 1) / GREEDY_BLOCKS;
    const int i0 = blockIdx.x * per, i1 = min(V, i0 + per);
    unsigned long long best = 0ull;
    for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
        unsigned long long w = ((unsigned long long)float_key(row[i]) << 32) | (uint32_t)(~(uint32_t)i);
        best = w > best ? w : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    if ((threadIdx.x & 31) == 0) s_best[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); w++) best = s_best[w] > best ? s_best[w] : best;
        atomicMax(word, best);
        __threadfence();
        if (atomicAdd(count, 1) == GREEDY_BLOCKS - 1) {
            __threadfence();
            unsigned long long win = atomicMax(word, 0ull);
            int tok = (int)(~(uint32_t)(win & 0xffffffffull));
            out_tokens[b] = tok;
            *word = 0ull;
            *count = 0;
            if (hist) {
                int slot = seq_slot[b];
                int *h = hist + (size_t)slot * hist_cap;
                int c = hist_count[slot];
                if (c < hist_cap) h[c] = tok;
                else { for (int i = 1; i < hist_cap; i++) h[i - 1] = h[i]; h[hist_cap - 1] = tok; }
                hist_count[slot] = c + 1;
            }
        }
    }
}

// ---- sampling without top-k (top_k <= 0) over a large vocabulary, on NUC_BLOCKS blocks a row.
// The candidates are everything above max - 20 * temp (fastgguf.c:4027-4034); top-p keeps the most probable of them
// whose mass reaches top_p * total (:4039-4047), here as a threshold on the logit found in two passes of 2,048 bins
// each over the candidates' range (entries that fall into the same one of the 4 million bins are kept or dropped
// together); the draw walks the kept entries in index order (the same law as the reference's walk in sorted
// order, another token for the same draw).  Masses are integers, exp((v - max) / temp) * 2^40: integer sums do not
// depend on the order in which blocks arrive, so a row's token depends on its logits and its generator alone.
// One block of 1,024 threads walking the whole row took 1.3 ms at a vocabulary of 128,256.
// State of a row in the caller's scratch (64-bit words; all zero on entry, zero again when the last kernel ends):
#define NUC_BLOCKS 32
#define NUC_BINS 2048
enum { NUC_MAX = 0, NUC_ARRIVE = 1, NUC_SUM = 2, NUC_NEED = 3, NUC_BIN1 = 4, NUC_BIN2 = 5, NUC_BLOCK = 6, NUC_REST = 7,
       NUC_HIST = 16, NUC_MASS = NUC_HIST + NUC_BINS, NUC_WORDS = NUC_MASS + NUC_BLOCKS };
static_assert(NUC_WORDS <= TOPK_CAND, "the state of a row fits the scratch row");

struct NucleusRow {
    float mx, inv_temp, width1, scale1, scale2;        // bins: width1 = 20 temp / 2048 of logit, scale = 1 / width
    float cut;
};
__device__ __forceinline__ NucleusRow nucleus_row(unsigned long long max_word, float temp) {
    NucleusRow r;
    r.mx = key_float((uint32_t)(max_word >> 32));
    r.inv_temp = 1.0f / temp;
    r.cut = r.mx - 20.0f * temp;
    r.width1 = 20.0f * temp / (float)NUC_BINS;
    r.scale1 = (float)NUC_BINS / (20.0f * temp);
    r.scale2 = r.scale1 * (float)NUC_BINS;
    return r;
}
// the same roundings wherever they are evaluated (no contraction left to the compiler)
__device__ __forceinline__ int nucleus_bin1(const NucleusRow &r, float v) {
    return min(NUC_BINS - 1, max(0, (int)__fmul_rn(__fsub_rn(r.mx, v), r.scale1)));
}
__device__ __forceinline__ int nucleus_bin2(const NucleusRow &r, float v, int bin1) {
    const float inside = __fsub_rn(__fsub_rn(r.mx, v), __fmul_rn((float)bin1, r.width1));
    return min(NUC_BINS - 1, max(0, (int)__fmul_rn(inside, r.scale2)));
}
__device__ __forceinline__ unsigned long long nucleus_mass(const NucleusRow &r, float v) {
    const unsigned long long m = (unsigned long long)__fmul_rn(expf(__fmul_rn(__fsub_rn(v, r.mx), r.inv_temp)), 1099511627776.0f);
    return m ? m : 1ull;
}
// bin1 < 0: no top-p, every candidate is kept
__device__ __forceinline__ bool nucleus_kept(const NucleusRow &r, float v, int bin1, int bin2) {
    if (!(v > r.cut)) return false;
    if (bin1 < 0) return true;
    const int b1 = nucleus_bin1(r, v);
    return b1 < bin1 || (b1 == bin1 && nucleus_bin2(r, v, bin1) <= bin2);
}
// true in every thread of the block that arrives last at the row's counter (which it resets)
__device__ __forceinline__ bool nucleus_last_block(unsigned long long *st) {
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const bool last = atomicAdd(&st[NUC_ARRIVE], 1ull) == (unsigned long long)(NUC_BLOCKS - 1);
        if (last) st[NUC_ARRIVE] = 0ull;
        s_last = last;
    }
    __syncthreads();
    __threadfence();
    return s_last != 0;
}
// The first bin, counting from bin 0, at which the running sum of hist[] reaches `need` (there is one: the bins hold
// at least `need`): its index and the sum before it.  256 threads, eight bins each; clears the histogram.
__device__ __forceinline__ void nucleus_scan(unsigned long long *hist, unsigned long long need, unsigned long long *bin_out,
                                             unsigned long long *before_out) {
    __shared__ unsigned long long s_sum[256];
    const int tid = threadIdx.x;
    unsigned long long h[NUC_BINS / 256], mine = 0ull;
#pragma unroll
    for (int j = 0; j < NUC_BINS / 256; j++) { h[j] = __ldcg(&hist[tid * (NUC_BINS / 256) + j]); mine += h[j]; hist[tid * (NUC_BINS / 256) + j] = 0ull; }
    s_sum[tid] = mine;
    __syncthreads();
    unsigned long long before = 0ull;
    for (int t = 0; t < tid; t++) before += s_sum[t];
    if (before < need && before + mine >= need) {
#pragma unroll
        for (int j = 0; j < NUC_BINS / 256; j++) {
            if (before + h[j] >= need) { *bin_out = (unsigned long long)(tid * (NUC_BINS / 256) + j); *before_out = before; break; }
            before += h[j];
        }
    }
}

// 1: the row's largest logit
__global__ void __launch_bounds__(256)
nucleus_max_kernel(const float *__restrict__ logits, int V, int ldl, unsigned long long *__restrict__ scratch, int stride) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ unsigned long long s_best[8];
    const int b = blockIdx.y;
    const float *row = logits + (size_t)b * ldl;
    const int per = (V + NUC_BLOCKS - 1) / NUC_BLOCKS, i0 = blockIdx.x * per, i1 = min(V, i0 + per);
    unsigned long long best = 0ull;
    for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
        const unsigned long long w = ((unsigned long long)float_key(row[i]) << 32) | (uint32_t)(~(uint32_t)i);
        best = w > best ? w : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    if ((threadIdx.x & 31) == 0) s_best[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++) best = s_best[w] > best ? s_best[w] : best;
        atomicMax(&scratch[(size_t)b * stride + NUC_MAX], best);
    }
}

// 2 and 3: masses of the candidates by bin (first pass: of the whole range; second pass: inside the bin where the first found
// the threshold); the block that arrives last finds the bin of the threshold
__global__ void __launch_bounds__(256)
nucleus_hist_kernel(const float *__restrict__ logits, int V, int ldl, float temp, float top_p, int pass,
                    unsigned long long *__restrict__ scratch, int stride) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ unsigned long long s_hist[NUC_BINS];
    unsigned long long *st = scratch + (size_t)blockIdx.y * stride;
    const float *row = logits + (size_t)blockIdx.y * ldl;
    const NucleusRow r = nucleus_row(__ldcg(&st[NUC_MAX]), temp);
    const int bin1 = pass == 2 ? (int)__ldcg(&st[NUC_BIN1]) : 0;
    const int per = (V + NUC_BLOCKS - 1) / NUC_BLOCKS, i0 = blockIdx.x * per, i1 = min(V, i0 + per);
    for (int i = threadIdx.x; i < NUC_BINS; i += blockDim.x) s_hist[i] = 0ull;
    __syncthreads();
    unsigned long long total = 0ull;
    for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
        const float v = row[i];
        if (!(v > r.cut)) continue;
        const unsigned long long m = nucleus_mass(r, v);
        if (pass == 1) { total += m; atomicAdd(&s_hist[nucleus_bin1(r, v)], m); }
        else if (nucleus_bin1(r, v) == bin1) atomicAdd(&s_hist[nucleus_bin2(r, v, bin1)], m);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < NUC_BINS; i += blockDim.x)
        if (s_hist[i]) atomicAdd(&st[NUC_HIST + i], s_hist[i]);
    if (pass == 1) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
        if ((threadIdx.x & 31) == 0 && total) atomicAdd(&st[NUC_SUM], total);
    }
    if (!nucleus_last_block(st)) return;
    unsigned long long need;
    if (pass == 1) {
        const unsigned long long sum = __ldcg(&st[NUC_SUM]);
        need = (unsigned long long)((double)sum * (double)top_p);
        need = need < 1ull ? 1ull : (need > sum ? sum : need);
    } else need = __ldcg(&st[NUC_NEED]);
    __shared__ unsigned long long s_bin, s_before;
    nucleus_scan(st + NUC_HIST, need, &s_bin, &s_before);
    __syncthreads();
    if (threadIdx.x == 0) {
        st[pass == 1 ? NUC_BIN1 : NUC_BIN2] = s_bin;
        st[NUC_NEED] = need - s_before;                 // what the next pass has to find inside the bin
    }
}

// 4: the kept mass of each block's entries; the block that arrives last draws and finds the block the draw falls into
__global__ void __launch_bounds__(256)
nucleus_mass_kernel(const float *__restrict__ logits, int V, int ldl, float temp, int with_top_p, const int *__restrict__ seq_slot,
                    unsigned long long *__restrict__ rng, unsigned long long *__restrict__ scratch, int stride) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ unsigned long long s_w[8];
    unsigned long long *st = scratch + (size_t)blockIdx.y * stride;
    const float *row = logits + (size_t)blockIdx.y * ldl;
    const NucleusRow r = nucleus_row(__ldcg(&st[NUC_MAX]), temp);
    const int bin1 = with_top_p ? (int)__ldcg(&st[NUC_BIN1]) : -1, bin2 = with_top_p ? (int)__ldcg(&st[NUC_BIN2]) : 0;
    const int per = (V + NUC_BLOCKS - 1) / NUC_BLOCKS, i0 = blockIdx.x * per, i1 = min(V, i0 + per);
    unsigned long long total = 0ull;
    for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
        const float v = row[i];
        if (nucleus_kept(r, v, bin1, bin2)) total += nucleus_mass(r, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    if ((threadIdx.x & 31) == 0) s_w[threadIdx.x >> 5] = total;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++) total += s_w[w];
        st[NUC_MASS + blockIdx.x] = total;
    }
    if (!nucleus_last_block(st)) return;
    if (threadIdx.x == 0) {
        unsigned long long tot = 0ull;
        for (int k = 0; k < NUC_BLOCKS; k++) tot += __ldcg(&st[NUC_MASS + k]);
        const int slot = seq_slot[blockIdx.y];
        uint64_t g = rng[slot];
        const unsigned long long u = xorshift64star(&g) >> 40;          // 24 bits, as rng_uniform (fastgguf.c:3979-3981)
        rng[slot] = g;
        // r = u / 2^24 * tot, in integers: tot < 2^58, so the product needs its high word
        unsigned long long rest = (__umul64hi(u, tot) << 40) | ((u * tot) >> 24);
        int blk = 0;
        for (; blk < NUC_BLOCKS - 1; blk++) {
            const unsigned long long m = __ldcg(&st[NUC_MASS + blk]);
            if (rest < m) break;
            rest -= m;
        }
        st[NUC_BLOCK] = (unsigned long long)blk;
        st[NUC_REST] = rest;
    }
}

// 5: the block the draw fell into walks its entries in index order; it also writes the token and clears the state
__global__ void __launch_bounds__(256)
nucleus_walk_kernel(const float *__restrict__ logits, int V, int ldl, float temp, int with_top_p, const int *__restrict__ seq_slot,
                    int *__restrict__ hist, int hist_cap, int *__restrict__ hist_count, int *__restrict__ out_tokens,
                    unsigned long long *__restrict__ scratch, int stride) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ unsigned long long s_part[256];
    unsigned long long *st = scratch + (size_t)blockIdx.x * stride;
    const float *row = logits + (size_t)blockIdx.x * ldl;
    const unsigned long long max_word = st[NUC_MAX];
    const NucleusRow r = nucleus_row(max_word, temp);
    const int bin1 = with_top_p ? (int)st[NUC_BIN1] : -1, bin2 = with_top_p ? (int)st[NUC_BIN2] : 0;
    const int blk = (int)st[NUC_BLOCK];
    const int per = (V + NUC_BLOCKS - 1) / NUC_BLOCKS, i0 = blk * per, i1 = min(V, i0 + per);
    // thread t takes the entries [i0 + t * span, i0 + (t + 1) * span): the threads in order cover the block in index order
    const int span = (per + 255) / 256, a0 = min(i1, i0 + (int)threadIdx.x * span), a1 = min(i1, a0 + span);
    unsigned long long mine = 0ull;
    for (int i = a0; i < a1; i++) { const float v = row[i]; if (nucleus_kept(r, v, bin1, bin2)) mine += nucleus_mass(r, v); }
    s_part[threadIdx.x] = mine;
    __syncthreads();
    if (threadIdx.x != 0) return;
    unsigned long long rest = st[NUC_REST];
    int t = 0;
    for (; t < 255; t++) { if (rest < s_part[t]) break; rest -= s_part[t]; }
    int chosen = (int)(~(uint32_t)(max_word & 0xffffffffull));           // (never used: the walk ends inside the kept entries)
    int last = -1;
    const int b0 = min(i1, i0 + t * span), b1 = min(i1, b0 + span);
    for (int i = b0; i < b1; i++) {
        const float v = row[i];
        if (!nucleus_kept(r, v, bin1, bin2)) continue;
        last = i;
        const unsigned long long m = nucleus_mass(r, v);
        if (rest < m) break;
        rest -= m;
    }
    if (last >= 0) chosen = last;
    out_tokens[blockIdx.x] = chosen;
    if (hist) {
        const int slot = seq_slot[blockIdx.x];
        int *h = hist + (size_t)slot * hist_cap;
        int c = hist_count[slot];
        if (c < hist_cap) h[c] = chosen;
        else { for (int i = 1; i < hist_cap; i++) h[i - 1] = h[i]; h[hist_cap - 1] = chosen; }
        hist_count[slot] = c + 1;
    }
    st[NUC_MAX] = 0ull; st[NUC_SUM] = 0ull; st[NUC_NEED] = 0ull; st[NUC_BIN1] = 0ull; st[NUC_BIN2] = 0ull;
    st[NUC_BLOCK] = 0ull; st[NUC_REST] = 0ull;
}

extern "C" int fg_sample(float *logits, int B, int V, int ldl, float temp, int top_k, float top_p,
                         float repeat_penalty, int repeat_last_n, const int *seq_slot,
                         unsigned long long *rng, int *hist, int hist_cap, int *hist_count,
                         const int *stop_ids, int n_stop, int *out_tokens, unsigned long long *scratch,
                         cudaStream_t stream) {
    if (B <= 0) return 0;
    if (top_k > MAX_TOP_K) return FG_ERR_BAD_SIZE;
    bool penalizes = hist && repeat_penalty > 0.f && repeat_penalty != 1.0f && repeat_last_n > 0;
    if (temp <= 0.f && !penalizes && (scratch ? B <= 65535 : B <= GREEDY_MAX_ROWS))
        return fg_launch(greedy_kernel, dim3(GREEDY_BLOCKS, B), dim3(256), 0, stream, (const float *)logits, V, ldl,
                         seq_slot, hist, hist_cap, hist_count, out_tokens, scratch, TOPK_CAND);
    SampleParams sp{temp, top_p, repeat_penalty, top_k, repeat_last_n};
    if (temp > 0.f && top_k > 0 && top_k <= TOPK_MAX_K && scratch && B <= 65535) {
        // two stages; `scratch` holds B * 4096 words
        int k = top_k < V ? top_k : V;
        int K = k <= 64 ? 64 : 128;                        // words a segment hands over (>= k); unused ones are zero
        int n_blocks = (V + TOPK_SEG - 1) / TOPK_SEG;
        int padded = 1;
        while (padded < n_blocks) padded <<= 1;               // the second stage merges a power of two of segments
        if (padded * K <= TOPK_CAND) {
            if (penalizes) {
                int e = fg_launch(penalty_kernel, dim3(B), dim3(64), 0, stream, logits, V, ldl, repeat_penalty,
                                  repeat_last_n, seq_slot, (const int *)hist, hist_cap, (const int *)hist_count, stop_ids, n_stop);
                if (e) return e;
            }
            int e = fg_launch(topk_stage1_kernel, dim3(n_blocks, B), dim3(256), 0, stream, (const float *)logits, V, ldl,
                              K, n_blocks, scratch);
            if (e) return e;
            return fg_launch(topk_stage2_kernel, dim3(B), dim3(256), 0, stream, (const unsigned long long *)scratch,
                             n_blocks, K, k, sp, seq_slot, rng, hist, hist_cap, hist_count, out_tokens);
        }
    }
    if (temp > 0.f && top_k <= 0 && scratch && B <= 65535 && V >= 8192) {
        // no top-k over a large vocabulary: NUC_BLOCKS blocks a row, five short kernels
        const int with_top_p = top_p > 0.f && top_p < 1.0f;
        int e = 0;
        if (penalizes)
            e = fg_launch(penalty_kernel, dim3(B), dim3(64), 0, stream, logits, V, ldl, repeat_penalty, repeat_last_n, seq_slot,
                          (const int *)hist, hist_cap, (const int *)hist_count, stop_ids, n_stop);
        if (!e) e = fg_launch(nucleus_max_kernel, dim3(NUC_BLOCKS, B), dim3(256), 0, stream, (const float *)logits, V, ldl, scratch, TOPK_CAND);
        for (int pass = 1; pass <= 2 && with_top_p && !e; pass++)
            e = fg_launch(nucleus_hist_kernel, dim3(NUC_BLOCKS, B), dim3(256), 0, stream, (const float *)logits, V, ldl, temp, top_p,
                          pass, scratch, TOPK_CAND);
        if (!e) e = fg_launch(nucleus_mass_kernel, dim3(NUC_BLOCKS, B), dim3(256), 0, stream, (const float *)logits, V, ldl, temp,
                              with_top_p, seq_slot, rng, scratch, TOPK_CAND);
        if (!e) e = fg_launch(nucleus_walk_kernel, dim3(B), dim3(256), 0, stream, (const float *)logits, V, ldl, temp, with_top_p,
                              seq_slot, hist, hist_cap, hist_count, out_tokens, scratch, TOPK_CAND);
        return e;
    }
    sample_kernel<<<B, SAMPLE_THREADS, 0, stream>>>(logits, V, ldl, sp, seq_slot, rng, hist, hist_cap,
                                                    hist_count, stop_ids, n_stop, out_tokens);
    return FG_LAUNCH_CHECK();
}

// plain argmax of each row (lowest index on ties), for callers that only want greedy tokens
__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float *__restrict__ logits, int V, int ldl, int *__restrict__ out) {
    int best = block_argmax(logits + (size_t)blockIdx.x * ldl, V, nullptr);
    if (threadIdx.x == 0) out[blockIdx.x] = best;
}

extern "C" int fg_argmax(const float *logits, int B, int V, int ldl, int *out, cudaStream_t stream) {
    if (B <= 0) return 0;
    argmax_kernel<<<B, SAMPLE_THREADS, 0, stream>>>(logits, V, ldl, out);
    return FG_LAUNCH_CHECK();
}
