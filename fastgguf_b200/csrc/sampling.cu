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

// ---- top-k sampling in two stages (k <= 128): the vocabulary of a row is split over TOPK_BLOCKS
// blocks; each selects the k best of its segment as 64-bit words (value key, then lower index first)
// with a radix select in shared memory; one block per row then sorts the TOPK_BLOCKS * k candidates
// and draws exactly as the single-block kernel does.  The k best of the row are among the k best of
// each segment, and the words order them totally, so the result is the single-block kernel's.
#define TOPK_SEG 4096                  // most vocabulary entries a stage-1 block takes
#define TOPK_CAND 2048                 // candidates per row after stage 1
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

__global__ void __launch_bounds__(256)
topk_stage1_kernel(const float *__restrict__ logits, int V, int ldl, int k, int n_blocks,
                   unsigned long long *__restrict__ cand) {        // [B, n_blocks * k], zero where unused
    __shared__ uint32_t keys[TOPK_SEG];
    __shared__ int hist[256];
    __shared__ int misc[4];
    __shared__ int wsum[8];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y, tid = threadIdx.x;
    const float *row = logits + (size_t)b * ldl;
    const int per = (V + n_blocks - 1) / n_blocks;
    const int i0 = blockIdx.x * per, n = max(0, min(V, i0 + per) - i0);
    unsigned long long *out = cand + ((size_t)b * n_blocks + blockIdx.x) * k;
    for (int i = tid; i < n; i += blockDim.x) keys[i] = float_key(row[i0 + i]);
    for (int i = tid; i < k; i += blockDim.x) out[i] = 0ull;
    __syncthreads();
    if (n == 0) return;
    const int kk = min(k, n);
    uint32_t prefix = 0, mask = 0;
    int need = kk;
    for (int shift = 24; shift >= 0; shift -= 8) {
        hist[tid] = 0;
        __syncthreads();
        for (int i = tid; i < n; i += blockDim.x)
            if ((keys[i] & mask) == prefix) atomicAdd(&hist[(keys[i] >> shift) & 255], 1);
        __syncthreads();
        // the bin that holds the `need`-th largest matching key, by a suffix sum over the 256 bins with 256 threads
        // (thread t takes bin 255 - t): the one whose running count reaches `need`.  One thread walking the bins took
        // as long as the counting itself.
        {
            const int x = hist[255 - tid], lane = tid & 31, w = tid >> 5;
            int incl = x;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { int y = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += y; }
            if (lane == 31) wsum[w] = incl;
            if (tid == 0) { misc[0] = 0; misc[1] = need; }       // never kept: the matching keys are at least `need`
            __syncthreads();
            int before = 0;
            for (int j = 0; j < w; j++) before += wsum[j];
            incl += before;
            if (incl >= need && incl - x < need) { misc[0] = 255 - tid; misc[1] = need - (incl - x); }
        }
        __syncthreads();
        prefix |= (uint32_t)misc[0] << shift;
        mask |= 255u << shift;
        need = misc[1];
        __syncthreads();
    }
    // everything above the k-th key, and the first `need` equal to it in index order
    if (tid == 0) misc[2] = 0;
    __syncthreads();
    int taken_eq = 0;
    for (int c0 = 0; c0 < n; c0 += blockDim.x) {
        int i = c0 + tid;
        uint32_t key = i < n ? keys[i] : 0u;
        int gt = i < n && key > prefix, eq = i < n && key == prefix;
        unsigned ball = __ballot_sync(0xffffffffu, eq);
        int lane = tid & 31, w = tid >> 5;
        if (lane == 0) wsum[w] = __popc(ball);
        __syncthreads();
        int before = 0, tot = 0;
        for (int j = 0; j < 8; j++) { if (j < w) before += wsum[j]; tot += wsum[j]; }
        int rank = taken_eq + before + __popc(ball & ((1u << lane) - 1));
        if (gt || (eq && rank < need)) {
            int at = atomicAdd(&misc[2], 1);
            out[at] = ((unsigned long long)key << 32) | (uint32_t)(~(uint32_t)(i0 + i));
        }
        taken_eq += tot;
        __syncthreads();
    }
}

__global__ void __launch_bounds__(1024)
topk_stage2_kernel(const unsigned long long *__restrict__ cand_in, int n_cand, int k, SampleParams sp,
                   const int *__restrict__ seq_slot, unsigned long long *__restrict__ rng,
                   int *__restrict__ hist, int hist_cap, int *__restrict__ hist_count, int *__restrict__ out_tokens) {
    __shared__ unsigned long long cand[TOPK_CAND];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x, tid = threadIdx.x, slot = seq_slot[b];
    for (int i = tid; i < TOPK_CAND; i += blockDim.x) cand[i] = i < n_cand ? cand_in[(size_t)b * n_cand + i] : 0ull;
    __syncthreads();
    for (int size = 2; size <= TOPK_CAND; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int i = tid; i < TOPK_CAND; i += blockDim.x) {
                int j = i ^ stride;
                if (j > i) {
                    unsigned long long x = cand[i], y = cand[j];
                    bool desc = (i & size) == 0;
                    if (desc ? x < y : x > y) { cand[i] = y; cand[j] = x; }
                }
            }
            __syncthreads();
        }
    }
    // the weights exp((v - top) / temp) of the k best, one thread each; the sums below add them in index order,
    // as the serial sampler does (the same floats in the same order: the same token)
    __shared__ float wgt[TOPK_MAX_K];
    if (tid < k) wgt[tid] = expf((key_float((uint32_t)(cand[tid] >> 32)) - key_float((uint32_t)(cand[0] >> 32))) / sp.temp);
    __syncthreads();
    if (tid == 0) {
        int n = 0;
        while (n < k && cand[n] != 0ull) n++;
        float sum = 0.f;
        for (int i = 0; i < n; i++) sum += wgt[i];
        int keep = n;
        if (sp.top_p > 0.f && sp.top_p < 1.0f) {
            float cum = 0.f, lim = sp.top_p * sum;
            for (int i = 0; i < n; i++) {
                cum += wgt[i];
                if (cum >= lim) { keep = i + 1; break; }
            }
        }
        float tot = 0.f;
        for (int i = 0; i < keep; i++) tot += wgt[i];
        uint64_t st = rng[slot];
        float r = (float)(xorshift64star(&st) >> 40) / 16777216.0f * tot;
        rng[slot] = st;
        int pick = keep - 1;
        for (int i = 0; i < keep; i++) {
            r -= wgt[i];
            if (r < 0.f) { pick = i; break; }
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
        // two stages; `scratch` holds B * 2048 words
        int k = top_k < V ? top_k : V;
        int n_blocks = TOPK_CAND / (k <= 64 ? 64 : 128);
        if ((V + n_blocks - 1) / n_blocks <= TOPK_SEG) {
            int kc = k <= 64 ? 64 : 128;                   // slots per block (>= k); unused ones stay zero
            if (penalizes) {
                int e = fg_launch(penalty_kernel, dim3(B), dim3(64), 0, stream, logits, V, ldl, repeat_penalty,
                                  repeat_last_n, seq_slot, (const int *)hist, hist_cap, (const int *)hist_count, stop_ids, n_stop);
                if (e) return e;
            }
            int e = fg_launch(topk_stage1_kernel, dim3(n_blocks, B), dim3(256), 0, stream, (const float *)logits, V, ldl,
                              kc < k ? kc : k, n_blocks, scratch);
            if (e) return e;
            int per_block = kc < k ? kc : k;
            return fg_launch(topk_stage2_kernel, dim3(B), dim3(1024), 0, stream, (const unsigned long long *)scratch,
                             n_blocks * per_block, k, sp, seq_slot, rng, hist, hist_cap, hist_count, out_tokens);
        }
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
