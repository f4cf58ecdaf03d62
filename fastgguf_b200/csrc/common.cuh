// Shared helpers of every kernel file: dtype codes, f32 <-> storage conversion, block
// reductions with a fixed order, and the launch-error convention (each extern "C" launcher
// returns the cudaError_t of its launch as an int; 0 is success).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

// dtype codes shared with the Python side (fastgguf_b200/ops/lib.py)
#define FG_F32 0
#define FG_BF16 1

// error codes above the CUDA range, returned by launchers for refused arguments
#define FG_ERR_BAD_DTYPE 10001
#define FG_ERR_BAD_SIZE 10002

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// store a float into a buffer whose dtype is only known at run time
__device__ __forceinline__ void store_as(void *base, int dtype, size_t idx, float v) {
    if (dtype == FG_F32) ((float *)base)[idx] = v;
    else ((bf16 *)base)[idx] = __float2bfloat16_rn(v);
}
__device__ __forceinline__ float load_as(const void *base, int dtype, size_t idx) {
    return dtype == FG_F32 ? ((const float *)base)[idx] : __bfloat162float(((const bf16 *)base)[idx]);
}

// The index of this thread's warp, read through a shuffle from lane 0.  The value is the same as threadIdx.x >> 5,
// but the compiler then knows that it does not differ between the lanes of a warp, and branches on it (the roles
// of a warp-specialised kernel) are uniform.  With the plain shift such branches counted as divergent, and warp
// shuffles inside them were measured at eight times their usual latency.
__device__ __forceinline__ int warp_index() { return __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum / max with a fixed order: xor-shuffle tree inside each warp, then the warp
// totals are added in warp order by every thread.  `scratch` holds at least 32 floats.  The
// result is the same in every thread.  Contains two __syncthreads().
__device__ __forceinline__ float block_sum(float v, float *scratch) {
    v = warp_sum(v);
    int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[w] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < nw; i++) t += scratch[i];
    return t;
}
__device__ __forceinline__ float block_max(float v, float *scratch) {
    v = warp_max(v);
    int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[w] = v;
    __syncthreads();
    float t = -INFINITY;
    for (int i = 0; i < nw; i++) t = fmaxf(t, scratch[i]);
    return t;
}

#define FG_LAUNCH_CHECK() ((int)cudaGetLastError())

// One lane of a converged warp (elect.sync).  A loop that the whole warp walks, with only the
// asynchronous instructions (tcgen05.mma, tcgen05.commit, TMA copies) under this predicate, keeps its
// counters, barrier addresses and descriptors in the uniform datapath; the same loop inside
// `if (lane == 0)` pays a move per operand and measured 490 against 290 cycles per K-block of four
// small MMAs.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile("{\n\t.reg .b32 rx;\n\t.reg .pred px;\n\telect.sync rx|px, %1;\n\t@px mov.s32 %0, 1;\n\t}"
                 : "+r"(pred) : "r"(0xffffffffu));
    return pred != 0;
}

// ------------------------------------------------------------------ dependent launches
// Every kernel of this library is launched with programmatic stream serialization: it may
// start while the kernel before it on the stream is still running.  Each kernel calls
// pdl_launch_dependents() at its start (its successor may be scheduled) and pdl_wait() before
// it first touches memory that an earlier kernel writes or reads; what it does before that
// wait (barrier set-up, fetching weights, which no kernel writes) overlaps the predecessor.
// The wait returns when every earlier kernel of the stream has finished (each of them waits too, so
// completion is transitive); BEFORE it, not only the predecessor but kernels further back may still
// run, because a kernel releases its successor at its start.  So a kernel may read before its wait
// only memory that nothing launched since the last full barrier of the stream writes - a full barrier
// being a memory copy, or the boundary of a graph launch.  Weights qualify always.  Positions, page
// tables and an entry's own cache pool qualify for the fused decode attention because the engine writes
// positions and tables only by the copy that opens a step or by `decode_advance_kernel`, the LAST
// node of the decode graph, and because an entry's pool is appended to by that entry's kernel alone.
// FASTGGUF_PDL=0 turns the attribute off; the two instructions are then no-ops.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

#include <cstdlib>
// Function attributes (the dynamic shared memory limit) belong to a kernel on ONE device: a launcher sets them the
// first time it runs on each device.  True once per device for the call site that owns `s`.
struct FgPerDevice { bool done[64]; };
static inline bool fg_needs_setup(FgPerDevice &s) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (s.done[dev]) return false;
    s.done[dev] = true;
    return true;
}

static inline bool fg_pdl_enabled() {
    static int v = -1;
    if (v < 0) { const char *e = getenv("FASTGGUF_PDL"); v = !(e && e[0] == '0'); }
    return v != 0;
}

template <typename... KArgs, typename... Args>
static inline int fg_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                            Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = fg_pdl_enabled() ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Plain stream order: the kernel starts when everything before it on the stream has finished (its
// griddepcontrol instructions are then no-ops; its successor may still be released early by it).
template <typename... KArgs, typename... Args>
static inline int fg_launch_in_order(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cfg.attrs = nullptr;
    cfg.numAttrs = 0;
    return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// the same, for a thread-block cluster of (1, 1, cluster_z) CTAs
template <typename... KArgs, typename... Args>
static inline int fg_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    int cluster_z, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (fg_pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        n++;
    }
    if (cluster_z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1; attr[n].val.clusterDim.y = 1; attr[n].val.clusterDim.z = cluster_z;
        n++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
