// The few kernels the host library itself needs while LOADING a model: dtype conversion, row gathers for
// fused / permuted weight matrices, seeded random weights, a scale.  None is on the path of a step.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "device.hpp"
#include "random_values.hpp"

namespace fg {

template <typename S>
__device__ __forceinline__ float load_as_float(const S *p, int64_t i);
template <> __device__ __forceinline__ float load_as_float<float>(const float *p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16 *p, int64_t i) { return __bfloat162float(p[i]); }
template <> __device__ __forceinline__ float load_as_float<__half>(const __half *p, int64_t i) { return __half2float(p[i]); }

template <typename S, typename D>
__global__ void convert_kernel(const S *__restrict__ src, D *__restrict__ dst, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        float v = load_as_float<S>(src, i);
        if constexpr (sizeof(D) == 4) dst[i] = v;
        else dst[i] = __float2bfloat16_rn(v);
    }
}

__global__ void convert_i64_i32_kernel(const long long *__restrict__ src, int *__restrict__ dst, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        dst[i] = (int)src[i];
}

static int grid_for(int64_t n) {
    int64_t g = (n + 255) / 256;
    return (int)(g < 1 ? 1 : g > 148 * 16 ? 148 * 16 : g);
}

void dev_convert(const void *src, int sd, void *dst, int dd, int64_t n, cudaStream_t s) {
    if (n <= 0) return;
    if (sd == dd) {
        FG_CUDA(cudaMemcpyAsync(dst, src, (size_t)n * elem_size(sd), cudaMemcpyDeviceToDevice, s));
        return;
    }
    int g = grid_for(n);
#define CONV(S, D) convert_kernel<S, D><<<g, 256, 0, s>>>((const S *)src, (D *)dst, n)
    if (sd == FG_F32 && dd == FG_BF16) CONV(float, __nv_bfloat16);
    else if (sd == FG_BF16 && dd == FG_F32) CONV(__nv_bfloat16, float);
    else if (sd == FG_F16 && dd == FG_F32) CONV(__half, float);
    else if (sd == FG_F16 && dd == FG_BF16) CONV(__half, __nv_bfloat16);
    else if (sd == FG_I64 && dd == FG_I32) convert_i64_i32_kernel<<<g, 256, 0, s>>>((const long long *)src, (int *)dst, n);
    else fail(FG_E_WEIGHTS, format("no conversion from dtype %d to dtype %d", sd, dd));
#undef CONV
    FG_CUDA(cudaGetLastError());
}

__global__ void gather_rows_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst,
                                   const long long *__restrict__ rows, int64_t row_bytes) {
    const uint8_t *s = src + rows[blockIdx.x] * row_bytes;
    uint8_t *d = dst + blockIdx.x * row_bytes;
    if (row_bytes % 4 == 0) {
        for (int64_t i = threadIdx.x; i < row_bytes / 4; i += blockDim.x) ((uint32_t *)d)[i] = ((const uint32_t *)s)[i];
    } else {
        for (int64_t i = threadIdx.x; i < row_bytes; i += blockDim.x) d[i] = s[i];
    }
}

void dev_gather_rows(const void *src, void *dst, const std::vector<int64_t> &rows, int64_t cols, int dtype, cudaStream_t s) {
    if (rows.empty()) return;
    long long *idx = nullptr;
    FG_CUDA(cudaMalloc(&idx, rows.size() * sizeof(long long)));
    std::vector<long long> host(rows.begin(), rows.end());
    cudaError_t e = cudaMemcpyAsync(idx, host.data(), host.size() * sizeof(long long), cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) {
        gather_rows_kernel<<<(unsigned)rows.size(), 128, 0, s>>>((const uint8_t *)src, (uint8_t *)dst, idx,
                                                                 cols * elem_size(dtype));
        e = cudaGetLastError();
    }
    cudaError_t e2 = cudaStreamSynchronize(s);       // `host` and `idx` go away with this call
    cudaFree(idx);
    FG_CUDA(e);
    FG_CUDA(e2);
}

template <typename D>
__global__ void fill_random_kernel(D *__restrict__ dst, int64_t n, uint64_t seed, uint64_t nh, int init, float std) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        float v = random_weight(seed, nh, (uint64_t)i, init, std);
        if constexpr (sizeof(D) == 4) dst[i] = v;
        else dst[i] = __float2bfloat16_rn(v);
    }
}

void dev_fill_random(void *dst, int dtype, int64_t n, uint64_t seed, uint64_t nh, int init, float std, cudaStream_t s) {
    if (n <= 0) return;
    if (dtype == FG_I32) {
        FG_CUDA(cudaMemsetAsync(dst, 0, (size_t)n * 4, s));
        return;
    }
    int g = grid_for(n);
    if (dtype == FG_F32) fill_random_kernel<float><<<g, 256, 0, s>>>((float *)dst, n, seed, nh, init, std);
    else if (dtype == FG_BF16) fill_random_kernel<__nv_bfloat16><<<g, 256, 0, s>>>((__nv_bfloat16 *)dst, n, seed, nh, init, std);
    else fail(FG_E_USAGE, "random weights are float32 or bfloat16");
    FG_CUDA(cudaGetLastError());
}

__global__ void scale_f32_kernel(float *x, int64_t n, float scale) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) x[i] *= scale;
}

void dev_scale_f32(float *x, int64_t n, float scale, cudaStream_t s) {
    if (n <= 0) return;
    scale_f32_kernel<<<grid_for(n), 256, 0, s>>>(x, n, scale);
    FG_CUDA(cudaGetLastError());
}

}  // namespace fg
