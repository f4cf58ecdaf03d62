// What the host needs from the device: checked CUDA calls, tensors as (pointer, dtype, shape, row stride),
// a bump allocator for a step's activations, and the kernel libraries' launchers looked up on first use.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <string>
#include <vector>

#include "../fastgguf_b200.h"
#include "../fastgguf_parts.h"
#include "errors.hpp"

namespace fg {

#define FG_CUDA(call)                                                                                        \
    do {                                                                                                     \
        cudaError_t e_ = (call);                                                                             \
        if (e_ != cudaSuccess)                                                                               \
            ::fg::fail(FG_E_DEVICE, ::fg::format("%s failed: %s", #call, cudaGetErrorString(e_)));           \
    } while (0)

// A launcher's return code -> exception (0 passes).
void check_kernel(int code, const char *what);

// A launcher of libfg_<module>.so, opened on first use from the folder of this library (or
// $FASTGGUF_LIB_DIR).  A missing library is an error: there is no other implementation to fall back to.
void *kernel_symbol(const char *module, const char *name);
#define FG_KERNEL(module, fn) (reinterpret_cast<decltype(&::fn)>(::fg::kernel_symbol(module, #fn)))
// every launcher call made so far (each launches at least one kernel)
long long launch_count();
void count_launch();
#define FG_LAUNCH(module, fn, ...)                                                                           \
    do {                                                                                                     \
        ::fg::count_launch();                                                                                \
        ::fg::ProfileScope fg_profile_scope_(#fn);                                                           \
        ::fg::check_kernel(FG_KERNEL(module, fn)(__VA_ARGS__), #fn);                                         \
    } while (0)
// Per-launcher device times, for `--profile`: while it is on, every launcher call is bracketed by two events on
// `stream` (which also ends the overlap of dependent launches: the times are those of kernels running one after
// another) and decode steps run eagerly, since events inside a recorded graph cannot be read.  One engine at a time.
void profile_enable(bool on, cudaStream_t stream);
bool profile_on();
// [{"name": launcher (and shape), "calls": n, "ms": total}, ...] by falling time; waits for the stream, clears the records
std::string profile_report_json();
struct ProfileScope {
    explicit ProfileScope(const char *name, const char *detail = nullptr);
    ~ProfileScope();
    int index = -1;
};
// Reads and clears the error flags of the kernel libraries that are loaded; throws FG_E_KERNEL if one is set.
void raise_on_device_error(const char *where);

struct Tensor {
    void *data = nullptr;
    int dtype = FG_F32;
    int64_t rows = 0, cols = 0;      // a matrix [rows, cols]; vectors have rows == 1
    int64_t ld = 0;                  // elements between rows
    bool defined() const { return data != nullptr; }
    int64_t numel() const { return rows * cols; }
    template <typename T> T *ptr() const { return (T *)data; }
    Tensor row_range(int64_t begin, int64_t end) const;
    fg_dev_tensor view() const;
};
int elem_size(int dtype);

// Device memory for the activations of one step.  Allocation bumps a cursor through a list of blocks; `reset`
// starts over.  The sequence of allocations of a step is deterministic, so a step that is run once to warm up and
// then recorded into a CUDA graph gets the same addresses both times; blocks are only added outside a recording.
// A step that needed more than a lane's first block got further blocks; the next `reset` replaces them by ONE block
// of the largest need seen so far, so that steps of changing shapes do not pile up memory.
// Three lanes keep a deep model's step small: what lives for the whole step (the residual stream, the step's
// integers, the logits) goes to lane 0, and the temporaries of layer i to lane 1 + (i & 1), which starts over when
// layer i begins - what layer i - 1 handed over (a started norm) lies in the other lane and stays until layer i + 1.
// All work of a step is ordered on one stream, so memory of layer i - 2 is free when layer i writes it.
class Arena {
public:
    explicit Arena(size_t block_bytes = (size_t)64 << 20) : block_bytes_(block_bytes) {}
    ~Arena();
    Arena(const Arena &) = delete;
    void *alloc(size_t bytes);
    Tensor matrix(int64_t rows, int64_t cols, int dtype);
    void reset();                       // a new step: every lane starts over
    void begin_layer(int i);            // allocations now go to the lane of layer i, which starts over
    void end_layers() { cur_ = 0; }     // back to the step's own lane
    void forbid_growth(bool v) { frozen_ = v; }
    size_t bytes_reserved() const;

private:
    struct Block { void *p; size_t size; };
    struct Lane {
        std::vector<Block> blocks;
        size_t block = 0, offset = 0, used = 0, peak = 0;
    };
    Lane lanes_[3];
    int cur_ = 0;
    size_t block_bytes_;
    bool frozen_ = false;
};

// Device memory that lives as long as its owner.
class DeviceBuffer {
public:
    DeviceBuffer() = default;
    explicit DeviceBuffer(size_t bytes, const char *what = "device memory");
    ~DeviceBuffer();
    DeviceBuffer(DeviceBuffer &&o) noexcept : p_(o.p_), bytes_(o.bytes_) { o.p_ = nullptr; o.bytes_ = 0; }
    DeviceBuffer &operator=(DeviceBuffer &&o) noexcept;
    DeviceBuffer(const DeviceBuffer &) = delete;
    void *get() const { return p_; }
    size_t bytes() const { return bytes_; }

private:
    void *p_ = nullptr;
    size_t bytes_ = 0;
};

// ---- small kernels of the host library (host_kernels.cu)
void dev_convert(const void *src, int src_dtype, void *dst, int dst_dtype, int64_t n, cudaStream_t s);
// dst[r, :] = src[rows[r], :] (rows on the host, uploaded by the call); cols elements of `dtype`
void dev_gather_rows(const void *src, void *dst, const std::vector<int64_t> &rows, int64_t cols, int dtype, cudaStream_t s);
void dev_fill_random(void *dst, int dtype, int64_t n, uint64_t seed, uint64_t name_hash, int init, float std, cudaStream_t s);
void dev_scale_f32(float *x, int64_t n, float scale, cudaStream_t s);

}  // namespace fg
