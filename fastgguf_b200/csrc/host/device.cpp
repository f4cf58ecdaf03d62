// See device.hpp.
#include "device.hpp"

#include <dlfcn.h>

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <map>
#include <mutex>
#include <vector>

namespace fg {

void check_kernel(int code, const char *what) {
    if (code == 0) return;
    const char *msg = nullptr;
    switch (code) {
    case 10001: msg = "unsupported dtype combination"; break;
    case 10002: msg = "a size outside what this kernel takes"; break;
    case 10003: msg = "device-side wait ran out (pipeline error flag set)"; break;
    case 10004: msg = "could not encode a TMA tensor map"; break;
    case 10005: msg = "the request exceeds the fixed scratch array of the no-allocation entry point"; break;
    }
    if (msg) fail(FG_E_KERNEL, format("%s: %s", what, msg));
    fail(FG_E_DEVICE, format("%s: CUDA error %d (%s)", what, code, cudaGetErrorString((cudaError_t)code)));
}

static std::mutex g_lib_mutex;
static std::map<std::string, void *> g_libs;
static std::atomic<long long> g_launches{0};

long long launch_count() { return g_launches.load(); }
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

// ---- per-launcher times
namespace {
struct ProfileRecord { std::string name; cudaEvent_t begin, end; };
struct ProfileState {
    bool on = false;
    cudaStream_t stream = nullptr;
    std::vector<ProfileRecord> records;
} g_profile;
}  // namespace

static void profile_clear() {
    for (auto &r : g_profile.records) { cudaEventDestroy(r.begin); cudaEventDestroy(r.end); }
    g_profile.records.clear();
}

void profile_enable(bool on, cudaStream_t stream) {
    if (g_profile.on && g_profile.stream) cudaStreamSynchronize(g_profile.stream);
    profile_clear();
    g_profile.on = on;
    g_profile.stream = stream;
}

bool profile_on() { return g_profile.on; }

ProfileScope::ProfileScope(const char *name, const char *detail) {
    if (!g_profile.on) return;
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(g_profile.stream, &st) != cudaSuccess || st != cudaStreamCaptureStatusNone) return;
    ProfileRecord r;
    r.name = detail ? std::string(name) + " " + detail : std::string(name);
    if (cudaEventCreate(&r.begin) != cudaSuccess) return;
    if (cudaEventCreate(&r.end) != cudaSuccess) { cudaEventDestroy(r.begin); return; }
    cudaEventRecord(r.begin, g_profile.stream);
    index = (int)g_profile.records.size();
    g_profile.records.push_back(std::move(r));
}

ProfileScope::~ProfileScope() {
    if (index >= 0 && index < (int)g_profile.records.size()) cudaEventRecord(g_profile.records[(size_t)index].end, g_profile.stream);
}

std::string profile_report_json() {
    if (g_profile.stream) FG_CUDA(cudaStreamSynchronize(g_profile.stream));
    std::map<std::string, std::pair<long long, double>> by_name;
    for (auto &r : g_profile.records) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, r.begin, r.end) != cudaSuccess) continue;
        auto &e = by_name[r.name];
        e.first++;
        e.second += ms;
    }
    profile_clear();
    std::vector<std::pair<std::string, std::pair<long long, double>>> rows(by_name.begin(), by_name.end());
    std::sort(rows.begin(), rows.end(), [](const auto &a, const auto &b) { return a.second.second > b.second.second; });
    std::string out = "[";
    for (size_t i = 0; i < rows.size(); i++) {
        std::string name;
        for (char c : rows[i].first) { if (c == '"' || c == '\\') name += '\\'; name += c; }
        out += format("%s{\"name\": \"%s\", \"calls\": %lld, \"ms\": %.6f}", i ? ", " : "", name.c_str(), rows[i].second.first, rows[i].second.second);
    }
    return out + "]";
}

static std::string own_folder() {
    Dl_info info;
    if (dladdr((void *)&own_folder, &info) && info.dli_fname) {
        std::string p = info.dli_fname;
        size_t slash = p.rfind('/');
        return slash == std::string::npos ? "." : p.substr(0, slash);
    }
    return ".";
}

static void *open_library(const std::string &module) {
    auto it = g_libs.find(module);
    if (it != g_libs.end()) return it->second;
    const char *env = getenv("FASTGGUF_LIB_DIR");
    std::string dir = env && *env ? env : own_folder();
    std::string path = dir + "/libfg_" + module + ".so";
    void *h = dlopen(path.c_str(), RTLD_NOW | RTLD_GLOBAL);
    if (!h) {
        const char *why = dlerror();
        fail(FG_E_DEVICE, "kernel library " + path + " could not be loaded (" + (why ? why : "unknown") +
                              "); build it with `python -m fastgguf_b200.csrc.build` - there is no fallback path");
    }
    g_libs[module] = h;
    return h;
}

void *kernel_symbol(const char *module, const char *name) {
    std::lock_guard<std::mutex> lock(g_lib_mutex);
    static std::map<std::string, void *> cache;
    std::string key = std::string(module) + ":" + name;
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    void *h = open_library(module);
    void *s = dlsym(h, name);
    if (!s) fail(FG_E_DEVICE, format("kernel library libfg_%s.so has no symbol %s (stale build?)", module, name));
    cache[key] = s;
    return s;
}

void raise_on_device_error(const char *where) {
    static const char *flags[][2] = {{"tc", "fg_gemm_tc_error"}, {"attn", "fg_attention_prefill_tc_error"}};
    for (auto &f : flags) {
        void *h = nullptr;
        {
            std::lock_guard<std::mutex> lock(g_lib_mutex);
            auto it = g_libs.find(f[0]);
            if (it == g_libs.end()) continue;      // never loaded: it launched nothing
            h = it->second;
        }
        auto reader = (int (*)(void))dlsym(h, f[1]);
        if (!reader) continue;
        int code = reader();
        if (code != 0)
            fail(FG_E_KERNEL, format("%s: a device-side wait ran out in library '%s' (code %d, role %d); its output is not valid",
                                     where, f[0], code >> 8, code & 255));
    }
}

// ------------------------------------------------------------------------------------ tensors
int elem_size(int dtype) {
    switch (dtype) {
    case FG_F32: return 4;
    case FG_BF16: return 2;
    case FG_F16: return 2;
    case FG_I32: return 4;
    case FG_I64: return 8;
    }
    return 0;
}

Tensor Tensor::row_range(int64_t begin, int64_t end) const {
    Tensor t = *this;
    t.data = (char *)data + begin * ld * elem_size(dtype);
    t.rows = end - begin;
    return t;
}

fg_dev_tensor Tensor::view() const {
    fg_dev_tensor v = {};
    v.data = data;
    v.dtype = dtype;
    v.ndim = 2;
    v.shape[0] = rows;
    v.shape[1] = cols;
    v.ld = ld;
    return v;
}

// ------------------------------------------------------------------------------------ memory
Arena::~Arena() {
    for (auto &l : lanes_)
        for (auto &b : l.blocks) cudaFree(b.p);
}

void Arena::reset() {
    cur_ = 0;
    for (auto &l : lanes_) {
        if (l.used > l.peak) l.peak = l.used;
        l.used = 0;
        l.block = 0;
        l.offset = 0;
        if (frozen_ || l.blocks.size() <= 1) continue;
        // the last step spilled into further blocks: one block for the largest step so far (cudaFree waits for the device)
        for (auto &b : l.blocks) cudaFree(b.p);
        l.blocks.clear();
        size_t size = l.peak + l.peak / 8;
        if (size < block_bytes_) size = block_bytes_;
        void *p = nullptr;
        if (cudaMalloc(&p, size) == cudaSuccess) l.blocks.push_back({p, size});
        else cudaGetLastError();             // alloc() asks again, block by block, and reports what fails
    }
}

void Arena::begin_layer(int i) {
    cur_ = 1 + (i & 1);
    Lane &l = lanes_[cur_];
    if (l.used > l.peak) l.peak = l.used;
    l.used = 0;
    l.block = 0;
    l.offset = 0;
}

void *Arena::alloc(size_t bytes) {
    bytes = (bytes + 255) / 256 * 256;
    if (bytes == 0) bytes = 256;
    Lane &l = lanes_[cur_];
    l.used += bytes;
    while (true) {
        if (l.block < l.blocks.size()) {
            Block &b = l.blocks[l.block];
            if (l.offset + bytes <= b.size) {
                void *p = (char *)b.p + l.offset;
                l.offset += bytes;
                return p;
            }
            l.block++;
            l.offset = 0;
            continue;
        }
        if (frozen_) fail(FG_E_INTERNAL, "a recorded step asked for more activation memory than its warm-up run");
        size_t size = bytes > block_bytes_ ? bytes : block_bytes_;
        void *p = nullptr;
        cudaError_t e = cudaMalloc(&p, size);
        if (e != cudaSuccess) {
            cudaGetLastError();
            fail(FG_E_DEVICE, format("out of device memory: the activations of this step need another %zu MiB (%s)",
                                     size >> 20, cudaGetErrorString(e)));
        }
        l.blocks.push_back({p, size});
    }
}

Tensor Arena::matrix(int64_t rows, int64_t cols, int dtype) {
    Tensor t;
    // rows of 16-bit tensors stay 16-byte aligned for TMA and vector loads
    int64_t ld = cols;
    t.data = alloc((size_t)(rows > 0 ? rows : 1) * (size_t)ld * elem_size(dtype));
    t.dtype = dtype;
    t.rows = rows;
    t.cols = cols;
    t.ld = ld;
    return t;
}

size_t Arena::bytes_reserved() const {
    size_t n = 0;
    for (auto &l : lanes_)
        for (auto &b : l.blocks) n += b.size;
    return n;
}

DeviceBuffer::DeviceBuffer(size_t bytes, const char *what) : bytes_(bytes) {
    if (bytes == 0) return;
    cudaError_t e = cudaMalloc(&p_, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        size_t free_b = 0, total_b = 0;
        cudaMemGetInfo(&free_b, &total_b);
        p_ = nullptr;
        fail(FG_E_DEVICE, format("out of device memory: %s needs %.1f MiB, %.1f MiB are free (%s)", what,
                                 bytes / 1048576.0, free_b / 1048576.0, cudaGetErrorString(e)));
    }
}
DeviceBuffer::~DeviceBuffer() {
    if (p_) cudaFree(p_);
}
DeviceBuffer &DeviceBuffer::operator=(DeviceBuffer &&o) noexcept {
    if (this != &o) {
        if (p_) cudaFree(p_);
        p_ = o.p_;
        bytes_ = o.bytes_;
        o.p_ = nullptr;
        o.bytes_ = 0;
    }
    return *this;
}

}  // namespace fg
