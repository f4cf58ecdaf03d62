// Reading and writing the safetensors container, and the sources named tensors come from.
//
// A safetensors file is an 8-byte little-endian header length, a JSON directory
// name -> {dtype, shape, data_offsets}, then the raw tensor bytes.  Role of the reference's GGUF reader
// (gguf_open, fastgguf.c:342-440): parse the directory with bounds checks, reject unsupported types by
// name (:421-425), reject tensors that reach past the end of the file (:432-435), and find tensors by
// exact name (tensor_find, :456-460).
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "errors.hpp"
#include "json.hpp"

namespace fg {

int dtype_size(int dtype);                 // bytes per element of FG_F32 / FG_BF16 / FG_F16 / FG_I32 / FG_I64
const char *dtype_name(int dtype);         // "F32", "BF16", ...
const char *dtype_long_name(int dtype);    // "float32", "bfloat16", ...
inline bool dtype_is_float(int dtype) { return dtype == FG_F32 || dtype == FG_BF16 || dtype == FG_F16; }

struct TensorInfo {
    std::string name;
    int dtype = FG_F32;
    std::vector<int64_t> shape;
    const void *data = nullptr;            // host memory (a view into a map, or the caller's)
    int64_t numel() const {
        int64_t n = 1;
        for (auto s : shape) n *= s;
        return n;
    }
    int64_t nbytes() const { return numel() * dtype_size(dtype); }
};

std::string shape_text(const std::vector<int64_t> &shape);   // "[3, 4]"

class SafetensorsFile {
public:
    explicit SafetensorsFile(const std::string &path);        // throws Error(FG_E_WEIGHTS)
    ~SafetensorsFile();
    SafetensorsFile(const SafetensorsFile &) = delete;
    const std::string &path() const { return path_; }
    const std::map<std::string, TensorInfo> &entries() const { return entries_; }
    const Json &metadata() const { return metadata_; }

private:
    std::string path_;
    int fd_ = -1;
    void *map_ = nullptr;
    size_t size_ = 0;
    std::map<std::string, TensorInfo> entries_;
    Json metadata_;
};

// Where named tensors come from: a model folder, or tensors already in host memory.
class TensorSource {
public:
    virtual ~TensorSource() = default;
    virtual const std::string &where() const = 0;
    virtual std::vector<std::string> names() const = 0;
    virtual const TensorInfo *find(const std::string &name) const = 0;
};

// model.safetensors, or the shards named by model.safetensors.index.json
class FolderSource : public TensorSource {
public:
    explicit FolderSource(const std::string &model_dir);
    const std::string &where() const override { return dir_; }
    std::vector<std::string> names() const override;
    const TensorInfo *find(const std::string &name) const override;

private:
    std::string dir_;
    std::vector<std::unique_ptr<SafetensorsFile>> files_;
    std::map<std::string, const TensorInfo *> where_is_;
};

class MemorySource : public TensorSource {
public:
    explicit MemorySource(std::vector<TensorInfo> tensors);
    const std::string &where() const override { return where_; }
    std::vector<std::string> names() const override;
    const TensorInfo *find(const std::string &name) const override;

private:
    std::string where_ = "tensors in memory";
    std::map<std::string, TensorInfo> t_;
};

// Writes tensors in name order; the header is padded to a multiple of 8 bytes.  `fill(info, dst)` produces
// each tensor's bytes when its `data` is null (random weights are generated tensor by tensor).
void write_safetensors(const std::string &path, const std::vector<TensorInfo> &tensors, const Json &metadata,
                       void (*fill)(const TensorInfo &, void *dst, void *ctx) = nullptr, void *ctx = nullptr);

// ---- seeded random weights (the same values on the host and on the device)
// Element `index` of the tensor `name_hash` of seed `seed`: a sum of eight 24-bit integers (Irwin-Hall,
// close to normal, |z| <= 4.9), centred and scaled by ONE float multiplication - integer arithmetic and one
// rounding, so a CPU and a GPU compute the same bits.  Role: the fixture generator tools/synth_gguf.py
// (seeded N(0, 0.02), :50, :83-86).
uint64_t name_hash64(const std::string &name);
float random_normal(uint64_t seed, uint64_t name_hash, uint64_t index);     // ~ N(0, 1)
uint16_t float_to_bf16(float f);                                            // round to nearest even
float bf16_to_float(uint16_t h);
float f16_to_float(uint16_t h);
// init 0: std * z; init 1: 1 + std * z
void fill_random_host(void *dst, int dtype, int64_t n, uint64_t seed, uint64_t name_hash, int init, float std);

}  // namespace fg
