// See safetensors.hpp.
#include "safetensors.hpp"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstring>
#include <fstream>
#include <set>
#include <thread>

#include "config.hpp"
#include "random_values.hpp"

namespace fg {

int dtype_size(int dtype) {
    switch (dtype) {
    case FG_F32: return 4;
    case FG_BF16: return 2;
    case FG_F16: return 2;
    case FG_I32: return 4;
    case FG_I64: return 8;
    }
    return 0;
}
const char *dtype_name(int dtype) {
    switch (dtype) {
    case FG_F32: return "F32";
    case FG_BF16: return "BF16";
    case FG_F16: return "F16";
    case FG_I32: return "I32";
    case FG_I64: return "I64";
    }
    return "?";
}
const char *dtype_long_name(int dtype) {
    switch (dtype) {
    case FG_F32: return "float32";
    case FG_BF16: return "bfloat16";
    case FG_F16: return "float16";
    case FG_I32: return "int32";
    case FG_I64: return "int64";
    }
    return "?";
}
static int dtype_from_name(const std::string &n) {
    if (n == "F32") return FG_F32;
    if (n == "BF16") return FG_BF16;
    if (n == "F16") return FG_F16;
    if (n == "I32") return FG_I32;
    if (n == "I64") return FG_I64;
    return -1;
}

std::string shape_text(const std::vector<int64_t> &shape) {
    std::string s = "[";
    for (size_t i = 0; i < shape.size(); i++) s += (i ? ", " : "") + std::to_string(shape[i]);
    return s + "]";
}

// ------------------------------------------------------------------------------------ reading
SafetensorsFile::SafetensorsFile(const std::string &path) : path_(path) {
    fd_ = open(path.c_str(), O_RDONLY);
    if (fd_ < 0) fail(FG_E_WEIGHTS, path + ": cannot open (" + strerror(errno) + ")");
    struct stat st;
    if (fstat(fd_, &st) != 0) {
        close(fd_);
        fail(FG_E_WEIGHTS, path + ": cannot stat (" + strerror(errno) + ")");
    }
    size_ = (size_t)st.st_size;
    auto bad = [&](const std::string &msg) {
        if (map_) munmap(map_, size_);
        close(fd_);
        map_ = nullptr;
        fd_ = -1;
        fail(FG_E_WEIGHTS, path + ": " + msg);
    };
    if (size_ < 8) bad(format("too short to be a safetensors file (%zu bytes)", size_));
    map_ = mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
    if (map_ == MAP_FAILED) {
        map_ = nullptr;
        bad(std::string("cannot map (") + strerror(errno) + ")");
    }
    const uint8_t *p = (const uint8_t *)map_;
    uint64_t hlen = 0;
    for (int i = 7; i >= 0; i--) hlen = (hlen << 8) | p[i];
    if (hlen > size_ - 8) bad(format("header length %llu exceeds the file (%zu bytes)", (unsigned long long)hlen, size_));
    Json header;
    try {
        header = Json::parse(std::string((const char *)p + 8, (size_t)hlen));
    } catch (const JsonError &e) {
        bad(std::string("header is not valid JSON (") + e.what() + ")");
    }
    if (!header.is_object()) bad("header must be a JSON object");
    const size_t data0 = 8 + (size_t)hlen;
    const uint64_t data_size = size_ - data0;
    for (auto &m : header.members()) {
        const std::string &name = m.first;
        const Json &info = m.second;
        if (name == "__metadata__") { metadata_ = info; continue; }
        const Json &dt = info.get("dtype"), &shape = info.get("shape"), &offs = info.get("data_offsets");
        bool ok = info.is_object() && dt.is_string() && shape.is_array() && offs.is_array() && offs.size() == 2 &&
                  offs[0].is_int() && offs[1].is_int();
        if (ok)
            for (auto &s : shape.items()) ok = ok && s.is_int() && s.as_int() >= 0;
        if (!ok) bad("tensor '" + name + "' has a malformed directory entry");
        TensorInfo t;
        t.name = name;
        t.dtype = dtype_from_name(dt.as_string());
        if (t.dtype < 0) bad("tensor '" + name + "': unsupported type " + dt.as_string());
        if (shape.size() > 4) bad("tensor '" + name + "' has more than 4 dimensions");
        for (auto &s : shape.items()) t.shape.push_back(s.as_int());
        long long b = offs[0].as_int(), e = offs[1].as_int();
        if (b < 0 || e < b || (uint64_t)e > data_size) bad("tensor '" + name + "' extends past the end of the file");
        if (e - b != t.nbytes())
            bad(format("tensor '%s' of shape %s %s needs %lld bytes, its directory entry gives %lld", name.c_str(),
                       shape_text(t.shape).c_str(), dt.as_string().c_str(), (long long)t.nbytes(), e - b));
        t.data = p + data0 + b;
        entries_[name] = std::move(t);
    }
}

SafetensorsFile::~SafetensorsFile() {
    if (map_) munmap(map_, size_);
    if (fd_ >= 0) close(fd_);
}

static bool file_exists(const std::string &p) {
    struct stat st;
    return stat(p.c_str(), &st) == 0;
}

FolderSource::FolderSource(const std::string &model_dir) : dir_(model_dir) {
    std::string single = model_dir + "/model.safetensors", index = model_dir + "/model.safetensors.index.json";
    std::vector<std::string> paths;
    if (file_exists(single)) paths.push_back(single);
    else if (file_exists(index)) {
        Json j;
        bool ok = true;
        try {
            j = Json::parse(read_text_file(index));
        } catch (const JsonError &) {
            ok = false;
        }
        const Json &wm = j.get("weight_map");
        if (!ok || !wm.is_object()) fail(FG_E_WEIGHTS, index + ": not a shard index (no 'weight_map')");
        std::set<std::string> shards;
        for (auto &m : wm.members())
            if (m.second.is_string()) shards.insert(m.second.as_string());
        for (auto &s : shards) paths.push_back(model_dir + "/" + s);
    } else {
        fail(FG_E_WEIGHTS, model_dir + ": neither model.safetensors nor model.safetensors.index.json found");
    }
    for (auto &p : paths) {
        files_.push_back(std::make_unique<SafetensorsFile>(p));
        SafetensorsFile *sf = files_.back().get();
        for (auto &kv : sf->entries()) {
            if (where_is_.count(kv.first)) {
                std::string other;
                for (auto &f : files_)
                    if (f.get() != sf && f->entries().count(kv.first)) other = f->path();
                fail(FG_E_WEIGHTS, p + ": tensor '" + kv.first + "' is also in " + other);
            }
            where_is_[kv.first] = &kv.second;
        }
    }
}
std::vector<std::string> FolderSource::names() const {
    std::vector<std::string> n;
    for (auto &kv : where_is_) n.push_back(kv.first);
    return n;
}
const TensorInfo *FolderSource::find(const std::string &name) const {
    auto it = where_is_.find(name);
    return it == where_is_.end() ? nullptr : it->second;
}

MemorySource::MemorySource(std::vector<TensorInfo> tensors) {
    for (auto &t : tensors) t_[t.name] = t;
}
std::vector<std::string> MemorySource::names() const {
    std::vector<std::string> n;
    for (auto &kv : t_) n.push_back(kv.first);
    return n;
}
const TensorInfo *MemorySource::find(const std::string &name) const {
    auto it = t_.find(name);
    return it == t_.end() ? nullptr : &it->second;
}

// ------------------------------------------------------------------------------------ writing
void write_safetensors(const std::string &path, const std::vector<TensorInfo> &tensors, const Json &metadata,
                       void (*fill)(const TensorInfo &, void *, void *), void *ctx) {
    std::vector<const TensorInfo *> order;
    for (auto &t : tensors) order.push_back(&t);
    std::sort(order.begin(), order.end(), [](const TensorInfo *a, const TensorInfo *b) { return a->name < b->name; });
    Json header = Json::object();
    if (metadata.is_object() && metadata.size()) header.set("__metadata__", metadata);
    int64_t off = 0;
    for (auto *t : order) {
        Json e = Json::object();
        e.set("dtype", dtype_name(t->dtype));
        Json shape = Json::array();
        for (auto s : t->shape) shape.push(Json((long long)s));
        e.set("shape", shape);
        Json offs = Json::array();
        offs.push(Json((long long)off));
        offs.push(Json((long long)(off + t->nbytes())));
        e.set("data_offsets", offs);
        header.set(t->name, e);
        off += t->nbytes();
    }
    std::string blob = header.dump();
    blob.append((8 - blob.size() % 8) % 8, ' ');
    std::string tmp = path + ".tmp";
    std::ofstream f(tmp, std::ios::binary | std::ios::trunc);
    if (!f) fail(FG_E_WEIGHTS, tmp + ": cannot write (" + strerror(errno) + ")");
    uint64_t hlen = blob.size();
    char lenb[8];
    for (int i = 0; i < 8; i++) lenb[i] = (char)((hlen >> (8 * i)) & 0xFF);
    f.write(lenb, 8);
    f.write(blob.data(), (std::streamsize)blob.size());
    std::vector<char> buf;
    for (auto *t : order) {
        if (t->nbytes() == 0) continue;
        if (t->data) f.write((const char *)t->data, (std::streamsize)t->nbytes());
        else {
            if (!fill) fail(FG_E_INTERNAL, "write_safetensors: tensor '" + t->name + "' has no data");
            buf.resize((size_t)t->nbytes());
            fill(*t, buf.data(), ctx);
            f.write(buf.data(), (std::streamsize)buf.size());
        }
    }
    f.close();
    if (!f) fail(FG_E_WEIGHTS, tmp + ": write failed");
    if (rename(tmp.c_str(), path.c_str()) != 0) fail(FG_E_WEIGHTS, path + ": cannot replace (" + strerror(errno) + ")");
}

// ------------------------------------------------------------------------------------ random weights
uint64_t name_hash64(const std::string &name) {     // FNV-1a, then mixed
    uint64_t h = 0xcbf29ce484222325ull;
    for (unsigned char c : name) { h ^= c; h *= 0x100000001b3ull; }
    return mix64(h);
}
float random_normal(uint64_t seed, uint64_t name_hash, uint64_t index) { return random_unit_normal(seed, name_hash, index); }
uint16_t float_to_bf16(float f) { return bf16_bits_rne(f); }
float bf16_to_float(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
float f16_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000) << 16, exp = (h >> 10) & 0x1F, man = h & 0x3FF, u;
    if (exp == 0) {
        if (man == 0) u = sign;
        else {
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400));
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FF) << 13);
        }
    } else if (exp == 31) u = sign | 0x7F800000u | (man << 13);
    else u = sign | ((exp + 127 - 15) << 23) | (man << 13);
    float f;
    memcpy(&f, &u, 4);
    return f;
}

void fill_random_host(void *dst, int dtype, int64_t n, uint64_t seed, uint64_t nh, int init, float std) {
    if (dtype == FG_I32) { memset(dst, 0, (size_t)n * 4); return; }
    unsigned hw = std::thread::hardware_concurrency();
    int n_threads = (int)std::min<int64_t>(hw ? hw : 4, std::max<int64_t>(1, n / (1 << 16)));
    auto work = [&](int64_t lo, int64_t hi) {
        if (dtype == FG_F32) {
            float *p = (float *)dst;
            for (int64_t i = lo; i < hi; i++) p[i] = random_weight(seed, nh, (uint64_t)i, init, std);
        } else {
            uint16_t *p = (uint16_t *)dst;
            for (int64_t i = lo; i < hi; i++) p[i] = bf16_bits_rne(random_weight(seed, nh, (uint64_t)i, init, std));
        }
    };
    if (dtype != FG_F32 && dtype != FG_BF16) fail(FG_E_USAGE, "random weights are written as float32 or bfloat16");
    if (n_threads <= 1) { work(0, n); return; }
    std::vector<std::thread> th;
    int64_t per = (n + n_threads - 1) / n_threads;
    for (int t = 0; t < n_threads; t++) {
        int64_t lo = t * per, hi = std::min(n, lo + per);
        if (lo < hi) th.emplace_back(work, lo, hi);
    }
    for (auto &t : th) t.join();
}

}  // namespace fg
