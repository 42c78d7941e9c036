// See gguf_file.h.
#include "gguf_file.h"
#include <cstring>
#include <fcntl.h>
#include <stdexcept>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace mk {

namespace {

struct Cursor {
    const uint8_t* p;
    const uint8_t* end;
    template <typename T> T read() {
        if ((size_t)(end - p) < sizeof(T)) throw std::runtime_error("GGUF header is truncated");
        T v;
        memcpy(&v, p, sizeof(T));
        p += sizeof(T);
        return v;
    }
    std::string read_string() {
        uint64_t n = read<uint64_t>();
        if ((uint64_t)(end - p) < n) throw std::runtime_error("GGUF string is truncated");
        std::string s(reinterpret_cast<const char*>(p), (size_t)n);
        p += n;
        return s;
    }
};

enum { T_U8 = 0, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STRING, T_ARRAY, T_U64, T_I64, T_F64 };

bool is_int_type(uint32_t t) { return t == T_U8 || t == T_I8 || t == T_U16 || t == T_I16 || t == T_U32 || t == T_I32 || t == T_U64 || t == T_I64; }

int64_t read_int(Cursor& c, uint32_t t) {
    switch (t) {
        case T_U8: return c.read<uint8_t>();
        case T_I8: return c.read<int8_t>();
        case T_U16: return c.read<uint16_t>();
        case T_I16: return c.read<int16_t>();
        case T_U32: return c.read<uint32_t>();
        case T_I32: return c.read<int32_t>();
        case T_U64: return (int64_t)c.read<uint64_t>();
        case T_I64: return c.read<int64_t>();
    }
    throw std::runtime_error("not an integer GGUF type");
}

int64_t row_bytes_of(int type, int64_t cols) {
    switch (type) {
        case 0: return cols * 4;
        case 1: return cols * 2;
        case 8: return cols / 32 * 34;
        case 12: return cols / 256 * 144;
        case 14: return cols / 256 * 210;
        default: return -1;
    }
}

}  // namespace

GgufFile::GgufFile(const std::string& path) {
    int fd = open(path.c_str(), O_RDONLY);
    if (fd < 0) throw std::runtime_error("cannot open GGUF file " + path);
    struct stat st;
    if (fstat(fd, &st) != 0) { close(fd); throw std::runtime_error("cannot stat GGUF file " + path); }
    map_len_ = (size_t)st.st_size;
    map_ = mmap(nullptr, map_len_, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (map_ == MAP_FAILED) { map_ = nullptr; throw std::runtime_error("cannot map GGUF file " + path); }
    const uint8_t* base = static_cast<const uint8_t*>(map_);
    Cursor c{base, base + map_len_};
    if (c.read<uint32_t>() != 0x46554747u) throw std::runtime_error(path + " is not a GGUF file");
    uint32_t version = c.read<uint32_t>();
    if (version != 3 && version != 2) throw std::runtime_error("unsupported GGUF version " + std::to_string(version));
    uint64_t n_tensors = c.read<uint64_t>();
    uint64_t n_kv = c.read<uint64_t>();
    for (uint64_t i = 0; i < n_kv; ++i) {
        std::string key = c.read_string();
        uint32_t t = c.read<uint32_t>();
        GgufValue val;
        if (is_int_type(t)) val.v = read_int(c, t);
        else if (t == T_F32) val.v = (double)c.read<float>();
        else if (t == T_F64) val.v = c.read<double>();
        else if (t == T_BOOL) val.v = (bool)(c.read<uint8_t>() != 0);
        else if (t == T_STRING) val.v = c.read_string();
        else if (t == T_ARRAY) {
            uint32_t et = c.read<uint32_t>();
            uint64_t n = c.read<uint64_t>();
            if (is_int_type(et) || et == T_BOOL) {
                std::vector<int64_t> a;
                a.reserve((size_t)n);
                for (uint64_t k = 0; k < n; ++k) a.push_back(et == T_BOOL ? (int64_t)c.read<uint8_t>() : read_int(c, et));
                val.v = std::move(a);
            } else if (et == T_F32 || et == T_F64) {
                std::vector<double> a;
                a.reserve((size_t)n);
                for (uint64_t k = 0; k < n; ++k) a.push_back(et == T_F32 ? (double)c.read<float>() : c.read<double>());
                val.v = std::move(a);
            } else if (et == T_STRING) {
                std::vector<std::string> a;
                a.reserve((size_t)n);
                for (uint64_t k = 0; k < n; ++k) a.push_back(c.read_string());
                val.v = std::move(a);
            } else {
                throw std::runtime_error("unsupported GGUF array element type in key " + key);
            }
        } else {
            throw std::runtime_error("unsupported GGUF value type in key " + key);
        }
        meta_[key] = std::move(val);
    }
    tensors_.reserve((size_t)n_tensors);
    for (uint64_t i = 0; i < n_tensors; ++i) {
        GgufTensor t;
        t.name = c.read_string();
        uint32_t nd = c.read<uint32_t>();
        if (nd == 0 || nd > 4) throw std::runtime_error("tensor " + t.name + " has unsupported rank");
        std::vector<int64_t> file_dims;
        for (uint32_t d = 0; d < nd; ++d) file_dims.push_back((int64_t)c.read<uint64_t>());
        t.dims.assign(file_dims.rbegin(), file_dims.rend());
        t.type = (int)c.read<uint32_t>();
        t.offset = c.read<uint64_t>();
        by_name_[t.name] = tensors_.size();
        tensors_.push_back(std::move(t));
    }
    uint64_t alignment = (uint64_t)get_int_or("general.alignment", 32);
    uint64_t header = (uint64_t)(c.p - base);
    uint64_t data_start = (header + alignment - 1) / alignment * alignment;
    for (GgufTensor& t : tensors_) {
        int64_t cols = t.dims.back();
        int64_t rows = t.elements() / cols;
        int64_t rb = row_bytes_of(t.type, cols);
        if (rb < 0) throw std::runtime_error("tensor " + t.name + " uses unsupported GGML type " + std::to_string(t.type));
        if (data_start + t.offset + (uint64_t)(rb * rows) > map_len_)
            throw std::runtime_error("tensor " + t.name + " extends past the end of the file");
        t.data = base + data_start + t.offset;
    }
}

GgufFile::~GgufFile() {
    if (map_) munmap(map_, map_len_);
}

int64_t GgufFile::get_int(const std::string& key) const {
    auto it = meta_.find(key);
    if (it == meta_.end()) throw std::runtime_error("GGUF metadata key `" + key + "` is missing");
    if (auto p = std::get_if<int64_t>(&it->second.v)) return *p;
    if (auto p = std::get_if<bool>(&it->second.v)) return *p ? 1 : 0;
    throw std::runtime_error("GGUF metadata key `" + key + "` is not an integer");
}

double GgufFile::get_float(const std::string& key) const {
    auto it = meta_.find(key);
    if (it == meta_.end()) throw std::runtime_error("GGUF metadata key `" + key + "` is missing");
    if (auto p = std::get_if<double>(&it->second.v)) return *p;
    if (auto p = std::get_if<int64_t>(&it->second.v)) return (double)*p;
    throw std::runtime_error("GGUF metadata key `" + key + "` is not a number");
}

std::string GgufFile::get_string(const std::string& key) const {
    auto it = meta_.find(key);
    if (it == meta_.end()) throw std::runtime_error("GGUF metadata key `" + key + "` is missing");
    if (auto p = std::get_if<std::string>(&it->second.v)) return *p;
    throw std::runtime_error("GGUF metadata key `" + key + "` is not a string");
}

int64_t GgufFile::array_len(const std::string& key) const {
    auto it = meta_.find(key);
    if (it == meta_.end()) return -1;
    if (auto p = std::get_if<std::vector<int64_t>>(&it->second.v)) return (int64_t)p->size();
    if (auto p = std::get_if<std::vector<double>>(&it->second.v)) return (int64_t)p->size();
    if (auto p = std::get_if<std::vector<std::string>>(&it->second.v)) return (int64_t)p->size();
    return -1;
}

const GgufTensor* GgufFile::tensor(const std::string& name) const {
    auto it = by_name_.find(name);
    return it == by_name_.end() ? nullptr : &tensors_[it->second];
}

const GgufTensor& GgufFile::require(const std::string& name) const {
    const GgufTensor* t = tensor(name);
    if (!t) throw std::runtime_error("GGUF tensor `" + name + "` is missing");
    return *t;
}

}  // namespace mk
