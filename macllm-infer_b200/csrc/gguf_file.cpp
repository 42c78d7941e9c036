// See gguf_file.h.
#include "gguf_file.h"
#include <cstdio>
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
        case 2: return cols / 32 * 18;     // Q4_0
        case 6: return cols / 32 * 22;     // Q5_0
        case 7: return cols / 32 * 24;     // Q5_1
        case 10: return cols / 256 * 84;   // Q2_K
        case 11: return cols / 256 * 110;  // Q3_K
        case 13: return cols / 256 * 176;  // Q5_K
        case 30: return cols * 2;          // BF16
        default: return -1;
    }
}

}  // namespace

// One file of a checkpoint: mapped, header parsed, tensor payloads bounds-checked.
GgufFile::Shard GgufFile::open_shard(const std::string& path, std::map<std::string, GgufValue>& meta_, std::vector<GgufTensor>& tensors_) {
    Shard sh;
    void*& map_ = sh.map;
    size_t& map_len_ = sh.len;
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
    const size_t first_tensor = tensors_.size();  // earlier shards' tensors stay as they are
    tensors_.reserve(first_tensor + (size_t)n_tensors);
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
        tensors_.push_back(std::move(t));
    }
    uint64_t alignment = 32;
    if (auto it = meta_.find("general.alignment"); it != meta_.end())
        if (auto pv = std::get_if<int64_t>(&it->second.v)) alignment = (uint64_t)*pv;
    if (alignment == 0 || (alignment & (alignment - 1)) != 0) throw std::runtime_error("GGUF alignment must be a power of two");
    uint64_t header = (uint64_t)(c.p - base);
    uint64_t data_start = (header + alignment - 1) / alignment * alignment;
    for (size_t ti = first_tensor; ti < tensors_.size(); ++ti) {
        GgufTensor& t = tensors_[ti];
        int64_t cols = t.dims.back();
        int64_t rows = t.elements() / cols;
        int64_t rb = row_bytes_of(t.type, cols);
        if (rb < 0) throw std::runtime_error("tensor " + t.name + " uses unsupported GGML type " + std::to_string(t.type));
        if (data_start + t.offset + (uint64_t)(rb * rows) > map_len_)
            throw std::runtime_error("tensor " + t.name + " extends past the end of the file");
        t.data = base + data_start + t.offset;
    }
    return sh;
}

GgufFile::Shard::Shard(Shard&& o) noexcept : map(o.map), len(o.len) { o.map = nullptr; o.len = 0; }
GgufFile::Shard::~Shard() { if (map) munmap(map, len); }

namespace {

// `<prefix>-00001-of-00003.gguf` -> (prefix, 0-based index, count); false when the name is not of that form
// (the reference's parse_gguf_split_filename, src/gguf.rs:492-514).
bool parse_split_name(const std::string& filename, std::string& prefix, int& index, int& count) {
    const std::string suffix = ".gguf";
    if (filename.size() <= suffix.size() || filename.compare(filename.size() - suffix.size(), suffix.size(), suffix) != 0) return false;
    std::string stem = filename.substr(0, filename.size() - suffix.size());
    size_t of = stem.rfind("-of-");
    if (of == std::string::npos) return false;
    std::string count_text = stem.substr(of + 4), indexed = stem.substr(0, of);
    size_t dash = indexed.rfind('-');
    if (dash == std::string::npos || dash == 0) return false;
    std::string index_text = indexed.substr(dash + 1);
    auto digits5 = [](const std::string& t) { return t.size() == 5 && t.find_first_not_of("0123456789") == std::string::npos; };
    if (!digits5(index_text) || !digits5(count_text)) return false;
    int file_index = std::stoi(index_text);
    count = std::stoi(count_text);
    if (file_index == 0 || count == 0 || file_index > count || count > 65535) return false;
    prefix = indexed.substr(0, dash);
    index = file_index - 1;
    return true;
}

struct SplitInfo { bool present = false; int64_t index = 0, count = 0, tensors = 0; };

// split.no / split.count / split.tensors.count (src/gguf.rs:956-993)
SplitInfo split_info(const std::map<std::string, GgufValue>& meta) {
    SplitInfo s;
    for (const auto& kv : meta)
        if (kv.first.compare(0, 6, "split.") == 0) s.present = true;
    if (!s.present) return s;
    auto need = [&](const char* key) {
        auto it = meta.find(key);
        if (it == meta.end()) throw std::runtime_error(std::string("required GGUF metadata `") + key + "` is missing");
        auto p = std::get_if<int64_t>(&it->second.v);
        if (p == nullptr || *p < 0) throw std::runtime_error(std::string("GGUF metadata `") + key + "` must be a non-negative integer");
        return *p;
    };
    s.index = need("split.no");
    s.count = need("split.count");
    s.tensors = need("split.tensors.count");
    if (s.count == 0 ? s.index != 0 : s.index >= s.count)
        throw std::runtime_error("GGUF metadata `split.no`=" + std::to_string(s.index) + " is outside split.count=" + std::to_string(s.count));
    return s;
}

constexpr int kMaxShards = 128;  // the reference's safety limit (src/gguf.rs:50)

}  // namespace

// A checkpoint is one file or a family `<prefix>-00001-of-000NN.gguf` opened through its first member
// (GgufFile::open, src/gguf.rs:576-660): siblings are found by name, must declare their own place in the same family,
// and contribute tensors only - the metadata of the first shard is the checkpoint's.
GgufFile::GgufFile(const std::string& path) {
    shards_.push_back(open_shard(path, meta_, tensors_));
    const SplitInfo first = split_info(meta_);
    const size_t slash = path.find_last_of('/');
    const std::string dir = slash == std::string::npos ? "" : path.substr(0, slash + 1);
    const std::string filename = slash == std::string::npos ? path : path.substr(slash + 1);
    std::string prefix;
    int name_index = 0, name_count = 0;
    const bool named = parse_split_name(filename, prefix, name_index, name_count);
    if ((!first.present || first.count <= 1) && named && name_count > 1)
        throw std::runtime_error("GGUF filename " + path + " declares an active shard family, but its metadata does not");
    if (first.present && first.count > 1) {
        if (first.index != 0) throw std::runtime_error("GGUF split " + path + " has split.no=" + std::to_string(first.index) + "; load the first shard instead");
        if (first.count > kMaxShards)
            throw std::runtime_error("GGUF declares " + std::to_string(first.count) + " shards, exceeding the supported safety limit " + std::to_string(kMaxShards));
        if (!named || name_index != 0 || name_count != first.count)
            throw std::runtime_error("GGUF first shard filename `" + filename + "` does not match split.no=0 and split.count=" + std::to_string(first.count));
        if ((int64_t)tensors_.size() > first.tensors) throw std::runtime_error("GGUF shard holds more tensors than split.tensors.count declares");
        for (int i = 1; i < (int)first.count; ++i) {
            char name[64];
            snprintf(name, sizeof name, "-%05d-of-%05d.gguf", i + 1, (int)first.count);
            const std::string shard_path = dir + prefix + name;
            std::map<std::string, GgufValue> shard_meta;
            try {
                shards_.push_back(open_shard(shard_path, shard_meta, tensors_));
            } catch (const std::exception& e) {
                throw std::runtime_error("failed to load GGUF shard " + std::to_string(i + 1) + " of " + std::to_string(first.count) + ": " + e.what());
            }
            const SplitInfo s = split_info(shard_meta);
            if (!s.present) throw std::runtime_error("GGUF shard " + shard_path + " is missing required split metadata");
            if (s.index != i) throw std::runtime_error("GGUF shard " + shard_path + " declares split.no=" + std::to_string(s.index) + ", expected " + std::to_string(i));
            if (s.count != first.count)
                throw std::runtime_error("GGUF shard " + shard_path + " declares split.count=" + std::to_string(s.count) + ", expected " + std::to_string(first.count));
            if (s.tensors != first.tensors)
                throw std::runtime_error("GGUF shard " + shard_path + " declares split.tensors.count=" + std::to_string(s.tensors) + ", expected " +
                                         std::to_string(first.tensors));
            // a later shard may repeat metadata of the first, never add or change any (src/gguf.rs:995-1017)
            for (const auto& kv : shard_meta) {
                if (kv.first.compare(0, 6, "split.") == 0 || kv.first == "general.alignment") continue;
                auto it = meta_.find(kv.first);
                if (it == meta_.end())
                    throw std::runtime_error("GGUF subsidiary shard " + shard_path + " contains metadata `" + kv.first + "` absent from the first shard");
                if (!(it->second.v == kv.second.v)) throw std::runtime_error("GGUF subsidiary shard " + shard_path + " has conflicting metadata `" + kv.first + "`");
            }
            if ((int64_t)tensors_.size() > first.tensors) throw std::runtime_error("GGUF shards hold more tensors than split.tensors.count declares");
        }
    }
    for (size_t i = 0; i < tensors_.size(); ++i)
        if (!by_name_.emplace(tensors_[i].name, i).second) throw std::runtime_error("GGUF tensor `" + tensors_[i].name + "` appears more than once");
    if (first.present && first.count > 1 && (int64_t)tensors_.size() != first.tensors)
        throw std::runtime_error("GGUF split checkpoint declares " + std::to_string(first.tensors) + " tensors, but " + std::to_string(tensors_.size()) +
                                 " unique tensors were loaded");
}
GgufFile::~GgufFile() = default;

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
