// GGUF v3 reader (memory-mapped): metadata key/values and tensor descriptors of one file or of a shard family
// `<prefix>-00001-of-000NN.gguf` opened through its first member (src/gguf.rs:576-660).  The header is parsed with the
// reference's rules and limits (parse_gguf, src/gguf.rs:2069-2240): bounded strings, arrays and index memory, no
// duplicate keys or names, canonical payload offsets, overflow-checked sizes.
// Format facts follow the reference's loader (src/gguf.rs:32-46,2155-2220): little-endian, default
// alignment 32, dims stored innermost-first, tensor data contiguous after the aligned header.
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <variant>
#include <vector>

namespace mk {

struct GgufTensor {
    std::string name;
    std::vector<int64_t> dims;  // logical order: outermost first (reversed from the file)
    int type = 0;
    uint64_t offset = 0;        // from the start of the data section
    const uint8_t* data = nullptr;
    int64_t elements() const { int64_t n = 1; for (int64_t d : dims) n *= d; return n; }
};

struct GgufValue {
    uint32_t type = 0;  // the GGUF value-type tag the file gave (an array's own tag, not its elements')
    std::variant<std::monostate, int64_t, double, bool, std::string, std::vector<int64_t>, std::vector<double>, std::vector<std::string>> v;
};

class GgufFile {
public:
    explicit GgufFile(const std::string& path);
    ~GgufFile();
    GgufFile(const GgufFile&) = delete;
    GgufFile& operator=(const GgufFile&) = delete;

    bool has(const std::string& key) const { return meta_.count(key) != 0; }
    int64_t get_int(const std::string& key) const;
    int64_t get_int_or(const std::string& key, int64_t def) const { return has(key) ? get_int(key) : def; }
    double get_float(const std::string& key) const;
    double get_float_or(const std::string& key, double def) const { return has(key) ? get_float(key) : def; }
    std::string get_string(const std::string& key) const;
    const GgufTensor* tensor(const std::string& name) const;
    const GgufTensor& require(const std::string& name) const;
    const std::vector<GgufTensor>& tensors() const { return tensors_; }
    int64_t array_len(const std::string& key) const;
    int shard_count() const { return (int)shards_.size(); }

private:
    struct Shard {  // one mapped file; tensors point into it
        void* map = nullptr;
        size_t len = 0;
        Shard() = default;
        Shard(Shard&& o) noexcept;
        Shard(const Shard&) = delete;
        Shard& operator=(const Shard&) = delete;
        ~Shard();
    };
    static Shard open_shard(const std::string& path, std::map<std::string, GgufValue>& meta, std::vector<GgufTensor>& tensors);
    std::vector<Shard> shards_;
    std::map<std::string, GgufValue> meta_;
    std::vector<GgufTensor> tensors_;
    std::map<std::string, size_t> by_name_;
};

}  // namespace mk
