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

// Limits of the reference's parser (src/gguf.rs:35-46): below the format's theoretical range so that a valid-looking
// sparse file cannot ask for gigabytes of index memory, far above any real vocabulary or tensor count.
constexpr uint64_t kMaxStringLength = 16ull << 20;
constexpr uint64_t kMaxCollectionEntries = 1ull << 20;
constexpr uint64_t kMaxDecodedAllocationBytes = 256ull << 20;
constexpr uint64_t kIndexAllocationBytesPerEntry = 256;
constexpr size_t kMaxMetadataKeyLength = 65535;
constexpr size_t kMaxTensorNameLength = 63;
constexpr uint32_t kMaxTensorDims = 4;
constexpr uint64_t kDecodedValueBytes = 32;  // charged per decoded array element

[[noreturn]] void fail(const std::string& what) { throw std::runtime_error(what); }

uint64_t checked_add(uint64_t a, uint64_t b, const char* label) {
    uint64_t r;
    if (__builtin_add_overflow(a, b, &r)) fail(std::string(label) + " overflow: " + std::to_string(a) + " + " + std::to_string(b));
    return r;
}

uint64_t checked_mul(uint64_t a, uint64_t b, const char* label) {
    uint64_t r;
    if (__builtin_mul_overflow(a, b, &r)) fail(std::string(label) + " overflow: " + std::to_string(a) + " * " + std::to_string(b));
    return r;
}

uint64_t align_up(uint64_t v, uint64_t a, const char* label) { return checked_add(v, a - 1, label) / a * a; }

// A bounds-checked cursor over the mapped file that also keeps the decoded-allocation budget (BoundedReader,
// src/gguf.rs:1940-2065): every read names the byte it failed at, every string and array is charged before it is built.
struct Cursor {
    const uint8_t* base;
    const uint8_t* p;
    const uint8_t* end;
    uint64_t charged = 0;
    uint64_t position() const { return (uint64_t)(p - base); }
    uint64_t remaining() const { return (uint64_t)(end - p); }
    void charge(uint64_t bytes, const char* label) {
        const uint64_t next = checked_add(charged, bytes, "decoded allocation accounting");
        if (next > kMaxDecodedAllocationBytes)
            fail(std::string("GGUF decoded allocation budget exceeded while reserving ") + label + ": requested " + std::to_string(bytes) +
                 " bytes with " + std::to_string(charged) + " of " + std::to_string(kMaxDecodedAllocationBytes) + " bytes already charged");
        charged = next;
    }
    template <typename T> T read() {
        if (remaining() < sizeof(T))
            fail("unexpected end of GGUF file at byte " + std::to_string(position()) + " while reading " + std::to_string(sizeof(T)) + " bytes");
        T v;
        memcpy(&v, p, sizeof(T));
        p += sizeof(T);
        return v;
    }
    std::string read_string() {
        const uint64_t n = read<uint64_t>();
        if (n > kMaxStringLength) fail("GGUF string length " + std::to_string(n) + " exceeds limit " + std::to_string(kMaxStringLength));
        if (n > remaining()) fail("GGUF string length " + std::to_string(n) + " exceeds " + std::to_string(remaining()) + " remaining bytes");
        charge(n, "string storage");
        std::string s(reinterpret_cast<const char*>(p), (size_t)n);
        p += n;
        return s;
    }
};

enum { T_U8 = 0, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STRING, T_ARRAY, T_U64, T_I64, T_F64 };

bool is_int_type(uint32_t t) { return t == T_U8 || t == T_I8 || t == T_U16 || t == T_I16 || t == T_U32 || t == T_I32 || t == T_U64 || t == T_I64; }

uint64_t minimum_disk_size(uint32_t t) {
    switch (t) {
        case T_U8: case T_I8: case T_BOOL: return 1;
        case T_U16: case T_I16: return 2;
        case T_U32: case T_I32: case T_F32: return 4;
        default: return 8;  // 64-bit scalars; a string is at least its length word
    }
}

void check_value_type(uint32_t t) {
    if (t > T_F64) fail("unknown GGUF metadata value type " + std::to_string(t));
}

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
    fail("not an integer GGUF type");
}

bool read_bool(Cursor& c) {
    const uint8_t b = c.read<uint8_t>();
    if (b > 1) fail("invalid GGUF boolean byte " + std::to_string(b) + "; expected 0 or 1");
    return b == 1;
}

void validate_count(uint64_t count, const char* label) {
    if (count > kMaxCollectionEntries)
        fail(std::string("GGUF ") + label + " count " + std::to_string(count) + " exceeds limit " + std::to_string(kMaxCollectionEntries));
}

// validate_metadata_key (src/gguf.rs:2326-2345)
void validate_metadata_key(const std::string& key) {
    if (key.empty()) fail("GGUF metadata key cannot be empty");
    if (key.size() > kMaxMetadataKeyLength)
        fail("GGUF metadata key is " + std::to_string(key.size()) + " bytes; maximum is " + std::to_string(kMaxMetadataKeyLength));
    for (unsigned char ch : key)
        if (ch >= 0x80) fail("GGUF metadata key '" + key + "' is not ASCII");
    bool segment_empty = true, ok = true;
    for (char ch : key) {
        if (ch == '.') { ok = ok && !segment_empty; segment_empty = true; continue; }
        ok = ok && ((ch >= 'a' && ch <= 'z') || (ch >= '0' && ch <= '9') || ch == '_' || ch == '-');
        segment_empty = false;
    }
    if (!ok || segment_empty) fail("GGUF metadata key '" + key + "' is not a dot-separated lowercase identifier");
}

struct BlockFormat { int weights, bytes; };

// GgufTensorType::from_tag with the block geometry (src/gguf.rs:283-349,351-423)
BlockFormat block_format_of(uint32_t tag) {
    switch (tag) {
        case 0: return {1, 4};
        case 1: return {1, 2};
        case 2: return {32, 18};     // Q4_0
        case 6: return {32, 22};     // Q5_0
        case 7: return {32, 24};     // Q5_1
        case 8: return {32, 34};     // Q8_0
        case 10: return {256, 84};   // Q2_K
        case 11: return {256, 110};  // Q3_K
        case 12: return {256, 144};  // Q4_K
        case 13: return {256, 176};  // Q5_K
        case 14: return {256, 210};  // Q6_K
        case 30: return {1, 2};      // BF16
    }
    fail("unsupported GGML tensor type " + std::to_string(tag) +
         "; this runtime currently supports F32 (0), F16 (1), Q4_0 (2), Q5_0 (6), Q5_1 (7), Q8_0 (8), Q2_K (10), Q3_K (11), Q4_K (12), "
         "Q5_K (13), Q6_K (14), and BF16 (30)");
}

const char* type_label(uint32_t tag) {
    switch (tag) {
        case 0: return "F32"; case 1: return "F16"; case 2: return "Q4_0"; case 6: return "Q5_0"; case 7: return "Q5_1"; case 8: return "Q8_0";
        case 10: return "Q2K"; case 11: return "Q3K"; case 12: return "Q4K"; case 13: return "Q5K"; case 14: return "Q6K"; case 30: return "BF16";
    }
    return "?";
}

// GgufTensorType::byte_len (src/gguf.rs:427-451): whole blocks per row, no overflow anywhere
uint64_t tensor_byte_len(uint32_t tag, const std::vector<int64_t>& dims, const std::string& name) {
    const BlockFormat f = block_format_of(tag);
    const uint64_t row_width = (uint64_t)dims.back();
    if (row_width % (uint64_t)f.weights != 0)
        fail("tensor '" + name + "' row width " + std::to_string(row_width) + " is not divisible by " + type_label(tag) + " block size " +
             std::to_string(f.weights));
    if ((tag == 6 || tag == 7) && (row_width / (uint64_t)f.weights) % 2 != 0)
        fail("tensor '" + name + "' row width " + std::to_string(row_width) + " is unsupported for " + type_label(tag) +
             "; Candle CPU kernels require paired 32-element blocks (a multiple of 64)");
    uint64_t elements = 1;
    for (int64_t d : dims)
        if (__builtin_mul_overflow(elements, (uint64_t)d, &elements)) fail("tensor '" + name + "' element count overflow");
    uint64_t bytes;
    if (__builtin_mul_overflow(elements / (uint64_t)f.weights, (uint64_t)f.bytes, &bytes)) fail("tensor '" + name + "' byte length overflow");
    return bytes;
}

}  // namespace

// One file of a checkpoint: mapped, header parsed with the reference's rules (parse_gguf, src/gguf.rs:2069-2240), tensor
// payloads bounds-checked.
GgufFile::Shard GgufFile::open_shard(const std::string& path, std::map<std::string, GgufValue>& meta_, std::vector<GgufTensor>& tensors_) {
    Shard sh;
    void*& map_ = sh.map;
    size_t& map_len_ = sh.len;
    int fd = open(path.c_str(), O_RDONLY | O_NONBLOCK);  // a FIFO with no writer must not block the loader (src/gguf.rs:3073-3098)
    if (fd < 0) throw std::runtime_error("cannot open GGUF file " + path);
    struct stat st;
    if (fstat(fd, &st) != 0) { close(fd); throw std::runtime_error("cannot stat GGUF file " + path); }
    if (!S_ISREG(st.st_mode)) { close(fd); throw std::runtime_error("GGUF path " + path + " is not a regular file"); }
    map_len_ = (size_t)st.st_size;
    if (map_len_ == 0) { close(fd); throw std::runtime_error(path + " is not a GGUF file: unexpected end of GGUF file at byte 0 while reading 4 bytes"); }
    map_ = mmap(nullptr, map_len_, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (map_ == MAP_FAILED) { map_ = nullptr; throw std::runtime_error("cannot map GGUF file " + path); }
    const uint8_t* base = static_cast<const uint8_t*>(map_);
    const uint64_t file_len = map_len_;
    Cursor c{base, base, base + map_len_};
    if (c.read<uint32_t>() != 0x46554747u) fail(path + " is not a GGUF file: bad GGUF magic");
    const uint32_t version = c.read<uint32_t>();
    if (__builtin_bswap32(version) == 3 && version != 3) fail("big-endian GGUF v3 is not supported");
    if (version != 3) fail("unsupported GGUF version " + std::to_string(version) + "; expected version 3");
    const uint64_t n_tensors = c.read<uint64_t>();
    const uint64_t n_kv = c.read<uint64_t>();
    validate_count(n_tensors, "tensor");
    validate_count(n_kv, "metadata");
    const uint64_t minimum_header = checked_add(checked_mul(n_kv, 13, "metadata header minimum"), checked_mul(n_tensors, 24, "tensor header minimum"),
                                                "combined header minimum");
    if (minimum_header > c.remaining())
        fail("declared tensor/metadata counts need at least " + std::to_string(minimum_header) + " bytes, but only " + std::to_string(c.remaining()) + " remain");
    c.charge(checked_mul(n_kv, kIndexAllocationBytesPerEntry, "metadata index allocation"), "metadata index entries");
    c.charge(checked_mul(n_tensors, kIndexAllocationBytesPerEntry, "tensor index allocation"), "tensor index entries");

    std::map<std::string, GgufValue> parsed;  // this file's own metadata: a repeated key is an error inside one file only
    for (uint64_t i = 0; i < n_kv; ++i) {
        std::string key = c.read_string();
        validate_metadata_key(key);
        const uint32_t t = c.read<uint32_t>();
        check_value_type(t);
        GgufValue val;
        val.type = t;
        if (is_int_type(t)) val.v = read_int(c, t);
        else if (t == T_F32) val.v = (double)c.read<float>();
        else if (t == T_F64) val.v = c.read<double>();
        else if (t == T_BOOL) val.v = read_bool(c);
        else if (t == T_STRING) val.v = c.read_string();
        else {  // T_ARRAY
            const uint32_t et = c.read<uint32_t>();
            check_value_type(et);
            if (et == T_ARRAY) fail("nested GGUF metadata arrays are not supported");
            const uint64_t n = c.read<uint64_t>();
            validate_count(n, "array element");
            const uint64_t minimum = checked_mul(n, minimum_disk_size(et), "array minimum byte length");
            if (minimum > c.remaining())
                fail("GGUF array of " + std::to_string(n) + " values of type " + std::to_string(et) + " needs at least " + std::to_string(minimum) +
                     " bytes, but only " + std::to_string(c.remaining()) + " remain");
            c.charge(checked_mul(n, kDecodedValueBytes, "decoded array allocation"), "metadata array elements");
            if (is_int_type(et) || et == T_BOOL) {
                std::vector<int64_t> a;
                a.reserve((size_t)n);
                for (uint64_t k = 0; k < n; ++k) a.push_back(et == T_BOOL ? (int64_t)read_bool(c) : read_int(c, et));
                val.v = std::move(a);
            } else if (et == T_F32 || et == T_F64) {
                std::vector<double> a;
                a.reserve((size_t)n);
                for (uint64_t k = 0; k < n; ++k) a.push_back(et == T_F32 ? (double)c.read<float>() : c.read<double>());
                val.v = std::move(a);
            } else {  // T_STRING
                std::vector<std::string> a;
                a.reserve((size_t)n);
                for (uint64_t k = 0; k < n; ++k) a.push_back(c.read_string());
                val.v = std::move(a);
            }
        }
        if (!parsed.emplace(key, std::move(val)).second) fail("duplicate GGUF metadata key '" + key + "'");
    }

    const size_t first_tensor = tensors_.size();  // earlier shards' tensors stay as they are
    tensors_.reserve(first_tensor + (size_t)n_tensors);
    std::vector<uint64_t> byte_lens;
    byte_lens.reserve((size_t)n_tensors);
    std::map<std::string, int> names;
    for (uint64_t i = 0; i < n_tensors; ++i) {
        GgufTensor t;
        t.name = c.read_string();
        c.charge(checked_mul((uint64_t)t.name.size(), 2, "tensor name clone allocation"), "tensor name clones");
        if (t.name.empty()) fail("GGUF tensor name cannot be empty");
        if (t.name.size() > kMaxTensorNameLength)
            fail("GGUF tensor name '" + t.name + "' is " + std::to_string(t.name.size()) + " bytes; maximum is " + std::to_string(kMaxTensorNameLength));
        const uint32_t nd = c.read<uint32_t>();
        if (nd < 1 || nd > kMaxTensorDims)
            fail("tensor '" + t.name + "' has rank " + std::to_string(nd) + "; supported ranks are 1..=" + std::to_string(kMaxTensorDims));
        std::vector<int64_t> file_dims;
        for (uint32_t d = 0; d < nd; ++d) {
            const uint64_t dim = c.read<uint64_t>();
            if (dim == 0) fail("tensor '" + t.name + "' has a zero-sized dimension");
            if (dim > (uint64_t)INT64_MAX) fail("tensor '" + t.name + "' dimension does not fit usize");
            file_dims.push_back((int64_t)dim);
        }
        t.dims.assign(file_dims.rbegin(), file_dims.rend());
        const uint32_t tag = c.read<uint32_t>();
        t.type = (int)tag;
        t.offset = c.read<uint64_t>();
        byte_lens.push_back(tensor_byte_len(tag, t.dims, t.name));
        if (!names.emplace(t.name, 0).second) fail("duplicate GGUF tensor name '" + t.name + "'");
        tensors_.push_back(std::move(t));
    }

    uint64_t alignment = 32;
    if (auto it = parsed.find("general.alignment"); it != parsed.end()) {
        if (it->second.type != T_U32) fail("general.alignment must be U32, found value type " + std::to_string(it->second.type));
        alignment = (uint64_t)std::get<int64_t>(it->second.v);
    }
    if (alignment < 8 || alignment % 8 != 0) fail("GGUF alignment " + std::to_string(alignment) + " must be a multiple of 8 bytes");
    const uint64_t data_start = n_tensors == 0 ? c.position() : align_up(c.position(), alignment, "GGUF data offset");
    if (data_start > file_len)
        fail("aligned GGUF tensor data offset " + std::to_string(data_start) + " exceeds file length " + std::to_string(file_len));
    uint64_t expected_offset = 0;
    for (size_t ti = first_tensor; ti < tensors_.size(); ++ti) {
        GgufTensor& t = tensors_[ti];
        const uint64_t byte_len = byte_lens[ti - first_tensor];
        if (t.offset != expected_offset)
            fail("tensor '" + t.name + "' has non-canonical offset " + std::to_string(t.offset) + ", expected " + std::to_string(expected_offset));
        const uint64_t start = checked_add(data_start, t.offset, "tensor absolute offset");
        const uint64_t stop = checked_add(start, byte_len, "tensor end offset");
        if (stop > file_len)
            fail("tensor '" + t.name + "' ends at byte " + std::to_string(stop) + ", past file length " + std::to_string(file_len) +
                 " (it extends past the end of the file)");
        t.data = base + start;
        expected_offset = checked_add(expected_offset, align_up(byte_len, alignment, "padded byte length"), "packed tensor data length");
    }
    if (checked_add(data_start, expected_offset, "GGUF packed data end") > file_len)
        fail("GGUF packed tensor data ends at byte " + std::to_string(data_start + expected_offset) + ", past file length " + std::to_string(file_len) +
             " (it extends past the end of the file)");
    for (auto& kv : parsed) meta_[kv.first] = std::move(kv.second);
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
    // validate_quantization_metadata (src/gguf.rs:664,1019-1037): block formats are only defined for quantisation version 2
    bool quantised = false;
    for (const GgufTensor& t : tensors_) quantised = quantised || (t.type != 0 && t.type != 1 && t.type != 30);
    if (quantised) {
        auto it = meta_.find("general.quantization_version");
        if (it == meta_.end()) throw std::runtime_error("quantized GGUF tensors require general.quantization_version");
        if (it->second.type != 4 /* U32 */)
            throw std::runtime_error("general.quantization_version must be U32, found value type " + std::to_string(it->second.type));
        const int64_t v = std::get<int64_t>(it->second.v);
        if (v != 2) throw std::runtime_error("unsupported GGUF quantization version " + std::to_string(v) + "; expected version 2");
    }
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
