// Weight upload: GGUF block bytes -> HBM layouts read by the kernels.
#include "device_util.h"
#include <cstring>
#include <map>
#include <mutex>
#include <vector>

namespace mk {

void ensure_dynamic_smem(const void* func, size_t bytes) {
    if (bytes <= 48 * 1024) return;
    static std::mutex mu;
    static std::map<std::pair<const void*, int>, size_t> done;
    int dev = 0;
    MK_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    size_t& have = done[{func, dev}];
    if (have >= bytes) return;
    MK_CUDA(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    have = bytes;
}

int device_sm_count() {
    static std::mutex mu;
    static std::map<int, int> cached;
    int dev = 0;
    MK_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    int& n = cached[dev];
    if (n == 0) MK_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    return n;
}

void unpermute_qk_rows_host(const uint8_t* src, int64_t rows, int64_t row_bytes, int heads, uint8_t* dst) {
    if (heads <= 0 || rows <= 0 || rows % heads != 0)
        throw std::runtime_error("cannot inverse-permute compressed Llama Q/K shape [" + std::to_string(rows) + " rows] across " +
                                 std::to_string(heads) + " heads");
    const int64_t d = rows / heads;
    if (d % 2 != 0) throw std::runtime_error("Llama Q/K head dimension " + std::to_string(d) + " must be even");
    for (int64_t h = 0; h < heads; ++h)
        for (int64_t lane = 0; lane < 2; ++lane)
            for (int64_t pair = 0; pair < d / 2; ++pair)
                memcpy(dst + (h * d + lane * (d / 2) + pair) * row_bytes, src + (h * d + 2 * pair + lane) * row_bytes, (size_t)row_bytes);
}

int64_t gguf_row_bytes(int type, int64_t cols) {
    switch (type) {
        case QT_F32: return cols * 4;
        case QT_F16: return cols * 2;
        case QT_Q8_0: return cols / 32 * 34;
        case QT_Q4_K: return cols / 256 * 144;
        case QT_Q6_K: return cols / 256 * 210;
        case QT_Q4_0: return cols / 32 * 18;
        case QT_Q5_0: return cols / 32 * 22;
        case QT_Q5_1: return cols / 32 * 24;
        case QT_Q2_K: return cols / 256 * 84;
        case QT_Q3_K: return cols / 256 * 110;
        case QT_Q5_K: return cols / 256 * 176;
        case QT_BF16: return cols * 2;
        default: return -1;
    }
}

static float half_bits_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            int e = -1;
            do { man <<= 1; ++e; } while ((man & 0x400u) == 0);
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
    else bits = sign | ((exp + 112u) << 23) | (man << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

// ---------------------------------------------------------------------------------------------------------------
// Host decoders of the block formats the kernels do not read in place (Q4_0, Q5_0, Q5_1, Q2_K, Q3_K, Q5_K, BF16; the
// public GGML layouts, type list src/gguf.rs:283-345, sizes :386-408).  A block is described by where its fields sit
// and how a weight's bits are gathered from them; `decode_block` writes the block's weights as f32.
namespace {

inline float f16_at(const uint8_t* p) { return half_bits_to_float((uint16_t)(p[0] | (p[1] << 8))); }

// six-bit (scale, min) pair j of the 12-byte packing shared by Q4_K and Q5_K
inline void k_scale_min(const uint8_t* s, int j, int& sc, int& mn) {
    if (j < 4) { sc = s[j] & 63; mn = s[j + 4] & 63; }
    else { sc = (s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4); mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4); }
}

void decode_block(int type, const uint8_t* b, float* y) {
    switch (type) {
        case QT_Q4_0: {  // d | 16 nibble bytes: weight i < 16 is the low nibble of byte i, weight i + 16 the high one; zero point 8
            const float d = f16_at(b);
            for (int i = 0; i < 32; ++i) y[i] = d * (float)(((b[2 + (i & 15)] >> (4 * (i >> 4))) & 0xF) - 8);
            break;
        }
        case QT_Q5_0:    // d | 32 fifth bits | 16 nibble bytes; zero point 16
        case QT_Q5_1: {  // d | m | 32 fifth bits | 16 nibble bytes; w = d * q + m
            const bool with_min = type == QT_Q5_1;
            const float d = f16_at(b), m = with_min ? f16_at(b + 2) : 0.f;
            const uint8_t* hb = b + (with_min ? 4 : 2);
            const uint8_t* qs = hb + 4;
            const uint32_t fifth = (uint32_t)hb[0] | ((uint32_t)hb[1] << 8) | ((uint32_t)hb[2] << 16) | ((uint32_t)hb[3] << 24);
            for (int i = 0; i < 32; ++i) {
                const int q = ((qs[i & 15] >> (4 * (i >> 4))) & 0xF) | (int)(((fifth >> i) & 1u) << 4);
                y[i] = with_min ? d * (float)q + m : d * (float)(q - 16);
            }
            break;
        }
        case QT_Q2_K: {  // 16 (scale | min << 4) bytes | 64 bytes of 2-bit values | d | dmin
            const float d = f16_at(b + 80), dmin = f16_at(b + 82);
            for (int i = 0; i < 256; ++i) {
                const int g = i >> 4, half = i >> 7, within = i & 127;         // 16-weight group, 128-weight half
                const int byte = 32 * half + (within & 31), shift = 2 * (within >> 5);
                const int q = (b[16 + byte] >> shift) & 3;
                y[i] = d * (float)(b[g] & 0xF) * (float)q - dmin * (float)(b[g] >> 4);
            }
            break;
        }
        case QT_Q3_K: {  // 32 high-bit bytes | 64 bytes of 2-bit values | 12 bytes of sixteen 6-bit scales | d
            const float d = f16_at(b + 108);
            const uint8_t* s = b + 96;
            for (int i = 0; i < 256; ++i) {
                const int g = i >> 4, half = i >> 7, within = i & 127;
                const int col = within & 31, plane = within >> 5;             // plane: which bit pair / high bit of the half
                const int low = (b[32 + 32 * half + col] >> (2 * plane)) & 3;
                const int high = (b[col] >> (4 * half + plane)) & 1;
                const int sl = g < 8 ? (s[g] & 0xF) : (s[g - 8] >> 4), sh = (s[8 + (g & 3)] >> (2 * (g >> 2))) & 3;
                y[i] = d * (float)((sl | (sh << 4)) - 32) * (float)(low - (high ? 0 : 4));
            }
            break;
        }
        case QT_Q5_K: {  // d | dmin | 12 scale bytes | 32 fifth-bit bytes | 128 nibble bytes
            const float d = f16_at(b), dmin = f16_at(b + 2);
            for (int i = 0; i < 256; ++i) {
                const int sub = i >> 5, col = i & 31, pair = sub >> 1;       // 32-weight sub-block; two sub-blocks share 32 bytes
                int sc, mn;
                k_scale_min(b + 4, sub, sc, mn);
                const int nib = (b[48 + 32 * pair + col] >> (4 * (sub & 1))) & 0xF;
                const int q = nib | (((b[16 + col] >> sub) & 1) << 4);
                y[i] = d * (float)sc * (float)q - dmin * (float)mn;
            }
            break;
        }
        default: throw std::runtime_error("decode_block: not a host-decoded block format");
    }
}

}  // namespace

bool decoded_at_load(int type) {
    return type == QT_Q4_0 || type == QT_Q5_0 || type == QT_Q5_1 || type == QT_Q2_K || type == QT_Q3_K || type == QT_Q5_K || type == QT_BF16;
}

void decode_rows_host(int type, const void* src, int64_t rows, int64_t cols, float* out) {
    const int64_t rb = gguf_row_bytes(type, cols);
    if (!decoded_at_load(type) || rb < 0) throw std::runtime_error("decode_rows_host: GGML type " + std::to_string(type) + " is not decoded on the host");
    const uint8_t* p = static_cast<const uint8_t*>(src);
    if (type == QT_BF16) {
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < rows * cols; ++i) {
            const uint32_t u = (uint32_t)(p[2 * i] | (p[2 * i + 1] << 8)) << 16;
            memcpy(out + i, &u, 4);
        }
        return;
    }
    const int per = (type == QT_Q4_0 || type == QT_Q5_0 || type == QT_Q5_1) ? 32 : 256;
    if (cols % per != 0) throw std::runtime_error("decode_rows_host: rows must be whole blocks of " + std::to_string(per) + " weights");
    const int64_t bb = rb / (cols / per), nblk = rows * (cols / per);
#pragma omp parallel for schedule(static)
    for (int64_t k = 0; k < nblk; ++k) decode_block(type, p + k * bb, out + k * per);
}

void upload_weight(int type, const void* src, int64_t rows, int64_t cols, DeviceWeight& out, cudaStream_t s) {
    if (decoded_at_load(type)) {
        // decoded once on the host and kept as a dense f32 matrix; the dense f16 GEMM serves it at every row count
        std::vector<float> dense((size_t)rows * cols);
        decode_rows_host(type, src, rows, cols, dense.data());
        upload_weight(QT_F32, dense.data(), rows, cols, out, s);
        out.file_type = type;
        return;
    }
    out.w = QWeight{};
    out.w.type = type;
    out.w.rows = rows;
    out.w.cols = cols;
    int64_t rb = gguf_row_bytes(type, cols);
    if (rb < 0) throw std::runtime_error("upload_weight: unsupported GGML type " + std::to_string(type));
    out.w.bytes = rb * rows;
    const uint8_t* p = static_cast<const uint8_t*>(src);
    switch (type) {
        case QT_F32:
            out.b0.upload(p, (size_t)rows * cols * 4, s);
            MK_CUDA(cudaStreamSynchronize(s));
            break;
        case QT_F16: {
            std::vector<float> tmp((size_t)rows * cols);
            const uint16_t* h = reinterpret_cast<const uint16_t*>(p);
            for (size_t i = 0; i < tmp.size(); ++i) tmp[i] = half_bits_to_float(h[i]);
            out.b0.upload(tmp.data(), tmp.size() * 4, s);
            MK_CUDA(cudaStreamSynchronize(s));
            out.w.type = QT_F32;
            break;
        }
        case QT_Q4_K:
            if (cols % 256) throw std::runtime_error("upload_weight: Q4_K needs cols % 256 == 0");
            out.b0.upload(p, (size_t)out.w.bytes, s);
            MK_CUDA(cudaStreamSynchronize(s));
            break;
        case QT_Q6_K: {
            if (cols % 256) throw std::runtime_error("upload_weight: Q6_K needs cols % 256 == 0");
            int64_t nblk = rows * (cols / 256);
            std::vector<uint8_t> ql((size_t)nblk * 128), qh((size_t)nblk * 64), sc((size_t)nblk * 16);
            std::vector<uint16_t> d((size_t)nblk);
#pragma omp parallel for schedule(static)
            for (int64_t b = 0; b < nblk; ++b) {
                const uint8_t* blk = p + b * 210;
                memcpy(&ql[b * 128], blk, 128);
                memcpy(&qh[b * 64], blk + 128, 64);
                memcpy(&sc[b * 16], blk + 192, 16);
                memcpy(&d[b], blk + 208, 2);
            }
            out.b0.upload(ql.data(), ql.size(), s);
            out.b1.upload(qh.data(), qh.size(), s);
            out.b2.upload(sc.data(), sc.size(), s);
            out.b3.upload(d.data(), d.size() * 2, s);
            MK_CUDA(cudaStreamSynchronize(s));
            break;
        }
        case QT_Q8_0: {
            if (cols % 32) throw std::runtime_error("upload_weight: Q8_0 needs cols % 32 == 0");
            int64_t nblk = rows * (cols / 32);
            std::vector<int8_t> qs((size_t)nblk * 32);
            std::vector<uint16_t> d((size_t)nblk);
#pragma omp parallel for schedule(static)
            for (int64_t b = 0; b < nblk; ++b) {
                const uint8_t* blk = p + b * 34;
                memcpy(&d[b], blk, 2);
                memcpy(&qs[b * 32], blk + 2, 32);
            }
            out.b0.upload(qs.data(), qs.size(), s);
            out.b1.upload(d.data(), d.size() * 2, s);
            MK_CUDA(cudaStreamSynchronize(s));
            break;
        }
    }
    out.w.p0 = out.b0.ptr();
    out.w.p1 = out.b1.ptr();
    out.w.p2 = out.b2.ptr();
    out.w.p3 = out.b3.ptr();
}

}  // namespace mk
