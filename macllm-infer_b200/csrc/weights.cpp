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

int64_t gguf_row_bytes(int type, int64_t cols) {
    switch (type) {
        case QT_F32: return cols * 4;
        case QT_F16: return cols * 2;
        case QT_Q8_0: return cols / 32 * 34;
        case QT_Q4_K: return cols / 256 * 144;
        case QT_Q6_K: return cols / 256 * 210;
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

void upload_weight(int type, const void* src, int64_t rows, int64_t cols, DeviceWeight& out, cudaStream_t s) {
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
