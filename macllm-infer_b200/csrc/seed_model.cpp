// Seed-model tensor generator: N(0, std) weights from a counter-based generator, quantised to the
// GGML block formats the loader accepts (block sizes: src/gguf.rs:386-408 of the reference).
//
// The quantisers here are simple min/max fits.  They need not equal llama.cpp's, because the B200
// path and the CPU oracle both read the bytes this writes; the block *layouts* are the public GGML
// ones and are checked against the `gguf` Python package's dequantisers in the tests.
#include "seed_model.h"
#include <cmath>
#include <cstring>
#include <algorithm>
#include <thread>
#include <vector>
#include <stdexcept>

namespace mk {

namespace {

inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// Standard normal for element `i` of stream (seed, stream): Box-Muller on two hashed uniforms.
inline float normal_at(uint64_t key, uint64_t i) {
    uint64_t a = splitmix64(key ^ splitmix64(2 * i + 1));
    uint64_t b = splitmix64(key ^ splitmix64(2 * i + 2));
    double u1 = ((double)(a >> 11) + 1.0) * (1.0 / 9007199254740993.0);  // (0, 1)
    double u2 = (double)(b >> 11) * (1.0 / 9007199254740992.0);          // [0, 1)
    return (float)(std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2));
}

inline uint16_t f2h(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    int32_t exp = (int32_t)((x >> 23) & 0xFF) - 127 + 15;
    uint32_t man = x & 0x7FFFFFu;
    if (((x >> 23) & 0xFF) == 0xFF) return (uint16_t)(sign | 0x7C00u | (man ? 0x200u : 0));
    if (exp >= 31) return (uint16_t)(sign | 0x7C00u);
    if (exp <= 0) {
        if (exp < -10) return (uint16_t)sign;
        man |= 0x800000u;
        int shift = 14 - exp;
        uint32_t half = man >> shift, rem = man & ((1u << shift) - 1), mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (half & 1))) ++half;
        return (uint16_t)(sign | half);
    }
    uint32_t half = ((uint32_t)exp << 10) | (man >> 13), rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) ++half;
    return (uint16_t)(sign | half);
}

inline float h2f(uint16_t h) {
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

void quantize_q8_0(const float* x, int64_t n, uint8_t* out) {
    for (int64_t b = 0; b < n / 32; ++b) {
        const float* xb = x + b * 32;
        float amax = 0.f;
        for (int i = 0; i < 32; ++i) amax = std::max(amax, std::fabs(xb[i]));
        float d = amax / 127.f;
        uint16_t dh = f2h(d);
        float id = d != 0.f ? 1.f / d : 0.f;
        uint8_t* o = out + b * 34;
        memcpy(o, &dh, 2);
        for (int i = 0; i < 32; ++i) o[2 + i] = (uint8_t)(int8_t)std::lround(xb[i] * id);
    }
}

void quantize_q4_k(const float* x, int64_t n, uint8_t* out) {
    for (int64_t b = 0; b < n / 256; ++b) {
        const float* xb = x + b * 256;
        float scales[8], mins[8];
        float max_scale = 0.f, max_min = 0.f;
        for (int j = 0; j < 8; ++j) {
            float mn = 0.f, mx = 0.f;
            for (int i = 0; i < 32; ++i) { mn = std::min(mn, xb[32 * j + i]); mx = std::max(mx, xb[32 * j + i]); }
            scales[j] = (mx - mn) / 15.f;
            mins[j] = -mn;
            max_scale = std::max(max_scale, scales[j]);
            max_min = std::max(max_min, mins[j]);
        }
        uint16_t dh = f2h(max_scale / 63.f), dmh = f2h(max_min / 63.f);
        float d = h2f(dh), dmin = h2f(dmh);
        uint8_t sc[8], mn[8];
        for (int j = 0; j < 8; ++j) {
            sc[j] = d > 0.f ? (uint8_t)std::min(63L, std::lround(scales[j] / d)) : 0;
            mn[j] = dmin > 0.f ? (uint8_t)std::min(63L, std::lround(mins[j] / dmin)) : 0;
        }
        uint8_t* o = out + b * 144;
        memcpy(o, &dh, 2);
        memcpy(o + 2, &dmh, 2);
        uint8_t* s = o + 4;
        memset(s, 0, 12);
        for (int j = 0; j < 8; ++j) {
            if (j < 4) { s[j] |= sc[j] & 63; s[j + 4] |= mn[j] & 63; }
            else {
                s[j + 4] = (sc[j] & 0xF) | ((mn[j] & 0xF) << 4);
                s[j - 4] |= (sc[j] >> 4) << 6;
                s[j] |= (mn[j] >> 4) << 6;
            }
        }
        uint8_t* qs = o + 16;
        for (int j = 0; j < 4; ++j) {
            float d0 = d * sc[2 * j], m0 = dmin * mn[2 * j], d1 = d * sc[2 * j + 1], m1 = dmin * mn[2 * j + 1];
            for (int l = 0; l < 32; ++l) {
                long q0 = d0 > 0.f ? std::lround((xb[64 * j + l] + m0) / d0) : 0;
                long q1 = d1 > 0.f ? std::lround((xb[64 * j + 32 + l] + m1) / d1) : 0;
                q0 = std::max(0L, std::min(15L, q0));
                q1 = std::max(0L, std::min(15L, q1));
                qs[32 * j + l] = (uint8_t)(q0 | (q1 << 4));
            }
        }
    }
}

void quantize_q6_k(const float* x, int64_t n, uint8_t* out) {
    for (int64_t b = 0; b < n / 256; ++b) {
        const float* xb = x + b * 256;
        float sub[16], max_sub = 0.f;
        for (int j = 0; j < 16; ++j) {
            float amax = 0.f;
            for (int i = 0; i < 16; ++i) amax = std::max(amax, std::fabs(xb[16 * j + i]));
            sub[j] = amax / 31.f;
            max_sub = std::max(max_sub, sub[j]);
        }
        uint16_t dh = f2h(max_sub / 127.f);
        float d = h2f(dh);
        int8_t sc[16];
        for (int j = 0; j < 16; ++j) sc[j] = d > 0.f ? (int8_t)std::min(127L, std::lround(sub[j] / d)) : 0;
        uint8_t q[256];
        for (int j = 0; j < 16; ++j) {
            float ds = d * sc[j];
            for (int i = 0; i < 16; ++i) {
                long v = ds > 0.f ? std::lround(xb[16 * j + i] / ds) : 0;
                v = std::max(-32L, std::min(31L, v));
                q[16 * j + i] = (uint8_t)(v + 32);
            }
        }
        uint8_t* o = out + b * 210;
        uint8_t* ql = o;
        uint8_t* qh = o + 128;
        memset(o, 0, 192);
        for (int h = 0; h < 2; ++h) {
            for (int l = 0; l < 32; ++l) {
                uint8_t q1 = q[128 * h + l], q2 = q[128 * h + l + 32], q3 = q[128 * h + l + 64], q4 = q[128 * h + l + 96];
                ql[64 * h + l] = (q1 & 0xF) | ((q3 & 0xF) << 4);
                ql[64 * h + l + 32] = (q2 & 0xF) | ((q4 & 0xF) << 4);
                qh[32 * h + l] = (q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6);
            }
        }
        memcpy(o + 192, sc, 16);
        memcpy(o + 208, &dh, 2);
    }
}

}  // namespace

int64_t seed_row_bytes(int type, int64_t cols) {
    switch (type) {
        case 0: return cols * 4;
        case 1: return cols * 2;
        case 8: return cols % 32 ? -1 : cols / 32 * 34;
        case 12: return cols % 256 ? -1 : cols / 256 * 144;
        case 14: return cols % 256 ? -1 : cols / 256 * 210;
        // formats written as random block bytes (see random_blocks below)
        case 2: return cols % 32 ? -1 : cols / 32 * 18;
        case 6: return cols % 32 ? -1 : cols / 32 * 22;
        case 7: return cols % 32 ? -1 : cols / 32 * 24;
        case 10: return cols % 256 ? -1 : cols / 256 * 84;
        case 11: return cols % 256 ? -1 : cols / 256 * 110;
        case 13: return cols % 256 ? -1 : cols / 256 * 176;
        case 30: return cols * 2;
        default: return -1;
    }
}

// The formats without a quantiser here (Q4_0, Q5_0, Q5_1, Q2_K, Q3_K, Q5_K) are written as seeded random block bytes: any
// bit pattern is a valid block once its f16 scale fields are finite, and the product and the oracle both read the bytes.
// The scale fields are set so that the decoded weights have about the asked standard deviation and zero mean (the
// divisors are the standard deviations of the decoded values of uniformly random bytes with unit scales).
struct RandomBlock { int type, bytes, d_at, m_at; float d_div, m_per_d; };
constexpr RandomBlock kRandomBlocks[] = {
    {2, 18, 0, -1, 4.612f, 0.f},  {6, 22, 0, -1, 9.227f, 0.f},   {7, 24, 0, 2, 9.231f, -15.5f},
    {10, 84, 80, 82, 13.873f, 1.5f}, {11, 110, 108, -1, 43.331f, 0.f}, {13, 176, 0, 2, 526.319f, 15.5f},
};

static bool random_blocks(int type, uint64_t key, float std_dev, int64_t n_bytes, uint8_t* o, int threads) {
    const RandomBlock* rb = nullptr;
    for (const RandomBlock& b : kRandomBlocks)
        if (b.type == type) rb = &b;
    if (rb == nullptr) return false;
    const int64_t blocks = n_bytes / rb->bytes;
    const uint16_t dh = f2h(std_dev / rb->d_div), mh = f2h(std_dev / rb->d_div * rb->m_per_d);
#pragma omp parallel for schedule(static) num_threads(threads)
    for (int64_t b = 0; b < blocks; ++b) {
        uint8_t* dst = o + b * rb->bytes;
        for (int i = 0; i < rb->bytes; i += 8) {
            const uint64_t w = splitmix64(key ^ splitmix64((uint64_t)(b * 32 + i / 8 + 1)));
            memcpy(dst + i, &w, (size_t)std::min(8, rb->bytes - i));
        }
        memcpy(dst + rb->d_at, &dh, 2);
        if (rb->m_at >= 0) memcpy(dst + rb->m_at, &mh, 2);
    }
    return true;
}

void seed_tensor(uint64_t seed, uint64_t stream, float std_dev, int type, int64_t rows, int64_t cols, void* out) {
    int64_t rb = seed_row_bytes(type, cols);
    if (rb < 0) throw std::runtime_error("seed_tensor: unsupported type or column count");
    uint64_t key = splitmix64(seed * 0x100000001B3ull + splitmix64(stream));
    uint8_t* o = static_cast<uint8_t*>(out);
    if (random_blocks(type, key, std_dev, rows * rb, o, std::max(1, (int)std::thread::hardware_concurrency()))) return;
    // every host core, whatever OMP_NUM_THREADS says: launchers of multi-process jobs export 1, which would turn the
    // seconds a seeded checkpoint takes into many minutes.  Rows are independent, so the bytes do not depend on it.
    const int threads = std::max(1, (int)std::thread::hardware_concurrency());
#pragma omp parallel num_threads(threads)
    {
        std::vector<float> row((size_t)cols);
#pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            for (int64_t c = 0; c < cols; ++c) row[c] = std_dev * normal_at(key, (uint64_t)(r * cols + c));
            uint8_t* dst = o + r * rb;
            switch (type) {
                case 0: memcpy(dst, row.data(), (size_t)cols * 4); break;
                case 1: for (int64_t c = 0; c < cols; ++c) { uint16_t h = f2h(row[c]); memcpy(dst + 2 * c, &h, 2); } break;
                case 30: for (int64_t c = 0; c < cols; ++c) { uint32_t u; memcpy(&u, &row[c], 4); uint16_t h = (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16); memcpy(dst + 2 * c, &h, 2); } break;
                case 8: quantize_q8_0(row.data(), cols, dst); break;
                case 12: quantize_q4_k(row.data(), cols, dst); break;
                case 14: quantize_q6_k(row.data(), cols, dst); break;
            }
        }
    }
}

}  // namespace mk
