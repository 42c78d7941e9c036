// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// A plain C++ restatement of the arithmetic on macllm-infer's CPU path for the
// continuous-batching step.  Nothing in the shipped library may link, load or
// call this file; only the parity tests, the smoke check and the CPU-baseline
// leg of the benchmark do, and only as the checker.
//
// Reference sources followed (paths inside the reference project):
//   src/model_weights.rs:346-377    LinearOp::forward (input forced to f32, QMatMul)
//   src/model_weights.rs:489-502    quantised embedding rows
//   src/model_weights.rs:563-565    rms_norm
//   src/decoder.rs:136-257          RoPE inverse frequencies, tables, half-split rotation
//   src/decoder.rs:298-305          dense feed-forward (SiLU / tanh-GELU gate * up, down)
//   src/decoder.rs:448-554          selected-softmax router and its (value desc, index asc) order
//   src/decoder.rs:4499-4541        causal / sliding visibility rule
//   src/decoder.rs:4580-4670        dense grouped-query attention (scale, softcap, mask, f32 softmax)
//   src/decoder.rs:4791-4796        tanh softcap
//   crates/macllm-kernels/src/paged_attention.rs:504-709   CPU paged online-softmax attention
//   src/sampling.rs:392-433         penalties, first-index argmax
//   src/gguf.rs:386-408             block sizes of Q4_K / Q6_K / Q8_0
//
// PARITY UNPINNED for the quantised matmul at bit level: the block dot products
// live in the un-vendored third-party crate candle-core 0.11.0
// (candle_core::quantized::QMatMul).  What is restated here is the published
// GGML block format and the published GGML rule that the CPU path quantises
// each activation row to 8-bit blocks (Q8_K for K-quants, Q8_0 for Q8_0) and
// takes integer block dot products scaled in f32.  Weight decoding is pinned
// against the `gguf` Python package's dequantisers in the tests; the float
// accumulation order across blocks is this file's own choice (sequential over
// blocks), because the third-party code's order depends on the host's SIMD path.

#include <cmath>
#include <cstdint>
#include <cstring>
#include <cstdlib>
#include <vector>
#include <algorithm>

#ifdef _OPENMP
#include <omp.h>
#endif
#if defined(__AVX2__) && !defined(ORC_NO_SIMD)
#include <immintrin.h>
#define ORC_AVX2 1
#endif

extern "C" {

enum { ORC_F32 = 0, ORC_F16 = 1, ORC_Q4_0 = 2, ORC_Q5_0 = 6, ORC_Q5_1 = 7, ORC_Q8_0 = 8, ORC_Q2_K = 10, ORC_Q3_K = 11, ORC_Q4_K = 12,
       ORC_Q5_K = 13, ORC_Q6_K = 14, ORC_BF16 = 30 };

// ---------------------------------------------------------------- f16 helpers
static inline float h2f(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do { man <<= 1; ++e; } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f; memcpy(&f, &bits, 4); return f;
}

static inline uint16_t f2h(float f) {  // round to nearest even
    uint32_t x; memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    int32_t exp = (int32_t)((x >> 23) & 0xFF) - 127 + 15;
    uint32_t man = x & 0x7FFFFFu;
    if (((x >> 23) & 0xFF) == 0xFF) return (uint16_t)(sign | 0x7C00u | (man ? 0x200u : 0));
    if (exp >= 31) return (uint16_t)(sign | 0x7C00u);
    if (exp <= 0) {
        if (exp < -10) return (uint16_t)sign;
        man |= 0x800000u;
        int shift = 14 - exp;
        uint32_t half = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1);
        uint32_t mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (half & 1))) ++half;
        return (uint16_t)(sign | half);
    }
    uint32_t half = ((uint32_t)exp << 10) | (man >> 13);
    uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) ++half;
    return (uint16_t)(sign | half);
}

uint16_t orc_f32_to_f16(float f) { return f2h(f); }
float orc_f16_to_f32(uint16_t h) { return h2f(h); }

// ---------------------------------------------------------------- block formats
// Sizes: src/gguf.rs:386-408.
#pragma pack(push, 1)
struct BlkQ80 { uint16_t d; int8_t qs[32]; };                                   // 34 B / 32 weights
struct BlkQ4K { uint16_t d; uint16_t dmin; uint8_t scales[12]; uint8_t qs[128]; };  // 144 B / 256
struct BlkQ6K { uint8_t ql[128]; uint8_t qh[64]; int8_t scales[16]; uint16_t d; };  // 210 B / 256
#pragma pack(pop)
static_assert(sizeof(BlkQ80) == 34 && sizeof(BlkQ4K) == 144 && sizeof(BlkQ6K) == 210, "block sizes");

static inline void q4k_scale_min(int j, const uint8_t* s, int* sc, int* mn) {
    if (j < 4) { *sc = s[j] & 63; *mn = s[j + 4] & 63; }
    else { *sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4); *mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4); }
}

int64_t orc_row_bytes(int type, int64_t cols) {
    switch (type) {
        case ORC_F32: return cols * 4;
        case ORC_F16: return cols * 2;
        case ORC_Q8_0: return cols / 32 * 34;
        case ORC_Q4_K: return cols / 256 * 144;
        case ORC_Q6_K: return cols / 256 * 210;
        // the other block formats the reference's loader accepts (src/gguf.rs:283-297, sizes :386-408)
        case ORC_Q4_0: return cols / 32 * 18;
        case ORC_Q5_0: return cols / 32 * 22;
        case ORC_Q5_1: return cols / 32 * 24;
        case ORC_Q2_K: return cols / 256 * 84;
        case ORC_Q3_K: return cols / 256 * 110;
        case ORC_Q5_K: return cols / 256 * 176;
        case ORC_BF16: return cols * 2;
    }
    return -1;
}

// The block formats below follow the published GGML layouts; the decoders are pinned against the `gguf` Python package on
// random block bytes (tests/test_oracle_formats.py).
static uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }
static uint32_t rd32(const uint8_t* p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }

// Q4_0: [d f16][16 bytes]; weight j = low nibble of byte j, weight j + 16 = its high nibble, both offset by 8.
static void dq_q4_0(const uint8_t* b, float* y) {
    float d = h2f(rd16(b));
    for (int j = 0; j < 16; ++j) { y[j] = d * ((b[2 + j] & 0xF) - 8); y[j + 16] = d * ((b[2 + j] >> 4) - 8); }
}
// Q5_0 / Q5_1: a fifth bit per weight in a 32-bit word: bit j for weight j, bit j + 16 for weight j + 16.
static void dq_q5_0(const uint8_t* b, float* y) {
    float d = h2f(rd16(b));
    uint32_t hi = rd32(b + 2);
    for (int j = 0; j < 16; ++j) {
        int lo0 = b[6 + j] & 0xF, lo1 = b[6 + j] >> 4;
        y[j] = d * ((lo0 | (int)(((hi >> j) & 1) << 4)) - 16);
        y[j + 16] = d * ((lo1 | (int)(((hi >> (j + 16)) & 1) << 4)) - 16);
    }
}
static void dq_q5_1(const uint8_t* b, float* y) {
    float d = h2f(rd16(b)), m = h2f(rd16(b + 2));
    uint32_t hi = rd32(b + 4);
    for (int j = 0; j < 16; ++j) {
        int lo0 = b[8 + j] & 0xF, lo1 = b[8 + j] >> 4;
        y[j] = d * (float)(lo0 | (int)(((hi >> j) & 1) << 4)) + m;
        y[j + 16] = d * (float)(lo1 | (int)(((hi >> (j + 16)) & 1) << 4)) + m;
    }
}
// Q2_K: [16 scale bytes: low nibble scale, high nibble min][64 bytes of 2-bit values][d f16][dmin f16]; sixteen groups of 16
// weights; group g of half n (128 weights) reads bit pair (g / 2) of bytes [32 n + 16 (g % 2), + 16).
static void dq_q2_k(const uint8_t* b, float* y) {
    const uint8_t* sc = b; const uint8_t* q = b + 16;
    float d = h2f(rd16(b + 80)), dmin = h2f(rd16(b + 82));
    for (int g = 0; g < 16; ++g) {
        int n = g / 8, gi = g % 8, shift = 2 * (gi / 2);
        const uint8_t* src = q + 32 * n + 16 * (gi % 2);
        float dl = d * (sc[g] & 0xF), ml = dmin * (sc[g] >> 4);
        for (int l = 0; l < 16; ++l) y[16 * g + l] = dl * ((src[l] >> shift) & 3) - ml;
    }
}
// Q3_K: [32 bytes: one high bit per weight][64 bytes of 2-bit values][12 bytes: sixteen 6-bit scales][d f16].
static void dq_q3_k(const uint8_t* b, float* y) {
    const uint8_t* hm = b; const uint8_t* q = b + 32; const uint8_t* s = b + 96;
    float d = h2f(rd16(b + 108));
    int scale[16];
    for (int i = 0; i < 16; ++i) {
        // low 4 bits: nibbles of bytes 0..7; high 2 bits: bit pairs of bytes 8..11
        int lo = i < 8 ? (s[i] & 0xF) : (s[i - 8] >> 4);
        int hi2 = (s[8 + (i % 4)] >> (2 * (i / 4))) & 3;
        scale[i] = (lo | (hi2 << 4)) - 32;
    }
    for (int g = 0; g < 16; ++g) {
        int n = g / 8, gi = g % 8, shift = 2 * (gi / 2), bit = 4 * n + gi / 2;
        const uint8_t* src = q + 32 * n + 16 * (gi % 2);
        const uint8_t* hsrc = hm + 16 * (gi % 2);
        float dl = d * scale[g];
        for (int l = 0; l < 16; ++l) {
            int v = (src[l] >> shift) & 3;
            if (!((hsrc[l] >> bit) & 1)) v -= 4;
            y[16 * g + l] = dl * v;
        }
    }
}
// Q5_K: [d f16][dmin f16][12 bytes: eight 6-bit scale / min pairs as in Q4_K][32 bytes: a fifth bit per weight][128 nibble bytes].
static void dq_q5_k(const uint8_t* b, float* y) {
    float d = h2f(rd16(b)), dmin = h2f(rd16(b + 2));
    const uint8_t* scales = b + 4; const uint8_t* qh = b + 16; const uint8_t* ql = b + 48;
    for (int j = 0; j < 4; ++j) {
        int sc0, m0, sc1, m1;
        q4k_scale_min(2 * j, scales, &sc0, &m0);
        q4k_scale_min(2 * j + 1, scales, &sc1, &m1);
        float d0 = d * sc0, mm0 = dmin * m0, d1 = d * sc1, mm1 = dmin * m1;
        for (int l = 0; l < 32; ++l) {
            int lo = ql[32 * j + l] & 0xF, hi = ql[32 * j + l] >> 4;
            y[64 * j + l] = d0 * (lo + (((qh[l] >> (2 * j)) & 1) << 4)) - mm0;
            y[64 * j + 32 + l] = d1 * (hi + (((qh[l] >> (2 * j + 1)) & 1) << 4)) - mm1;
        }
    }
}

// Dequantise one row of `cols` weights.
void orc_dequant_row(int type, const void* src, int64_t cols, float* dst) {
    const uint8_t* raw = (const uint8_t*)src;
    switch (type) {
        case ORC_Q4_0: for (int64_t i = 0; i < cols / 32; ++i) dq_q4_0(raw + i * 18, dst + i * 32); break;
        case ORC_Q5_0: for (int64_t i = 0; i < cols / 32; ++i) dq_q5_0(raw + i * 22, dst + i * 32); break;
        case ORC_Q5_1: for (int64_t i = 0; i < cols / 32; ++i) dq_q5_1(raw + i * 24, dst + i * 32); break;
        case ORC_Q2_K: for (int64_t i = 0; i < cols / 256; ++i) dq_q2_k(raw + i * 84, dst + i * 256); break;
        case ORC_Q3_K: for (int64_t i = 0; i < cols / 256; ++i) dq_q3_k(raw + i * 110, dst + i * 256); break;
        case ORC_Q5_K: for (int64_t i = 0; i < cols / 256; ++i) dq_q5_k(raw + i * 176, dst + i * 256); break;
        case ORC_BF16: for (int64_t i = 0; i < cols; ++i) { uint32_t u = (uint32_t)rd16(raw + 2 * i) << 16; memcpy(dst + i, &u, 4); } break;
        case ORC_F32: memcpy(dst, src, cols * 4); break;
        case ORC_F16: { const uint16_t* h = (const uint16_t*)src; for (int64_t i = 0; i < cols; ++i) dst[i] = h2f(h[i]); break; }
        case ORC_Q8_0: {
            const BlkQ80* b = (const BlkQ80*)src;
            for (int64_t i = 0; i < cols / 32; ++i) { float d = h2f(b[i].d); for (int k = 0; k < 32; ++k) dst[i * 32 + k] = d * b[i].qs[k]; }
            break;
        }
        case ORC_Q4_K: {
            const BlkQ4K* b = (const BlkQ4K*)src;
            for (int64_t i = 0; i < cols / 256; ++i) {
                float d = h2f(b[i].d), dmin = h2f(b[i].dmin);
                float* y = dst + i * 256;
                for (int j = 0; j < 4; ++j) {
                    int sc0, m0, sc1, m1;
                    q4k_scale_min(2 * j, b[i].scales, &sc0, &m0);
                    q4k_scale_min(2 * j + 1, b[i].scales, &sc1, &m1);
                    float d0 = d * sc0, mm0 = dmin * m0, d1 = d * sc1, mm1 = dmin * m1;
                    const uint8_t* q = b[i].qs + 32 * j;
                    for (int l = 0; l < 32; ++l) { y[64 * j + l] = d0 * (q[l] & 0xF) - mm0; y[64 * j + 32 + l] = d1 * (q[l] >> 4) - mm1; }
                }
            }
            break;
        }
        case ORC_Q6_K: {
            const BlkQ6K* b = (const BlkQ6K*)src;
            for (int64_t i = 0; i < cols / 256; ++i) {
                float d = h2f(b[i].d);
                float* y = dst + i * 256;
                for (int h = 0; h < 2; ++h) {
                    const uint8_t* ql = b[i].ql + 64 * h; const uint8_t* qh = b[i].qh + 32 * h; const int8_t* sc = b[i].scales + 8 * h;
                    for (int l = 0; l < 32; ++l) {
                        int is = l / 16;
                        int q1 = (int)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
                        int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                        int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                        int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                        y[128 * h + l] = d * sc[is] * q1; y[128 * h + l + 32] = d * sc[is + 2] * q2;
                        y[128 * h + l + 64] = d * sc[is + 4] * q3; y[128 * h + l + 96] = d * sc[is + 6] * q4;
                    }
                }
            }
            break;
        }
    }
}

void orc_dequant(int type, const void* src, int64_t rows, int64_t cols, float* dst) {
    int64_t rb = orc_row_bytes(type, cols);
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) orc_dequant_row(type, (const char*)src + r * rb, cols, dst + r * cols);
}

// ---------------------------------------------------------------- activation quantisation
// 8-bit activation blocks of 256 (for K-quant weights): one f32 scale, 256 int8,
// sixteen 16-element partial sums.  Rule: the scale maps the element of largest
// magnitude to -128 (clamped to 127), values round half away from zero.
void orc_quantize_q8k(const float* x, int64_t n, int8_t* qs, float* d, int16_t* bsums) {
    for (int64_t b = 0; b < n / 256; ++b) {
        const float* xb = x + b * 256; int8_t* q = qs + b * 256;
        float amax = 0.f, mx = 0.f;
        for (int j = 0; j < 256; ++j) { float ax = fabsf(xb[j]); if (ax > amax) { amax = ax; mx = xb[j]; } }
        if (amax == 0.f) { d[b] = 0.f; memset(q, 0, 256); for (int j = 0; j < 16; ++j) bsums[b * 16 + j] = 0; continue; }
        float iscale = -128.f / mx;
        for (int j = 0; j < 256; ++j) { float v = roundf(iscale * xb[j]); q[j] = (int8_t)(v > 127.f ? 127.f : v); }
        for (int j = 0; j < 16; ++j) { int s = 0; for (int k = 0; k < 16; ++k) s += q[j * 16 + k]; bsums[b * 16 + j] = (int16_t)s; }
        d[b] = 1.0f / iscale;
    }
}

// 8-bit activation blocks of 32 (for Q8_0 weights): scale = amax/127 stored as f16.
void orc_quantize_q80(const float* x, int64_t n, int8_t* qs, uint16_t* d) {
    for (int64_t b = 0; b < n / 32; ++b) {
        const float* xb = x + b * 32; float amax = 0.f;
        for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(xb[j]));
        float dd = amax / 127.f; float id = dd != 0.f ? 1.0f / dd : 0.f;
        d[b] = f2h(dd);
        for (int j = 0; j < 32; ++j) qs[b * 32 + j] = (int8_t)roundf(xb[j] * id);
    }
}

// ---------------------------------------------------------------- quantised matmul
#ifdef ORC_AVX2
static inline int32_t hsum_i32(__m256i v) {
    __m128i s = _mm_add_epi32(_mm256_castsi256_si128(v), _mm256_extracti128_si256(v, 1));
    s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0x4E));
    s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0xB1));
    return _mm_cvtsi128_si32(s);
}
#endif
static float dot_q4k_q8k(const BlkQ4K* w, const int8_t* qs, const float* dx, const int16_t* bs, int64_t nb, bool rev) {
    float acc = 0.f;
    for (int64_t bi = 0; bi < nb; ++bi) {
        int64_t b = rev ? nb - 1 - bi : bi;
        const int8_t* q8 = qs + b * 256;
        int32_t isum = 0, msum = 0;
#ifdef ORC_AVX2
        __m256i vsum = _mm256_setzero_si256();   // exact 32-bit integer sums: any order gives the same isum
#endif
        for (int j = 0; j < 4; ++j) {
            int sc0, m0, sc1, m1;
            q4k_scale_min(2 * j, w[b].scales, &sc0, &m0);
            q4k_scale_min(2 * j + 1, w[b].scales, &sc1, &m1);
            const uint8_t* q = w[b].qs + 32 * j;
#ifdef ORC_AVX2
            // 4-bit x 8-bit pairs: |sum of two| <= 2*15*128 fits 16 bits; times a 6-bit scale, pairwise, fits 32 bits.
            const __m256i qv = _mm256_loadu_si256((const __m256i*)q), nib = _mm256_set1_epi8(0xF);
            const __m256i p0 = _mm256_maddubs_epi16(_mm256_and_si256(qv, nib), _mm256_loadu_si256((const __m256i*)(q8 + 64 * j)));
            const __m256i p1 = _mm256_maddubs_epi16(_mm256_and_si256(_mm256_srli_epi16(qv, 4), nib), _mm256_loadu_si256((const __m256i*)(q8 + 64 * j + 32)));
            vsum = _mm256_add_epi32(vsum, _mm256_add_epi32(_mm256_madd_epi16(p0, _mm256_set1_epi16((short)sc0)), _mm256_madd_epi16(p1, _mm256_set1_epi16((short)sc1))));
#else
            int32_t s0 = 0, s1 = 0;
            for (int l = 0; l < 32; ++l) { s0 += (int)(q[l] & 0xF) * q8[64 * j + l]; s1 += (int)(q[l] >> 4) * q8[64 * j + 32 + l]; }
            isum += sc0 * s0 + sc1 * s1;
#endif
            msum += m0 * ((int)bs[b * 16 + 4 * j] + bs[b * 16 + 4 * j + 1]) + m1 * ((int)bs[b * 16 + 4 * j + 2] + bs[b * 16 + 4 * j + 3]);
        }
#ifdef ORC_AVX2
        isum = hsum_i32(vsum);
#endif
        float d = h2f(w[b].d), dmin = h2f(w[b].dmin);
        acc += dx[b] * (d * (float)isum - dmin * (float)msum);
    }
    return acc;
}

static float dot_q6k_q8k(const BlkQ6K* w, const int8_t* qs, const float* dx, int64_t nb, bool rev) {
    float acc = 0.f;
    for (int64_t bi = 0; bi < nb; ++bi) {
        int64_t b = rev ? nb - 1 - bi : bi;
        const int8_t* q8 = qs + b * 256;
        int32_t isum = 0;
#ifdef ORC_AVX2
        // (q - 32) * y = q * y - 32 * y with q in 0..63: pair sums stay within 16 bits (<= 2*63*128 + 2*32*128), and
        // the 8-bit scale of each 16-element run multiplies pairwise into exact 32-bit sums.  A 32-byte vector holds
        // two runs: the low half takes scale 2k, the high half scale 2k+1.
        __m256i vsum = _mm256_setzero_si256();
        const __m256i nib = _mm256_set1_epi8(0xF), two = _mm256_set1_epi8(3), off = _mm256_set1_epi8(32);
        for (int h = 0; h < 2; ++h) {
            const __m256i l0 = _mm256_loadu_si256((const __m256i*)(w[b].ql + 64 * h)), l1 = _mm256_loadu_si256((const __m256i*)(w[b].ql + 64 * h + 32));
            const __m256i hv = _mm256_loadu_si256((const __m256i*)(w[b].qh + 32 * h));
            const int8_t* sc = w[b].scales + 8 * h; const int8_t* y = q8 + 128 * h;
            __m256i qv[4];
            qv[0] = _mm256_or_si256(_mm256_and_si256(l0, nib), _mm256_slli_epi16(_mm256_and_si256(hv, two), 4));
            qv[1] = _mm256_or_si256(_mm256_and_si256(l1, nib), _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(hv, 2), two), 4));
            qv[2] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(l0, 4), nib), _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(hv, 4), two), 4));
            qv[3] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(l1, 4), nib), _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(hv, 6), two), 4));
            for (int k = 0; k < 4; ++k) {
                const __m256i yv = _mm256_loadu_si256((const __m256i*)(y + 32 * k));
                const __m256i p = _mm256_sub_epi16(_mm256_maddubs_epi16(qv[k], yv), _mm256_maddubs_epi16(off, yv));
                const __m256i sv = _mm256_set_m128i(_mm_set1_epi16((short)sc[2 * k + 1]), _mm_set1_epi16((short)sc[2 * k]));
                vsum = _mm256_add_epi32(vsum, _mm256_madd_epi16(p, sv));
            }
        }
        isum = hsum_i32(vsum);
#else
        for (int h = 0; h < 2; ++h) {
            const uint8_t* ql = w[b].ql + 64 * h; const uint8_t* qh = w[b].qh + 32 * h; const int8_t* sc = w[b].scales + 8 * h;
            const int8_t* y = q8 + 128 * h;
            int32_t s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int l = 0; l < 32; ++l) {
                int is = l / 16;
                int q1 = (int)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
                int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                s[is] += q1 * y[l]; s[is + 2] += q2 * y[l + 32]; s[is + 4] += q3 * y[l + 64]; s[is + 6] += q4 * y[l + 96];
            }
            for (int k = 0; k < 8; ++k) isum += (int)sc[k] * s[k];
        }
#endif
        acc += dx[b] * (h2f(w[b].d) * (float)isum);
    }
    return acc;
}

static float dot_q80_q80(const BlkQ80* w, const int8_t* qs, const uint16_t* dx, int64_t nb, bool rev) {
    float acc = 0.f;
    for (int64_t bi = 0; bi < nb; ++bi) {
        int64_t b = rev ? nb - 1 - bi : bi;
        int32_t s = 0;
        for (int k = 0; k < 32; ++k) s += (int)w[b].qs[k] * qs[b * 32 + k];
        acc += (float)s * (h2f(w[b].d) * h2f(dx[b]));
    }
    return acc;
}

// y[t, n] = sum_k x[t, k] * W[n, k]   (W block-quantised along k, row-major [out, in]).
// mode 1: activations quantised per row, integer block dots (the CPU path's behaviour).
// mode 2: weights dequantised to f32, plain f32 dot (the reference's own validation mode,
//         src/weights.rs:274-300).
// mode 3: mode 1 with the f32 accumulation over blocks taken in reverse order - the same arithmetic under
//         another association, used to measure how far two valid evaluation orders of the reference's
//         CPU path drift apart (its own tests allow for this: tests/smollm3_gguf_reference.rs:46-55).
void orc_qmatmul(int type, const void* W, int64_t out, int64_t in, const float* x, int64_t T, float* y, int mode) {
    int64_t rb = orc_row_bytes(type, in);
    bool quantised = (type == ORC_Q4_K || type == ORC_Q6_K || type == ORC_Q8_0);
    if ((mode == 1 || mode == 3) && quantised) {
        const bool rev = mode == 3;
        std::vector<int8_t> qs((size_t)T * in);
        if (type == ORC_Q8_0) {
            std::vector<uint16_t> dx((size_t)T * (in / 32));
#pragma omp parallel for schedule(static)
            for (int64_t t = 0; t < T; ++t) orc_quantize_q80(x + t * in, in, qs.data() + t * in, dx.data() + t * (in / 32));
#pragma omp parallel for schedule(static)
            for (int64_t n = 0; n < out; ++n) {
                const BlkQ80* w = (const BlkQ80*)((const char*)W + n * rb);
                for (int64_t t = 0; t < T; ++t) y[t * out + n] = dot_q80_q80(w, qs.data() + t * in, dx.data() + t * (in / 32), in / 32, rev);
            }
            return;
        }
        int64_t nb = in / 256;
        std::vector<float> dx((size_t)T * nb);
        std::vector<int16_t> bs((size_t)T * nb * 16);
#pragma omp parallel for schedule(static)
        for (int64_t t = 0; t < T; ++t) orc_quantize_q8k(x + t * in, in, qs.data() + t * in, dx.data() + t * nb, bs.data() + t * nb * 16);
#pragma omp parallel for schedule(static)
        for (int64_t n = 0; n < out; ++n) {
            const char* w = (const char*)W + n * rb;
            for (int64_t t = 0; t < T; ++t) {
                y[t * out + n] = type == ORC_Q4_K
                    ? dot_q4k_q8k((const BlkQ4K*)w, qs.data() + t * in, dx.data() + t * nb, bs.data() + t * nb * 16, nb, rev)
                    : dot_q6k_q8k((const BlkQ6K*)w, qs.data() + t * in, dx.data() + t * nb, nb, rev);
            }
        }
        return;
    }
#pragma omp parallel
    {
        std::vector<float> row((size_t)in);
#pragma omp for schedule(static)
        for (int64_t n = 0; n < out; ++n) {
            orc_dequant_row(type, (const char*)W + n * rb, in, row.data());
            for (int64_t t = 0; t < T; ++t) {
                const float* xt = x + t * in; float acc = 0.f;
                for (int64_t k = 0; k < in; ++k) acc += xt[k] * row[k];
                y[t * out + n] = acc;
            }
        }
    }
}

// The Q8_K-dequantised activation row (what mode 1 effectively multiplies the weights by);
// used to bound the error of the tensor-core path, which consumes these values in f16.
void orc_fake_quant_rows(int type, const float* x, int64_t T, int64_t in, float* out) {
    std::vector<int8_t> qs((size_t)in);
    for (int64_t t = 0; t < T; ++t) {
        if (type == ORC_Q8_0) {
            std::vector<uint16_t> d((size_t)in / 32);
            orc_quantize_q80(x + t * in, in, qs.data(), d.data());
            for (int64_t k = 0; k < in; ++k) out[t * in + k] = h2f(d[k / 32]) * qs[k];
        } else {
            std::vector<float> d((size_t)in / 256); std::vector<int16_t> bs((size_t)in / 16);
            orc_quantize_q8k(x + t * in, in, qs.data(), d.data(), bs.data());
            for (int64_t k = 0; k < in; ++k) out[t * in + k] = d[k / 256] * qs[k];
        }
    }
}

// Embedding rows: dequantise the selected rows (src/model_weights.rs:489-502), then scale.
void orc_embed(int type, const void* W, int64_t cols, const uint32_t* ids, int64_t T, float scale, float* out) {
    int64_t rb = orc_row_bytes(type, cols);
    for (int64_t t = 0; t < T; ++t) {
        orc_dequant_row(type, (const char*)W + (int64_t)ids[t] * rb, cols, out + t * cols);
        if (scale != 1.0f) for (int64_t k = 0; k < cols; ++k) out[t * cols + k] *= scale;
    }
}

// ---------------------------------------------------------------- elementwise
// RMSNorm in f32: x / sqrt(mean(x^2) + eps) * w   (src/model_weights.rs:563-565).
void orc_rmsnorm(const float* x, const float* w, float eps, int64_t rows, int64_t dim, float* y) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const float* xr = x + r * dim; float ss = 0.f;
        for (int64_t k = 0; k < dim; ++k) ss += xr[k] * xr[k];
        float m = sqrtf(ss / (float)dim + eps);
        for (int64_t k = 0; k < dim; ++k) y[r * dim + k] = xr[k] / m * w[k];
    }
}

static inline float silu_f(float v) { return v / (1.0f + expf(-v)); }
static inline float gelu_tanh_f(float v) {
    return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * v * (1.0f + 0.044715f * v * v)));
}

// act(gate) * up, act 0 = SiLU, 1 = tanh-GELU   (src/decoder.rs:298-305).
void orc_act_mul(const float* gate, const float* up, int64_t n, int act, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = (act == 0 ? silu_f(gate[i]) : gelu_tanh_f(gate[i])) * up[i];
}

void orc_softcap(float* x, int64_t n, float cap) {
    for (int64_t i = 0; i < n; ++i) x[i] = tanhf(x[i] * (1.0f / cap)) * cap;
}

// RoPE tables (src/decoder.rs:136-201): inv_freq in f64 then f32; angle = f32(pos) * inv_freq.
// factors (may be null): per-frequency divisors, f32(base / f64(factor)) as RotaryEmbedding::new does for GGUF
// `rope_freqs.weight` (src/decoder.rs:136-152).
void orc_rope_tables(double theta, int rotary_dim, int64_t capacity, const float* factors, float* cos_t, float* sin_t) {
    int half = rotary_dim / 2;
    std::vector<float> inv((size_t)half);
    for (int i = 0; i < half; ++i) {
        double base = 1.0 / pow(theta, (double)(2 * i) / (double)rotary_dim);
        inv[i] = factors ? (float)(base / (double)factors[i]) : (float)base;
    }
    for (int64_t p = 0; p < capacity; ++p)
        for (int i = 0; i < half; ++i) { float a = (float)p * inv[i]; cos_t[p * half + i] = cosf(a); sin_t[p * half + i] = sinf(a); }
}

// Half-split rotation of the first rotary_dim dims of every head of x [T, heads, d],
// token t at absolute position pos[t]   (src/decoder.rs:203-257).
void orc_rope_apply(float* x, int64_t T, int heads, int d, int rotary_dim, const int32_t* pos, const float* cos_t, const float* sin_t) {
    int half = rotary_dim / 2;
    for (int64_t t = 0; t < T; ++t) {
        const float* c = cos_t + (int64_t)pos[t] * half; const float* s = sin_t + (int64_t)pos[t] * half;
        for (int h = 0; h < heads; ++h) {
            float* v = x + (t * heads + h) * d;
            for (int i = 0; i < half; ++i) {
                float x1 = v[i], x2 = v[i + half];
                v[i] = x1 * c[i] - x2 * s[i];
                v[i + half] = x1 * s[i] + x2 * c[i];
            }
        }
    }
}

// ---------------------------------------------------------------- attention
// Paged causal GQA attention for a ragged batch, restating the CPU custom op
// (crates/macllm-kernels/src/paged_attention.rs:614-709): one key at a time, online softmax.
// Extended with the sliding-window visibility rule of src/decoder.rs:4515-4532 (window 0 = full).
//   q, out:   [T, q_heads, d] f32 (token-major)
//   k_pool,v_pool: [blocks, layers, kv_heads, block_tokens, d] f32, or f16 when kv_f16 != 0
//   page_table: lane l's pages are block ids page_table[page_off[l] + i]
// mode 0 = online softmax (C1), mode 1 = dense two-pass softmax (D1: max, exp, sum, divide, then P.V)
void orc_paged_attention(const float* q, float* out, const void* k_pool, const void* v_pool, int kv_f16,
                         const uint32_t* page_table, const int32_t* page_off, const int32_t* start_pos,
                         const int32_t* lane_len, int lanes, int q_heads, int kv_heads, int d, int block_tokens,
                         int layers, int layer, float scale, float softcap, int window, int mode) {
    std::vector<int64_t> q_off((size_t)lanes + 1, 0);
    for (int l = 0; l < lanes; ++l) q_off[l + 1] = q_off[l] + lane_len[l];
    int groups = q_heads / kv_heads;
    int64_t total_rows = q_off[lanes];
    // flatten (lane,row) for parallelism
    std::vector<int> row_lane((size_t)total_rows);
    for (int l = 0; l < lanes; ++l) for (int64_t r = q_off[l]; r < q_off[l + 1]; ++r) row_lane[r] = l;
#pragma omp parallel
    {
        std::vector<float> acc((size_t)d), scores;
#pragma omp for schedule(dynamic, 4) collapse(2)
        for (int64_t row = 0; row < total_rows; ++row) {
            for (int h = 0; h < q_heads; ++h) {
                int l = row_lane[row];
                int kvh = h / groups;
                int64_t p = (int64_t)start_pos[l] + (row - q_off[l]);  // absolute position of this query
                int64_t first = 0;
                if (window > 0 && p - (window - 1) > 0) first = p - (window - 1);
                const float* qv = q + (row * q_heads + h) * d;
                auto kv_ptr = [&](const void* pool, int64_t pos) -> int64_t {
                    int64_t blk = page_table[page_off[l] + pos / block_tokens];
                    return (((blk * layers + layer) * kv_heads + kvh) * block_tokens + pos % block_tokens) * (int64_t)d;
                };
                auto ld = [&](const void* pool, int64_t idx) -> float {
                    return kv_f16 ? h2f(((const uint16_t*)pool)[idx]) : ((const float*)pool)[idx];
                };
                float* o = out + (row * q_heads + h) * d;
                if (mode == 0) {
                    float mx = -INFINITY, norm = 0.f;
                    std::fill(acc.begin(), acc.end(), 0.f);
                    for (int64_t pos = first; pos <= p; ++pos) {
                        int64_t ki = kv_ptr(k_pool, pos);
                        float s = 0.f;
                        for (int i = 0; i < d; ++i) s += qv[i] * ld(k_pool, ki + i);
                        s *= scale;
                        if (softcap != 0.f) s = tanhf(s / softcap) * softcap;
                        float nm = fmaxf(mx, s);
                        float ow = std::isfinite(mx) ? expf(mx - nm) : 0.f;
                        float nw = expf(s - nm);
                        for (int i = 0; i < d; ++i) acc[i] = acc[i] * ow + ld(v_pool, ki + i) * nw;
                        norm = norm * ow + nw; mx = nm;
                    }
                    for (int i = 0; i < d; ++i) o[i] = acc[i] / norm;
                } else {
                    int64_t n = p - first + 1;
                    scores.resize((size_t)n);
                    float mx = -INFINITY;
                    for (int64_t j = 0; j < n; ++j) {
                        int64_t ki = kv_ptr(k_pool, first + j);
                        float s = 0.f;
                        for (int i = 0; i < d; ++i) s += qv[i] * ld(k_pool, ki + i);
                        s *= scale;
                        if (softcap != 0.f) s = tanhf(s * (1.0f / softcap)) * softcap;
                        scores[j] = s; mx = fmaxf(mx, s);
                    }
                    float sum = 0.f;
                    for (int64_t j = 0; j < n; ++j) { scores[j] = expf(scores[j] - mx); sum += scores[j]; }
                    for (int64_t j = 0; j < n; ++j) scores[j] /= sum;
                    std::fill(acc.begin(), acc.end(), 0.f);
                    for (int64_t j = 0; j < n; ++j) {
                        int64_t vi = kv_ptr(v_pool, first + j);
                        float pj = scores[j];
                        for (int i = 0; i < d; ++i) acc[i] += pj * ld(v_pool, vi + i);
                    }
                    for (int i = 0; i < d; ++i) o[i] = acc[i];
                }
            }
        }
    }
}

// Scatter k,v [T, kv_heads, d] f32 of one layer into the pool at slots[t] = block*block_tokens + row
// (crates/macllm-kv/src/cache.rs:2543-2643: token at absolute position p -> block p / bt, row p % bt).
void orc_kv_scatter(const float* k, const float* v, void* k_pool, void* v_pool, int kv_f16, const int64_t* slots,
                    int64_t T, int kv_heads, int d, int block_tokens, int layers, int layer) {
    for (int64_t t = 0; t < T; ++t) {
        int64_t blk = slots[t] / block_tokens, row = slots[t] % block_tokens;
        for (int h = 0; h < kv_heads; ++h) {
            int64_t dst = (((blk * layers + layer) * kv_heads + h) * block_tokens + row) * (int64_t)d;
            const float* ks = k + (t * kv_heads + h) * d; const float* vs = v + (t * kv_heads + h) * d;
            if (kv_f16) {
                for (int i = 0; i < d; ++i) { ((uint16_t*)k_pool)[dst + i] = f2h(ks[i]); ((uint16_t*)v_pool)[dst + i] = f2h(vs[i]); }
            } else {
                memcpy((float*)k_pool + dst, ks, d * 4); memcpy((float*)v_pool + dst, vs, d * 4);
            }
        }
    }
}

// ---------------------------------------------------------------- MoE routing
// Top-k by (logit desc, index asc), softmax over the selected k only (src/decoder.rs:448-554).
// experts_out [T, k] in selection order (best first); weights_out [T, k].
void orc_moe_route(const float* logits, int64_t T, int experts, int k, int32_t* experts_out, float* weights_out) {
    std::vector<int> cand((size_t)experts);
    for (int64_t t = 0; t < T; ++t) {
        const float* row = logits + t * experts;
        for (int e = 0; e < experts; ++e) cand[e] = e;
        std::sort(cand.begin(), cand.end(), [&](int a, int b) {
            if (row[a] > row[b]) return true;
            if (row[a] < row[b]) return false;
            return a < b;
        });
        float mx = -INFINITY;
        for (int i = 0; i < k; ++i) mx = fmaxf(mx, row[cand[i]]);
        float den = 0.f;
        for (int i = 0; i < k; ++i) den += expf(row[cand[i]] - mx);
        for (int i = 0; i < k; ++i) { experts_out[t * k + i] = cand[i]; weights_out[t * k + i] = expf(row[cand[i]] - mx) / den; }
    }
}

// ---------------------------------------------------------------- recurrent mixers
// Stable softplus as the reference writes it: max(x, 0) + ln(1 + exp(-|x|)).
static inline float softplus_stable(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

// Gated DeltaNet decay: exp(softplus(alpha + time_bias[h]) * state_decay[h]) for alpha [tokens][heads]
// (crates/macllm-kernels/src/gated_delta.rs:96-104).
void orc_gated_delta_decay(const float* alpha, const float* time_bias, const float* state_decay, int64_t tokens, int heads, float* out) {
    for (int64_t i = 0; i < tokens * heads; ++i) {
        int h = (int)(i % heads);
        out[i] = expf(softplus_stable(alpha[i] + time_bias[h]) * state_decay[h]);
    }
}

// Gated DeltaNet recurrence over ragged lanes (crates/macllm-kernels/src/gated_delta.rs:396-431).  Rows of lane l are
// cu[l] .. cu[l+1]; query / key [rows][heads][key_dim] (already normalised, query already scaled), value / out
// [rows][heads][value_dim], decay / beta [rows][heads]; state [lanes][heads][key_dim][value_dim], read from state_in and
// written to state_out (the input stays as it was: a failed forward must be able to fall back to it).  Per head and value
// column: memory = sum_k S[k] * decay * key[k]; delta = (value - memory) * beta; S[k] = S[k] * decay + key[k] * delta;
// out = sum_k S[k] * query[k] - every product and sum rounded on its own, in this order.
void orc_gated_delta_recurrence(const float* query, const float* key, const float* value, const float* decay, const float* beta,
                                const int32_t* cu, int lanes, int heads, int key_dim, int value_dim, const float* state_in,
                                float* state_out, float* out) {
    for (int l = 0; l < lanes; ++l)
        for (int h = 0; h < heads; ++h) {
            const int64_t sb = ((int64_t)l * heads + h) * key_dim * value_dim;
            for (int v = 0; v < value_dim; ++v) {
                for (int k = 0; k < key_dim; ++k) state_out[sb + (int64_t)k * value_dim + v] = state_in[sb + (int64_t)k * value_dim + v];
                for (int64_t r = cu[l]; r < cu[l + 1]; ++r) {
                    const int64_t th = r * heads + h;
                    const float* kk = key + th * key_dim; const float* qq = query + th * key_dim;
                    float memory = 0.f;
                    for (int k = 0; k < key_dim; ++k) memory += state_out[sb + (int64_t)k * value_dim + v] * decay[th] * kk[k];
                    const float delta = (value[th * value_dim + v] - memory) * beta[th];
                    float projected = 0.f;
                    for (int k = 0; k < key_dim; ++k) {
                        float* sp = state_out + sb + (int64_t)k * value_dim + v;
                        const float next = *sp * decay[th] + kk[k] * delta;
                        *sp = next;
                        projected += next * qq[k];
                    }
                    out[th * value_dim + v] = projected;
                }
            }
        }
}

// Mamba2 selective scan over ragged lanes (crates/macllm-kernels/src/mamba2.rs:255-289).  xbc [rows][H*P + 2*G*N] laid out
// [x | B | C], raw_dt [rows][H], dt_bias / a / d [H], state [lanes][H][P][N]; out [rows][H][P].  Per token and head:
// delta = softplus(dt + dt_bias), decay = exp(delta * a); per position: S[n] = decay * S[n] + delta * x * B[n],
// out = sum_n S[n] * C[n] + d * x.  Heads are divided evenly into G contiguous groups that share B and C.
void orc_mamba2_scan(const float* xbc, const float* raw_dt, const float* dt_bias, const float* a, const float* d, const int32_t* cu,
                     int lanes, int heads, int head_dim, int state_size, int groups, const float* state_in, float* state_out, float* out) {
    const int64_t inner = (int64_t)heads * head_dim, gsw = (int64_t)groups * state_size, width = inner + 2 * gsw;
    const int hpg = heads / groups;
    for (int l = 0; l < lanes; ++l) {
        float* S = state_out + (int64_t)l * inner * state_size;
        memcpy(S, state_in + (int64_t)l * inner * state_size, sizeof(float) * (size_t)(inner * state_size));
        for (int64_t r = cu[l]; r < cu[l + 1]; ++r) {
            const float* row = xbc + r * width;
            for (int h = 0; h < heads; ++h) {
                const float delta = softplus_stable(raw_dt[r * heads + h] + dt_bias[h]);
                const float dec = expf(delta * a[h]);
                const float* B = row + inner + (int64_t)(h / hpg) * state_size;
                const float* Cv = row + inner + gsw + (int64_t)(h / hpg) * state_size;
                for (int p = 0; p < head_dim; ++p) {
                    const int64_t lane_i = (int64_t)h * head_dim + p;
                    const float x = row[lane_i];
                    float projected = 0.f;
                    for (int n = 0; n < state_size; ++n) {
                        float* sp = S + lane_i * state_size + n;
                        const float next = dec * *sp + delta * x * B[n];
                        *sp = next;
                        projected += next * Cv[n];
                    }
                    out[r * inner + lane_i] = projected + d[h] * x;
                }
            }
        }
    }
}

// Short convolution over ragged lanes (ShortConvolution::forward_lane after the input projection and before the output
// projection, src/decoder.rs:1436-1492): bcx [rows][3*hidden] laid out [B | C | x]; Bx = B * x; a causal depthwise
// cross-correlation of Bx with kernel [hidden][K] (tap K-1 meets the current token) over the lane's tail of the last
// K-1 Bx rows [lanes][K-1][hidden] followed by its new rows, summed from the oldest tap on; out = C * that.  The new
// tail is the last K-1 rows of the window.
void orc_short_conv(const float* bcx, const float* kernel, const int32_t* cu, int lanes, int hidden, int K, const float* tail_in,
                    float* tail_out, float* out) {
    const int hist = K - 1;
    for (int l = 0; l < lanes; ++l) {
        const int64_t n = cu[l + 1] - cu[l];
        std::vector<float> window((size_t)((hist + n) * hidden));
        for (int64_t i = 0; i < (int64_t)hist * hidden; ++i) window[(size_t)i] = tail_in[(int64_t)l * hist * hidden + i];
        for (int64_t t = 0; t < n; ++t)
            for (int c = 0; c < hidden; ++c) {
                const float* row = bcx + (cu[l] + t) * 3 * hidden;
                window[(size_t)((hist + t) * hidden + c)] = row[c] * row[2 * hidden + c];
            }
        for (int64_t t = 0; t < n; ++t)
            for (int c = 0; c < hidden; ++c) {
                float sum = window[(size_t)(t * hidden + c)] * kernel[(int64_t)c * K];
                for (int j = 1; j < K; ++j) sum += window[(size_t)((t + j) * hidden + c)] * kernel[(int64_t)c * K + j];
                out[(cu[l] + t) * hidden + c] = bcx[(cu[l] + t) * 3 * hidden + hidden + c] * sum;
            }
        for (int64_t i = 0; i < (int64_t)hist * hidden; ++i) tail_out[(int64_t)l * hist * hidden + i] = window[(size_t)(n * hidden + i)];
    }
}

// ---------------------------------------------------------------- sampling
// First-index argmax under a total order on floats (src/sampling.rs:425-433).
static inline int32_t total_key(float f) { int32_t b; memcpy(&b, &f, 4); return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1); }
int64_t orc_argmax(const float* v, int64_t n) {
    int64_t best = 0;
    for (int64_t i = 1; i < n; ++i) if (total_key(v[i]) > total_key(v[best])) best = i;
    return best;
}

// Threads the OpenMP loops of this library use from now on (launchers such as torchrun export OMP_NUM_THREADS=1).
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int orc_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

}  // extern "C"
