// Quantised GEMM on the 5th-generation tensor cores (tcgen05) for prefill chunks and wide decode
// batches:  y[t][n] = sum_k xh[t][k] * dequant(W)[n][k].
//
// Replaces LinearOp::Quantized forward (src/model_weights.rs:346-377 of the reference) when many
// activation rows share one pass over the weights.  Weights stay in GGUF block format in HBM and are
// dequantised to f16 on their way into shared memory; activations are the f16 image of the same
// 8-bit-quantised rows the integer path uses, so both paths see identical operands up to one f16
// rounding each.  Accumulation is f32 in tensor memory.
//
// Shape of one CTA: 128 weight rows (the MMA M dimension, one TMEM lane per row) x BN tokens (the MMA
// N dimension, one TMEM column per token), K walked in stages of 128.  Operands sit in shared memory
// in the K-major "interleaved" (no swizzle) canonical layout: 8 rows x 16 bytes form one 128-byte
// core matrix, core matrices of consecutive 8-row groups are 128 bytes apart (stride byte offset),
// consecutive 16-byte K chunks are rows/8*128 bytes apart (leading byte offset).  One elected thread
// issues eight K=16 MMAs per stage and commits them to the stage's mbarrier; the other threads are
// already dequantising the next stage.  Small matrices are split along K across CTAs and reduced in
// split order by a second kernel, so results do not depend on scheduling.
//
// Every wait on an mbarrier is bounded: after the limit the kernel records a status word and carries
// on to its teardown (tensor memory is always released).
#include "qgemm_tc.h"
#include "kernels.h"

namespace mk {

namespace {

constexpr int TC_THREADS = 256;
constexpr int TC_BM = 128;
constexpr int TC_BK = 128;
constexpr uint32_t TC_SPIN_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

// Bounded wait; returns false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit) {
    uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i <= limit; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version for sm_100
    return d;                // layout type 0 = no swizzle, base offset 0
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ uint32_t scale_byte(uint32_t y, uint32_t z, uint32_t w, int i) {
    uint32_t word = (i >> 2) == 0 ? y : ((i >> 2) == 1 ? z : w);
    return (word >> ((i & 3) * 8)) & 0xFFu;
}

__device__ __forceinline__ void q4k_scale_min_reg(uint32_t y, uint32_t z, uint32_t w, int j, int& sc, int& mn) {
    if (j < 4) {
        sc = scale_byte(y, z, w, j) & 63;
        mn = scale_byte(y, z, w, j + 4) & 63;
    } else {
        uint32_t a = scale_byte(y, z, w, j + 4);
        sc = (a & 0xF) | ((scale_byte(y, z, w, j - 4) >> 6) << 4);
        mn = (a >> 4) | ((scale_byte(y, z, w, j) >> 6) << 4);
    }
}

// Four bytes b0..b3 (each < 64) -> two half2 holding (b0, b1) and (b2, b3) minus `bias`, times `scale`,
// plus `neg_offset`, rounded once per element.
__device__ __forceinline__ void bytes_to_half4(uint32_t bytes, __half2 bias, __half2 scale, __half2 neg_offset, uint32_t& o01,
                                               uint32_t& o23) {
    uint32_t p01 = __byte_perm(bytes, 0x64646464u, 0x4140);
    uint32_t p23 = __byte_perm(bytes, 0x64646464u, 0x4342);
    __half2 h01 = __hsub2(*reinterpret_cast<__half2*>(&p01), bias);
    __half2 h23 = __hsub2(*reinterpret_cast<__half2*>(&p23), bias);
    h01 = __hfma2(h01, scale, neg_offset);
    h23 = __hfma2(h23, scale, neg_offset);
    o01 = *reinterpret_cast<uint32_t*>(&h01);
    o23 = *reinterpret_cast<uint32_t*>(&h23);
}

// Same for w = q * s - o where s and o are f32 values split into an f16 head and an f16 tail, so the
// f16 result carries one rounding relative to w itself instead of the (larger) roundings of s and o:
// w = fma(q, s_hi, -o_hi) + fma(q, s_lo, -o_lo).
struct SplitScale {
    __half2 s_hi, s_lo, o_hi, o_lo;  // o_* hold the negated offset
};
__device__ __forceinline__ SplitScale make_split(float s, float o) {
    SplitScale r;
    __half sh = __float2half_rn(s), oh = __float2half_rn(-o);
    r.s_hi = __half2half2(sh);
    r.o_hi = __half2half2(oh);
    r.s_lo = __float2half2_rn(s - __half2float(sh));
    r.o_lo = __float2half2_rn(-o - __half2float(oh));
    return r;
}
__device__ __forceinline__ void nibbles_to_half4(uint32_t bytes, __half2 bias, const SplitScale& sp, uint32_t& o01, uint32_t& o23) {
    uint32_t p01 = __byte_perm(bytes, 0x64646464u, 0x4140);
    uint32_t p23 = __byte_perm(bytes, 0x64646464u, 0x4342);
    __half2 q01 = __hsub2(*reinterpret_cast<__half2*>(&p01), bias);
    __half2 q23 = __hsub2(*reinterpret_cast<__half2*>(&p23), bias);
    __half2 h01 = __hadd2(__hfma2(q01, sp.s_hi, sp.o_hi), __hfma2(q01, sp.s_lo, sp.o_lo));
    __half2 h23 = __hadd2(__hfma2(q23, sp.s_hi, sp.o_hi), __hfma2(q23, sp.s_lo, sp.o_lo));
    o01 = *reinterpret_cast<uint32_t*>(&h01);
    o23 = *reinterpret_cast<uint32_t*>(&h23);
}

struct TcParams {
    QWeight W;
    const __half* xh;
    int T, K, out;
    float* y;         // direct output when splits == 1
    int ldy;
    float* partial;   // [splits][T][out] when splits > 1
    int splits, stages_per_split;
    float out_scale, softcap;
    int32_t* status;
};

// Dequantise 64 consecutive K elements of one weight row into eight 16-byte chunks of the A tile.
__device__ __forceinline__ void dequant_store_a(const TcParams& p, int row_global, int ks, int c, uint8_t* a_stage, int row) {
    auto chunk_ptr = [&](int chunk) -> uint4* {
        return reinterpret_cast<uint4*>(a_stage + chunk * (TC_BM / 8 * 128) + (row >> 3) * 128 + (row & 7) * 16);
    };
    if (row_global >= p.out) {
        uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int i = 0; i < 8; ++i) *chunk_ptr(8 * c + i) = z;
        return;
    }
    if (p.W.type == QT_Q4_K) {
        int nb = p.K / 256;
        int ib = ks >> 1, j = (ks & 1) * 2 + c;
        const uint8_t* blk = (const uint8_t*)p.W.p0 + ((int64_t)row_global * nb + ib) * 144;
        uint4 hdr = *reinterpret_cast<const uint4*>(blk);
        uint4 q0 = *reinterpret_cast<const uint4*>(blk + 16 + 32 * j);
        uint4 q1 = *reinterpret_cast<const uint4*>(blk + 16 + 32 * j + 16);
        float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFF)));
        float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
        int sc0, m0, sc1, m1;
        q4k_scale_min_reg(hdr.y, hdr.z, hdr.w, 2 * j, sc0, m0);
        q4k_scale_min_reg(hdr.y, hdr.z, hdr.w, 2 * j + 1, sc1, m1);
        SplitScale sp0 = make_split(d * (float)sc0, dmin * (float)m0);
        SplitScale sp1 = make_split(d * (float)sc1, dmin * (float)m1);
        __half2 bias = __float2half2_rn(1024.f);
        uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint4 lo, hi;
            nibbles_to_half4(words[2 * i] & 0x0F0F0F0Fu, bias, sp0, lo.x, lo.y);
            nibbles_to_half4(words[2 * i + 1] & 0x0F0F0F0Fu, bias, sp0, lo.z, lo.w);
            nibbles_to_half4((words[2 * i] >> 4) & 0x0F0F0F0Fu, bias, sp1, hi.x, hi.y);
            nibbles_to_half4((words[2 * i + 1] >> 4) & 0x0F0F0F0Fu, bias, sp1, hi.z, hi.w);
            *chunk_ptr(8 * c + i) = lo;
            *chunk_ptr(8 * c + 4 + i) = hi;
        }
    } else if (p.W.type == QT_Q6_K) {
        int nb = p.K / 256;
        int64_t b = (int64_t)row_global * nb + (ks >> 1);
        int hf = ks & 1;
        uint4 qa = *reinterpret_cast<const uint4*>((const uint8_t*)p.W.p0 + b * 128 + hf * 64 + 16 * c);
        uint4 qb = *reinterpret_cast<const uint4*>((const uint8_t*)p.W.p0 + b * 128 + hf * 64 + 32 + 16 * c);
        uint4 qh = *reinterpret_cast<const uint4*>((const uint8_t*)p.W.p1 + b * 64 + hf * 32 + 16 * c);
        const int8_t* sc = (const int8_t*)p.W.p2 + b * 16 + hf * 8 + c;
        float d = __half2float(((const __half*)p.W.p3)[b]);
        __half2 bias = __float2half2_rn(1056.f);  // 1024 (magic exponent) + 32 (re-centring)
        __half2 zero = __float2half2_rn(0.f);
        uint32_t a[4] = {qa.x, qa.y, qa.z, qa.w}, bq[4] = {qb.x, qb.y, qb.z, qb.w}, h[4] = {qh.x, qh.y, qh.z, qh.w};
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            __half2 s = __float2half2_rn(d * (float)sc[2 * g]);
#pragma unroll
            for (int half8 = 0; half8 < 2; ++half8) {
                uint4 o;
                uint32_t v0, v1;
                {
                    uint32_t src = (g & 1) ? bq[2 * half8] : a[2 * half8];
                    uint32_t nib = ((g >> 1) ? (src >> 4) : src) & 0x0F0F0F0Fu;
                    v0 = nib | (((h[2 * half8] >> (2 * g)) & 0x03030303u) << 4);
                    src = (g & 1) ? bq[2 * half8 + 1] : a[2 * half8 + 1];
                    nib = ((g >> 1) ? (src >> 4) : src) & 0x0F0F0F0Fu;
                    v1 = nib | (((h[2 * half8 + 1] >> (2 * g)) & 0x03030303u) << 4);
                }
                bytes_to_half4(v0, bias, s, zero, o.x, o.y);
                bytes_to_half4(v1, bias, s, zero, o.z, o.w);
                *chunk_ptr(4 * g + 2 * c + half8) = o;
            }
        }
    } else {  // QT_Q8_0 planes
        int nbk = p.K / 32;
        const int8_t* qs = (const int8_t*)p.W.p0 + (int64_t)row_global * p.K + ks * TC_BK + 64 * c;
        const __half* dd = (const __half*)p.W.p1 + (int64_t)row_global * nbk + ks * 4 + 2 * c;
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            float d = __half2float(dd[blk]);
            uint4 q0 = *reinterpret_cast<const uint4*>(qs + 32 * blk);
            uint4 q1 = *reinterpret_cast<const uint4*>(qs + 32 * blk + 16);
            uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                __half2 hv[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    uint32_t word = w[2 * i + (e >> 1)];
                    int b0 = (int)(int8_t)((word >> ((e & 1) * 16)) & 0xFF);
                    int b1 = (int)(int8_t)((word >> ((e & 1) * 16 + 8)) & 0xFF);
                    hv[e] = __floats2half2_rn(d * (float)b0, d * (float)b1);
                }
                *chunk_ptr(8 * c + 4 * blk + i) = *reinterpret_cast<uint4*>(hv);
            }
        }
    }
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(TC_THREADS, 1) qgemm_tc_kernel(TcParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int A_BYTES = TC_BM * TC_BK * 2;
    constexpr int B_BYTES = BN * TC_BK * 2;
    constexpr int A_LBO = TC_BM / 8 * 128, B_LBO = BN / 8 * 128;
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~(uintptr_t)127);
    uint8_t* a_base = smem;
    uint8_t* b_base = smem + STAGES * A_BYTES;
    __shared__ uint64_t bars[STAGES];
    __shared__ uint32_t tmem_base_slot;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row0 = blockIdx.x * TC_BM;
    const int tok0 = blockIdx.y * BN;
    const int split = blockIdx.z;
    const int total_stages = p.K / TC_BK;
    const int s_begin = split * p.stages_per_split;
    const int s_end = min(total_stages, s_begin + p.stages_per_split);
    const int n_local = s_end - s_begin;

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < STAGES; ++i) mbar_init(&bars[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"((uint32_t)BN)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    // instruction descriptor: D = f32, A = B = f16, both K-major, N = BN, M = 128
    const uint32_t idesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
    bool gave_up = false;
    const int a_row = tid & 127, a_c = tid >> 7;

    for (int it = 0; it < n_local; ++it) {
        const int st = it % STAGES, use = it / STAGES;
        const int ks = s_begin + it;
        if (use > 0 && !gave_up) {
            if (!mbar_wait(&bars[st], (uint32_t)((use - 1) & 1), TC_SPIN_LIMIT)) {
                gave_up = true;
                atomicExch(p.status, 1);
            }
        }
        uint8_t* a_stage = a_base + st * A_BYTES;
        uint8_t* b_stage = b_base + st * B_BYTES;
        dequant_store_a(p, row0 + a_row, ks, a_c, a_stage, a_row);
        // activations: BN rows x 16 chunks of 8 halves
#pragma unroll
        for (int i = 0; i < BN * 16 / TC_THREADS; ++i) {
            int idx = tid + i * TC_THREADS;
            int n = idx % BN, chunk = idx / BN;
            int tok = tok0 + n;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (tok < p.T) v = *reinterpret_cast<const uint4*>(p.xh + (int64_t)tok * p.K + ks * TC_BK + chunk * 8);
            *reinterpret_cast<uint4*>(b_stage + chunk * B_LBO + (n >> 3) * 128 + (n & 7) * 16) = v;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t a_addr = smem_u32(a_stage), b_addr = smem_u32(b_stage);
#pragma unroll
            for (int k = 0; k < TC_BK / 16; ++k) {
                uint64_t adesc = make_smem_desc(a_addr + k * 2 * A_LBO, A_LBO, 128);
                uint64_t bdesc = make_smem_desc(b_addr + k * 2 * B_LBO, B_LBO, 128);
                umma_f16(tmem_base, adesc, bdesc, idesc, (it > 0 || k > 0) ? 1u : 0u);
            }
            umma_commit(&bars[st]);
        }
    }

    // all MMAs of this CTA complete when the last commit arrives
    if (n_local > 0 && !gave_up) {
        int last = n_local - 1;
        if (!mbar_wait(&bars[last % STAGES], (uint32_t)((last / STAGES) & 1), TC_SPIN_LIMIT)) {
            gave_up = true;
            atomicExch(p.status, 2);
        }
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    if (n_local > 0) {
        const int quad = warp & 3, chalf = warp >> 2;
        const int row = row0 + quad * 32 + lane;
        float* dst = p.splits > 1 ? p.partial + (int64_t)split * p.T * p.out : p.y;
        const int ld = p.splits > 1 ? p.out : p.ldy;
#pragma unroll
        for (int cb = 0; cb < BN / 2; cb += 16) {
            int col = chalf * (BN / 2) + cb;
            uint32_t r[16];
            tmem_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)col, r);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (row < p.out) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    int tok = tok0 + col + i;
                    if (tok < p.T) {
                        float v = __uint_as_float(r[i]);
                        if (p.splits == 1) {
                            v *= p.out_scale;
                            if (p.softcap != 0.f) v = tanhf(v * (1.0f / p.softcap)) * p.softcap;
                        }
                        dst[(int64_t)tok * ld + row] = v;
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN) : "memory");
    }
}

__global__ void splitk_reduce_kernel(const float* partial, int splits, int64_t n, int out, float* y, int ldy, float out_scale,
                                     float softcap) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += partial[(int64_t)s * n + i];
    acc *= out_scale;
    if (softcap != 0.f) acc = tanhf(acc * (1.0f / softcap)) * softcap;
    int64_t t = i / out, c = i - t * out;
    y[t * ldy + c] = acc;
}

struct TcPlan {
    int bn, stages, row_tiles, n_tiles, splits, stages_per_split;
    size_t smem;
};

TcPlan make_plan(const QWeight& W, int T) {
    TcPlan pl;
    pl.bn = T <= 32 ? 32 : (T <= 64 ? 64 : 128);
    pl.stages = pl.bn <= 64 ? 4 : 3;
    pl.row_tiles = (int)((W.rows + TC_BM - 1) / TC_BM);
    pl.n_tiles = (T + pl.bn - 1) / pl.bn;
    int total_stages = (int)(W.cols / TC_BK);
    int tiles = pl.row_tiles * pl.n_tiles;
    int want = (148 + tiles - 1) / tiles;
    int max_splits = total_stages / 2 > 0 ? total_stages / 2 : 1;
    pl.splits = want < 1 ? 1 : (want > max_splits ? max_splits : want);
    pl.stages_per_split = (total_stages + pl.splits - 1) / pl.splits;
    pl.splits = (total_stages + pl.stages_per_split - 1) / pl.stages_per_split;
    pl.smem = (size_t)pl.stages * (TC_BM * TC_BK * 2 + pl.bn * TC_BK * 2) + 256;
    return pl;
}

template <int BN, int STAGES>
void launch_variant(const TcParams& p, const TcPlan& pl, cudaStream_t s) {
    ensure_dynamic_smem(reinterpret_cast<const void*>(&qgemm_tc_kernel<BN, STAGES>), pl.smem);
    dim3 grid((unsigned)pl.row_tiles, (unsigned)pl.n_tiles, (unsigned)pl.splits);
    qgemm_tc_kernel<BN, STAGES><<<grid, TC_THREADS, pl.smem, s>>>(p);
    MK_LAUNCH_CHECK();
}

}  // namespace

bool qgemm_tc_preferred(const QWeight& W, int T) {
    if (W.type != QT_Q4_K && W.type != QT_Q6_K && W.type != QT_Q8_0) return false;
    if (W.cols % 256 != 0) return false;
    return T > 8;
}

size_t qgemm_tc_partial_floats(const QWeight& W, int T) {
    TcPlan pl = make_plan(W, T);
    return pl.splits > 1 ? (size_t)pl.splits * T * W.rows : 0;
}

void launch_qgemm_tc_scratch(const QWeight& W, const ActQ& x, int T, float* y, int ldy, float out_scale, float softcap,
                             float* partial, int32_t* status, cudaStream_t s) {
    if (T <= 0) return;
    if (x.xh == nullptr) throw std::runtime_error("launch_qgemm_tc: f16 activations missing");
    if (W.cols % 256 != 0) throw std::runtime_error("launch_qgemm_tc: K must be a multiple of 256");
    TcPlan pl = make_plan(W, T);
    TcParams p;
    p.W = W;
    p.xh = x.xh;
    p.T = T;
    p.K = (int)W.cols;
    p.out = (int)W.rows;
    p.y = y;
    p.ldy = ldy;
    p.partial = partial;
    p.splits = pl.splits;
    p.stages_per_split = pl.stages_per_split;
    p.out_scale = out_scale;
    p.softcap = softcap;
    p.status = status;
    if (pl.bn == 32) launch_variant<32, 4>(p, pl, s);
    else if (pl.bn == 64) launch_variant<64, 4>(p, pl, s);
    else launch_variant<128, 3>(p, pl, s);
    if (pl.splits > 1) {
        int64_t n = (int64_t)T * W.rows;
        splitk_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(partial, pl.splits, n, (int)W.rows, y, ldy, out_scale,
                                                                          softcap);
        MK_LAUNCH_CHECK();
    }
}

void launch_qgemm_tc(const QWeight& W, const ActQ& x, int act_kind, int T, float* y, int ldy, float out_scale, float softcap,
                     QgemmWorkspace& ws, cudaStream_t s) {
    (void)act_kind;
    size_t need = qgemm_tc_partial_floats(W, T);
    ws.partial.ensure(need * sizeof(float));
    if (ws.status.size() == 0) {
        ws.status.alloc(sizeof(int32_t));
        ws.status.zero(s);
    }
    launch_qgemm_tc_scratch(W, x, T, y, ldy, out_scale, softcap, ws.partial.as<float>(), ws.status.as<int32_t>(), s);
}

}  // namespace mk
