// Narrow-batch matmul for decode ticks: y[t][n] = sum_k xh[t][k] * dequant(W)[n][k] with W in GGUF Q4_K blocks,
// read from HBM exactly once per call.
//
// Replaces LinearOp::Quantized forward (src/model_weights.rs:346-377 of the reference) when at most 64 activation
// rows share a matrix - the decode tick of a continuous batch, where the matmuls are bound by the bytes of the
// weights.  Keeping the weights in their 4.5-bit block format makes those bytes 3.5x fewer than an f16 image.
//
// The work is cut into (128-row tile, 256-column block) units, shared out evenly over at most one persistent CTA per
// SM; a CTA's contiguous range of units usually covers the tail of one row tile, some whole row tiles and the head
// of another.  608 threads in five roles:
//   warp 0      - one lane streams the raw blocks of the units (18 KiB bulk copies) into a four-deep ring;
//   warp 2      - one lane loads the matching 256 columns of the f16 activations (four 64-column TMA boxes,
//                 128-byte swizzle) plus their per-group sums into a two-deep ring;
//   warps 3-10  - two threads per weight row turn the nibbles of the block, 128 columns at a time, into one of two
//                 f16 operand slots in the K-major no-swizzle core-matrix layout (8 rows x 16 bytes) - as the exact
//                 integers sc * q - and the eight group minimums into a small second operand;
//   warp 1      - one lane issues, per unit, sixteen K = 16 tcgen05 MMAs of sc * q against the activations and one of
//                 the minimums against the activation group sums, into two of four accumulators in tensor memory
//                 (M = 128 rows, N = BN tokens), and commits slots, stages and accumulators back to their producers;
//   warps 11-18 - per unit, read both accumulators (one TMEM lane quadrant and one half of the token columns each) and add d * main - dmin * minimums (d and dmin are f16 in the
//                 file, the arithmetic here is f32) to running sums in registers; at the end of the CTA's piece of a
//                 row tile they store the sums - to the result when every row tile has one piece, else to that
//                 piece's slot of the partial-sum scratch, whose slots the consumer kernel adds in slot order.
// No weight is ever rounded: the only rounding left is the f16 image of the activations.
// Every mbarrier wait is bounded; a wait that gives up records a status word and the role leaves its loop.
#include "qstream_tc.h"
#include "hgemm_tc.h"
#include "kernels.h"
#include <cuda.h>
#include <algorithm>

namespace mk {

namespace {

constexpr int QS_BM = 128;
constexpr int QS_THREADS = 608;  // weight loader, MMA, activation loader warps; eight converting, eight epilogue warps
constexpr int QS_RAW_STAGES = 4;  // weight blocks in flight (HBM latency)
constexpr int QS_X_STAGES = 2;    // activation blocks in flight (L2 latency)
constexpr int QS_RAW_BYTES = QS_BM * 144;         // one block column of 128 rows
constexpr int QS_A_SLOT_BYTES = QS_BM * 128 * 2;  // 128 rows x 128 columns f16
constexpr int QS_A_LBO = QS_BM / 8 * 128;         // bytes between consecutive 16-byte K chunks
constexpr uint32_t QS_SPIN_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
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
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const void* tmap, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
// One contiguous run of bytes (a multiple of 16, both ends 16-byte aligned) into this CTA's shared memory.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// K-major, no swizzle: core matrices of 8 rows x 16 bytes; lbo = bytes between K chunks, sbo = between 8-row groups.
__device__ __forceinline__ uint64_t make_nosw_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}
// K-major, 128-byte rows, 128-byte swizzle: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_sw128_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
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
template <int N>
__device__ __forceinline__ void tmem_ld_n(uint32_t taddr, uint32_t (&r)[N]);
template <>
__device__ __forceinline__ void tmem_ld_n<16>(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld16(taddr, r); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]);
template <>
__device__ __forceinline__ void tmem_ld_n<32>(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld32(taddr, r); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

// ---- Q4_K block -> tensor-core operands -----------------------------------------------------------------------
// A 256-wide block of row n is d * (sc_g * q) - dmin * m_g over its eight groups g of 32.  sc_g * q is an integer
// below 1024 and m_g one below 64: both are exact in f16.  So the MMA multiplies the activations by sc_g * q (main
// accumulator) and the per-group sums of the activations by m_g (second accumulator); d and dmin, which are f16 in
// the file, scale the two accumulators in f32 once per block.  No weight is ever rounded.

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
// Four nibbles in the low halves of four bytes -> (1024 + q) as f16 by byte permutation, then
// fma(1024 + q, sc, -1024 sc) = sc * q: the product is exact and the result has at most 10 bits.
__device__ __forceinline__ void nibbles_times_scale(uint32_t bytes, __half2 sc, __half2 nbias, uint32_t& o01, uint32_t& o23) {
    uint32_t p01 = __byte_perm(bytes, 0x64646464u, 0x4140);
    uint32_t p23 = __byte_perm(bytes, 0x64646464u, 0x4342);
    __half2 h01 = __hfma2(*reinterpret_cast<__half2*>(&p01), sc, nbias);
    __half2 h23 = __hfma2(*reinterpret_cast<__half2*>(&p23), sc, nbias);
    o01 = *reinterpret_cast<uint32_t*>(&h01);
    o23 = *reinterpret_cast<uint32_t*>(&h23);
}

// Row `row` of the stage, columns [128 * half + 64 * c, + 64) of its 256-wide block, into operand slot `a_slot`.
__device__ __forceinline__ void convert_chunk(const uint8_t* blk, int row, int half, int c, uint8_t* a_slot) {
    const uint4 hdr = *reinterpret_cast<const uint4*>(blk);
    uint8_t* dst_row = a_slot + (row >> 3) * 128 + (row & 7) * 16;
    const int j = half * 2 + c;  // 64-column chunk of the block: low nibbles = group 2j, high nibbles = 2j + 1
    const uint4 q0 = *reinterpret_cast<const uint4*>(blk + 16 + 32 * j);
    const uint4 q1 = *reinterpret_cast<const uint4*>(blk + 16 + 32 * j + 16);
    int sc0, m0, sc1, m1;
    q4k_scale_min_reg(hdr.y, hdr.z, hdr.w, 2 * j, sc0, m0);
    q4k_scale_min_reg(hdr.y, hdr.z, hdr.w, 2 * j + 1, sc1, m1);
    const __half2 s0 = __float2half2_rn((float)sc0), s1 = __float2half2_rn((float)sc1);
    const __half2 nb0 = __float2half2_rn(-1024.f * (float)sc0), nb1 = __float2half2_rn(-1024.f * (float)sc1);
    const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint4 lo, hi;
        nibbles_times_scale(words[2 * i] & 0x0F0F0F0Fu, s0, nb0, lo.x, lo.y);
        nibbles_times_scale(words[2 * i + 1] & 0x0F0F0F0Fu, s0, nb0, lo.z, lo.w);
        nibbles_times_scale((words[2 * i] >> 4) & 0x0F0F0F0Fu, s1, nb1, hi.x, hi.y);
        nibbles_times_scale((words[2 * i + 1] >> 4) & 0x0F0F0F0Fu, s1, nb1, hi.z, hi.w);
        *reinterpret_cast<uint4*>(dst_row + (8 * c + i) * QS_A_LBO) = lo;
        *reinterpret_cast<uint4*>(dst_row + (8 * c + 4 + i) * QS_A_LBO) = hi;
    }
}

// The eight group minimums of the block as f16, twice (once for the head, once for the tail of the activation sums),
// and d, dmin as f32 for the epilogue.
__device__ __forceinline__ void write_mins(const uint8_t* blk, int row, uint8_t* extra, float2* dd) {
    const uint4 hdr = *reinterpret_cast<const uint4*>(blk);
    __half m[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        int sc, mn;
        q4k_scale_min_reg(hdr.y, hdr.z, hdr.w, g, sc, mn);
        m[g] = __float2half_rn((float)mn);
    }
    uint8_t* dst = extra + (row >> 3) * 128 + (row & 7) * 16;
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<uint4*>(m);
    *reinterpret_cast<uint4*>(dst + QS_A_LBO) = *reinterpret_cast<uint4*>(m);
    dd[row] = make_float2(__half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFF))),
                          __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16))));
}

struct QsParams {
    int T, rows, n_blocks;        // n_blocks = cols / 256
    float* y;
    int ldy;
    int row_tiles;
    int units;                    // row_tiles * n_blocks (row tile, block) units, shared out evenly over the CTAs
    int slots;                    // most pieces any row tile is cut into; > 1: pieces go to partial[slot][T][rows]
    float* partial;
    int32_t* status;
};

template <int BN>
struct QsSmem {
    static constexpr int X_BYTES = 4 * BN * 128 + 2 * BN * 16;   // four 64-column boxes + the group sums (head, tail)
    static constexpr int EXTRA_BYTES = 2 * QS_BM * 16;           // the group minimums, twice
    static constexpr size_t TOTAL = (size_t)QS_RAW_STAGES * QS_RAW_BYTES + (size_t)QS_X_STAGES * X_BYTES + 2 * QS_A_SLOT_BYTES +
                                    2 * EXTRA_BYTES + 4 * QS_BM * sizeof(float2) + 1024 + 256;
};

template <int BN>
__global__ void __launch_bounds__(QS_THREADS, 1)
qstream_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                  const __grid_constant__ CUtensorMap tm_gs, QsParams p) {
    using L = QsSmem<BN>;
    extern __shared__ uint8_t qs_smem_raw[];
    uint8_t* raw_ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(qs_smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* x_ring = raw_ring + (size_t)QS_RAW_STAGES * QS_RAW_BYTES;
    uint8_t* a_slots = x_ring + (size_t)QS_X_STAGES * L::X_BYTES;
    uint8_t* extras = a_slots + 2 * QS_A_SLOT_BYTES;
    float2* dd = reinterpret_cast<float2*>(extras + 2 * L::EXTRA_BYTES);  // [4][128] (d, dmin)
    uint64_t* bars = reinterpret_cast<uint64_t*>(dd + 4 * QS_BM);
    uint64_t* raw_full = bars;                              // [RAW] loader -> converters
    uint64_t* raw_empty = raw_full + QS_RAW_STAGES;         // [RAW] converters -> loader
    uint64_t* x_full = raw_empty + QS_RAW_STAGES;           // [X]   loader -> MMA
    uint64_t* x_empty = x_full + QS_X_STAGES;               // [X]   MMA -> loader
    uint64_t* a_full = x_empty + QS_X_STAGES;               // [2]   converters -> MMA
    uint64_t* a_empty = a_full + 2;                         // [2]   MMA -> converters
    uint64_t* acc_full = a_empty + 2;                       // [2]   MMA -> epilogue
    uint64_t* acc_empty = acc_full + 2;                     // [2]   epilogue -> MMA
    __shared__ uint32_t tmem_base_slot;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // this CTA's share of the units: a contiguous range, usually the tail of one row tile, some whole row tiles and
    // the head of another; a "piece" is the part of a row tile one CTA covers
    const int u0 = (int)((int64_t)blockIdx.x * p.units / gridDim.x), u1 = (int)((int64_t)(blockIdx.x + 1) * p.units / gridDim.x);
    const int n_local = u1 - u0;
    auto cta_of_unit = [&](int u) {
        int c = (int)((int64_t)u * gridDim.x / p.units);
        while ((int64_t)(c + 1) * p.units / gridDim.x <= u) ++c;
        while ((int64_t)c * p.units / gridDim.x > u) --c;
        return c;
    };
    constexpr uint32_t TMEM_COLS = 4 * BN;  // two sets of (main, minimums) accumulators

    if (threadIdx.x == 0) {
        for (int i = 0; i < QS_RAW_STAGES; ++i) {
            mbar_init(&raw_full[i], 1);
            mbar_init(&raw_empty[i], 8);   // one arrival per converting warp
        }
        for (int i = 0; i < QS_X_STAGES; ++i) {
            mbar_init(&x_full[i], 1);
            mbar_init(&x_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&a_full[i], 8);
            mbar_init(&a_empty[i], 1);
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], 8);   // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;
    // Everything above is private to the CTA.  The weights do not depend on the predecessor kernel either, so the
    // loader fills the weight ring first and only then waits for the predecessor, whose output (the activations) it
    // loads next.  Every other access to global memory of this kernel (the epilogue's stores) is ordered after
    // those loads through the mbarriers.
    pdl_trigger();

    if (warp == 0) {
        // ---- weight loader: the weights depend on no predecessor kernel, so this lane never waits for one
        if (lane == 0) {
            for (int i = 0; i < n_local; ++i) {
                const uint32_t st = i % QS_RAW_STAGES, ph = (i / QS_RAW_STAGES) & 1;
                if (!mbar_wait(&raw_empty[st], ph ^ 1, QS_SPIN_LIMIT)) { atomicExch(p.status, 22); break; }
                mbar_expect_tx(&raw_full[st], (uint32_t)QS_RAW_BYTES);
                // units are stored one after the other, 18 KiB each: fetched as one box of 144 full 128-byte lines
                tma_load_2d(raw_ring + (size_t)st * QS_RAW_BYTES, &tm_w, 0, (u0 + i) * (QS_RAW_BYTES / 128), &raw_full[st]);
            }
        }
    } else if (warp == 2) {
        // ---- activation loader (its own warp, so that a full activation ring never holds back the weight stream)
        if (lane == 0) {
            pdl_wait();
            for (int i = 0; i < n_local; ++i) {
                const uint32_t st = i % QS_X_STAGES, ph = (i / QS_X_STAGES) & 1;
                if (!mbar_wait(&x_empty[st], ph ^ 1, QS_SPIN_LIMIT)) { atomicExch(p.status, 21); break; }
                uint8_t* xb = x_ring + (size_t)st * L::X_BYTES;
                const int blk = (u0 + i) % p.n_blocks;
                mbar_expect_tx(&x_full[st], (uint32_t)L::X_BYTES);
#pragma unroll
                for (int q = 0; q < 4; ++q) tma_load_2d(xb + q * BN * 128, &tm_x, blk * 256 + q * 64, 0, &x_full[st]);
                tma_load_2d(xb + 4 * BN * 128, &tm_gs, blk * 8, 0, &x_full[st]);
                tma_load_2d(xb + 4 * BN * 128 + BN * 16, &tm_gs, p.n_blocks * 8 + blk * 8, 0, &x_full[st]);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(QS_BM >> 4) << 24);
            // every descriptor this lane will ever need, built once: the issue loop below is a single thread's
            // dependent instruction stream, and anything computed per MMA there delays the tensor cores
            uint64_t a_desc[2], e_adesc[2], b_desc[QS_X_STAGES][4], e_bdesc[QS_X_STAGES];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                a_desc[h] = make_nosw_desc(smem_u32(a_slots + h * QS_A_SLOT_BYTES), QS_A_LBO, 128);
                e_adesc[h] = make_nosw_desc(smem_u32(extras + h * L::EXTRA_BYTES), QS_A_LBO, 128);
            }
#pragma unroll
            for (int xs = 0; xs < QS_X_STAGES; ++xs) {
                const uint32_t xb_addr = smem_u32(x_ring + (size_t)xs * L::X_BYTES);
#pragma unroll
                for (int q = 0; q < 4; ++q) b_desc[xs][q] = make_sw128_desc(xb_addr + q * BN * 128);
                e_bdesc[xs] = make_nosw_desc(xb_addr + 4 * BN * 128, BN * 16, 128);
            }
            constexpr uint64_t A_K_STEP = (2 * QS_A_LBO) >> 4;  // two 16-byte K chunks further, in descriptor units
            bool ok = true;
            for (int i = 0; i < n_local && ok; ++i) {
                const uint32_t set = i & 1, aph = (i >> 1) & 1;
                const uint32_t xs = i % QS_X_STAGES, xph = (i / QS_X_STAGES) & 1;
                if (!mbar_wait(&acc_empty[set], aph ^ 1, QS_SPIN_LIMIT)) { atomicExch(p.status, 23); break; }
                if (!mbar_wait(&x_full[xs], xph, QS_SPIN_LIMIT)) { atomicExch(p.status, 24); break; }
                const uint32_t d_main = tmem_base + set * 2 * BN, d_mins = d_main + BN;
                for (int half = 0; half < 2; ++half) {
                    if (!mbar_wait(&a_full[half], (uint32_t)(i & 1), QS_SPIN_LIMIT)) { atomicExch(p.status, 25); ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                    for (int k = 0; k < 8; ++k)
                        umma_f16(d_main, a_desc[half] + A_K_STEP * k, b_desc[xs][half * 2 + (k >> 2)] + (uint64_t)(2 * (k & 3)), idesc,
                                 (half > 0 || k > 0) ? 1u : 0u);
                    // the group minimums against the group sums of the activations (head and tail): one K = 16 step
                    if (half == 0) umma_f16(d_mins, e_adesc[i & 1], e_bdesc[xs], idesc, 0u);
                    umma_commit(&a_empty[half]);
                }
                if (ok) {
                    umma_commit(&x_empty[xs]);
                    umma_commit(&acc_full[set]);
                }
            }
        }
    } else if (warp < 11) {
        // ---- converters (warps 3-10): two threads per weight row of the tile, 64 columns each per half block
        const int r = ((int)threadIdx.x - 96) & 127, csel = ((int)threadIdx.x - 96) >> 7;
        bool ok = true;
        for (int i = 0; i < n_local && ok; ++i) {
            const uint32_t st = i % QS_RAW_STAGES, ph = (i / QS_RAW_STAGES) & 1;
            if (!mbar_wait(&raw_full[st], ph, QS_SPIN_LIMIT)) {
                if (lane == 0) atomicExch(p.status, 26);
                break;
            }
            const uint8_t* blk = raw_ring + (size_t)st * QS_RAW_BYTES + r * 144;
            for (int half = 0; half < 2; ++half) {
                if (!mbar_wait(&a_empty[half], (uint32_t)((i & 1) ^ 1), QS_SPIN_LIMIT)) {
                    if (lane == 0) atomicExch(p.status, 27);
                    ok = false;
                    break;
                }
                convert_chunk(blk, r, half, csel, a_slots + half * QS_A_SLOT_BYTES);
                if (half == 0 && csel == 0) write_mins(blk, r, extras + (i & 1) * L::EXTRA_BYTES, dd + (i & 3) * QS_BM);
                // every lane makes its stores visible to the async proxy, then one lane arrives for the warp
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&a_full[half]);
            }
            if (ok) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&raw_empty[st]);
            }
        }
    } else {
        // ---- epilogue warps 11-18: warp w reads TMEM lanes 32 (w % 4) .. + 31 (weight rows) and one half of the
        // token columns; per block, y += d * main - dmin * minimums, running sums in registers
        constexpr int HN = BN / 2;  // token columns per warp
        const int quad = warp & 3, chalf = (warp - 11) >> 2;
        const int row_in_tile = quad * 32 + lane;
        float acc[HN];
#pragma unroll
        for (int t = 0; t < HN; ++t) acc[t] = 0.f;
        bool ok = true;
        for (int i = 0; i < n_local; ++i) {
            const uint32_t set = i & 1, aph = (i >> 1) & 1;
            if (!mbar_wait(&acc_full[set], aph, QS_SPIN_LIMIT)) {
                if (lane == 0) atomicExch(p.status, 28);
                ok = false;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float2 dm = dd[(i & 3) * QS_BM + row_in_tile];
            const uint32_t t_main = tmem_base + ((uint32_t)(quad * 32) << 16) + set * 2 * BN + chalf * HN;
            {
                uint32_t vm[HN], vn[HN];
                tmem_ld_n<HN>(t_main, vm);
                tmem_ld_n<HN>(t_main + BN, vn);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int t = 0; t < HN; ++t)
                    acc[t] = __fmaf_rn(-dm.y, __uint_as_float(vn[t]), __fmaf_rn(dm.x, __uint_as_float(vm[t]), acc[t]));
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[set]);
            // end of this CTA's piece of the row tile: store it and start the next piece from zero
            const int u = u0 + i, tile = u / p.n_blocks;
            if (i + 1 == n_local || (u + 1) / p.n_blocks != tile) {
                const int row = tile * QS_BM + row_in_tile;
                const int t0 = chalf * HN;
                if (p.slots == 1) {
                    if (row < p.rows) {
#pragma unroll
                        for (int t = 0; t < HN; ++t)
                            if (t0 + t < p.T) p.y[(int64_t)(t0 + t) * p.ldy + row] = acc[t];
                    }
                } else {
                    const int first = cta_of_unit(tile * p.n_blocks);
                    const int64_t slot_stride = (int64_t)p.T * p.rows;
                    float* dst = p.partial + (int64_t)((int)blockIdx.x - first) * slot_stride;
                    const bool last_piece = u + 1 == (tile + 1) * p.n_blocks;
                    if (row < p.rows) {
#pragma unroll
                        for (int t = 0; t < HN; ++t)
                            if (t0 + t < p.T) dst[(int64_t)(t0 + t) * p.rows + row] = acc[t];
                        if (last_piece) {  // the slots this row tile does not use read as zero
                            for (int sl = (int)blockIdx.x - first + 1; sl < p.slots; ++sl)
                                for (int t = t0; t < min(p.T, t0 + HN); ++t) p.partial[sl * slot_stride + (int64_t)t * p.rows + row] = 0.f;
                        }
                    }
                }
#pragma unroll
                for (int t = 0; t < HN; ++t) acc[t] = 0.f;
            }
        }
        (void)ok;
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// Row-major Q4_K blocks [rows][nb][144 bytes] -> unit-major [row tile][block][128 rows][144 bytes], rows past the end
// zero (a zero block dequantises to zero).  16 bytes per thread.
__global__ void retile_q4k_kernel(const uint4* src, int64_t rows, int nb, uint4* dst, int64_t chunks) {
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= chunks) return;
    const int64_t unit = c / (QS_RAW_BYTES / 16);
    const int in_unit = (int)(c - unit * (QS_RAW_BYTES / 16));
    const int r = in_unit / 9, part = in_unit - r * 9;  // 144 bytes = 9 chunks
    const int64_t tile = unit / nb, blk = unit - tile * nb;
    const int64_t row = tile * QS_BM + r;
    dst[c] = row < rows ? src[(row * nb + blk) * 9 + part] : make_uint4(0, 0, 0, 0);
}

template <int BN>
void launch_qs(const CUtensorMap& tw, const CUtensorMap& tx, const CUtensorMap& tg, const QsParams& p, int ctas, cudaStream_t s) {
    constexpr size_t smem = QsSmem<BN>::TOTAL;
    static bool configured = false;
    if (!configured) {
        MK_CUDA(cudaFuncSetAttribute(qstream_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    launch_pdl(qstream_tc_kernel<BN>, dim3(ctas), dim3(QS_THREADS), smem, s, tw, tx, tg, p);
    MK_LAUNCH_CHECK();
}

}  // namespace

void build_qstream_weight(const void* q4k_blocks, int64_t rows, int64_t cols, QStreamWeight& out, cudaStream_t s) {
    if (cols <= 0 || cols % 256 != 0 || rows <= 0) throw std::runtime_error("build_qstream_weight: cols must be a positive multiple of 256");
    out.rows = rows;
    out.cols = cols;
    const int nb = (int)(cols / 256);
    const int64_t row_tiles = (rows + QS_BM - 1) / QS_BM;
    out.tiled.alloc((size_t)row_tiles * nb * QS_RAW_BYTES);
    const int64_t chunks = row_tiles * nb * (QS_RAW_BYTES / 16);
    retile_q4k_kernel<<<(unsigned)((chunks + 255) / 256), 256, 0, s>>>(reinterpret_cast<const uint4*>(q4k_blocks), rows, nb,
                                                                        out.tiled.as<uint4>(), chunks);
    MK_LAUNCH_CHECK();
    // the unit-major copy seen as rows of 128 bytes: one unit = one box of 144 rows
    encode_tma_2d(out.tmap, true, out.tiled.ptr(), 128, (uint64_t)row_tiles * nb * (QS_RAW_BYTES / 128), 128, 128, QS_RAW_BYTES / 128, false);
    out.ready = true;
}

QStreamPlan qstream_plan(int64_t rows, int64_t cols, int T, int max_splits) {
    QStreamPlan pl;
    pl.bn = T <= 32 ? 32 : 64;
    pl.row_tiles = (int)((rows + QS_BM - 1) / QS_BM);
    const int nb = (int)(cols / 256);
    pl.units = pl.row_tiles * nb;
    const int sms = 148;
    auto pieces = [&](int ctas) {  // most CTAs any row tile is spread over
        int worst = 1;
        auto cta_of = [&](int64_t u) {
            int64_t c = u * ctas / pl.units;
            while ((c + 1) * pl.units / ctas <= u) ++c;
            while (c * pl.units / ctas > u) --c;
            return (int)c;
        };
        for (int t = 0; t < pl.row_tiles; ++t) worst = std::max(worst, cta_of((int64_t)t * nb + nb - 1) - cta_of((int64_t)t * nb) + 1);
        return worst;
    };
    if (max_splits <= 1) {
        pl.ctas = pl.row_tiles;  // whole row tiles only: the result is complete in y
        pl.slots = 1;
    } else {
        // as many CTAs as there are SMs, at least two blocks each; fewer while a row tile would be cut into more
        // pieces than the consumer may add or the pieces would not fit in 16 MiB
        int ctas = std::max(1, std::min(sms, pl.units));
        while (ctas > 1) {
            int s = pieces(ctas);
            if (s <= std::min(max_splits, 16) && (size_t)s * T * rows * 4 <= ((size_t)16 << 20)) break;
            ctas = ctas * 3 / 4;
        }
        pl.ctas = ctas;
        pl.slots = pieces(ctas);
    }
    pl.partial_floats = pl.slots > 1 ? (size_t)pl.slots * T * rows : 0;
    return pl;
}

int launch_qstream_tc(const QStreamWeight& W, const __half* xh, const __half* gs, int T, float* y, int ldy, float* partial,
                      size_t partial_floats, int32_t* status, cudaStream_t s, int max_splits) {
    if (T <= 0) return 1;
    if (!W.ready) throw std::runtime_error("launch_qstream_tc: the matrix descriptor was not built");
    if (T > kQStreamMaxRows) throw std::runtime_error("launch_qstream_tc: more activation rows than the kernel covers");
    if (xh == nullptr || gs == nullptr) throw std::runtime_error("launch_qstream_tc: f16 activations or their group sums missing");
    if (partial == nullptr) max_splits = 1;
    QStreamPlan pl = qstream_plan(W.rows, W.cols, T, max_splits);
    if (pl.slots > 1 && pl.partial_floats > partial_floats) pl = qstream_plan(W.rows, W.cols, T, 1);
    alignas(64) CUtensorMap tx;
    encode_tma_2d(&tx, false, xh, (uint64_t)W.cols, (uint64_t)T, (uint64_t)W.cols * 2, 64, (uint32_t)pl.bn, true);
    // group sums [T][2 * cols/32] f16: boxes of 8 halves (the eight groups of one block) x BN rows land as one
    // 16-byte K chunk of the no-swizzle operand layout
    alignas(64) CUtensorMap tg;
    encode_tma_2d(&tg, false, gs, (uint64_t)W.cols / 16, (uint64_t)T, (uint64_t)W.cols / 16 * 2, 8, (uint32_t)pl.bn, false);
    QsParams p;
    p.T = T;
    p.rows = (int)W.rows;
    p.n_blocks = (int)(W.cols / 256);
    p.y = y;
    p.ldy = ldy;
    p.row_tiles = pl.row_tiles;
    p.units = pl.units;
    p.slots = pl.slots;
    p.partial = partial;
    p.status = status;
    const CUtensorMap& tw = *reinterpret_cast<const CUtensorMap*>(W.tmap);
    if (pl.bn == 32) launch_qs<32>(tw, tx, tg, p, pl.ctas, s);
    else launch_qs<64>(tw, tx, tg, p, pl.ctas, s);
    return pl.slots;
}

}  // namespace mk
