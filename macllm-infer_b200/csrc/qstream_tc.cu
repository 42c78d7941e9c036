// Narrow-batch matmul for decode ticks: y[t][n] = sum_k xh[t][k] * dequant(W)[n][k] with W in GGUF Q4_K or Q6_K
// blocks, read from HBM exactly once per call and dequantised straight into tensor memory.
//
// Replaces LinearOp::Quantized forward (src/model_weights.rs:346-377 of the reference) when at most 64 activation
// rows share a matrix - the decode tick of a continuous batch, where the matmuls are bound by the bytes of the
// weights.  Keeping the weights in their 4.5 / 6.6-bit block format makes those bytes 3.5x / 2.4x fewer than an f16
// image.
//
// The matrix is cut into (128-row tile, 256-column block) units, stored one after the other so that a unit is one
// contiguous bulk copy.  R row tiles that follow one another form a group; an item is (group, block): the R units
// that multiply the same 256 activation columns.  Items are shared out evenly over at most one persistent CTA per
// SM; the part of a group one CTA covers is a piece.  864 threads in five roles:
//   warp 0       - streams the raw units into a ring of shared-memory stages (up to 8 x 18 KiB in flight; one elected
//                  lane issues, the warp walks the item list together so that ring counters stay warp-uniform); the
//                  weights depend on no predecessor kernel, so this role never waits for one;
//   warp 2       - loads the 256 columns of the f16 activations of an item (four 64-column TMA boxes, 128-byte swizzle)
//                  into a three-deep ring, once per item, whatever R is;
//   warps 3-18   - converters, two groups of eight warps: group i owns A buffer i and the units of parity i, so one
//                  group converts while the MMAs of the other group's buffer run.  Thread (row, 64-column chunk) turns
//                  its nibbles into f16 weights in registers, sixteen at a time, and writes them with tcgen05.st into the
//                  A operand buffer in TENSOR memory (row = TMEM lane, two weights per 32-bit column).  Shared memory
//                  carries the raw bytes only; the dequantised operand never touches it;
//   warp 1       - allocates tensor memory (overlapped with the first weight copies) and issues, per unit, sixteen
//                  K = 16 tcgen05.mma with A from tensor memory and B (the activations) from shared memory into the
//                  accumulator of the unit's row tile (M = 128, N = BN tokens, up to four accumulators), and commits
//                  buffers, stages and accumulators back;
//   warps 19-26  - at the end of a piece read its accumulators (each warp a lane quadrant and a column half) and store
//                  them: to the result when every group has one piece, else to that piece's slot of the partial-sum
//                  scratch, whose slots the consumer kernel adds in slot order; or, for an interleaved gate|up matrix,
//                  act(gate) * up as f16.
// Expert-grouped form (sparse-MoE layers): the matrix is a bank of experts, the activation rows are grouped by expert,
// and the row ranges live on the device (they come from the routing kernels of the same forward).  Warp 0 first builds
// this CTA's share of the job list - (expert, chunk of up to BN of its rows, group of row tiles) - from the ranges, with
// no host round trip; a job then runs like a whole group of the plain form.
// Q4_K arithmetic: sc * q (an integer below 1024) is formed exactly, then w = fma(sc * q, d, -f16(dmin * m)): the f16
// weight carries the rounding of the product and that of dmin * m.  Q6_K: w = (q - 32) * f16(d * sc).
// Every mbarrier wait is bounded; a wait that gives up records a status word and the role leaves its loop.
#include "qstream_tc.h"
#include "hgemm_tc.h"
#include "kernels.h"
#include <cuda.h>
#include <algorithm>

namespace mk {

namespace {

constexpr int QS_BM = 128;
constexpr int QS_CONV_WARPS = 16;
constexpr int QS_EPI_WARPS = 8;
constexpr int QS_THREADS = (3 + QS_CONV_WARPS + QS_EPI_WARPS) * 32;  // 864
constexpr int QS_MAX_STAGES = 8;
constexpr int QS_X_STAGES = 3;    // activation blocks in flight (L2 latency)
constexpr int QS_Q4K_UNIT = QS_BM * 144;                         // 18432
constexpr int QS_Q6K_UNIT = QS_BM * (128 + 64 + 16) + 256;       // 26880: ql, qh, scales planes + d (f16, padded)
constexpr int QS_ACC = 4;                                        // accumulators in tensor memory
constexpr uint32_t QS_SPIN_LIMIT = 1u << 22;
constexpr uint32_t QS_TMEM_COLS = 512;
constexpr uint32_t QS_A_COL0 = 256;                              // two A buffers of 128 columns
constexpr int QS_MAX_JOBS = 320;                                 // jobs one CTA can be handed in the expert-grouped form

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
// D[tmem] (+)= A[tmem] * B[smem]: A is M = 128 rows (lanes) x 16 f16 (8 columns), K-major.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
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
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
          "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
          "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// ---- Q4_K ------------------------------------------------------------------------------------------------------
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
// Four nibbles in the low halves of four bytes -> (1024 + q) as f16 by byte permutation; fma(1024 + q, sc, -1024 sc)
// = sc * q exactly (below 1024); then fma(sc * q, d, -dmin * m): the dequantised weight, rounded once.
__device__ __forceinline__ void nibbles_to_weights(uint32_t bytes, __half2 sc, __half2 nbias, __half2 d, __half2 nmin, uint32_t& o01,
                                                   uint32_t& o23) {
    uint32_t p01 = __byte_perm(bytes, 0x64646464u, 0x4140);
    uint32_t p23 = __byte_perm(bytes, 0x64646464u, 0x4342);
    __half2 h01 = __hfma2(__hfma2(*reinterpret_cast<__half2*>(&p01), sc, nbias), d, nmin);
    __half2 h23 = __hfma2(__hfma2(*reinterpret_cast<__half2*>(&p23), sc, nbias), d, nmin);
    o01 = *reinterpret_cast<uint32_t*>(&h01);
    o23 = *reinterpret_cast<uint32_t*>(&h23);
}
// Group G (32 weights, columns [32 G, 32 G + 32)) of a 256-wide block -> 32 f16 weights, two per register.  `blk` is
// the row's 144-byte block, `hdr` its first 16 bytes (d, dmin, the twelve scale bytes).  Groups 2J and 2J + 1 share the
// 32 bytes at 16 + 32 J: low nibbles / high nibbles.  G is a template argument so that the scale bytes are picked apart
// with constant shifts.
template <int G>
__device__ __forceinline__ void convert_q4k_group(const uint8_t* blk, const uint4& hdr, uint32_t (&out)[16]) {
    constexpr int J = G >> 1, SH = (G & 1) * 4;
    const uint4 q0 = *reinterpret_cast<const uint4*>(blk + 16 + 32 * J);
    const uint4 q1 = *reinterpret_cast<const uint4*>(blk + 16 + 32 * J + 16);
    int sc, m;
    q4k_scale_min_reg(hdr.y, hdr.z, hdr.w, G, sc, m);
    const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
    const __half2 d2 = __half2half2(__ushort_as_half((unsigned short)(hdr.x & 0xFFFF)));
    const __half2 s2 = __float2half2_rn((float)sc);
    const __half2 nb = __float2half2_rn(-1024.f * (float)sc);
    const __half2 nm = __float2half2_rn(-dmin * (float)m);
    const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) nibbles_to_weights((words[i] >> SH) & 0x0F0F0F0Fu, s2, nb, d2, nm, out[2 * i], out[2 * i + 1]);
}

// ---- Q6_K ------------------------------------------------------------------------------------------------------
// Unit layout: ql plane [128 rows][128 B], qh plane [128][64 B], scales plane [128][16 B], d [128] f16.  The 16-byte
// chunks of a row of the ql and qh planes are stored at chunk ^ (row & 7) / chunk ^ (row & 3) so that the 32 rows a
// warp reads at once fall into different banks.
constexpr int Q6_QL = 0, Q6_QH = QS_BM * 128, Q6_SC = Q6_QH + QS_BM * 64, Q6_D = Q6_SC + QS_BM * 16;
// Four 6-bit values (low nibbles in `lo4`, the two high bits in bits 0-1 of each byte of `hi2`) -> (q - 32) * s.
__device__ __forceinline__ void q6_to_weights(uint32_t lo4, uint32_t hi2, __half2 s, uint32_t& o01, uint32_t& o23) {
    const uint32_t q = lo4 | (hi2 << 4);
    uint32_t p01 = __byte_perm(q, 0x64646464u, 0x4140);
    uint32_t p23 = __byte_perm(q, 0x64646464u, 0x4342);
    const __half2 bias = __float2half2_rn(-1056.f);  // 1024 + q - 1056 = q - 32, exact
    __half2 h01 = __hmul2(__hadd2(*reinterpret_cast<__half2*>(&p01), bias), s);
    __half2 h23 = __hmul2(__hadd2(*reinterpret_cast<__half2*>(&p23), bias), s);
    o01 = *reinterpret_cast<uint32_t*>(&h01);
    o23 = *reinterpret_cast<uint32_t*>(&h23);
}
// Group G (32 weights, columns [32 G, 32 G + 32)) of the block: half n = G / 4 of the block, quarter qq = G % 4 of that
// half: weight l of the group comes from ql[64 n + 32 (qq & 1) + l] (low nibbles for qq < 2, high nibbles otherwise) with
// its two high bits in qh[32 n + l] at bit 2 qq; scales sc[8 n + 2 qq] for l < 16 and sc[8 n + 2 qq + 1] for l >= 16.
__device__ __forceinline__ void convert_q6k_group(const uint8_t* raw, int row, int G, uint32_t (&out)[16]) {
    const int n = G >> 2, qq = G & 3;
    const uint8_t* ql_row = raw + Q6_QL + row * 128;
    const uint8_t* qh_row = raw + Q6_QH + row * 64;
    const int8_t* sc = reinterpret_cast<const int8_t*>(raw + Q6_SC + row * 16) + 8 * n + 2 * qq;
    const float d = __half2float(*reinterpret_cast<const __half*>(raw + Q6_D + row * 2));
    const __half2 s0 = __float2half2_rn(d * (float)sc[0]), s1 = __float2half2_rn(d * (float)sc[1]);
    const int sh_lo = (qq >> 1) * 4, sh_hi = 2 * qq;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const uint4 a = *reinterpret_cast<const uint4*>(ql_row + (((4 * n + 2 * (qq & 1) + c) ^ (row & 7)) << 4));
        const uint4 h = *reinterpret_cast<const uint4*>(qh_row + (((2 * n + c) ^ (row & 3)) << 4));
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, hw[4] = {h.x, h.y, h.z, h.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
            q6_to_weights((aw[i] >> sh_lo) & 0x0F0F0F0Fu, (hw[i] >> sh_hi) & 0x03030303u, c == 0 ? s0 : s1, out[8 * c + 2 * i], out[8 * c + 2 * i + 1]);
    }
}

struct QsParams {
    int T, rows;                  // activation rows; weight rows (all segments)
    int n_blocks;                 // cols / 256
    int row_tiles, groups, R;     // R row tiles per group
    int items;                    // groups * n_blocks
    int whole_groups;             // 1: CTAs own whole groups (every result complete in one CTA)
    int slots;                    // most pieces any group is cut into; > 1: pieces go to partial[slot][T][rows]
    int tiles_a;                  // row tiles of the first segment (Q4_K); the rest are Q6_K
    int fmt_a, fmt_b;             // 0 = Q4_K, 1 = Q6_K
    int stage_bytes, n_stages;
    // expert-grouped form: the matrix is `experts` matrices of tiles_pe row tiles back to back; the activation rows
    // [offsets[e], offsets[e + 1]) belong to expert e and are multiplied by its matrix only.  A job is (expert, chunk of
    // BN rows, group of R row tiles); jobs are shared out evenly over the CTAs, whole jobs only.  rows = rows per expert.
    int grouped, experts, tiles_pe, groups_pe;
    const int32_t* offsets;
    int mode;                     // 0 plain, 1 gated (rows interleaved gate/up; writes f16 act(gate) * up)
    int act;                      // gated: 0 SiLU, 1 tanh GELU
    const uint8_t* w_a;           // units of segment a, then of segment b
    const uint8_t* w_b;
    float* y;
    int ldy;
    __half* yh;                   // gated output [T][rows / 2]
    int ldyh;
    float* partial;
    int32_t* status;
    long long* prof;              // optional [5][8]: cycles per role of CTA 0 (measuring aid)
    int dbg;                      // with prof only: 1 skip the conversion arithmetic, 2 skip the TMEM stores, 4 skip the MMAs
};

template <int BN>
struct QsSmem {
    static constexpr int X_BYTES = 4 * BN * 128;   // four 64-column boxes
};

__device__ __forceinline__ float act_fn(float g, int act) {
    if (act == 0) return g / (1.f + __expf(-g));
    const float c = 0.7978845608028654f;
    return 0.5f * g * (1.f + tanhf(c * (g + 0.044715f * g * g * g)));
}

// PROF: CTA 0 accumulates the cycles every role spends in each of its waits and in its whole loop, and stamps a
// timeline into shared memory (a measuring aid; the production instantiation carries none of it).
#define QS_WAIT(site, bar, parity) (PROF ? prof_wait(prof_acc[site], bar, parity) : mbar_wait(bar, parity, QS_SPIN_LIMIT))
__device__ __forceinline__ bool prof_wait(long long& acc, uint64_t* bar, uint32_t parity) {
    const long long t0 = clock64();
    const bool ok = mbar_wait(bar, parity, QS_SPIN_LIMIT);
    acc += clock64() - t0;
    return ok;
}
// One lane of a converged warp.  The roles that issue TMA copies and MMAs run their loops with the whole warp and
// elect a lane for the issue itself: addresses and descriptors then are warp-uniform values and live in uniform
// registers instead of being moved there one by one before every instruction.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xFFFFFFFF;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

// GROUPED is a template parameter so that the plain form carries none of the job-table lookups.
template <int BN, bool PROF, bool GROUPED>
__global__ void __launch_bounds__(QS_THREADS, 1)
qstream_tc_kernel(const __grid_constant__ CUtensorMap tm_x, QsParams p) {
    using L = QsSmem<BN>;
    long long prof_acc[4] = {0, 0, 0, 0};
    const long long prof_t0 = PROF ? clock64() : 0;
    __shared__ uint32_t tlog[PROF ? 5 : 1][PROF ? 400 : 1];
    int tcnt = 0;
#define QS_LOG(role, ev) do { if (PROF && blockIdx.x == 0 && (threadIdx.x & 31) == 0 && tcnt < 400) { \
        tlog[role][tcnt++] = ((uint32_t)(ev) << 28) | (uint32_t)((clock64() - prof_t0) & 0x0FFFFFFF); } } while (0)
    extern __shared__ uint8_t qs_smem_raw[];
    uint8_t* x_ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(qs_smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* raw_ring = x_ring + (size_t)QS_X_STAGES * L::X_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(raw_ring + (size_t)p.n_stages * p.stage_bytes);
    uint64_t* raw_full = bars;                              // [stages] loader -> converters
    uint64_t* raw_empty = raw_full + QS_MAX_STAGES;         // [stages] converters -> loader
    uint64_t* x_full = raw_empty + QS_MAX_STAGES;           // [X]   loader -> MMA
    uint64_t* x_empty = x_full + QS_X_STAGES;               // [X]   MMA -> loader
    uint64_t* a_full = x_empty + QS_X_STAGES;               // [2]   converters -> MMA
    uint64_t* a_empty = a_full + 2;                         // [2]   MMA -> converters
    uint64_t* acc_full = a_empty + 2;                       // [4]   MMA -> epilogue
    uint64_t* acc_empty = acc_full + QS_ACC;                // [4]   epilogue -> MMA
    uint64_t* tmem_ready = acc_empty + QS_ACC;              // [1]   allocating warp -> everyone
    __shared__ uint32_t tmem_base_slot;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int C = (int)gridDim.x, c = (int)blockIdx.x;
    const int R = p.R, nb = p.n_blocks;
    // expert-grouped form: this CTA's jobs, looked up by the roles as "group" g = 0, 1, ...
    constexpr int JOBS = GROUPED ? QS_MAX_JOBS : 1;
    __shared__ int16_t job_expert[JOBS], job_rows[JOBS], job_group[JOBS];
    __shared__ int32_t job_row0[JOBS];
    __shared__ int32_t job_range[2];
    if (GROUPED) {
        // the row ranges come from the routing kernels: nothing of this launch can start before they are final
        pdl_wait();
        if (warp == 0) {
            // jobs of expert e: ceil(rows_e / BN) chunks x groups_pe; two passes over the experts, 32 at a time: the
            // total first, then the entries of this CTA's share
            int total = 0;
            for (int base = 0; base < p.experts; base += 32) {
                const int e = base + lane;
                int cnt = e < p.experts ? (p.offsets[e + 1] - p.offsets[e] + BN - 1) / BN * p.groups_pe : 0;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
                total += cnt;
            }
            const int j0 = (int)((int64_t)c * total / C), j1 = (int)((int64_t)(c + 1) * total / C);
            int running = 0;
            for (int base = 0; base < p.experts; base += 32) {
                const int e = base + lane;
                const int n_e = e < p.experts ? p.offsets[e + 1] - p.offsets[e] : 0;
                const int cnt = (n_e + BN - 1) / BN * p.groups_pe;
                int incl = cnt;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int t = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += t;
                }
                const int start = running + incl - cnt;
                for (int j = max(start, j0); j < min(start + cnt, j1); ++j) {
                    const int idx = j - j0;
                    if (idx < QS_MAX_JOBS) {
                        const int q = j - start, chunk = q / p.groups_pe;
                        job_expert[idx] = (int16_t)e;
                        job_group[idx] = (int16_t)(q - chunk * p.groups_pe);
                        job_row0[idx] = p.offsets[e] + chunk * BN;
                        job_rows[idx] = (int16_t)min(BN, n_e - chunk * BN);
                    }
                }
                running += __shfl_sync(0xffffffffu, incl, 31);
            }
            if (lane == 0) {
                job_range[0] = j0;
                job_range[1] = j1;
                if (j1 - j0 > QS_MAX_JOBS) atomicExch(p.status, 30);
            }
        }
        __syncthreads();
    }
    // this CTA's contiguous range of items
    int i0, i1;
    if (GROUPED) {
        i0 = 0;
        i1 = min(job_range[1] - job_range[0], QS_MAX_JOBS) * nb;
    } else if (p.whole_groups) {
        i0 = (int)((int64_t)c * p.groups / C) * nb;
        i1 = (int)((int64_t)(c + 1) * p.groups / C) * nb;
    } else {
        i0 = (int)((int64_t)c * p.items / C);
        i1 = (int)((int64_t)(c + 1) * p.items / C);
    }
    const int g0 = i0 / nb, b0 = i0 - g0 * nb;       // the only division of the item walk: (g, b) advance by counting
    const int acc_shift = R == 1 ? 2 : (R == 2 ? 1 : 0);  // QS_ACC / R accumulator sets
    const int n_stages = p.n_stages;
    // row tile r of group g: its index inside its matrix, whether it exists, and the index of its first unit
    const int tiles_limit = GROUPED ? p.tiles_pe : p.row_tiles;
    auto tile_of = [&](int g, int r) { return (GROUPED ? (int)job_group[g] : g) * R + r; };
    auto unit_tile = [&](int g, int tile) { return GROUPED ? (int64_t)job_expert[g] * p.tiles_pe + tile : (int64_t)tile; };

    if (warp == 0) {
        // one barrier per lane
        if (lane < n_stages) mbar_init(&raw_full[lane], 1);
        else if (lane < 2 * QS_MAX_STAGES && lane >= QS_MAX_STAGES && lane - QS_MAX_STAGES < n_stages) mbar_init(&raw_empty[lane - QS_MAX_STAGES], QS_CONV_WARPS / 2);
        else if (lane >= 16 && lane < 16 + QS_X_STAGES) mbar_init(&x_full[lane - 16], 1);
        else if (lane >= 20 && lane < 20 + QS_X_STAGES) mbar_init(&x_empty[lane - 20], 1);
        else if (lane >= 24 && lane < 26) mbar_init(&a_full[lane - 24], QS_CONV_WARPS / 2);
        else if (lane >= 26 && lane < 28) mbar_init(&a_empty[lane - 26], 1);
        else if (lane == 28) mbar_init(tmem_ready, 1);
        if (lane < QS_ACC) {
            mbar_init(&acc_full[lane], 1);
            mbar_init(&acc_empty[lane], QS_EPI_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // From here on the roles meet only through the mbarriers.  The weights depend on no predecessor kernel, so their
    // loader starts at once; the activation loader waits for the predecessor; every other access to global memory
    // (the epilogue's stores) is ordered after the activation loads through the mbarriers.
    pdl_trigger();
    QS_LOG(warp <= 3 ? warp : 4, 0);

    if (warp == 0) {
        // ---- weight loader
        int g = g0, b = b0;
        uint32_t st = 0, use = 0;
        for (int it = i0; it < i1; ++it) {
            for (int r = 0; r < R; ++r) {
                const int tile = tile_of(g, r);
                if (tile >= tiles_limit) break;
                if (!QS_WAIT(0, &raw_empty[st], (use & 1) ^ 1)) { if (lane == 0) atomicExch(p.status, 22); it = i1; break; }
                const bool seg_b = !GROUPED && tile >= p.tiles_a;
                const uint32_t bytes = (uint32_t)((seg_b ? p.fmt_b : p.fmt_a) ? QS_Q6K_UNIT : QS_Q4K_UNIT);
                const uint8_t* src = seg_b ? p.w_b + ((int64_t)(tile - p.tiles_a) * nb + b) * bytes : p.w_a + (unit_tile(g, tile) * nb + b) * bytes;
                if (elect_one()) {
                    mbar_expect_tx(&raw_full[st], bytes);
                    bulk_load(raw_ring + (size_t)st * p.stage_bytes, src, bytes, &raw_full[st]);
                }
                __syncwarp();
                QS_LOG(0, 2);
                if (++st == (uint32_t)n_stages) { st = 0; ++use; }
            }
            if (++b == nb) { b = 0; ++g; }
        }
    } else if (warp == 2) {
        // ---- activation loader: one block of 256 columns per item
        pdl_wait();
        QS_LOG(2, 1);
        int g = g0, b = b0;
        uint32_t st = 0, ph = 0;
        for (int it = i0; it < i1; ++it) {
            if (!QS_WAIT(0, &x_empty[st], ph ^ 1)) { if (lane == 0) atomicExch(p.status, 21); break; }
            uint8_t* xb = x_ring + (size_t)st * L::X_BYTES;
            if (elect_one()) {
                mbar_expect_tx(&x_full[st], (uint32_t)L::X_BYTES);
#pragma unroll
                for (int q = 0; q < 4; ++q) tma_load_2d(xb + q * BN * 128, &tm_x, b * 256 + q * 64, GROUPED ? job_row0[g] : 0, &x_full[st]);
            }
            __syncwarp();
            QS_LOG(2, 2);
            if (++b == nb) { b = 0; ++g; }
            if (++st == QS_X_STAGES) { st = 0; ph ^= 1; }
        }
    } else if (warp == 1) {
        // ---- tensor memory, then the MMA issuer
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"(QS_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(tmem_ready);
        mbar_wait(tmem_ready, 0, QS_SPIN_LIMIT);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&tmem_base_slot);
        QS_LOG(1, 8);
        const uint32_t idesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(QS_BM >> 4) << 24);
        // descriptor of 64-column box q of activation stage xs = b_desc0 + (xs * X_BYTES + q * BN * 128) / 16
        const uint64_t b_desc0 = make_sw128_desc(smem_u32(x_ring));
        int g = g0, b = b0, piece = 0;
        uint32_t n = 0, xs = 0, xph = 0;
        bool ok = true;
        for (int it = i0; it < i1 && ok; ++it) {
            const bool first = it == i0 || b == 0, last = it + 1 == i1 || b + 1 == nb;
            if (!QS_WAIT(0, &x_full[xs], xph)) { if (lane == 0) atomicExch(p.status, 24); break; }
            QS_LOG(1, 1);
            const int set = piece & ((QS_ACC >> (2 - acc_shift)) - 1), set_use = piece >> acc_shift;
            const uint64_t b_stage = b_desc0 + (uint64_t)((xs * L::X_BYTES) >> 4);
            for (int r = 0; r < R; ++r) {
                if (tile_of(g, r) >= tiles_limit) break;
                const int slot = set * R + r;
                if (first && !QS_WAIT(1, &acc_empty[slot], (uint32_t)(set_use & 1) ^ 1)) { if (lane == 0) atomicExch(p.status, 23); ok = false; break; }
                const uint32_t buf = n & 1;
                if (!QS_WAIT(2, &a_full[buf], (n >> 1) & 1)) { if (lane == 0) atomicExch(p.status, 25); ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                QS_LOG(1, 2);
                const uint32_t d_acc = tmem_base + (uint32_t)slot * BN;
                const uint32_t a_addr = tmem_base + QS_A_COL0 + buf * 128;
                if (elect_one()) {
                    if (!(PROF && (p.dbg & 4))) {
#pragma unroll
                        for (int k = 0; k < 16; ++k)
                            umma_f16_ts(d_acc, a_addr + 8 * k, b_stage + (uint64_t)(((k >> 2) * BN * 128) >> 4) + (uint64_t)(2 * (k & 3)), idesc,
                                        (first && k == 0) ? 0u : 1u);
                    }
                    umma_commit(&a_empty[buf]);
                    if (last) umma_commit(&acc_full[slot]);
                }
                __syncwarp();
                QS_LOG(1, 3);
                ++n;
            }
            if (ok && elect_one()) umma_commit(&x_empty[xs]);
            __syncwarp();
            if (last) ++piece;
            if (++b == nb) { b = 0; ++g; }
            if (++xs == QS_X_STAGES) { xs = 0; xph ^= 1; }
        }
    } else if (warp < 3 + QS_CONV_WARPS) {
        // ---- converters: two groups of eight warps; group i converts the units of odd/even order into A buffer i, so
        // that one group's hand-shakes (barrier waits, TMEM store, fences) run under the other group's arithmetic.
        // Warp w covers TMEM lanes 32 (w % 4) .. + 31 (weight rows) and two 64-column chunks of the block.
        const int quad = warp & 3, grp = (warp - 3) >> 3, h = ((warp - 3) >> 2) & 1;
        const int row = quad * 32 + lane;
        const uint32_t buf = (uint32_t)grp;
        int g = g0, b = b0;
        uint32_t n = 0, st = 0, use = 0, k = 0;  // unit counter; its ring stage and wrap count; units this group converted
        uint32_t tmem_base = 0;
        bool ok = true;
        for (int it = i0; it < i1 && ok; ++it) {
            for (int r = 0; r < R; ++r) {
                const int tile = tile_of(g, r);
                if (tile >= tiles_limit) break;
                if ((n & 1) == buf) {
                    if (!QS_WAIT(0, &raw_full[st], use & 1)) {
                        if (lane == 0) atomicExch(p.status, 26);
                        ok = false;
                        break;
                    }
                    if (warp == 3) QS_LOG(3, 1);
                    const uint8_t* raw = raw_ring + (size_t)st * p.stage_bytes;
                    if (k == 0) {  // the allocation ran while the first unit was on its way
                        if (!mbar_wait(tmem_ready, 0, QS_SPIN_LIMIT)) { if (lane == 0) atomicExch(p.status, 29); ok = false; break; }
                        tmem_base = *reinterpret_cast<volatile uint32_t*>(&tmem_base_slot);
                    }
                    if (!QS_WAIT(1, &a_empty[buf], (k & 1) ^ 1)) {
                        if (lane == 0) atomicExch(p.status, 27);
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (warp == 3) QS_LOG(3, 3);
                    const uint32_t t_dst = tmem_base + ((uint32_t)(quad * 32) << 16) + QS_A_COL0 + buf * 128 + 64 * h;
                    const bool q6 = ((!GROUPED && tile >= p.tiles_a) ? p.fmt_b : p.fmt_a) != 0;
                    uint32_t w[16];
                    if (PROF && (p.dbg & 1)) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) w[i] = n + i;
#pragma unroll
                        for (int q = 0; q < 4; ++q) tmem_st16(t_dst + 16 * q, w);
                    } else if (!q6) {
                        const uint8_t* blk = raw + row * 144;
                        const uint4 hdr = *reinterpret_cast<const uint4*>(blk);
                        if (h == 0) {
                            convert_q4k_group<0>(blk, hdr, w); tmem_st16(t_dst, w);
                            convert_q4k_group<1>(blk, hdr, w); tmem_st16(t_dst + 16, w);
                            convert_q4k_group<2>(blk, hdr, w); tmem_st16(t_dst + 32, w);
                            convert_q4k_group<3>(blk, hdr, w); tmem_st16(t_dst + 48, w);
                        } else {
                            convert_q4k_group<4>(blk, hdr, w); tmem_st16(t_dst, w);
                            convert_q4k_group<5>(blk, hdr, w); tmem_st16(t_dst + 16, w);
                            convert_q4k_group<6>(blk, hdr, w); tmem_st16(t_dst + 32, w);
                            convert_q4k_group<7>(blk, hdr, w); tmem_st16(t_dst + 48, w);
                        }
                    } else {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            convert_q6k_group(raw, row, 4 * h + q, w);
                            tmem_st16(t_dst + 16 * q, w);
                        }
                    }
                    if (warp == 3) QS_LOG(3, 2);
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(&a_full[buf]);
                        mbar_arrive(&raw_empty[st]);
                    }
                    if (warp == 3) QS_LOG(3, 5);
                    ++k;
                }
                ++n;
                if (++st == (uint32_t)n_stages) { st = 0; ++use; }
            }
            if (++b == nb) { b = 0; ++g; }
        }
    } else {
        // ---- epilogue warps: warp w reads TMEM lanes 32 (w % 4) .. + 31 (weight rows); the two warps of a lane quadrant
        // share a tile's token columns (first half / second half)
        const int quad = warp & 3, chalf = (warp - 3 - QS_CONV_WARPS) >> 2;
        const int row_in_tile = quad * 32 + lane;
        constexpr int CH = BN >= 64 ? 32 : (BN >= 32 ? 16 : 8);  // token columns per warp and tile
        int g = g0, b = b0, piece = 0;
        uint32_t tmem_base = 0;
        auto cta_of_item = [&](int i) {
            int cc = (int)((int64_t)i * C / p.items);
            while ((int)((int64_t)(cc + 1) * p.items / C) <= i) ++cc;
            while ((int)((int64_t)cc * p.items / C) > i) --cc;
            return cc;
        };
        bool ok = true;
        for (int it = i0; it < i1 && ok; ++it) {
            const bool last = it + 1 == i1 || b + 1 == nb;
            if (last) {
                if (piece == 0) {
                    if (!mbar_wait(tmem_ready, 0, QS_SPIN_LIMIT)) { if (lane == 0) atomicExch(p.status, 29); break; }
                    tmem_base = *reinterpret_cast<volatile uint32_t*>(&tmem_base_slot);
                }
                const int set = piece & ((QS_ACC >> (2 - acc_shift)) - 1), set_use = piece >> acc_shift;
                // split results: this piece's slot of the scratch
                int my_slot = 0;
                if (p.mode == 0 && p.slots > 1) my_slot = c - cta_of_item(g * nb);
                // token rows of this piece: the call's rows, or the chunk of one expert's rows
                const int tok0 = GROUPED ? job_row0[g] : 0, T_here = GROUPED ? (int)job_rows[g] : p.T;
                for (int r = 0; r < R && ok; ++r) {
                    const int tile = tile_of(g, r);
                    if (tile >= tiles_limit) break;
                    const int slot = set * R + r;
                    if (!QS_WAIT(0, &acc_full[slot], (uint32_t)(set_use & 1))) {
                        if (lane == 0) atomicExch(p.status, 28);
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (warp == 3 + QS_CONV_WARPS) QS_LOG(4, 1);
                    const uint32_t t_acc = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)slot * BN;
                    const int row = tile * QS_BM + row_in_tile;
                    {
                        const int c0 = chalf * CH;
                        uint32_t v[CH];
                        if constexpr (CH == 32) tmem_ld32(t_acc + c0, v);
                        else if constexpr (CH == 16) tmem_ld16(t_acc + c0, v);
                        else tmem_ld8(t_acc + c0, v);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        if (p.mode == 1) {
#pragma unroll
                            for (int t = 0; t < CH; t += 2) {
                                // rows 2f / 2f + 1 of the tile are gate / up of feature f: the even lane holds gate(t), gate(t+1),
                                // the odd lane up(t), up(t+1).  They swap one value: the even lane receives up(t) and finishes
                                // token t, the odd lane receives gate(t+1) and finishes token t + 1.
                                const float a0 = __uint_as_float(v[t]), a1 = __uint_as_float(v[t + 1]);
                                const float recv = __shfl_xor_sync(0xffffffffu, (lane & 1) ? a0 : a1, 1);
                                const float gate = (lane & 1) ? recv : a0;
                                const float up = (lane & 1) ? a1 : recv;
                                const int tok = c0 + t + (lane & 1);
                                if (row < p.rows && tok < T_here) p.yh[(int64_t)(tok0 + tok) * p.ldyh + (row >> 1)] = __float2half_rn(act_fn(gate, p.act) * up);
                            }
                        } else if (row < p.rows) {
                            const bool direct = p.slots == 1;
                            const int64_t ld = direct ? p.ldy : p.rows;
                            float* dst = (direct ? p.y : p.partial + (int64_t)my_slot * p.T * p.rows) + (int64_t)(tok0 + c0) * ld + row;
#pragma unroll
                            for (int t = 0; t < CH; ++t)
                                if (c0 + t < T_here) dst[(int64_t)t * ld] = __uint_as_float(v[t]);
                            if (!direct && b + 1 == nb) {  // the group's last piece: the slots this group does not use read as zero
                                for (int sl = my_slot + 1; sl < p.slots; ++sl) {
                                    float* z = p.partial + (int64_t)sl * p.T * p.rows + (int64_t)c0 * ld + row;
                                    for (int t = 0; t < CH && c0 + t < p.T; ++t) z[(int64_t)t * ld] = 0.f;
                                }
                            }
                        }
                    }
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (warp == 3 + QS_CONV_WARPS) QS_LOG(4, 2);
                    if (lane == 0) mbar_arrive(&acc_empty[slot]);
                }
                ++piece;
            }
            if (++b == nb) { b = 0; ++g; }
        }
    }

    if (PROF && p.prof != nullptr && blockIdx.x == 0 && lane == 0 && (warp <= 3 || warp == 3 + QS_CONV_WARPS)) {
        // rows: 0 weight loader, 1 MMA, 2 activation loader, 3 first converter warp, 4 first epilogue warp
        const int role = warp <= 3 ? warp : 4;
        for (int k = 0; k < tcnt; ++k) p.prof[41 + role * 400 + k] = tlog[role][k];
        long long* o = p.prof + role * 8;
        o[0] = clock64() - prof_t0;
        for (int i = 0; i < 4; ++i) o[1 + i] = prof_acc[i];
        o[5] = i1 - i0;
        o[6] = tcnt;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&tmem_base_slot);
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(QS_TMEM_COLS) : "memory");
    }
}

// Row-major Q4_K blocks [rows][nb][144 bytes] -> unit-major [row tile][block][128 rows][144 bytes], rows past the end
// zero (a zero block dequantises to zero).  `interleave` > 0: the source holds `interleave` gate rows followed by as
// many up rows and the destination row 2f is gate row f, row 2f + 1 up row f.  16 bytes per thread.
__global__ void retile_q4k_kernel(const uint4* src, int64_t rows, int nb, uint4* dst, int64_t chunks, int64_t interleave) {
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= chunks) return;
    const int64_t unit = c / (QS_Q4K_UNIT / 16);
    const int in_unit = (int)(c - unit * (QS_Q4K_UNIT / 16));
    const int r = in_unit / 9, part = in_unit - r * 9;  // 144 bytes = 9 chunks
    const int64_t tile = unit / nb, blk = unit - tile * nb;
    int64_t row = tile * QS_BM + r;
    if (interleave > 0 && row < rows) row = (row & 1) ? interleave + (row >> 1) : (row >> 1);
    dst[c] = row < rows ? src[(row * nb + blk) * 9 + part] : make_uint4(0, 0, 0, 0);
}

// Q6_K planes (QWeight layout: ql [rows*nb][128], qh [rows*nb][64], scales [rows*nb][16], d [rows*nb] f16) -> units of
// QS_Q6K_UNIT bytes with the chunk swizzle convert_q6k expects.  One thread per 16 bytes of a unit.
__global__ void retile_q6k_kernel(const uint8_t* ql, const uint8_t* qh, const uint8_t* sc, const __half* d, int64_t rows, int nb,
                                  uint8_t* dst, int64_t chunks) {
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= chunks) return;
    constexpr int CH = QS_Q6K_UNIT / 16;  // 1680
    const int64_t unit = c / CH;
    const int in_unit = (int)(c - unit * CH);
    const int64_t tile = unit / nb, blk = unit - tile * nb;
    uint4 v = make_uint4(0, 0, 0, 0);
    uint8_t* out = dst + unit * QS_Q6K_UNIT;
    if (in_unit < QS_BM * 8) {  // ql: 8 chunks per row
        const int r = in_unit >> 3, ch = in_unit & 7;
        const int64_t row = tile * QS_BM + r;
        if (row < rows) v = *reinterpret_cast<const uint4*>(ql + ((row * nb + blk) * 128 + ch * 16));
        *reinterpret_cast<uint4*>(out + Q6_QL + r * 128 + ((ch ^ (r & 7)) << 4)) = v;
    } else if (in_unit < QS_BM * 12) {  // qh: 4 chunks per row
        const int k = in_unit - QS_BM * 8, r = k >> 2, ch = k & 3;
        const int64_t row = tile * QS_BM + r;
        if (row < rows) v = *reinterpret_cast<const uint4*>(qh + ((row * nb + blk) * 64 + ch * 16));
        *reinterpret_cast<uint4*>(out + Q6_QH + r * 64 + ((ch ^ (r & 3)) << 4)) = v;
    } else if (in_unit < QS_BM * 13) {  // scales: 1 chunk per row
        const int r = in_unit - QS_BM * 12;
        const int64_t row = tile * QS_BM + r;
        if (row < rows) v = *reinterpret_cast<const uint4*>(sc + (row * nb + blk) * 16);
        *reinterpret_cast<uint4*>(out + Q6_SC + r * 16) = v;
    } else {  // d: 8 rows per chunk
        const int k = in_unit - QS_BM * 13;
        __half h[8];
        for (int i = 0; i < 8; ++i) {
            const int64_t row = tile * QS_BM + k * 8 + i;
            h[i] = row < rows ? d[row * nb + blk] : __float2half(0.f);
        }
        *reinterpret_cast<uint4*>(out + Q6_D + k * 16) = *reinterpret_cast<uint4*>(h);
    }
}

template <int BN>
size_t qs_smem_bytes(int n_stages, int stage_bytes) {
    return (size_t)QS_X_STAGES * QsSmem<BN>::X_BYTES + (size_t)n_stages * stage_bytes + 64 * sizeof(uint64_t) + 1024;
}

template <int BN>
void launch_qs(const CUtensorMap& tx, const QsParams& p, int ctas, cudaStream_t s) {
    const size_t smem = qs_smem_bytes<BN>(p.n_stages, p.stage_bytes);
    if (p.grouped) {
        ensure_dynamic_smem(reinterpret_cast<const void*>(&qstream_tc_kernel<BN, false, true>), smem);
        launch_pdl(qstream_tc_kernel<BN, false, true>, dim3(ctas), dim3(QS_THREADS), smem, s, tx, p);
    } else if (p.prof != nullptr) {
        ensure_dynamic_smem(reinterpret_cast<const void*>(&qstream_tc_kernel<BN, true, false>), smem);
        launch_pdl(qstream_tc_kernel<BN, true, false>, dim3(ctas), dim3(QS_THREADS), smem, s, tx, p);
    } else {
        ensure_dynamic_smem(reinterpret_cast<const void*>(&qstream_tc_kernel<BN, false, false>), smem);
        launch_pdl(qstream_tc_kernel<BN, false, false>, dim3(ctas), dim3(QS_THREADS), smem, s, tx, p);
    }
    MK_LAUNCH_CHECK();
}

}  // namespace

void build_qstream_weight(const void* q4k_blocks, int64_t rows, int64_t cols, QStreamWeight& out, cudaStream_t s, int64_t interleave) {
    if (cols <= 0 || cols % 256 != 0 || rows <= 0) throw std::runtime_error("build_qstream_weight: cols must be a positive multiple of 256");
    if (interleave > 0 && rows != 2 * interleave) throw std::runtime_error("build_qstream_weight: an interleaved matrix is gate rows then as many up rows");
    out.rows = rows;
    out.cols = cols;
    out.fmt = 0;
    out.gated = interleave > 0;
    const int nb = (int)(cols / 256);
    const int64_t row_tiles = (rows + QS_BM - 1) / QS_BM;
    out.row_tiles = (int)row_tiles;
    out.tiled.alloc((size_t)row_tiles * nb * QS_Q4K_UNIT);
    const int64_t chunks = row_tiles * nb * (QS_Q4K_UNIT / 16);
    retile_q4k_kernel<<<(unsigned)((chunks + 255) / 256), 256, 0, s>>>(reinterpret_cast<const uint4*>(q4k_blocks), rows, nb,
                                                                        out.tiled.as<uint4>(), chunks, interleave);
    MK_LAUNCH_CHECK();
    out.ready = true;
}

void build_qstream_weight_q6k(const QWeight& w, QStreamWeight& out, cudaStream_t s) {
    if (w.type != QT_Q6_K || w.cols <= 0 || w.cols % 256 != 0 || w.rows <= 0) throw std::runtime_error("build_qstream_weight_q6k: a Q6_K matrix with cols a multiple of 256");
    out.rows = w.rows;
    out.cols = w.cols;
    out.fmt = 1;
    out.gated = false;
    const int nb = (int)(w.cols / 256);
    const int64_t row_tiles = (w.rows + QS_BM - 1) / QS_BM;
    out.row_tiles = (int)row_tiles;
    out.tiled.alloc((size_t)row_tiles * nb * QS_Q6K_UNIT);
    const int64_t chunks = row_tiles * nb * (QS_Q6K_UNIT / 16);
    retile_q6k_kernel<<<(unsigned)((chunks + 255) / 256), 256, 0, s>>>(reinterpret_cast<const uint8_t*>(w.p0), reinterpret_cast<const uint8_t*>(w.p1),
                                                                        reinterpret_cast<const uint8_t*>(w.p2), reinterpret_cast<const __half*>(w.p3),
                                                                        w.rows, nb, out.tiled.as<uint8_t>(), chunks);
    MK_LAUNCH_CHECK();
    out.ready = true;
}

QStreamPlan qstream_plan(int row_tiles, int n_blocks, int64_t rows, int T, int max_splits, bool whole_groups, int sms) {
    QStreamPlan best;
    const int bn = T <= 16 ? 16 : (T <= 32 ? 32 : 64);
    double best_cost = 1e30;
    for (int R : {1, 2, 4}) {
        QStreamPlan pl;
        pl.bn = bn;
        pl.R = R;
        pl.row_tiles = row_tiles;
        pl.groups = (row_tiles + R - 1) / R;
        pl.items = pl.groups * n_blocks;
        pl.whole_groups = whole_groups || max_splits <= 1;
        int ctas;
        if (pl.whole_groups) {
            ctas = std::max(1, std::min(sms, pl.groups));
            pl.slots = 1;
        } else {
            ctas = std::max(1, std::min(sms, pl.items));
            auto pieces = [&](int cc) {  // most CTAs any group is spread over
                auto cta_of = [&](int64_t i) {
                    int64_t k = i * cc / pl.items;
                    while ((k + 1) * pl.items / cc <= i) ++k;
                    while (k * pl.items / cc > i) --k;
                    return (int)k;
                };
                int worst = 1;
                for (int g = 0; g < pl.groups; ++g) worst = std::max(worst, cta_of((int64_t)g * n_blocks + n_blocks - 1) - cta_of((int64_t)g * n_blocks) + 1);
                return worst;
            };
            while (ctas > pl.groups) {
                int sl = pieces(ctas);
                if (sl <= std::min(max_splits, 16) && (size_t)sl * T * rows * 4 <= kSplitScratchBytes) break;
                ctas = ctas * 3 / 4;
            }
            if (ctas <= pl.groups) {  // no cut fits the scratch or the cap on slots: whole groups per CTA
                pl.whole_groups = true;
                ctas = std::max(1, std::min(sms, pl.groups));
                pl.slots = 1;
            } else {
                pl.slots = pieces(ctas);
            }
        }
        pl.ctas = ctas;
        pl.partial_floats = pl.slots > 1 ? (size_t)pl.slots * T * rows : 0;
        // cost model: the busiest CTA's units (weights streamed and converted) plus its activation blocks (one per item,
        // about a unit's worth of L2 traffic each at 64 rows) plus the partial-sum traffic of the consumer
        int64_t worst_items;
        if (pl.whole_groups) worst_items = (int64_t)((pl.groups + ctas - 1) / ctas) * n_blocks;
        else worst_items = (pl.items + ctas - 1) / ctas;
        const int last_group_tiles = row_tiles - (pl.groups - 1) * R;
        (void)last_group_tiles;
        double cost = (double)worst_items * R + 0.5 * (double)worst_items * bn / 64.0 + 0.15 * pl.slots;
        if (cost < best_cost) {
            best_cost = cost;
            best = pl;
        }
    }
    return best;
}

static long long* g_qs_prof = nullptr;
void qstream_set_profile_buffer(long long* dev_buffer) { g_qs_prof = dev_buffer; }

int launch_qstream_tc(const QStreamWeight& W, const __half* xh, int T, float* y, int ldy, float* partial, size_t partial_floats,
                      int32_t* status, cudaStream_t s, int max_splits, const QStreamWeight* W2, int gated_act, __half* yh, int ldyh) {
    if (T <= 0) return 1;
    if (!W.ready || (W2 != nullptr && !W2->ready)) throw std::runtime_error("launch_qstream_tc: the matrix was not re-tiled");
    if (T > kQStreamMaxRows) throw std::runtime_error("launch_qstream_tc: more activation rows than the kernel covers");
    if (xh == nullptr) throw std::runtime_error("launch_qstream_tc: f16 activations missing");
    if (W2 != nullptr && (W2->cols != W.cols || W.rows % QS_BM != 0)) throw std::runtime_error("launch_qstream_tc: stacked matrices need equal widths and a first part of whole row tiles");
    const bool gated = gated_act >= 0;
    if (gated && (!W.gated || yh == nullptr || W2 != nullptr)) throw std::runtime_error("launch_qstream_tc: the gated form needs an interleaved gate|up matrix and an f16 output");
    if (partial == nullptr) max_splits = 1;
    const int nb = (int)(W.cols / 256);
    const int64_t rows = W.rows + (W2 ? W2->rows : 0);
    const int row_tiles = W.row_tiles + (W2 ? W2->row_tiles : 0);
    const int sms = device_sm_count();
    QStreamPlan pl = qstream_plan(row_tiles, nb, rows, T, gated ? 1 : max_splits, gated, sms);
    if (pl.slots > 1 && pl.partial_floats > partial_floats) pl = qstream_plan(row_tiles, nb, rows, T, 1, true, sms);
    alignas(64) CUtensorMap tx;
    encode_tma_2d(&tx, false, xh, (uint64_t)W.cols, (uint64_t)T, (uint64_t)W.cols * 2, 64, (uint32_t)pl.bn, true);
    QsParams p{};
    p.T = T;
    p.rows = (int)rows;
    p.n_blocks = nb;
    p.row_tiles = row_tiles;
    p.groups = pl.groups;
    p.R = pl.R;
    p.items = pl.items;
    p.whole_groups = pl.whole_groups ? 1 : 0;
    p.slots = pl.slots;
    p.tiles_a = W.row_tiles;
    p.fmt_a = W.fmt;
    p.fmt_b = W2 ? W2->fmt : W.fmt;
    p.stage_bytes = (p.fmt_a || p.fmt_b) ? QS_Q6K_UNIT : QS_Q4K_UNIT;
    const size_t x_bytes = (size_t)QS_X_STAGES * 4 * pl.bn * 128;
    p.n_stages = (int)std::min<size_t>(QS_MAX_STAGES, ((size_t)200 * 1024 - x_bytes) / (size_t)p.stage_bytes);
    p.mode = gated ? 1 : 0;
    p.act = gated ? gated_act : 0;
    p.w_a = W.tiled.as<uint8_t>();
    p.w_b = W2 ? W2->tiled.as<uint8_t>() : nullptr;
    p.y = y;
    p.ldy = ldy;
    p.yh = yh;
    p.ldyh = ldyh;
    p.partial = partial;
    p.status = status;
    p.prof = g_qs_prof;
    { const char* e = getenv("MACLLM_B200_QS_DBG"); p.dbg = (g_qs_prof != nullptr && e != nullptr) ? atoi(e) : 0; }
    if (pl.bn == 16) launch_qs<16>(tx, p, pl.ctas, s);
    else if (pl.bn == 32) launch_qs<32>(tx, p, pl.ctas, s);
    else launch_qs<64>(tx, p, pl.ctas, s);
    return pl.slots;
}

// Expert-grouped form (SparseMoeFeedForward::forward, src/decoder.rs:394-441: every expert multiplies the rows routed to it).
int launch_qstream_tc_grouped(const QStreamWeight& W, int experts, const int32_t* offsets_dev, const __half* xh, int rows_total,
                              int max_rows_per_expert, float* y, int ldy, int32_t* status, cudaStream_t s, int gated_act, __half* yh, int ldyh, bool rows_known) {
    if (rows_total <= 0) return 1;
    if (!W.ready) throw std::runtime_error("launch_qstream_tc_grouped: the matrix was not re-tiled");
    if (experts <= 0 || W.rows % experts != 0 || (W.rows / experts) % QS_BM != 0)
        throw std::runtime_error("launch_qstream_tc_grouped: every expert needs a whole number of 128-row tiles");
    if (xh == nullptr || offsets_dev == nullptr) throw std::runtime_error("launch_qstream_tc_grouped: activations or row ranges missing");
    const bool gated = gated_act >= 0;
    if (gated && (!W.gated || yh == nullptr)) throw std::runtime_error("launch_qstream_tc_grouped: the gated form needs an interleaved gate|up bank and an f16 output");
    const int nb = (int)(W.cols / 256);
    const int tiles_pe = (int)(W.rows / experts / QS_BM);
    const int bound = std::max(1, std::min(max_rows_per_expert, kQStreamMaxRows));
    const int bn = bound <= 16 ? 16 : (bound <= 32 ? 32 : 64);
    const int R = tiles_pe % 2 == 0 ? 2 : 1;
    const int sms = device_sm_count();
    // a bound on the jobs any CTA is handed: every expert may add one partly filled chunk
    const int64_t max_jobs = ((int64_t)rows_total / bn + experts) * (tiles_pe / R);
    if (rows_known && (max_jobs + sms - 1) / sms + 1 > QS_MAX_JOBS) throw std::runtime_error("launch_qstream_tc_grouped: more jobs per CTA than the kernel's table holds");
    alignas(64) CUtensorMap tx;
    encode_tma_2d(&tx, false, xh, (uint64_t)W.cols, (uint64_t)rows_total, (uint64_t)W.cols * 2, 64, (uint32_t)bn, true);
    QsParams p{};
    p.T = rows_total;
    p.rows = (int)(W.rows / experts);
    p.n_blocks = nb;
    p.row_tiles = W.row_tiles;
    p.R = R;
    p.groups = 0;
    p.items = 0;
    p.whole_groups = 1;
    p.slots = 1;
    p.tiles_a = W.row_tiles;
    p.fmt_a = p.fmt_b = W.fmt;
    p.stage_bytes = W.fmt ? QS_Q6K_UNIT : QS_Q4K_UNIT;
    const size_t x_bytes = (size_t)QS_X_STAGES * 4 * bn * 128;
    p.n_stages = (int)std::min<size_t>(QS_MAX_STAGES, ((size_t)200 * 1024 - x_bytes) / (size_t)p.stage_bytes);
    p.grouped = 1;
    p.experts = experts;
    p.tiles_pe = tiles_pe;
    p.groups_pe = tiles_pe / R;
    p.offsets = offsets_dev;
    p.mode = gated ? 1 : 0;
    p.act = gated ? gated_act : 0;
    p.w_a = W.tiled.as<uint8_t>();
    p.y = y;
    p.ldy = ldy;
    p.yh = yh;
    p.ldyh = ldyh;
    p.status = status;
    p.prof = nullptr;
    if (bn == 16) launch_qs<16>(tx, p, sms, s);
    else if (bn == 32) launch_qs<32>(tx, p, sms, s);
    else launch_qs<64>(tx, p, sms, s);
    return 1;
}

}  // namespace mk
