// Wide-batch matmul on the tcgen05 tensor cores over an f16 image of the weights.
//
// Replaces LinearOp::Quantized forward (src/model_weights.rs:346-377 of the reference) for prefill
// chunks: when hundreds of activation rows share one pass over a matrix, dequantising the GGUF blocks
// inside the GEMM repeats that work once per 128 tokens and the CUDA cores, not the tensor cores,
// set the pace.  A B200 has room to keep a second, f16 copy of every matrix (2 bytes per weight), made
// once at load time: w = f16(dequant(block)), one rounding per weight.  The GEMM is then the plain
// y[t][n] = sum_k xh[t][k] * wh[n][k] with f32 accumulation in tensor memory.
//
// One persistent CTA per SM, 192 threads in three roles:
//   warp 0   - one lane issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of a 128 x 64 weight
//              box and a BN x 64 activation box per stage into a ring of shared-memory stages;
//   warp 1   - one lane issues the MMAs (tcgen05.mma kind::f16, M = 128 weight rows, N = BN tokens,
//              four K = 16 steps per stage), commits each stage back to the loader, and commits the tile
//              to the epilogue; two accumulators in tensor memory alternate so the next tile's main
//              loop runs under the previous tile's epilogue;
//   warps 2-5 - read the accumulator (tcgen05.ld, one lane per weight row), apply scale / soft cap and
//              store f32 results (32 consecutive rows of one token per store instruction).
// Every mbarrier wait is bounded; a wait that gives up records a status word and the role leaves its
// loop, the other roles run into their own limits, and tensor memory is always released.
#include "hgemm_tc.h"
#include "kernels.h"
#include <cuda.h>
#include <mutex>

namespace mk {

namespace {

constexpr int HG_BM = 128;
constexpr int HG_BK = 64;  // 64 halves = 128 bytes = one swizzle row
constexpr int HG_THREADS = 192;
constexpr uint32_t HG_SPIN_LIMIT = 1u << 22;

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
// One 2-D box into this CTA's own shared memory; completes its bytes on the mbarrier.
__device__ __forceinline__ void tma_load_2d(void* dst, const void* tmap, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
// K-major operand tile with 128-byte rows and the 128-byte swizzle: 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t make_sw128_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;                    // leading byte offset: unused for swizzled K-major tiles
    d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset
    d |= (uint64_t)1 << 46;                    // descriptor version for sm_100
    d |= (uint64_t)2 << 61;                    // layout type: 128-byte swizzle
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

// ---- load-time dequantisation to f16 (values as the reference's dequantize: crates candle k_quants
// to_float order of operations: (d * scale) * q - (dmin * min) in f32, then one rounding to f16) -------

__device__ __forceinline__ void q4k_scale_min(const uint8_t* sc, int j, int& s, int& m) {
    if (j < 4) {
        s = sc[j] & 63;
        m = sc[j + 4] & 63;
    } else {
        s = (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4);
        m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4);
    }
}

// One warp per 256-element block; lane l produces elements 8l .. 8l+7.  Row r of W goes to out + r * row_stride.
__global__ void dequant_f16_kernel(QWeight W, __half* out, int64_t row_stride) {
    const int64_t nb = W.cols / 256;
    const int64_t b = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (b >= W.rows * nb) return;
    const int lane = threadIdx.x & 31;
    __half h[8];
    if (W.type == QT_Q4_K) {
        const uint8_t* blk = (const uint8_t*)W.p0 + b * 144;
        float d = __half2float(*reinterpret_cast<const __half*>(blk));
        float dmin = __half2float(*reinterpret_cast<const __half*>(blk + 2));
        int j = lane >> 2;  // 32-element group
        int s, m;
        q4k_scale_min(blk + 4, j, s, m);
        float d1 = __fmul_rn(d, (float)s), m1 = __fmul_rn(dmin, (float)m);
        const uint8_t* qs = blk + 16 + (j >> 1) * 32 + (lane & 3) * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            int q = (j & 1) ? (qs[i] >> 4) : (qs[i] & 0xF);
            h[i] = __float2half_rn(__fsub_rn(__fmul_rn(d1, (float)q), m1));
        }
    } else if (W.type == QT_Q6_K) {
        const uint8_t* ql = (const uint8_t*)W.p0 + b * 128;
        const uint8_t* qh = (const uint8_t*)W.p1 + b * 64;
        const int8_t* sc = (const int8_t*)W.p2 + b * 16;
        float d = __half2float(((const __half*)W.p3)[b]);
        int e0 = lane * 8;
        int hf = e0 >> 7, r = e0 & 127;     // 128-element half, offset inside it
        int grp = r >> 5, l0 = r & 31;       // which of the four 32-element quarters, first l
        float ds = __fmul_rn(d, (float)sc[hf * 8 + (l0 >> 4) + 2 * grp]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            int l = l0 + i;
            uint8_t lo = ql[hf * 64 + (grp & 1) * 32 + l];
            int nib = (grp >> 1) ? (lo >> 4) : (lo & 0xF);
            int q = (nib | (((qh[hf * 32 + l] >> (2 * grp)) & 3) << 4)) - 32;
            h[i] = __float2half_rn(__fmul_rn(ds, (float)q));
        }
    } else if (W.type == QT_Q8_0) {
        int64_t row = b / nb, ib = b - row * nb;
        const int8_t* qs = (const int8_t*)W.p0 + row * W.cols + ib * 256 + lane * 8;
        float d = __half2float(((const __half*)W.p1)[row * (W.cols / 32) + ib * 8 + (lane >> 2)]);
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] = __float2half_rn(__fmul_rn(d, (float)qs[i]));
    } else {  // QT_F32
        const float* src = (const float*)W.p0 + b * 256 + lane * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] = __float2half_rn(src[i]);
    }
    const int64_t out_row = b / nb, out_blk = b - out_row * nb;
    *reinterpret_cast<uint4*>(out + out_row * row_stride + out_blk * 256 + lane * 8) = *reinterpret_cast<uint4*>(h);
}

// ---- the GEMM ------------------------------------------------------------------------------------

struct HgParams {
    int T, K, rows;
    float* y;
    int ldy;
    float out_scale, softcap;
    int row_tiles, n_tiles;
    // split-K (narrow batches, long K): work item = (output tile, K share); every share writes its f32
    // partial sums to partial[share][T][rows] and the kernel that consumes the result adds the shares in
    // share order, so the value does not depend on scheduling and no extra pass over the output is needed
    int splits, kb_per_split;
    float* partial;
    int32_t* status;
    // gated epilogue (splits == 1): weight rows 2j / 2j+1 are the gate / up projections of feature j and the kernel
    // writes yh[t][j] = f16(act(gate) * up) instead of y; 0 = off, 1 = SiLU, 2 = tanh GELU
    int gated;
    __half* yh;
    int ldyh;
};

template <int BN, int STAGES>
struct HgSmem {
    static constexpr int A_BYTES = HG_BM * HG_BK * 2;   // 16 KiB
    static constexpr int B_BYTES = BN * HG_BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr size_t TOTAL = (size_t)STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
};

__device__ __forceinline__ float finish_value(float v, const HgParams& p) {
    v *= p.out_scale;
    if (p.softcap != 0.f) v = tanhf(v * (1.0f / p.softcap)) * p.softcap;
    return v;
}

// The activations of the gated feed-forward, as the SwiGLU kernel of quantize.cu computes them.
__device__ __forceinline__ float hg_silu(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float hg_gelu_tanh(float x) {
    return 0.5f * x * (1.0f + tanhf(0.7978845608028654f * x * (1.0f + 0.044715f * x * x)));
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(HG_THREADS, 1)
hgemm_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, HgParams p) {
    using L = HgSmem<BN, STAGES>;
    constexpr int LD_COLS = BN >= 32 ? 32 : BN;
    extern __shared__ uint8_t hg_smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(hg_smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + (size_t)STAGES * L::STAGE_BYTES);
    uint64_t* full = bars;                  // [STAGES]  loader -> MMA
    uint64_t* empty = bars + STAGES;        // [STAGES]  MMA -> loader
    uint64_t* acc_full = bars + 2 * STAGES; // [2]       MMA -> epilogue
    uint64_t* acc_empty = acc_full + 2;     // [2]       epilogue -> MMA
    __shared__ uint32_t tmem_base_slot;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = p.K / HG_BK;
    const int mn_tiles = p.row_tiles * p.n_tiles;
    const int total_items = mn_tiles * p.splits;
    constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], 128);
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
    // Everything above is private to the CTA.  The weights do not depend on the predecessor kernel either, so
    // the loader fills the ring with weight boxes first and only then waits for the predecessor, whose output
    // (the activations) it loads next.  Every other access to global memory of this kernel (the epilogue's
    // stores) is ordered after those loads through the mbarriers.
    pdl_trigger();

    // work item -> (row tile, token tile, K share); token tiles vary fastest, so the CTAs that run side by side cover
    // a few row tiles across every token tile: each weight box comes from HBM once and the activations stay in L2
    auto decode = [&](int item, int& m_tile, int& n_tile, int& kb0, int& kb1) {
        int mn = item % mn_tiles, split = item / mn_tiles;
        m_tile = mn / p.n_tiles;
        n_tile = mn % p.n_tiles;
        kb0 = split * p.kb_per_split;
        kb1 = min(k_blocks, kb0 + p.kb_per_split);
    };

    if (warp == 0) {
        // ---- loader
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true, waited = false;
            int held_x[STAGES], held_y[STAGES];  // activation boxes of the stages filled before the wait
            for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
                int m_tile, n_tile, kb0, kb1;
                decode(item, m_tile, n_tile, kb0, kb1);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const uint32_t st = it % STAGES, ph = (it / STAGES) & 1;
                    if (it == STAGES && !waited) {  // the ring is full of weights: now the activations
                        pdl_wait();
                        waited = true;
                        for (int h = 0; h < STAGES; ++h)
                            tma_load_2d(tiles + (size_t)h * L::STAGE_BYTES + L::A_BYTES, &tm_x, held_x[h], held_y[h], &full[h]);
                    }
                    if (!mbar_wait(&empty[st], ph ^ 1, HG_SPIN_LIMIT)) {
                        atomicExch(p.status, 11);
                        ok = false;
                        break;
                    }
                    uint8_t* a_dst = tiles + (size_t)st * L::STAGE_BYTES;
                    uint8_t* b_dst = a_dst + L::A_BYTES;
                    mbar_expect_tx(&full[st], (uint32_t)L::STAGE_BYTES);
                    tma_load_2d(a_dst, &tm_w, kb * HG_BK, m_tile * HG_BM, &full[st]);
                    if (waited) {
                        tma_load_2d(b_dst, &tm_x, kb * HG_BK, n_tile * BN, &full[st]);
                    } else {
                        held_x[st] = kb * HG_BK;
                        held_y[st] = n_tile * BN;
                    }
                }
            }
            if (!waited) {  // fewer stages of work than the ring holds
                pdl_wait();
                for (uint32_t h = 0; h < it && h < (uint32_t)STAGES; ++h)
                    tma_load_2d(tiles + (size_t)h * L::STAGE_BYTES + L::A_BYTES, &tm_x, held_x[h], held_y[h], &full[h]);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(HG_BM >> 4) << 24);
            uint32_t it = 0, tile_it = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++tile_it) {
                int m_tile, n_tile, kb0, kb1;
                decode(item, m_tile, n_tile, kb0, kb1);
                const uint32_t acc = tile_it & 1, acc_ph = (tile_it >> 1) & 1;
                if (!mbar_wait(&acc_empty[acc], acc_ph ^ 1, HG_SPIN_LIMIT)) {
                    atomicExch(p.status, 12);
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const uint32_t st = it % STAGES, ph = (it / STAGES) & 1;
                    if (!mbar_wait(&full[st], ph, HG_SPIN_LIMIT)) {
                        atomicExch(p.status, 13);
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_u32(tiles + (size_t)st * L::STAGE_BYTES);
                    const uint32_t b_addr = a_addr + L::A_BYTES;
                    const uint64_t adesc = make_sw128_desc(a_addr), bdesc = make_sw128_desc(b_addr);
#pragma unroll
                    for (int k = 0; k < HG_BK / 16; ++k) {
                        // 16 halves = 32 bytes further along K inside the swizzled row: +2 in 16-byte units
                        umma_f16(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty[st]);
                }
                if (ok) umma_commit(&acc_full[acc]);
            }
        }
    } else {
        // ---- epilogue: warps 2..5 own TMEM lane quadrants (warp % 4)
        const int quad = warp & 3;
        const int etid = (int)threadIdx.x - 64;  // 0..127 among the epilogue threads
        uint32_t tile_it = 0;
        for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++tile_it) {
            int m_tile, n_tile, kb0, kb1;
            decode(item, m_tile, n_tile, kb0, kb1);
            const int split = item / mn_tiles;
            const uint32_t acc = tile_it & 1, acc_ph = (tile_it >> 1) & 1;
            // every epilogue warp waits for itself, then the four agree on the outcome, so that a wait that
            // gave up takes all of them out of the loop together (they meet again at named barrier 1)
            const uint32_t got = mbar_wait(&acc_full[acc], acc_ph, HG_SPIN_LIMIT) ? 1u : 0u;
            uint32_t all_got;
            asm volatile(
                "{\n\t.reg .pred p, q;\n\t"
                "setp.ne.u32 q, %1, 0;\n\t"
                "bar.red.and.pred p, 1, 128, q;\n\t"
                "selp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(all_got)
                : "r"(got)
                : "memory");
            if (!all_got) {
                if (etid == 0) atomicExch(p.status, 14);
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = m_tile * HG_BM + quad * 32 + lane;
            const int tok0 = n_tile * BN;
            float* dst = p.splits > 1 ? p.partial + (int64_t)split * p.T * p.rows : p.y;
            const int ld = p.splits > 1 ? p.rows : p.ldy;
#pragma unroll 1
            for (int cb = 0; cb < BN; cb += LD_COLS) {
                if (tok0 + cb >= p.T) break;  // uniform over the CTA: nothing but padding from here on
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN + (uint32_t)cb, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (p.gated != 0) {
                    // lanes 2i / 2i+1 hold gate / up of one feature: the even lane finishes the even token columns,
                    // the odd lane the odd ones, after one exchange per pair of columns
                    const bool odd = (lane & 1) != 0;
                    const int feature = row >> 1;
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        float mine = __uint_as_float(odd ? r[i] : r[i + 1]);       // what the partner needs
                        float theirs = __shfl_xor_sync(0xffffffffu, mine, 1);
                        float g = odd ? theirs : __uint_as_float(r[i]);
                        float u = odd ? __uint_as_float(r[i + 1]) : theirs;
                        int tok = tok0 + cb + i + (odd ? 1 : 0);
                        if (row < p.rows && tok < p.T) {
                            float a = p.gated == 1 ? hg_silu(g) : hg_gelu_tanh(g);
                            p.yh[(int64_t)tok * p.ldyh + feature] = __float2half_rn(a * u);
                        }
                    }
                } else if (row < p.rows) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        int tok = tok0 + cb + i;
                        if (tok < p.T) {
                            float v = __uint_as_float(r[i]);
                            if (p.splits == 1) v = finish_value(v, p);
                            dst[(int64_t)tok * ld + row] = v;
                        }
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&acc_empty[acc]);
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---- host side --------------------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q);
        if (e == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    if (fn == nullptr) throw std::runtime_error("the CUDA driver does not provide cuTensorMapEncodeTiled");
    return fn;
}

// f16 matrix [n_rows][cols] row-major, boxes of box_rows x 64 columns, 128-byte swizzle, zero fill.
void encode_half_matrix(CUtensorMap* out, const void* base, int64_t n_rows, int64_t cols, int box_rows) {
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) throw std::runtime_error("hgemm: matrix base must be 16-byte aligned");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)n_rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)HG_BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = encode_fn()(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
}

template <int BN, int STAGES>
void launch_hg(const CUtensorMap& tw, const CUtensorMap& tx, const HgParams& p, int grid, cudaStream_t s) {
    constexpr size_t smem = HgSmem<BN, STAGES>::TOTAL;
    ensure_dynamic_smem(reinterpret_cast<const void*>(&hgemm_tc_kernel<BN, STAGES>), smem);
    launch_pdl(hgemm_tc_kernel<BN, STAGES>, dim3(grid), dim3(HG_THREADS), smem, s, tw, tx, p);
    MK_LAUNCH_CHECK();
}

}  // namespace

void encode_tma_2d(void* out_map, bool bytes_not_halves, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                   uint32_t box_inner, uint32_t box_outer, bool swizzle_128b) {
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || row_stride_bytes % 16 != 0)
        throw std::runtime_error("TMA descriptor: base and row stride must be multiples of 16 bytes");
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)row_stride_bytes};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = encode_fn()(reinterpret_cast<CUtensorMap*>(out_map),
                             bytes_not_halves ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                             const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             swizzle_128b ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
}



bool hgemm_tc_supported(const QWeight& W) {
    if (W.type != QT_Q4_K && W.type != QT_Q6_K && W.type != QT_Q8_0 && W.type != QT_F32) return false;
    return W.cols % 256 == 0 && W.rows > 0;
}

void build_half_weight_stacked(const QWeight* const* parts, int n_parts, HalfWeight& out, cudaStream_t s) {
    if (n_parts <= 0) throw std::runtime_error("build_half_weight: nothing to build");
    int64_t rows = 0;
    const int64_t cols = parts[0]->cols;
    for (int i = 0; i < n_parts; ++i) {
        if (!hgemm_tc_supported(*parts[i]) || parts[i]->cols != cols) throw std::runtime_error("build_half_weight: unsupported matrix");
        rows += parts[i]->rows;
    }
    out.rows = rows;
    out.cols = cols;
    out.values.alloc((size_t)rows * (size_t)cols * 2);
    int64_t row0 = 0;
    for (int i = 0; i < n_parts; ++i) {
        const QWeight& W = *parts[i];
        const int64_t blocks = W.rows * (W.cols / 256);
        const int warps_per_cta = 8;
        dequant_f16_kernel<<<(unsigned)((blocks + warps_per_cta - 1) / warps_per_cta), warps_per_cta * 32, 0, s>>>(
            W, out.values.as<__half>() + row0 * cols, cols);
        MK_LAUNCH_CHECK();
        row0 += W.rows;
    }
    static_assert(sizeof(CUtensorMap) <= sizeof(out.tmap), "descriptor storage too small");
    encode_half_matrix(reinterpret_cast<CUtensorMap*>(out.tmap), out.values.ptr(), rows, cols, HG_BM);
    out.ready = true;
}

void build_half_weight_interleaved(const QWeight& gate, const QWeight& up, HalfWeight& out, cudaStream_t s) {
    if (!hgemm_tc_supported(gate) || !hgemm_tc_supported(up) || gate.cols != up.cols || gate.rows != up.rows)
        throw std::runtime_error("build_half_weight_interleaved: unsupported pair of matrices");
    const int64_t cols = gate.cols;
    out.rows = 2 * gate.rows;
    out.cols = cols;
    out.values.alloc((size_t)out.rows * (size_t)cols * 2);
    const QWeight* parts[2] = {&gate, &up};
    for (int i = 0; i < 2; ++i) {
        const int64_t blocks = parts[i]->rows * (cols / 256);
        const int warps_per_cta = 8;
        dequant_f16_kernel<<<(unsigned)((blocks + warps_per_cta - 1) / warps_per_cta), warps_per_cta * 32, 0, s>>>(
            *parts[i], out.values.as<__half>() + i * cols, 2 * cols);
        MK_LAUNCH_CHECK();
    }
    encode_half_matrix(reinterpret_cast<CUtensorMap*>(out.tmap), out.values.ptr(), out.rows, cols, HG_BM);
    out.ready = true;
}

void build_half_weight(const QWeight& W, HalfWeight& out, cudaStream_t s) {
    const QWeight* one = &W;
    build_half_weight_stacked(&one, 1, out, s);
}

HgemmPlan hgemm_tc_plan(int64_t rows, int64_t cols, int T, int max_splits) {
    HgemmPlan pl;
    pl.bn = T <= 64 ? 64 : 128;
    if (T > 128) {
        // 256-token tiles do about 10 % more per unit of time (less shared-memory traffic per MMA, half the epilogue
        // hand-offs), 128-token tiles fill the last round of CTAs better: take the one with fewer (rounds x tile time)
        const int64_t mt = (rows + HG_BM - 1) / HG_BM;
        const double cost256 = (double)((mt * ((T + 255) / 256) + 147) / 148) * 2.0;
        const double cost128 = (double)((mt * ((T + 127) / 128) + 147) / 148) * 1.1;
        pl.bn = cost128 < cost256 ? 128 : 256;
    }
    pl.row_tiles = (int)((rows + HG_BM - 1) / HG_BM);
    pl.n_tiles = (T + pl.bn - 1) / pl.bn;
    const int kb = (int)(cols / HG_BK);
    const int tiles = pl.row_tiles * pl.n_tiles;
    const int sms = 148;
    // shares of K per output tile: fewest "waves x (K blocks per share + fixed cost)" with shares of at least
    // four K blocks and at most 16 MiB of partial sums
    int best = 1;
    long best_cost = -1;
    for (int s = 1; s <= std::max(1, std::min(max_splits, 16)); ++s) {
        int per = (kb + s - 1) / s;
        if (s > 1 && (per < 4 || (size_t)s * T * rows * 4 > ((size_t)16 << 20))) break;
        if ((kb + per - 1) / per != s) continue;  // not a distinct split
        long waves = ((long)tiles * s + sms - 1) / sms;
        long cost = waves * (per + 3) + (s > 1 ? 1 : 0);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = s; }
    }
    pl.splits = best;
    pl.kb_per_split = (kb + best - 1) / best;
    pl.partial_floats = best > 1 ? (size_t)best * T * rows : 0;
    return pl;
}

namespace {
int launch_hgemm_any(const HalfWeight& W, const __half* xh, int T, float* y, int ldy, float out_scale, float softcap,
                     const HgemmScratch& ws, cudaStream_t s, int max_splits, int gated, __half* yh, int ldyh);
}

int launch_hgemm_tc(const HalfWeight& W, const __half* xh, int T, float* y, int ldy, float out_scale, float softcap,
                    const HgemmScratch& ws, cudaStream_t s, int max_splits) {
    return launch_hgemm_any(W, xh, T, y, ldy, out_scale, softcap, ws, s, max_splits, 0, nullptr, 0);
}

void launch_hgemm_tc_gated(const HalfWeight& W, const __half* xh, int T, int act, __half* yh, int ldyh, const HgemmScratch& ws,
                           cudaStream_t s) {
    if (W.rows % 2 != 0 || yh == nullptr) throw std::runtime_error("launch_hgemm_tc_gated: needs an interleaved gate/up image and an output");
    launch_hgemm_any(W, xh, T, nullptr, 0, 1.0f, 0.f, ws, s, 1, act == 0 ? 1 : 2, yh, ldyh);
}

namespace {
int launch_hgemm_any(const HalfWeight& W, const __half* xh, int T, float* y, int ldy, float out_scale, float softcap,
                     const HgemmScratch& ws, cudaStream_t s, int max_splits, int gated, __half* yh, int ldyh) {
    if (T <= 0) return 1;
    if (!W.ready) throw std::runtime_error("launch_hgemm_tc: the f16 image of the matrix was not built");
    if (xh == nullptr) throw std::runtime_error("launch_hgemm_tc: f16 activations missing");
    if (out_scale != 1.0f || softcap != 0.f || ws.partial == nullptr) max_splits = 1;
    HgemmPlan pl = hgemm_tc_plan(W.rows, W.cols, T, max_splits);
    if (pl.splits > 1 && pl.partial_floats > ws.partial_floats) {
        pl.splits = 1;
        pl.kb_per_split = (int)(W.cols / HG_BK);
    }
    alignas(64) CUtensorMap tx;
    encode_half_matrix(&tx, xh, T, W.cols, pl.bn);
    HgParams p;
    p.T = T;
    p.K = (int)W.cols;
    p.rows = (int)W.rows;
    p.y = y;
    p.ldy = ldy;
    p.out_scale = out_scale;
    p.softcap = softcap;
    p.row_tiles = pl.row_tiles;
    p.n_tiles = pl.n_tiles;
    p.splits = pl.splits;
    p.kb_per_split = pl.kb_per_split;
    p.partial = ws.partial;
    p.status = ws.status;
    p.gated = gated;
    p.yh = yh;
    p.ldyh = ldyh;
    const int grid = std::min(device_sm_count(), p.row_tiles * p.n_tiles * p.splits);
    const CUtensorMap& tw = *reinterpret_cast<const CUtensorMap*>(W.tmap);
    if (pl.bn == 256) launch_hg<256, 4>(tw, tx, p, grid, s);
    else if (pl.bn == 128) launch_hg<128, 6>(tw, tx, p, grid, s);
    else launch_hg<64, 8>(tw, tx, p, grid, s);
    return pl.splits;
}
}  // namespace

}  // namespace mk
