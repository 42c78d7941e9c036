// C ABI, part 1: kernel-level entry points used for unit parity.  Host buffers in, host buffers out;
// each call stages its operands in HBM, runs the sm_100a kernel and reads the result back.
#include "../../include/macllm_b200.h"
#include "c_api_util.h"
#include "device_util.h"
#include "kernels.h"
#include "hgemm_tc.h"
#include "qstream_tc.h"
#include "host_sampler.h"
#include "attention_tc.h"
#include "qgemm_tc.h"
#include "recurrent.h"
#include <vector>
#include <cstring>

using namespace mk;

namespace {

struct ActBufs {
    DevBuf qs, d, bs, xh;
    ActQ view(int T, int K, int kind, bool want_f16 = false) {
        qs.ensure((size_t)T * K);
        d.ensure((size_t)T * (kind == ACT_Q8K ? K / 256 : K / 32) * 4);
        bs.ensure((size_t)T * (K / 16) * 2 + 16);
        ActQ a;
        a.qs = qs.as<int8_t>();
        a.d = d.as<float>();
        a.bsums = bs.as<int16_t>();
        if (want_f16) {
            xh.ensure((size_t)T * K * 2);
            a.xh = xh.as<__half>();
        }
        return a;
    }
};

int act_kind_for(int wtype) { return wtype == QT_Q8_0 ? ACT_Q80 : ACT_Q8K; }

}  // namespace

extern "C" {

int32_t mk_k_quantize(int32_t act_kind, const float* x, int32_t T, int32_t K, int8_t* qs, float* d, int16_t* bsums) {
    return guarded([&] {
        require_device();
        if (K % 256 != 0 && act_kind == ACT_Q8K) throw std::runtime_error("mk_k_quantize: K must be a multiple of 256");
        if (K % 32 != 0) throw std::runtime_error("mk_k_quantize: K must be a multiple of 32");
        DevBuf dx((size_t)T * K * 4);
        dx.upload(x, (size_t)T * K * 4);
        ActBufs ab;
        ActQ a = ab.view(T, K, act_kind);
        NormQuantArgs na;
        na.h = dx.as<float>();
        na.rows = T;
        na.dim = K;
        na.act_kind = act_kind;
        na.out = a;
        launch_add_norm_quant(na, nullptr);
        MK_CUDA(cudaDeviceSynchronize());
        ab.qs.download(qs, (size_t)T * K);
        ab.d.download(d, (size_t)T * (act_kind == ACT_Q8K ? K / 256 : K / 32) * 4);
        if (act_kind == ACT_Q8K && bsums) ab.bs.download(bsums, (size_t)T * (K / 16) * 2);
        MK_CUDA(cudaDeviceSynchronize());
    });
}

int32_t mk_k_add_norm(float* h, const float* a, float a_scale, const float* post_w, const float* norm_w, float eps,
                      int32_t rows, int32_t dim, float* normed_out) {
    return guarded([&] {
        require_device();
        size_t n = (size_t)rows * dim * 4;
        DevBuf dh(n), da, dpw, dnw, dout(n);
        dh.upload(h, n);
        NormQuantArgs na;
        na.h = dh.as<float>();
        if (a) { da.upload(a, n); na.a = da.as<float>(); }
        if (post_w) { dpw.upload(post_w, (size_t)dim * 4); na.post_w = dpw.as<float>(); }
        if (norm_w) { dnw.upload(norm_w, (size_t)dim * 4); na.norm_w = dnw.as<float>(); }
        na.a_scale = a_scale;
        na.eps = eps;
        na.rows = rows;
        na.dim = dim;
        na.normed_out = dout.as<float>();
        launch_add_norm_quant(na, nullptr);
        MK_CUDA(cudaDeviceSynchronize());
        dh.download(h, n);
        if (normed_out) dout.download(normed_out, n);
        MK_CUDA(cudaDeviceSynchronize());
    });
}

namespace {

// Shared body of mk_k_qmatmul and mk_k_qmatmul_time: upload, quantise the activations once, then run the
// chosen matmul `iters` times (timed one by one with the L2 flushed in between when avg_ms is wanted).
void qmatmul_case(int32_t type, const void* w, int64_t rows, int64_t cols, const float* x, int32_t T, float* y, int32_t path,
                  int iters, float* avg_ms) {
    require_device();
    if (path < MK_PATH_AUTO || path > MK_PATH_STREAM) throw std::runtime_error("mk_k_qmatmul: unknown path selector");
    DeviceWeight dw;
    upload_weight(type, w, rows, cols, dw);
    int kind = act_kind_for(type);
    DevBuf dx((size_t)T * cols * 4), dy((size_t)T * rows * 4);
    dx.upload(x, (size_t)T * cols * 4);
    ActBufs ab;
    const bool half = path == MK_PATH_HALF;
    const bool stream = path == MK_PATH_STREAM;
    QStreamWeight qsw;
    // MACLLM_B200_QS_SPLITS=1 keeps whole groups of row tiles in one CTA (no partial sums), for tests of that form
    const int stream_splits = [] { const char* e = getenv("MACLLM_B200_QS_SPLITS"); return e != nullptr ? std::max(1, atoi(e)) : 16; }();  // read per call
    DevBuf qs_partial;
    int qs_splits = 1;
    if (stream) {
        if ((type != MK_TYPE_Q4_K && type != MK_TYPE_Q6_K) || T > kQStreamMaxRows)
            throw std::runtime_error("mk_k_qmatmul: the streamed matmul covers Q4_K and Q6_K matrices and at most 64 rows");
        if (type == MK_TYPE_Q4_K) build_qstream_weight(dw.w.p0, rows, cols, qsw, nullptr);
        else build_qstream_weight_q6k(dw.w, qsw, nullptr);
        qs_partial.alloc(kSplitScratchBytes);
    }
    if (half) {
        if (!hgemm_tc_supported(dw.w)) throw std::runtime_error("mk_k_qmatmul: the f16-image GEMM does not cover this matrix");
        build_half_weight(dw.w, dw.half, nullptr);
        // narrow batches share K out over CTAs, as the model's decode ticks do; the shares are added below
        if (T <= kQStreamMaxRows) qs_partial.alloc(kSplitScratchBytes);
    }
    const bool tensor = !half && !stream && (path == MK_PATH_TENSOR || (path == MK_PATH_AUTO && qgemm_tc_preferred(dw.w, T)));
    ActQ a = ab.view(T, (int)cols, kind, tensor || half || stream);
    NormQuantArgs na;
    na.h = dx.as<float>();
    na.rows = T;
    na.dim = (int)cols;
    na.act_kind = kind;
    na.out = a;
    launch_add_norm_quant(na, nullptr);
    QgemmWorkspace ws;
    ws.status.alloc(sizeof(int32_t));
    ws.status.zero(nullptr);
    HgemmScratch hs;
    hs.status = ws.status.as<int32_t>();
    if (half && qs_partial.size() > 0) {
        hs.partial = qs_partial.as<float>();
        hs.partial_floats = qs_partial.size() / 4;
    }
    auto run = [&] {
        if (stream) qs_splits = launch_qstream_tc(qsw, a.xh, T, dy.as<float>(), (int)rows, qs_partial.as<float>(), qs_partial.size() / 4,
                                                  ws.status.as<int32_t>(), nullptr, stream_splits);
        else if (half) qs_splits = launch_hgemm_tc(dw.half, a.xh, T, dy.as<float>(), (int)rows, 1.0f, 0.f, hs, nullptr, hs.partial ? 16 : 1);
        else if (tensor) launch_qgemm_tc(dw.w, a, kind, T, dy.as<float>(), (int)rows, 1.0f, 0.f, ws, nullptr);
        else launch_qgemv(dw.w, a, T, dy.as<float>(), (int)rows, 1.0f, 0.f, nullptr);
    };
    if (avg_ms == nullptr) {
        run();
    } else {
        DevBuf flush((size_t)256 << 20);  // larger than the L2
        cudaEvent_t e0, e1;
        MK_CUDA(cudaEventCreate(&e0));
        MK_CUDA(cudaEventCreate(&e1));
        double total = 0;
        for (int i = 0; i < iters + 2; ++i) {
            flush.zero(nullptr);
            MK_CUDA(cudaEventRecord(e0, nullptr));
            run();
            MK_CUDA(cudaEventRecord(e1, nullptr));
            MK_CUDA(cudaEventSynchronize(e1));
            float ms = 0;
            MK_CUDA(cudaEventElapsedTime(&ms, e0, e1));
            if (i >= 2) total += ms;
        }
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        *avg_ms = (float)(total / iters);
    }
    MK_CUDA(cudaDeviceSynchronize());
    if (stream && getenv("MACLLM_B200_QS_PROF") != nullptr) {
        // one more launch with CTA 0 recording where each of its roles waited (printed to stderr)
        DevBuf prof((41 + 2000) * sizeof(long long));
        prof.zero(nullptr);
        qstream_set_profile_buffer(prof.as<long long>());
        run();
        qstream_set_profile_buffer(nullptr);
        MK_CUDA(cudaDeviceSynchronize());
        std::vector<long long> hv(41 + 2000);
        prof.download(hv.data(), hv.size() * sizeof(long long));
        MK_CUDA(cudaDeviceSynchronize());
        const long long* h = hv.data();
        if (getenv("MACLLM_B200_QS_TRACE") != nullptr) {
            for (int role = 0; role < 5; ++role)
                for (long long k = 0; k < h[role * 8 + 6]; ++k) {
                    const long long e = h[41 + role * 400 + k];
                    fprintf(stderr, "[qstream trace] role %d ev %lld t %lld\n", role, (e >> 28) & 0xF, e & 0x0FFFFFFF);
                }
        }
        static const char* role[5] = {"weight loader", "mma issuer", "activation loader", "converter", "epilogue"};
        for (int r = 0; r < 5; ++r)
            fprintf(stderr, "[qstream prof] %-18s total %8lld  wait0 %8lld  wait1 %8lld  wait2 %8lld  wait3 %8lld  items %lld\n", role[r], h[r * 8],
                    h[r * 8 + 1], h[r * 8 + 2], h[r * 8 + 3], h[r * 8 + 4], h[r * 8 + 5]);
    }
    int32_t st = 0;
    ws.status.download(&st, 4);
    MK_CUDA(cudaDeviceSynchronize());
    if (st != 0) throw std::runtime_error("tensor-core matmul: a bounded wait inside the kernel gave up (status " + std::to_string(st) + ")");
    if (y != nullptr && (stream || half) && qs_splits > 1) {
        // the shares are added in share order, as the consumer kernels of the model do
        std::vector<float> parts((size_t)qs_splits * T * rows);
        qs_partial.download(parts.data(), parts.size() * 4);
        MK_CUDA(cudaDeviceSynchronize());
        const size_t n = (size_t)T * rows;
        for (size_t i = 0; i < n; ++i) {
            float v = parts[i];
            for (int sp = 1; sp < qs_splits; ++sp) v += parts[(size_t)sp * n + i];
            y[i] = v;
        }
    } else if (y != nullptr) dy.download(y, (size_t)T * rows * 4);
    MK_CUDA(cudaDeviceSynchronize());
}

}  // namespace

int32_t mk_k_qmatmul(int32_t type, const void* w, int64_t rows, int64_t cols, const float* x, int32_t T, float* y,
                     int32_t path) {
    return guarded([&] { qmatmul_case(type, w, rows, cols, x, T, y, path, 1, nullptr); });
}

int32_t mk_k_qmatmul_time(int32_t type, const void* w, int64_t rows, int64_t cols, const float* x, int32_t T, int32_t path,
                          int32_t iters, float* avg_ms) {
    return guarded([&] {
        if (iters <= 0 || avg_ms == nullptr) throw std::runtime_error("mk_k_qmatmul_time: iters must be positive and avg_ms non-null");
        qmatmul_case(type, w, rows, cols, x, T, nullptr, path, iters, avg_ms);
    });
}

int32_t mk_k_embed(int32_t type, const void* w, int64_t rows, int64_t cols, const uint32_t* ids, int32_t T, float scale,
                   float* out) {
    return guarded([&] {
        require_device();
        for (int i = 0; i < T; ++i)
            if ((int64_t)ids[i] >= rows) throw std::runtime_error("mk_k_embed: token id out of range");
        DeviceWeight dw;
        upload_weight(type, w, rows, cols, dw);
        DevBuf di((size_t)T * 4), dout((size_t)T * cols * 4);
        di.upload(ids, (size_t)T * 4);
        launch_embed(dw.w, di.as<uint32_t>(), T, scale, dout.as<float>(), nullptr);
        MK_CUDA(cudaDeviceSynchronize());
        dout.download(out, (size_t)T * cols * 4);
        MK_CUDA(cudaDeviceSynchronize());
    });
}

int32_t mk_k_actmul(const float* gate, const float* up, int32_t T, int32_t F, int32_t act, float* out) {
    return guarded([&] {
        require_device();
        size_t n = (size_t)T * F * 4;
        DevBuf dg(n), du(n), dout(n);
        dg.upload(gate, n);
        du.upload(up, n);
        launch_actmul_quant(dg.as<float>(), du.as<float>(), F, T, F, act, ACT_Q8K, ActQ{}, dout.as<float>(), nullptr);
        MK_CUDA(cudaDeviceSynchronize());
        dout.download(out, n);
        MK_CUDA(cudaDeviceSynchronize());
    });
}

int32_t mk_k_gated_ffn(int32_t type, const void* gate_w, const void* up_w, int64_t F, int64_t cols, const float* x, int32_t T,
                       int32_t act, float* out, int32_t iters, float* avg_ms) {
    return guarded([&] {
        require_device();
        DeviceWeight dg, du;
        upload_weight(type, gate_w, F, cols, dg);
        upload_weight(type, up_w, F, cols, du);
        if (!hgemm_tc_supported(dg.w)) throw std::runtime_error("mk_k_gated_ffn: the f16-image GEMM does not cover this matrix");
        HalfWeight image;
        build_half_weight_interleaved(dg.w, du.w, image, nullptr);
        int kind = act_kind_for(type);
        DevBuf dx((size_t)T * cols * 4), dy((size_t)T * F * 2);
        dx.upload(x, (size_t)T * cols * 4);
        ActBufs ab;
        ActQ a = ab.view(T, (int)cols, kind, true);
        NormQuantArgs na;
        na.h = dx.as<float>();
        na.rows = T;
        na.dim = (int)cols;
        na.act_kind = kind;
        na.out = a;
        launch_add_norm_quant(na, nullptr);
        DevBuf status(4);
        status.zero(nullptr);
        HgemmScratch hs;
        hs.status = status.as<int32_t>();
        auto run = [&] { launch_hgemm_tc_gated(image, a.xh, T, act, dy.as<__half>(), (int)F, hs, nullptr); };
        run();
        if (iters > 0 && avg_ms != nullptr) {
            DevBuf flush((size_t)256 << 20);  // larger than the L2
            cudaEvent_t e0, e1;
            MK_CUDA(cudaEventCreate(&e0));
            MK_CUDA(cudaEventCreate(&e1));
            double total = 0;
            for (int i = 0; i < iters + 2; ++i) {
                flush.zero(nullptr);
                MK_CUDA(cudaEventRecord(e0, nullptr));
                run();
                MK_CUDA(cudaEventRecord(e1, nullptr));
                MK_CUDA(cudaEventSynchronize(e1));
                float ms = 0;
                MK_CUDA(cudaEventElapsedTime(&ms, e0, e1));
                if (i >= 2) total += ms;
            }
            cudaEventDestroy(e0);
            cudaEventDestroy(e1);
            *avg_ms = (float)(total / iters);
        }
        MK_CUDA(cudaDeviceSynchronize());
        int32_t st = 0;
        status.download(&st, 4);
        MK_CUDA(cudaDeviceSynchronize());
        if (st != 0) throw std::runtime_error("tensor-core matmul: a bounded wait inside the kernel gave up (status " + std::to_string(st) + ")");
        if (out != nullptr) {
            std::vector<__half> h((size_t)T * F);
            dy.download(h.data(), h.size() * 2);
            MK_CUDA(cudaDeviceSynchronize());
            for (size_t i = 0; i < h.size(); ++i) out[i] = __half2float(h[i]);
        }
    });
}

int32_t mk_k_attention_step(const mk_attn_case* c) {
    return guarded([&] {
        require_device();
        const int T = c->total_tokens, lanes = c->lanes, d = c->head_dim;
        const int esz = c->kv_f16 ? 2 : 4;
        size_t pool_elems = (size_t)c->pool_blocks * c->layers * c->kv_heads * c->block_tokens * d;
        DevBuf kpool(pool_elems * esz), vpool(pool_elems * esz);
        kpool.upload(c->k_pool, pool_elems * esz);
        vpool.upload(c->v_pool, pool_elems * esz);
        size_t qn = (size_t)T * c->q_heads * d * 4, kn = (size_t)T * c->kv_heads * d * 4;
        DevBuf dq(qn), dk(kn), dv(kn), dout(qn);
        dq.upload(c->q, qn);
        dk.upload(c->k, kn);
        dv.upload(c->v, kn);

        std::vector<LaneHeader> hdr(lanes);
        int total_blocks = 0, tiles = 0;
        int q_tile = attention_q_tile(c->q_heads, c->kv_heads);
        for (int l = 0; l < lanes; ++l) {
            hdr[l].start_pos = c->start_pos[l];
            hdr[l].n_tokens = c->lane_len[l];
            hdr[l].table_off = c->table_off[l];
            hdr[l].n_blocks = c->table_len[l];
            total_blocks = std::max(total_blocks, c->table_off[l] + c->table_len[l]);
            tiles += (c->lane_len[l] + q_tile - 1) / q_tile;
        }
        DevBuf dhdr((size_t)lanes * sizeof(LaneHeader)), dtab((size_t)std::max(total_blocks, 1) * 4);
        dhdr.upload(hdr.data(), (size_t)lanes * sizeof(LaneHeader));
        dtab.upload(c->tables, (size_t)total_blocks * 4);
        DevBuf cu((size_t)(lanes + 1) * 4), pos((size_t)T * 4), tl((size_t)T * 4), slots((size_t)T * 8), last((size_t)lanes * 4),
            tile_lane((size_t)tiles * 4), tile_row((size_t)tiles * 4), ntiles(4), err(4);
        err.zero();
        BatchDesc b;
        b.lanes = lanes;
        b.T = T;
        b.max_tiles = tiles;
        b.hdr = dhdr.as<LaneHeader>();
        b.tables = dtab.as<uint32_t>();
        b.cu_seqlens = cu.as<int32_t>();
        b.positions = pos.as<int32_t>();
        b.token_lane = tl.as<int32_t>();
        b.slots = slots.as<int64_t>();
        b.last_index = last.as<int32_t>();
        b.tile_lane = tile_lane.as<int32_t>();
        b.tile_row0 = tile_row.as<int32_t>();
        b.n_tiles = ntiles.as<int32_t>();
        b.error_flag = err.as<int32_t>();
        launch_build_batch(b, c->block_tokens, q_tile, nullptr);

        DevBuf dcos, dsin, dqn, dkn;
        RopeKvArgs r;
        r.q = dq.as<float>();
        r.k = dk.as<float>();
        r.v = dv.as<float>();
        r.ldq = c->q_heads * d;
        r.ldk = r.ldv = c->kv_heads * d;
        if (c->q_norm_w) { dqn.upload(c->q_norm_w, (size_t)d * 4); r.q_norm_w = dqn.as<float>(); }
        if (c->k_norm_w) { dkn.upload(c->k_norm_w, (size_t)d * 4); r.k_norm_w = dkn.as<float>(); }
        r.norm_eps = c->norm_eps;
        if (c->cos_table && c->rotary_dim > 0) {
            size_t tn = (size_t)c->rope_capacity * (c->rotary_dim / 2) * 4;
            dcos.upload(c->cos_table, tn);
            dsin.upload(c->sin_table, tn);
            r.cos_t = dcos.as<float>();
            r.sin_t = dsin.as<float>();
            r.rotary_dim = c->rotary_dim;
        }
        r.positions = b.positions;
        r.slots = b.slots;
        r.k_pool = kpool.ptr();
        r.v_pool = vpool.ptr();
        r.kv_f16 = c->kv_f16;
        r.T = T;
        r.q_heads = c->q_heads;
        r.kv_heads = c->kv_heads;
        r.d = d;
        r.block_tokens = c->block_tokens;
        r.layers = c->layers;
        r.layer = c->layer;
        launch_rope_kv(r, nullptr);

        AttnArgs at;
        at.q = dq.as<float>();
        at.out = dout.as<float>();
        at.k_pool = kpool.ptr();
        at.v_pool = vpool.ptr();
        at.kv_f16 = c->kv_f16;
        at.batch = b;
        at.q_heads = c->q_heads;
        at.kv_heads = c->kv_heads;
        at.d = d;
        at.block_tokens = c->block_tokens;
        at.layers = c->layers;
        at.layer = c->layer;
        at.scale = c->scale;
        at.softcap = c->softcap;
        at.window = c->window;
        at.q_tile = q_tile;
        const bool tc_ok = attention_tc_supported(c->q_heads, c->kv_heads, d, c->block_tokens, c->kv_f16 != 0);
        if (c->kernel == 2 && !tc_ok) throw std::runtime_error("mk_k_attention_step: the tensor-core kernel does not cover this shape");
        if (c->kernel < 0 || c->kernel > 2) throw std::runtime_error("mk_k_attention_step: unknown kernel selector");
        DevBuf work, part_o, part_ml;
        if (tc_ok && c->kernel != 1) {
            AttnTcPlan plan;
            // the kernels address block tables through LaneHeader::table_off; the plan assumes tables packed in lane order
            for (int l = 0, off = 0; l < lanes; off += c->table_len[l], ++l)
                if (c->table_off[l] != off) throw std::runtime_error("mk_k_attention_step: block tables must be packed in lane order");
            plan_attention_tc(c->start_pos, c->lane_len, c->table_len, lanes, c->q_heads, c->kv_heads, plan);
            std::vector<int32_t> lists;
            lists.insert(lists.end(), plan.entries.begin(), plan.entries.end());
            lists.insert(lists.end(), plan.tiles.begin(), plan.tiles.end());
            lists.insert(lists.end(), plan.dec_lanes.begin(), plan.dec_lanes.end());
            work.alloc(std::max<size_t>(lists.size(), 1) * 4);
            if (!lists.empty()) work.upload(lists.data(), lists.size() * 4);
            part_o.alloc(std::max<size_t>((size_t)plan.n_entries() * c->kv_heads * 16 * d, 1) * 4);
            part_ml.alloc(std::max<size_t>((size_t)plan.n_entries() * c->kv_heads * 32, 1) * 4);
            AttnTcArgs ta;
            ta.q = at.q;
            ta.out = at.out;
            ta.k_pool = at.k_pool;
            ta.v_pool = at.v_pool;
            ta.hdr = b.hdr;
            ta.tables = b.tables;
            ta.cu_seqlens = b.cu_seqlens;
            ta.entries = work.as<int32_t>();
            ta.tiles = ta.entries + plan.entries.size();
            ta.dec_lanes = ta.tiles + plan.tiles.size();
            ta.n_tiles = plan.n_tiles();
            ta.n_entries = plan.n_entries();
            ta.n_dec_lanes = plan.n_dec_lanes();
            ta.part_o = part_o.as<float>();
            ta.part_ml = part_ml.as<float>();
            DevBuf counters((size_t)std::max(lanes, 1) * c->kv_heads * 4);
            counters.zero(nullptr);
            ta.counters = counters.as<int32_t>();
            ta.q_heads = c->q_heads;
            ta.kv_heads = c->kv_heads;
            ta.d = d;
            ta.block_tokens = c->block_tokens;
            ta.layers = c->layers;
            ta.layer = c->layer;
            ta.scale = c->scale;
            ta.softcap = c->softcap;
            ta.window = c->window;
            launch_paged_attention_tc(ta, nullptr);
        } else {
            launch_paged_attention(at, nullptr);
        }
        MK_CUDA(cudaDeviceSynchronize());

        int32_t flag = 0;
        err.download(&flag, 4);
        dout.download(c->out, qn);
        if (c->q_rot_out) dq.download(c->q_rot_out, qn);
        if (c->slots_out) slots.download(c->slots_out, (size_t)T * 8);
        if (c->positions_out) pos.download(c->positions_out, (size_t)T * 4);
        if (c->last_index_out) last.download(c->last_index_out, (size_t)lanes * 4);
        if (c->cu_seqlens_out) cu.download(c->cu_seqlens_out, (size_t)(lanes + 1) * 4);
        kpool.download(c->k_pool, pool_elems * esz);
        vpool.download(c->v_pool, pool_elems * esz);
        MK_CUDA(cudaDeviceSynchronize());
        if (flag != 0) throw std::runtime_error("mk_k_attention_step: batch descriptor index out of range (flag " + std::to_string(flag) + ")");
    });
}

namespace {

// cu_seqlens as the launchers want it: on the device, rising from 0 to the number of rows
int32_t checked_rows(const int32_t* cu, int32_t lanes, const char* what) {
    if (cu == nullptr || lanes <= 0 || cu[0] != 0) throw std::runtime_error(std::string(what) + ": lane boundaries must rise from 0 to the number of rows");
    for (int32_t l = 0; l < lanes; ++l)
        if (cu[l + 1] < cu[l]) throw std::runtime_error(std::string(what) + ": lane boundaries must rise from 0 to the number of rows");
    return cu[lanes];
}

}  // namespace

int32_t mk_k_gated_delta_decay(const float* alpha, const float* time_bias, const float* state_decay, int32_t tokens, int32_t heads, float* out) {
    return guarded([&] {
        require_device();
        if (tokens <= 0 || heads <= 0) throw std::runtime_error("Gated DeltaNet decay requires non-empty token and head dimensions");
        const size_t n = (size_t)tokens * heads * 4;
        DevBuf da(n), db((size_t)heads * 4), ds((size_t)heads * 4), dout(n);
        da.upload(alpha, n);
        db.upload(time_bias, (size_t)heads * 4);
        ds.upload(state_decay, (size_t)heads * 4);
        launch_gated_delta_decay(da.as<float>(), db.as<float>(), ds.as<float>(), tokens, heads, dout.as<float>(), nullptr);
        MK_CUDA(cudaDeviceSynchronize());
        dout.download(out, n);
        MK_CUDA(cudaDeviceSynchronize());
    });
}

int32_t mk_k_gated_delta_recurrence(const float* query, const float* key, const float* value, const float* decay, const float* beta,
                                    const int32_t* cu_seqlens, int32_t lanes, int32_t heads, int32_t key_dim, int32_t value_dim,
                                    const float* state_in, float* state_out, float* out) {
    return guarded([&] {
        require_device();
        if (heads <= 0 || key_dim <= 0 || value_dim <= 0) throw std::runtime_error("Gated DeltaNet decode has incompatible query/key geometry");
        const int32_t rows = checked_rows(cu_seqlens, lanes, "mk_k_gated_delta_recurrence");
        if (rows <= 0) throw std::runtime_error("mk_k_gated_delta_recurrence: no rows");
        const size_t qk = (size_t)rows * heads * key_dim * 4, vv = (size_t)rows * heads * value_dim * 4, ctl = (size_t)rows * heads * 4;
        const size_t st = (size_t)lanes * heads * key_dim * value_dim * 4;
        DevBuf dq(qk), dk(qk), dv(vv), dd(ctl), db(ctl), dcu((size_t)(lanes + 1) * 4), dsi(st), dso(st), dout(vv);
        dq.upload(query, qk);
        dk.upload(key, qk);
        dv.upload(value, vv);
        dd.upload(decay, ctl);
        db.upload(beta, ctl);
        dcu.upload(cu_seqlens, (size_t)(lanes + 1) * 4);
        dsi.upload(state_in, st);
        GatedDeltaArgs a;
        a.query = dq.as<float>(); a.key = dk.as<float>(); a.value = dv.as<float>(); a.decay = dd.as<float>(); a.beta = db.as<float>();
        a.cu = dcu.as<int32_t>(); a.state_in = dsi.as<float>(); a.state_out = dso.as<float>(); a.out = dout.as<float>();
        a.lanes = lanes; a.heads = heads; a.key_dim = key_dim; a.value_dim = value_dim;
        launch_gated_delta_recurrence(a, nullptr);
        MK_CUDA(cudaDeviceSynchronize());
        dso.download(state_out, st);
        dout.download(out, vv);
        MK_CUDA(cudaDeviceSynchronize());
    });
}

int32_t mk_k_mamba2_scan(const float* xbc, int64_t xbc_width, const float* raw_dt, const float* dt_bias, const float* a_decay, const float* d_skip,
                         const int32_t* cu_seqlens, int32_t lanes, int32_t heads, int32_t head_dim, int32_t state_size, const float* state_in,
                         float* state_out, float* out) {
    return guarded([&] {
        require_device();
        const int groups = mamba2_groups(xbc_width, heads, head_dim, state_size);
        const int32_t rows = checked_rows(cu_seqlens, lanes, "mk_k_mamba2_scan");
        if (rows <= 0) throw std::runtime_error("Mamba2 scan requires non-empty dimensions");
        const size_t xb = (size_t)rows * xbc_width * 4, dt = (size_t)rows * heads * 4, hv = (size_t)heads * 4;
        const size_t st = (size_t)lanes * heads * head_dim * state_size * 4, ob = (size_t)rows * heads * head_dim * 4;
        DevBuf dx(xb), ddt(dt), dbias(hv), da(hv), dd(hv), dcu((size_t)(lanes + 1) * 4), dsi(st), dso(st), dout(ob);
        dx.upload(xbc, xb);
        ddt.upload(raw_dt, dt);
        dbias.upload(dt_bias, hv);
        da.upload(a_decay, hv);
        dd.upload(d_skip, hv);
        dcu.upload(cu_seqlens, (size_t)(lanes + 1) * 4);
        dsi.upload(state_in, st);
        Mamba2Args m;
        m.xbc = dx.as<float>(); m.raw_dt = ddt.as<float>(); m.dt_bias = dbias.as<float>(); m.a = da.as<float>(); m.d = dd.as<float>();
        m.cu = dcu.as<int32_t>(); m.state_in = dsi.as<float>(); m.state_out = dso.as<float>(); m.out = dout.as<float>();
        m.lanes = lanes; m.heads = heads; m.head_dim = head_dim; m.state_size = state_size; m.groups = groups;
        launch_mamba2_scan(m, nullptr);
        MK_CUDA(cudaDeviceSynchronize());
        dso.download(state_out, st);
        dout.download(out, ob);
        MK_CUDA(cudaDeviceSynchronize());
    });
}

int32_t mk_k_short_conv(const float* bcx, const float* kernel, const int32_t* cu_seqlens, int32_t lanes, int32_t hidden, int32_t taps,
                        const float* tail_in, float* tail_out, float* out) {
    return guarded([&] {
        require_device();
        if (hidden <= 0 || taps < 1) throw std::runtime_error("short-convolution state geometry does not match its layer");
        const int32_t rows = checked_rows(cu_seqlens, lanes, "mk_k_short_conv");
        if (rows <= 0) throw std::runtime_error("mk_k_short_conv: no rows");
        const size_t xb = (size_t)rows * 3 * hidden * 4, kb = (size_t)hidden * taps * 4, ob = (size_t)rows * hidden * 4;
        const size_t tb = (size_t)lanes * (taps - 1) * hidden * 4;
        DevBuf dx(xb), dk(kb), dcu((size_t)(lanes + 1) * 4), dti(std::max<size_t>(tb, 4)), dto(std::max<size_t>(tb, 4)), dout(ob);
        dx.upload(bcx, xb);
        dk.upload(kernel, kb);
        dcu.upload(cu_seqlens, (size_t)(lanes + 1) * 4);
        if (tb > 0) dti.upload(tail_in, tb);
        ShortConvArgs c;
        c.bcx = dx.as<float>(); c.kernel = dk.as<float>(); c.cu = dcu.as<int32_t>(); c.tail_in = dti.as<float>(); c.tail_out = dto.as<float>();
        c.out = dout.as<float>(); c.rows = rows; c.lanes = lanes; c.hidden = hidden; c.K = taps;
        launch_short_conv(c, nullptr);
        MK_CUDA(cudaDeviceSynchronize());
        if (tb > 0) dto.download(tail_out, tb);
        dout.download(out, ob);
        MK_CUDA(cudaDeviceSynchronize());
    });
}

int32_t mk_k_recurrent_time(int32_t kind, int32_t lanes, int32_t rows_per_lane, int32_t heads, int32_t dim_a, int32_t dim_b, int32_t iters,
                            float* avg_ms, double* state_bytes) {
    return guarded([&] {
        require_device();
        if (kind < 0 || kind > 1 || lanes <= 0 || rows_per_lane <= 0 || heads <= 0 || dim_a <= 0 || dim_b <= 0 || iters <= 0 || avg_ms == nullptr)
            throw std::runtime_error("mk_k_recurrent_time: bad arguments");
        const int64_t rows = (int64_t)lanes * rows_per_lane;
        std::vector<int32_t> cu((size_t)lanes + 1);
        for (int l = 0; l <= lanes; ++l) cu[(size_t)l] = l * rows_per_lane;
        DevBuf dcu((size_t)(lanes + 1) * 4);
        dcu.upload(cu.data(), (size_t)(lanes + 1) * 4);
        const size_t st = (size_t)lanes * heads * dim_a * dim_b * 4;   // [key_dim][value_dim] or [head_dim][state_size] per (lane, head)
        DevBuf s0(st), s1(st);
        s0.zero(nullptr);
        s1.zero(nullptr);
        if (state_bytes != nullptr) *state_bytes = 2.0 * (double)st;   // read once, written once per launch
        cudaEvent_t e0, e1;
        MK_CUDA(cudaEventCreate(&e0));
        MK_CUDA(cudaEventCreate(&e1));
        float total = 0.f;
        auto timed = [&](auto&& launch) {
            for (int it = -3; it < iters; ++it) {   // three warm-up launches; the two state buffers change roles every launch
                const bool flip = (it & 1) != 0;
                MK_CUDA(cudaEventRecord(e0, nullptr));
                launch(flip ? s1.as<float>() : s0.as<float>(), flip ? s0.as<float>() : s1.as<float>());
                MK_CUDA(cudaEventRecord(e1, nullptr));
                MK_CUDA(cudaEventSynchronize(e1));
                float ms = 0.f;
                MK_CUDA(cudaEventElapsedTime(&ms, e0, e1));
                if (it >= 0) total += ms;
            }
        };
        if (kind == 0) {   // Gated DeltaNet: dim_a = key_dim, dim_b = value_dim
            const size_t qk = (size_t)rows * heads * dim_a * 4, vv = (size_t)rows * heads * dim_b * 4, ctl = (size_t)rows * heads * 4;
            DevBuf dq(qk), dk(qk), dv(vv), dd(ctl), db(ctl), dout(vv);
            for (DevBuf* b : {&dq, &dk, &dv, &dd, &db}) b->zero(nullptr);
            GatedDeltaArgs a;
            a.query = dq.as<float>(); a.key = dk.as<float>(); a.value = dv.as<float>(); a.decay = dd.as<float>(); a.beta = db.as<float>();
            a.cu = dcu.as<int32_t>(); a.out = dout.as<float>(); a.lanes = lanes; a.heads = heads; a.key_dim = dim_a; a.value_dim = dim_b;
            timed([&](const float* in, float* out) { a.state_in = in; a.state_out = out; launch_gated_delta_recurrence(a, nullptr); });
        } else {           // Mamba2: dim_a = head_dim, dim_b = state_size, one group
            const int64_t width = (int64_t)heads * dim_a + 2 * (int64_t)dim_b;
            const size_t xb = (size_t)rows * width * 4, dt = (size_t)rows * heads * 4, hv = (size_t)heads * 4, ob = (size_t)rows * heads * dim_a * 4;
            DevBuf dx(xb), ddt(dt), dbias(hv), da(hv), dd(hv), dout(ob);
            for (DevBuf* b : {&dx, &ddt, &dbias, &da, &dd}) b->zero(nullptr);
            Mamba2Args m;
            m.xbc = dx.as<float>(); m.raw_dt = ddt.as<float>(); m.dt_bias = dbias.as<float>(); m.a = da.as<float>(); m.d = dd.as<float>();
            m.cu = dcu.as<int32_t>(); m.out = dout.as<float>(); m.lanes = lanes; m.heads = heads; m.head_dim = dim_a; m.state_size = dim_b; m.groups = 1;
            timed([&](const float* in, float* out) { m.state_in = in; m.state_out = out; launch_mamba2_scan(m, nullptr); });
        }
        MK_CUDA(cudaEventDestroy(e0));
        MK_CUDA(cudaEventDestroy(e1));
        *avg_ms = total / (float)iters;
    });
}

int32_t mk_k_argmax(const float* logits, int32_t B, int32_t vocab, uint32_t* out) {
    return guarded([&] {
        require_device();
        DevBuf dl((size_t)B * vocab * 4), dout((size_t)B * 4);
        dl.upload(logits, (size_t)B * vocab * 4);
        DevBuf scratch(argmax_scratch_bytes(B));
        scratch.zero(nullptr);
        launch_argmax(dl.as<float>(), B, vocab, dout.as<uint32_t>(), scratch.ptr(), nullptr);
        MK_CUDA(cudaDeviceSynchronize());
        dout.download(out, (size_t)B * 4);
        MK_CUDA(cudaDeviceSynchronize());
    });
}

int32_t mk_k_grouped_qmatmul(int32_t type, const void* w, const void* up_w, int32_t experts, int64_t rows_pe, int64_t cols, const float* x,
                             const int32_t* offsets, float* y, int32_t path, int32_t act) {
    return guarded([&] {
        require_device();
        if (experts <= 0 || rows_pe <= 0 || cols <= 0 || offsets == nullptr) throw std::runtime_error("mk_k_grouped_qmatmul: bad arguments");
        const int P = offsets[experts];
        int most = 0;
        for (int e = 0; e < experts; ++e) {
            if (offsets[e + 1] < offsets[e]) throw std::runtime_error("mk_k_grouped_qmatmul: row ranges must not decrease");
            most = std::max(most, offsets[e + 1] - offsets[e]);
        }
        if (P <= 0) return;
        const bool gated = up_w != nullptr;
        if (gated && path != MK_PATH_STREAM) throw std::runtime_error("mk_k_grouped_qmatmul: the gated form exists on the streamed path only");
        const int64_t rb = gguf_row_bytes(type, cols);
        DeviceWeight bank;
        if (!gated) {
            upload_weight(type, w, rows_pe * experts, cols, bank);
        } else {
            // [gate bank; up bank] in one buffer, as the model stacks them
            std::vector<uint8_t> both((size_t)(2 * rows_pe * experts * rb));
            memcpy(both.data(), w, both.size() / 2);
            memcpy(both.data() + both.size() / 2, up_w, both.size() / 2);
            upload_weight(type, both.data(), 2 * rows_pe * experts, cols, bank);
        }
        int kind = act_kind_for(type);
        DevBuf dx((size_t)P * cols * 4), dy((size_t)P * rows_pe * 4), doff((size_t)(experts + 1) * 4), status(4);
        dx.upload(x, (size_t)P * cols * 4);
        doff.upload(offsets, (size_t)(experts + 1) * 4);
        status.zero(nullptr);
        ActBufs ab;
        ActQ a = ab.view(P, (int)cols, kind, path == MK_PATH_STREAM);
        NormQuantArgs na;
        na.h = dx.as<float>();
        na.rows = P;
        na.dim = (int)cols;
        na.act_kind = kind;
        na.out = a;
        launch_add_norm_quant(na, nullptr);
        if (path == MK_PATH_GEMV) {
            QWeight one = bank.w;
            one.rows = rows_pe;
            launch_qgemv_grouped(one, experts, doff.as<int32_t>(), nullptr, a, dy.as<float>(), (int)rows_pe, nullptr);
        } else if (path == MK_PATH_STREAM) {
            if (type != MK_TYPE_Q4_K && !(type == MK_TYPE_Q6_K && !gated)) throw std::runtime_error("mk_k_grouped_qmatmul: the streamed path covers Q4_K (and Q6_K when not gated)");
            QStreamWeight qsw;
            if (type == MK_TYPE_Q4_K) build_qstream_weight(bank.w.p0, bank.w.rows, cols, qsw, nullptr, gated ? rows_pe * experts : 0);
            else build_qstream_weight_q6k(bank.w, qsw, nullptr);
            DevBuf yh;
            if (gated) yh.alloc((size_t)P * rows_pe * 2);
            launch_qstream_tc_grouped(qsw, experts, doff.as<int32_t>(), a.xh, P, most, dy.as<float>(), (int)rows_pe, status.as<int32_t>(), nullptr,
                                      gated ? act : -1, gated ? yh.as<__half>() : nullptr, (int)rows_pe);
            MK_CUDA(cudaDeviceSynchronize());
            if (gated) {
                std::vector<uint16_t> h((size_t)P * rows_pe);
                yh.download(h.data(), h.size() * 2);
                MK_CUDA(cudaDeviceSynchronize());
                for (size_t i = 0; i < h.size(); ++i) y[i] = __half2float(__ushort_as_half(h[i]));
            }
        } else {
            throw std::runtime_error("mk_k_grouped_qmatmul: path must be the integer GEMV or the streamed kernel");
        }
        MK_CUDA(cudaDeviceSynchronize());
        int32_t st = 0;
        status.download(&st, 4);
        if (!(gated && path == MK_PATH_STREAM)) dy.download(y, (size_t)P * rows_pe * 4);
        MK_CUDA(cudaDeviceSynchronize());
        if (st != 0) throw std::runtime_error("grouped matmul: a bounded wait inside the kernel gave up (status " + std::to_string(st) + ")");
    });
}

int32_t mk_k_ep_exchange_emulated(int32_t ranks, int32_t local_experts, int32_t hidden, int32_t cap_rows, const uint16_t* rows,
                                  const int32_t* offsets, int32_t exchanges, int32_t silent_rank, int64_t wait_ns, float* results,
                                  int32_t* merged_ranges, int32_t* status) {
    return guarded([&] {
        require_device();
        if (ranks < 1 || ranks > kEpMaxRanks || local_experts < 1 || local_experts > 128 || hidden <= 0 || hidden % 8 != 0 || cap_rows <= 0 ||
            exchanges < 1 || rows == nullptr || offsets == nullptr || results == nullptr || merged_ranges == nullptr || status == nullptr)
            throw std::runtime_error("mk_k_ep_exchange_emulated: bad arguments");
        const int N = ranks, EL = local_experts, E = N * EL;
        for (int r = 0; r < N; ++r) {
            const int32_t* o = offsets + (size_t)r * (E + 1);
            if (o[0] != 0 || o[E] > cap_rows) throw std::runtime_error("mk_k_ep_exchange_emulated: row ranges start at 0 and fit cap_rows");
            for (int e = 0; e < E; ++e)
                if (o[e + 1] < o[e]) throw std::runtime_error("mk_k_ep_exchange_emulated: row ranges must not decrease");
        }
        // the blocks of all ranks live on this device; every rank's view of them is the same table with its own rank
        auto up = [](int64_t v) { return (v + 255) / 256 * 256; };
        EpDispatch d0;
        d0.ranks = N;
        d0.local_experts = EL;
        d0.hidden = hidden;
        d0.cap_rows = cap_rows;
        int64_t at = 0;
        d0.rows_in_off = at;
        at = up(at + (int64_t)2 * N * cap_rows * hidden * 2);
        d0.off_in_off = at;
        at = up(at + (int64_t)2 * N * (EL + 1) * 4);
        d0.flag_in_off = at;
        at = up(at + (int64_t)2 * N * 4);
        d0.out_back_off = at;
        at = up(at + (int64_t)2 * cap_rows * hidden * 4);
        d0.flag_back_off = at;
        at = up(at + (int64_t)2 * N * 4);
        std::vector<DevBuf> block((size_t)N), x((size_t)N), off((size_t)N), merged((size_t)N), out((size_t)N), comb((size_t)N), start((size_t)N),
            done((size_t)N), st((size_t)N);
        for (int r = 0; r < N; ++r) {
            block[(size_t)r].alloc((size_t)at);
            block[(size_t)r].zero(nullptr);
            d0.base[r] = block[(size_t)r].as<uint8_t>();
            x[(size_t)r].alloc((size_t)cap_rows * hidden * 2);
            x[(size_t)r].upload(rows + (size_t)r * cap_rows * hidden, (size_t)cap_rows * hidden * 2);
            off[(size_t)r].alloc((size_t)(E + 1) * 4);
            off[(size_t)r].upload(offsets + (size_t)r * (E + 1), (size_t)(E + 1) * 4);
            merged[(size_t)r].alloc((size_t)N * cap_rows * hidden * 2);
            out[(size_t)r].alloc((size_t)N * cap_rows * hidden * 4);
            comb[(size_t)r].alloc((size_t)(EL + 1) * 4);
            comb[(size_t)r].zero(nullptr);
            start[(size_t)r].alloc((size_t)N * EL * 4);
            start[(size_t)r].zero(nullptr);
            done[(size_t)r].alloc((size_t)2 * kEpMaxRanks * 4);
            done[(size_t)r].zero(nullptr);
            st[(size_t)r].alloc(4);
            st[(size_t)r].zero(nullptr);
        }
        MK_CUDA(cudaDeviceSynchronize());
        auto view = [&](int r) { EpDispatch d = d0; d.rank = r; return d; };
        // one stream, stage by stage over all ranks: every flag a kernel waits for was published by an earlier launch (or,
        // for the silent rank, never is - those waits run out after wait_ns and leave their status code)
        const uint64_t wns = wait_ns > 0 ? (uint64_t)wait_ns : kEpWaitNs;
        for (uint32_t epoch = 1; epoch <= (uint32_t)exchanges; ++epoch) {
            for (int r = 0; r < N; ++r)
                if (r != silent_rank) launch_ep_dispatch(x[(size_t)r].as<__half>(), off[(size_t)r].as<int32_t>(), view(r), epoch, done[(size_t)r].as<int32_t>(), st[(size_t)r].as<int32_t>(), nullptr);
            for (int r = 0; r < N; ++r)
                if (r != silent_rank)
                    launch_ep_regroup(view(r), epoch, merged[(size_t)r].as<__half>(), comb[(size_t)r].as<int32_t>(), start[(size_t)r].as<int32_t>(), st[(size_t)r].as<int32_t>(), nullptr, wns);
            if (silent_rank >= 0) break;  // the ranks that waited hold empty ranges and their status; nothing to return
            for (int r = 0; r < N; ++r)
                launch_ep_scale_rows(merged[(size_t)r].as<__half>(), comb[(size_t)r].as<int32_t>(), EL, r * EL, hidden, out[(size_t)r].as<float>(), nullptr);
            for (int r = 0; r < N; ++r)
                launch_ep_return(out[(size_t)r].as<float>(), start[(size_t)r].as<int32_t>(), view(r), epoch, done[(size_t)r].as<int32_t>() + kEpMaxRanks, nullptr);
            for (int r = 0; r < N; ++r) launch_ep_wait_back(view(r), epoch, st[(size_t)r].as<int32_t>(), nullptr, wns);
        }
        MK_CUDA(cudaDeviceSynchronize());
        const uint32_t last = silent_rank >= 0 ? 1u : (uint32_t)exchanges;
        for (int r = 0; r < N; ++r) {
            EpDispatch d = view(r);
            MK_CUDA(cudaMemcpy(results + (size_t)r * cap_rows * hidden, ep_result_area(d, last), (size_t)cap_rows * hidden * 4, cudaMemcpyDeviceToHost));
            comb[(size_t)r].download(merged_ranges + (size_t)r * (EL + 1), (size_t)(EL + 1) * 4);
            st[(size_t)r].download(status + r, 4);
        }
        MK_CUDA(cudaDeviceSynchronize());
    });
}

int32_t mk_k_penalties(float* logits, int32_t vocab, const uint32_t* history, int32_t n_history, float repetition_penalty,
                       const uint32_t* generated, int32_t n_generated, float presence_penalty, float frequency_penalty) {
    return guarded([&] {
        apply_penalties(logits, vocab, history, n_history, repetition_penalty, generated, n_generated, presence_penalty, frequency_penalty);
    });
}

int32_t mk_k_sample(const float* logits, int32_t B, int32_t vocab, const mk_lane_sampling* settings, int32_t where, uint32_t* out) {
    return guarded([&] {
        if (B <= 0 || vocab <= 0 || logits == nullptr || settings == nullptr || out == nullptr) throw std::runtime_error("mk_k_sample: bad arguments");
        if (where == 0) {
            for (int32_t r = 0; r < B; ++r) {
                const float* row = logits + (int64_t)r * vocab;
                const mk_lane_sampling& s = settings[r];
                out[r] = s.temperature > 0.f ? sample_top_k_top_p(row, vocab, s.temperature, s.top_k, s.top_p, s.u) : (uint32_t)argmax_first(row, vocab);
            }
            return;
        }
        require_device();
        std::vector<LaneSampling> ls((size_t)B);
        for (int32_t r = 0; r < B; ++r) {
            if (!device_sampling_covers(settings[r].temperature, settings[r].top_k, vocab))
                throw std::runtime_error("mk_k_sample: the device sampler covers greedy selection and 1 <= top_k <= 1024");
            ls[(size_t)r] = LaneSampling{settings[r].temperature, settings[r].top_k, settings[r].top_p, settings[r].u};
        }
        DevBuf dl((size_t)B * vocab * 4), dp((size_t)B * sizeof(LaneSampling)), dout((size_t)B * 4), status(4);
        dl.upload(logits, (size_t)B * vocab * 4);
        dp.upload(ls.data(), ls.size() * sizeof(LaneSampling));
        status.zero(nullptr);
        launch_sample(dl.as<float>(), B, vocab, dp.as<LaneSampling>(), dout.as<uint32_t>(), status.as<int32_t>(), nullptr);
        MK_CUDA(cudaDeviceSynchronize());
        dout.download(out, (size_t)B * 4);
        int32_t st = 0;
        status.download(&st, 4);
        MK_CUDA(cudaDeviceSynchronize());
        if ((st & 0xFFFF0000) == kSampleEmptyStatus) throw std::runtime_error("sampling distribution is empty (row " + std::to_string(st & 0xFFFF) + ")");
    });
}

int32_t mk_k_moe_route(const float* logits, int32_t T, int32_t experts, int32_t k, int32_t* sel_experts, float* sel_weights) {
    return guarded([&] {
        require_device();
        if (T <= 0 || experts <= 0) throw std::runtime_error("mk_k_moe_route: bad arguments");
        if (k <= 0 || k > experts) throw std::runtime_error("experts per token " + std::to_string(k) + " must be in 1..=" + std::to_string(experts));  // src/decoder.rs:456-458
        DevBuf dl((size_t)T * experts * 4), de((size_t)T * k * 4), dw((size_t)T * k * 4);
        dl.upload(logits, (size_t)T * experts * 4);
        DevBuf status(4);
        status.zero(nullptr);
        launch_moe_route(dl.as<float>(), T, experts, k, de.as<int32_t>(), dw.as<float>(), status.as<int32_t>(), nullptr);
        MK_CUDA(cudaDeviceSynchronize());
        de.download(sel_experts, (size_t)T * k * 4);
        dw.download(sel_weights, (size_t)T * k * 4);
        int32_t st = 0;
        status.download(&st, 4);
        MK_CUDA(cudaDeviceSynchronize());
        // the choices are written (in range) even for a refused row, so a caller can inspect them
        if ((st & 0xFFFF0000) == kMoeRouteStatus) throw std::runtime_error("router produced non-finite logits for token row " + std::to_string(st & 0xFFFF));
    });
}

int32_t mk_k_matmul_plan(int32_t path, int64_t rows, int64_t cols, int32_t T, int32_t max_splits, int64_t* out8) {
    return guarded([&] {
        if (rows <= 0 || cols <= 0 || T <= 0 || out8 == nullptr) throw std::runtime_error("mk_k_matmul_plan: arguments out of range");
        if (path == MK_PATH_HALF) {
            if (cols % 64 != 0) throw std::runtime_error("mk_k_matmul_plan: the f16-image GEMM needs columns in multiples of 64");
            HgemmPlan p = hgemm_tc_plan(rows, cols, T, max_splits);
            const int64_t v[8] = {p.bn, p.row_tiles, p.n_tiles, p.splits, p.kb_per_split, (int64_t)p.partial_floats, 0, 0};
            memcpy(out8, v, sizeof v);
        } else if (path == MK_PATH_STREAM) {
            if (cols % 256 != 0 || T > kQStreamMaxRows) throw std::runtime_error("mk_k_matmul_plan: the streamed matmul covers 256-wide blocks and at most 64 rows");
            QStreamPlan p = qstream_plan((int)((rows + 127) / 128), (int)(cols / 256), rows, T, max_splits, false);
            const int64_t v[8] = {p.bn, p.row_tiles, p.items, p.ctas, p.slots, (int64_t)p.partial_floats, p.R, p.groups};
            memcpy(out8, v, sizeof v);
        } else {
            throw std::runtime_error("mk_k_matmul_plan: only the f16-image and the streamed path are planned on the host");
        }
    });
}

int32_t mk_k_attention_plan(const int32_t* start_pos, const int32_t* n_tokens, int32_t lanes, int32_t q_heads, int32_t kv_heads,
                            int32_t block_tokens, int32_t* shares_out, int32_t* tiles_out, int32_t* max_entries_out) {
    return guarded([&] {
        if (lanes <= 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0 || block_tokens <= 0)
            throw std::runtime_error("mk_k_attention_plan: arguments out of range");
        std::vector<int32_t> n_blocks((size_t)lanes);
        for (int i = 0; i < lanes; ++i) n_blocks[(size_t)i] = (start_pos[i] + n_tokens[i] + block_tokens - 1) / block_tokens;
        AttnTcPlan plan;
        plan_attention_tc(start_pos, n_tokens, n_blocks.data(), lanes, q_heads, kv_heads, plan);
        for (int i = 0; i < lanes; ++i) shares_out[i] = 0;
        for (int e = 0; e < plan.n_entries(); ++e) shares_out[plan.entries[(size_t)e * 8]] = plan.entries[(size_t)e * 8 + 2];
        *tiles_out = plan.n_tiles();
        *max_entries_out = attention_tc_max_entries(lanes, kv_heads);
        if (plan.n_entries() > *max_entries_out) throw std::runtime_error("mk_k_attention_plan: the plan exceeds its own bound");
    });
}

int32_t mk_k_moe_combine_exchange(const float* expert_out, const int32_t* sel, const float* weights, int32_t T, int32_t k,
                                  int32_t hidden, int32_t e_lo, int32_t e_hi, int32_t ranks, int32_t rank, const float* peer_rows,
                                  int32_t deliver, int32_t wait_ms, int32_t epochs, float* out, float* pushed, int32_t* status_out) {
    return guarded([&] {
        require_device();
        if (ranks < 2 || ranks > kEpMaxRanks || rank < 0 || rank >= ranks || T <= 0 || epochs <= 0 || wait_ms <= 0 || wait_ms > 2000)
            throw std::runtime_error("mk_k_moe_combine_exchange: arguments out of range");
        const size_t pairs = (size_t)T * k, row_floats = (size_t)T * hidden;
        DevBuf d_eo(pairs * hidden * 4), d_sel(pairs * 4), d_w(pairs * 4), d_pos(pairs * 4), d_out(row_floats * 4), d_status(4);
        d_eo.upload(expert_out, pairs * hidden * 4);
        d_sel.upload(sel, pairs * 4);
        d_w.upload(weights, pairs * 4);
        std::vector<int32_t> pos(pairs);
        for (size_t i = 0; i < pairs; ++i) pos[i] = (int32_t)i;
        d_pos.upload(pos.data(), pairs * 4);
        d_status.zero(nullptr);
        // every rank's block, laid out as EpComm::open_exchange does: gather [2][ranks][T*hidden] floats, then flags [2][ranks][T]
        const size_t gather_bytes = (size_t)2 * ranks * row_floats * 4, flag_bytes = (size_t)2 * ranks * T * 4;
        std::vector<DevBuf> blocks((size_t)ranks);
        EpPeers peers;
        peers.rank = rank;
        peers.ranks = ranks;
        peers.max_tokens = T;
        peers.slot_floats = (int64_t)row_floats;
        for (int r = 0; r < ranks; ++r) {
            blocks[(size_t)r].alloc(gather_bytes + flag_bytes);
            blocks[(size_t)r].zero(nullptr);
            peers.gather[r] = blocks[(size_t)r].as<float>();
            peers.flags[r] = reinterpret_cast<uint32_t*>(static_cast<char*>(blocks[(size_t)r].ptr()) + gather_bytes);
        }
        MK_CUDA(cudaDeviceSynchronize());
        for (int e = 1; e <= epochs; ++e) {
            const int buf = e & 1;
            if (deliver != 0) {
                std::vector<uint32_t> flags((size_t)T, (uint32_t)e);
                for (int r = 0; r < ranks; ++r) {
                    if (r == rank) continue;
                    MK_CUDA(cudaMemcpy(peers.gather[rank] + ((size_t)buf * ranks + r) * row_floats, peer_rows + (size_t)r * row_floats,
                                       row_floats * 4, cudaMemcpyHostToDevice));
                    MK_CUDA(cudaMemcpy(peers.flags[rank] + ((size_t)buf * ranks + r) * T, flags.data(), (size_t)T * 4, cudaMemcpyHostToDevice));
                }
            }
            launch_moe_combine_exchange(d_eo.as<float>(), d_sel.as<int32_t>(), d_w.as<float>(), d_pos.as<int32_t>(), T, k, hidden, e_lo,
                                        e_hi, peers, (uint32_t)e, d_out.as<float>(), d_status.as<int32_t>(), nullptr,
                                        (uint64_t)wait_ms * 1000000ull);
            MK_CUDA(cudaDeviceSynchronize());
        }
        d_out.download(out, row_floats * 4);
        d_status.download(status_out, 4);
        const int buf = epochs & 1;
        for (int r = 0; r < ranks; ++r)
            MK_CUDA(cudaMemcpy(pushed + (size_t)r * row_floats, peers.gather[r] + ((size_t)buf * ranks + rank) * row_floats, row_floats * 4,
                               cudaMemcpyDeviceToHost));
        MK_CUDA(cudaDeviceSynchronize());
    });
}

}  // extern "C"
