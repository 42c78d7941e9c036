"""Parity of the sm_100a kernels against the CPU oracle, through the C ABI (needs a GPU)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

QTYPES = {"q4_k": 12, "q6_k": 14, "q8_0": 8}


@pytest.fixture(scope="module")
def ops(mk):
    import importlib
    return importlib.import_module("macllm_infer_b200.ops")


def _weights(ops, qtype, rows, cols, stream=1):
    return ops.seed_tensor(0, stream, 0.02, qtype, rows, cols)


@pytest.mark.parametrize("kind", [0, 1])
def test_quantize_bit_exact(ops, orc, kind):
    rng = np.random.default_rng(1)
    x = rng.standard_normal((7, 1024)).astype(np.float32)
    x[2, 256:512] = 0.0                      # an all-zero block
    x[3, 5] = -x[3, 9]                       # a sign tie on the block maximum
    x[3, 5] = abs(x[3]).max() + 1.0
    x[3, 9] = -x[3, 5]
    qs, d, bs = ops.quantize(x, kind)
    if kind == 0:
        oq, od, ob = orc.quantize_q8k(x)
        assert np.array_equal(bs, ob)
    else:
        oq, od = orc.quantize_q80(x)
    assert np.array_equal(qs, oq)
    assert np.array_equal(d, od)


@pytest.mark.parametrize("name", list(QTYPES))
@pytest.mark.parametrize("T", [1, 3, 8, 19])
def test_qgemv_matches_oracle(ops, orc, name, T):
    qtype = QTYPES[name]
    rows, cols = 384, 2048
    w = _weights(ops, qtype, rows, cols)
    rng = np.random.default_rng(T)
    x = rng.standard_normal((T, cols)).astype(np.float32)
    got = ops.qmatmul(qtype, w, rows, cols, x, 1)
    want = orc.qmatmul(qtype, w, rows, cols, x, 1)
    # integer block dots are exact; only the f32 accumulation order over blocks differs
    assert np.max(np.abs(got - want)) <= 2e-5 * max(1.0, np.max(np.abs(want)))


@pytest.mark.parametrize("name", list(QTYPES))
@pytest.mark.parametrize("T,rows,cols", [(9, 128, 256), (40, 300, 1024), (64, 2048, 2048), (130, 512, 5632), (257, 256, 768)])
def test_qgemm_tensor_matches_oracle(ops, orc, name, T, rows, cols):
    qtype = QTYPES[name]
    w = _weights(ops, qtype, rows, cols, stream=3)
    rng = np.random.default_rng(T + rows)
    x = rng.standard_normal((T, cols)).astype(np.float32)
    got = ops.qmatmul(qtype, w, rows, cols, x, 2)
    want = orc.qmatmul(qtype, w, rows, cols, x, 1)
    # operands rounded once to f16 (rel 2^-11 each), f32 accumulation
    scale = np.sqrt(cols) * 0.02
    assert np.max(np.abs(got - want)) <= 2e-3 * scale
    cos = float((got * want).sum() / np.sqrt((got * got).sum() * (want * want).sum()))
    assert cos >= 0.999999


@pytest.mark.parametrize("name", list(QTYPES))
@pytest.mark.parametrize("T,rows,cols", [(9, 128, 256), (40, 2048, 2048), (64, 512, 5632), (100, 300, 1024), (130, 300, 1024),
                                          (257, 2048, 2048), (700, 512, 5632), (2048, 1152, 768)])
def test_f16_image_gemm_matches_oracle(ops, orc, name, T, rows, cols):
    """The wide-batch path: weights rounded once to f16 at load time, TMA-fed tcgen05 GEMM.  Ragged edges on
    purpose: T and rows that are not multiples of the tile, several K blocks, more tiles than SMs."""
    qtype = QTYPES[name]
    w = _weights(ops, qtype, rows, cols, stream=4)
    rng = np.random.default_rng(T + rows)
    x = rng.standard_normal((T, cols)).astype(np.float32)
    got = ops.qmatmul(qtype, w, rows, cols, x, 3)
    want = orc.qmatmul(qtype, w, rows, cols, x, 1)
    assert np.isfinite(got).all()
    # both operands rounded once to f16 (rel 2^-11 each), f32 accumulation
    scale = np.sqrt(cols) * 0.02
    assert np.max(np.abs(got - want)) <= 2e-3 * scale
    cos = float((got * want).sum() / np.sqrt((got * got).sum() * (want * want).sum()))
    assert cos >= 0.999999
    # against the in-kernel dequant path the only difference is how the weight was rounded
    other = ops.qmatmul(qtype, w, rows, cols, x, 2)
    assert np.max(np.abs(got - other)) <= 2e-3 * scale


@pytest.mark.parametrize("name", list(QTYPES))
@pytest.mark.parametrize("act", [0, 1])
@pytest.mark.parametrize("T,F,cols", [(9, 64, 256), (40, 96, 1024), (100, 1024, 2048), (257, 300, 1024), (301, 2048, 512), (2048, 672, 768)])
def test_gated_gemm_equals_gemm_then_activation(ops, orc, name, act, T, F, cols):
    """The wide-tick feed-forward front: gate and up rows interleaved in one f16 image, the activation and the product
    finished in the GEMM's epilogue and written as f16.  Against the separate kernels (plain f16-image GEMM of each
    matrix, then the SwiGLU kernel) the accumulators and the activation arithmetic are the same, so the halves must
    be identical (above 64 rows, where neither side splits K); against the oracle the usual f16-operand tolerance applies.  Odd T, F with a partial last tile."""
    qtype = QTYPES[name]
    gate_w = _weights(ops, qtype, F, cols, stream=7)
    up_w = _weights(ops, qtype, F, cols, stream=8)
    rng = np.random.default_rng(T + F)
    x = rng.standard_normal((T, cols)).astype(np.float32)
    got = ops.gated_ffn(qtype, gate_w, up_w, F, cols, x, act)
    g = ops.qmatmul(qtype, gate_w, F, cols, x, 3)
    u = ops.qmatmul(qtype, up_w, F, cols, x, 3)
    want = ops.actmul(g, u, act).astype(np.float16).astype(np.float32)
    if T > 64:
        assert np.array_equal(got, want)
    else:
        # up to 64 rows the plain GEMM shares K out over CTAs and adds the shares afterwards: another association
        assert np.allclose(got, want, rtol=4e-3, atol=2e-4)
    og = orc.qmatmul(qtype, gate_w, F, cols, x, 1)
    ou = orc.qmatmul(qtype, up_w, F, cols, x, 1)
    ref = orc.act_mul(og, ou, act)
    # gate and up each carry the f16-operand error of the GEMM (2e-3 * scale); the product adds them, then one f16 rounding
    scale = np.sqrt(cols) * 0.02
    assert np.max(np.abs(got - ref)) <= 2e-3 * scale * (2 * np.max(np.abs(og)) + np.max(np.abs(ou)) + 1)


@pytest.mark.parametrize("splits", [16, 1])
@pytest.mark.parametrize("name,T,rows,cols", [("q4_k", 9, 128, 256), ("q4_k", 33, 300, 1024), ("q4_k", 64, 2048, 2048), ("q4_k", 64, 512, 5632),
                                               ("q4_k", 40, 2560, 2048), ("q4_k", 64, 1000, 11008), ("q4_k", 17, 22016, 2048), ("q4_k", 4, 2048, 2048),
                                               ("q4_k", 16, 3000, 2048), ("q6_k", 9, 128, 256), ("q6_k", 64, 512, 2048), ("q6_k", 33, 1000, 1024),
                                               ("q6_k", 2, 3072, 2048), ("q4_k", 1, 2048, 2048), ("q4_k", 1, 12288, 4096), ("q6_k", 1, 1000, 1024)])
def test_streamed_matmul_matches_oracle(ops, orc, monkeypatch, name, T, rows, cols, splits):
    """The decode-tick path: raw Q4_K / Q6_K units by bulk copy, dequantised by the converter warps straight into tensor
    memory, tcgen05 MMA with A from tensor memory.  Ragged row counts, one to 43 block columns, token tiles of 16 / 32 /
    64, with the work cut into partial-sum slots (16) and with whole groups of row tiles per CTA (1)."""
    qtype = QTYPES[name]
    monkeypatch.setenv("MACLLM_B200_QS_SPLITS", str(splits))
    w = _weights(ops, qtype, rows, cols, stream=6)
    rng = np.random.default_rng(T + rows)
    x = rng.standard_normal((T, cols)).astype(np.float32)
    got = ops.qmatmul(qtype, w, rows, cols, x, 4)
    want = orc.qmatmul(qtype, w, rows, cols, x, 1)
    assert np.isfinite(got).all()
    # the f16 weight carries two roundings (Q4_K: the product sc*q*d and dmin*m; Q6_K: d*sc and the product), the
    # activations one: a little wider than the f16-image GEMM's single rounding per weight
    scale = np.sqrt(cols) * 0.02
    assert np.max(np.abs(got - want)) <= 3e-3 * scale
    cos = float((got * want).sum() / np.sqrt((got * got).sum() * (want * want).sum()))
    assert cos >= 0.999999


@pytest.mark.parametrize("label,T,rows,cols,path", [("decode_gate_up", 64, 22016, 2048, 4), ("decode_down", 64, 2048, 11008, 4),
                                                     ("decode_qkv_image", 64, 3072, 2048, 3), ("decode_down_image", 64, 2048, 11008, 3),
                                                     ("prefill_gate_up", 2048, 22016, 2048, 3), ("prefill_down", 2048, 2048, 11008, 3)])
def test_matmul_timing_entry_on_the_benchmark_shapes(ops, label, T, rows, cols, path):
    """mk_k_qmatmul_time on the feed-forward matrices of the headline workload (device-resident operands, L2
    flushed before every launch): the launch must take a sane, positive time.  Also the command the profiler
    captures of these two GEMM kernels run."""
    w = _weights(ops, 12, rows, cols, stream=8)
    x = np.random.default_rng(1).standard_normal((T, cols)).astype(np.float32)
    ms = ops.qmatmul_time(12, w, rows, cols, x, path, 3)
    assert 0.0 < ms < 50.0
    print(label, "ms per launch", ms, "TFLOP/s", 2.0 * T * rows * cols / ms / 1e9)


def test_gated_gemm_timing_entry_on_the_benchmark_shape(ops):
    """The gate|up GEMM of one 2048-token tick of the headline workload with the activation in its epilogue (operands
    resident, L2 flushed before every launch).  Also the command the profiler captures of this kernel run."""
    F, cols, T = 11008, 2048, 2048
    gate_w = _weights(ops, 12, F, cols, stream=8)
    up_w = _weights(ops, 12, F, cols, stream=9)
    x = np.random.default_rng(1).standard_normal((T, cols)).astype(np.float32)
    out, ms = ops.gated_ffn(12, gate_w, up_w, F, cols, x, 0, iters=3)
    assert ms > 0.0 and np.isfinite(out).all()
    print("gated prefill_gate_up ms per launch", ms, "TFLOP/s", 2.0 * T * 2 * F * cols / ms / 1e9)


@pytest.mark.parametrize("name", ["q4_k", "q6_k", "q8_0", "f32"])
def test_embed_rows_exact(ops, orc, name):
    qtype = {"f32": 0, **QTYPES}[name]
    rows, cols = 300, 512
    w = _weights(ops, qtype, rows, cols, stream=5)
    ids = np.array([0, 299, 17, 17, 123], dtype=np.uint32)
    got = ops.embed(qtype, w, rows, cols, ids, 1.0)
    want = orc.embed(qtype, w, cols, ids, 1.0)
    assert np.array_equal(got, want)
    got = ops.embed(qtype, w, rows, cols, ids, 59.866)
    want = orc.embed(qtype, w, cols, ids, 59.866)
    assert np.array_equal(got, want)


def test_add_norm(ops, orc):
    rng = np.random.default_rng(3)
    rows, dim = 5, 2048
    h = rng.standard_normal((rows, dim)).astype(np.float32)
    a = rng.standard_normal((rows, dim)).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    pw = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    h2, n = ops.add_norm(h, a, 1.0, None, w, 1e-5)
    assert np.array_equal(h2, h + a)
    want = orc.rmsnorm(h + a, w, 1e-5)
    assert np.max(np.abs(n - want)) < 1e-5
    # sandwich form: post-norm on the branch output before the residual add
    h3, n3 = ops.add_norm(h, a, 1.0, pw, w, 1e-6)
    want_h = h + orc.rmsnorm(a, pw, 1e-6)
    assert np.max(np.abs(h3 - want_h)) < 1e-5
    assert np.max(np.abs(n3 - orc.rmsnorm(want_h, w, 1e-6))) < 2e-5


@pytest.mark.parametrize("act", [0, 1])
def test_actmul(ops, orc, act):
    rng = np.random.default_rng(4)
    g = (3 * rng.standard_normal((3, 5632))).astype(np.float32)
    u = rng.standard_normal((3, 5632)).astype(np.float32)
    got = ops.actmul(g, u, act)
    want = orc.act_mul(g, u, act)
    assert np.max(np.abs(got - want)) < 2e-6 * max(1.0, np.max(np.abs(want)))


def test_argmax_first_index_and_total_order(ops, orc):
    rng = np.random.default_rng(5)
    logits = rng.standard_normal((6, 32000)).astype(np.float32)
    logits[1, 100] = logits[1, 20000] = 9.0          # tie: first index wins
    logits[2, :] = -0.0
    logits[2, 7] = 0.0                                # +0 > -0 in the total order
    logits[3, :] = -5.0
    logits[4, 31999] = 50.0
    got = ops.argmax(logits)
    want = [orc.argmax(r) for r in logits]
    assert list(got) == want
    assert got[1] == 100 and got[2] == 7 and got[3] == 0 and got[4] == 31999


def test_moe_route(ops, orc):
    rng = np.random.default_rng(6)
    logits = rng.standard_normal((33, 128)).astype(np.float32)
    logits[0, 3] = logits[0, 90] = 4.0               # tie -> lower index first
    logits[1, :] = 0.5                                # all equal -> experts 0..7
    logits[2, 10] = 0.0
    logits[2, 4] = -0.0
    sel, w = ops.moe_route(logits, 8)
    osel, ow = orc.moe_route(logits, 8)
    assert np.array_equal(sel, osel)
    assert np.max(np.abs(w - ow)) < 1e-6
    assert list(sel[1]) == list(range(8))


def _attn_case(rng, lanes_spec, q_heads, kv_heads, d, bt, layers, layer, kv_dtype):
    """lanes_spec: list of (start_pos, n_tokens).  Builds pools with random history and disjoint tables."""
    blocks_needed = [-(-(s + n) // bt) for s, n in lanes_spec]
    pool_blocks = sum(blocks_needed) + 3
    perm = rng.permutation(pool_blocks)
    tables, off = [], 0
    for nb in blocks_needed:
        tables.append([int(b) for b in perm[off:off + nb]])
        off += nb
    shape = (pool_blocks, layers, kv_heads, bt, d)
    k_pool = rng.standard_normal(shape).astype(np.float32).astype(kv_dtype)
    v_pool = rng.standard_normal(shape).astype(np.float32).astype(kv_dtype)
    T = sum(n for _, n in lanes_spec)
    q = rng.standard_normal((T, q_heads * d)).astype(np.float32)
    k = rng.standard_normal((T, kv_heads * d)).astype(np.float32)
    v = rng.standard_normal((T, kv_heads * d)).astype(np.float32)
    return tables, k_pool, v_pool, q, k, v


@pytest.mark.parametrize("kv_dtype", [np.float32, np.float16])
@pytest.mark.parametrize("geom", [(32, 4, 64), (16, 4, 128), (16, 8, 256), (2, 1, 4)])
@pytest.mark.parametrize("window,softcap", [(0, 0.0), (24, 0.0), (0, 50.0)])
def test_attention_step_matches_oracle(ops, orc, kv_dtype, geom, window, softcap):
    q_heads, kv_heads, d = geom
    bt, layers, layer = 16, 3, 1
    rng = np.random.default_rng(q_heads * 1000 + d + window)
    lanes_spec = [(0, 17), (40, 1), (5, 33), (63, 1), (16, 16), (0, 1), (100, 70)]
    tables, k_pool, v_pool, q, k, v = _attn_case(rng, lanes_spec, q_heads, kv_heads, d, bt, layers, layer, kv_dtype)
    rotary = d
    cos, sin = orc.rope_tables(10000.0, rotary, 256)
    qn = (1 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    kn = (1 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    scale = 1.0 / np.sqrt(d)
    kp, vp = k_pool.copy(), v_pool.copy()
    res = ops.attention_step(q, k, v, kp, vp, tables, [s for s, _ in lanes_spec], [n for _, n in lanes_spec],
                             q_heads=q_heads, kv_heads=kv_heads, head_dim=d, block_tokens=bt, layers=layers, layer=layer,
                             scale=scale, softcap=softcap, window=window, cos_table=cos, sin_table=sin, rotary_dim=rotary,
                             q_norm_w=qn, k_norm_w=kn, norm_eps=1e-6)
    # oracle: same steps
    pos = np.concatenate([np.arange(s, s + n) for s, n in lanes_spec]).astype(np.int32)
    slots = np.concatenate([[tables[i][p // bt] * bt + p % bt for p in range(s, s + n)]
                            for i, (s, n) in enumerate(lanes_spec)]).astype(np.int64)
    assert np.array_equal(res["positions"], pos)
    assert np.array_equal(res["slots"], slots)
    cu = np.concatenate([[0], np.cumsum([n for _, n in lanes_spec])])
    assert np.array_equal(res["cu_seqlens"], cu)
    assert np.array_equal(res["last_index"], cu[1:] - 1)
    T = len(pos)
    qh = orc.rmsnorm(q.reshape(T * q_heads, d), qn, 1e-6).reshape(T, q_heads * d)
    kh = orc.rmsnorm(k.reshape(T * kv_heads, d), kn, 1e-6).reshape(T, kv_heads * d)
    q_rot = orc.rope_apply(qh, q_heads, d, rotary, pos, cos, sin)
    k_rot = orc.rope_apply(kh, kv_heads, d, rotary, pos, cos, sin)
    assert np.max(np.abs(res["q_rot"] - q_rot)) < 2e-6
    okp, ovp = k_pool.copy(), v_pool.copy()
    orc.kv_scatter(k_rot, v, okp, ovp, slots, kv_heads, d, bt, layers, layer)
    tol_pool = 0 if kv_dtype == np.float32 else 2e-3
    assert np.max(np.abs(kp.astype(np.float32) - okp.astype(np.float32))) <= max(tol_pool, 2e-6)
    assert np.array_equal(vp, ovp)
    flat = np.concatenate(tables).astype(np.uint32)
    page_off = np.concatenate([[0], np.cumsum([len(t) for t in tables])[:-1]]).astype(np.int32)
    for mode in (0, 1):
        want = orc.paged_attention(q_rot, okp, ovp, flat, page_off, [s for s, _ in lanes_spec], [n for _, n in lanes_spec],
                                   q_heads=q_heads, kv_heads=kv_heads, d=d, block_tokens=bt, layers=layers, layer=layer,
                                   scale=scale, softcap=softcap, window=window, mode=mode)
        assert np.max(np.abs(res["out"] - want)) < (2e-5 if kv_dtype == np.float32 else 2e-3)


@pytest.mark.parametrize("geom", [(32, 4, 64), (16, 4, 128), (8, 4, 128), (4, 4, 64), (16, 8, 256)])
@pytest.mark.parametrize("window,softcap,bt", [(0, 0.0, 16), (100, 0.0, 16), (0, 30.0, 32)])
def test_tensor_core_attention_long_contexts(ops, orc, geom, window, softcap, bt):
    """The tensor-core kernel on its own (kernel=2): prefill chunks that span several query tiles and key
    tiles, one-token lanes long enough to be split over several CTAs, against the oracle and against
    the scalar kernel (kernel=1) on the same pools."""
    q_heads, kv_heads, d = geom
    layers, layer = 2, 1
    rng = np.random.default_rng(q_heads * 77 + d + window + bt)
    lanes_spec = [(0, 150), (700, 1), (333, 200), (1500, 1), (63, 1), (64, 1), (0, 1), (129, 67), (2047, 1)]
    tables, k_pool, v_pool, q, k, v = _attn_case(rng, lanes_spec, q_heads, kv_heads, d, bt, layers, layer, np.float16)
    scale = 1.0 / np.sqrt(d)
    outs = {}
    for kernel in (1, 2):
        kp, vp = k_pool.copy(), v_pool.copy()
        res = ops.attention_step(q, k, v, kp, vp, tables, [s for s, _ in lanes_spec], [n for _, n in lanes_spec],
                                 q_heads=q_heads, kv_heads=kv_heads, head_dim=d, block_tokens=bt, layers=layers, layer=layer,
                                 scale=scale, softcap=softcap, window=window, kernel=kernel)
        outs[kernel] = res["out"]
    flat = np.concatenate(tables).astype(np.uint32)
    page_off = np.concatenate([[0], np.cumsum([len(t) for t in tables])[:-1]]).astype(np.int32)
    want = orc.paged_attention(q, kp, vp, flat, page_off, [s for s, _ in lanes_spec], [n for _, n in lanes_spec],
                               q_heads=q_heads, kv_heads=kv_heads, d=d, block_tokens=bt, layers=layers, layer=layer,
                               scale=scale, softcap=softcap, window=window, mode=0)
    assert np.isfinite(outs[2]).all()
    assert np.max(np.abs(outs[1] - want)) < 2e-5
    # queries and probabilities are rounded to f16 for the tensor cores: 2^-11 relative on operands of size <= 1
    assert np.max(np.abs(outs[2] - want)) < 2e-3


def test_decode_attention_at_the_benchmark_shape(ops, orc):
    """64 one-token lanes with 100..1000 tokens of history each, 16 query heads over 4 KV heads of 128: the
    decode tick of the headline workload, one layer of it."""
    q_heads, kv_heads, d, bt = 16, 4, 128, 16
    rng = np.random.default_rng(64)
    lanes_spec = [(int(c), 1) for c in rng.integers(100, 1000, size=64)]
    tables, k_pool, v_pool, q, k, v = _attn_case(rng, lanes_spec, q_heads, kv_heads, d, bt, 1, 0, np.float16)
    scale = 1.0 / np.sqrt(d)
    kp, vp = k_pool.copy(), v_pool.copy()
    res = ops.attention_step(q, k, v, kp, vp, tables, [s for s, _ in lanes_spec], [n for _, n in lanes_spec], q_heads=q_heads,
                             kv_heads=kv_heads, head_dim=d, block_tokens=bt, layers=1, layer=0, scale=scale, kernel=2)
    flat = np.concatenate(tables).astype(np.uint32)
    page_off = np.concatenate([[0], np.cumsum([len(t) for t in tables])[:-1]]).astype(np.int32)
    want = orc.paged_attention(q, kp, vp, flat, page_off, [s for s, _ in lanes_spec], [n for _, n in lanes_spec], q_heads=q_heads,
                               kv_heads=kv_heads, d=d, block_tokens=bt, layers=1, layer=0, scale=scale, softcap=0.0, window=0, mode=0)
    assert np.max(np.abs(res["out"] - want)) < 2e-3


def test_decode_attention_with_one_long_history_among_many_short_ones(ops, orc):
    """48 one-token lanes x 4 KV heads fill the GPU by themselves, so lanes are not cut - except the one whose history is
    many times the mean, which is shared out over several CTAs and merged; every lane must still match the oracle."""
    q_heads, kv_heads, d, bt = 16, 4, 128, 16
    rng = np.random.default_rng(65)
    lanes_spec = [(int(c), 1) for c in rng.integers(40, 300, size=47)] + [(5000, 1)]
    tables, k_pool, v_pool, q, k, v = _attn_case(rng, lanes_spec, q_heads, kv_heads, d, bt, 1, 0, np.float16)
    scale = 1.0 / np.sqrt(d)
    kp, vp = k_pool.copy(), v_pool.copy()
    res = ops.attention_step(q, k, v, kp, vp, tables, [s for s, _ in lanes_spec], [n for _, n in lanes_spec], q_heads=q_heads,
                             kv_heads=kv_heads, head_dim=d, block_tokens=bt, layers=1, layer=0, scale=scale, kernel=2)
    flat = np.concatenate(tables).astype(np.uint32)
    page_off = np.concatenate([[0], np.cumsum([len(t) for t in tables])[:-1]]).astype(np.int32)
    want = orc.paged_attention(q, kp, vp, flat, page_off, [s for s, _ in lanes_spec], [n for _, n in lanes_spec], q_heads=q_heads,
                               kv_heads=kv_heads, d=d, block_tokens=bt, layers=1, layer=0, scale=scale, softcap=0.0, window=0, mode=0)
    assert np.max(np.abs(res["out"] - want)) < 2e-3


def test_tensor_core_attention_is_refused_for_f32_pools(ops):
    rng = np.random.default_rng(3)
    tables, k_pool, v_pool, q, k, v = _attn_case(rng, [(0, 4)], 4, 2, 64, 16, 1, 0, np.float32)
    with pytest.raises(RuntimeError, match="does not cover"):
        ops.attention_step(q, k, v, k_pool, v_pool, tables, [0], [4], q_heads=4, kv_heads=2, head_dim=64, block_tokens=16,
                           layers=1, layer=0, scale=0.125, kernel=2)


def test_attention_nope_layer_leaves_queries_unrotated(ops, orc):
    rng = np.random.default_rng(9)
    q_heads, kv_heads, d, bt = 8, 2, 64, 16
    lanes_spec = [(3, 5), (20, 1)]
    tables, k_pool, v_pool, q, k, v = _attn_case(rng, lanes_spec, q_heads, kv_heads, d, bt, 1, 0, np.float32)
    res = ops.attention_step(q, k, v, k_pool, v_pool, tables, [3, 20], [5, 1], q_heads=q_heads, kv_heads=kv_heads,
                             head_dim=d, block_tokens=bt, layers=1, layer=0, scale=0.125)
    assert np.array_equal(res["q_rot"], q)


def _expert_partial(expert_out, sel, weights, e_lo, e_hi):
    """A token's choices held by one rank, weighted and added in ascending expert order, in f32."""
    T, k = sel.shape
    out = np.zeros((T, expert_out.shape[1]), dtype=np.float32)
    for t in range(T):
        for c in np.argsort(sel[t], kind="stable"):
            if e_lo <= sel[t, c] < e_hi:
                out[t] = out[t] + expert_out[t * k + c] * weights[t, c]
    return out


@pytest.mark.parametrize("T,ranks,rank,epochs", [(1, 2, 0, 1), (37, 4, 2, 3), (300, 2, 1, 2)])
def test_expert_exchange_kernel_combines_pushes_and_adds_in_rank_order(ops, T, ranks, rank, epochs):
    """The fused expert-parallel kernel from one rank's side, every rank's exchange block on this GPU: its own partial
    rows must land in all blocks, and the result must be the ranks' rows added in rank order, bit for bit; more than
    148 tokens (several rows per CTA) and several epochs (alternating buffers) included."""
    k, hidden, experts = 4, 512, 16
    rng = np.random.default_rng(T)
    sel = np.stack([rng.choice(experts, k, replace=False) for _ in range(T)]).astype(np.int32)
    weights = rng.random((T, k)).astype(np.float32)
    expert_out = rng.standard_normal((T * k, hidden)).astype(np.float32)
    per = experts // ranks
    e_lo, e_hi = rank * per, (rank + 1) * per
    peer_rows = rng.standard_normal((ranks, T, hidden)).astype(np.float32)
    out, pushed, status = ops.moe_combine_exchange(expert_out, sel, weights, e_lo, e_hi, ranks, rank, peer_rows, epochs=epochs)
    assert status == 0
    partial = _expert_partial(expert_out, sel, weights, e_lo, e_hi)
    for r in range(ranks):
        assert np.array_equal(pushed[r], partial)
    rows = peer_rows.copy()
    rows[rank] = partial
    want = rows[0]
    for r in range(1, ranks):
        want = want + rows[r]
    assert np.array_equal(out, want)


def test_expert_exchange_kernel_gives_up_when_a_peer_never_delivers(ops):
    """Nothing sets the other rank's flags: the wait is bounded (50 ms here), the kernel returns, the status word names
    the missing peer and the context stays usable."""
    T, k, hidden = 5, 2, 256
    rng = np.random.default_rng(0)
    sel = np.stack([rng.choice(8, k, replace=False) for _ in range(T)]).astype(np.int32)
    weights = rng.random((T, k)).astype(np.float32)
    expert_out = rng.standard_normal((T * k, hidden)).astype(np.float32)
    out, pushed, status = ops.moe_combine_exchange(expert_out, sel, weights, 0, 4, 2, 0, None, wait_ms=50)
    assert status == (0x4550000 | 1)
    assert np.array_equal(pushed[1], _expert_partial(expert_out, sel, weights, 0, 4))
    # the device still answers
    assert ops.argmax(np.eye(3, dtype=np.float32)).tolist() == [0, 1, 2]


@pytest.mark.parametrize("name", ["q4_k", "q6_k"])
@pytest.mark.parametrize("case", ["decode", "ragged", "wide"])
def test_expert_grouped_streamed_matmul_matches_oracle(ops, orc, name, case):
    """The expert-grouped form of the decode matmul (the row ranges are read on the device): experts with no rows, with a
    handful, and with more than one 64-row chunk; against the oracle's integer arithmetic per expert and against the
    grouped integer GEMV."""
    qtype = QTYPES[name]
    experts, rows_pe, cols = 8, 256, 512
    counts = {"decode": [1, 0, 3, 2, 0, 1, 4, 1], "ragged": [0, 17, 64, 5, 33, 0, 1, 40], "wide": [130, 0, 64, 65, 7, 200, 1, 0]}[case]
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    P = int(offsets[-1])
    rng = np.random.default_rng(len(case))
    x = rng.standard_normal((P, cols)).astype(np.float32)
    w = _weights(ops, qtype, experts * rows_pe, cols, stream=11)
    rb = len(w) // (experts * rows_pe)
    want = np.zeros((P, rows_pe), np.float32)
    for e in range(experts):
        lo, hi = offsets[e], offsets[e + 1]
        if hi > lo:
            want[lo:hi] = orc.qmatmul(qtype, w[e * rows_pe * rb:(e + 1) * rows_pe * rb], rows_pe, cols, x[lo:hi], 1)
    got = ops.grouped_qmatmul(qtype, w, experts, rows_pe, cols, x, offsets, 4)
    scale = np.sqrt(cols) * 0.02
    assert np.isfinite(got).all() and np.max(np.abs(got - want)) <= 3e-3 * scale
    gemv = ops.grouped_qmatmul(qtype, w, experts, rows_pe, cols, x, offsets, 1)
    assert np.max(np.abs(gemv - want)) <= 2e-5 * max(1.0, np.max(np.abs(want)))


@pytest.mark.parametrize("act", [0, 1])
def test_expert_grouped_gated_matmul_matches_oracle(ops, orc, act):
    """gate and up banks interleaved per expert, act(gate) * up in the epilogue, f16 out."""
    experts, F, cols = 4, 384, 512
    counts = [5, 0, 70, 12]
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    P = int(offsets[-1])
    rng = np.random.default_rng(act)
    x = rng.standard_normal((P, cols)).astype(np.float32)
    gate = _weights(ops, 12, experts * F, cols, stream=12)
    up = _weights(ops, 12, experts * F, cols, stream=13)
    rb = len(gate) // (experts * F)
    want = np.zeros((P, F), np.float32)
    gmax = umax = 0.0
    for e in range(experts):
        lo, hi = offsets[e], offsets[e + 1]
        if hi > lo:
            g = orc.qmatmul(12, gate[e * F * rb:(e + 1) * F * rb], F, cols, x[lo:hi], 1)
            u = orc.qmatmul(12, up[e * F * rb:(e + 1) * F * rb], F, cols, x[lo:hi], 1)
            gmax, umax = max(gmax, float(np.abs(g).max())), max(umax, float(np.abs(u).max()))
            want[lo:hi] = orc.act_mul(g, u, act)
    got = ops.grouped_qmatmul(12, gate, experts, F, cols, x, offsets, 4, up_bank=up, act=act)
    scale = np.sqrt(cols) * 0.02
    assert np.isfinite(got).all()
    # gate and up each carry the f16-operand error of the matmul; the product adds them, then one f16 rounding
    assert np.max(np.abs(got - want)) <= 3e-3 * scale * (2 * gmax + umax + 1)


def test_expert_grouped_gated_matmul_on_the_moe_decode_shape(ops, orc):
    """One MoE layer's gate|up bank of the 30B-A3B shape (128 experts of 768 x 2048 Q4_K each for gate and for up) with the
    routed rows of a 72-lane decode tick (576 rows, a few per expert, some experts idle); checked against the oracle on
    every eighth expert.  Also the launch the profiler capture of the expert-grouped kernel runs."""
    experts, F, cols, P = 128, 768, 2048, 576
    rng = np.random.default_rng(30)
    counts = np.bincount(rng.integers(0, experts, P), minlength=experts)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    x = rng.standard_normal((P, cols)).astype(np.float32)
    gate = _weights(ops, 12, experts * F, cols, stream=14)
    up = _weights(ops, 12, experts * F, cols, stream=15)
    rb = len(gate) // (experts * F)
    got = ops.grouped_qmatmul(12, gate, experts, F, cols, x, offsets, 4, up_bank=up, act=0)
    assert np.isfinite(got).all()
    scale = np.sqrt(cols) * 0.02
    for e in range(0, experts, 8):
        lo, hi = offsets[e], offsets[e + 1]
        if hi == lo:
            continue
        g = orc.qmatmul(12, gate[e * F * rb:(e + 1) * F * rb], F, cols, x[lo:hi], 1)
        u = orc.qmatmul(12, up[e * F * rb:(e + 1) * F * rb], F, cols, x[lo:hi], 1)
        want = orc.act_mul(g, u, 0)
        assert np.max(np.abs(got[lo:hi] - want)) <= 3e-3 * scale * (2 * float(np.abs(g).max()) + float(np.abs(u).max()) + 1), e
