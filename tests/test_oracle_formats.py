"""Pins the oracle's block decoders (and the seed-model quantisers) against the `gguf` Python
package's dequantisers - the public GGML block layouts."""
import numpy as np
import pytest

gguf = pytest.importorskip("gguf")
from gguf import quants  # noqa: E402

CASES = [("q4_k", 12, gguf.GGMLQuantizationType.Q4_K), ("q6_k", 14, gguf.GGMLQuantizationType.Q6_K),
         ("q8_0", 8, gguf.GGMLQuantizationType.Q8_0)]


@pytest.fixture(scope="module")
def ops(mk):
    import importlib
    return importlib.import_module("macllm_infer_b200.ops")


@pytest.mark.parametrize("name,qtype,gtype", CASES)
def test_dequant_matches_gguf_package(ops, orc, name, qtype, gtype):
    rows, cols = 24, 1024
    w = ops.seed_tensor(7, 11, 0.02, qtype, rows, cols)
    rb = ops.row_bytes(qtype, cols)
    assert w.size == rows * rb and rb == orc.row_bytes(qtype, cols)
    want = quants.dequantize(w.reshape(rows, rb), gtype)
    got = orc.dequant(qtype, w, rows, cols)
    assert got.shape == want.shape
    assert np.max(np.abs(got - want)) <= 1e-7


@pytest.mark.parametrize("name,qtype,gtype", CASES)
def test_random_block_bytes_decode_like_gguf_package(orc, name, qtype, gtype):
    """Arbitrary block bytes (not produced by our quantiser) decode identically: layout, not values."""
    rng = np.random.default_rng(3)
    rows, cols = 8, 512
    rb = orc.row_bytes(qtype, cols)
    raw = rng.integers(0, 256, size=(rows, rb), dtype=np.uint8)
    # keep the f16 scale fields finite
    blk = {12: 144, 14: 210, 8: 34}[qtype]
    view = raw.reshape(rows, rb // blk, blk)
    if qtype == 12:
        view[:, :, 1] &= 0x3B
        view[:, :, 3] &= 0x3B
    elif qtype == 14:
        view[:, :, 209] &= 0x3B
    else:
        view[:, :, 1] &= 0x3B
    want = quants.dequantize(raw, gtype)
    got = orc.dequant(qtype, raw, rows, cols)
    assert np.allclose(got, want, rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("name,qtype,gtype", CASES)
def test_seed_quantiser_error_is_small(ops, orc, name, qtype, gtype):
    rows, cols = 16, 2048
    ref = np.frombuffer(ops.seed_tensor(3, 5, 0.02, 0, rows, cols).tobytes(), dtype=np.float32).reshape(rows, cols)
    assert abs(ref.std() - 0.02) < 0.001 and abs(ref.mean()) < 0.001
    w = ops.seed_tensor(3, 5, 0.02, qtype, rows, cols)
    deq = orc.dequant(qtype, w, rows, cols)
    rel = np.sqrt(np.mean((deq - ref) ** 2)) / ref.std()
    assert rel < {12: 0.09, 14: 0.03, 8: 0.01}[qtype]


def test_quantised_matmul_close_to_dense(ops, orc):
    """The reference's own bound for this boundary: quantised matmul within 0.05 of the same weights
    dequantised (src/model_weights.rs:624-683)."""
    rng = np.random.default_rng(0)
    rows, cols = 64, 512
    for qtype in (12, 14, 8):
        w = ops.seed_tensor(1, 2, 0.5, qtype, rows, cols)
        x = rng.standard_normal((2, cols)).astype(np.float32)
        y1 = orc.qmatmul(qtype, w, rows, cols, x, 1)
        y2 = orc.qmatmul(qtype, w, rows, cols, x, 2)
        assert np.max(np.abs(y1 - y2)) < 0.05 * max(1.0, float(np.max(np.abs(y2))))
        fq = orc.fake_quant_rows(qtype, x)
        y3 = fq @ orc.dequant(qtype, w, rows, cols).T
        assert np.max(np.abs(y1 - y3)) < 1e-4 * max(1.0, float(np.max(np.abs(y2))))


def test_embedding_rows_equal_dequantised_rows(ops, orc):
    rows, cols = 40, 512
    for qtype in (12, 14, 8):
        w = ops.seed_tensor(1, 9, 0.02, qtype, rows, cols)
        ids = [3, 39, 0]
        assert np.array_equal(orc.embed(qtype, w, cols, ids), orc.dequant(qtype, w, rows, cols)[ids])


# The block formats no kernel reads in place: the oracle's decoder and the product's load-time host decoder are two
# independent restatements of the public layouts; both are pinned against the `gguf` package on seeded random blocks
# (any bit pattern is a valid block once its f16 scale fields are finite) and on arbitrary bytes.
LOAD_DECODED = [("q4_0", 2, gguf.GGMLQuantizationType.Q4_0, 18, 32), ("q5_0", 6, gguf.GGMLQuantizationType.Q5_0, 22, 32),
                ("q5_1", 7, gguf.GGMLQuantizationType.Q5_1, 24, 32), ("q2_k", 10, gguf.GGMLQuantizationType.Q2_K, 84, 256),
                ("q3_k", 11, gguf.GGMLQuantizationType.Q3_K, 110, 256), ("q5_k", 13, gguf.GGMLQuantizationType.Q5_K, 176, 256)]
F16_FIELDS = {2: [0], 6: [0], 7: [0, 2], 10: [80, 82], 11: [108], 13: [0, 2]}


@pytest.mark.parametrize("name,qtype,gtype,block_bytes,block_weights", LOAD_DECODED)
def test_load_decoded_formats_match_gguf_package(ops, orc, name, qtype, gtype, block_bytes, block_weights):
    rows, cols = 6, 1024
    rb = ops.row_bytes(qtype, cols)
    assert rb == cols // block_weights * block_bytes == orc.row_bytes(qtype, cols)
    # seeded blocks as the checkpoint writer makes them: decoded weights of about the asked spread, zero mean
    w = ops.seed_tensor(5, 9, 0.02, qtype, rows, cols)
    want = quants.dequantize(w.reshape(rows, rb), gtype)
    assert np.isfinite(want).all() and 0.012 < want.std() < 0.03 and abs(want.mean()) < 0.004
    assert np.array_equal(orc.dequant(qtype, w, rows, cols), want.astype(np.float32))
    assert np.array_equal(ops.decode_rows(qtype, w, rows, cols), want.astype(np.float32))
    # arbitrary bytes, scale fields kept finite
    raw = np.random.default_rng(qtype).integers(0, 256, size=(rows, rb), dtype=np.uint8)
    view = raw.reshape(rows, rb // block_bytes, block_bytes)
    for off in F16_FIELDS[qtype]:
        view[:, :, off + 1] &= 0x3B
    want = quants.dequantize(raw, gtype).astype(np.float32)
    assert np.allclose(orc.dequant(qtype, raw, rows, cols), want, rtol=1e-6, atol=1e-7)
    assert np.allclose(ops.decode_rows(qtype, raw, rows, cols), want, rtol=1e-6, atol=1e-7)


def test_bf16_rows_decode_exactly(ops, orc):
    rows, cols = 3, 64
    w = ops.seed_tensor(1, 2, 0.02, 30, rows, cols)
    assert w.size == rows * cols * 2
    want = (w.view(np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(rows, cols)
    ref = np.frombuffer(ops.seed_tensor(1, 2, 0.02, 0, rows, cols).tobytes(), dtype=np.float32).reshape(rows, cols)
    assert np.max(np.abs(want - ref)) <= np.max(np.abs(ref)) * 2 ** -8       # round-to-nearest-even truncation to 8 bits of mantissa
    assert np.array_equal(orc.dequant(30, w, rows, cols), want)
    assert np.array_equal(ops.decode_rows(30, w, rows, cols), want)


def test_host_decoder_refuses_what_it_does_not_decode(ops, mk):
    import importlib
    capi = importlib.import_module("macllm_infer_b200._capi")
    raw = np.zeros(144 * 4, dtype=np.uint8)
    for qtype, cols in ((12, 256), (8, 32), (99, 32)):     # formats the kernels read in place, and an unknown id
        with pytest.raises(capi.MkError):
            ops.decode_rows(qtype, raw, 1, cols)
    with pytest.raises(capi.MkError):
        ops.decode_rows(13, raw, 1, 300)                    # not a whole number of 256-weight blocks


def test_vector_inner_sums_equal_the_scalar_loops(orc, tmp_path):
    """The oracle's Q4_K / Q6_K dots take their integer inner sums with AVX2 where the host has it. Integer sums are
    exact in any order, so the result must equal the scalar loops' bit for bit: the same file built without the
    vector path is the check. Random block bytes cover every nibble, high-bit and scale pattern."""
    import ctypes as C
    import os
    import subprocess
    src = os.path.join(os.path.dirname(orc.__file__), "oracle_math.cpp")
    so = str(tmp_path / "liboracle_scalar.so")
    cxx = "/usr/bin/g++" if os.access("/usr/bin/g++", os.X_OK) else "g++"
    subprocess.run([cxx, "-O2", "-std=c++17", "-fPIC", "-fopenmp", "-mavx2", "-mfma", "-ffp-contract=off", "-fno-fast-math",
                    "-DORC_NO_SIMD", "-shared", "-o", so, src], check=True)
    scalar = C.CDLL(so)
    rng = np.random.default_rng(11)
    for qtype, block_bytes, scale_at in ((12, 144, (0, 4)), (14, 210, (208, 210))):
        for rows, cols, T in ((96, 1024, 3), (33, 256, 1)):
            nb = cols // 256
            w = rng.integers(0, 256, size=(rows, nb, block_bytes), dtype=np.uint8)
            halves = rng.uniform(0.001, 0.05, size=(rows, nb, (scale_at[1] - scale_at[0]) // 2)).astype(np.float16)
            w[:, :, scale_at[0]:scale_at[1]] = halves.view(np.uint8).reshape(rows, nb, -1)
            w = np.ascontiguousarray(w.reshape(rows, nb * block_bytes))
            x = (rng.standard_normal((T, cols)) * 3).astype(np.float32)
            x[0, :40] = 0
            for mode in (1, 3):
                want = np.empty((T, rows), np.float32)
                scalar.orc_qmatmul(C.c_int(qtype), C.c_void_p(w.ctypes.data), C.c_int64(rows), C.c_int64(cols),
                                   C.c_void_p(x.ctypes.data), C.c_int64(T), C.c_void_p(want.ctypes.data), C.c_int(mode))
                got = orc.qmatmul(qtype, w, rows, cols, x, mode)
                assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (qtype, rows, cols, T, mode)


def test_q4_0_and_q8_0_golden_blocks_of_the_reference(ops, orc):
    """src/gguf.rs:3882-3971: one hand-made block of each format and the weights it must decode to - Q4_0 with scale 0.125
    walks -1.0 ... 0.875 and back; Q8_0 with scale 0.007873535 (f16 0x2008) times the signed bytes."""
    q4 = np.array([0x00, 0x30, 0xf0, 0xe1, 0xd2, 0xc3, 0xb4, 0xa5, 0x96, 0x87, 0x78, 0x69, 0x5a, 0x4b, 0x3c, 0x2d, 0x1e, 0x0f], np.uint8)
    q8 = np.array([0x08, 0x20, 0x81, 0xc0, 0xe0, 0xf0, 0xf3, 0xff, 0x00, 0x01, 0x0d, 0x10, 0x20, 0x40, 0x7f, 0x5f, 0xa1, 0x2a, 0xd6, 0x19,
                   0xe7, 0x03, 0xfd, 0x72, 0x8e, 0x4c, 0xb4, 0x33, 0xcd, 0x06, 0xfa, 0x01, 0xff, 0x00], np.uint8)
    assert ops.row_bytes(2, 32) == orc.row_bytes(2, 32) == 18 and ops.row_bytes(8, 32) == orc.row_bytes(8, 32) == 34
    want_q4 = np.array([-1.0 + i * 0.125 for i in range(16)] + [0.875 - i * 0.125 for i in range(16)], np.float32)
    assert np.array_equal(orc.dequant(2, q4, 1, 32)[0], want_q4)
    assert np.array_equal(ops.decode_rows(2, q4, 1, 32)[0], want_q4)
    signed = np.array([-127, -64, -32, -16, -13, -1, 0, 1, 13, 16, 32, 64, 127, 95, -95, 42, -42, 25, -25, 3, -3, 114, -114, 76, -76, 51,
                       -51, 6, -6, 1, -1, 0], np.float32)
    want_q8 = signed * np.float32(0.007873535)
    assert np.array_equal(orc.dequant(8, q8, 1, 32)[0], want_q8)
    assert np.float32(np.frombuffer(q8[:2].tobytes(), np.float16)[0]) == np.float32(0.007873535)
    # the product reads Q8_0 in place: the embedding-row path decodes the same block on the host side of the oracle only;
    # the device decoders of Q8_0 are held to the oracle in the GPU kernel tests


def test_llama_query_key_rows_are_unpermuted_like_the_reference(ops, orc):
    """src/gguf.rs:3663-3683,4328-4395: eight rows across two heads go to the order 0 2 1 3 4 6 5 7; rows of Q8_0 and Q4_0
    blocks move as whole byte strings and decode to the same first weights as the reference's."""
    from oracle import decoder
    import importlib
    capi = importlib.import_module("macllm_infer_b200._capi")
    dense = np.arange(8, dtype=np.float32)
    want = np.array([0, 2, 1, 3, 4, 6, 5, 7], np.float32)
    assert np.array_equal(ops.unpermute_qk_rows(dense.view(np.uint8), 8, 2).view(np.float32), want)
    assert np.array_equal(decoder._unpermute(dense.view(np.uint8), 8, 2, 4).view(np.float32), want)
    one = np.frombuffer(np.float16(1.0).tobytes(), np.uint8)
    q8 = np.concatenate([np.concatenate([one, np.full(32, v, np.uint8)] * 2) for v in range(1, 9)])
    q4 = np.concatenate([np.concatenate([one, np.full(16, c | (c << 4), np.uint8)] * 2) for c in range(8)])
    for qtype, raw, first in ((8, q8, [1, 3, 2, 4, 5, 7, 6, 8]), (2, q4, [-8, -6, -7, -5, -4, -2, -3, -1])):
        assert raw.size == 8 * orc.row_bytes(qtype, 64)
        moved = ops.unpermute_qk_rows(raw, 8, 2)
        assert np.array_equal(moved, decoder._unpermute(raw, 8, 2, raw.size // 8))
        rows = orc.dequant(qtype, moved, 8, 64)
        assert list(rows[:, 0]) == first and all(np.all(rows[r] == rows[r, 0]) for r in range(8))
    with pytest.raises(capi.MkError, match="across 3 heads"):
        ops.unpermute_qk_rows(dense.view(np.uint8), 8, 3)
    with pytest.raises(capi.MkError, match="head dimension 1 must be even"):
        ops.unpermute_qk_rows(dense.view(np.uint8), 8, 8)
