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
