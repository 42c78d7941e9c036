"""Known answers the reference's own tests hold for the arithmetic of the path, run against the oracle (no GPU) and, where
a kernel-level entry exists, against the CUDA kernels (GPU):

  * paged decode row against materialised GQA attention across slabs, with and without soft cap
    (crates/macllm-kernels/src/paged_attention.rs:1340-1406);
  * a ragged batch against serial per-lane attention (paged_attention.rs:1409-1501), and direct pages against a fresh
    chunked prefill followed by decode (paged_attention.rs:1504-1593);
  * router: only the top-k are normalised, ties go to the lower expert, signed zeros tie, k = experts
    (src/decoder.rs:8600-8642);
  * sparse MoE exact outputs [4/7, 6/7, 9/4, 11/4] (src/decoder.rs:8645-8717).
The expected values are computed in the tests in float64 from the definitions, not by the code under test.
"""
import importlib

import numpy as np
import pytest


@pytest.fixture(scope="module")
def ops(mk):
    return importlib.import_module("macllm_infer_b200.ops")


def dense_gqa(q, keys, values, start, scale, softcap=0.0, window=0):
    """dense_causal_attention (src/decoder.rs:4580-4670) in float64.  q [n, H, d]; keys/values [ctx, KV, d]; row r of q sits
    at position start + r and sees keys 0..start + r (and, with a window, only the last `window` of them)."""
    n, H, d = q.shape
    KV = keys.shape[1]
    out = np.zeros((n, H, d))
    for r in range(n):
        p = start + r
        lo = max(0, p - window + 1) if window else 0
        for h in range(H):
            kh = h // (H // KV)
            s = keys[lo:p + 1, kh].astype(np.float64) @ q[r, h].astype(np.float64) * scale
            if softcap:
                s = np.tanh(s / softcap) * softcap
            w = np.exp(s - s.max())
            w /= w.sum()
            out[r, h] = w @ values[lo:p + 1, kh].astype(np.float64)
    return out


def pools(blocks, kv_heads, bt, d, dtype=np.float32):
    shape = (blocks, 1, kv_heads, bt, d)
    return np.zeros(shape, dtype), np.zeros(shape, dtype)


def scatter(k_pool, v_pool, table, keys, values, bt):
    for p in range(len(keys)):
        k_pool[table[p // bt], 0, :, p % bt] = keys[p]
        v_pool[table[p // bt], 0, :, p % bt] = values[p]


SLAB_CASE = dict(
    # K/V [head][token][d] of the reference's case, three tokens over two 2-token blocks that live in different slabs
    k=np.array([[[1, 0], [0, 1], [1, 1]], [[-1, 0], [0, -1], [-1, -1]]], np.float32),
    v=np.array([[[1, 2], [3, 4], [5, 6]], [[-1, -2], [-3, -4], [-5, -6]]], np.float32),
    q=np.array([[1, 0], [0, 1], [-1, 0], [0, -1]], np.float32),   # four query heads, one row at position 2
)


@pytest.mark.parametrize("softcap", [0.0, 1.5])
def test_paged_decode_row_matches_materialised_gqa_across_slabs_on_the_oracle(orc, softcap):
    c = SLAB_CASE
    keys, values = c["k"].transpose(1, 0, 2), c["v"].transpose(1, 0, 2)       # [token][head][d]
    k_pool, v_pool = pools(4, 2, 2, 2)
    table = [0, 1]                                                            # slab_blocks = 1: every block its own slab
    scatter(k_pool, v_pool, table, keys, values, 2)
    want = dense_gqa(c["q"][None], keys, values, 2, 0.5, softcap)[0]
    for mode in (1, 2):
        got = orc.paged_attention(c["q"].reshape(1, 8), k_pool, v_pool, table, [0], [2], [1], q_heads=4, kv_heads=2, d=2, block_tokens=2,
                                  layers=1, layer=0, scale=0.5, softcap=softcap, mode=mode)
        assert np.abs(got.reshape(4, 2) - want).max() <= 1e-6


def ragged_case(seed=0):
    """Lanes of 2, 5 and 3 fresh tokens, four query heads over two KV heads of width 3, 2-token blocks."""
    rng = np.random.default_rng(seed)
    lens = [2, 5, 3]
    H, KV, d, bt = 4, 2, 3, 2
    q = [rng.standard_normal((n, H, d)).astype(np.float32) for n in lens]
    k = [rng.standard_normal((n, KV, d)).astype(np.float32) for n in lens]
    v = [rng.standard_normal((n, KV, d)).astype(np.float32) for n in lens]
    tables, nxt = [], 0
    for n in lens:
        nb = -(-n // bt)
        tables.append(list(range(nxt, nxt + nb)))
        nxt += nb
    return lens, H, KV, d, bt, q, k, v, tables, nxt


@pytest.mark.parametrize("softcap", [0.0, 1.5])
def test_ragged_batch_matches_serial_attention_on_the_oracle(orc, softcap):
    lens, H, KV, d, bt, q, k, v, tables, blocks = ragged_case()
    k_pool, v_pool = pools(blocks, KV, bt, d)
    for t, kk, vv in zip(tables, k, v):
        scatter(k_pool, v_pool, t, kk, vv, bt)
    flat = [b for t in tables for b in t]
    off = np.concatenate([[0], np.cumsum([len(t) for t in tables])[:-1]])
    got = orc.paged_attention(np.concatenate([x.reshape(len(x), -1) for x in q]), k_pool, v_pool, flat, off, [0, 0, 0], lens, q_heads=H,
                              kv_heads=KV, d=d, block_tokens=bt, layers=1, layer=0, scale=0.41, softcap=softcap, mode=1)
    want = np.concatenate([dense_gqa(qq, kk, vv, 0, 0.41, softcap).reshape(len(qq), -1) for qq, kk, vv in zip(q, k, v)])
    assert np.abs(got - want).max() <= 1e-6


def test_direct_pages_match_chunked_prefill_then_decode_on_the_oracle(orc):
    """A 7-token history written in chunks of 3, 3 and 1 (decode) gives, row for row, what one pass over all 7 gives."""
    rng = np.random.default_rng(3)
    H, KV, d, bt, n = 4, 2, 3, 2, 7
    q = rng.standard_normal((n, H, d)).astype(np.float32)
    k = rng.standard_normal((n, KV, d)).astype(np.float32)
    v = rng.standard_normal((n, KV, d)).astype(np.float32)
    table = [2, 0, 3, 1]
    k_pool, v_pool = pools(4, KV, bt, d)
    rows = []
    for lo, hi in ((0, 3), (3, 6), (6, 7)):
        scatter(k_pool, v_pool, table, k[:hi], v[:hi], bt)
        rows.append(orc.paged_attention(q[lo:hi].reshape(hi - lo, -1), k_pool, v_pool, table, [0], [lo], [hi - lo], q_heads=H, kv_heads=KV, d=d,
                                        block_tokens=bt, layers=1, layer=0, scale=0.5, mode=1))
    want = dense_gqa(q, k, v, 0, 0.5).reshape(n, -1)
    assert np.abs(np.concatenate(rows) - want).max() <= 1e-6


def test_router_known_answers_on_the_oracle(orc):
    """selected_softmax_routes_only_normalizes_top_k_with_stable_ties and ..._treats_signed_zero_as_a_tie_and_supports_k_equal_e."""
    sel, w = orc.moe_route(np.array([[1.0, 3.0, 2.0, -5.0], [4.0, 4.0, 0.0, -1.0]], np.float32), 2)
    assert sel.tolist() == [[1, 2], [0, 1]]
    logistic = 1.0 / (1.0 + np.exp(-1.0))
    assert abs(w[0, 0] - logistic) < 1e-7 and abs(w[0, 1] - (1 - logistic)) < 1e-7
    assert abs(w[1, 0] - 0.5) < 1e-7 and abs(w[1, 1] - 0.5) < 1e-7
    sel, _ = orc.moe_route(np.array([[0.0, -0.0]], np.float32), 1)
    assert sel.tolist() == [[0]]                                              # -0.0 == 0.0: the lower index wins
    sel, w = orc.moe_route(np.array([[3.0, 1.0, 2.0, 0.0]], np.float32), 4)
    assert sorted(sel[0].tolist()) == [0, 1, 2, 3] and abs(float(w.sum()) - 1.0) < 1e-6


def test_sparse_moe_exact_outputs_on_the_oracle(orc):
    """sparse_moe_dense_bank_routes_and_index_adds_exact_outputs: hidden 2, three experts of width 1, top-2, SiLU; router
    rows ln 4 / 0, ln 3 / ln 2, 0 / ln 6; gate and up all ones; down scaled by 1 / silu(1).  Tokens (1, 0) and (0, 1) give
    [4/7, 6/7] and [9/4, 11/4]."""
    inv = 1.0 + np.exp(-1.0)
    router = np.array([[np.log(4.0), 0.0], [np.log(3.0), np.log(2.0)], [0.0, np.log(6.0)]], np.float32)
    gate = np.ones((3, 1, 2), np.float32)
    up = np.ones((3, 1, 2), np.float32)
    down = np.array([[[inv], [0.0]], [[0.0], [2 * inv]], [[3 * inv], [3 * inv]]], np.float32)
    x = np.array([[1.0, 0.0], [0.0, 1.0]], np.float32)
    sel, w = orc.moe_route(x @ router.T, 2)
    out = np.zeros_like(x)
    for e in range(3):                                    # experts in index order, index_add (src/decoder.rs:424-439)
        rows, choice = np.nonzero(sel == e)
        if len(rows) == 0:
            continue
        h = orc.act_mul(x[rows] @ gate[e].T, x[rows] @ up[e].T, 0)
        out[rows] += (h @ down[e].T) * w[rows, choice][:, None]
    assert np.abs(out.reshape(-1) - np.array([4 / 7, 6 / 7, 9 / 4, 11 / 4])).max() < 1e-5


# ---- the same attention cases on the CUDA kernels -----------------------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("softcap", [0.0, 1.5])
def test_paged_decode_row_across_slabs_on_the_gpu(ops, softcap):
    c = SLAB_CASE
    keys, values = c["k"].transpose(1, 0, 2), c["v"].transpose(1, 0, 2)
    pad = lambda a: np.concatenate([a, np.zeros(a.shape[:-1] + (2,), np.float32)], axis=-1)   # head widths come in multiples of 4
    k_pool, v_pool = pools(4, 2, 2, 4)
    scatter(k_pool, v_pool, [0, 1], pad(keys[:2]), pad(values[:2]), 2)        # the first two tokens are history
    r = ops.attention_step(pad(c["q"]).reshape(1, 16), pad(keys[2]).reshape(1, 8), pad(values[2]).reshape(1, 8), k_pool, v_pool, [[0, 1]], [2], [1],
                           q_heads=4, kv_heads=2, head_dim=4, block_tokens=2, layers=1, layer=0, scale=0.5, softcap=softcap, kernel=1)
    want = dense_gqa(c["q"][None], keys, values, 2, 0.5, softcap)[0]
    got = r["out"].reshape(4, 4)
    assert np.abs(got[:, :2] - want).max() <= 2e-6 and np.abs(got[:, 2:]).max() == 0.0
    assert np.array_equal(k_pool[1, 0, :, 0, :2], keys[2]) and np.array_equal(v_pool[1, 0, :, 0, :2], values[2])   # the new row landed in slab 1


@pytest.mark.gpu
@pytest.mark.parametrize("softcap", [0.0, 1.5])
def test_ragged_batch_matches_serial_attention_on_the_gpu(ops, softcap):
    lens, H, KV, d, bt, q, k, v, tables, blocks = ragged_case()
    d4 = 4                                                # the kernels take head widths in multiples of 4: pad with zeros
    pad = lambda a: np.concatenate([a, np.zeros(a.shape[:-1] + (d4 - d,), np.float32)], axis=-1)
    k_pool, v_pool = pools(blocks, KV, bt, d4)
    r = ops.attention_step(np.concatenate([pad(x).reshape(len(x), -1) for x in q]), np.concatenate([pad(x).reshape(len(x), -1) for x in k]),
                           np.concatenate([pad(x).reshape(len(x), -1) for x in v]), k_pool, v_pool, tables, [0, 0, 0], lens, q_heads=H,
                           kv_heads=KV, head_dim=d4, block_tokens=bt, layers=1, layer=0, scale=0.41, softcap=softcap, kernel=1)
    want = np.concatenate([dense_gqa(qq, kk, vv, 0, 0.41, softcap) for qq, kk, vv in zip(q, k, v)])
    got = r["out"].reshape(-1, H, d4)
    assert np.abs(got[..., :d] - want).max() <= 2e-6 and np.abs(got[..., d:]).max() == 0.0


def test_router_refuses_non_finite_logits_and_bad_counts_on_the_oracle(orc):
    """selected_softmax_routes_rejects_invalid_or_non_finite_logits (src/decoder.rs:8620-8629)."""
    with pytest.raises(ValueError, match="non-finite logits for token row 0"):
        orc.moe_route(np.array([[1.0, np.nan]], np.float32), 1)
    with pytest.raises(ValueError, match="non-finite logits for token row 1"):
        orc.moe_route(np.array([[1.0, 2.0], [np.inf, 0.0]], np.float32), 1)
    for k in (0, 3):
        with pytest.raises(ValueError, match=r"experts per token \d must be in 1\.\.=2"):
            orc.moe_route(np.array([[1.0, 2.0]], np.float32), k)


@pytest.mark.gpu
def test_router_refuses_non_finite_logits_and_bad_counts_on_the_gpu(ops, mk):
    """The same refusals from the device kernel: a row with a NaN records a status that names the row (the choices written
    for it stay in range, so nothing downstream indexes out of bounds); counts outside 1..=experts are refused before any
    launch."""
    import importlib
    capi = importlib.import_module("macllm_infer_b200._capi")
    with pytest.raises(capi.MkError, match="non-finite logits for token row 1"):
        ops.moe_route(np.array([[1.0, 2.0, 3.0, 0.5], [0.0, np.nan, 1.0, 2.0]], np.float32), 2)
    for k in (0, 5):
        with pytest.raises(capi.MkError, match=r"experts per token \d must be in 1\.\.=4"):
            ops.moe_route(np.array([[1.0, 2.0, 3.0, 0.5]], np.float32), k)
    sel, w = ops.moe_route(np.array([[1.0, 2.0, 3.0, 0.5]], np.float32), 2)    # the device still answers
    assert sel.tolist() == [[2, 1]]


def test_partial_rope_rotates_only_the_configured_prefix_on_the_oracle(orc):
    """partial_rope_rotates_only_the_configured_prefix (src/decoder.rs:8464-8500): head_dim 4, rotary_dim 2, theta 10000,
    position 1 - the last two dimensions of every head pass through untouched, the first two turn by one radian."""
    cos, sin = orc.rope_tables(10_000.0, 2, 8)
    q = np.array([[1.0, 2.0, 30.0, 40.0, 3.0, 4.0, 50.0, 60.0]], np.float32)
    k = np.array([[5.0, 6.0, 70.0, 80.0, 7.0, 8.0, 90.0, 100.0]], np.float32)
    for x in (q, k):
        got = orc.rope_apply(x, 2, 4, 2, [1], cos, sin).reshape(2, 4)
        src = x.reshape(2, 4)
        assert np.array_equal(got[:, 2:], src[:, 2:])
        assert np.max(np.abs(got[:, :2] - src[:, :2])) > 1e-3
        c, s = np.float32(np.cos(1.0)), np.float32(np.sin(1.0))
        want = np.stack([src[:, 0] * c - src[:, 1] * s, src[:, 1] * c + src[:, 0] * s], axis=1)
        assert np.allclose(got[:, :2], want, rtol=1e-6, atol=1e-6)


def test_grouped_attention_maps_adjacent_query_groups_on_the_oracle(orc):
    """grouped_attention_maps_adjacent_query_groups (src/decoder.rs:7752-7776): two KV heads of width 1 with keys [1, 0] and
    [0, 1] and values [1, 10] and [-1, -10], four query heads of 1.0 in two groups of two, one query row that sees both
    positions: heads 0 and 1 give 0.7310586 * 1 + 0.2689414 * 10, heads 2 and 3 give -0.2689414 - 0.7310586 * 10."""
    keys = np.array([[[1.0], [0.0]], [[0.0], [1.0]]], np.float32)          # [token][kv head][d]
    values = np.array([[[1.0], [-1.0]], [[10.0], [-10.0]]], np.float32)
    k_pool, v_pool = pools(1, 2, 2, 1)
    scatter(k_pool, v_pool, [0], keys, values, 2)
    q = np.ones((1, 4), np.float32)
    first = np.float32(0.7310586) * 1.0 + np.float32(0.2689414) * 10.0
    second = -np.float32(0.2689414) - np.float32(0.7310586) * 10.0
    for mode in (1, 2):
        got = orc.paged_attention(q, k_pool, v_pool, [0], [0], [1], [1], q_heads=4, kv_heads=2, d=1, block_tokens=2, layers=1, layer=0,
                                  scale=1.0, softcap=0.0, mode=mode).reshape(4)
        assert np.max(np.abs(got - np.array([first, first, second, second], np.float32))) <= 1e-4
    assert np.max(np.abs(dense_gqa(q.reshape(1, 4, 1), keys, values, 1, 1.0)[0, :, 0] - [first, first, second, second])) <= 1e-4


def test_sliding_window_masks_expired_positions_in_prefill_and_decode_on_the_oracle(orc):
    """sliding_mask_applies_during_prefill_and_single_token_decode (src/decoder.rs:9524-9585): window 2. A decode row at position
    2 over keys 0..2 sees keys 1 and 2 only; in a three-row prefill row 0 sees key 0, row 1 keys 0-1, row 2 keys 1-2. With
    one-hot values the output of each row is the softmax weight of every key, so the masked cells read exactly 0."""
    d, bt, ctx = 1, 2, 3
    keys = np.zeros((ctx, 1, d), np.float32)                    # equal scores: the weights are uniform over what is visible
    values = np.zeros((ctx, 1, ctx), np.float32)
    k_pool, _ = pools(2, 1, bt, d)
    for p in range(ctx):
        k_pool[p // bt, 0, 0, p % bt] = keys[p]
    # the oracle's value rows have the key width, so each of the three "which key" indicators is run as its own value plane
    def weights(rows, start):
        out = np.zeros((rows, ctx), np.float32)
        for key in range(ctx):
            v_pool = np.zeros_like(k_pool)
            v_pool[key // bt, 0, 0, key % bt] = 1.0
            got = orc.paged_attention(np.ones((rows, 1), np.float32), k_pool, v_pool, [0, 1], [0], [start], [rows], q_heads=1, kv_heads=1, d=1,
                                      block_tokens=bt, layers=1, layer=0, scale=1.0, softcap=0.0, window=2, mode=2)
            out[:, key] = got[:, 0]
        return out
    decode = weights(1, 2)
    assert decode[0, 0] == 0.0 and np.allclose(decode[0, 1:], [0.5, 0.5], atol=1e-6)
    prefill = weights(3, 0)
    assert np.allclose(prefill, [[1.0, 0.0, 0.0], [0.5, 0.5, 0.0], [0.0, 0.5, 0.5]], atol=1e-6)
    assert prefill[0, 1] == 0.0 and prefill[2, 0] == 0.0
