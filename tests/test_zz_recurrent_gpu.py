"""The recurrent mixers' sm_100a kernels against the oracle, through the C ABI (mk_k_gated_delta_decay,
mk_k_gated_delta_recurrence, mk_k_mamba2_scan, mk_k_short_conv): the reference's known answers first
(crates/macllm-kernels/src/gated_delta.rs:756-870, crates/macllm-kernels/src/mamba2.rs:692-776, src/decoder.rs:6673-6754), then
ragged batches at the sizes the register kernels are built for.

Tolerances.  The delta-rule recurrence and the short convolution take their controls as inputs and round every product and sum
on its own in the reference's order: bit-exact.  The decay controls and the Mamba2 scan evaluate exp and log1p on the device,
whose last bit may differ from the host library's: 2e-6 relative to the largest magnitude of the compared tensor."""
import importlib

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(mk):
    return importlib.import_module("macllm_infer_b200.ops")


def close(got, want, rel=2e-6):
    scale = max(1.0, float(np.max(np.abs(want))))
    err = float(np.max(np.abs(got - want)))
    assert np.isfinite(got).all() and err <= rel * scale, (err, scale)


def exact(got, want):
    assert np.array_equal(got, want), float(np.max(np.abs(got - want)))


def cu_of(lens):
    return np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)


def test_gated_delta_known_answers(ops, orc):
    alpha = np.array([[-3.0, 1.5], [20.0, -20.0]], np.float32)
    bias, sd = np.array([0.25, -0.5], np.float32), np.array([-0.75, -0.125], np.float32)
    close(ops.gated_delta_decay(alpha, bias, sd), orc.gated_delta_decay(alpha, bias, sd), 1e-6)
    out, state = ops.gated_delta_recurrence(np.array([[[0.5, -1.0]]]), np.array([[[0.25, 0.75]]]), np.array([[[1.0, 2.0]]]),
                                            np.array([[0.8]]), np.array([[0.5]]), np.array([[[[1.0, 2.0], [3.0, 4.0]]]]))
    assert np.max(np.abs(state.reshape(-1) - np.array([0.675, 1.5, 2.025, 2.9], np.float32))) <= 1e-6
    assert np.max(np.abs(out.reshape(-1) - np.array([-1.6875, -2.15], np.float32))) <= 1e-6


@pytest.mark.parametrize("key_dim,value_dim", [(128, 128), (64, 96), (24, 70)])
def test_gated_delta_recurrence_ragged_batch(ops, orc, key_dim, value_dim):
    """Register kernels (key_dim 128 and 64) and the in-place kernel (any key_dim); value_dim 96 and 70 leave a partly filled
    CTA; lanes of 9, 1, 0 and 30 rows: prefill chunks, a decode lane and a lane that only carries its state through."""
    rng = np.random.default_rng(key_dim)
    heads, lens = 4, [9, 1, 0, 30]
    cu = cu_of(lens)
    rows = int(cu[-1])
    Q, K = (rng.standard_normal((2, rows, heads, key_dim)) / np.sqrt(key_dim)).astype(np.float32)
    V = rng.standard_normal((rows, heads, value_dim)).astype(np.float32)
    D = rng.uniform(0.6, 1.0, (rows, heads)).astype(np.float32)
    B = rng.uniform(0.0, 1.0, (rows, heads)).astype(np.float32)
    S = rng.standard_normal((len(lens), heads, key_dim, value_dim)).astype(np.float32)
    before = S.copy()
    want_out, want_state = orc.gated_delta_recurrence(Q, K, V, D, B, S, cu)
    out, state = ops.gated_delta_recurrence(Q, K, V, D, B, S, cu)
    exact(out, want_out)
    exact(state, want_state)
    exact(state[2], S[2])
    exact(S, before)
    # the 30-row lane in chunks of 16 and 14 from the carried state: the same rows and the same final state
    a, b = int(cu[3]), int(cu[4])
    o1, s1 = ops.gated_delta_recurrence(Q[a:a + 16], K[a:a + 16], V[a:a + 16], D[a:a + 16], B[a:a + 16], S[3:4])
    o2, s2 = ops.gated_delta_recurrence(Q[a + 16:b], K[a + 16:b], V[a + 16:b], D[a + 16:b], B[a + 16:b], s1)
    exact(np.concatenate([o1, o2]), out[a:b])
    exact(s2, state[3:4])


def test_gated_delta_decay_extremes(ops, orc):
    rng = np.random.default_rng(1)
    alpha = np.concatenate([rng.standard_normal((63, 8)).astype(np.float32) * 4, np.array([[100.0, -100.0, 0.0, 30.0, -30.0, 88.0, -88.0, 1e-8]], np.float32)])
    bias = rng.standard_normal(8).astype(np.float32)
    sd = -rng.uniform(0.05, 1.0, 8).astype(np.float32)
    close(ops.gated_delta_decay(alpha, bias, sd), orc.gated_delta_decay(alpha, bias, sd))


def test_mamba2_known_fixture_chunking_and_decode(ops, orc):
    """mamba2.rs:520-572,692-776: the reference's fixture (3 tokens, 4 heads of 2 positions, state 3, 2 groups, dt of +-100)."""
    T, H, P, N, G = 3, 4, 2, 3, 2
    inner, gsw = H * P, G * N
    xbc = []
    for token in range(T):
        xbc += [((token * 11 + i * 7) % 19) * 0.07 - 0.5 for i in range(inner)]
        xbc += [((token * 5 + i * 3) % 13) * 0.04 - 0.2 for i in range(gsw)]
        xbc += [((token * 7 + i * 5) % 17) * 0.03 - 0.18 for i in range(gsw)]
    f = lambda v: np.array(v, np.float32)
    xbc = f(xbc).reshape(T, inner + 2 * gsw)
    dt = f([100.0, -100.0, 0.2, -0.7, -1.3, 0.9, 1.4, -0.2, 0.0, 0.4, -0.8, 1.1]).reshape(T, H)
    bias, a, d = f([-0.15, 0.25, -0.4, 0.05]), f([-0.03, -0.2, -0.45, -0.1]), f([0.2, -0.3, 0.5, 0.1])
    S = f([(i - 11.0) * 0.015 for i in range(inner * N)]).reshape(1, H, P, N)
    want_out, want_state = orc.mamba2_scan(xbc, dt, bias, a, d, S)
    out, state = ops.mamba2_scan(xbc, dt, bias, a, d, S)
    close(out, want_out)
    close(state, want_state)
    o1, s1 = ops.mamba2_scan(xbc[:2], dt[:2], bias, a, d, S)
    o2, s2 = ops.mamba2_scan(xbc[2:], dt[2:], bias, a, d, s1)
    exact(np.concatenate([o1, o2]), out)
    exact(s2, state)


@pytest.mark.parametrize("head_dim,state_size,groups", [(64, 128, 1), (64, 64, 2), (40, 16, 4), (12, 20, 2)])
def test_mamba2_scan_ragged_batch(ops, orc, head_dim, state_size, groups):
    """Register kernels (state 128, 64, 16) and the in-place kernel (state 20); head_dim 40 and 12 leave idle threads."""
    rng = np.random.default_rng(state_size)
    heads, lens = 8, [7, 1, 0, 21]
    cu = cu_of(lens)
    rows = int(cu[-1])
    width = heads * head_dim + 2 * groups * state_size
    xbc = (rng.standard_normal((rows, width)) * 0.5).astype(np.float32)
    dt = rng.standard_normal((rows, heads)).astype(np.float32)
    bias = (rng.standard_normal(heads) * 0.3).astype(np.float32)
    a = -rng.uniform(0.02, 0.5, heads).astype(np.float32)
    d = rng.standard_normal(heads).astype(np.float32)
    S = rng.standard_normal((len(lens), heads, head_dim, state_size)).astype(np.float32)
    want_out, want_state = orc.mamba2_scan(xbc, dt, bias, a, d, S, cu)
    out, state = ops.mamba2_scan(xbc, dt, bias, a, d, S, cu)
    close(out, want_out, 1e-5)
    close(state, want_state, 1e-5)
    exact(state[2], S[2])


def test_short_convolution_known_answer_and_ragged_batch(ops, orc):
    x = np.array([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]], np.float32)
    bcx = np.concatenate([x, x, x], axis=1)
    kernel = np.array([[1.0, 10.0, 100.0], [-1.0, 0.5, 2.0]], np.float32)
    out, tail = ops.short_conv(bcx, kernel, np.zeros((1, 2, 2), np.float32))
    exact(out, np.array([[100.0, 16.0], [2730.0, 136.0], [12955.0, 456.0]], np.float32))
    exact(tail, np.array([[[9.0, 16.0], [25.0, 36.0]]], np.float32))
    rng = np.random.default_rng(5)
    for K in (1, 3, 4):
        hidden, lens = 1536, [33, 1, 0, 2, 100]
        cu = cu_of(lens)
        rows = int(cu[-1])
        bcx = rng.standard_normal((rows, 3 * hidden)).astype(np.float32)
        kernel = rng.standard_normal((hidden, K)).astype(np.float32)
        tail = rng.standard_normal((len(lens), K - 1, hidden)).astype(np.float32)
        want_out, want_tail = orc.short_conv(bcx, kernel, tail, cu)
        out, nxt = ops.short_conv(bcx, kernel, tail, cu)
        exact(out, want_out)
        exact(nxt, want_tail)


def test_geometry_refusals_come_back_as_errors(ops, mk):
    capi = importlib.import_module("macllm_infer_b200._capi")
    z = lambda *s: np.zeros(s, np.float32)
    with pytest.raises(capi.MkError, match="cannot encode paired B/C states of width 3"):
        ops.mamba2_scan(z(2, 8 + 7), z(2, 4), z(4), z(4), z(4), z(1, 4, 2, 3))
    with pytest.raises(capi.MkError, match="head count 4 is not divisible by inferred group count 3"):
        ops.mamba2_scan(z(2, 8 + 18), z(2, 4), z(4), z(4), z(4), z(1, 4, 2, 3))
    with pytest.raises(capi.MkError, match="kernel size 9 exceeds 8"):
        ops.short_conv(z(2, 6), z(2, 9), z(1, 8, 2))
    with pytest.raises(capi.MkError, match="lane boundaries must rise"):
        ops.gated_delta_recurrence(z(2, 1, 4), z(2, 1, 4), z(2, 1, 4), z(2, 1), z(2, 1), z(2, 1, 4, 4), [0, 3, 2])


def test_launch_times_of_a_decode_tick_and_a_prefill_chunk(ops):
    """CUDA-event time per launch at the shapes the register kernels are built for; the state is read once and written once per
    launch, so a decode tick of 64 lanes moves 2 x 134 MB of state and little else.  Printed for the record (run with -s); the
    assertion only says that the launches ran."""
    cases = (("gated_delta", 64, 1, 32, 128, 128), ("gated_delta", 1, 512, 32, 128, 128),
             ("mamba2", 64, 1, 64, 64, 128), ("mamba2", 1, 512, 64, 64, 128))
    for kind, lanes, rows, heads, dim_a, dim_b in cases:
        ms, nbytes = ops.recurrent_time(kind, lanes, rows, heads, dim_a, dim_b, iters=10)
        assert ms > 0.0 and nbytes == 2.0 * lanes * heads * dim_a * dim_b * 4
        print(f"RECURRENT_TIME {kind} lanes={lanes} rows_per_lane={rows} heads={heads} dims={dim_a}x{dim_b}: {ms * 1e3:.1f} us per launch, "
              f"state {nbytes / 1e6:.1f} MB -> {nbytes / ms / 1e6:.0f} GB/s")
