"""The recurrent mixers' arithmetic, restated in the oracle and pinned to the reference's own known answers: Gated DeltaNet
decay and recurrence (crates/macllm-kernels/src/gated_delta.rs:756-870), the Mamba2 selective scan against a scalar loop on
the reference's fixture (crates/macllm-kernels/src/mamba2.rs:520-776), and the short convolution's hand calculation
(src/decoder.rs:6673-6754).  CPU only."""
import math

import numpy as np
import pytest


def test_gated_delta_decay_matches_the_stable_scalar_formula(orc):
    """gated_delta.rs:756-777."""
    alpha = np.array([[-3.0, 1.5], [20.0, -20.0]], np.float32)
    bias = np.array([0.25, -0.5], np.float32)
    state_decay = np.array([-0.75, -0.125], np.float32)
    got = orc.gated_delta_decay(alpha, bias, state_decay).reshape(-1)
    for i, value in enumerate(got):
        h = i % 2
        shifted = float(alpha.reshape(-1)[i] + bias[h])
        softplus = max(shifted, 0.0) + math.log1p(math.exp(-abs(shifted)))
        assert abs(value - math.exp(softplus * float(state_decay[h]))) <= 1e-7
    with pytest.raises(ValueError, match="alpha shape \\[2, 2\\], time bias \\[3\\]"):
        orc.gated_delta_decay(alpha, np.zeros(3, np.float32), state_decay)


def test_gated_delta_recurrence_matches_the_scalar_golden(orc):
    """gated_delta.rs:779-809: one head, key_dim 2, value_dim 2, state [[1, 2], [3, 4]] - next state 0.675 1.5 2.025 2.9 and
    output -1.6875 -2.15."""
    out, state = orc.gated_delta_recurrence(np.array([[[0.5, -1.0]]]), np.array([[[0.25, 0.75]]]), np.array([[[1.0, 2.0]]]),
                                            np.array([[0.8]]), np.array([[0.5]]), np.array([[[[1.0, 2.0], [3.0, 4.0]]]]))
    assert np.max(np.abs(state.reshape(-1) - np.array([0.675, 1.5, 2.025, 2.9], np.float32))) <= 1e-6
    assert np.max(np.abs(out.reshape(-1) - np.array([-1.6875, -2.15], np.float32))) <= 1e-6


def test_gated_delta_prefill_equals_sequential_steps_and_lanes_do_not_mix(orc):
    """gated_delta.rs:811-870, and the decoder's ragged case (src/decoder.rs:7106-7174): two tokens at once equal two single
    steps bit for bit; a lane in a ragged batch equals the same lane alone."""
    q = np.array([[[0.5, -1.0]], [[0.25, 0.75]]], np.float32)
    k = np.array([[[0.25, 0.75]], [[-0.5, 0.5]]], np.float32)
    v = np.array([[[1.0, 2.0]], [[-1.0, 0.5]]], np.float32)
    decay = np.array([[0.8], [0.9]], np.float32)
    beta = np.array([[0.5], [0.25]], np.float32)
    s0 = np.array([[[[1.0, 2.0], [3.0, 4.0]]]], np.float32)
    one_out, one_state = orc.gated_delta_recurrence(q, k, v, decay, beta, s0)
    state, outs = s0, []
    for t in range(2):
        o, state = orc.gated_delta_recurrence(q[t:t + 1], k[t:t + 1], v[t:t + 1], decay[t:t + 1], beta[t:t + 1], state)
        outs.append(o)
    assert np.array_equal(one_out, np.concatenate(outs)) and np.array_equal(one_state, state)
    assert np.array_equal(s0, np.array([[[[1.0, 2.0], [3.0, 4.0]]]], np.float32))      # the input state is left as it was
    rng = np.random.default_rng(3)
    heads, kd, vd, lens = 3, 8, 5, [4, 1, 6]
    rows = sum(lens)
    Q, K = rng.standard_normal((2, rows, heads, kd)).astype(np.float32) * 0.3
    V = rng.standard_normal((rows, heads, vd)).astype(np.float32)
    D = rng.uniform(0.5, 1.0, (rows, heads)).astype(np.float32)
    B = rng.uniform(0.0, 1.0, (rows, heads)).astype(np.float32)
    S = rng.standard_normal((3, heads, kd, vd)).astype(np.float32)
    cu = np.concatenate([[0], np.cumsum(lens)])
    out, nxt = orc.gated_delta_recurrence(Q, K, V, D, B, S, cu)
    for l in range(3):
        a, b = cu[l], cu[l + 1]
        o, s = orc.gated_delta_recurrence(Q[a:b], K[a:b], V[a:b], D[a:b], B[a:b], S[l:l + 1])
        assert np.array_equal(out[a:b], o) and np.array_equal(nxt[l:l + 1], s)
    with pytest.raises(ValueError, match="incompatible query/key geometry"):
        orc.gated_delta_recurrence(Q, K[:, :, :4], V, D, B, S, cu)


# the reference's fixture (mamba2.rs:520-572)
TOKENS, HEADS, HEAD_DIM, STATE_SIZE, GROUPS = 3, 4, 2, 3, 2
INNER, GSW = HEADS * HEAD_DIM, GROUPS * STATE_SIZE


def mamba2_fixture():
    xbc = []
    for token in range(TOKENS):
        xbc += [((token * 11 + i * 7) % 19) * 0.07 - 0.5 for i in range(INNER)]
        xbc += [((token * 5 + i * 3) % 13) * 0.04 - 0.2 for i in range(GSW)]
        xbc += [((token * 7 + i * 5) % 17) * 0.03 - 0.18 for i in range(GSW)]
    f = lambda v: np.array(v, np.float32)
    return dict(xbc=f(xbc).reshape(TOKENS, INNER + 2 * GSW),
                raw_dt=f([100.0, -100.0, 0.2, -0.7, -1.3, 0.9, 1.4, -0.2, 0.0, 0.4, -0.8, 1.1]).reshape(TOKENS, HEADS),
                dt_bias=f([-0.15, 0.25, -0.4, 0.05]), a=f([-0.03, -0.2, -0.45, -0.1]), d=f([0.2, -0.3, 0.5, 0.1]),
                state=f([(i - 11.0) * 0.015 for i in range(INNER * STATE_SIZE)]).reshape(1, HEADS, HEAD_DIM, STATE_SIZE))


def scalar_scan(fx, tokens):
    """The scalar loop of the reference's test (mamba2.rs:632-668), in float32 step by step."""
    f = np.float32
    state = fx["state"].reshape(-1).copy()
    out = np.zeros(tokens * INNER, np.float32)
    hpg = HEADS // GROUPS
    for token in range(tokens):
        row = fx["xbc"][token]
        for head in range(HEADS):
            shifted = f(fx["raw_dt"][token, head] + fx["dt_bias"][head])
            delta = f(max(shifted, f(0)) + f(math.log1p(f(math.exp(-abs(shifted))))))
            decay = f(math.exp(f(delta * fx["a"][head])))
            b0 = INNER + (head // hpg) * STATE_SIZE
            c0 = INNER + GSW + (head // hpg) * STATE_SIZE
            for pos in range(HEAD_DIM):
                lane = head * HEAD_DIM + pos
                value = row[lane]
                projected = f(0)
                for n in range(STATE_SIZE):
                    i = lane * STATE_SIZE + n
                    state[i] = f(f(decay * state[i]) + f(f(delta * value) * row[b0 + n]))
                    projected = f(projected + f(state[i] * row[c0 + n]))
                out[token * INNER + lane] = f(projected + f(fx["d"][head] * value))
    return out, state


def test_mamba2_scan_handles_extreme_dt_chunking_decode_and_final_state(orc):
    """mamba2.rs:692-776: the whole sequence against the scalar loop (dt of +-100 locks the stable softplus), then a two-token
    chunk followed by a one-token decode from the chunk's state; the initial state is not modified."""
    fx = mamba2_fixture()
    before = fx["state"].copy()
    out, state = orc.mamba2_scan(fx["xbc"], fx["raw_dt"], fx["dt_bias"], fx["a"], fx["d"], fx["state"])
    want_out, want_state = scalar_scan(fx, TOKENS)
    assert np.isfinite(out).all() and np.isfinite(state).all()
    assert np.max(np.abs(out.reshape(-1) - want_out)) <= 1e-6 and np.max(np.abs(state.reshape(-1) - want_state)) <= 1e-6
    o1, s1 = orc.mamba2_scan(fx["xbc"][:2], fx["raw_dt"][:2], fx["dt_bias"], fx["a"], fx["d"], fx["state"])
    o2, s2 = orc.mamba2_scan(fx["xbc"][2:], fx["raw_dt"][2:], fx["dt_bias"], fx["a"], fx["d"], s1)
    assert np.array_equal(np.concatenate([o1, o2]), out) and np.array_equal(s2, state)
    assert np.array_equal(fx["state"], before)
    # two lanes in one call: the sequence twice, the second from another state
    other = (fx["state"] * np.float32(-0.5)).astype(np.float32)
    both_out, both_state = orc.mamba2_scan(np.concatenate([fx["xbc"], fx["xbc"][:1]]), np.concatenate([fx["raw_dt"], fx["raw_dt"][:1]]),
                                           fx["dt_bias"], fx["a"], fx["d"], np.concatenate([fx["state"], other]), [0, 3, 4])
    lone_out, lone_state = orc.mamba2_scan(fx["xbc"][:1], fx["raw_dt"][:1], fx["dt_bias"], fx["a"], fx["d"], other)
    assert np.array_equal(both_out[:3], out) and np.array_equal(both_out[3:], lone_out)
    assert np.array_equal(both_state[:1], state) and np.array_equal(both_state[1:], lone_state)


def test_mamba2_geometry_refusals(orc):
    """ScanGeometry::validate (mamba2.rs:64-150)."""
    assert orc.mamba2_geometry(INNER + 2 * GSW, HEADS, HEAD_DIM, STATE_SIZE) == GROUPS
    with pytest.raises(ValueError, match="xBC width 7 is smaller than inner size 8"):
        orc.mamba2_geometry(7, HEADS, HEAD_DIM, STATE_SIZE)
    with pytest.raises(ValueError, match="cannot encode paired B/C states of width 3"):
        orc.mamba2_geometry(INNER + 7, HEADS, HEAD_DIM, STATE_SIZE)
    with pytest.raises(ValueError, match="head count 4 is not divisible by inferred group count 3"):
        orc.mamba2_geometry(INNER + 2 * 3 * STATE_SIZE, HEADS, HEAD_DIM, STATE_SIZE)
    with pytest.raises(ValueError, match="non-empty dimensions"):
        orc.mamba2_geometry(8, 0, HEAD_DIM, STATE_SIZE)


def test_short_convolution_matches_the_hand_calculation_and_chunked_state(orc):
    """src/decoder.rs:6673-6754: B = C = x = the input rows [1, 2], [3, 4], [5, 6], kernel rows [1, 10, 100] and [-1, 0.5, 2]:
    outputs [100, 16], [2730, 136], [12955, 456]; the tail keeps the last two B*x rows [9, 16], [25, 36]; one token then two
    give the same outputs and tail."""
    x = np.array([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]], np.float32)
    bcx = np.concatenate([x, x, x], axis=1)
    kernel = np.array([[1.0, 10.0, 100.0], [-1.0, 0.5, 2.0]], np.float32)
    zero_tail = np.zeros((1, 2, 2), np.float32)
    out, tail = orc.short_conv(bcx, kernel, zero_tail)
    assert np.array_equal(out, np.array([[100.0, 16.0], [2730.0, 136.0], [12955.0, 456.0]], np.float32))
    assert np.array_equal(tail, np.array([[[9.0, 16.0], [25.0, 36.0]]], np.float32))
    o1, t1 = orc.short_conv(bcx[:1], kernel, zero_tail)
    o2, t2 = orc.short_conv(bcx[1:], kernel, t1)
    assert np.array_equal(np.concatenate([o1, o2]), out) and np.array_equal(t2, tail)
    assert np.array_equal(t1, np.array([[[0.0, 0.0], [1.0, 4.0]]], np.float32))
    # ragged lanes keep their own tails (src/decoder.rs:6847-6921)
    both, tails = orc.short_conv(np.concatenate([bcx, bcx[1:]]), kernel, np.concatenate([zero_tail, t1]), [0, 3, 5])
    assert np.array_equal(both[:3], out) and np.array_equal(both[3:], o2) and np.array_equal(tails, np.concatenate([tail, t2]))
    with pytest.raises(ValueError, match="short-convolution tail has shape \\[1, 1, 2\\], expected \\[1, 2, 2\\]"):
        orc.short_conv(bcx, kernel, np.zeros((1, 1, 2), np.float32))
