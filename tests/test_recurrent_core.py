"""The per-thread steps the recurrent kernels are made of (macllm-infer_b200/csrc/recurrent_core.cuh), compiled for the host
and walked thread by thread with the kernels' state indexing, against the oracle: equal bit for bit, since both round every
product and sum on its own in the reference's order.  No GPU; the kernels themselves are compared in the GPU suite."""
import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def emu(tmp_path_factory):
    so = tmp_path_factory.mktemp("emu") / "librecurrent_emulation.so"
    cxx = "/usr/bin/g++" if os.access("/usr/bin/g++", os.X_OK) else "g++"
    subprocess.run([cxx, "-O2", "-std=c++17", "-fPIC", "-ffp-contract=off", "-fno-fast-math", "-shared", "-I", str(ROOT / "macllm-infer_b200" / "csrc"),
                    "-o", str(so), str(ROOT / "tests" / "recurrent_emulation.cpp")], check=True)
    return C.CDLL(str(so))


def p(a):
    return a.ctypes.data_as(C.c_void_p)


def ragged(rng, lens):
    return np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)


@pytest.mark.parametrize("variant,key_dim", [(0, 5), (0, 8), (1, 4), (1, 8)])
def test_gated_delta_threads_equal_the_oracle(emu, orc, variant, key_dim):
    rng = np.random.default_rng(key_dim + variant)
    heads, vd, lens = 3, 70, [5, 1, 0, 7]           # 70 columns: more than one CTA's 64; a lane with no rows keeps its state
    cu = ragged(rng, lens)
    rows = int(cu[-1])
    Q, K = (rng.standard_normal((2, rows, heads, key_dim)) * 0.4).astype(np.float32)
    V = rng.standard_normal((rows, heads, vd)).astype(np.float32)
    D = rng.uniform(0.5, 1.0, (rows, heads)).astype(np.float32)
    B = rng.uniform(0.0, 1.0, (rows, heads)).astype(np.float32)
    S = rng.standard_normal((len(lens), heads, key_dim, vd)).astype(np.float32)
    want_out, want_state = orc.gated_delta_recurrence(Q, K, V, D, B, S, cu)
    out, state = np.empty_like(want_out), np.empty_like(S)
    emu.emu_gated_delta(variant, p(Q), p(K), p(V), p(D), p(B), p(cu), len(lens), heads, key_dim, vd, p(S), p(state), p(out))
    assert np.array_equal(out, want_out) and np.array_equal(state, want_state)
    assert np.array_equal(state[2], S[2])


def test_gated_delta_decay_threads_equal_the_oracle(emu, orc):
    rng = np.random.default_rng(0)
    alpha = np.concatenate([rng.standard_normal((6, 4)).astype(np.float32) * 4, np.array([[100.0, -100.0, 0.0, 30.0]], np.float32)])
    bias = rng.standard_normal(4).astype(np.float32)
    sd = -rng.uniform(0.05, 1.0, 4).astype(np.float32)
    out = np.empty_like(alpha)
    emu.emu_gated_delta_decay(p(alpha), p(bias), p(sd), C.c_int64(alpha.shape[0]), 4, p(out))
    assert np.array_equal(out, orc.gated_delta_decay(alpha, bias, sd)) and np.isfinite(out).all()


@pytest.mark.parametrize("variant,state_size", [(0, 5), (1, 3)])
def test_mamba2_threads_equal_the_oracle(emu, orc, variant, state_size):
    rng = np.random.default_rng(10 + variant)
    heads, head_dim, groups, lens = 4, 6, 2, [3, 0, 4, 1]
    cu = ragged(rng, lens)
    rows = int(cu[-1])
    width = heads * head_dim + 2 * groups * state_size
    xbc = (rng.standard_normal((rows, width)) * 0.5).astype(np.float32)
    dt = np.concatenate([rng.standard_normal((rows - 1, heads)), [[100.0, -100.0, 0.0, 1.0]]]).astype(np.float32)
    bias, a, d = rng.standard_normal(heads).astype(np.float32) * 0.3, -rng.uniform(0.02, 0.5, heads).astype(np.float32), rng.standard_normal(heads).astype(np.float32)
    S = rng.standard_normal((len(lens), heads, head_dim, state_size)).astype(np.float32)
    want_out, want_state = orc.mamba2_scan(xbc, dt, bias, a, d, S, cu)
    out, state = np.empty_like(want_out), np.empty_like(S)
    emu.emu_mamba2(variant, p(xbc), p(dt), p(bias), p(a), p(d), p(cu), len(lens), heads, head_dim, state_size, groups, p(S), p(state), p(out))
    assert np.array_equal(out, want_out) and np.array_equal(state, want_state)


@pytest.mark.parametrize("K", [1, 3, 4])
def test_short_convolution_threads_equal_the_oracle(emu, orc, K):
    rng = np.random.default_rng(K)
    hidden, lens = 10, [4, 1, 0, 2, 6]              # lanes shorter than the window take part of their new tail from the old one
    cu = ragged(rng, lens)
    rows = int(cu[-1])
    bcx = rng.standard_normal((rows, 3 * hidden)).astype(np.float32)
    kernel = rng.standard_normal((hidden, K)).astype(np.float32)
    tail = rng.standard_normal((len(lens), K - 1, hidden)).astype(np.float32)
    want_out, want_tail = orc.short_conv(bcx, kernel, tail, cu)
    out, nxt = np.empty_like(want_out), np.empty_like(tail)
    emu.emu_short_conv(p(bcx), p(kernel), p(cu), len(lens), hidden, K, p(tail), p(nxt), p(out))
    assert np.array_equal(out, want_out) and np.array_equal(nxt, want_tail)
