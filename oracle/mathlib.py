"""ctypes/NumPy front of oracle_math.cpp (the C++ restatement of the reference's CPU arithmetic).

TEST INFRASTRUCTURE ONLY - see oracle/__init__.py.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "liboracle_math.so"

F32, F16, Q8_0, Q4_K, Q6_K = 0, 1, 8, 12, 14

_lib = None


def build(force: bool = False) -> Path:
    src = HERE / "oracle_math.cpp"
    if force or not LIB.exists() or LIB.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "-B" if force else "-s", "liboracle_math.so"], check=True,
                       capture_output=True)
    return LIB


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB.exists():
            build()
        h = C.CDLL(str(LIB))
        h.orc_row_bytes.restype = C.c_int64
        h.orc_row_bytes.argtypes = [C.c_int, C.c_int64]
        h.orc_argmax.restype = C.c_int64
        h.orc_f16_to_f32.restype = C.c_float
        h.orc_f16_to_f32.argtypes = [C.c_uint16]
        h.orc_f32_to_f16.restype = C.c_uint16
        h.orc_f32_to_f16.argtypes = [C.c_float]
        h.orc_num_threads.restype = C.c_int
        _lib = h
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def row_bytes(t: int, cols: int) -> int:
    return int(lib().orc_row_bytes(t, C.c_int64(cols)))


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    """Threads of the oracle's OpenMP loops from now on (torchrun exports OMP_NUM_THREADS=1)."""
    lib().orc_set_num_threads(int(n))


def dequant(t: int, w: np.ndarray, rows: int, cols: int) -> np.ndarray:
    w = np.ascontiguousarray(w)
    out = np.empty((rows, cols), dtype=np.float32)
    lib().orc_dequant(t, _p(w), C.c_int64(rows), C.c_int64(cols), _p(out))
    return out


def quantize_q8k(x: np.ndarray):
    x = _f32(x)
    T, K = x.shape
    qs = np.empty((T, K), np.int8)
    d = np.empty((T, K // 256), np.float32)
    bs = np.empty((T, K // 16), np.int16)
    for t in range(T):
        lib().orc_quantize_q8k(_p(x[t]), C.c_int64(K), _p(qs[t]), _p(d[t]), _p(bs[t]))
    return qs, d, bs


def quantize_q80(x: np.ndarray):
    x = _f32(x)
    T, K = x.shape
    qs = np.empty((T, K), np.int8)
    d = np.empty((T, K // 32), np.uint16)
    for t in range(T):
        lib().orc_quantize_q80(_p(x[t]), C.c_int64(K), _p(qs[t]), _p(d[t]))
    return qs, d.view(np.float16).astype(np.float32)


def qmatmul(t: int, w: np.ndarray, rows: int, cols: int, x: np.ndarray, mode: int = 1) -> np.ndarray:
    """y [T, rows] = x [T, cols] . W^T ; mode 1 = 8-bit activation blocks + integer dots, 2 = dequantised f32."""
    x = _f32(x)
    w = np.ascontiguousarray(w)
    T = x.shape[0]
    y = np.empty((T, rows), dtype=np.float32)
    lib().orc_qmatmul(t, _p(w), C.c_int64(rows), C.c_int64(cols), _p(x), C.c_int64(T), _p(y), mode)
    return y


def fake_quant_rows(t: int, x: np.ndarray) -> np.ndarray:
    x = _f32(x)
    out = np.empty_like(x)
    lib().orc_fake_quant_rows(t, _p(x), C.c_int64(x.shape[0]), C.c_int64(x.shape[1]), _p(out))
    return out


def embed(t: int, w: np.ndarray, cols: int, ids, scale: float = 1.0) -> np.ndarray:
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    w = np.ascontiguousarray(w)
    out = np.empty((len(ids), cols), dtype=np.float32)
    lib().orc_embed(t, _p(w), C.c_int64(cols), _p(ids), C.c_int64(len(ids)), C.c_float(scale), _p(out))
    return out


def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    x = _f32(x)
    w = _f32(w)
    rows, dim = x.shape
    y = np.empty_like(x)
    lib().orc_rmsnorm(_p(x), _p(w), C.c_float(eps), C.c_int64(rows), C.c_int64(dim), _p(y))
    return y


def act_mul(gate: np.ndarray, up: np.ndarray, act: int) -> np.ndarray:
    gate, up = _f32(gate), _f32(up)
    out = np.empty_like(gate)
    lib().orc_act_mul(_p(gate), _p(up), C.c_int64(gate.size), act, _p(out))
    return out


def softcap(x: np.ndarray, cap: float) -> np.ndarray:
    x = _f32(x).copy()
    lib().orc_softcap(_p(x), C.c_int64(x.size), C.c_float(cap))
    return x


def rope_tables(theta: float, rotary_dim: int, capacity: int, factors=None):
    cos = np.empty((capacity, rotary_dim // 2), np.float32)
    sin = np.empty_like(cos)
    f = _f32(factors) if factors is not None else None
    lib().orc_rope_tables(C.c_double(theta), rotary_dim, C.c_int64(capacity), _p(f) if f is not None else None, _p(cos), _p(sin))
    return cos, sin


def rope_apply(x: np.ndarray, heads: int, d: int, rotary_dim: int, pos, cos, sin) -> np.ndarray:
    """x [T, heads*d]; returns rotated copy."""
    x = _f32(x).copy()
    pos = np.ascontiguousarray(pos, dtype=np.int32)
    lib().orc_rope_apply(_p(x), C.c_int64(x.shape[0]), heads, d, rotary_dim, _p(pos), _p(cos), _p(sin))
    return x


def kv_scatter(k, v, k_pool, v_pool, slots, kv_heads, d, block_tokens, layers, layer):
    k, v = _f32(k), _f32(v)
    slots = np.ascontiguousarray(slots, dtype=np.int64)
    f16 = 1 if k_pool.dtype == np.float16 else 0
    lib().orc_kv_scatter(_p(k), _p(v), _p(k_pool), _p(v_pool), f16, _p(slots), C.c_int64(len(slots)), kv_heads, d,
                         block_tokens, layers, layer)


def paged_attention(q, k_pool, v_pool, page_table, page_off, start_pos, lane_len, *, q_heads, kv_heads, d, block_tokens,
                    layers, layer, scale, softcap=0.0, window=0, mode=1) -> np.ndarray:
    q = _f32(q)
    out = np.empty_like(q)
    pt = np.ascontiguousarray(page_table, dtype=np.uint32)
    po = np.ascontiguousarray(page_off, dtype=np.int32)
    sp = np.ascontiguousarray(start_pos, dtype=np.int32)
    ll = np.ascontiguousarray(lane_len, dtype=np.int32)
    f16 = 1 if k_pool.dtype == np.float16 else 0
    lib().orc_paged_attention(_p(q), _p(out), _p(k_pool), _p(v_pool), f16, _p(pt), _p(po), _p(sp), _p(ll), len(ll), q_heads,
                              kv_heads, d, block_tokens, layers, layer, C.c_float(scale), C.c_float(softcap), window, mode)
    return out


def moe_route(logits: np.ndarray, k: int):
    """selected_softmax_routes (src/decoder.rs:448-554), with its refusals (:453-483)."""
    logits = _f32(logits)
    T, E = logits.shape
    if k == 0 or k > E:
        raise ValueError(f"experts per token {k} must be in 1..={E}")
    bad = np.flatnonzero(~np.isfinite(logits).all(axis=1))
    if bad.size:
        raise ValueError(f"router produced non-finite logits for token row {int(bad[0])}")
    sel = np.empty((T, k), np.int32)
    w = np.empty((T, k), np.float32)
    lib().orc_moe_route(_p(logits), C.c_int64(T), E, k, _p(sel), _p(w))
    return sel, w


def _cu(cu_seqlens, rows):
    cu = np.ascontiguousarray(cu_seqlens, dtype=np.int32)
    if cu.ndim != 1 or cu.size < 2 or cu[0] != 0 or cu[-1] != rows or np.any(np.diff(cu) < 0):
        raise ValueError("lane boundaries must rise from 0 to the number of rows")
    return cu


def gated_delta_decay(alpha, time_bias, state_decay) -> np.ndarray:
    """exp(softplus(alpha + time_bias) * state_decay) for alpha [tokens, heads] (crates/macllm-kernels/src/gated_delta.rs:13-60,96-104)."""
    alpha, time_bias, state_decay = _f32(alpha), _f32(time_bias), _f32(state_decay)
    if alpha.ndim != 2 or 0 in alpha.shape:
        raise ValueError("Gated DeltaNet decay requires non-empty token and head dimensions")
    if time_bias.shape != (alpha.shape[1],) or state_decay.shape != (alpha.shape[1],):
        raise ValueError(f"Gated DeltaNet decay has alpha shape {list(alpha.shape)}, time bias {list(time_bias.shape)} and state decay {list(state_decay.shape)}")
    out = np.empty_like(alpha)
    lib().orc_gated_delta_decay(_p(alpha), _p(time_bias), _p(state_decay), C.c_int64(alpha.shape[0]), alpha.shape[1], _p(out))
    return out


def gated_delta_recurrence(query, key, value, decay, beta, state, cu_seqlens=None):
    """query / key [rows, heads, key_dim], value [rows, heads, value_dim], decay / beta [rows, heads], state
    [lanes, heads, key_dim, value_dim]; returns (out [rows, heads, value_dim], next state).  One lane unless `cu_seqlens`
    says otherwise (crates/macllm-kernels/src/gated_delta.rs:139-170,236-270,396-431)."""
    query, key, value, decay, beta, state = (_f32(t) for t in (query, key, value, decay, beta, state))
    rows, heads, key_dim = query.shape
    if heads == 0 or key_dim == 0 or key.shape != query.shape:
        raise ValueError("Gated DeltaNet decode has incompatible query/key geometry")
    value_dim = value.shape[2] if value.ndim == 3 else 0
    cu = _cu([0, rows] if cu_seqlens is None else cu_seqlens, rows)
    lanes = cu.size - 1
    if (value.shape[:2] != (rows, heads) or value_dim == 0 or decay.shape != (rows, heads) or beta.shape != (rows, heads)
            or state.shape != (lanes, heads, key_dim, value_dim)):
        raise ValueError(f"Gated DeltaNet decode has query {list(query.shape)}, key {list(key.shape)}, value {list(value.shape)}, "
                         f"decay {list(decay.shape)}, beta {list(beta.shape)} and state {list(state.shape)}")
    out = np.empty((rows, heads, value_dim), np.float32)
    nxt = np.empty_like(state)
    lib().orc_gated_delta_recurrence(_p(query), _p(key), _p(value), _p(decay), _p(beta), _p(cu), lanes, heads, key_dim, value_dim,
                                     _p(state), _p(nxt), _p(out))
    return out, nxt


def mamba2_geometry(xbc_width: int, heads: int, head_dim: int, state_size: int) -> int:
    """The group count a projection width implies, with the refusals of ScanGeometry::validate
    (crates/macllm-kernels/src/mamba2.rs:64-150)."""
    if min(heads, head_dim, state_size) <= 0:
        raise ValueError("Mamba2 scan requires non-empty dimensions")
    inner = heads * head_dim
    if xbc_width < inner:
        raise ValueError(f"Mamba2 xBC width {xbc_width} is smaller than inner size {inner}")
    bc = xbc_width - inner
    if bc == 0 or bc % (2 * state_size) != 0:
        raise ValueError(f"Mamba2 xBC width {xbc_width} cannot encode paired B/C states of width {state_size}")
    groups = bc // (2 * state_size)
    if heads % groups != 0:
        raise ValueError(f"Mamba2 scan head count {heads} is not divisible by inferred group count {groups}")
    return groups


def mamba2_scan(xbc, raw_dt, dt_bias, a, d, state, cu_seqlens=None):
    """xbc [rows, H*P + 2*G*N] laid out [x | B | C], raw_dt [rows, H], dt_bias / a / d [H], state [lanes, H, P, N]; returns
    (out [rows, H, P], final state) (crates/macllm-kernels/src/mamba2.rs:17-150,255-289)."""
    xbc, raw_dt, dt_bias, a, d, state = (_f32(t) for t in (xbc, raw_dt, dt_bias, a, d, state))
    rows, width = xbc.shape
    cu = _cu([0, rows] if cu_seqlens is None else cu_seqlens, rows)
    lanes = cu.size - 1
    if state.ndim != 4 or state.shape[0] != lanes:
        raise ValueError("Mamba2 scan state must be [lanes, heads, head_dim, state_size]")
    _, heads, head_dim, state_size = state.shape
    if rows == 0:
        raise ValueError("Mamba2 scan requires non-empty dimensions")
    if raw_dt.shape != (rows, heads) or dt_bias.shape != (heads,) or a.shape != (heads,) or d.shape != (heads,):
        raise ValueError(f"Mamba2 scan has xBC {list(xbc.shape)}, dt {list(raw_dt.shape)}, dt bias {list(dt_bias.shape)}, A {list(a.shape)}, "
                         f"D {list(d.shape)}, and state {list(state.shape[1:])}")
    groups = mamba2_geometry(width, heads, head_dim, state_size)
    out = np.empty((rows, heads, head_dim), np.float32)
    nxt = np.empty_like(state)
    lib().orc_mamba2_scan(_p(xbc), _p(raw_dt), _p(dt_bias), _p(a), _p(d), _p(cu), lanes, heads, head_dim, state_size, groups,
                          _p(state), _p(nxt), _p(out))
    return out, nxt


def short_conv(bcx, kernel, tail, cu_seqlens=None):
    """bcx [rows, 3*hidden] laid out [B | C | x], kernel [hidden, K], tail [lanes, K-1, hidden]; returns (C * conv(B * x), new tail)
    (src/decoder.rs:1430-1492)."""
    bcx, kernel, tail = _f32(bcx), _f32(kernel), _f32(tail)
    rows = bcx.shape[0]
    hidden, K = kernel.shape
    cu = _cu([0, rows] if cu_seqlens is None else cu_seqlens, rows)
    lanes = cu.size - 1
    if bcx.shape != (rows, 3 * hidden) or K < 1:
        raise ValueError("short-convolution state geometry does not match its layer")
    if tail.shape != (lanes, K - 1, hidden):
        raise ValueError(f"short-convolution tail has shape {list(tail.shape)}, expected [{lanes}, {K - 1}, {hidden}]")
    out = np.empty((rows, hidden), np.float32)
    nxt = np.empty_like(tail)
    lib().orc_short_conv(_p(bcx), _p(kernel), _p(cu), lanes, hidden, K, _p(tail), _p(nxt), _p(out))
    return out, nxt


def argmax(v: np.ndarray) -> int:
    v = _f32(v)
    return int(lib().orc_argmax(_p(v), C.c_int64(v.size)))


def apply_penalties(logits, history, rep, generated, presence, frequency) -> np.ndarray:
    """apply_repetition_penalty then apply_openai_penalties (src/sampling.rs:392-423), in numpy f32: the repetition
    penalty touches every distinct history token once (negative logits are multiplied, the others divided); the
    presence / frequency penalties subtract frequency * count + presence per distinct generated token.  Tokens outside
    the row are ignored.  Written apart from the product's host sampler on purpose."""
    out = _f32(logits).copy()
    rep = np.float32(rep)
    if rep > 0 and abs(rep - np.float32(1.0)) >= np.finfo(np.float32).eps:
        for t in sorted({int(t) for t in history}):
            if t < out.size:
                out[t] = out[t] * rep if out[t] < 0 else out[t] / rep
    if (presence != 0 or frequency != 0) and len(generated) > 0:
        counts = {}
        for t in generated:
            counts[int(t)] = counts.get(int(t), 0) + 1
        for t, c in counts.items():
            if t < out.size:
                out[t] = out[t] - (np.float32(frequency) * np.float32(c) + np.float32(presence))
    return out
