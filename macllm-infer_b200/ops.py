"""NumPy-facing wrappers of the kernel-level C ABI entry points (mk_k_*).

Each function mirrors one operator of the reference's path (cited in include/macllm_b200.h) and runs
the sm_100a kernel through the shared library; host arrays in, host arrays out.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _capi as capi


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def row_bytes(qtype: int, cols: int) -> int:
    return int(capi.lib().mk_row_bytes(qtype, cols))


def decode_rows(qtype: int, w: np.ndarray, rows: int, cols: int) -> np.ndarray:
    """The load-time host decoder of the block formats no kernel reads in place (Q4_0, Q5_0, Q5_1, Q2_K, Q3_K, Q5_K, BF16)."""
    w = np.ascontiguousarray(w)
    out = np.empty((rows, cols), dtype=np.float32)
    capi.check(capi.lib().mk_decode_rows(qtype, _p(w), rows, cols, _p(out)))
    return out


def unpermute_qk_rows(raw: np.ndarray, rows: int, heads: int) -> np.ndarray:
    """The loader's un-permutation of Llama Q/K rows on raw row bytes (any block format)."""
    raw = np.ascontiguousarray(raw).reshape(-1).view(np.uint8)
    out = np.empty_like(raw)
    capi.check(capi.lib().mk_unpermute_qk_rows(_p(raw), rows, raw.size // max(rows, 1), heads, _p(out)))
    return out


def seed_tensor(seed: int, stream: int, std: float, qtype: int, rows: int, cols: int) -> np.ndarray:
    """N(0, std) weights from the counter-based generator, quantised to `qtype`; returns raw block bytes."""
    rb = row_bytes(qtype, cols)
    if rb < 0:
        raise capi.MkError(f"unsupported type {qtype} for {cols} columns")
    out = np.empty(rows * rb, dtype=np.uint8)
    capi.check(capi.lib().mk_seed_tensor(seed, stream, std, qtype, rows, cols, _p(out)))
    return out


def quantize(x: np.ndarray, act_kind: int = 0):
    x = _f32(x)
    T, K = x.shape
    qs = np.empty((T, K), dtype=np.int8)
    d = np.empty((T, K // (256 if act_kind == 0 else 32)), dtype=np.float32)
    bs = np.zeros((T, K // 16), dtype=np.int16)
    capi.check(capi.lib().mk_k_quantize(act_kind, _p(x), T, K, _p(qs), _p(d), _p(bs)))
    return qs, d, bs


def add_norm(h, a=None, a_scale=1.0, post_w=None, norm_w=None, eps=1e-5):
    """Returns (updated residual, normed output)."""
    h = _f32(h).copy()
    rows, dim = h.shape
    a = None if a is None else _f32(a)
    post_w = None if post_w is None else _f32(post_w)
    norm_w = None if norm_w is None else _f32(norm_w)
    out = np.empty_like(h)
    capi.check(capi.lib().mk_k_add_norm(_p(h), _p(a), a_scale, _p(post_w), _p(norm_w), eps, rows, dim, _p(out)))
    return h, out


def qmatmul(qtype: int, w_bytes: np.ndarray, rows: int, cols: int, x: np.ndarray, path: int = capi.PATH_AUTO) -> np.ndarray:
    x = _f32(x)
    T = x.shape[0]
    w_bytes = np.ascontiguousarray(w_bytes)
    y = np.empty((T, rows), dtype=np.float32)
    capi.check(capi.lib().mk_k_qmatmul(qtype, _p(w_bytes), rows, cols, _p(x), T, _p(y), path))
    return y


def qmatmul_time(qtype: int, w_bytes: np.ndarray, rows: int, cols: int, x: np.ndarray, path: int, iters: int = 10) -> float:
    """Mean launch duration (ms) of the matmul on the chosen path, operands resident, L2 flushed per launch."""
    x = _f32(x)
    w_bytes = np.ascontiguousarray(w_bytes)
    ms = C.c_float(0)
    capi.check(capi.lib().mk_k_qmatmul_time(qtype, _p(w_bytes), rows, cols, _p(x), x.shape[0], path, iters, C.byref(ms)))
    return float(ms.value)


def embed(qtype: int, w_bytes: np.ndarray, rows: int, cols: int, ids, scale: float = 1.0) -> np.ndarray:
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    out = np.empty((len(ids), cols), dtype=np.float32)
    w_bytes = np.ascontiguousarray(w_bytes)
    capi.check(capi.lib().mk_k_embed(qtype, _p(w_bytes), rows, cols, _p(ids), len(ids), scale, _p(out)))
    return out


def actmul(gate, up, act: int = 0) -> np.ndarray:
    gate, up = _f32(gate), _f32(up)
    T, F = gate.shape
    out = np.empty_like(gate)
    capi.check(capi.lib().mk_k_actmul(_p(gate), _p(up), T, F, act, _p(out)))
    return out


def gated_ffn(qtype: int, gate_w, up_w, F: int, cols: int, x, act: int = 0, iters: int = 0):
    """f16(act(x @ gate.T) * (x @ up.T)) from one tensor-core GEMM over the interleaved gate/up image, as f32 [T][F];
    with iters > 0 also the average milliseconds of the GEMM."""
    x = _f32(x)
    T = x.shape[0]
    out = np.empty((T, F), dtype=np.float32)
    ms = C.c_float(0)
    capi.check(capi.lib().mk_k_gated_ffn(qtype, _p(gate_w), _p(up_w), F, cols, _p(x), T, act, _p(out), iters,
                                         C.byref(ms) if iters > 0 else None))
    return (out, float(ms.value)) if iters > 0 else out


def _cu32(cu_seqlens, rows: int) -> np.ndarray:
    return np.ascontiguousarray([0, rows] if cu_seqlens is None else cu_seqlens, dtype=np.int32)


def gated_delta_decay(alpha, time_bias, state_decay) -> np.ndarray:
    """exp(softplus(alpha + time_bias) * state_decay) for alpha [tokens, heads]."""
    alpha, time_bias, state_decay = _f32(alpha), _f32(time_bias), _f32(state_decay)
    tokens, heads = alpha.shape
    if time_bias.shape != (heads,) or state_decay.shape != (heads,):
        raise ValueError(f"Gated DeltaNet decay has alpha shape {list(alpha.shape)}, time bias {list(time_bias.shape)} and state decay {list(state_decay.shape)}")
    out = np.empty_like(alpha)
    capi.check(capi.lib().mk_k_gated_delta_decay(_p(alpha), _p(time_bias), _p(state_decay), tokens, heads, _p(out)))
    return out


def gated_delta_recurrence(query, key, value, decay, beta, state, cu_seqlens=None):
    """query / key [rows, heads, key_dim], value [rows, heads, value_dim], decay / beta [rows, heads], state
    [lanes, heads, key_dim, value_dim] -> (out [rows, heads, value_dim], next state)."""
    query, key, value, decay, beta, state = (_f32(t) for t in (query, key, value, decay, beta, state))
    rows, heads, key_dim = query.shape
    cu = _cu32(cu_seqlens, rows)
    lanes = cu.size - 1
    value_dim = value.shape[2]
    if (key.shape != query.shape or value.shape[:2] != (rows, heads) or decay.shape != (rows, heads) or beta.shape != (rows, heads)
            or state.shape != (lanes, heads, key_dim, value_dim) or cu[-1] != rows):
        raise ValueError(f"Gated DeltaNet decode has query {list(query.shape)}, key {list(key.shape)}, value {list(value.shape)}, "
                         f"decay {list(decay.shape)}, beta {list(beta.shape)} and state {list(state.shape)}")
    out = np.empty((rows, heads, value_dim), np.float32)
    nxt = np.empty_like(state)
    capi.check(capi.lib().mk_k_gated_delta_recurrence(_p(query), _p(key), _p(value), _p(decay), _p(beta), _p(cu), lanes, heads, key_dim,
                                                      value_dim, _p(state), _p(nxt), _p(out)))
    return out, nxt


def mamba2_scan(xbc, raw_dt, dt_bias, a, d, state, cu_seqlens=None):
    """xbc [rows, H*P + 2*G*N] laid out [x | B | C], raw_dt [rows, H], dt_bias / a / d [H], state [lanes, H, P, N] ->
    (out [rows, H, P], final state)."""
    xbc, raw_dt, dt_bias, a, d, state = (_f32(t) for t in (xbc, raw_dt, dt_bias, a, d, state))
    rows, width = xbc.shape
    cu = _cu32(cu_seqlens, rows)
    lanes = cu.size - 1
    _, heads, head_dim, state_size = state.shape
    if (state.shape[0] != lanes or raw_dt.shape != (rows, heads) or dt_bias.shape != (heads,) or a.shape != (heads,) or d.shape != (heads,)
            or cu[-1] != rows):
        raise ValueError(f"Mamba2 scan has xBC {list(xbc.shape)}, dt {list(raw_dt.shape)}, dt bias {list(dt_bias.shape)}, A {list(a.shape)}, "
                         f"D {list(d.shape)}, and state {list(state.shape[1:])}")
    out = np.empty((rows, heads, head_dim), np.float32)
    nxt = np.empty_like(state)
    capi.check(capi.lib().mk_k_mamba2_scan(_p(xbc), width, _p(raw_dt), _p(dt_bias), _p(a), _p(d), _p(cu), lanes, heads, head_dim, state_size,
                                           _p(state), _p(nxt), _p(out)))
    return out, nxt


def short_conv(bcx, kernel, tail, cu_seqlens=None):
    """bcx [rows, 3*hidden] laid out [B | C | x], kernel [hidden, K], tail [lanes, K-1, hidden] -> (C * conv(B * x), new tail)."""
    bcx, kernel, tail = _f32(bcx), _f32(kernel), _f32(tail)
    rows = bcx.shape[0]
    hidden, K = kernel.shape
    cu = _cu32(cu_seqlens, rows)
    lanes = cu.size - 1
    if bcx.shape != (rows, 3 * hidden) or cu[-1] != rows:
        raise ValueError("short-convolution state geometry does not match its layer")
    if tail.shape != (lanes, K - 1, hidden):
        raise ValueError(f"short-convolution tail has shape {list(tail.shape)}, expected [{lanes}, {K - 1}, {hidden}]")
    out = np.empty((rows, hidden), np.float32)
    nxt = np.empty_like(tail)
    capi.check(capi.lib().mk_k_short_conv(_p(bcx), _p(kernel), _p(cu), lanes, hidden, K, _p(tail) if tail.size else None,
                                          _p(nxt) if nxt.size else None, _p(out)))
    return out, nxt


def recurrent_time(kind: str, lanes: int, rows_per_lane: int, heads: int, dim_a: int, dim_b: int, iters: int = 10):
    """(average ms per launch, state bytes read + written per launch) of 'gated_delta' (dim_a key_dim, dim_b value_dim) or 'mamba2'
    (dim_a head_dim, dim_b state_size)."""
    ms, nbytes = C.c_float(), C.c_double()
    capi.check(capi.lib().mk_k_recurrent_time({"gated_delta": 0, "mamba2": 1}[kind], lanes, rows_per_lane, heads, dim_a, dim_b, iters,
                                              C.byref(ms), C.byref(nbytes)))
    return float(ms.value), float(nbytes.value)


def argmax(logits) -> np.ndarray:
    logits = _f32(logits)
    B, V = logits.shape
    out = np.empty(B, dtype=np.uint32)
    capi.check(capi.lib().mk_k_argmax(_p(logits), B, V, _p(out)))
    return out


def moe_route(logits, k: int):
    logits = _f32(logits)
    T, E = logits.shape
    sel = np.empty((T, k), dtype=np.int32)
    w = np.empty((T, k), dtype=np.float32)
    capi.check(capi.lib().mk_k_moe_route(_p(logits), T, E, k, _p(sel), _p(w)))
    return sel, w


def grouped_qmatmul(qtype: int, w_bank, experts: int, rows_pe: int, cols: int, x: np.ndarray, offsets, path: int, up_bank=None, act: int = 0):
    """Expert-grouped matmul: rows [offsets[e], offsets[e+1]) of x go through expert e's matrix of the bank."""
    x = _f32(x)
    off = np.ascontiguousarray(offsets, dtype=np.int32)
    y = np.zeros((x.shape[0], rows_pe), dtype=np.float32)
    w_bank = np.ascontiguousarray(w_bank)
    up = None if up_bank is None else np.ascontiguousarray(up_bank)
    capi.check(capi.lib().mk_k_grouped_qmatmul(qtype, _p(w_bank), None if up is None else _p(up), experts, rows_pe, cols, _p(x), _p(off), _p(y), path, act))
    return y


def ep_exchange_emulated(rows: np.ndarray, offsets: np.ndarray, local_experts: int, exchanges: int = 1, silent_rank: int = -1, wait_ns: int = 0):
    """The dispatch / return exchange of data-parallel expert parallelism with all ranks on one device.  rows: f16
    [ranks][cap_rows][hidden]; offsets: [ranks][ranks * local_experts + 1].  Returns (results f32 like rows, merged
    ranges [ranks][local_experts + 1], status [ranks])."""
    rows = np.ascontiguousarray(rows, dtype=np.float16)
    off = np.ascontiguousarray(offsets, dtype=np.int32)
    ranks, cap, hidden = rows.shape
    results = np.zeros((ranks, cap, hidden), dtype=np.float32)
    ranges = np.zeros((ranks, local_experts + 1), dtype=np.int32)
    status = np.zeros(ranks, dtype=np.int32)
    capi.check(capi.lib().mk_k_ep_exchange_emulated(ranks, local_experts, hidden, cap, _p(rows), _p(off), exchanges, silent_rank, wait_ns,
                                                    _p(results), _p(ranges), _p(status)))
    return results, ranges, status


def penalties(logits, history, repetition, generated, presence, frequency) -> np.ndarray:
    """Repetition penalty over the set of history tokens, then presence / frequency penalties over generated counts."""
    row = np.array(logits, dtype=np.float32)
    h = np.ascontiguousarray(history, dtype=np.uint32)
    g = np.ascontiguousarray(generated, dtype=np.uint32)
    capi.check(capi.lib().mk_k_penalties(_p(row), len(row), _p(h), len(h), repetition, _p(g), len(g), presence, frequency))
    return row


def sample(logits: np.ndarray, settings, where: int) -> np.ndarray:
    """settings: one (temperature, top_k, top_p, u) per row.  where 0 = host sampler, 1 = device kernel."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    B, V = logits.shape
    arr = (capi.LaneSampling * B)(*[capi.LaneSampling(float(t), int(k), float(p), float(u)) for t, k, p, u in settings])
    out = np.zeros(B, dtype=np.uint32)
    capi.check(capi.lib().mk_k_sample(_p(logits), B, V, arr, where, _p(out)))
    return out


def matmul_plan(path: int, rows: int, cols: int, T: int, max_splits: int = 16) -> dict:
    """Host-only: how a launch of the f16-image GEMM (PATH_HALF) or the streamed matmul (PATH_STREAM) is cut."""
    out = np.zeros(8, dtype=np.int64)
    capi.check(capi.lib().mk_k_matmul_plan(path, rows, cols, T, max_splits, _p(out)))
    names = ("bn", "row_tiles", "n_tiles", "splits", "kb_per_split", "partial_floats") if path == capi.PATH_HALF else \
        ("bn", "row_tiles", "items", "ctas", "slots", "partial_floats", "tiles_per_group", "groups")
    return dict(zip(names, map(int, out)))


def attention_plan(start_pos, n_tokens, q_heads: int, kv_heads: int, block_tokens: int = 16):
    """Host-only: (key shares per lane, query tiles, entry bound) of one tick's attention plan."""
    sp = np.ascontiguousarray(start_pos, dtype=np.int32)
    nt = np.ascontiguousarray(n_tokens, dtype=np.int32)
    shares = np.zeros(len(sp), dtype=np.int32)
    tiles, bound = C.c_int32(0), C.c_int32(0)
    capi.check(capi.lib().mk_k_attention_plan(_p(sp), _p(nt), len(sp), q_heads, kv_heads, block_tokens, _p(shares), C.byref(tiles),
                                              C.byref(bound)))
    return shares, int(tiles.value), int(bound.value)


def moe_combine_exchange(expert_out, sel, weights, e_lo: int, e_hi: int, ranks: int, rank: int, peer_rows=None, wait_ms: int = 50,
                         epochs: int = 1):
    """One rank's launch(es) of the fused expert-parallel combine + exchange kernel with every rank's exchange block on
    this GPU.  peer_rows [ranks][T][hidden] plays the other ranks' deliveries; None leaves their flags unset, so the
    kernel's bounded wait runs out.  Returns (out [T][hidden], pushed [ranks][T][hidden], status word)."""
    sel = np.ascontiguousarray(sel, dtype=np.int32)
    weights = _f32(weights)
    T, k = sel.shape
    expert_out = _f32(expert_out)
    hidden = expert_out.shape[1]
    out = np.empty((T, hidden), dtype=np.float32)
    pushed = np.empty((ranks, T, hidden), dtype=np.float32)
    status = C.c_int32(0)
    rows = _f32(peer_rows) if peer_rows is not None else None
    capi.check(capi.lib().mk_k_moe_combine_exchange(_p(expert_out), _p(sel), _p(weights), T, k, hidden, e_lo, e_hi, ranks, rank,
                                                    _p(rows) if rows is not None else None, 1 if rows is not None else 0, wait_ms,
                                                    epochs, _p(out), _p(pushed), C.byref(status)))
    return out, pushed, int(status.value)


def attention_step(q, k, v, k_pool, v_pool, tables, start_pos, lane_len, *, q_heads, kv_heads, head_dim, block_tokens,
                   layers, layer, scale, softcap=0.0, window=0, cos_table=None, sin_table=None, rotary_dim=0,
                   q_norm_w=None, k_norm_w=None, norm_eps=1e-6, kernel=0):
    """One attention layer step of a ragged batch.  `tables` is a list of per-lane block-id lists.
    k_pool / v_pool ([blocks, layers, kv_heads, block_tokens, head_dim], f16 or f32) are updated in place.
    Returns dict(out, q_rot, slots, positions, last_index, cu_seqlens)."""
    q = _f32(q).copy()
    k, v = _f32(k), _f32(v)
    lanes = len(lane_len)
    T = int(sum(lane_len))
    assert k_pool.dtype == v_pool.dtype and k_pool.dtype in (np.float16, np.float32)
    flat, offs, lens = [], [], []
    for t in tables:
        offs.append(len(flat))
        lens.append(len(t))
        flat.extend(int(b) for b in t)
    tab = np.asarray(flat if flat else [0], dtype=np.uint32)
    sp = np.asarray(start_pos, dtype=np.int32)
    ll = np.asarray(lane_len, dtype=np.int32)
    to = np.asarray(offs, dtype=np.int32)
    tl = np.asarray(lens, dtype=np.int32)
    out = np.empty_like(q)
    q_rot = np.empty_like(q)
    slots = np.empty(T, dtype=np.int64)
    pos = np.empty(T, dtype=np.int32)
    last = np.empty(lanes, dtype=np.int32)
    cu = np.empty(lanes + 1, dtype=np.int32)
    cos_table = None if cos_table is None else _f32(cos_table)
    sin_table = None if sin_table is None else _f32(sin_table)
    q_norm_w = None if q_norm_w is None else _f32(q_norm_w)
    k_norm_w = None if k_norm_w is None else _f32(k_norm_w)
    c = capi.AttnCase()
    c.lanes, c.total_tokens = lanes, T
    c.q_heads, c.kv_heads, c.head_dim = q_heads, kv_heads, head_dim
    c.block_tokens, c.layers, c.layer, c.pool_blocks = block_tokens, layers, layer, k_pool.shape[0]
    c.kv_f16 = 1 if k_pool.dtype == np.float16 else 0
    c.scale, c.softcap, c.window = scale, softcap, window
    c.rotary_dim = rotary_dim if cos_table is not None else 0
    c.rope_capacity = 0 if cos_table is None else cos_table.shape[0]
    c.norm_eps = norm_eps
    c.kernel = kernel  # 0 auto, 1 scalar f32 kernel, 2 tensor-core kernel
    for name, arr in (("start_pos", sp), ("lane_len", ll), ("table_off", to), ("table_len", tl), ("tables", tab), ("q", q),
                      ("k", k), ("v", v), ("q_norm_w", q_norm_w), ("k_norm_w", k_norm_w), ("cos_table", cos_table),
                      ("sin_table", sin_table), ("k_pool", k_pool), ("v_pool", v_pool), ("out", out), ("q_rot_out", q_rot),
                      ("slots_out", slots), ("positions_out", pos), ("last_index_out", last), ("cu_seqlens_out", cu)):
        setattr(c, name, None if arr is None else arr.ctypes.data)
    capi.check(capi.lib().mk_k_attention_step(C.byref(c)))
    return dict(out=out, q_rot=q_rot, slots=slots, positions=pos, last_index=last, cu_seqlens=cu)
