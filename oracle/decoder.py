"""CPU ORACLE - TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

The decoder forward of the reference's CPU path, restated over oracle_math.cpp:
  src/decoder.rs:3146-3358   forward_inner_batch (embedding, layers, last-row gather, logits tail)
  src/decoder.rs:808-1161    packed attention: projections, per-head QK norm before RoPE, per-lane
                             rotation, paged write, causal / sliding attention
  src/decoder.rs:2684-2699   finish_mixer (post norms, residuals, FFN norm)
  src/decoder.rs:298-305,394-554   dense and sparse-MoE feed-forward
  src/gguf.rs:1888-1924      llama-style Q/K row un-permutation at load
  src/gguf_model.rs:1400-1494,2313-2324  Gemma 2 layer pattern, SmolLM3 NoPE layers
All activations f32; the quantised matmuls quantise the activation rows to 8-bit blocks (mode 1) or
run on dequantised weights (mode 2).  KV pool f32 like the reference CPU backend, or f16 when asked.
"""
from __future__ import annotations

import mmap
import struct
from pathlib import Path

import numpy as np

from . import mathlib as M

_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<B", 10: "<Q", 11: "<q", 12: "<d"}


class Gguf:
    """One GGUF file, or a shard family `<prefix>-00001-of-000NN.gguf` entered through its first member
    (src/gguf.rs:576-660): later members add tensors, the metadata is the first member's."""

    def __init__(self, path, _member=False):
        self.f = open(path, "rb")
        self.mm = mmap.mmap(self.f.fileno(), 0, access=mmap.ACCESS_READ)
        self.buf = np.frombuffer(self.mm, dtype=np.uint8)
        self.p = 0
        magic, version, n_tensors, n_kv = self._unpack("<IIQQ")
        assert magic == 0x46554747 and version in (2, 3)
        self.meta = {}
        for _ in range(n_kv):
            key = self._string()
            (t,) = self._unpack("<I")
            self.meta[key] = self._value(t)
        self.tensors = {}
        order = []
        for _ in range(n_tensors):
            name = self._string()
            (nd,) = self._unpack("<I")
            dims = [self._unpack("<Q")[0] for _ in range(nd)][::-1]
            qtype, off = self._unpack("<IQ")
            self.tensors[name] = dict(dims=dims, type=qtype, offset=off)
            order.append(name)
        align = self.meta.get("general.alignment", 32)
        self.data_start = (self.p + align - 1) // align * align
        for t in self.tensors.values():
            t["file"] = self
        self.members = [self]
        count = int(self.meta.get("split.count", 0))
        if not _member and count > 1:
            path = Path(path)
            stem = path.name[:-len(".gguf")]
            prefix, index = stem.rsplit("-of-", 1)[0].rsplit("-", 1)
            assert int(index) == 1 and int(self.meta["split.no"]) == 0, "a shard family is entered through its first member"
            for i in range(1, count):
                g = Gguf(path.with_name(f"{prefix}-{i + 1:05d}-of-{count:05d}.gguf"), _member=True)
                assert int(g.meta["split.no"]) == i and int(g.meta["split.count"]) == count
                assert not set(g.tensors) & set(self.tensors), "a tensor appears in two shards"
                self.tensors.update(g.tensors)
                self.members.append(g)
            assert len(self.tensors) == int(self.meta["split.tensors.count"])

    def _unpack(self, fmt):
        n = struct.calcsize(fmt)
        v = struct.unpack_from(fmt, self.mm, self.p)
        self.p += n
        return v

    def _string(self):
        (n,) = self._unpack("<Q")
        s = self.mm[self.p:self.p + n].decode("utf-8")
        self.p += n
        return s

    def _value(self, t):
        if t == 8:
            return self._string()
        if t == 9:
            et, n = self._unpack("<IQ")
            if et == 8:
                out = None  # token strings are not needed by the oracle; skip them quickly
                for _ in range(n):
                    (ln,) = self._unpack("<Q")
                    self.p += ln
                return out
            size = struct.calcsize(_SCALAR[et])
            arr = np.frombuffer(self.mm, dtype=np.dtype(_SCALAR[et]), count=n, offset=self.p)
            self.p += size * n
            return arr
        return self._unpack(_SCALAR[t])[0]

    def raw(self, name):
        t = self.tensors[name]
        cols = t["dims"][-1]
        rows = int(np.prod(t["dims"][:-1])) if len(t["dims"]) > 1 else 1
        n = rows * M.row_bytes(t["type"], cols)
        src = t["file"]
        start = src.data_start + t["offset"]
        return src.buf[start:start + n], t["type"], rows, cols

    def f32(self, name):
        raw, qtype, rows, cols = self.raw(name)
        assert qtype == 0
        return np.frombuffer(raw.tobytes(), dtype=np.float32).copy()


def _unpermute(raw: np.ndarray, rows: int, heads: int, row_bytes: int) -> np.ndarray:
    """llama.cpp pair-interleaved Q/K rows -> half-split order: source row head*d + 2*pair + lane goes to
    dest head*d + lane*d/2 + pair (src/gguf.rs:1912-1921)."""
    d = rows // heads
    src = raw.reshape(heads, d // 2, 2, row_bytes)
    return np.ascontiguousarray(src.transpose(0, 2, 1, 3)).reshape(-1)


class Decoder:
    def __init__(self, path, kv_dtype="f32", matmul_mode=1):
        g = self.g = Gguf(path)
        m = g.meta
        a = self.arch = m["general.architecture"]
        self.layers = int(m[f"{a}.block_count"])
        self.hidden = int(m[f"{a}.embedding_length"])
        self.q_heads = int(m[f"{a}.attention.head_count"])
        self.kv_heads = int(m.get(f"{a}.attention.head_count_kv", self.q_heads))
        self.d = int(m.get(f"{a}.attention.key_length", self.hidden // self.q_heads))
        self.ffn = int(m.get(f"{a}.feed_forward_length", 0))
        self.eps = float(np.float32(m[f"{a}.attention.layer_norm_rms_epsilon"]))
        self.max_context = int(m[f"{a}.context_length"])
        self.vocab = int(m.get(f"{a}.vocab_size", g.tensors["token_embd.weight"]["dims"][0]))
        self.tied = "output.weight" not in g.tensors
        self.rotary = int(m.get(f"{a}.rope.dimension_count", self.d))
        theta = float(m.get(f"{a}.rope.freq_base", 10000.0))
        self.permute = a in ("llama", "smollm3")
        # RoPE frequency factors: the Llama profile reads them (src/gguf_model.rs:1855,2015-2033), the others refuse the tensor
        self.rope_factors = None
        if "rope_freqs.weight" in g.tensors:
            if a != "llama":
                raise ValueError(f"GGUF {a} rope frequency factors are not supported")
            self.rope_factors = g.f32("rope_freqs.weight")
            if len(self.rope_factors) != self.d // 2 or not (np.isfinite(self.rope_factors).all() and (self.rope_factors > 0).all()):
                raise ValueError("GGUF `rope_freqs.weight` factors must be head_dim / 2 finite positive values")
        self.embedding_scale = 1.0
        self.final_softcap = 0.0
        self.experts = int(m.get("qwen3moe.expert_count", 0))
        self.experts_used = int(m.get("qwen3moe.expert_used_count", 0))
        self.expert_ffn = int(m.get("qwen3moe.expert_feed_forward_length", 0))
        self.stop_ids = (int(m["tokenizer.ggml.eos_token_id"]),) if "tokenizer.ggml.eos_token_id" in m else ()
        self.lspec = []
        for l in range(self.layers):
            s = dict(sliding=False, window=0, rope=True, theta=theta, qk_norm=a in ("qwen3", "qwen3moe"), act=0, sandwich=False,
                     moe=a == "qwen3moe", scale=float(np.float32(1.0 / np.sqrt(float(self.d)))), softcap=0.0)
            if a == "smollm3":
                s["rope"] = (l + 1) % 4 != 0
            if a == "gemma2":
                s["sliding"] = l % 2 == 0
                s["window"] = int(m.get("gemma2.attention.sliding_window", 4096)) if s["sliding"] else 0
                s["softcap"] = float(np.float32(m["gemma2.attn_logit_softcapping"]))
                s["act"], s["sandwich"] = 1, True
            self.lspec.append(s)
        if a == "gemma2":
            self.embedding_scale = float(np.float32(np.sqrt(float(self.hidden))))
            self.final_softcap = float(np.float32(m.get("gemma2.final_logit_softcapping", 0.0)))
            self.rotary = self.d
        self.kv_dtype = np.float16 if kv_dtype == "f16" else np.float32
        self.mode = matmul_mode
        self.w = {}
        for name, t in g.tensors.items():
            raw, qtype, rows, cols = g.raw(name)
            if len(t["dims"]) == 1:
                self.w[name] = g.f32(name)
                continue
            if self.permute and (name.endswith("attn_q.weight") or name.endswith("attn_k.weight")):
                heads = self.q_heads if name.endswith("attn_q.weight") else self.kv_heads
                raw = _unpermute(raw, rows, heads, M.row_bytes(qtype, cols))
            self.w[name] = (np.ascontiguousarray(raw), qtype, rows, cols)
        self.rope_tables = {}
        self.pool = None

    def bind_pool(self, pool):
        self.pool = pool
        shape = (pool.max_blocks, self.layers, self.kv_heads, pool.block_tokens, self.d)
        self.k_pool = np.zeros(shape, self.kv_dtype)
        self.v_pool = np.zeros(shape, self.kv_dtype)

    def _mm(self, name, x, expert=None):
        raw, qtype, rows, cols = self.w[name]
        if expert is not None:
            E = self.experts
            per = rows // E
            rb = M.row_bytes(qtype, cols)
            raw = raw[expert * per * rb:(expert + 1) * per * rb]
            rows = per
        if qtype == 0:
            return (x @ np.frombuffer(raw.tobytes(), np.float32).reshape(rows, cols).T).astype(np.float32)
        return M.qmatmul(qtype, raw, rows, cols, x, self.mode)

    def _rope(self, theta):
        if theta not in self.rope_tables:
            cap = min(self.max_context, max(self.pool.max_blocks * self.pool.block_tokens, 256))
            self.rope_tables[theta] = M.rope_tables(theta, self.rotary, cap, self.rope_factors)
        return self.rope_tables[theta]

    def forward(self, lanes, reservation):
        """lanes: (session, ids, start_pos); reservation: oracle.kv.Reservation.  Returns [lanes, vocab] logits."""
        bt = self.pool.block_tokens
        ids = np.concatenate([np.asarray(i, np.uint32) for _, i, _ in lanes])
        lane_len = [len(i) for _, i, _ in lanes]
        start = [s for _, _, s in lanes]
        T = len(ids)
        pos = np.concatenate([np.arange(s, s + n) for s, n in zip(start, lane_len)]).astype(np.int32)
        tables = [[b[0] for b in lane["provisional"]] for lane in reservation.lanes]
        slots = np.concatenate([[tables[i][p // bt] * bt + p % bt for p in range(s, s + n)]
                                for i, (s, n) in enumerate(zip(start, lane_len))]).astype(np.int64)
        flat = np.concatenate([np.asarray(t, np.uint32) for t in tables])
        page_off = np.concatenate([[0], np.cumsum([len(t) for t in tables])[:-1]]).astype(np.int32)
        for src, dst, rows in reservation.cows:  # copy_paged_prefix, cache.rs:3042-3089
            self.k_pool[dst, :, :, :rows] = self.k_pool[src, :, :, :rows]
            self.v_pool[dst, :, :, :rows] = self.v_pool[src, :, :, :rows]
        raw, qtype, rows, cols = self.w["token_embd.weight"]
        h = M.embed(qtype, raw, cols, ids, self.embedding_scale)
        for l, ls in enumerate(self.lspec):
            p = f"blk.{l}."
            n = M.rmsnorm(h, self.w[p + "attn_norm.weight"], self.eps)
            q = self._mm(p + "attn_q.weight", n)
            k = self._mm(p + "attn_k.weight", n)
            v = self._mm(p + "attn_v.weight", n)
            if ls["qk_norm"]:
                q = M.rmsnorm(q.reshape(T * self.q_heads, self.d), self.w[p + "attn_q_norm.weight"], self.eps).reshape(T, -1)
                k = M.rmsnorm(k.reshape(T * self.kv_heads, self.d), self.w[p + "attn_k_norm.weight"], self.eps).reshape(T, -1)
            if ls["rope"]:
                cos, sin = self._rope(ls["theta"])
                q = M.rope_apply(q, self.q_heads, self.d, self.rotary, pos, cos, sin)
                k = M.rope_apply(k, self.kv_heads, self.d, self.rotary, pos, cos, sin)
            M.kv_scatter(k, v, self.k_pool, self.v_pool, slots, self.kv_heads, self.d, bt, self.layers, l)
            att = M.paged_attention(q, self.k_pool, self.v_pool, flat, page_off, start, lane_len, q_heads=self.q_heads,
                                    kv_heads=self.kv_heads, d=self.d, block_tokens=bt, layers=self.layers, layer=l,
                                    scale=ls["scale"], softcap=ls["softcap"], window=ls["window"], mode=1)
            o = self._mm(p + "attn_output.weight", att)
            if ls["sandwich"]:
                o = M.rmsnorm(o, self.w[p + "post_attention_norm.weight"], self.eps)
            h = h + o
            f_in = M.rmsnorm(h, self.w[p + "ffn_norm.weight"], self.eps)
            if not ls["moe"]:
                gate = self._mm(p + "ffn_gate.weight", f_in)
                up = self._mm(p + "ffn_up.weight", f_in)
                f = self._mm(p + "ffn_down.weight", M.act_mul(gate, up, ls["act"]))
            else:
                router = f_in @ self.w_router(p)
                sel, wts = M.moe_route(router, self.experts_used)
                f = np.zeros_like(h)
                for e in range(self.experts):  # experts in index order, index_add (decoder.rs:424-439)
                    rows_e, choice = np.nonzero(sel == e)
                    if len(rows_e) == 0:
                        continue
                    x = np.ascontiguousarray(f_in[rows_e])
                    gate = self._mm(p + "ffn_gate_exps.weight", x, e)
                    up = self._mm(p + "ffn_up_exps.weight", x, e)
                    out = self._mm(p + "ffn_down_exps.weight", M.act_mul(gate, up, ls["act"]), e)
                    contrib = (out * wts[rows_e, choice][:, None]).astype(np.float32)
                    f[rows_e] = f[rows_e] + contrib
            if ls["sandwich"]:
                f = M.rmsnorm(f, self.w[p + "post_ffw_norm.weight"], self.eps)
            h = h + f
        last = np.cumsum(lane_len) - 1
        hl = M.rmsnorm(np.ascontiguousarray(h[last]), self.w["output_norm.weight"], self.eps)
        logits = self._mm("token_embd.weight" if self.tied else "output.weight", hl)
        if self.final_softcap:
            logits = M.softcap(logits, self.final_softcap)
        return logits

    def w_router(self, p):
        raw, qtype, rows, cols = self.w[p + "ffn_gate_inp.weight"]
        return np.frombuffer(raw.tobytes(), np.float32).reshape(rows, cols).T
