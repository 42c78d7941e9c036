"""Host-only paged-KV pool, block tables and exact-token prefix cache over the C ABI (mk_kvpool_*,
mk_kvtable_*, mk_prefix_cache_*).  Mirrors crates/macllm-kv of the reference; no GPU is touched.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _capi as capi


class KvPool:
    def __init__(self, block_tokens: int, slab_blocks: int, max_blocks: int):
        h = C.c_void_p()
        capi.check(capi.lib().mk_kvpool_new(block_tokens, slab_blocks, max_blocks, C.byref(h)))
        self._h = h

    def stats(self) -> dict:
        s = capi.PoolStats()
        capi.check(capi.lib().mk_kvpool_stats(self._h, C.byref(s)))
        return s.as_dict()

    def new_table(self) -> "KvTable":
        h = C.c_void_p()
        capi.check(capi.lib().mk_kvtable_new(self._h, C.byref(h)))
        return KvTable(self, h)

    def _tables(self, tables):
        arr = (C.c_void_p * len(tables))(*[t._h for t in tables])
        return arr

    def append_batch(self, tables, n_tokens, commit=True):
        """reserve_batch + commit (or rollback).  Returns the copy-on-write (src, dst, rows) triples.
        Raises KvExhausted without mutating anything when the pool cannot serve the batch."""
        arr = self._tables(tables)
        n = np.ascontiguousarray(n_tokens, dtype=np.int32)
        copies = np.empty(3 * max(len(tables), 1), np.int64)
        nc = C.c_int32(len(tables))
        capi.check(capi.lib().mk_kvpool_append_batch(self._h, arr, n.ctypes.data, len(tables), 1 if commit else 0,
                                                     copies.ctypes.data, C.byref(nc)))
        return [tuple(int(x) for x in copies[3 * i:3 * i + 3]) for i in range(nc.value)]

    def append_touch_rollback(self, tables, n_tokens) -> int:
        """reserve_batch, mark every page of the reservation as touched by the device, roll back: what a forward that
        failed midway leaves behind.  Returns the epoch the reservation had taken."""
        arr = self._tables(tables)
        n = np.ascontiguousarray(n_tokens, dtype=np.int32)
        capi.check(capi.lib().mk_kvpool_append_batch(self._h, arr, n.ctypes.data, len(tables), 2, None, None))
        return self.submitted_epoch()

    def page_table(self, tables, n_tokens):
        """The compact page table a reservation of this batch would expose (then rolls it back)."""
        arr = self._tables(tables)
        n = np.ascontiguousarray(n_tokens, dtype=np.int32)
        cap = 1 << 16
        pages = np.empty((cap, 2), np.uint32)
        rows = C.c_int32(cap)
        lo = np.empty(len(tables), np.int32)
        lc = np.empty(len(tables), np.int32)
        ll = np.empty(len(tables), np.int32)
        capi.check(capi.lib().mk_kvpool_page_table(self._h, arr, n.ctypes.data, len(tables), pages.ctypes.data, C.byref(rows),
                                                   lo.ctypes.data, lc.ctypes.data, ll.ctypes.data))
        return pages[: rows.value].tolist(), lo.tolist(), lc.tolist(), ll.tolist()

    def submitted_epoch(self) -> int:
        e = C.c_int64()
        capi.check(capi.lib().mk_kvpool_submit_epoch(self._h, C.byref(e)))
        return int(e.value)

    def complete_epoch(self, epoch: int) -> None:
        capi.check(capi.lib().mk_kvpool_complete_epoch(self._h, epoch))

    def __del__(self):
        try:
            if self._h:
                capi.lib().mk_kvpool_free(self._h)
                self._h = None
        except Exception:
            pass


class KvTable:
    def __init__(self, pool: KvPool, handle):
        self.pool = pool
        self._h = handle

    def __len__(self) -> int:
        n = C.c_int64()
        capi.check(capi.lib().mk_kvtable_len(self._h, C.byref(n)))
        return int(n.value)

    def blocks(self):
        cap = 1 << 16
        slots = np.empty(cap, np.uint32)
        gens = np.empty(cap, np.uint64)
        n = C.c_int32(cap)
        capi.check(capi.lib().mk_kvtable_blocks(self._h, slots.ctypes.data, gens.ctypes.data, C.byref(n)))
        return [(int(s), int(g)) for s, g in zip(slots[: n.value], gens[: n.value])]

    def clear(self) -> None:
        capi.check(capi.lib().mk_kvtable_clear(self._h))

    def fork_prefix(self, tokens: int) -> "KvTable":
        h = C.c_void_p()
        capi.check(capi.lib().mk_kvtable_fork_prefix(self._h, tokens, C.byref(h)))
        return KvTable(self.pool, h)

    def attach_prefix(self, src: "KvTable", tokens: int) -> None:
        capi.check(capi.lib().mk_kvtable_attach_prefix(self._h, src._h, tokens))

    def free(self) -> None:
        if self._h:
            capi.lib().mk_kvtable_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class PrefixCache:
    def __init__(self, block_tokens: int, capacity_blocks: int):
        h = C.c_void_p()
        capi.check(capi.lib().mk_prefix_cache_new(block_tokens, capacity_blocks, C.byref(h)))
        self._h = h

    def insert(self, tokens, value: int, cost: int) -> list[int]:
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        ev = np.empty(4096, np.int64)
        n = C.c_int32(4096)
        capi.check(capi.lib().mk_prefix_cache_insert(self._h, t.ctypes.data, len(t), value, cost, ev.ctypes.data, C.byref(n)))
        return [int(x) for x in ev[: n.value]]

    def lookup(self, tokens):
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        v = C.c_int64()
        m = C.c_int64()
        capi.check(capi.lib().mk_prefix_cache_lookup(self._h, t.ctypes.data, len(t), C.byref(v), C.byref(m)))
        return None if v.value < 0 else (int(m.value), int(v.value))

    def lookup_exact(self, tokens, exclusive_max=None):
        """TokenPrefixCache::lookup: (matched tokens, value) of the longest stored prefix that is an exact endpoint strictly
        below the prompt length and below `exclusive_max`; None on a miss."""
        hit = self._bounded(1, tokens, exclusive_max)
        return None if hit is None else hit[:2]

    def lookup_aligned(self, tokens, exclusive_max=None):
        """lookup_aligned_common_prefix with its bound: (matched tokens, snapshot tokens, value) or None."""
        hit = self._bounded(0, tokens, exclusive_max)
        return None if hit is None else (hit[0], hit[2], hit[1])

    def _bounded(self, exact, tokens, exclusive_max):
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        v, m, s = C.c_int64(), C.c_int64(), C.c_int64()
        capi.check(capi.lib().mk_prefix_cache_lookup_bounded(self._h, exact, t.ctypes.data if len(t) else None, len(t),
                                                             -1 if exclusive_max is None else int(exclusive_max),
                                                             C.byref(v), C.byref(m), C.byref(s)))
        return None if v.value < 0 else (int(m.value), int(v.value), int(s.value))

    def set_max_cost(self, max_cost: int) -> list[int]:
        """The new budget evicts least recently used snapshots until the cache fits; returns their values."""
        ev = np.empty(4096, np.int64)
        n = C.c_int32(4096)
        capi.check(capi.lib().mk_prefix_cache_set_max_cost(self._h, max_cost, ev.ctypes.data, C.byref(n)))
        return [int(x) for x in ev[: n.value]]

    def force_collisions(self) -> None:
        capi.check(capi.lib().mk_prefix_cache_force_collisions(self._h))

    def evict_lru(self):
        v = C.c_int64()
        capi.check(capi.lib().mk_prefix_cache_evict_lru(self._h, C.byref(v)))
        return None if v.value < 0 else int(v.value)

    def stats(self) -> dict:
        d = capi.PrefixDiagnostics()
        capi.check(capi.lib().mk_prefix_cache_diagnostics(self._h, C.byref(d)))
        return d.as_dict()

    def __del__(self):
        try:
            if self._h:
                capi.lib().mk_prefix_cache_free(self._h)
                self._h = None
        except Exception:
            pass


def block_digests(block_tokens: int, tokens) -> list[bytes]:
    t = np.ascontiguousarray(tokens, dtype=np.uint32)
    n = C.c_int32(len(t) // block_tokens + 1)
    out = np.empty((n.value, 32), np.uint8)
    capi.check(capi.lib().mk_prefix_block_digests(block_tokens, t.ctypes.data, len(t), out.ctypes.data, C.byref(n)))
    return [bytes(out[i]) for i in range(n.value)]


def sha256(data: bytes) -> bytes:
    buf = np.frombuffer(data, dtype=np.uint8) if data else np.empty(0, np.uint8)
    out = np.empty(32, np.uint8)
    capi.check(capi.lib().mk_sha256(buf.ctypes.data if len(buf) else None, len(buf), out.ctypes.data))
    return bytes(out)
