"""One interface over the product's host KV pool (C ABI) and the oracle's Python restatement, so the
reference's known-answer cases and the randomised differential run against both."""
from __future__ import annotations

import importlib


class OraclePool:
    def __init__(self, bt, slab, max_blocks):
        from oracle import kv
        self.kv = kv
        self.p = kv.Pool(bt, slab, max_blocks)

    def new_table(self):
        return OracleTable(self, self.kv.Table(self.p))

    def append(self, tables, ns, commit=True):
        try:
            r = self.p.reserve_batch([t.t for t in tables], list(ns))
        except self.kv.Exhausted:
            return None
        cows = list(r.cows)
        if commit:
            r.mark_all_used()
            r.commit()
        else:
            r.rollback()
        return cows

    def append_touch_rollback(self, tables, ns):
        r = self.p.reserve_batch([t.t for t in tables], list(ns))
        r.mark_all_used()
        epoch = r.epoch
        r.rollback()
        return epoch

    def page_table(self, tables, ns):
        r = self.p.reserve_batch([t.t for t in tables], list(ns))
        out = r.page_table()
        r.rollback()
        return out

    def stats(self):
        return self.p.stats()

    def submitted(self):
        return self.p.submitted_epoch

    def complete(self, epoch):
        self.p.mark_completed_through(epoch)


class OracleTable:
    def __init__(self, pool, t):
        self.pool, self.t = pool, t

    def blocks(self):
        return list(self.t.blocks)

    def __len__(self):
        return self.t.logical_len

    def fork_prefix(self, n):
        return OracleTable(self.pool, self.t.fork_prefix(n))

    def clear(self):
        self.t.clear()

    def free(self):
        self.t.drop()


class ProductPool:
    def __init__(self, bt, slab, max_blocks):
        self.kv = importlib.import_module("macllm_infer_b200.kv")
        self.capi = importlib.import_module("macllm_infer_b200._capi")
        self.p = self.kv.KvPool(bt, slab, max_blocks)

    def new_table(self):
        return ProductTable(self, self.p.new_table())

    def append(self, tables, ns, commit=True):
        try:
            return self.p.append_batch([t.t for t in tables], list(ns), commit)
        except self.capi.KvExhausted:
            return None

    def append_touch_rollback(self, tables, ns):
        return self.p.append_touch_rollback([t.t for t in tables], list(ns))

    def page_table(self, tables, ns):
        return self.p.page_table([t.t for t in tables], list(ns))

    def stats(self):
        return self.p.stats()

    def submitted(self):
        return self.p.submitted_epoch()

    def complete(self, epoch):
        self.p.complete_epoch(epoch)


class ProductTable:
    def __init__(self, pool, t):
        self.pool, self.t = pool, t

    def blocks(self):
        return self.t.blocks()

    def __len__(self):
        return len(self.t)

    def fork_prefix(self, n):
        return ProductTable(self.pool, self.t.fork_prefix(n))

    def clear(self):
        self.t.clear()

    def free(self):
        self.t.free()
