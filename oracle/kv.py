"""CPU ORACLE - TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Python restatement of the reference's paged-KV bookkeeping and exact-token prefix cache:
  crates/macllm-kv/src/cache.rs        PagedKvPool :588-1370, PagedKvBlockTable :1434-1865,
                                       reserve_batch :2216-2445, PagedKvBatchReservation :2453-3005
  crates/macllm-kv/src/prefix_cache.rs TokenPrefixCache :123-547, digest format :556-654
Integer / byte work only; pinned by the reference's own known-answer tests (tests/test_oracle_kv.py).
"""
from __future__ import annotations

import hashlib
import struct
from collections import OrderedDict
from dataclasses import dataclass, field

FREE, RESERVED, LIVE, RETIRED = "free", "reserved", "live", "retired"


class Exhausted(Exception):
    def __init__(self, requested, free_blocks, unallocated, boundary_message=None):
        super().__init__(boundary_message or
                         f"paged KV pool exhausted: requested {requested} blocks, {free_blocks} free and {unallocated} unallocated")
        self.requested, self.free_blocks, self.unallocated = requested, free_blocks, unallocated


class Invalid(Exception):
    pass


@dataclass
class Slot:
    generation: int = 0
    state: str = FREE
    transaction: int = 0
    references: int = 0
    until: int = 0
    last_use: int = 0


def div_ceil(a, b):
    return (a + b - 1) // b


class Pool:
    def __init__(self, block_tokens: int, slab_blocks: int, max_blocks: int):
        for value, name in ((block_tokens, "block_tokens"), (slab_blocks, "slab_blocks"), (max_blocks, "max_blocks")):  # cache.rs:126-147
            if value <= 0:
                raise Invalid(f"invalid paged KV config: {name} must be positive")
        if max_blocks > 0xFFFFFFFF:
            raise Invalid("invalid paged KV config: max_blocks exceeds the generational block-ID range")
        self.block_tokens, self.slab_blocks, self.max_blocks = block_tokens, slab_blocks, max_blocks
        self.slots: list[Slot] = []
        self.slabs = 0
        self.next_transaction = 0
        self.active_transaction = None
        self.submitted_epoch = 0
        self.completed_epoch = 0

    # ---- occupancy (scan form: the oracle keeps no maintained counters, cache.rs:1350-1369)
    def stats(self) -> dict:
        res = sum(s.state == RESERVED for s in self.slots)
        live = sum(s.state == LIVE for s in self.slots)
        refs = sum(s.references for s in self.slots if s.state == LIVE)
        shared = sum(s.state == LIVE and s.references > 1 for s in self.slots)
        ret = sum(s.state == RETIRED for s in self.slots)
        return dict(allocated_blocks=len(self.slots), free_blocks=len(self.slots) - res - live - ret, live_blocks=live,
                    reserved_blocks=res, retired_blocks=ret, shared_blocks=shared, live_references=refs, slabs=self.slabs,
                    submitted_epoch=self.submitted_epoch, completed_epoch=self.completed_epoch)

    def free_blocks(self) -> int:
        return sum(s.state == FREE for s in self.slots)

    def ensure_free_blocks(self, requested: int) -> None:  # cache.rs:649-715
        free_now = self.free_blocks()
        unallocated = self.max_blocks - len(self.slots)
        if requested > free_now + unallocated:
            raise Exhausted(requested, free_now, unallocated)
        missing = requested - free_now
        planned = 0
        while planned < missing:
            blocks = min(self.slab_blocks, self.max_blocks - len(self.slots))
            if blocks == 0:
                raise Exhausted(requested, free_now, unallocated)
            self.slots.extend(Slot(last_use=self.completed_epoch) for _ in range(blocks))
            self.slabs += 1
            planned += blocks

    def _begin(self):  # cache.rs:717-733
        if self.active_transaction is not None:
            raise Invalid(f"paged KV transaction {self.active_transaction} is still active")
        self.next_transaction += 1
        self.active_transaction = self.next_transaction
        self.submitted_epoch += 1
        return self.active_transaction, self.submitted_epoch

    def _reserve_blocks(self, count: int, transaction: int):  # cache.rs:735-809: lowest-index free slots
        if count == 0:
            return []
        self.ensure_free_blocks(count)
        ids = []
        for i, s in enumerate(self.slots):
            if s.state == FREE:
                ids.append((i, s.generation + 1))
                if len(ids) == count:
                    break
        for i, g in ids:
            s = self.slots[i]
            s.generation, s.state, s.transaction, s.last_use = g, RESERVED, transaction, self.completed_epoch
        return ids

    def _slot(self, bid):
        i, g = bid
        if i >= len(self.slots) or self.slots[i].generation != g:
            raise Invalid(f"stale paged KV block id for slot {i}")
        return self.slots[i]

    def _validate_owned(self, bid, transaction=None):  # cache.rs:851-871
        s = self._slot(bid)
        if not (s.state == LIVE or (s.state == RESERVED and transaction is not None and s.transaction == transaction)):
            raise Invalid(f"block {bid[0]} is not owned by the append transaction")

    def live_references(self, bid) -> int:
        s = self._slot(bid)
        if s.state != LIVE:
            raise Invalid(f"block {bid[0]} is not live")
        return s.references

    def retain_live(self, ids) -> None:  # cache.rs:929-983
        for b in ids:
            if self._slot(b).state != LIVE:
                raise Invalid(f"block {b[0]} is not live")
        for b in ids:
            self.slots[b[0]].references += 1

    def release_live(self, ids) -> None:  # cache.rs:987-1100
        counts: dict[int, int] = {}
        for b in ids:
            if self._slot(b).state != LIVE:
                raise Invalid(f"block {b[0]} is not live")
            counts[b[0]] = counts.get(b[0], 0) + 1
        for i, c in counts.items():
            if self.slots[i].references < c:
                raise Invalid("block has fewer references than the release requires")
        for i, c in counts.items():
            s = self.slots[i]
            s.references -= c
            if s.references == 0:
                if s.last_use <= self.completed_epoch:
                    s.state = FREE
                else:
                    s.state, s.until = RETIRED, s.last_use

    def mark_use(self, ids, transaction, epoch) -> None:  # cache.rs:1127-1146
        for b in ids:
            self._validate_owned(b, transaction)
        for b in ids:
            s = self.slots[b[0]]
            s.last_use = max(s.last_use, epoch)

    def commit_reserved_replacing(self, ids, superseded, transaction) -> None:  # cache.rs:1152-1212
        if self.active_transaction != transaction:
            raise Invalid("transaction is not the active paged KV transaction")
        for b in ids:
            s = self._slot(b)
            if s.state != RESERVED or s.transaction != transaction:
                raise Invalid(f"block {b[0]} is not reserved by this transaction")
        for b in ids:
            s = self.slots[b[0]]
            s.state, s.references = LIVE, 1
        self.release_live(superseded)
        self.active_transaction = None

    def rollback_reserved(self, ids, transaction) -> None:  # cache.rs:1214-1276
        if self.active_transaction != transaction:
            return
        for i, g in dict.fromkeys(ids):
            if i >= len(self.slots) or self.slots[i].generation != g:
                continue
            s = self.slots[i]
            if s.state != RESERVED or s.transaction != transaction:
                continue
            if s.last_use <= self.completed_epoch:
                s.state = FREE
            else:
                s.state, s.until = RETIRED, s.last_use
        self.active_transaction = None

    def mark_completed_through(self, epoch: int) -> None:  # cache.rs:1278-1319
        if self.active_transaction is not None:
            raise Invalid("cannot publish device completion while a paged KV transaction is active")
        if epoch < self.completed_epoch or epoch > self.submitted_epoch:
            raise Invalid(f"invalid completion epoch {epoch}")
        self.completed_epoch = epoch
        for s in self.slots:
            if s.state == RETIRED and s.until <= epoch:
                s.state = FREE

    # ---- reserve_batch (cache.rs:2216-2445)
    def reserve_batch(self, tables, new_tokens) -> "Reservation":
        if not tables:
            raise Invalid("paged KV reservation batch cannot be empty")
        if self.active_transaction is not None:
            raise Invalid(f"paged KV transaction {self.active_transaction} is still active")
        bt = self.block_tokens
        lanes = []
        total = 0
        for i, (t, n) in enumerate(zip(tables, new_tokens)):
            if t.pool is not self:
                raise Invalid("lane table belongs to another paged KV pool")
            if t.in_flight is not None:
                raise Invalid("lane table is unavailable or already reserved")
            if any(t is u for u in tables[:i]):
                raise Invalid(f"lane {i} duplicates an earlier table")
            if n <= 0:
                raise Invalid("lane append token count must be positive")
            for b in t.blocks:
                self._validate_owned(b)
            if len(t.blocks) != div_ceil(t.logical_len, bt):
                raise Invalid("lane block table disagrees with its logical length")
            cow = None
            if t.logical_len % bt != 0 and self.live_references(t.blocks[-1]) > 1:
                cow = (len(t.blocks) - 1, t.blocks[-1], t.logical_len % bt)
            new_len = t.logical_len + n
            if new_len > t.limit:
                raise Invalid("sequence exceeds the context limit")
            growth = max(0, div_ceil(new_len, bt) - len(t.blocks))
            reserved = growth + (1 if cow else 0)
            total += reserved
            lanes.append(dict(table=t, old_len=t.logical_len, new_len=new_len, new_tokens=n, growth=growth, reserved=reserved,
                              provisional=list(t.blocks), cow=cow))
        self.ensure_free_blocks(total)
        transaction, epoch = self._begin()
        try:
            reserved_ids = self._reserve_blocks(total, transaction)
        except Exception:
            self.rollback_reserved([], transaction)
            raise
        superseded, cows, off = [], [], 0
        for lane in lanes:
            blocks = reserved_ids[off:off + lane["reserved"]]
            g0 = 0
            if lane["cow"]:
                idx, source, valid = lane["cow"]
                lane["provisional"][idx] = blocks[0]
                superseded.append(source)
                cows.append((source[0], blocks[0][0], valid))
                g0 = 1
            lane["provisional"].extend(blocks[g0:])
            off += lane["reserved"]
        for lane in lanes:
            lane["table"].in_flight = transaction
        return Reservation(self, transaction, epoch, lanes, reserved_ids, superseded, cows)


class Table:
    def __init__(self, pool: Pool, limit: int = 1 << 40):
        self.pool, self.limit = pool, limit
        self.blocks: list[tuple[int, int]] = []
        self.logical_len = 0
        self.in_flight = None

    def attach_prefix(self, source: "Table", logical_len: int) -> None:  # cache.rs:1486-1563
        if source is self:
            raise Invalid("a paged KV table cannot attach itself as a prefix")
        if source.pool is not self.pool:
            raise Invalid("prefix source belongs to another paged KV pool")
        if self.in_flight is not None or self.blocks or self.logical_len:
            raise Invalid("prefix destination must be a live, empty, unlocked table")
        if source.in_flight is not None:
            raise Invalid("prefix source must be live and unlocked")
        if logical_len > source.logical_len:
            raise Invalid("prefix length exceeds source length")
        if logical_len > self.limit:
            raise Invalid("prefix length exceeds the context limit")
        prefix = source.blocks[:div_ceil(logical_len, self.pool.block_tokens)]
        self.pool.retain_live(prefix)
        self.blocks = list(prefix)
        self.logical_len = logical_len

    def fork_prefix(self, logical_len: int) -> "Table":
        f = Table(self.pool, self.limit)
        f.attach_prefix(self, logical_len)
        return f

    def clear(self) -> bool:  # cache.rs:1840-1852
        if self.in_flight is not None:
            return False
        self.pool.release_live(self.blocks)
        self.blocks = []
        self.logical_len = 0
        return True

    def drop(self) -> None:
        self.pool.release_live(self.blocks)
        self.blocks = []


class Reservation:
    def __init__(self, pool, transaction, epoch, lanes, reserved, superseded, cows):
        self.pool, self.transaction, self.epoch = pool, transaction, epoch
        self.lanes, self.reserved, self.superseded, self.cows = lanes, reserved, superseded, cows
        self.finalized = False

    def mark_all_used(self) -> None:
        ids = [b for lane in self.lanes for b in lane["provisional"]] + list(self.superseded)
        self.pool.mark_use(ids, self.transaction, self.epoch)

    def page_table(self):  # cache.rs:2707-2851
        remap: dict[int, int] = {}
        pages, offsets, counts, lens = [], [], [], []
        for lane in self.lanes:
            offsets.append(len(pages))
            counts.append(len(lane["provisional"]))
            lens.append(lane["new_len"])
            for b in lane["provisional"]:
                self.pool._validate_owned(b, self.transaction)
                slab, off = divmod(b[0], self.pool.slab_blocks)
                if slab not in remap:
                    remap[slab] = len(remap)
                pages.append([remap[slab], off])
        self.pool.mark_use([b for lane in self.lanes for b in lane["provisional"]], self.transaction, self.epoch)
        return pages, offsets, counts, lens

    def commit(self) -> int:  # cache.rs:2947-2979
        if self.finalized:
            raise Invalid("paged KV reservation was already finalized")
        self.pool.commit_reserved_replacing(self.reserved, self.superseded, self.transaction)
        for lane in self.lanes:
            t = lane["table"]
            t.blocks, t.logical_len, t.in_flight = lane["provisional"], lane["new_len"], None
        self.finalized = True
        return self.epoch

    def rollback(self) -> None:  # cache.rs:2985-2998
        if self.finalized:
            return
        self.pool.rollback_reserved(self.reserved, self.transaction)
        for lane in self.lanes:
            if lane["table"].in_flight == self.transaction:
                lane["table"].in_flight = None
        self.finalized = True


# ------------------------------------------------------------------------------------------ prefix cache

HASH_DOMAIN = b"macllm-infer/token-prefix\0"


def hash_block(previous: bytes, block_tokens: int, block_index: int, tokens) -> bytes:  # prefix_cache.rs:563-586
    h = hashlib.sha256()
    h.update(HASH_DOMAIN)
    h.update(struct.pack("<IIII", 1, block_tokens, block_index, len(tokens)))
    h.update(previous)
    h.update(struct.pack(f"<{len(tokens)}I", *tokens))
    return h.digest()


def endpoint_digest(tokens, n: int, bt: int) -> bytes:
    chain = bytes(32)
    for b in range(div_ceil(n, bt)):
        chain = hash_block(chain, bt, b, list(tokens[b * bt:min((b + 1) * bt, n)]))
    return chain


def full_block_digests(tokens, bt: int) -> list[bytes]:
    out, chain = [], bytes(32)
    for b in range(len(tokens) // bt):
        chain = hash_block(chain, bt, b, list(tokens[b * bt:(b + 1) * bt]))
        out.append(chain)
    return out


@dataclass
class _Entry:
    tokens: tuple
    snapshot: object
    cost: int
    digest: bytes
    block_digests: list = field(default_factory=list)


class PrefixCache:
    def __init__(self, block_tokens: int, max_cost: int, drop=None):
        """`drop(snapshot)` runs for every snapshot the cache lets go of inside insert(): the one an
        identical key replaces and the ones evicted for room (in Rust these are dropped values)."""
        self.bt, self.max_cost = block_tokens, max_cost
        self.drop = drop
        self.resident = 0
        self.next_id = 0
        self.entries: "OrderedDict[int, _Entry]" = OrderedDict()  # order = LRU (front = least recent)
        self.hits = self.misses = self.matched_tokens = self.evictions = self.insertions = 0
        self.forced = False

    def insert(self, tokens, snapshot, cost: int):  # prefix_cache.rs:181-249; returns evicted snapshots
        tokens = tuple(int(t) for t in tokens)
        if not tokens or cost > self.max_cost:
            return None
        digest = endpoint_digest(tokens, len(tokens), self.bt)
        evicted = []
        for eid, e in list(self.entries.items()):
            if e.digest == digest and e.tokens == tokens:
                old = self._remove(eid, False)
                if self.drop:
                    self.drop(old)
                break
        while self.resident > self.max_cost - cost:
            ev = self.evict_lru()
            if ev is None:
                break
            evicted.append(ev)
            if self.drop:
                self.drop(ev)
        eid = self.next_id
        self.next_id += 1
        self.resident += cost
        self.entries[eid] = _Entry(tokens, snapshot, cost, digest, full_block_digests(tokens, self.bt))
        self.insertions += 1
        return evicted

    def force_collisions(self):   # force_collisions_for_tests: hits can then only come from the exact comparison
        assert not self.entries
        self.forced = True

    def lookup(self, prompt, exclusive_max=None):  # prefix_cache.rs:250-304: the longest exact endpoint below both bounds
        prompt = tuple(int(t) for t in prompt)
        limit = len(prompt) if exclusive_max is None else min(len(prompt), exclusive_max)
        best = None
        for eid, e in self.entries.items():
            n = len(e.tokens)
            if n < limit and e.tokens == prompt[:n] and (best is None or n > len(self.entries[best].tokens)):
                best = eid
        if best is None:
            self.misses += 1
            return None
        e = self.entries[best]
        self.hits += 1
        self.matched_tokens += len(e.tokens)
        self.entries.move_to_end(best)
        return len(e.tokens), e.snapshot

    def set_max_cost(self, max_cost):  # prefix_cache.rs:395-409; returns the evicted snapshots
        self.max_cost = max_cost
        evicted = []
        while self.resident > self.max_cost:
            ev = self.evict_lru()
            if ev is None:
                break
            evicted.append(ev)
            if self.drop:
                self.drop(ev)
        return evicted

    def lookup_aligned_common_prefix(self, prompt, exclusive_max=None):  # prefix_cache.rs:316-359
        prompt = tuple(int(t) for t in prompt)
        limit = len(prompt) if exclusive_max is None else min(len(prompt), exclusive_max)
        lengths = sorted({(b + 1) * self.bt for e in self.entries.values() for b in range(len(e.block_digests))
                          if (b + 1) * self.bt < limit}, reverse=True)
        if not lengths:
            self.misses += 1
            return None
        chains = full_block_digests(prompt[:lengths[0]], self.bt)
        for matched in lengths:
            digest = chains[matched // self.bt - 1]
            for eid in reversed(self.entries):  # most recently used first
                e = self.entries[eid]
                b = matched // self.bt - 1
                if b < len(e.block_digests) and e.block_digests[b] == digest and e.tokens[:matched] == prompt[:matched]:
                    self.hits += 1
                    self.matched_tokens += matched
                    self.entries.move_to_end(eid)
                    return matched, e.snapshot
        self.misses += 1
        return None

    def evict_lru(self):
        if not self.entries:
            return None
        eid = next(iter(self.entries))
        return self._remove(eid, True)

    def _remove(self, eid, count):
        e = self.entries.pop(eid)
        self.resident -= e.cost
        if count:
            self.evictions += 1
        return e.snapshot

    def stats(self) -> dict:
        return dict(entries=len(self.entries), cached_blocks=self.resident, capacity_blocks=self.max_cost, hits=self.hits,
                    misses=self.misses, matched_tokens=self.matched_tokens, insertions=self.insertions, evictions=self.evictions)
