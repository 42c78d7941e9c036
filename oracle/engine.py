"""CPU ORACLE - TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Python restatement of the reference's scheduler tick and per-sequence phase machine
(src/engine.rs:1654-2614, src/generation.rs:787-1266) and of the model-side glue between sessions,
the paged KV pool and the prefix cache (src/decoder.rs:3392-3758,4125-4201).  The arithmetic of a
forward is supplied by a `forward` callable: oracle.decoder.Decoder for real checkpoints, or
`fake_forward` (one-hot logits) for scheduler-only cases.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

import math
import numpy as np

from . import kv


def fake_next_token(token: int, pos: int, vocab: int) -> int:
    return (31 * int(token) + 7 * int(pos) + 3) % vocab


class OracleModel:
    """Sessions + pool + prefix cache + transactional forward (the DecoderModel glue)."""

    def __init__(self, vocab, max_context, block_tokens=16, slab_blocks=8, kv_capacity_tokens=4096, prefix_capacity_tokens=0,
                 decoder=None, stop_ids=()):
        self.vocab, self.max_context = vocab, max_context
        self.pool = kv.Pool(block_tokens, slab_blocks, kv.div_ceil(kv_capacity_tokens, block_tokens))  # src/runtime.rs:194
        self.prefix = None
        if prefix_capacity_tokens > 0:
            budget = min(kv.div_ceil(prefix_capacity_tokens, block_tokens), self.pool.max_blocks)  # decoder.rs:3403-3412
            self.prefix = kv.PrefixCache(block_tokens, budget, drop=lambda snap: snap.drop())
        self.decoder = decoder
        self.stop_ids = tuple(stop_ids)
        if decoder is not None:
            decoder.bind_pool(self.pool)

    def new_session(self):
        return dict(table=kv.Table(self.pool, self.max_context), len=0)

    def clear_session(self, s):
        old = s["table"].logical_len
        s["table"].clear()
        if old != 0 and s["table"].logical_len != 0:
            return
        s["len"] = 0

    def reset_session_for_prompt(self, s, prompt) -> int:  # decoder.rs:3494-3532
        self.clear_session(s)
        if self.prefix is None:
            return 0
        hit = self.prefix.lookup_aligned_common_prefix(prompt, len(prompt))
        if hit is None:
            return 0
        matched, snapshot = hit
        s["table"].attach_prefix(snapshot, matched)
        s["len"] = matched
        return matched

    def publish_prompt_prefix(self, s, tokens) -> None:  # decoder.rs:3534-3603
        if self.prefix is None:
            return
        bt = self.prefix.bt
        n = len(tokens) // bt * bt
        if n == 0 or s["len"] < n:
            return
        fork = s["table"].fork_prefix(n)
        if self.prefix.insert(tokens[:n], fork, max(len(fork.blocks), 1)) is None:
            fork.drop()  # the cost exceeds the whole budget: the fork is dropped again

    def reserve_batch(self, lanes):  # decoder.rs:3696-3758; lanes: (session, start_pos, n_tokens)
        for s, start, n in lanes:
            if n <= 0:
                raise kv.Invalid("input sequence cannot be empty")
            if s["len"] != start:
                raise kv.Invalid(f"start_pos {start} does not match decoder sequence length {s['len']}")
        while True:
            try:
                return self.pool.reserve_batch([s["table"] for s, _, _ in lanes], [n for _, _, n in lanes])
            except kv.Exhausted as e:
                snap = self.prefix.evict_lru() if self.prefix is not None else None
                if snap is not None:
                    snap.drop()
                    continue
                st = self.pool.stats()   # classify_reservation_error, decoder.rs:3970-3994; KvCacheExhausted, architecture.rs:928-953
                free_now = st["free_blocks"] + (self.pool.max_blocks - st["allocated_blocks"])
                raise kv.Exhausted(e.requested, e.free_blocks, e.unallocated,
                                   f"KV cache requires {e.requested} additional blocks, but only {free_now} of {self.pool.max_blocks} are free "
                                   f"({st['retired_blocks']} retired, {self.pool.block_tokens} tokens/block)")

    def forward(self, lanes, reservation, want_logits=True):
        """lanes: (session, ids, start_pos).  Returns logits [lanes, vocab] (or next tokens for the fake)."""
        reservation.mark_all_used()
        if self.decoder is None:
            out = np.zeros((len(lanes), self.vocab), np.float32)
            for i, (_, ids, start) in enumerate(lanes):
                out[i, fake_next_token(ids[-1], start + len(ids) - 1, self.vocab)] = 1.0
        else:
            out = self.decoder.forward(lanes, reservation)
        reservation.commit()
        for s, ids, start in lanes:
            s["len"] = start + len(ids)
        self.pool.mark_completed_through(self.pool.submitted_epoch)  # CPU path: decoder.rs:4191-4199
        return out


@dataclass
class Req:
    prompt: list
    max_new_tokens: int
    ignore_stop_tokens: bool = True
    temperature: float = 0.0
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    publish_prompt_prefix: bool = True
    event_capacity: int = 0              # mpsc::channel(event_capacity), engine.rs:755-767; 0 = no bound
    event_send_timeout_ms: float = 0.0


@dataclass
class _Seq:
    rid: int
    req: Req
    session: dict
    history: list
    prompt_tokens: int
    phase: str = "prefill"
    cursor: int = 0
    decode_token: int = 0
    generated: int = 0
    delivering: bool = False
    reclaimed: dict | None = None
    pending_events: int = 0
    in_channel: int = 0
    blocked_since: float | None = None


@dataclass
class Result:
    tokens: list = field(default_factory=list)
    state: str = "running"
    message: str = ""
    cached_tokens: int = 0
    logits: list = field(default_factory=list)


class OracleEngine:
    def __init__(self, model: OracleModel, max_active_sequences=2, scheduler_token_budget=256, prefill_token_quantum=128,
                 queue_capacity=8, record_logits=False, sampler=None):
        # EngineConfig::validate, engine.rs:350-367
        for value, what in ((queue_capacity, "queue capacity"), (max_active_sequences, "maximum active sequences"),
                            (scheduler_token_budget, "scheduler token budget"), (prefill_token_quantum, "prefill token quantum")):
            if value <= 0:
                raise ValueError(f"{what} must be positive")
        if prefill_token_quantum > scheduler_token_budget:
            raise ValueError("prefill token quantum cannot exceed the scheduler token budget")
        self.m = model
        self.max_active, self.budget, self.quantum, self.queue_capacity = (max_active_sequences, scheduler_token_budget,
                                                                            prefill_token_quantum, queue_capacity)
        self.record_logits = record_logits
        self.sampler = sampler
        self.sessions = [model.new_session() for _ in range(max_active_sequences)]  # engine.rs:1336-1360
        self.queue: deque = deque()
        self.pending_atomic: list = []
        self.active: deque = deque()
        self.results: dict[int, Result] = {}
        self.trace: list = []
        self.next_id = self.next_batch = 0
        self.round_visits = self.round_budget = 0
        self.kv_shrinks = 0
        self.cancelled: set[int] = set()   # EngineTicket::cancel, engine.rs:1136-1145: sticky
        self.tick_kinds: list = []
        self.on_barrier = None             # test hook: called once after the next forward's completion barrier

    def cancel(self, rid):
        self.cancelled.add(rid)

    def _finish_cancelled(self, rid):
        if self.results[rid].state == "running":
            self.results[rid].state = "cancelled"

    def submit(self, reqs, atomic_batch=False):  # submit_batch_with_policy, engine.rs:976-1053 (order and wording: 394-426)
        if not reqs:
            raise RuntimeError("inference batch must not be empty")
        limit = min(self.queue_capacity, self.max_active)
        if atomic_batch and len(reqs) > limit:
            raise RuntimeError(f"inference batch contains {len(reqs)} requests, but the atomic admission limit is {limit}")
        if len(self.queue) + len(reqs) > self.queue_capacity:
            raise RuntimeError("inference queue is full")
        batch = None
        if atomic_batch:
            batch = (self.next_batch, len(reqs))
            self.next_batch += 1
        ids = []
        for r in reqs:
            rid = self.next_id
            self.next_id += 1
            self.results[rid] = Result()
            self.queue.append((rid, r, batch))
            ids.append(rid)
        return ids

    def pending(self):
        return len(self.queue) + len(self.pending_atomic) + len(self.active)

    def _fail(self, rid, msg):
        self.results[rid].state, self.results[rid].message = "failed", msg

    def _admit(self, rid, r: Req):  # engine.rs:1654-1808
        if rid in self.cancelled:  # skipped before preflight and model work, engine.rs:1671-1674
            return self._finish_cancelled(rid)
        # prepare_request for token-id input, engine.rs:2976-3021
        if not r.prompt:
            return self._fail(rid, "raw token prompt must not be empty")
        for i, t in enumerate(r.prompt):
            if t >= self.m.vocab:
                return self._fail(rid, f"raw prompt token {t} at index {i} exceeds model vocabulary {self.m.vocab}")
        if len(r.prompt) + max(r.max_new_tokens - 1, 0) > self.m.max_context:
            return self._fail(rid, f"This model's maximum context length is {self.m.max_context} tokens; the prompt ({len(r.prompt)} tokens) "
                                   f"plus requested output ({r.max_new_tokens} tokens) exceeds it")
        why = None  # Sampler::new + set_penalties, sampling.rs:43-79; reported as in engine.rs:3022-3032
        top_p = getattr(r, "top_p", 1.0)
        if not (math.isfinite(r.temperature) and r.temperature >= 0.0):
            why = "temperature must be finite and non-negative"
        elif not (math.isfinite(top_p) and 0.0 < top_p <= 1.0):
            why = "top_p must be finite and in (0, 1]"
        elif not (math.isfinite(r.repetition_penalty) and r.repetition_penalty > 0.0):
            why = "repetition_penalty must be finite and positive"
        elif not (math.isfinite(r.presence_penalty) and -2.0 <= r.presence_penalty <= 2.0):
            why = "invalid presence_penalty"
        elif not (math.isfinite(r.frequency_penalty) and -2.0 <= r.frequency_penalty <= 2.0):
            why = "invalid frequency_penalty"
        if why is not None:
            return self._fail(rid, "invalid sampling parameters: " + why)
        max_cached = 0 if r.max_new_tokens == 0 else len(r.prompt) + r.max_new_tokens - 1  # engine.rs:2839-2863
        if max_cached > self.m.pool.max_blocks * self.m.pool.block_tokens:
            return self._fail(rid, f"request requires up to {max_cached} cached tokens, exceeding the configured shared KV capacity of "
                                   f"{self.m.pool.max_blocks} blocks \u00d7 {self.m.pool.block_tokens} tokens")
        session = self.sessions.pop()  # LIFO, engine.rs:1719-1722
        seq = _Seq(rid, r, session, list(r.prompt), len(r.prompt))
        cached = self.m.reset_session_for_prompt(session, seq.history)  # generation.rs:799
        assert cached < len(seq.history)
        seq.cursor = cached
        self.results[rid].cached_tokens = cached
        self.active.append(seq)

    def _admit_pending_atomic(self):  # engine.rs:1886-1936
        if not self.pending_atomic:
            return
        if len(self.pending_atomic) > self.max_active - len(self.active):
            return
        batch, self.pending_atomic = self.pending_atomic, []
        for rid, r in batch:
            self._admit(rid, r)

    def _try_admit(self):  # engine.rs:1810-1881
        self._admit_pending_atomic()
        if self.pending_atomic:
            return
        while len(self.active) < self.max_active and self.queue:
            rid, r, batch = self.queue.popleft()
            if batch is None:
                self._admit(rid, r)
                continue
            self.pending_atomic = [(rid, r)]
            while len(self.pending_atomic) < batch[1]:
                rid2, r2, b2 = self.queue.popleft()
                assert b2 == batch
                self.pending_atomic.append((rid2, r2))
            self._admit_pending_atomic()
            if self.pending_atomic:
                break

    def _reclaim(self, s: _Seq):
        if s.reclaimed is None:
            self.m.clear_session(s.session)
            s.reclaimed = s.session
            s.session = None

    def consume(self, rid, n=1):  # the receiver side of the request's event channel
        for s in self.active:
            if s.rid == rid:
                s.in_channel = max(0, s.in_channel - n)

    def _flush(self, s: _Seq, now_ms: float) -> str:  # ActiveSequence::flush_pending, engine.rs:1408-1465
        if s.rid in self.cancelled:
            s.pending_events = 0
            return "abandoned"
        if s.req.event_capacity <= 0:
            s.pending_events = 0
            return "drained"
        while s.pending_events > 0:
            if s.in_channel < s.req.event_capacity:
                s.in_channel += 1
                s.pending_events -= 1
                s.blocked_since = None
                continue
            if s.blocked_since is None:
                s.blocked_since = now_ms
            if now_ms - s.blocked_since >= s.req.event_send_timeout_ms:
                self.cancelled.add(s.rid)
                s.pending_events = 0
                return "abandoned"
            return "blocked"
        return "drained"

    def step(self, now_ms: float = 0.0) -> int:  # drive_once, engine.rs:1938-1964
        self._try_admit()
        if not self.active:
            return 0
        if self.round_visits == 0 or self.round_budget == 0:
            self.round_visits, self.round_budget = len(self.active), self.budget
        visit_limit = min(self.round_visits, len(self.active))
        actions = []
        token_budget = self.round_budget
        for index in range(visit_limit):  # collect_visits, engine.rs:2005-2095
            if token_budget == 0:
                break
            s = self.active[index]
            initial = self._flush(s, now_ms)
            if initial == "abandoned":  # engine.rs:1409-1417,2024-2029
                actions.append(dict(kind="remove"))
                continue
            if initial == "blocked":    # engine.rs:2030-2032
                actions.append(dict(kind="keep"))
                continue
            if s.delivering:
                actions.append(dict(kind="remove"))
                continue
            step_budget = min(self.quantum, token_budget)
            if s.phase == "finished" or s.req.max_new_tokens == 0:
                actions.append(dict(kind="complete", finished=True))
                continue
            if s.phase == "prefill":
                start, n, was_prefill = s.cursor, min(s.prompt_tokens - s.cursor, step_budget), True
            else:
                start, n, was_prefill = s.prompt_tokens + max(s.generated - 1, 0), 1, False
            assert s.session["len"] == start
            token_budget -= n
            actions.append(dict(kind="preview", start=start, n=n, was_prefill=was_prefill))
        visits = len(actions)
        for i, a in enumerate(actions):
            if a["kind"] == "remove":
                self._reclaim(self.active[i])
                if self.active[i].rid in self.cancelled:
                    self._finish_cancelled(self.active[i].rid)
        candidates = [i for i, a in enumerate(actions) if a["kind"] == "preview"]
        reservation = None
        input_tokens = 0
        selected = len(candidates)
        if candidates:  # reserve_and_prepare_visits, engine.rs:2097-2167
            while True:
                lanes = [(self.active[i].session, actions[i]["start"], actions[i]["n"]) for i in candidates[:selected]]
                try:
                    reservation = self.m.reserve_batch(lanes)
                    break
                except kv.Exhausted as e:
                    if selected > 1:
                        selected -= 1
                        self.kv_shrinks += 1
                        continue
                    for i in candidates:
                        actions[i] = dict(kind="keep")
                    s = self.active[candidates[0]]
                    self._fail(s.rid, str(e))
                    s.pending_events += 1
                    s.delivering = True
                    self._reclaim(s)
                    selected = 0
                    break
            for i in candidates[selected:]:
                actions[i] = dict(kind="keep")
            for i in candidates[:selected]:
                a, s = actions[i], self.active[i]
                a["ready"] = (not a["was_prefill"]) or a["start"] + a["n"] == s.prompt_tokens
                a["kind"] = "forward"
                input_tokens += a["n"]
        fwd = [i for i, a in enumerate(actions) if a["kind"] == "forward"]
        if fwd:  # execute_prepared_visits, engine.rs:2233-2269
            lanes, tick, phases = [], [], []
            for i in fwd:
                a, s = actions[i], self.active[i]
                ids = s.history[a["start"]:a["start"] + a["n"]] if a["was_prefill"] else [s.decode_token]
                lanes.append((s.session, ids, a["start"]))
                tick.append((s.rid, a["start"], a["n"]))
                phases.append("decode" if not a["was_prefill"] else ("first_token" if a["ready"] else "suffix_prefill"))
            logits = self.m.forward(lanes, reservation)
            self.trace.append(tick)
            # BenchmarkForwardKind of the packed forward, engine.rs:2347-2356
            self.tick_kinds.append(dict(kind=phases[0] if all(p == phases[0] for p in phases) else "mixed", phases=phases,
                                        lane_count=len(fwd), input_tokens=input_tokens))
            if self.on_barrier is not None:
                hook, self.on_barrier = self.on_barrier, None
                hook()
            for row, i in enumerate(fwd):  # complete_mixed_rows, engine.rs:2411-2523
                a, s = actions[i], self.active[i]
                nxt = a["start"] + a["n"]
                if s.req.publish_prompt_prefix and a["was_prefill"] and 0 < nxt <= s.prompt_tokens:
                    self.m.publish_prompt_prefix(s.session, s.history[:nxt])  # generation.rs:505-509
                a["kind"], a["finished"] = "complete", False
                if s.rid in self.cancelled:  # generation.rs:1201-1204: the row is consumed, nothing is sampled
                    s.phase, a["finished"] = "finished", True
                    self._finish_cancelled(s.rid)
                    continue
                if not a["ready"]:
                    s.phase, s.cursor = "prefill", nxt
                    continue
                lrow = np.array(logits[row], dtype=np.float32)
                if self.record_logits:
                    self.results[s.rid].logits.append(lrow.copy())
                token = self._sample(s, lrow)
                res = self.results[s.rid]
                if not s.req.ignore_stop_tokens and token in self.m.stop_ids:  # generation.rs:1221-1225
                    s.phase, a["finished"] = "finished", True
                    continue
                reaches = s.generated + 1 == s.req.max_new_tokens
                s.generated += 1
                s.history.append(token)
                res.tokens.append(token)
                s.pending_events += 1
                if reaches:
                    s.phase, a["finished"] = "finished", True
                    continue
                s.phase, s.decode_token = "decode", token
        elif reservation is not None:
            reservation.rollback()
        for i, a in enumerate(actions):  # finalize_visits, engine.rs:2525-2614
            s = self.active[i]
            if a["kind"] == "complete":
                if a["finished"]:
                    if self.results[s.rid].state == "running":
                        self.results[s.rid].state = "done"
                        s.pending_events += 1
                    self._reclaim(s)
                    s.delivering = True
                a["kind"] = "keep"
        for i, a in enumerate(actions):
            s = self.active[i]
            if a["kind"] == "remove":
                continue
            final = self._flush(s, now_ms)   # engine.rs:2559-2580
            if final == "drained" and s.delivering:
                self._reclaim(s)
                a["kind"] = "remove"
            elif final == "abandoned":
                a["kind"] = "remove" if s.reclaimed is not None else "keep"
        for a in actions:
            slot = self.active.popleft()
            if a["kind"] == "remove":
                self.sessions.append(slot.reclaimed)
            else:
                self.active.append(slot)
        self.round_visits -= visits
        self.round_budget -= input_tokens
        if not self.active:
            self.round_visits = self.round_budget = 0
        return len(fwd)

    def _sample(self, s: _Seq, row: np.ndarray) -> int:  # sampling.rs:95-142 (greedy path)
        from . import mathlib
        r = s.req
        generated = s.history[len(s.history) - s.generated:] if s.generated else []
        row = mathlib.apply_penalties(row, s.history, r.repetition_penalty, generated, r.presence_penalty, r.frequency_penalty)
        if r.temperature > 0:
            raise NotImplementedError("the oracle grades greedy sampling only (stochastic parity is unpinned)")
        return mathlib.argmax(row)

    def run(self):
        idle = 0
        while self.pending() > 0:
            idle = 0 if self.step() > 0 else idle + 1
            if idle > 4 * (self.max_active + 4):
                raise RuntimeError("scheduler made no progress")
