"""Python mirror of the reference's model / session / engine surface over the C ABI.

`Model` follows the CausalLm trait (src/architecture.rs:1038-1246 of the reference): sessions,
prompt-prefix reset/publish, KV reservation, packed ragged forward, completion barrier.  `Engine`
follows EngineHandle / ServingScheduler (src/engine.rs): submit requests of raw token ids, drive
scheduler ticks, read back generated tokens.  Everything runs in libmacllm_b200.so.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _capi as capi


@dataclass
class Request:
    prompt: list | np.ndarray
    max_new_tokens: int
    ignore_stop_tokens: bool = True
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    seed: int = 0
    publish_prompt_prefix: bool = True
    event_capacity: int = 0             # events (one per token, one terminal) that may wait for `Engine.consume`; 0 = no bound
    event_send_timeout_ms: float = 0.0  # how long a full channel is tolerated before the request is given up


class Session:
    def __init__(self, model: "Model", _handle=None):
        self.model = model
        if _handle is not None:
            self._h = _handle
            return
        h = C.c_void_p()
        capi.check(capi.lib().mk_session_new(model._h, C.byref(h)))
        self._h = h

    def fork_prefix(self, logical_len: int) -> "Session":
        """A new session sharing this one's first logical_len tokens (copy-on-write on a shared partial tail)."""
        h = C.c_void_p()
        capi.check(capi.lib().mk_session_fork_prefix(self.model._h, self._h, logical_len, C.byref(h)))
        return Session(self.model, _handle=h)

    def __len__(self) -> int:
        n = C.c_int64()
        capi.check(capi.lib().mk_session_len(self._h, C.byref(n)))
        return int(n.value)

    def clear(self) -> None:
        capi.check(capi.lib().mk_session_clear(self._h))

    def block_table(self):
        cap = 1 << 16
        slots = np.empty(cap, np.uint32)
        gens = np.empty(cap, np.uint64)
        n = C.c_int32(cap)
        capi.check(capi.lib().mk_session_block_table(self._h, slots.ctypes.data, gens.ctypes.data, C.byref(n)))
        return slots[: n.value].copy(), gens[: n.value].copy()

    def close(self) -> None:
        if self._h:
            capi.lib().mk_session_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Model:
    """A decoder resident on one GPU (or the host-only fake used for scheduler tests)."""

    def __init__(self, handle, keep=None):
        self._h = handle
        self._keep = keep

    @staticmethod
    def _config(device=0, block_tokens=16, slab_blocks=8, kv_capacity_tokens=4096, prefix_capacity_tokens=0, kv_dtype="f16",
                max_batch_tokens=2048, max_batch_lanes=64, matmul_path=capi.PATH_AUTO, ep_rank=0, ep_size=1, ep_mode=0) -> capi.LoadConfig:
        cfg = capi.LoadConfig()
        cfg.device_ordinal = device
        cfg.block_tokens = block_tokens
        cfg.slab_blocks = slab_blocks
        cfg.kv_capacity_tokens = kv_capacity_tokens
        cfg.prefix_capacity_tokens = prefix_capacity_tokens
        cfg.kv_dtype = capi.TYPE_F16 if kv_dtype == "f16" else capi.TYPE_F32
        cfg.max_batch_tokens = max_batch_tokens
        cfg.max_batch_lanes = max_batch_lanes
        cfg.matmul_path = matmul_path
        cfg.ep_rank = ep_rank
        cfg.ep_size = ep_size
        cfg.ep_mode = ep_mode
        return cfg

    EP_ID_BYTES = 128

    @staticmethod
    def ep_unique_id() -> bytes:
        """Rank 0's id of a new expert-parallel group; hand it to the other ranks (file, store, socket)."""
        buf = (C.c_uint8 * Model.EP_ID_BYTES)()
        capi.check(capi.lib().mk_ep_unique_id(buf))
        return bytes(buf)

    def ep_init(self, unique_id: bytes) -> None:
        """Joins the expert-parallel group (collective: returns once all ep_size ranks have called it)."""
        if len(unique_id) != Model.EP_ID_BYTES:
            raise ValueError("expert-parallel id must be 128 bytes")
        buf = (C.c_uint8 * Model.EP_ID_BYTES).from_buffer_copy(unique_id)
        capi.check(capi.lib().mk_model_ep_init(self._h, buf))

    def ep_idle_tick(self) -> None:
        """Data-parallel expert parallelism: take part in this tick's exchanges without lanes of one's own."""
        capi.check(capi.lib().mk_model_ep_idle_tick(self._h))

    @staticmethod
    def inspect_gguf(path) -> dict:
        """Host-only audit of a checkpoint (container, family spec, every decoder tensor); raises MkError with the
        loader's message when load_gguf would refuse the file.  Needs no GPU."""
        s = capi.GgufSummary()
        capi.check(capi.lib().mk_gguf_inspect(str(path).encode(), C.byref(s)))
        out = {name: getattr(s, name) for name, _ in capi.GgufSummary._fields_}
        out["architecture"] = s.architecture.decode()
        return out

    @classmethod
    def load_gguf(cls, path, **kw) -> "Model":
        cfg = cls._config(**kw)
        h = C.c_void_p()
        capi.check(capi.lib().mk_model_load_gguf(str(path).encode(), C.byref(cfg), C.byref(h)))
        return cls(h)

    @classmethod
    def fake(cls, vocab=32, max_context=4096, fail_forward_at=-1, **kw) -> "Model":
        cfg = cls._config(**kw)
        h = C.c_void_p()
        capi.check(capi.lib().mk_model_new_fake(vocab, max_context, C.byref(cfg), fail_forward_at, C.byref(h)))
        return cls(h)

    def inject_failure(self, site: str, index: int) -> None:
        """Fake model only: make call number `index` at 'forward' | 'read_output' | 'admission' | 'synchronize' fail;
        'clear_session' counts from this call on."""
        sites = {"forward": 0, "read_output": 1, "admission": 2, "synchronize": 3, "clear_session": 4}
        capi.check(capi.lib().mk_model_fake_inject(self._h, sites[site], index))

    def script(self, stop_ids=(), logits_row=()) -> None:
        """Fake model only: stop token ids, and one logits row that every forward returns for every lane (empty: the one-hot rows)."""
        stops = np.asarray(list(stop_ids), np.uint32)
        row = np.asarray(list(logits_row), np.float32)
        capi.check(capi.lib().mk_model_fake_script(self._h, stops.ctypes.data if len(stops) else None, len(stops),
                                                   row.ctypes.data if len(row) else None, len(row)))

    def on_next_barrier(self, fn) -> None:
        """Fake model only: call `fn()` once inside the next completion barrier (while the engine waits for a forward)."""
        self._barrier_cb = C.CFUNCTYPE(None, C.c_void_p)(lambda _user: fn())   # kept alive until it has run
        capi.check(capi.lib().mk_model_fake_on_barrier(self._h, C.cast(self._barrier_cb, C.c_void_p), None))

    def spec(self) -> capi.RuntimeSpec:
        s = capi.RuntimeSpec()
        capi.check(capi.lib().mk_model_spec(self._h, C.byref(s)))
        return s

    def new_session(self) -> Session:
        return Session(self)

    def reset_session_for_prompt(self, session: Session, tokens) -> int:
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        cached = C.c_int64()
        capi.check(capi.lib().mk_reset_session_for_prompt(self._h, session._h, t.ctypes.data, len(t), C.byref(cached)))
        return int(cached.value)

    def publish_prompt_prefix(self, session: Session, tokens) -> None:
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        capi.check(capi.lib().mk_publish_prompt_prefix(self._h, session._h, t.ctypes.data, len(t)))

    def pool_stats(self) -> dict:
        s = capi.PoolStats()
        capi.check(capi.lib().mk_pool_stats_query(self._h, C.byref(s)))
        return s.as_dict()

    def kv_capacity(self) -> dict:
        c = capi.KvCapacity()
        capi.check(capi.lib().mk_kv_capacity_query(self._h, C.byref(c)))
        return {n: getattr(c, n) for n, _ in c._fields_}

    def prefix_diagnostics(self) -> dict:
        d = capi.PrefixDiagnostics()
        capi.check(capi.lib().mk_prefix_diagnostics_query(self._h, C.byref(d)))
        return d.as_dict()

    def _lanes(self, lanes):
        """lanes: list of (session, token ids, start_pos).  Returns (ctypes array, keep-alive list)."""
        arr = (capi.Lane * len(lanes))()
        keep = []
        for i, (session, ids, start_pos) in enumerate(lanes):
            t = np.ascontiguousarray(ids, dtype=np.uint32)
            keep.append(t)
            arr[i].session = session._h
            arr[i].input_ids = t.ctypes.data_as(C.POINTER(C.c_uint32))
            arr[i].n_tokens = len(t)
            arr[i].start_pos = start_pos
        return arr, keep

    def forward_batch(self, lanes, want_logits=True, want_tokens=True):
        """reserve_batch_kv + forward_batch_tokens_reserved + read_output_to_cpu for one packed ragged
        batch.  Returns (logits [lanes, vocab] or None, tokens [lanes] or None)."""
        arr, keep = self._lanes(lanes)
        r = C.c_void_p()
        capi.check(capi.lib().mk_reserve_batch(self._h, arr, len(lanes), C.byref(r)))
        flags = (capi.FWD_WANT_LOGITS if want_logits else 0) | (capi.FWD_WANT_TOKENS if want_tokens else 0)
        capi.check(capi.lib().mk_forward_batch_reserved(self._h, arr, len(lanes), r, flags))
        vocab = self.spec().vocab_size
        logits = np.empty((len(lanes), vocab), np.float32) if want_logits else None
        tokens = np.empty(len(lanes), np.uint32) if want_tokens else None
        capi.check(capi.lib().mk_read_output(self._h, None if logits is None else logits.ctypes.data,
                                             None if tokens is None else tokens.ctypes.data))
        del keep
        return logits, tokens

    def last_forward_ms(self) -> float:
        v = C.c_float()
        capi.check(capi.lib().mk_last_forward_ms(self._h, C.byref(v)))
        return float(v.value)

    def launch_count(self) -> int:
        v = C.c_int64()
        capi.check(capi.lib().mk_launch_count(self._h, C.byref(v)))
        return int(v.value)

    def transfer_bytes(self) -> tuple[int, int]:
        """(host-to-device, device-to-host) bytes moved by forwards since load."""
        a, b = C.c_int64(), C.c_int64()
        capi.check(capi.lib().mk_transfer_bytes(self._h, C.byref(a), C.byref(b)))
        return int(a.value), int(b.value)

    def profile_enable(self, on: bool) -> None:
        capi.check(capi.lib().mk_profile_enable(self._h, 1 if on else 0))

    def profile_query(self) -> list[dict]:
        """Per kernel class: launches, summed device ms (CUDA events), algorithmic bytes and flops."""
        n = C.c_int32(32)
        arr = (capi.KernelProfile * 32)()
        capi.check(capi.lib().mk_profile_query(self._h, arr, C.byref(n)))
        return [dict(name=arr[i].name.decode(), launches=arr[i].launches, ms=arr[i].ms, bytes=arr[i].bytes, flops=arr[i].flops)
                for i in range(n.value)]

    def synchronize(self) -> None:
        capi.check(capi.lib().mk_synchronize(self._h))

    def close(self) -> None:
        if self._h:
            capi.lib().mk_model_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_STATES = ("running", "done", "failed", "cancelled")
FORWARD_KINDS = ("suffix_prefill", "first_token", "decode", "mixed")


class Engine:
    """The continuous-batching scheduler over one model."""

    def __init__(self, model: Model, max_active_sequences=2, scheduler_token_budget=256, prefill_token_quantum=128,
                 queue_capacity=8, record_logits=False, host_sampling=False):
        self.model = model
        cfg = capi.EngineConfig(max_active_sequences, scheduler_token_budget, prefill_token_quantum, queue_capacity,
                                1 if record_logits else 0, 1 if host_sampling else 0)
        h = C.c_void_p()
        capi.check(capi.lib().mk_engine_new(model._h, C.byref(cfg), C.byref(h)))
        self._h = h

    def submit(self, requests, atomic_batch=False) -> list[int]:
        n = len(requests)
        arr = (capi.Request * n)()
        keep = []
        for i, r in enumerate(requests):
            t = np.ascontiguousarray(r.prompt, dtype=np.uint32)
            keep.append(t)
            arr[i].prompt = t.ctypes.data_as(C.POINTER(C.c_uint32))
            arr[i].n_prompt = len(t)
            arr[i].max_new_tokens = r.max_new_tokens
            arr[i].ignore_stop_tokens = 1 if r.ignore_stop_tokens else 0
            arr[i].temperature = r.temperature
            arr[i].top_k = r.top_k
            arr[i].top_p = r.top_p
            arr[i].repetition_penalty = r.repetition_penalty
            arr[i].presence_penalty = r.presence_penalty
            arr[i].frequency_penalty = r.frequency_penalty
            arr[i].seed = r.seed
            arr[i].no_prefix_publication = 0 if r.publish_prompt_prefix else 1
            arr[i].event_capacity = r.event_capacity
            arr[i].event_send_timeout_ms = r.event_send_timeout_ms
        ids = np.empty(n, np.int32)
        capi.check(capi.lib().mk_engine_submit(self._h, arr, n, 1 if atomic_batch else 0, ids.ctypes.data))
        return [int(x) for x in ids]

    def step(self, now_ms: float | None = None) -> int:
        """One scheduler tick; `now_ms` is the clock that event-channel timeouts are measured against (the engine's own if None)."""
        lanes = C.c_int32()
        if now_ms is None:
            capi.check(capi.lib().mk_engine_step(self._h, C.byref(lanes)))
        else:
            capi.check(capi.lib().mk_engine_step_at(self._h, float(now_ms), C.byref(lanes)))
        return int(lanes.value)

    def consume(self, request_id: int, n: int = 1) -> None:
        """The host took `n` events of the request out of its channel."""
        capi.check(capi.lib().mk_engine_consume_events(self._h, request_id, n))

    def run(self) -> None:
        capi.check(capi.lib().mk_engine_run(self._h))

    def pending(self) -> int:
        n = C.c_int32()
        capi.check(capi.lib().mk_engine_pending(self._h, C.byref(n)))
        return int(n.value)

    def cancel(self, request_id: int) -> None:
        """EngineTicket::cancel of the reference (src/engine.rs:1136-1145): sticky; the scheduler drops the request at its
        next look at it. May be called from another thread while `step` runs."""
        capi.check(capi.lib().mk_engine_cancel(self._h, request_id))

    def keep_trace(self, keep: bool) -> None:
        """Turn the per-tick records on or off (off drops those kept so far); a server runs with them off."""
        capi.check(capi.lib().mk_engine_keep_trace(self._h, 1 if keep else 0))

    def release(self, request_id: int) -> None:
        """Drop the stored result of a request that has ended."""
        capi.check(capi.lib().mk_engine_release_request(self._h, request_id))

    def progress(self, request_id: int):
        """(generated tokens so far, state, prompt tokens served from the prefix cache) without copying the tokens."""
        n = C.c_int32(0)
        fin = C.c_int32()
        cached = C.c_int64()
        capi.check(capi.lib().mk_engine_result(self._h, request_id, None, C.byref(n), C.byref(fin), C.byref(cached)))
        return int(n.value), _STATES[fin.value], int(cached.value)

    def result(self, request_id: int):
        """Returns dict(tokens, state ('running' | 'done' | 'failed' | 'cancelled'), cached_tokens, message, kind)."""
        count, _, _ = self.progress(request_id)
        toks = np.empty(max(count, 1), np.uint32)
        n = C.c_int32(len(toks))
        fin = C.c_int32()
        cached = C.c_int64()
        capi.check(capi.lib().mk_engine_result(self._h, request_id, toks.ctypes.data, C.byref(n), C.byref(fin), C.byref(cached)))
        state = _STATES[fin.value]
        msg = capi.lib().mk_last_error().decode() if state == "failed" else ""
        kind = C.c_int32()
        capi.check(capi.lib().mk_engine_failure_kind(self._h, request_id, C.byref(kind)))
        return dict(tokens=toks[: n.value].copy(), state=state, cached_tokens=int(cached.value), message=msg,
                    kind=("none", "invalid_request", "resource_exhausted", "internal", "fatal")[kind.value])

    def status(self) -> str:
        """EngineStatus of the reference: 'ready', 'busy' or 'poisoned'."""
        st = C.c_int32()
        capi.check(capi.lib().mk_engine_status(self._h, C.byref(st)))
        return {1: "ready", 2: "busy", 3: "poisoned"}.get(st.value, "stopped")

    def logits(self, request_id: int) -> np.ndarray:
        rows = C.c_int32()
        capi.check(capi.lib().mk_engine_logits(self._h, request_id, None, C.byref(rows)))
        vocab = self.model.spec().vocab_size
        out = np.empty((rows.value, vocab), np.float32)
        if rows.value:
            capi.check(capi.lib().mk_engine_logits(self._h, request_id, out.ctypes.data, C.byref(rows)))
        return out

    def trace(self) -> list[list[tuple[int, int, int]]]:
        """Every packed forward so far: [(request id, start position, token count), ...] per tick."""
        out = []
        tick = 0
        while True:
            n = C.c_int32(0)
            st = capi.lib().mk_engine_trace(self._h, tick, None, C.byref(n))
            if st != 0:
                break
            arr = (capi.TickLane * max(n.value, 1))()
            m = C.c_int32(n.value)
            capi.check(capi.lib().mk_engine_trace(self._h, tick, arr, C.byref(m)))
            out.append([(arr[i].request_id, arr[i].start_pos, arr[i].n_tokens) for i in range(m.value)])
            tick += 1
        return out

    def metrics(self, request_id: int) -> dict:
        """The model-side GenerationMetrics of a request (src/generation.rs:35-58): token counts, decode steps, finish reason
        and the device time of the forwards it joined, by the phase its lane was in."""
        m = capi.RequestMetrics()
        capi.check(capi.lib().mk_engine_request_metrics(self._h, request_id, C.byref(m)))
        out = {name: getattr(m, name) for name, _ in m._fields_ if name != "reserved_"}
        out["finish_reason"] = (None, "length", "stop", "cancelled")[m.finish_reason]
        return out

    def tick_info(self, tick: int) -> dict:
        """Kind ('suffix_prefill' | 'first_token' | 'decode' | 'mixed'), lane count, input tokens, device time and the lanes'
        phases of one packed forward - the reference's BenchmarkPackedForwardRecord (src/engine.rs:452-460)."""
        info = capi.TickInfo()
        capi.check(capi.lib().mk_engine_tick_info(self._h, tick, C.byref(info)))
        arr = (capi.TickLane * max(info.lane_count, 1))()
        m = C.c_int32(max(info.lane_count, 1))
        capi.check(capi.lib().mk_engine_trace(self._h, tick, arr, C.byref(m)))
        return dict(kind=FORWARD_KINDS[info.kind], lane_count=info.lane_count, input_tokens=info.input_tokens, model_ms=info.model_ms,
                    phases=[FORWARD_KINDS[arr[i].phase] for i in range(m.value)])

    def batch_trace(self, member_request_id: int) -> dict:
        """EngineBatchTrace of the atomic batch the request was submitted in (src/engine.rs:462-484); `complete` turns true
        once admission ran and every member has ended."""
        t = capi.BatchTrace()
        n = C.c_int32(0)
        capi.check(capi.lib().mk_engine_batch_trace(self._h, member_request_id, C.byref(t), None, C.byref(n)))
        ticks = (C.c_int64 * max(n.value, 1))()
        m = C.c_int32(max(n.value, 1))
        capi.check(capi.lib().mk_engine_batch_trace(self._h, member_request_id, C.byref(t), ticks, C.byref(m)))
        out = {name: getattr(t, name) for name, _ in t._fields_ if name != "reserved_"}
        out["complete"] = bool(out["complete"])
        out["forward_ticks"] = [int(ticks[i]) for i in range(m.value)]
        return out

    def stats(self) -> dict:
        s = capi.EngineStats()
        capi.check(capi.lib().mk_engine_stats_query(self._h, C.byref(s)))
        return {n: getattr(s, n) for n, _ in s._fields_}

    def close(self) -> None:
        if self._h:
            capi.lib().mk_engine_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def run_expert_parallel(engine: Engine, model: Model, all_reduce_sum, outstanding=None, on_tick=None) -> int:
    """Drives `engine` in lock step with the other ranks of an expert-parallel group with data-parallel lanes
    (ep_mode=1): every rank schedules its own sequences, and every MoE layer of every tick is one exchange that all ranks
    take part in, so a rank without a lane to run takes the tick idle.  `all_reduce_sum(n)` returns the sum of n over all
    ranks (torch.distributed, MPI, a socket: the library does not care); `outstanding()` is this rank's count of requests
    not yet finished, including ones it has yet to submit (default: the engine's pending count); `on_tick()` runs before
    each tick (a place to submit arrivals).  Returns the number of ticks."""
    ticks = 0
    while True:
        if on_tick is not None:
            on_tick()
        if all_reduce_sum(engine.pending() if outstanding is None else outstanding()) <= 0:
            break
        if engine.step() == 0:
            model.ep_idle_tick()
        ticks += 1
    model.synchronize()
    return ticks
