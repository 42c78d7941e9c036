"""The raw `/completion` surface in front of the continuous-batching engine.

Mirrors the reference's benchmark endpoint (`raw_completion`, src/server.rs:633-666; request contract
`RawCompletionRequest::validate`, src/server.rs:326-458; response projection `RawCompletionEvent`, src/server.rs:473-622;
streaming `next_raw_stream_event`, src/server.rs:721-806), plus `/healthz` and `/v1/models` (src/server.rs:273-322).
Chat Completions, templates and tool calls are not part of this path.

One difference from the reference: its `prompt` is text and goes through the model's tokenizer, which this library does
not carry.  Here `prompt` may be an array of token ids, or a string when the server was given a `tokenizer` (an object
with `encode(str) -> list[int]` and `decode(list[int]) -> str`); without one, `content` stays empty and the sampled
token ids travel in the `tokens` field of the streamed fragments, as they do in the reference.

Threads: the engine and its model handles belong to ONE inference worker thread (src/engine.rs:849-862); HTTP handler
threads only enqueue jobs and read each job's event queue.
"""
from __future__ import annotations

import json
import math
import queue
import select
import socket
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

from . import engine as _engine

# RAW_COMPLETION_RESPONSE_FIELDS (crates/macllm-chat/src/openai.rs:29-52)
RAW_COMPLETION_RESPONSE_FIELDS = [
    "index", "content", "stop", "tokens_predicted", "tokens_evaluated", "truncated", "stop_type",
    "generation_settings/seed", "generation_settings/temperature", "generation_settings/top_k", "generation_settings/top_p",
    "generation_settings/repeat_penalty", "generation_settings/ignore_eos", "generation_settings/stream",
    "generation_settings/max_tokens", "generation_settings/n_predict", "generation_settings/n_keep",
    "timings/cache_n", "timings/prompt_n", "timings/prompt_ms", "timings/predicted_n", "timings/predicted_ms",
]

_FIELDS = {  # name -> kind, in the order of RawCompletionRequest
    "prompt": "prompt", "n_predict": "usize", "temperature": "f64", "top_k": "usize", "top_p": "f64", "seed": "u64",
    "cache_prompt": "bool", "stream": "bool", "return_tokens": "bool", "id_slot": "usize", "ignore_eos": "bool",
    "repeat_penalty": "f64", "response_fields": "strings",
}


class ApiError(Exception):
    """The OpenAI-shaped error object (crates/macllm-chat/src/openai.rs:1382-1424)."""

    def __init__(self, status: int, message: str, error_type: str, param=None, code=None):
        super().__init__(message)
        self.status, self.message, self.error_type, self.param, self.code = status, message, error_type, param, code

    @classmethod
    def invalid_request(cls, message, param=None, code=None):
        return cls(400, message, "invalid_request_error", param, code)

    @classmethod
    def server_error(cls, message, status=500):
        return cls(status, message, "server_error", None, "internal_error")

    def body(self) -> dict:
        return {"error": {"message": self.message, "type": self.error_type, "param": self.param, "code": self.code}}


def _is_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def parse_raw_request(body: bytes) -> dict:
    """serde's part of the contract: a JSON object with exactly the thirteen fields, each of its type."""
    def bad(detail):
        return ApiError.invalid_request(f"invalid /completion request: {detail}", None, "invalid_json")
    try:
        v = json.loads(body)
    except (ValueError, UnicodeDecodeError) as e:
        raise bad(str(e))
    if not isinstance(v, dict):
        raise bad("expected a JSON object")
    for k in v:
        if k not in _FIELDS:
            raise bad(f"unknown field `{k}`")
    for k, kind in _FIELDS.items():
        if k not in v:
            raise bad(f"missing field `{k}`")
        x = v[k]
        ok = {
            "prompt": isinstance(x, str) or (isinstance(x, list) and all(_is_int(t) and 0 <= t < 2 ** 32 for t in x)),
            "usize": _is_int(x) and 0 <= x < 2 ** 64,
            "u64": _is_int(x) and 0 <= x < 2 ** 64,
            "f64": isinstance(x, (int, float)) and not isinstance(x, bool),
            "bool": isinstance(x, bool),
            "strings": isinstance(x, list) and all(isinstance(s, str) for s in x),
        }[kind]
        if not ok:
            raise bad(f"invalid type for field `{k}`")
    return v


def validate_raw_request(v: dict, max_context: int, tokenizer=None):
    """RawCompletionRequest::validate (src/server.rs:348-458): same checks, order, messages, params and codes.
    Returns (token ids, generation settings)."""
    def inv(message, param, code="invalid_value"):
        return ApiError.invalid_request(message, param, code)
    prompt = v["prompt"]
    if len(prompt) == 0:
        raise inv("prompt must not be empty", "prompt")
    if v["n_predict"] == 0 or v["n_predict"] > max_context:
        raise inv(f"n_predict must be in 1..={max_context}", "n_predict")
    t = float(v["temperature"])
    if not math.isfinite(t) or t < 0.0:
        raise inv("temperature must be finite and non-negative", "temperature")
    p = float(v["top_p"])
    if not math.isfinite(p) or p <= 0.0 or p > 1.0:
        raise inv("top_p must be finite and in (0, 1]", "top_p")
    if v["id_slot"] >= 8:
        raise inv("id_slot must be in 0..8", "id_slot")
    if not v["ignore_eos"]:
        raise inv("ignore_eos must be true for fixed-length benchmark completions", "ignore_eos", "unsupported_value")
    if not v["return_tokens"]:
        raise inv("return_tokens must be true for benchmark token-parity evidence", "return_tokens", "unsupported_value")
    if float(v["repeat_penalty"]) != 1.0 or math.copysign(1.0, float(v["repeat_penalty"])) != 1.0:
        raise inv("repeat_penalty must be 1.0 for the shared benchmark contract", "repeat_penalty", "unsupported_value")
    if list(v["response_fields"]) != RAW_COMPLETION_RESPONSE_FIELDS:
        raise inv("response_fields must exactly match the benchmark response projection", "response_fields", "unsupported_value")
    if isinstance(prompt, str):
        if tokenizer is None:
            raise inv("this server has no tokenizer: send the prompt as an array of token ids", "prompt", "unsupported_value")
        prompt = list(tokenizer.encode(prompt))
        if not prompt:
            raise inv("prompt must not be empty", "prompt")
    settings = {"seed": v["seed"], "temperature": t, "top_k": v["top_k"], "top_p": p, "repeat_penalty": 1.0, "ignore_eos": True,
                "stream": v["stream"], "max_tokens": v["n_predict"], "n_predict": v["n_predict"], "n_keep": 0}
    return [int(x) for x in prompt], settings


def fragment_event(content: str, token_id: int, n_decoded: int, prompt_tokens: int) -> dict:
    """RawCompletionEvent::fragment (src/server.rs:553-581)."""
    return {"index": 0, "content": content, "tokens": [token_id], "stop": False, "id_slot": -1,
            "tokens_predicted": n_decoded, "tokens_evaluated": prompt_tokens}


def terminal_event(content: str, settings: dict, m: dict) -> dict:
    """RawCompletionEvent::terminal (src/server.rs:583-622): exactly the 22 projected fields."""
    out = {"index": 0, "content": content, "stop": True, "tokens_predicted": m["generated_tokens"],
           "tokens_evaluated": m["prompt_tokens"], "truncated": False, "stop_type": m["stop_type"]}
    for k in ("seed", "temperature", "top_k", "top_p", "repeat_penalty", "ignore_eos", "stream", "max_tokens", "n_predict", "n_keep"):
        out[f"generation_settings/{k}"] = settings[k]
    out["timings/cache_n"] = m["cached_prompt_tokens"]
    out["timings/prompt_n"] = m["prompt_tokens"] - m["cached_prompt_tokens"]
    out["timings/prompt_ms"] = m["prefill_ms"]
    out["timings/predicted_n"] = m["generated_tokens"]
    out["timings/predicted_ms"] = max(0.0, m["total_ms"] - m["ttft_ms"])
    return out


class _Job:
    def __init__(self, tokens, settings, publish_prefix=True):
        self.tokens, self.settings, self.publish_prefix = tokens, settings, publish_prefix
        self.events: queue.Queue = queue.Queue()
        self.request_id = None
        self.seen = 0
        self.t_submit = time.perf_counter()
        self.t_first = None
        # set by the handler when its client is gone (EngineTicket's Drop, src/engine.rs:1141-1145): sticky; the worker passes
        # it on to the engine, which drops the request at its next look at it
        self.cancelled = threading.Event()
        self.cancel_sent = False
        # the request's event channel: the handler counts the events it has dealt with, the worker tells the engine
        self.taken = 0
        self.taken_sent = 0


class CompletionServer:
    """`engine_factory()` is called on the worker thread and returns (engine, model); the server owns both from then on.
    `metadata`: served_model / device / dtype strings of `/healthz` and `/v1/models`."""

    def __init__(self, engine_factory, bind=("127.0.0.1", 0), tokenizer=None, metadata=None, idle_wait_s=0.001,
                 event_capacity=0, event_send_timeout_s=30.0):
        self._factory = engine_factory
        self._tokenizer = tokenizer
        self._meta = dict(served_model="macllm-b200", device="cuda", dtype="f16")
        self._meta.update(metadata or {})
        self._inbox: queue.Queue = queue.Queue()
        self._stop = threading.Event()
        self._ready = threading.Event()
        self._status = "starting"
        self._max_context = 0
        self._idle_wait_s = idle_wait_s
        # EngineConfig::event_capacity / event_send_timeout (src/engine.rs:320-323; the reference's defaults are 16 events and
        # 30 s): how many events of a request may wait for its connection, and for how long a full channel is tolerated before
        # the request is given up.  0 = no bound.
        self._event_capacity = int(event_capacity)
        self._event_send_timeout_ms = float(event_send_timeout_s) * 1e3
        self._worker_error = None
        self._worker = threading.Thread(target=self._run_worker, name="inference-worker", daemon=True)
        server = self

        class Handler(BaseHTTPRequestHandler):
            protocol_version = "HTTP/1.1"

            def log_message(self, *a):  # quiet
                pass

            def _json(self, status, obj):
                data = json.dumps(obj, separators=(",", ":")).encode()
                try:
                    self.send_response(status)
                    self.send_header("Content-Type", "application/json")
                    self.send_header("Content-Length", str(len(data)))
                    self.end_headers()
                    self.wfile.write(data)
                except (BrokenPipeError, ConnectionResetError):   # the client left before its answer
                    self.close_connection = True

            def do_GET(self):
                if self.path == "/healthz":
                    st = server.status()
                    healthy = st in ("ready", "busy")
                    self._json(200 if healthy else 503, {"status": "ok" if healthy else "error", "worker": st, "model": server._meta["served_model"],
                                                         "device": server._meta["device"], "dtype": server._meta["dtype"]})
                elif self.path == "/v1/models":
                    self._json(200, {"object": "list", "data": [{"id": server._meta["served_model"], "object": "model", "created": 0,
                                                                  "owned_by": "macllm-infer"}]})
                else:
                    self._json(404, ApiError(404, "not found", "invalid_request_error", None, "not_found").body())

            def do_POST(self):
                if self.path != "/completion":
                    self._json(404, ApiError(404, "not found", "invalid_request_error", None, "not_found").body())
                    return
                body = self.rfile.read(int(self.headers.get("Content-Length", "0") or 0))
                try:
                    v = parse_raw_request(body)
                    tokens, settings = validate_raw_request(v, server._max_context, server._tokenizer)
                    # cache_prompt = false selects EngineRequestPolicy::benchmark_measured() (src/server.rs:434-438)
                    job = server._submit(tokens, settings, publish_prefix=bool(v["cache_prompt"]))
                except ApiError as e:
                    self._json(e.status, e.body())
                    return
                if settings["stream"]:
                    self._stream(job)
                else:
                    self._collect(job)

            def _client_gone(self) -> bool:
                """True once the peer has closed its side: a readable socket that yields no byte."""
                try:
                    readable, _, _ = select.select([self.connection], [], [], 0)
                    return bool(readable) and self.connection.recv(1, socket.MSG_PEEK) == b""
                except (OSError, ValueError):
                    return True

            def _next_event(self, job):
                """The job's next event, or None when the client went away first (the request is then given up)."""
                while True:
                    now = time.monotonic()
                    if now - getattr(self, "_last_peek", 0.0) >= 0.1:   # also while events keep coming (a collected response)
                        self._last_peek = now
                        if self._client_gone():
                            job.cancelled.set()
                            return None
                    try:
                        return job.events.get(timeout=0.1)
                    except queue.Empty:
                        pass

            def _collect(self, job):
                content = ""
                while True:
                    ev = self._next_event(job)
                    if ev is None:
                        self.close_connection = True
                        return
                    job.taken += 1
                    if ev[0] == "token":
                        content += ev[3]
                    elif ev[0] == "finished":
                        err = _check_terminal(job.settings, ev[1])
                        if err is not None:
                            self._json(500, err.body())
                        else:
                            self._json(200, terminal_event(content, job.settings, ev[1]))
                        return
                    else:
                        e = _engine_failure(ev[1], ev[2])
                        self._json(e.status, e.body())
                        return

            def _stream(self, job):
                self.send_response(200)
                self.send_header("Content-Type", "text/event-stream")
                self.send_header("Cache-Control", "no-cache")
                self.send_header("Connection", "close")
                self.end_headers()

                def send(obj):
                    self.wfile.write(b"data: " + json.dumps(obj, separators=(",", ":")).encode() + b"\n\n")
                    self.wfile.flush()
                last = 0
                try:
                    while True:
                        ev = self._next_event(job)
                        if ev is None:
                            break
                        if ev[0] == "token":
                            _, token_id, n_decoded, text = ev
                            if not (last < n_decoded <= job.settings["n_predict"]):
                                send(ApiError.server_error("inference worker emitted inconsistent raw token metadata").body())
                                break
                            last = n_decoded
                            send(fragment_event(text, token_id, n_decoded, len(job.tokens)))
                            job.taken += 1            # the event has left for the client: its place in the channel is free
                        elif ev[0] == "finished":
                            err = _check_terminal(job.settings, ev[1])
                            if err is None and last != ev[1]["generated_tokens"]:
                                err = ApiError.server_error("inference worker raw token metadata did not reconcile with terminal metrics")
                            send(err.body() if err is not None else terminal_event("", job.settings, ev[1]))
                            break
                        else:
                            send(_engine_failure(ev[1], ev[2]).body())
                            break
                except (BrokenPipeError, ConnectionResetError):
                    job.cancelled.set()
                self.close_connection = True

        class Httpd(ThreadingHTTPServer):
            request_queue_size = 1024   # the listen backlog: a wave of clients connecting at once must not wait for SYN retries
            daemon_threads = True

        self._httpd = Httpd(bind, Handler)
        self._http_thread = threading.Thread(target=self._httpd.serve_forever, name="http", daemon=True)

    # ------------------------------------------------------------------ lifecycle
    @property
    def port(self) -> int:
        return self._httpd.server_address[1]

    def start(self, timeout=120.0) -> "CompletionServer":
        self._worker.start()
        if not self._ready.wait(timeout):
            raise RuntimeError("inference worker did not start")
        if self._worker_error is not None:
            raise self._worker_error
        self._http_thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        self._inbox.put(None)
        self._httpd.shutdown()
        self._httpd.server_close()
        self._worker.join(timeout=30)

    def status(self) -> str:
        return self._status

    # ------------------------------------------------------------------ handler side
    def _submit(self, tokens, settings, publish_prefix=True) -> _Job:
        if self._status in ("poisoned", "stopped", "starting"):
            label = self._status.capitalize()
            raise ApiError.server_error(f"inference worker is unavailable ({label})", 503)
        job = _Job(tokens, settings, publish_prefix)
        reply: queue.Queue = queue.Queue()
        self._inbox.put((job, reply))
        err = reply.get()
        if err is not None:
            raise err
        return job

    # ------------------------------------------------------------------ worker side
    def _run_worker(self):
        try:
            engine, model = self._factory()
            self._max_context = int(model.spec().max_context)
        except Exception as e:  # the server never starts
            self._worker_error = e
            self._status = "stopped"
            self._ready.set()
            return
        if hasattr(engine, "keep_trace"):
            engine.keep_trace(False)      # a server lives long: no per-tick records, results released once delivered
        self._status = "ready"
        self._ready.set()
        active: dict[int, _Job] = {}
        draining: dict[int, _Job] = {}     # answered requests whose last events the engine still holds for their channel
        try:
            while not self._stop.is_set():
                # admit what the handlers queued; block only when there is nothing to run
                try:
                    item = self._inbox.get(timeout=self._idle_wait_s) if not active else self._inbox.get_nowait()
                except queue.Empty:
                    item = False
                while item:
                    job, reply = item
                    try:
                        s = job.settings
                        (rid,) = engine.submit([_engine.Request(job.tokens, s["n_predict"], ignore_stop_tokens=True, temperature=s["temperature"],
                                                                top_k=s["top_k"], top_p=s["top_p"], seed=s["seed"],
                                                                publish_prompt_prefix=job.publish_prefix,
                                                                event_capacity=self._event_capacity,
                                                                event_send_timeout_ms=self._event_send_timeout_ms)])
                        job.request_id = rid
                        active[rid] = job
                        reply.put(None)
                    except Exception as e:
                        msg = str(e)
                        if "queue is full" in msg:
                            reply.put(ApiError.server_error("inference queue is full", 429))
                        else:
                            reply.put(ApiError.server_error(msg, 503))
                    try:
                        item = self._inbox.get_nowait()
                    except queue.Empty:
                        item = False
                if item is None:
                    break
                if not active and not draining:
                    continue
                if self._event_capacity > 0:
                    for rid, job in list(active.items()) + list(draining.items()):
                        taken = job.taken
                        if taken > job.taken_sent:
                            engine.consume(rid, taken - job.taken_sent)
                            job.taken_sent = taken
                try:
                    engine.step()
                except Exception:
                    pass  # a failure that escapes a tick poisons the engine; the requests report it below
                self._status = engine.status()
                now = time.perf_counter()
                for rid in list(active):
                    job = active[rid]
                    if job.cancelled.is_set() and not job.cancel_sent:
                        engine.cancel(rid)
                        job.cancel_sent = True
                    n, state, cached = engine.progress(rid)
                    if n > job.seen:
                        toks = engine.result(rid)["tokens"]
                        if job.t_first is None:
                            job.t_first = now
                        for i in range(job.seen, n):
                            text = self._tokenizer.decode([int(toks[i])]) if self._tokenizer is not None else ""
                            job.events.put(("token", int(toks[i]), i + 1, text))
                        job.seen = n
                    if state == "done":
                        first = job.t_first if job.t_first is not None else now
                        reason = engine.metrics(rid)["finish_reason"]     # the engine's own FinishReason, not a guess from the count
                        job.events.put(("finished", dict(generated_tokens=n, prompt_tokens=len(job.tokens), cached_prompt_tokens=int(cached),
                                                         stop_type={"length": "limit", "stop": "stop"}.get(reason, "cancelled"),
                                                         prefill_ms=(first - job.t_submit) * 1e3, ttft_ms=(first - job.t_submit) * 1e3,
                                                         total_ms=(now - job.t_submit) * 1e3)))
                        draining[rid] = active.pop(rid)
                    elif state == "failed":
                        r = engine.result(rid)
                        job.events.put(("failed", r["kind"], r["message"]))
                        draining[rid] = active.pop(rid)
                    elif state == "cancelled":   # nobody is listening any more: no event
                        draining[rid] = active.pop(rid)
                for rid in list(draining):       # the result is dropped once the engine has let go of the slot
                    try:
                        engine.release(rid)
                        del draining[rid]
                    except Exception as e:
                        if "still has events to deliver" not in str(e):
                            del draining[rid]
                if self._status not in ("poisoned",) and not active and not draining:
                    self._status = "ready"
        except Exception as e:  # a scheduler panic (src/engine.rs:1600-1647): fatal for everything in flight, the worker is gone
            self._status = "poisoned"
            for job in active.values():
                job.events.put(("failed", "fatal", f"inference worker failed: {e}"))
            active.clear()
            while not self._stop.is_set():   # keep refusing what handlers had already queued
                try:
                    item = self._inbox.get(timeout=0.05)
                except queue.Empty:
                    continue
                if item is None:
                    break
                item[1].put(ApiError.server_error("inference worker is unavailable (Poisoned)", 503))
        for job in active.values():
            job.events.put(("failed", "internal", "inference worker stopped before completing the request"))
        if self._status != "poisoned":
            self._status = "stopped"
        try:
            engine.close()
        except Exception:
            pass


def _check_terminal(settings, m):
    """validate_raw_completion_metrics (src/server.rs:808-820)."""
    if m["stop_type"] != "limit" or m["generated_tokens"] != settings["n_predict"]:
        reason = {"limit": "Length", "stop": "Stop"}.get(m["stop_type"], "Cancelled")
        return ApiError.server_error(f"raw completion ended after {m['generated_tokens']} tokens with {reason}; expected the fixed "
                                     f"{settings['n_predict']}-token limit")
    return None


def _engine_failure(kind: str, message: str) -> ApiError:
    """engine_failure_error / engine_failure_response (src/server.rs:822-841)."""
    if kind == "invalid_request":
        return ApiError.invalid_request(message, None, "invalid_request")
    return ApiError.server_error(message, 503 if kind == "resource_exhausted" else 500)
