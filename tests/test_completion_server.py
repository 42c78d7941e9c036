"""The raw `/completion` surface over the engine, on the host-only model (no GPU): the request contract, the response
projection, the streamed form and the error mapping of the reference's endpoint (src/server.rs:326-841; its own tests
`raw_completion_uses_the_untemplated_fixed_length_contract`, `raw_completion_streams_visible_text_then_exact_terminal_evidence`,
`health_and_models_report_the_single_loaded_runtime`, src/server.rs:5085-5230)."""
import http.client
import importlib
import json
import threading

import pytest


@pytest.fixture()
def srv_mod(mk):
    return importlib.import_module("macllm_infer_b200.server")


def body(srv_mod, **over):
    b = {"prompt": [5, 6, 7], "n_predict": 2, "temperature": 0.0, "top_k": 1, "top_p": 1.0, "seed": 7, "cache_prompt": True,
         "stream": False, "return_tokens": True, "id_slot": 3, "ignore_eos": True, "repeat_penalty": 1.0,
         "response_fields": list(srv_mod.RAW_COMPLETION_RESPONSE_FIELDS)}
    b.update(over)
    return b


def start(mk, srv_mod, tokenizer=None, queue_capacity=8, max_active=4, inject=None, **model_kw):
    eng = importlib.import_module("macllm_infer_b200.engine")

    def factory():
        model = eng.Model.fake(vocab=64, max_context=256, kv_capacity_tokens=2048, **model_kw)
        if inject is not None:
            model.inject_failure(*inject)
        return eng.Engine(model, max_active_sequences=max_active, scheduler_token_budget=64, prefill_token_quantum=32, queue_capacity=queue_capacity), model
    return srv_mod.CompletionServer(factory, tokenizer=tokenizer, metadata=dict(served_model="test-model", device="cpu", dtype="f32")).start()


def call(server, method, path, payload=None, raw=None):
    conn = http.client.HTTPConnection("127.0.0.1", server.port, timeout=30)
    data = raw if raw is not None else (json.dumps(payload).encode() if payload is not None else None)
    conn.request(method, path, body=data, headers={"Content-Type": "application/json"} if data is not None else {})
    r = conn.getresponse()
    out = r.read()
    conn.close()
    return r.status, r.getheader("Content-Type"), out


def test_health_and_models_report_the_single_loaded_runtime(mk, srv_mod):
    s = start(mk, srv_mod)
    try:
        st, _, b = call(s, "GET", "/healthz")
        h = json.loads(b)
        assert st == 200 and h["status"] == "ok" and h["worker"] == "ready" and h["device"] == "cpu" and h["dtype"] == "f32"
        st, _, b = call(s, "GET", "/v1/models")
        assert st == 200 and json.loads(b)["data"][0]["id"] == "test-model" and json.loads(b)["data"][0]["owned_by"] == "macllm-infer"
    finally:
        s.stop()


def test_completion_uses_the_fixed_length_contract(mk, srv_mod):
    s = start(mk, srv_mod)
    try:
        st, ctype, b = call(s, "POST", "/completion", body(srv_mod))
        assert st == 200 and ctype == "application/json"
        r = json.loads(b)
        # exactly the projected fields: no token list, no prompt echo
        assert list(r.keys()) == srv_mod.RAW_COMPLETION_RESPONSE_FIELDS
        assert r["stop"] is True and r["stop_type"] == "limit" and r["truncated"] is False and r["index"] == 0
        assert r["tokens_predicted"] == 2 and r["tokens_evaluated"] == 3
        assert r["generation_settings/ignore_eos"] is True and r["generation_settings/repeat_penalty"] == 1.0
        assert r["generation_settings/n_predict"] == 2 and r["generation_settings/max_tokens"] == 2 and r["generation_settings/n_keep"] == 0
        assert r["generation_settings/seed"] == 7 and r["generation_settings/top_k"] == 1
        assert r["timings/cache_n"] == 0 and r["timings/prompt_n"] == 3 and r["timings/predicted_n"] == 2
        assert r["timings/prompt_ms"] >= 0.0 and r["timings/predicted_ms"] >= 0.0
    finally:
        s.stop()


def test_completion_streams_token_evidence_then_the_terminal_event(mk, srv_mod):
    s = start(mk, srv_mod)
    try:
        # what the engine generates for this prompt, from the non-streamed path's sibling: run it through the engine directly
        eng = importlib.import_module("macllm_infer_b200.engine")
        model = eng.Model.fake(vocab=64, max_context=256, kv_capacity_tokens=2048)
        e = eng.Engine(model, max_active_sequences=4, scheduler_token_budget=64, prefill_token_quantum=32)
        (rid,) = e.submit([eng.Request([5, 6, 7], 3)])
        e.run()
        want = [int(t) for t in e.result(rid)["tokens"]]
        e.close()

        st, ctype, b = call(s, "POST", "/completion", body(srv_mod, stream=True, n_predict=3, cache_prompt=False))
        assert st == 200 and ctype == "text/event-stream"
        text = b.decode()
        assert "[DONE]" not in text and "keep-alive" not in text
        events = [json.loads(line[len("data: "):]) for line in text.split("\n\n") if line.startswith("data: ")]
        assert len(events) == 4
        for i, ev in enumerate(events[:3]):
            assert ev["tokens"] == [want[i]] and ev["stop"] is False and ev["id_slot"] == -1
            assert ev["tokens_predicted"] == i + 1 and ev["tokens_evaluated"] == 3 and ev["index"] == 0
        last = events[3]
        assert list(last.keys()) == srv_mod.RAW_COMPLETION_RESPONSE_FIELDS
        assert last["content"] == "" and last["stop"] is True and last["tokens_predicted"] == 3 and last["stop_type"] == "limit"
        assert last["generation_settings/stream"] is True
    finally:
        s.stop()


def test_text_prompts_need_a_tokenizer_and_content_is_decoded_text(mk, srv_mod):
    class Toy:
        def encode(self, text):
            return [ord(c) % 60 + 1 for c in text]

        def decode(self, ids):
            return "".join(chr(97 + i % 26) for i in ids)
    s = start(mk, srv_mod)
    try:
        st, _, b = call(s, "POST", "/completion", body(srv_mod, prompt="a b"))
        err = json.loads(b)["error"]
        assert st == 400 and err["param"] == "prompt" and err["type"] == "invalid_request_error"
    finally:
        s.stop()
    s = start(mk, srv_mod, tokenizer=Toy())
    try:
        st, _, b = call(s, "POST", "/completion", body(srv_mod, prompt="a b"))
        r = json.loads(b)
        assert st == 200 and r["tokens_evaluated"] == 3 and len(r["content"]) == 2 and r["content"].isalpha()
    finally:
        s.stop()


@pytest.mark.parametrize("change,param,code,message", [
    (dict(prompt=[]), "prompt", "invalid_value", "prompt must not be empty"),
    (dict(n_predict=0), "n_predict", "invalid_value", "n_predict must be in 1..=256"),
    (dict(n_predict=257), "n_predict", "invalid_value", "n_predict must be in 1..=256"),
    (dict(temperature=-0.5), "temperature", "invalid_value", "temperature must be finite and non-negative"),
    (dict(top_p=0.0), "top_p", "invalid_value", "top_p must be finite and in (0, 1]"),
    (dict(top_p=1.5), "top_p", "invalid_value", "top_p must be finite and in (0, 1]"),
    (dict(id_slot=8), "id_slot", "invalid_value", "id_slot must be in 0..8"),
    (dict(ignore_eos=False), "ignore_eos", "unsupported_value", "ignore_eos must be true for fixed-length benchmark completions"),
    (dict(return_tokens=False), "return_tokens", "unsupported_value", "return_tokens must be true for benchmark token-parity evidence"),
    (dict(repeat_penalty=1.1), "repeat_penalty", "unsupported_value", "repeat_penalty must be 1.0 for the shared benchmark contract"),
    (dict(response_fields=["content"]), "response_fields", "unsupported_value", "response_fields must exactly match the benchmark response projection"),
])
def test_requests_outside_the_contract_are_refused_with_the_reference_wording(mk, srv_mod, change, param, code, message):
    s = start(mk, srv_mod)
    try:
        st, _, b = call(s, "POST", "/completion", body(srv_mod, **change))
        err = json.loads(b)["error"]
        assert st == 400
        assert err == {"message": message, "type": "invalid_request_error", "param": param, "code": code}
    finally:
        s.stop()


def test_malformed_unknown_and_missing_fields_fail_closed(mk, srv_mod):
    s = start(mk, srv_mod)
    try:
        for raw in (b"{not json", json.dumps({**body(srv_mod), "extra": 1}).encode(),
                    json.dumps({k: v for k, v in body(srv_mod).items() if k != "seed"}).encode(),
                    json.dumps(body(srv_mod, n_predict="2")).encode(), json.dumps(body(srv_mod, stream=1)).encode()):
            st, _, b = call(s, "POST", "/completion", raw=raw)
            err = json.loads(b)["error"]
            assert st == 400 and err["code"] == "invalid_json" and err["message"].startswith("invalid /completion request: ")
        assert call(s, "POST", "/v1/chat/completions", {"model": "x"})[0] == 404
    finally:
        s.stop()


def test_concurrent_requests_share_the_batch_and_each_gets_its_own_tokens(mk, srv_mod):
    eng = importlib.import_module("macllm_infer_b200.engine")
    prompts = [[3 + i, 9, 4 + 2 * i, 11] for i in range(6)]
    model = eng.Model.fake(vocab=64, max_context=256, kv_capacity_tokens=2048)
    e = eng.Engine(model, max_active_sequences=4, scheduler_token_budget=64, prefill_token_quantum=32, queue_capacity=8)
    want = []
    for p in prompts:  # one at a time: the host-only model's tokens depend only on the sequence
        (rid,) = e.submit([eng.Request(p, 5)])
        e.run()
        want.append([int(t) for t in e.result(rid)["tokens"]])
    e.close()
    s = start(mk, srv_mod)
    got = [None] * len(prompts)

    def one(i):
        st, _, b = call(s, "POST", "/completion", body(srv_mod, prompt=prompts[i], n_predict=5, stream=True))
        evs = [json.loads(line[6:]) for line in b.decode().split("\n\n") if line.startswith("data: ")]
        got[i] = (st, [ev["tokens"][0] for ev in evs[:-1]], evs[-1])
    try:
        threads = [threading.Thread(target=one, args=(i,)) for i in range(len(prompts))]
        for t in threads:
            t.start()
        for t in threads:
            t.join(60)
        for i, (st, toks, last) in enumerate(got):
            assert st == 200 and toks == want[i] and last["tokens_predicted"] == 5 and last["tokens_evaluated"] == 4
    finally:
        s.stop()


def test_a_poisoned_worker_fails_the_request_and_turns_health_red(mk, srv_mod):
    """A forward that fails poisons the engine (src/engine.rs:1577-1647): the request in flight gets a server error, later
    submissions answer 503 `inference worker is unavailable (Poisoned)`, `/healthz` reports the worker poisoned."""
    s = start(mk, srv_mod, inject=("forward", 1))
    try:
        st, _, b = call(s, "POST", "/completion", body(srv_mod, n_predict=4))
        err = json.loads(b)["error"]
        assert st == 500 and err["type"] == "server_error" and err["code"] == "internal_error" and "inference worker failed" in err["message"]
        st, _, b = call(s, "GET", "/healthz")
        assert st == 503 and json.loads(b)["worker"] == "poisoned" and json.loads(b)["status"] == "error"
        st, _, b = call(s, "POST", "/completion", body(srv_mod))
        assert st == 503 and "unavailable (Poisoned)" in json.loads(b)["error"]["message"]
    finally:
        s.stop()


def test_cache_prompt_false_hits_the_prefix_cache_but_publishes_nothing(mk, srv_mod):
    """EngineRequestPolicy::benchmark_measured (src/engine.rs:222-241, selected by cache_prompt = false,
    src/server.rs:434-438): measured requests leave the cache as they found it."""
    prompt = list(range(3, 3 + 48))
    s = start(mk, srv_mod, prefix_capacity_tokens=1024)
    try:
        def cached(cache_prompt):
            st, _, b = call(s, "POST", "/completion", body(srv_mod, prompt=prompt, cache_prompt=cache_prompt))
            assert st == 200
            return json.loads(b)["timings/cache_n"]
        assert cached(False) == 0 and cached(False) == 0      # nothing was published by the measured requests
        assert cached(True) == 0                               # this one publishes its prompt prefix ...
        hit = cached(False)
        assert hit > 0 and hit % 16 == 0 and hit < len(prompt)  # ... which a measured request may use (whole blocks, not the last token)
        assert cached(True) == hit
    finally:
        s.stop()


def test_the_benchmark_step_through_the_endpoint_counts_every_token(mk):
    """bench.http_step on the host-only model: every request of a workload goes through POST /completion from concurrent
    clients and the step's token count is prompt + generated tokens of all of them."""
    import bench
    eng = importlib.import_module("macllm_infer_b200.engine")
    wl = bench.workloads_module()
    w = wl.Workload("http-test", "none", 10, (2, 6), 16, 64, 91, prompt=(4, 30))
    reqs = wl.make_requests(w, 64, 0, 0)
    model = eng.Model.fake(vocab=64, max_context=512, kv_capacity_tokens=4096)
    out = bench.http_step(eng, model, w, reqs, 4, 3)
    want = sum(len(p) for p in reqs[0]) + int(sum(reqs[1]))
    assert out["requests"] == 10 and out["clients"] == 3
    assert abs(out["value"] * out["wall_s"] - want) <= 0.02 * want          # wall_s is rounded to a millisecond


def test_a_worker_exception_fails_everything_in_flight_and_the_server_keeps_answering(mk, srv_mod):
    """A panic of the worker itself (src/engine.rs:1600-1647), here a tokenizer that raises while a fragment is decoded:
    the request in flight ends with a server error naming the cause, later requests get 503, `/healthz` turns red."""
    class Broken:
        def encode(self, text):
            return [1, 2, 3]

        def decode(self, ids):
            raise RuntimeError("detokeniser exploded")
    s = start(mk, srv_mod, tokenizer=Broken())
    try:
        st, _, b = call(s, "POST", "/completion", body(srv_mod, prompt="abc"))
        err = json.loads(b)["error"]
        assert st == 500 and err["type"] == "server_error" and "inference worker failed: detokeniser exploded" in err["message"]
        st, _, b = call(s, "POST", "/completion", body(srv_mod))
        assert st == 503 and "unavailable (Poisoned)" in json.loads(b)["error"]["message"]
        st, _, b = call(s, "GET", "/healthz")
        assert st == 503 and json.loads(b)["worker"] == "poisoned"
    finally:
        s.stop()


class _SlowEngine:
    """The engine with a pause in every tick, so that a client can leave while its request runs; records the cancellations."""

    def __init__(self, inner, pause_s):
        self._inner, self._pause_s, self.cancelled, self.final = inner, pause_s, [], {}

    def release(self, rid):
        self.final[rid] = self._inner.result(rid)      # what the engine held when the server let go of the request
        return self._inner.release(rid)

    def step(self):
        import time
        time.sleep(self._pause_s)
        return self._inner.step()

    def cancel(self, rid):
        self.cancelled.append(rid)
        return self._inner.cancel(rid)

    def __getattr__(self, name):
        return getattr(self._inner, name)


@pytest.mark.parametrize("stream", [True, False])
def test_a_client_that_leaves_cancels_its_request_and_the_peer_finishes(mk, srv_mod, stream):
    """Dropping the ticket sets the sticky cancellation flag (src/engine.rs:1141-1145,4397-4411; the endpoint's own case
    `dropping_a_started_sse_body_cancels_the_worker_ticket`, src/server.rs:7192-7250): the request of a client that
    closed its connection stops taking ticks, its pages return to the pool, and a peer in the same batch is served in full."""
    import socket
    import time
    eng = importlib.import_module("macllm_infer_b200.engine")
    made = {}

    def factory():
        model = eng.Model.fake(vocab=64, max_context=4096, kv_capacity_tokens=16384)
        made["model"] = model
        made["engine"] = _SlowEngine(eng.Engine(model, max_active_sequences=4, scheduler_token_budget=64, prefill_token_quantum=32,
                                                queue_capacity=8), 0.004)
        return made["engine"], model
    s = srv_mod.CompletionServer(factory, metadata=dict(served_model="test-model", device="cpu", dtype="f32")).start()
    try:
        payload = json.dumps(body(srv_mod, n_predict=2000, stream=stream)).encode()
        sock = socket.create_connection(("127.0.0.1", s.port), timeout=30)
        sock.sendall(b"POST /completion HTTP/1.1\r\nHost: x\r\nContent-Type: application/json\r\nContent-Length: " +
                     str(len(payload)).encode() + b"\r\n\r\n" + payload)
        peer = {}
        t = threading.Thread(target=lambda: peer.update(r=call(s, "POST", "/completion", body(srv_mod, prompt=[9, 8], n_predict=40))))
        t.start()
        if stream:
            got = b""
            while b"data: " not in got:              # the first fragments arrive
                chunk = sock.recv(4096)
                assert chunk, got
                got += chunk
        else:
            time.sleep(0.1)
        sock.close()
        t.join(timeout=30)
        assert peer["r"][0] == 200 and json.loads(peer["r"][2])["tokens_predicted"] == 40
        deadline = time.time() + 20
        while time.time() < deadline and made["engine"].pending() > 0:
            time.sleep(0.02)
        e = made["engine"]
        assert e.cancelled == [0]
        r = e.final[0]
        assert r["state"] == "cancelled" and 0 < len(r["tokens"]) < 2000
        with pytest.raises(RuntimeError, match="unknown request id 0"):      # delivered or given up: the engine keeps nothing
            e.result(0)
        assert e.trace() == []                                               # and no per-tick records in a server
        assert e.pending() == 0 and made["model"].pool_stats()["live_blocks"] == 0
        st, _, b = call(s, "GET", "/healthz")
        assert st == 200 and json.loads(b)["worker"] == "ready"
    finally:
        s.stop()


class _ShortEngine:
    """An engine that ends every request after one token, whatever was asked: the endpoint must notice."""

    def __init__(self, inner, eng):
        self._inner, self._eng = inner, eng

    def submit(self, requests, atomic_batch=False):
        short = [self._eng.Request(list(r.prompt), 1, ignore_stop_tokens=True) for r in requests]
        return self._inner.submit(short, atomic_batch)

    def __getattr__(self, name):
        return getattr(self._inner, name)


@pytest.mark.parametrize("stream", [False, True])
def test_completion_requires_the_exact_requested_token_boundary(mk, srv_mod, stream):
    """validate_raw_completion_metrics (src/server.rs:808-820; its test at src/server.rs:5361-5388): a generation that ends short
    of n_predict is an error of the server, never a shorter success - collected or streamed (src/server.rs:5250-5304: the
    body must not carry the terminal "stop_type":"limit")."""
    eng = importlib.import_module("macllm_infer_b200.engine")

    def factory():
        model = eng.Model.fake(vocab=64, max_context=256, kv_capacity_tokens=2048)
        return _ShortEngine(eng.Engine(model, max_active_sequences=2, scheduler_token_budget=64, prefill_token_quantum=32), eng), model
    s = srv_mod.CompletionServer(factory, metadata=dict(served_model="test-model", device="cpu", dtype="f32")).start()
    try:
        st, ctype, b = call(s, "POST", "/completion", body(srv_mod, n_predict=3, stream=stream))
        text = b.decode()
        assert "raw completion ended after 1 tokens with Length; expected the fixed 3-token limit" in text
        assert '"stop_type":"limit"' not in text
        if stream:
            assert st == 200 and ctype == "text/event-stream"
            events = [json.loads(line[6:]) for line in text.split("\n\n") if line.startswith("data: ")]
            assert events[0]["tokens"] and events[-1]["error"]["type"] == "server_error"
        else:
            assert st == 500 and json.loads(b)["error"]["type"] == "server_error"
        # the unit rule itself (src/server.rs:5361-5388)
        settings = {"n_predict": 32}
        good = dict(generated_tokens=32, stop_type="limit")
        assert srv_mod._check_terminal(settings, good) is None
        assert srv_mod._check_terminal(settings, dict(good, generated_tokens=31)) is not None
        assert srv_mod._check_terminal(settings, dict(good, stop_type="stop")) is not None
    finally:
        s.stop()


def test_a_connection_that_stops_taking_events_pauses_its_request_and_is_given_up(mk, srv_mod):
    """The request's event channel at the endpoint (EngineConfig::event_capacity / event_send_timeout, src/engine.rs:320-323,
    1408-1465): with room for two events and 0.3 s of patience, a request whose connection takes nothing stops after its
    first events while a peer is served in full, and is given up once its channel has stayed full for the timeout."""
    import time
    eng = importlib.import_module("macllm_infer_b200.engine")
    made = {}

    def factory():
        model = eng.Model.fake(vocab=64, max_context=4096, kv_capacity_tokens=16384)
        made["model"] = model
        made["engine"] = _SlowEngine(eng.Engine(model, max_active_sequences=4, scheduler_token_budget=64, prefill_token_quantum=32,
                                                queue_capacity=8), 0.002)
        return made["engine"], model
    s = srv_mod.CompletionServer(factory, metadata=dict(served_model="test-model", device="cpu", dtype="f32"),
                                 event_capacity=2, event_send_timeout_s=0.3).start()
    try:
        settings = dict(n_predict=200, temperature=0.0, top_k=1, top_p=1.0, seed=1)
        stuck = s._submit([5, 6, 7], settings)                       # a job nobody reads from
        st, _, b = call(s, "POST", "/completion", body(srv_mod, prompt=[9, 8], n_predict=60))
        assert st == 200 and json.loads(b)["tokens_predicted"] == 60       # the peer ran to its end through the same ticks
        assert 2 <= stuck.events.qsize() <= 4, "two events in the channel, at most two more waiting in the engine"
        deadline = time.time() + 10
        while time.time() < deadline and made["engine"].pending() > 0:
            time.sleep(0.02)
        e = made["engine"]
        assert e.pending() == 0
        r = e.final[stuck.request_id]
        assert r["state"] == "cancelled" and len(r["tokens"]) <= 4
        assert made["model"].pool_stats()["live_blocks"] == 0
        st, _, b = call(s, "GET", "/healthz")
        assert st == 200 and json.loads(b)["worker"] == "ready"
    finally:
        s.stop()
