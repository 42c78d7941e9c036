"""Scheduler-tick parity on the host-only fake model: the schedules the reference's own tests assert
(src/engine.rs:4701-5014) and a randomised differential of traces, tokens, block tables, prefix-cache
counters and pool stats between the product's C++ engine and the oracle's Python restatement."""
import importlib
import random

import pytest


@pytest.fixture(scope="module")
def eng(mk):
    return importlib.import_module("macllm_infer_b200.engine")


def product_engine(eng, model_kw, engine_kw):
    model = eng.Model.fake(**model_kw)
    return model, eng.Engine(model, **engine_kw)


def oracle_engine(model_kw, engine_kw):
    from oracle import engine as oe
    m = oe.OracleModel(model_kw.get("vocab", 32), model_kw.get("max_context", 4096), model_kw.get("block_tokens", 16),
                       model_kw.get("slab_blocks", 8), model_kw.get("kv_capacity_tokens", 4096),
                       model_kw.get("prefix_capacity_tokens", 0))
    return m, oe.OracleEngine(m, **engine_kw)


def both(eng, model_kw, engine_kw):
    return product_engine(eng, model_kw, engine_kw), oracle_engine(model_kw, engine_kw)


def submit_both(eng, pe, oe_, prompts, max_new, atomic=False):
    from oracle import engine as oe
    ids_p = pe.submit([eng.Request(p, n) for p, n in zip(prompts, max_new)], atomic)
    ids_o = oe_.submit([oe.Req(list(p), n) for p, n in zip(prompts, max_new)], atomic)
    assert ids_p == ids_o
    return ids_p


def assert_tick_kinds_agree(pe, oe_):
    """Whole-forward kinds, lane phases, lane counts and input tokens of every tick; the device-time buckets add up."""
    assert len(oe_.tick_kinds) == len(pe.trace())
    for tick, want in enumerate(oe_.tick_kinds):
        got = pe.tick_info(tick)
        assert {k: got[k] for k in ("kind", "phases", "lane_count", "input_tokens")} == want, tick
    st = pe.stats()
    assert abs(st["suffix_prefill_ms"] + st["first_token_ms"] + st["decode_ms"] + st["mixed_ms"] - st["device_ms"]) < 1e-6


def test_ragged_prefill_and_decode_schedule(eng):
    """engine.rs:4701-4765: budget 4, quantum 2, two active; a 6-token prompt with 1 new token and a
    1-token prompt with 2 new tokens."""
    (pm, pe), (om, oe_) = both(eng, dict(vocab=32), dict(max_active_sequences=2, scheduler_token_budget=4, prefill_token_quantum=2))
    submit_both(eng, pe, oe_, [[1, 2, 3, 4, 1, 2], [2]], [1, 2])
    for e in (pe, oe_):
        for _ in range(3):
            e.step()
    want = [[(0, 0, 2), (1, 0, 1)], [(0, 2, 2), (1, 1, 1)], [(0, 4, 2)]]
    assert pe.trace() == want
    assert [[tuple(l) for l in t] for t in oe_.trace] == want
    assert pe.pending() == 0 and oe_.pending() == 0
    assert len(pe.result(0)["tokens"]) == 1 and len(pe.result(1)["tokens"]) == 2
    assert list(pe.result(1)["tokens"]) == oe_.results[1].tokens


def test_budget_smaller_than_active_count_keeps_the_round_robin_cursor(eng):
    """engine.rs:4968-5014: three 4-token prompts, budget 2, quantum 1 -> lanes [a,b], [c,a], [b,c]."""
    (pm, pe), (om, oe_) = both(eng, dict(vocab=32), dict(max_active_sequences=3, scheduler_token_budget=2, prefill_token_quantum=1))
    submit_both(eng, pe, oe_, [[1] * 4, [2] * 4, [4] * 4], [1, 1, 1])
    for e in (pe, oe_):
        for _ in range(3):
            e.step()
    assert [[l[0] for l in t] for t in pe.trace()] == [[0, 1], [2, 0], [1, 2]]
    assert [[l[0] for l in t] for t in oe_.trace] == [[0, 1], [2, 0], [1, 2]]


def test_kv_pressure_shrinks_the_batch_from_the_back(eng):
    """engine.rs:4845-4895: three one-token requests, room for two blocks."""
    mkw = dict(vocab=32, block_tokens=16, slab_blocks=2, kv_capacity_tokens=32)
    (pm, pe), (om, oe_) = both(eng, mkw, dict(max_active_sequences=3, scheduler_token_budget=3, prefill_token_quantum=1))
    submit_both(eng, pe, oe_, [[1], [2], [3]], [1, 1, 1])
    for e in (pe, oe_):
        e.step()
    assert [len(t) for t in pe.trace()] == [2] and pe.pending() == 1
    assert pe.stats()["kv_shrinks"] == 1 and oe_.kv_shrinks == 1
    for e in (pe, oe_):
        e.step()
    assert [[l[0] for l in t] for t in pe.trace()] == [[0, 1], [2]]
    assert all(pe.result(i)["state"] == "done" for i in range(3))


def test_irreducible_kv_pressure_fails_only_that_request(eng):
    """engine.rs:4898-4966: a lane that can never be served fails alone; its peers continue."""
    mkw = dict(vocab=32, block_tokens=2, slab_blocks=2, kv_capacity_tokens=4)
    (pm, pe), (om, oe_) = both(eng, mkw, dict(max_active_sequences=2, scheduler_token_budget=8, prefill_token_quantum=4))
    # each request fits the pool on its own (4 cached tokens), but after the first tick each holds one of the
    # two blocks and the first lane's decode needs a third: not even a one-lane batch can be reserved
    submit_both(eng, pe, oe_, [[1, 2], [4, 5]], [3, 3])
    for e in (pe, oe_):
        e.run()
    states = [pe.result(i)["state"] for i in range(2)]
    assert states == [oe_.results[i].state for i in range(2)]
    assert states == ["failed", "done"]
    # KvCacheExhausted as the model boundary words it (src/architecture.rs:928-953, src/decoder.rs:3970-3994)
    assert pe.result(0)["message"] == oe_.results[0].message == "KV cache requires 1 additional blocks, but only 0 of 2 are free (0 retired, 2 tokens/block)"
    assert pe.result(0)["kind"] == "resource_exhausted"
    assert len(pe.result(1)["tokens"]) == 3
    assert pm.pool_stats()["live_blocks"] == 0


def test_atomic_batch_waits_until_every_member_fits(eng):
    """engine.rs:1886-1936."""
    (pm, pe), (om, oe_) = both(eng, dict(vocab=32), dict(max_active_sequences=3, scheduler_token_budget=16, prefill_token_quantum=8,
                                                        queue_capacity=8))
    submit_both(eng, pe, oe_, [[1, 2, 3]], [6])
    for e in (pe, oe_):
        e.step()
    submit_both(eng, pe, oe_, [[4], [5], [6]], [2, 2, 2], atomic=True)
    for e in (pe, oe_):
        e.run()
    tr = pe.trace()
    assert tr == [[tuple(l) for l in t] for t in oe_.trace]
    # no member of the batch runs before request 0 has left and all three fit
    first_batch_tick = next(i for i, t in enumerate(tr) if any(l[0] in (1, 2, 3) for l in t))
    assert sorted(l[0] for l in tr[first_batch_tick]) == [1, 2, 3]
    assert all(all(l[0] == 0 for l in t) for t in tr[:first_batch_tick])


def test_requests_that_can_never_fit_are_rejected_at_admission(eng):
    """kv_capacity_rejection, engine.rs:2839-2863, and validate_request, generation.rs:1308-1337."""
    model, e = product_engine(eng, dict(vocab=32, max_context=64, block_tokens=16, kv_capacity_tokens=32),
                              dict(max_active_sequences=2, queue_capacity=8))
    ids = e.submit([eng.Request(list(range(1, 30)), 8), eng.Request([1, 2], 100), eng.Request([40], 1), eng.Request([], 1),
                    eng.Request([3], 2)])
    e.run()
    assert [e.result(i)["state"] for i in ids] == ["failed", "failed", "failed", "failed", "done"]
    # the reference's wording and kind (reject_preflight with ResourceExhausted, engine.rs:1694-1701,2856-2861)
    assert e.result(ids[0])["message"] == "request requires up to 36 cached tokens, exceeding the configured shared KV capacity of 2 blocks \u00d7 16 tokens"
    assert e.result(ids[0])["kind"] == "resource_exhausted" and e.result(ids[1])["kind"] == "invalid_request"
    assert "maximum context length is 64 tokens" in e.result(ids[1])["message"]


def test_forward_failure_rolls_back_every_lane(eng):
    """decoder.rs:4146-4162 / cache.rs:3001-3005, the case failed_mixed_batch_rolls_back_every_lane_and_retries
    (decoder.rs:9325-9388): a failed forward leaves sessions and pool untouched, and the same batch then runs."""
    capi = importlib.import_module("macllm_infer_b200._capi")
    model = eng.Model.fake(vocab=32, fail_forward_at=1)
    a, b = model.new_session(), model.new_session()
    model.forward_batch([(a, [1, 2, 3], 0), (b, [4], 0)])
    before = model.pool_stats()
    with pytest.raises(capi.MkError, match="injected"):
        model.forward_batch([(a, [5], 3), (b, [6, 7], 1)])
    after = model.pool_stats()
    assert len(a) == 3 and len(b) == 1
    assert after["live_blocks"] == before["live_blocks"] and after["reserved_blocks"] == 0
    logits, toks = model.forward_batch([(a, [5], 3), (b, [6, 7], 1)])
    assert list(toks) == [(31 * 5 + 7 * 3 + 3) % 32, (31 * 7 + 7 * 2 + 3) % 32]


def test_lane_validation_happens_before_any_mutation(eng):
    """mixed_batch_prevalidation_is_atomic_across_lanes (decoder.rs:9266-9323): a bad second lane - wrong start, a token
    outside the vocabulary, the first lane's session again - is found before the first lane is touched."""
    capi = importlib.import_module("macllm_infer_b200._capi")
    model = eng.Model.fake(vocab=32)
    a, b = model.new_session(), model.new_session()
    with pytest.raises(capi.MkError, match="start_pos"):
        model.forward_batch([(a, [1], 0), (b, [2], 5)])
    with pytest.raises(capi.MkError):
        model.forward_batch([(a, [1], 0), (b, [99], 0)])     # token outside the vocabulary
    with pytest.raises(capi.MkError, match="duplicates"):
        model.forward_batch([(a, [1], 0), (a, [2], 0)])
    assert len(a) == 0 and len(b) == 0 and model.pool_stats()["live_blocks"] == 0


@pytest.mark.parametrize("seed", range(6))
def test_randomised_differential_with_prefix_cache(eng, seed):
    """Shared-prefix workloads under KV pressure: schedules, tokens, cached-token counts, block tables
    (through pool stats) and prefix-cache counters agree tick by tick."""
    rng = random.Random(seed)
    bt = rng.choice([4, 16])
    mkw = dict(vocab=64, max_context=2048, block_tokens=bt, slab_blocks=rng.choice([2, 8]),
               kv_capacity_tokens=rng.choice([40 * bt, 200 * bt]), prefix_capacity_tokens=rng.choice([0, 12 * bt, 64 * bt]))
    ekw = dict(max_active_sequences=rng.choice([2, 4, 7]), scheduler_token_budget=rng.choice([8, 48, 256]),
               prefill_token_quantum=rng.choice([3, 16, 64]), queue_capacity=64)
    (pm, pe), (om, oe_) = both(eng, mkw, ekw)
    stems = [[rng.randrange(3, 64) for _ in range(rng.randint(bt, 6 * bt))] for _ in range(3)]
    submitted = 0
    for wave in range(4):
        prompts, max_new = [], []
        for _ in range(rng.randint(1, 6)):
            stem = rng.choice(stems)
            prompts.append(stem[: rng.randint(1, len(stem))] + [rng.randrange(3, 64) for _ in range(rng.randint(1, 2 * bt))])
            max_new.append(rng.randint(1, 12))
        submit_both(eng, pe, oe_, prompts, max_new, atomic=rng.random() < 0.3 and len(prompts) <= ekw["max_active_sequences"])
        submitted += len(prompts)
        for _ in range(rng.randint(1, 30)):
            lp, lo = pe.step(), oe_.step()
            assert lp == lo
            assert pm.pool_stats() == om.pool.stats()
            if mkw["prefix_capacity_tokens"]:
                assert pm.prefix_diagnostics() == om.prefix.stats()
    pe.run()
    oe_.run()
    assert pe.trace() == [[tuple(l) for l in t] for t in oe_.trace]
    assert_tick_kinds_agree(pe, oe_)
    for rid in range(submitted):
        rp, ro = pe.result(rid), oe_.results[rid]
        assert rp["state"] == ro.state
        assert list(rp["tokens"]) == ro.tokens
        assert rp["cached_tokens"] == ro.cached_tokens
    assert pm.pool_stats() == om.pool.stats()
    if mkw["prefix_capacity_tokens"]:
        assert pm.prefix_diagnostics() == om.prefix.stats()
        assert pm.prefix_diagnostics()["hits"] + pm.prefix_diagnostics()["misses"] > 0


# ---- worker poisoning (src/engine.rs:1577-1647,2719-2770; tests at src/engine.rs:5603-5760) ----------------------

def test_forward_failure_poisons_the_engine_and_fans_out_fatal(eng):
    """scheduler_panic_is_caught_and_fanned_out_as_fatal (src/engine.rs:5603-5637) and
    fatal_model_error_poisons_active_and_queued_requests (src/engine.rs:5799-5858): the tick that fails had both
    requests packed; both, and the one still queued, end Fatal; one cleanup drain, no completion barrier; the sessions
    are gone and later submissions are refused."""
    capi = importlib.import_module("macllm_infer_b200._capi")
    model = eng.Model.fake(vocab=32, fail_forward_at=1)
    e = eng.Engine(model, max_active_sequences=2, scheduler_token_budget=8, prefill_token_quantum=2, queue_capacity=8)
    ids = e.submit([eng.Request([1, 2, 3], 4), eng.Request([4, 5], 4), eng.Request([6], 2)])
    assert e.step() == 2            # tick 0 runs
    assert e.status() == "busy"
    assert e.step() == 0            # tick 1: the injected failure escapes the tick
    assert e.status() == "poisoned"
    for i in ids:
        r = e.result(i)
        assert r["state"] == "failed" and r["kind"] == "fatal"
        assert r["message"].startswith("inference worker failed: ") and "injected forward failure" in r["message"]
    assert e.pending() == 0
    assert e.stats()["cleanup_drains"] == 1 and e.stats()["failed_requests"] == 3
    assert len(e.trace()) == 1      # the failed tick never completed
    assert e.step() == 0            # a poisoned engine does nothing more
    with pytest.raises(capi.MkError, match=r"inference worker is unavailable \(Poisoned\)"):
        e.submit([eng.Request([1], 1)])
    # the model rolled the failed tick back (src/decoder.rs:4146-4162): nothing is reserved, the sessions' pages
    # were released with the sessions
    st = model.pool_stats()
    assert st["reserved_blocks"] == 0 and st["live_blocks"] == 0


def test_completion_barrier_failure_poisons_without_a_second_drain(eng):
    """shared_completion_failure_poison_is_atomic_and_not_retried (src/engine.rs:5687-5760): once the read-back has
    been entered a failure poisons the engine and no cleanup drain follows."""
    model = eng.Model.fake(vocab=32)
    model.inject_failure("read_output", 0)
    e = eng.Engine(model, max_active_sequences=2, scheduler_token_budget=8, prefill_token_quantum=4, queue_capacity=8)
    ids = e.submit([eng.Request([1], 1), eng.Request([2], 1), eng.Request([1, 2], 1)])
    e.run()
    assert e.status() == "poisoned"
    assert [e.result(i)["kind"] for i in ids] == ["fatal"] * 3
    assert "injected completion barrier failure" in e.result(ids[2])["message"]
    assert e.stats()["cleanup_drains"] == 0


def test_cleanup_drain_failure_is_appended_to_the_fatal_message(eng):
    """src/engine.rs:2723-2736."""
    model = eng.Model.fake(vocab=32, fail_forward_at=0)
    model.inject_failure("synchronize", 0)
    e = eng.Engine(model, max_active_sequences=2, queue_capacity=4)
    (i,) = e.submit([eng.Request([1, 2], 2)])
    e.run()
    msg = e.result(i)["message"]
    assert "injected forward failure" in msg and "forward-error cleanup synchronization also failed" in msg


def test_admission_failure_poisons_and_loses_no_session(eng):
    """An error during request admission poisons the worker too (src/engine.rs:1607-1621); with the engine alive
    the slot's session goes back to the reusable list before the error travels on."""
    model = eng.Model.fake(vocab=32)
    model.inject_failure("admission", 1)
    e = eng.Engine(model, max_active_sequences=2, queue_capacity=4)
    ids = e.submit([eng.Request([1], 1), eng.Request([2], 1)])
    e.run()
    assert e.status() == "poisoned"
    assert [e.result(i)["kind"] for i in ids] == ["fatal", "fatal"]
    assert "injected admission failure" in e.result(ids[0])["message"]


def test_kv_exhaustion_fails_one_request_with_resource_exhausted_not_fatal(eng):
    """fail_kv_exhausted_visit (src/engine.rs:2205-2231): request-local, the engine stays healthy."""
    model = eng.Model.fake(vocab=32, kv_capacity_tokens=64, block_tokens=16)
    e = eng.Engine(model, max_active_sequences=2, scheduler_token_budget=64, prefill_token_quantum=64, queue_capacity=4)
    ids = e.submit([eng.Request(list(range(1, 31)) * 2, 2), eng.Request(list(range(1, 31)), 8)])
    e.run()
    kinds = sorted(e.result(i)["kind"] for i in ids)
    assert e.status() == "ready"
    assert "fatal" not in kinds


def test_second_forward_before_the_read_is_refused(eng):
    """One tick in flight: the staging and result buffers of a tick are reused by the next one."""
    import ctypes as C
    capi = importlib.import_module("macllm_infer_b200._capi")
    model = eng.Model.fake(vocab=32)
    a, b = model.new_session(), model.new_session()
    def enqueue(lanes):
        arr, keep = model._lanes(lanes)
        r = C.c_void_p()
        capi.check(capi.lib().mk_reserve_batch(model._h, arr, len(lanes), C.byref(r)))
        st = capi.lib().mk_forward_batch_reserved(model._h, arr, len(lanes), r, capi.FWD_WANT_TOKENS)
        return st, keep
    st, _ = enqueue([(a, [1, 2], 0)])
    assert st == 0
    st, _ = enqueue([(b, [3], 0)])
    assert st != 0 and "previous forward was not read" in capi.lib().mk_last_error().decode()
    assert len(b) == 0 and len(a) == 2      # the refused forward changed nothing
    toks = (C.c_uint32 * 1)()
    capi.check(capi.lib().mk_read_output(model._h, None, toks))
    assert toks[0] == (31 * 2 + 7 * 1 + 3) % 32
    st, _ = enqueue([(b, [3], 0)])          # after the read the next tick goes through
    assert st == 0
    model.synchronize()
    assert capi.lib().mk_read_output(model._h, None, toks) != 0   # nothing left to read


def test_scheduler_limits_must_be_positive_and_internally_consistent(eng):
    """engine.rs:4376-4395 with EngineConfig::validate's wording (engine.rs:350-367)."""
    from oracle import engine as oe
    capi = importlib.import_module("macllm_infer_b200._capi")
    cases = [(dict(max_active_sequences=0), "maximum active sequences must be positive"),
             (dict(scheduler_token_budget=0), "scheduler token budget must be positive"),
             (dict(prefill_token_quantum=0), "prefill token quantum must be positive"),
             (dict(queue_capacity=0), "queue capacity must be positive"),
             (dict(scheduler_token_budget=4, prefill_token_quantum=5), "prefill token quantum cannot exceed the scheduler token budget")]
    model = eng.Model.fake(vocab=8)
    om = oe.OracleModel(8, 4096, 16, 8, 4096, 0)
    eng.Engine(model).close()                      # the defaults are valid
    oe.OracleEngine(om)
    for kw, message in cases:
        with pytest.raises(capi.MkError, match=message):
            eng.Engine(model, **kw)
        with pytest.raises(ValueError, match=message):
            oe.OracleEngine(om, **kw)


def test_token_prompts_are_validated_with_the_reference_wording(eng):
    """engine.rs:4341-4364 (empty and out-of-vocabulary token prompts) and engine.rs:4315-4338 (context overflow leads
    with the phrase clients recognise): each fails only its own request, as an invalid request, before any model work."""
    (pm, pe), (om, oe_) = both(eng, dict(vocab=6, max_context=32, kv_capacity_tokens=256),
                               dict(max_active_sequences=2, scheduler_token_budget=8, prefill_token_quantum=4))
    prompts = [[], [1, 6], [1, 2, 3], [1] * 30, [1] * 29, [2, 3]]
    max_new = [4, 4, 33, 4, 4, 2]
    ids = submit_both(eng, pe, oe_, prompts, max_new)
    pe.run()
    oe_.run()
    want = {0: "raw token prompt must not be empty",
            1: "raw prompt token 6 at index 1 exceeds model vocabulary 6",
            2: "This model's maximum context length is 32 tokens; the prompt (3 tokens) plus requested output (33 tokens) exceeds it",
            3: "This model's maximum context length is 32 tokens; the prompt (30 tokens) plus requested output (4 tokens) exceeds it"}
    for rid in ids:
        rp, ro = pe.result(rid), oe_.results[rid]
        if rid in want:
            assert rp["state"] == ro.state == "failed" and rp["kind"] == "invalid_request"
            assert rp["message"] == ro.message == want[rid]
        else:   # 29 + 4 - 1 = 32 tokens of context is exactly the limit
            assert rp["state"] == ro.state == "done" and list(rp["tokens"]) == ro.tokens
    assert all(lane[0] in (4, 5) for tick in pe.trace() for lane in tick)     # the refused requests never reached the model
    assert pe.trace() == [[tuple(l) for l in t] for t in oe_.trace]


def test_scheduler_fills_available_slots_before_the_first_iteration(eng):
    """engine.rs:4811-4842: three queued one-token requests, three slots, budget 3, quantum 1 - the first tick already packs
    all three in submission order, with one completion barrier and no cleanup drain."""
    (pm, pe), (om, oe_) = both(eng, dict(vocab=32), dict(max_active_sequences=3, scheduler_token_budget=3, prefill_token_quantum=1,
                                                          queue_capacity=3))
    submit_both(eng, pe, oe_, [[1], [2], [3]], [1, 1, 1])
    assert pe.step() == 3
    oe_.step()
    assert pe.trace() == [[(0, 0, 1), (1, 0, 1), (2, 0, 1)]] == [[tuple(l) for l in t] for t in oe_.trace]
    s = pe.stats()
    assert s["ticks"] == 1 and s["cleanup_drains"] == 0 and s["completed_requests"] == 3


def test_invalid_sampling_parameters_fail_the_request_with_the_reference_wording(eng):
    """rejects_invalid_sampling_parameters (src/sampling.rs:812-829) as the engine reports it (engine.rs:3022-3032):
    Sampler::new's three checks, then set_penalties' two, each failing only its own request."""
    from oracle import engine as oe
    (pm, pe), (om, oe_) = both(eng, dict(vocab=16), dict(max_active_sequences=2, scheduler_token_budget=8, prefill_token_quantum=4, queue_capacity=16))
    cases = [(dict(temperature=-1.0), "temperature must be finite and non-negative"),
             (dict(temperature=float("nan")), "temperature must be finite and non-negative"),
             (dict(repetition_penalty=0.0), "repetition_penalty must be finite and positive"),
             (dict(presence_penalty=2.5), "invalid presence_penalty"),
             (dict(frequency_penalty=-3.0), "invalid frequency_penalty"),
             (dict(presence_penalty=2.0, frequency_penalty=-2.0), None)]
    ids_p = pe.submit([eng.Request([1, 2], 2, **kw) for kw, _ in cases])
    ids_o = oe_.submit([oe.Req([1, 2], 2, **kw) for kw, _ in cases])
    assert ids_p == ids_o
    pe.run()
    oe_.run()
    for rid, (_, why) in zip(ids_p, cases):
        rp, ro = pe.result(rid), oe_.results[rid]
        if why is None:
            assert rp["state"] == ro.state == "done"
        else:
            assert rp["state"] == ro.state == "failed" and rp["kind"] == "invalid_request"
            assert rp["message"] == ro.message == "invalid sampling parameters: " + why
    # top_p lives on the product's request only (the oracle's engine has no stochastic sampler of its own)
    (rid,) = pe.submit([eng.Request([1, 2], 2, top_p=0.0)])
    pe.run()
    assert pe.result(rid)["message"] == "invalid sampling parameters: top_p must be finite and in (0, 1]"


# ---- cancellation (EngineTicket::cancel, src/engine.rs:1136-1145; tests at src/engine.rs:4931-4966,5016-5131,5284-5346) --------

def cancel_both(pe, oe_, rid):
    pe.cancel(rid)
    oe_.cancel(rid)


def test_cancelled_queued_request_is_skipped_before_preflight_and_model_work(eng):
    """engine.rs:5016-5058: one active slot, budget 1, quantum 1; "a a a a", "b b" and "y" queue up. After the first tick
    the queued second request and the running first are cancelled: the first leaves without another forward, the second
    never gets validated, a session or a forward, and the third runs once the slot is free."""
    (pm, pe), (om, oe_) = both(eng, dict(vocab=32), dict(max_active_sequences=1, scheduler_token_budget=1, prefill_token_quantum=1))
    submit_both(eng, pe, oe_, [[1, 1, 1, 1], [2, 2], [4]], [1, 1, 1])
    for e in (pe, oe_):
        assert e.step() == 1
    cancel_both(pe, oe_, 1)
    cancel_both(pe, oe_, 0)
    for e in (pe, oe_):
        assert e.step() == 0          # the first request leaves; nothing is forwarded
    assert pm.pool_stats()["live_blocks"] == 0 and om.pool.stats()["live_blocks"] == 0
    for e in (pe, oe_):
        e.step()                      # the cancelled queued request is popped and skipped; the third is admitted
        e.run()
    trace = pe.trace()
    assert trace == [[tuple(l) for l in t] for t in oe_.trace]
    assert not any(l[0] == 1 for t in trace for l in t)
    assert any(l[0] == 2 for t in trace for l in t)
    assert [pe.result(i)["state"] for i in range(3)] == ["cancelled", "cancelled", "done"]
    assert [oe_.results[i].state for i in range(3)] == ["cancelled", "cancelled", "done"]
    assert pe.result(1)["message"] == "" and pe.result(1)["kind"] == "none"    # no preflight answer of any kind
    assert pe.stats()["cancelled_requests"] == 2 and pe.stats()["failed_requests"] == 0


def test_a_cancelled_request_is_not_validated(eng):
    """engine.rs:1671-1674 comes before prepare_request: a cancelled request with an invalid prompt is skipped, not refused."""
    pm, pe = product_engine(eng, dict(vocab=32), dict(max_active_sequences=1, scheduler_token_budget=4, prefill_token_quantum=4))
    ids = pe.submit([eng.Request([1, 2], 4), eng.Request([99], 1)])
    pe.cancel(ids[1])
    pe.run()
    assert pe.result(ids[1])["state"] == "cancelled"
    assert pe.result(ids[0])["state"] == "done"
    with pytest.raises(RuntimeError, match="unknown request id"):
        pe.cancel(7)


def test_active_limit_delays_admission_until_a_cancelled_slot_is_reclaimed(eng):
    """engine.rs:5059-5131: two active slots, three requests. The third waits; cancelling the first frees its session (cleared
    once), the third is admitted on the next tick and reuses that slot."""
    ekw = dict(max_active_sequences=2, scheduler_token_budget=4, prefill_token_quantum=2)
    (pm, pe), (om, oe_) = both(eng, dict(vocab=32), ekw)
    submit_both(eng, pe, oe_, [[1, 1, 1, 1], [2, 2, 2, 2], [4, 2]], [3, 3, 1])
    for e in (pe, oe_):
        e.step()
        e.step()
    assert pe.pending() == 3 and not any(l[0] == 2 for t in pe.trace() for l in t)
    cancel_both(pe, oe_, 0)
    for e in (pe, oe_):
        e.step()
    # the tick that sees the cancellation forwards only the peer and returns the pages before that forward
    assert [l[0] for l in pe.trace()[-1]] == [1]
    assert pe.result(0)["state"] == "cancelled" and oe_.results[0].state == "cancelled"
    assert pm.pool_stats() == om.pool.stats()
    for e in (pe, oe_):
        e.run()
    assert pe.trace() == [[tuple(l) for l in t] for t in oe_.trace]
    assert pe.result(2)["state"] == "done" and list(pe.result(2)["tokens"]) == oe_.results[2].tokens
    assert pe.result(1)["state"] == "done" and len(pe.result(1)["tokens"]) == 3


def test_cancellation_after_the_shared_completion_barrier_drops_only_its_lane(eng):
    """engine.rs:4931-4966: two one-token requests share a forward; the first is cancelled while the forward runs (the fake
    model flips the flag inside the completion barrier). Both lanes were in the packed forward, the cancelled one gets no
    token, the peer gets its own row's token, both sessions are back, one barrier, no cleanup drain."""
    (pm, pe), (om, oe_) = both(eng, dict(vocab=32), dict(max_active_sequences=2, scheduler_token_budget=8, prefill_token_quantum=4))
    submit_both(eng, pe, oe_, [[1], [2]], [1, 1])
    pm.on_next_barrier(lambda: pe.cancel(0))
    oe_.on_barrier = lambda: oe_.cancel(0)
    for e in (pe, oe_):
        assert e.step() == 2
    assert pe.trace() == [[(0, 0, 1), (1, 0, 1)]] == [[tuple(l) for l in t] for t in oe_.trace]
    assert pe.result(0)["state"] == "cancelled" and len(pe.result(0)["tokens"]) == 0
    assert oe_.results[0].state == "cancelled" and oe_.results[0].tokens == []
    assert pe.result(1)["state"] == "done" and list(pe.result(1)["tokens"]) == oe_.results[1].tokens
    assert list(pe.result(1)["tokens"]) == [(31 * 2 + 3) % 32]      # row 1 of the forward, not row 0
    assert pe.pending() == 0 and oe_.pending() == 0
    assert pe.stats()["cleanup_drains"] == 0 and pe.stats()["ticks"] == 1
    assert pm.pool_stats()["live_blocks"] == 0


def test_cancelled_prefix_slot_is_removed_before_the_peers_rows_are_mapped(eng):
    """engine.rs:5284-5346: three active one-token prompts, the first cancelled before the tick: the packed forward holds the
    two peers at rows 0 and 1 with their own tokens, and the cancelled slot's pages were returned before that forward."""
    mkw = dict(vocab=32, block_tokens=16, slab_blocks=2, kv_capacity_tokens=32)   # two blocks: three lanes would not fit
    ekw = dict(max_active_sequences=3, scheduler_token_budget=3, prefill_token_quantum=1)
    (pm, pe), (om, oe_) = both(eng, mkw, ekw)
    submit_both(eng, pe, oe_, [[1, 1], [2], [3]], [2, 1, 1])
    # one tick with a budget that reaches only the first slot would not do here; cancel before anything ran
    cancel_both(pe, oe_, 0)
    for e in (pe, oe_):
        assert e.step() == 2
    assert pe.trace() == [[(1, 0, 1), (2, 0, 1)]] == [[tuple(l) for l in t] for t in oe_.trace]
    assert pe.stats()["kv_shrinks"] == 0 and oe_.kv_shrinks == 0
    assert list(pe.result(1)["tokens"]) == [(31 * 2 + 3) % 32] and list(pe.result(2)["tokens"]) == [(31 * 3 + 3) % 32]
    assert pe.result(0)["state"] == "cancelled"
    assert pe.stats()["cleanup_drains"] == 0


def test_cancellation_between_quanta_skips_the_next_decode(eng):
    """generation.rs:2476-2516: a sequence cancelled after its first token never runs the next decode; the tokens it had stay
    readable. generation.rs:2289-2311: one cancelled before its first prefill chunk never reaches the model."""
    (pm, pe), (om, oe_) = both(eng, dict(vocab=32), dict(max_active_sequences=2, scheduler_token_budget=8, prefill_token_quantum=4))
    submit_both(eng, pe, oe_, [[1, 2]], [4])
    for e in (pe, oe_):
        e.step()
    assert len(pe.result(0)["tokens"]) == 1
    cancel_both(pe, oe_, 0)
    for e in (pe, oe_):
        assert e.step() == 0
        assert e.pending() == 0
    assert pe.stats()["ticks"] == 1 and pe.stats()["decode_tokens"] == 0
    assert pe.result(0)["state"] == "cancelled" and list(pe.result(0)["tokens"]) == oe_.results[0].tokens
    submit_both(eng, pe, oe_, [[3, 4, 5]], [2])
    cancel_both(pe, oe_, 1)
    for e in (pe, oe_):
        assert e.step() == 0
    assert pe.stats()["ticks"] == 1 and pe.stats()["prefill_tokens"] == 2


def test_cancelling_a_finished_request_changes_nothing(eng):
    pm, pe = product_engine(eng, dict(vocab=32), dict(max_active_sequences=1, scheduler_token_budget=4, prefill_token_quantum=4))
    rid = pe.submit([eng.Request([1, 2], 2)])[0]
    pe.run()
    before = pe.result(rid)
    pe.cancel(rid)
    pe.step()
    after = pe.result(rid)
    assert after["state"] == "done" and list(after["tokens"]) == list(before["tokens"])
    assert pe.stats()["cancelled_requests"] == 0


def test_a_cancelled_member_does_not_hold_back_its_atomic_batch(eng):
    """engine.rs:1886-1936 with 1671-1674: the batch is admitted as a whole; the cancelled member is skipped at its own admission."""
    (pm, pe), (om, oe_) = both(eng, dict(vocab=32), dict(max_active_sequences=3, scheduler_token_budget=8, prefill_token_quantum=4))
    submit_both(eng, pe, oe_, [[1], [2], [3]], [2, 2, 2], atomic=True)
    cancel_both(pe, oe_, 1)
    for e in (pe, oe_):
        e.run()
    assert pe.trace() == [[tuple(l) for l in t] for t in oe_.trace]
    assert [pe.result(i)["state"] for i in range(3)] == ["done", "cancelled", "done"]
    assert [l[0] for l in pe.trace()[0]] == [0, 2]


def test_a_failed_session_clearing_keeps_every_slot_for_the_fatal_fan_out(eng):
    """engine.rs:5640-5682: the first of two active requests is cancelled and the clearing of its session fails: nothing was
    forwarded, no barrier and no drain ran, and the fatal message reaches the cancelled request as well as its peer."""
    pm, pe = product_engine(eng, dict(vocab=32), dict(max_active_sequences=2, scheduler_token_budget=8, prefill_token_quantum=4))
    pe.submit([eng.Request([1] * 8, 1), eng.Request([2] * 8, 1)])
    assert pe.step() == 2                     # both are active, half of each prompt is in
    pe.cancel(0)
    pm.inject_failure("clear_session", 0)     # the next clearing is the cancelled slot's
    assert pe.step() == 0
    assert pe.status() == "poisoned"
    assert len(pe.trace()) == 1 and pe.stats()["ticks"] == 1 and pe.stats()["cleanup_drains"] == 0
    for rid in (0, 1):
        r = pe.result(rid)
        assert r["state"] == "failed" and r["kind"] == "fatal"
        assert r["message"] == "inference worker failed: injected session clearing failure"
    with pytest.raises(RuntimeError, match=r"inference worker is unavailable \(Poisoned\)"):
        pe.submit([eng.Request([1], 1)])


@pytest.mark.parametrize("seed", range(8))
def test_randomised_differential_with_cancellations(eng, seed):
    """Requests are given up at random moments - queued, in the middle of their prefill, between decodes, after they ended:
    schedules, tokens, states, pool statistics and prefix-cache counters agree with the oracle tick by tick."""
    rng = random.Random(1000 + seed)
    bt = rng.choice([4, 16])
    mkw = dict(vocab=64, max_context=2048, block_tokens=bt, slab_blocks=rng.choice([2, 8]),
               kv_capacity_tokens=rng.choice([40 * bt, 200 * bt]), prefix_capacity_tokens=rng.choice([0, 12 * bt, 64 * bt]))
    ekw = dict(max_active_sequences=rng.choice([2, 4, 7]), scheduler_token_budget=rng.choice([8, 48, 256]),
               prefill_token_quantum=rng.choice([3, 16, 64]), queue_capacity=64)
    ekw["prefill_token_quantum"] = min(ekw["prefill_token_quantum"], ekw["scheduler_token_budget"])
    (pm, pe), (om, oe_) = both(eng, mkw, ekw)
    stems = [[rng.randrange(3, 64) for _ in range(rng.randint(bt, 6 * bt))] for _ in range(3)]
    submitted = 0
    for wave in range(4):
        prompts, max_new = [], []
        for _ in range(rng.randint(2, 6)):
            stem = rng.choice(stems)
            prompts.append(stem[: rng.randint(1, len(stem))] + [rng.randrange(3, 64) for _ in range(rng.randint(1, 2 * bt))])
            max_new.append(rng.randint(1, 12))
        submit_both(eng, pe, oe_, prompts, max_new, atomic=rng.random() < 0.3 and len(prompts) <= ekw["max_active_sequences"])
        submitted += len(prompts)
        for _ in range(rng.randint(1, 30)):
            if rng.random() < 0.25:
                cancel_both(pe, oe_, rng.randrange(submitted))
            lp, lo = pe.step(), oe_.step()
            assert lp == lo
            assert pm.pool_stats() == om.pool.stats()
            if mkw["prefix_capacity_tokens"]:
                assert pm.prefix_diagnostics() == om.prefix.stats()
    pe.run()
    oe_.run()
    assert pe.trace() == [[tuple(l) for l in t] for t in oe_.trace]
    assert_tick_kinds_agree(pe, oe_)
    states = set()
    for rid in range(submitted):
        rp, ro = pe.result(rid), oe_.results[rid]
        assert rp["state"] == ro.state
        assert list(rp["tokens"]) == ro.tokens
        states.add(rp["state"])
    assert pm.pool_stats() == om.pool.stats()
    if not mkw["prefix_capacity_tokens"]:
        assert pm.pool_stats()["live_blocks"] == 0       # every cancelled request gave its pages back
    assert "cancelled" in states


# ---- benchmark traces (src/engine.rs:430-484; tests at src/engine.rs:4454-4619) ---------------------------------------

def test_atomic_batch_is_fully_admitted_before_its_first_forward(eng):
    """engine.rs:4454-4540: three one-token requests in one atomic batch, three active slots, budget 3, quantum 1 - one tick
    admits all three and runs one packed first-token forward of three lanes; the batch's trace is complete after it."""
    pm, pe = product_engine(eng, dict(vocab=32, max_context=8), dict(max_active_sequences=3, scheduler_token_budget=3, prefill_token_quantum=1))
    ids = pe.submit([eng.Request([1], 1, publish_prompt_prefix=False) for _ in range(3)], True)
    assert pe.batch_trace(ids[0])["complete"] is False
    assert pe.step() == 3
    t = pe.batch_trace(ids[2])
    assert t["complete"] is True
    assert (t["expected_members"], t["admitted_members"], t["terminal_members"], t["rejected_members"]) == (3, 3, 3, 0)
    assert t["admission_active_sequences"] == 3
    assert t["packed_forwards"] == 1 and t["forward_ticks"] == [0]
    info = pe.tick_info(0)
    assert info["kind"] == "first_token" and info["lane_count"] == 3 and info["phases"] == ["first_token"] * 3
    assert t["first_token_ms"] == info["model_ms"]
    assert t["suffix_prefill_ms"] == 0.0 and t["decode_ms"] == 0.0 and t["mixed_ms"] == 0.0


def test_benchmark_trace_retains_each_packed_decode_forward(eng):
    """engine.rs:4541-4619: two two-token requests, budget 2, quantum 1: the trace is unreadable after the first tick and holds
    a first-token forward and a decode forward, two lanes and two input tokens each, after the second."""
    pm, pe = product_engine(eng, dict(vocab=32, max_context=8), dict(max_active_sequences=2, scheduler_token_budget=2, prefill_token_quantum=1))
    ids = pe.submit([eng.Request([1], 2, publish_prompt_prefix=False), eng.Request([1], 2, publish_prompt_prefix=False)], True)
    pe.step()
    assert pe.batch_trace(ids[0])["complete"] is False
    pe.step()
    t = pe.batch_trace(ids[0])
    assert t["complete"] is True and t["forward_ticks"] == [0, 1]
    infos = [pe.tick_info(k) for k in t["forward_ticks"]]
    assert [i["kind"] for i in infos] == ["first_token", "decode"]
    assert all(i["lane_count"] == 2 and i["input_tokens"] == 2 for i in infos)
    assert t["decode_ms"] == infos[1]["model_ms"] and t["mixed_ms"] == 0.0


def test_a_mixed_forward_is_counted_once_in_its_own_bucket(eng):
    """engine.rs:430-439,2347-2356: a forward whose lanes differ in phase is Mixed as a whole; the lanes keep their own phases,
    and a batch whose member shared the forward with an outsider records the whole forward."""
    pm, pe = product_engine(eng, dict(vocab=32), dict(max_active_sequences=3, scheduler_token_budget=8, prefill_token_quantum=2))
    outsider = pe.submit([eng.Request([1, 2, 3, 4, 5], 2)])[0]
    batch = pe.submit([eng.Request([1], 3), eng.Request([2, 3, 4], 1)], True)
    pe.run()
    kinds = [pe.tick_info(k) for k in range(len(pe.trace()))]
    # tick 0: outsider chunk 0-2 (suffix), member 0 first token, member 1 chunk 0-2 (suffix)
    assert kinds[0]["kind"] == "mixed" and kinds[0]["phases"] == ["suffix_prefill", "first_token", "suffix_prefill"]
    # tick 1: outsider chunk 2-4 (suffix), member 0 decode, member 1 last chunk (first token)
    assert kinds[1]["kind"] == "mixed" and kinds[1]["phases"] == ["suffix_prefill", "decode", "first_token"]
    t = pe.batch_trace(batch[0])
    assert t["complete"] and (t["expected_members"], t["admitted_members"], t["rejected_members"]) == (2, 2, 0)
    st = pe.stats()
    assert abs(t["mixed_ms"] - sum(k["model_ms"] for i, k in enumerate(kinds) if i in t["forward_ticks"] and k["kind"] == "mixed")) < 1e-9
    assert abs(st["suffix_prefill_ms"] + st["first_token_ms"] + st["decode_ms"] + st["mixed_ms"] - st["device_ms"]) < 1e-9
    with pytest.raises(RuntimeError, match="was not submitted in an atomic batch"):
        pe.batch_trace(outsider)


def test_rejected_and_cancelled_members_end_the_trace(eng):
    """engine.rs:517-543,3027-3040: a member refused at preflight counts as rejected and terminal, a cancelled one as terminal;
    the trace completes without them ever running."""
    pm, pe = product_engine(eng, dict(vocab=32), dict(max_active_sequences=3, scheduler_token_budget=8, prefill_token_quantum=4))
    ids = pe.submit([eng.Request([1, 2], 1), eng.Request([99], 1), eng.Request([3], 1)], True)
    pe.cancel(ids[2])
    pe.run()
    t = pe.batch_trace(ids[0])
    assert t["complete"] is True
    assert (t["expected_members"], t["admitted_members"], t["terminal_members"], t["rejected_members"]) == (3, 1, 3, 1)
    assert t["admission_active_sequences"] == 1 and t["packed_forwards"] == 1


def test_a_request_local_preflight_failure_does_not_poison_the_worker(eng):
    """engine.rs:5347-5379: an invalid request (top_p = 0) ahead of a healthy one is refused with InvalidRequest; the healthy
    one is admitted and finishes, the engine stays usable and both reusable sessions are still there (two more requests run
    side by side afterwards). engine.rs:4412-4453: a full queue and a poisoned engine are told apart at submission."""
    pm, pe = product_engine(eng, dict(vocab=32), dict(max_active_sequences=2, scheduler_token_budget=8, prefill_token_quantum=4, queue_capacity=2))
    bad, good = pe.submit([eng.Request([1], 1, top_p=0.0), eng.Request([2], 1)])
    with pytest.raises(RuntimeError, match="inference queue is full"):
        pe.submit([eng.Request([3], 1)])
    pe.run()
    assert pe.result(bad)["state"] == "failed" and pe.result(bad)["kind"] == "invalid_request"
    assert pe.result(good)["state"] == "done" and pe.status() == "ready"
    a, b = pe.submit([eng.Request([4, 5], 2), eng.Request([6], 2)])
    pe.run()
    assert all(len(t) == 2 for t in pe.trace()[1:])          # both sessions serve again
    assert pe.result(a)["state"] == pe.result(b)["state"] == "done"
    pm.inject_failure("forward", 3)
    pe.submit([eng.Request([7], 1)])
    pe.run()
    assert pe.status() == "poisoned"
    with pytest.raises(RuntimeError, match=r"inference worker is unavailable \(Poisoned\)"):
        pe.submit([eng.Request([8], 1)])


def test_a_long_lived_host_turns_records_off_and_releases_results(eng):
    """The reference keeps per-forward records only for benchmark submissions (capture_benchmark_trace, engine.rs:1037-1053) and a
    request's result lives in its ticket: here the host says so - no per-tick records, a result dropped once read."""
    pm, pe = product_engine(eng, dict(vocab=32), dict(max_active_sequences=2, scheduler_token_budget=8, prefill_token_quantum=4))
    a, b = pe.submit([eng.Request([1, 2], 2), eng.Request([3], 5)], True)
    pe.step()
    assert len(pe.trace()) == 1
    pe.keep_trace(False)
    assert pe.trace() == []
    with pytest.raises(RuntimeError, match="still running"):
        pe.release(b)
    pe.run()
    assert pe.trace() == [] and pe.stats()["ticks"] == 5          # counters and time buckets keep running
    st = pe.stats()
    assert abs(st["first_token_ms"] + st["decode_ms"] + st["mixed_ms"] + st["suffix_prefill_ms"] - st["device_ms"]) < 1e-6
    assert pe.batch_trace(a)["complete"] and pe.batch_trace(a)["forward_ticks"] == [0]   # what was recorded before the switch stays
    tokens = list(pe.result(a)["tokens"])
    pe.release(a)
    with pytest.raises(RuntimeError, match=f"unknown request id {a}"):
        pe.result(a)
    t = pe.batch_trace(b)                                          # the other member still reaches the batch's trace
    assert t["complete"] and t["terminal_members"] == 2
    pe.release(b)
    with pytest.raises(RuntimeError, match="was not submitted in an atomic batch"):
        pe.batch_trace(b)
    with pytest.raises(RuntimeError, match="unknown request id 99"):
        pe.release(99)
    assert len(tokens) == 2
    pe.keep_trace(True)
    c, d = pe.submit([eng.Request([4], 1), eng.Request([5], 1)], True)
    pe.run()
    assert pe.trace() == [[(c, 0, 1), (d, 0, 1)]] and pe.tick_info(0)["kind"] == "first_token"
    assert pe.batch_trace(c)["forward_ticks"] == [0]              # numbered among the records that are kept


def test_an_atomic_batch_that_does_not_fit_the_queue_leaves_nothing_behind(eng):
    """partial_atomic_batch_send_aborts_queued_members_without_waiting (engine.rs:4620-4662): a batch is queued whole or not at
    all - a refused one leaves no member waiting and takes no request ids that a later submission would skip."""
    pm, pe = product_engine(eng, dict(vocab=32), dict(max_active_sequences=3, scheduler_token_budget=8, prefill_token_quantum=4, queue_capacity=2))
    with pytest.raises(RuntimeError, match="inference batch contains 3 requests, but the atomic admission limit is 2"):
        pe.submit([eng.Request([1], 1), eng.Request([2], 1), eng.Request([3], 1)], True)      # the limit is min(queue, active slots)
    with pytest.raises(RuntimeError, match="inference batch must not be empty"):
        pe.submit([], True)
    first = pe.submit([eng.Request([9], 1)])
    with pytest.raises(RuntimeError, match="inference queue is full"):
        pe.submit([eng.Request([1], 1), eng.Request([2], 1)], True)                         # one place left for two members
    assert pe.pending() == 1
    pe.run()
    ids = pe.submit([eng.Request([1], 1), eng.Request([2], 1)], True)
    assert first == [0] and ids == [1, 2]                                                  # the refused batches took no ids
    pe.run()
    assert all(pe.result(i)["state"] == "done" for i in ids)


def test_a_sequence_keeps_its_own_random_stream_and_history_across_interleaved_steps(eng):
    """resumable_steps_preserve_sampler_rng_and_history (generation.rs:2640-2693): a seeded stochastic request draws the same
    tokens whether it runs alone or takes turns with a neighbour under a one-token budget; another seed draws others."""
    def run(seed, with_neighbour):
        model = eng.Model.fake(vocab=8)
        model.script(logits_row=[1.0, 0.9, 0.8, 0.7, 0.6, 0.5, 0.4, 0.3])
        e = eng.Engine(model, max_active_sequences=2, scheduler_token_budget=1, prefill_token_quantum=1)
        reqs = [eng.Request([1, 2], 12, temperature=1.0, top_k=8, top_p=1.0, seed=seed)]
        if with_neighbour:
            reqs.append(eng.Request([3], 9, temperature=1.0, top_k=8, top_p=1.0, seed=seed + 1))
        ids = e.submit(reqs)
        e.run()
        return list(e.result(ids[0])["tokens"])
    alone, shared, other = run(7, False), run(7, True), run(8, False)
    assert alone == shared and len(alone) == 12
    assert alone != other and len(set(alone)) > 1


# ---- event-channel back-pressure (ActiveSequence::flush_pending, src/engine.rs:1408-1465; tests at src/engine.rs:5132-5283) ----

def step_both(pe, oe_, now_ms):
    lp, lo = pe.step(now_ms), oe_.step(now_ms)
    assert lp == lo
    return lp


def lanes_of(pe, rid):
    return sum(1 for t in pe.trace() for l in t if l[0] == rid)


def test_a_backpressured_slot_is_skipped_while_its_peer_finishes(eng):
    """engine.rs:5132-5237: quantum 1; "a" wants 3 tokens through a channel of ONE event with a 10 ms timeout, "b" 2 tokens
    through a roomy one. After five ticks "a" has run twice and waits with one event pending while "b" has finished. Polling
    the full channel does not restart its clock; once the host takes an event, "a" runs again and the next full channel gets
    a fresh clock; 9 ms later it is still waiting, 11 ms later it is given up and both sessions are back."""
    from oracle import engine as oe
    ekw = dict(max_active_sequences=2, scheduler_token_budget=8, prefill_token_quantum=1)
    (pm, pe), (om, oe_) = both(eng, dict(vocab=32), ekw)
    slow, peer = pe.submit([eng.Request([1], 3, event_capacity=1, event_send_timeout_ms=10.0),
                            eng.Request([2], 2, event_capacity=8, event_send_timeout_ms=10.0)])
    assert [slow, peer] == oe_.submit([oe.Req([1], 3, event_capacity=1, event_send_timeout_ms=10.0),
                                      oe.Req([2], 2, event_capacity=8, event_send_timeout_ms=10.0)])
    for _ in range(5):
        step_both(pe, oe_, 0.0)
    assert lanes_of(pe, slow) == 2, "the slow slot pauses with one event pending"
    assert pe.result(peer)["state"] == "done" and len(pe.result(peer)["tokens"]) == 2
    assert pe.result(slow)["state"] == "running" and len(pe.result(slow)["tokens"]) == 2
    assert pm.pool_stats() == om.pool.stats()
    step_both(pe, oe_, 5.0)
    assert lanes_of(pe, slow) == 2, "a blocked slot runs no forward"
    pe.consume(slow, 1)
    oe_.consume(slow, 1)
    step_both(pe, oe_, 5.0)                       # the waiting event goes out, the third token is produced, the channel is full again
    assert lanes_of(pe, slow) == 3
    step_both(pe, oe_, 5.0 + 9.0)
    assert pe.pending() == 1 and pe.result(slow)["state"] == "done", "9 ms into the new wait the request is still held"
    step_both(pe, oe_, 5.0 + 11.0)
    step_both(pe, oe_, 5.0 + 11.0)
    assert pe.pending() == 0 and oe_.pending() == 0, "the timed-out slot has left"
    assert pe.trace() == [[tuple(l) for l in t] for t in oe_.trace]
    assert pm.pool_stats()["live_blocks"] == 0
    a, b = pe.submit([eng.Request([3], 1), eng.Request([4], 1)])       # both sessions are back
    pe.run()
    assert pe.result(a)["state"] == pe.result(b)["state"] == "done" and len(pe.trace()[-1]) == 2


def test_polling_a_full_channel_does_not_restart_its_timeout(eng):
    """engine.rs:5195-5215: the wait is timed from the moment the event first met a full channel."""
    pm, pe = product_engine(eng, dict(vocab=32), dict(max_active_sequences=1, scheduler_token_budget=8, prefill_token_quantum=4))
    rid = pe.submit([eng.Request([1], 4, event_capacity=1, event_send_timeout_ms=10.0)])[0]
    pe.step(0.0)
    pe.step(1.0)                                   # second token: the channel is full from t = 1
    for now in (3.0, 6.0, 9.0, 10.9):
        assert pe.step(now) == 0 and pe.pending() == 1
    pe.step(11.0)                                  # 10 ms after t = 1
    pe.step(11.0)
    assert pe.pending() == 0 and pe.result(rid)["state"] == "cancelled" and len(pe.result(rid)["tokens"]) == 2


def test_a_blocked_middle_slot_is_filtered_without_shifting_packed_rows(eng):
    """engine.rs:5238-5283: three active one-token prompts with 3 new tokens each, budget 3, quantum 1; the middle one has a
    channel of one event. Ticks 1 and 2 pack all three; in tick 3 the middle slot is held and the forward carries the first
    and the third at rows 0 and 1 with their own inputs and positions."""
    from oracle import engine as oe
    ekw = dict(max_active_sequences=3, scheduler_token_budget=3, prefill_token_quantum=1)
    (pm, pe), (om, oe_) = both(eng, dict(vocab=32), ekw)
    caps = (8, 1, 8)
    ids = pe.submit([eng.Request([p], 3, event_capacity=c, event_send_timeout_ms=1000.0) for p, c in zip((1, 2, 3), caps)])
    assert ids == oe_.submit([oe.Req([p], 3, event_capacity=c, event_send_timeout_ms=1000.0) for p, c in zip((1, 2, 3), caps)])
    for _ in range(3):
        step_both(pe, oe_, 0.0)
    trace = pe.trace()
    assert trace == [[tuple(l) for l in t] for t in oe_.trace]
    assert [[l[0] for l in t] for t in trace] == [[0, 1, 2], [0, 1, 2], [0, 2]]
    assert trace[2] == [(0, 2, 1), (2, 2, 1)]
    assert lanes_of(pe, 1) == 2, "the blocked middle slot does not run in the third tick"
    assert pe.stats()["cleanup_drains"] == 0 and pe.stats()["ticks"] == 3
    # the third tick's tokens are those of rows 0 and 1 of that forward, not shifted by the missing lane
    fake = lambda t, p: (31 * t + 7 * p + 3) % 32
    for rid, first in ((0, 1), (2, 3)):
        want, tok = [], first
        for pos in range(3):
            tok = fake(tok, pos)
            want.append(tok)
        assert list(pe.result(rid)["tokens"]) == want


def test_an_unbounded_channel_never_blocks_and_needs_no_consumer(eng):
    pm, pe = product_engine(eng, dict(vocab=32), dict(max_active_sequences=1, scheduler_token_budget=8, prefill_token_quantum=4))
    rid = pe.submit([eng.Request([1], 50)])[0]
    pe.run()
    assert pe.result(rid)["state"] == "done" and len(pe.result(rid)["tokens"]) == 50
    with pytest.raises(RuntimeError, match="unknown request id 5"):
        pe.consume(5, 1)
    pe.consume(rid, 3)                             # a request that has left the scheduler has no channel: nothing happens


@pytest.mark.parametrize("seed", range(6))
def test_randomised_differential_with_backpressure(eng, seed):
    """Channels of one to three events, hosts that take events at random moments, a clock that advances: schedules, tokens,
    states and pool statistics agree with the oracle tick by tick."""
    from oracle import engine as oe
    rng = random.Random(2000 + seed)
    ekw = dict(max_active_sequences=rng.choice([2, 3, 5]), scheduler_token_budget=rng.choice([4, 16]), prefill_token_quantum=rng.choice([1, 4]),
               queue_capacity=64)
    (pm, pe), (om, oe_) = both(eng, dict(vocab=64, block_tokens=4, kv_capacity_tokens=4096), ekw)
    reqs = [([rng.randrange(3, 64) for _ in range(rng.randint(1, 9))], rng.randint(1, 10), rng.choice([0, 1, 2, 3]), rng.choice([5.0, 40.0, 1e9]))
            for _ in range(12)]
    ids = pe.submit([eng.Request(p, n, event_capacity=c, event_send_timeout_ms=t) for p, n, c, t in reqs])
    assert ids == oe_.submit([oe.Req(p, n, event_capacity=c, event_send_timeout_ms=t) for p, n, c, t in reqs])
    now = 0.0
    for _ in range(400):
        if pe.pending() == 0:
            break
        now += rng.choice([0.0, 1.0, 7.0])
        for rid in ids:
            if rng.random() < 0.3:
                n = rng.randint(1, 2)
                pe.consume(rid, n)
                oe_.consume(rid, n)
        step_both(pe, oe_, now)
        assert pm.pool_stats() == om.pool.stats()
    assert pe.pending() == 0 and oe_.pending() == 0
    assert pe.trace() == [[tuple(l) for l in t] for t in oe_.trace]
    for rid in ids:
        rp, ro = pe.result(rid), oe_.results[rid]
        assert rp["state"] == ro.state and list(rp["tokens"]) == ro.tokens
    assert pm.pool_stats()["live_blocks"] == 0


def test_run_waits_out_a_full_channel_instead_of_reporting_no_progress(eng):
    """A host that drives the engine with run() and never takes events: the request pauses when its channel is full and is
    given up when the send timeout has passed on the engine's own clock; the wait is not mistaken for a stuck scheduler."""
    pm, pe = product_engine(eng, dict(vocab=32), dict(max_active_sequences=2, scheduler_token_budget=8, prefill_token_quantum=4))
    held, free = pe.submit([eng.Request([1], 20, event_capacity=2, event_send_timeout_ms=30.0), eng.Request([2], 20)])
    pe.run()
    assert pe.pending() == 0
    assert pe.result(free)["state"] == "done" and len(pe.result(free)["tokens"]) == 20
    assert pe.result(held)["state"] == "cancelled" and 2 <= len(pe.result(held)["tokens"]) <= 3
    assert pe.status() == "ready" and pm.pool_stats()["live_blocks"] == 0


def test_token_prompts_pass_through_unchanged_and_health_is_explicit(eng):
    """raw_token_input_bypasses_chat_rendering_and_preserves_ids (engine.rs:4178-4194): the ids [4, 0, 2] reach the model as
    they are - id 0 included - and ignore_stop_tokens stays in force. status_health_is_explicit (engine.rs:4366-4374): Ready
    and Busy accept work, Poisoned does not."""
    pm, pe = product_engine(eng, dict(vocab=32), dict(max_active_sequences=1, scheduler_token_budget=8, prefill_token_quantum=8))
    pm.script(stop_ids=[(31 * 2 + 7 * 2 + 3) % 32])          # the first sampled token would stop a request that honoured stop ids
    assert pe.status() == "ready"
    rid = pe.submit([eng.Request([4, 0, 2], 2, ignore_stop_tokens=True)])[0]
    assert pe.status() == "busy"
    pe.run()
    assert pe.trace()[0] == [(rid, 0, 3)]                     # three prompt tokens, none dropped or added
    fake = lambda t, p: (31 * t + 7 * p + 3) % 32
    first = fake(2, 2)
    assert list(pe.result(rid)["tokens"]) == [first, fake(first, 3)] and pe.metrics(rid)["finish_reason"] == "length"
    assert pe.status() == "ready"
    pm.inject_failure("forward", 2)
    pe.submit([eng.Request([1], 1)])
    pe.run()
    assert pe.status() == "poisoned"
    with pytest.raises(RuntimeError, match="unavailable"):
        pe.submit([eng.Request([1], 1)])
