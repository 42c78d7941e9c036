"""The host side of the five benchmark workloads at their full size, on the host-only fake model: schedules, tokens,
prefix hits, block tables (through the pool counters and cached-token counts) and evictions of the product's C++
engine must equal the oracle's Python restatement of the reference's scheduler, KV pool and prefix cache bit for bit.
No arithmetic is involved, so no GPU is needed; the logits side of parity is covered by the GPU tests."""
import importlib

import pytest


@pytest.fixture(scope="module")
def env(mk):
    return importlib.import_module("macllm_infer_b200.engine"), importlib.import_module("macllm_infer_b200.workloads")


def engines(eng, wl, w, prompts, new, vocab=4096):
    from oracle import engine as oe
    cap = wl.kv_capacity_tokens(w, prompts, new)
    mkw = dict(vocab=vocab, max_context=1 << 16, kv_capacity_tokens=cap, prefix_capacity_tokens=w.prefix_capacity_tokens)
    ekw = dict(max_active_sequences=w.max_active(), scheduler_token_budget=w.budget, prefill_token_quantum=w.quantum,
               queue_capacity=len(prompts) + 8)
    pm = eng.Model.fake(**mkw)
    pe = eng.Engine(pm, **ekw)
    om = oe.OracleModel(vocab, 1 << 16, 16, 8, cap, w.prefix_capacity_tokens)
    oe_ = oe.OracleEngine(om, **ekw)
    return pm, pe, om, oe_


def compare(pm, pe, om, oe_, ids):
    assert pe.trace() == [[tuple(l) for l in t] for t in oe_.trace]
    for i in ids:
        rp, ro = pe.result(i), oe_.results[i]
        assert rp["state"] == ro.state and list(rp["tokens"]) == ro.tokens and rp["cached_tokens"] == ro.cached_tokens
    assert pm.pool_stats() == om.pool.stats()
    if om.prefix is not None:
        assert pm.prefix_diagnostics() == om.prefix.stats()


@pytest.mark.parametrize("name", ["tinyllama-1.1b-batch4", "smollm3-3b-ragged64", "gemma2-9b-long128"])
def test_one_atomic_batch_workloads(env, name):
    """Configurations 1, 2 and 4: the whole batch admitted at once."""
    eng, wl = env
    from oracle import engine as oe
    w = wl.WORKLOADS[name]
    prompts, new, _ = wl.make_requests(w, 4096)
    pm, pe, om, oe_ = engines(eng, wl, w, prompts, new)
    ids = pe.submit([eng.Request(p, n) for p, n in zip(prompts, new)], atomic_batch=True)
    assert ids == oe_.submit([oe.Req([int(t) for t in p], n) for p, n in zip(prompts, new)], atomic_batch=True)
    pe.run()
    oe_.run()
    compare(pm, pe, om, oe_, ids)
    st = pe.stats()
    assert st["completed_requests"] == w.seqs and st["failed_requests"] == 0
    assert st["prefill_tokens"] == sum(len(p) for p in prompts) and st["decode_tokens"] == sum(n - 1 for n in new)


@pytest.mark.parametrize("rank", [0, 1])
def test_prefix_reuse_workload_per_replica(env, rank):
    """Configuration 3, one replica: request 0 alone, then the other 31 in submission order; 2048 shared tokens.  Hits,
    misses, matched tokens, insertions and evictions of the prefix cache are compared exactly."""
    eng, wl = env
    from oracle import engine as oe
    w = wl.WORKLOADS["qwen3-8b-prefix32"]
    prompts, new, _ = wl.make_requests(w, 4096, rank)
    pm, pe, om, oe_ = engines(eng, wl, w, prompts, new)
    ids = []
    for lo, hi in ((0, 1), (1, len(prompts))):
        a = pe.submit([eng.Request(p, n) for p, n in zip(prompts[lo:hi], new[lo:hi])])
        assert a == oe_.submit([oe.Req([int(t) for t in p], n) for p, n in zip(prompts[lo:hi], new[lo:hi])])
        ids += a
        pe.run()
        oe_.run()
    compare(pm, pe, om, oe_, ids)
    d = pm.prefix_diagnostics()
    assert d["hits"] == 31 and d["misses"] == 1 and d["matched_tokens"] == 31 * 2048
    assert all(pe.result(i)["cached_tokens"] == 2048 for i in ids[1:])


def test_poisson_arrival_workload(env):
    """Configuration 5, the first 700 arrivals: requests are submitted when a virtual clock (20 ms per scheduler tick)
    passes their arrival time and at most 512 run at once (the KV pool holds the 512 longest sequences).  Every tick of
    both engines must agree."""
    eng, wl = env
    from oracle import engine as oe
    w = wl.WORKLOADS["qwen3-30b-a3b-poisson"]
    prompts, new, arrivals = wl.make_requests(w, 4096, 0, limit=700)
    pm, pe, om, oe_ = engines(eng, wl, w, prompts, new)
    ids, nxt, now = [], 0, 0.0
    while nxt < len(prompts) or pe.pending() > 0:
        wave = []
        while nxt < len(prompts) and arrivals[nxt] <= now:
            wave.append(nxt)
            nxt += 1
        if wave:
            a = pe.submit([eng.Request(prompts[i], new[i]) for i in wave])
            assert a == oe_.submit([oe.Req([int(t) for t in prompts[i]], new[i]) for i in wave])
            ids += a
        assert pe.step() == oe_.step()
        now += 0.020
    assert oe_.pending() == 0
    compare(pm, pe, om, oe_, ids)
    assert pe.stats()["completed_requests"] == 700
