"""Token selection: the reference's own sampler cases (src/sampling.rs:467-511,632-648) on the oracle and on the product's
host sampler, the stochastic rule (src/sampling.rs:145-169,337-390) against an independent numpy restatement, and the
device kernel against the host sampler for the same uniform draws (needs a GPU)."""
import importlib

import numpy as np
import pytest


@pytest.fixture(scope="module")
def ops(mk):
    return importlib.import_module("macllm_infer_b200.ops")


# ---- the reference's known answers ---------------------------------------------------------------------------------

def test_greedy_cases_of_the_reference(ops, orc):
    """greedy_chooses_largest_logit, greedy_ties_choose_the_first_token (src/sampling.rs:467-476,504-506)."""
    for row, want in (([0.0, 3.0, 2.0], 1), ([3.0, 3.0, 2.0], 0), ([-0.0, 0.0, -1.0], 1)):   # total order: -0.0 < +0.0
        assert orc.argmax(np.array(row, np.float32)) == want
        assert int(ops.sample(np.array([row], np.float32), [(0.0, 0, 1.0, 0.0)], 0)[0]) == want


def test_penalty_cases_of_the_reference(ops, orc):
    """penalty_changes_seen_positive_and_negative_logits (src/sampling.rs:497-501) and
    openai_penalties_use_generated_counts_and_follow_repetition (src/sampling.rs:632-648)."""
    for fn in (orc.apply_penalties, ops.penalties):
        assert list(fn([2.0, -2.0, 1.0], [0, 1, 0], 2.0, [], 0.0, 0.0)) == [1.0, -4.0, 1.0]
        step = fn([4.0, -2.0, 3.0, 1.0], [0, 1, 2], 2.0, [], 0.0, 0.0)
        assert list(fn(step, [], 1.0, [1, 1, 2, 99], 1.5, 0.5)) == [2.0, -6.5, -0.5, 1.0]
        original = np.array([-0.0, np.inf, 3.0], np.float32)
        same = fn(original, [], 1.0, [0, 1, 1], 0.0, 0.0)
        assert same.view(np.uint32).tolist() == original.view(np.uint32).tolist()
        assert list(fn([1.0, 2.0], [], 1.0, [0, 0], -1.0, -0.5)) == [3.0, 2.0]


def test_zero_target_never_selects_a_masked_token(ops):
    """src/sampling.rs:508-511: probabilities [0, 1, 0] and a draw of 0 give token 1."""
    row = np.array([[-np.inf, 2.0, -np.inf]], np.float32)
    assert int(ops.sample(row, [(1.0, 0, 1.0, 0.0)], 0)[0]) == 1
    assert int(ops.sample(row, [(1.0, 3, 1.0, 0.0)], 0)[0]) == 1


# ---- the stochastic rule against an independent restatement -------------------------------------------------------------

def numpy_sampler(row, temperature, top_k, top_p, u):
    """Sampler::sample_stochastic in numpy (float64 softmax: only draws away from a boundary are compared)."""
    v = row.astype(np.float64) / temperature
    order = sorted(range(len(v)), key=lambda i: (-v[i], i))
    if 0 < top_k < len(v):
        order = order[:top_k]
    p = np.zeros(len(v))
    p[order] = np.exp(v[order] - v[order[0]])
    p /= p.sum()
    ranked = sorted(order, key=lambda i: (-p[i], i))
    if top_p < 1.0:
        c = np.cumsum(p[ranked])
        keep = int(np.searchsorted(c, top_p, side="left")) + 1
        for i in ranked[keep:]:
            p[i] = 0.0
    cum = np.cumsum(p)
    target = u * cum[-1]
    edge = np.min(np.abs(cum - target)) / cum[-1]
    return int(np.searchsorted(cum, target, side="right")), edge


@pytest.mark.parametrize("temperature,top_k,top_p", [(0.7, 20, 0.8), (0.6, 20, 0.95), (1.0, 1, 1.0), (1.0, 5, 1.0), (1.3, 100, 0.5),
                                                      (0.7, 0, 0.8), (0.9, 0, 0.3)])   # the settings of src/sampling.rs:652-661
def test_host_sampler_follows_the_rule(ops, temperature, top_k, top_p):
    rng = np.random.default_rng(int(temperature * 10) + top_k)
    rows = rng.standard_normal((40, 500)).astype(np.float32) * 3
    us = rng.random(40).astype(np.float32)
    got = ops.sample(rows, [(temperature, top_k, top_p, float(u)) for u in us], 0)
    for r in range(40):
        want, edge = numpy_sampler(rows[r], temperature, top_k, top_p, float(us[r]))
        if edge > 1e-5:   # a draw within float rounding of a boundary may fall on either side
            assert int(got[r]) == want, (r, us[r])


def test_top_k_one_and_tiny_top_p_always_return_the_best(ops):
    rng = np.random.default_rng(5)
    rows = rng.standard_normal((8, 300)).astype(np.float32)
    best = rows.argmax(axis=1)
    for u in (0.0, 0.37, 0.999999):
        assert list(ops.sample(rows, [(0.9, 1, 1.0, u)] * 8, 0)) == list(best)
        assert list(ops.sample(rows, [(0.9, 0, 1e-6, u)] * 8, 0)) == list(best)


def test_draws_follow_the_softmax(ops):
    """A grid of draws reproduces the truncated, renormalised softmax of the kept candidates."""
    row = np.array([2.0, 1.0, 0.0, -1.0, 5.0, -3.0], np.float32)
    n = 4000
    toks = ops.sample(np.repeat(row[None], n, axis=0), [(1.0, 4, 1.0, (i + 0.5) / n) for i in range(n)], 0)
    kept = [4, 0, 1, 2]
    p = np.exp(row[kept] - row[kept].max())
    p /= p.sum()
    freq = np.array([(toks == k).mean() for k in kept])
    assert np.all(np.abs(freq - p) < 2e-3) and set(toks) <= set(kept)


# ---- device == host ---------------------------------------------------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("vocab", [1000, 32000, 128256])
def test_device_sampler_equals_host_sampler(ops, vocab):
    """Same arithmetic, same order of operations, same uniform draw: the same token, on random rows, on rows full of
    ties (values on a coarse grid) and on rows whose top_k cut falls inside a run of equal values."""
    rng = np.random.default_rng(vocab)
    rows = []
    for i in range(48):
        kind = i % 3
        if kind == 0:
            rows.append(rng.standard_normal(vocab) * rng.choice([0.5, 2.0, 6.0]))
        elif kind == 1:
            rows.append(np.round(rng.standard_normal(vocab) * 2) / 2)          # heavy ties
        else:
            r = rng.standard_normal(vocab) * 0.1
            r[rng.choice(vocab, size=min(vocab, 300), replace=False)] = 3.0    # the cut falls among equals
            rows.append(r)
    rows = np.array(rows, np.float32)
    settings = []
    for i in range(48):
        t = float(rng.choice([0.0, 0.3, 0.7, 1.0, 1.5]))
        k = int(rng.choice([1, 5, 40, 100, 1000, 1024]))
        settings.append((t, min(k, vocab), float(rng.choice([0.3, 0.8, 0.95, 1.0])), float(rng.random())))
    host = ops.sample(rows, settings, 0)
    dev = ops.sample(rows, settings, 1)
    assert list(dev) == list(host)
    # and many draws on one row
    row = np.repeat(rows[:1], 256, axis=0)
    st = [(0.8, 50, 0.9, (i + 0.25) / 256) for i in range(256)]
    assert list(ops.sample(row, st, 1)) == list(ops.sample(row, st, 0))


@pytest.mark.gpu
def test_device_sampler_refuses_what_it_does_not_cover(ops):
    capi = importlib.import_module("macllm_infer_b200._capi")
    rows = np.zeros((1, 2000), np.float32)
    for k in (0, 1025):
        with pytest.raises(capi.MkError, match="1 <= top_k <= 1024"):
            ops.sample(rows, [(1.0, k, 1.0, 0.5)], 1)
    with pytest.raises(capi.MkError, match="sampling distribution is empty"):
        ops.sample(np.full((1, 2000), -np.inf, np.float32), [(1.0, 10, 1.0, 0.5)], 1)


@pytest.mark.gpu
def test_engine_samples_on_the_device_like_on_the_host(mk, tmp_path_factory):
    """A request with temperature / top-k / top-p: the engine picks its tokens on the device (one u32 per lane crosses
    PCIe) and gets the tokens the host sampler picks from the read-back logits, draw for draw."""
    eng = importlib.import_module("macllm_infer_b200.engine")
    seed = importlib.import_module("macllm_infer_b200.seed_gguf")
    spec = seed.scaled("tinyllama-1.1b", layers=2, vocab=2048)
    path = tmp_path_factory.mktemp("samp") / "llama.gguf"
    seed.write_seed_gguf(path, spec, seed=0)
    rng = np.random.default_rng(3)
    prompts = [rng.integers(3, spec.vocab, size=n) for n in (9, 30, 17)]
    def run(host_sampling):
        model = eng.Model.load_gguf(path, kv_dtype="f16", matmul_path=0, max_batch_tokens=128, max_batch_lanes=4)
        e = eng.Engine(model, max_active_sequences=4, scheduler_token_budget=64, prefill_token_quantum=32, host_sampling=host_sampling)
        reqs = [eng.Request(prompts[0], 12, temperature=0.8, top_k=40, top_p=0.9, seed=11),
                eng.Request(prompts[1], 12),                                                   # greedy lane in the same ticks
                eng.Request(prompts[2], 12, temperature=1.2, top_k=5, top_p=1.0, seed=12)]
        ids = e.submit(reqs, atomic_batch=True)
        e.run()
        out = [list(e.result(i)["tokens"]) for i in ids]
        st = e.stats()
        e.close()
        model.close()
        return out, st
    dev, st_dev = run(False)
    host, st_host = run(True)
    assert dev == host
    assert st_dev["device_sampled"] == 24 and st_host["device_sampled"] == 0
