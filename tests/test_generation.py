"""The per-sequence phase machine on the host-only model: the known answers of the reference's generation tests
(src/generation.rs:2052-2288,2404-2475,2517-2585,2694-2756) asked of the engine, one request at a time unless the case is
about interleaving. The fake model answers token t at position p with (31 t + 7 p + 3) mod vocab, or a scripted logits row."""
import importlib

import pytest


@pytest.fixture(scope="module")
def eng(mk):
    return importlib.import_module("macllm_infer_b200.engine")


def one(eng, prompt, max_new, model_kw=None, engine_kw=None, stop_ids=(), logits_row=(), **request_kw):
    model = eng.Model.fake(**dict(dict(vocab=16), **(model_kw or {})))
    if stop_ids or logits_row:
        model.script(stop_ids=stop_ids, logits_row=logits_row)
    e = eng.Engine(model, **dict(dict(max_active_sequences=1, scheduler_token_budget=8, prefill_token_quantum=8), **(engine_kw or {})))
    rid = e.submit([eng.Request(prompt, max_new, **request_kw)])[0]
    e.run()
    return model, e, rid


def test_every_successful_prefill_quantum_publishes_its_exact_endpoint(eng):
    """generation.rs:2052-2074: a five-token prompt in quanta of two publishes the prefixes of 2, 4 and 5 tokens."""
    model, e, rid = one(eng, [0, 1, 2, 0, 1], 1, dict(block_tokens=1, prefix_capacity_tokens=64),
                        dict(scheduler_token_budget=2, prefill_token_quantum=2))
    d = model.prefix_diagnostics()
    assert d["insertions"] == 3 and d["entries"] == 3 and d["cached_blocks"] == 2 + 4 + 5
    assert e.trace() == [[(rid, 0, 2)], [(rid, 2, 2)], [(rid, 4, 1)]]


def test_a_sequence_can_disable_prompt_prefix_publication(eng):
    """generation.rs:2076-2096."""
    model, e, rid = one(eng, [0, 1, 2, 0, 1], 1, dict(block_tokens=1, prefix_capacity_tokens=64),
                        dict(scheduler_token_budget=2, prefill_token_quantum=2), publish_prompt_prefix=False)
    assert model.prefix_diagnostics()["insertions"] == 0 and e.result(rid)["state"] == "done"


def test_metrics_split_prefill_without_double_counting_the_first_token_forward(eng):
    """generation.rs:2098-2123: five prompt tokens in quanta of two, two new tokens: prefill time is suffix time plus the
    first-token forward's time, one decode step; each forward's time is in exactly one bucket."""
    model, e, rid = one(eng, [0, 1, 2, 0, 1], 2, engine_kw=dict(scheduler_token_budget=2, prefill_token_quantum=2))
    m = e.metrics(rid)
    assert m["prefill_ms"] == m["suffix_prefill_ms"] + m["first_token_ms"]
    assert m["decode_steps"] == 1 and m["generated_tokens"] == 2 and m["prompt_tokens"] == 5
    times = [e.tick_info(k)["model_ms"] for k in range(4)]
    assert m["suffix_prefill_ms"] == times[0] + times[1] and m["first_token_ms"] == times[2] and m["decode_ms"] == times[3]
    assert [e.tick_info(k)["kind"] for k in range(4)] == ["suffix_prefill", "suffix_prefill", "first_token", "decode"]


def test_a_stop_token_after_a_decode_counts_the_model_step(eng):
    """generation.rs:2125-2144: the first token is visible, the decode step samples a stop token: one generated token, one
    decode step, finish reason Stop; the stop token is not part of the output."""
    # prompt [0] -> 3 at position 0; 3 at position 1 -> (93 + 7 + 3) mod 8 = 7, the stop token
    model, e, rid = one(eng, [0], 3, dict(vocab=8), stop_ids=[7], ignore_stop_tokens=False)
    m = e.metrics(rid)
    assert list(e.result(rid)["tokens"]) == [3]
    assert (m["generated_tokens"], m["decode_steps"], m["finish_reason"]) == (1, 1, "stop")


def test_benchmark_mode_ignores_stop_tokens(eng):
    """generation.rs:2268-2287: with ignore_stop_tokens the same sequence runs to its length limit through the stop token."""
    model, e, rid = one(eng, [0], 3, dict(vocab=8), stop_ids=[7], ignore_stop_tokens=True)
    m = e.metrics(rid)
    assert list(e.result(rid)["tokens"])[:2] == [3, 7]
    assert (m["generated_tokens"], m["decode_steps"], m["finish_reason"]) == (3, 2, "length")


def test_a_stop_token_as_the_first_token_ends_without_output(eng):
    """generation.rs:1221-1225 at the first-token forward: nothing visible, no decode step, reason Stop."""
    model, e, rid = one(eng, [0], 3, dict(vocab=8), stop_ids=[3], ignore_stop_tokens=False)
    m = e.metrics(rid)
    assert list(e.result(rid)["tokens"]) == [] and e.result(rid)["state"] == "done"
    assert (m["generated_tokens"], m["decode_steps"], m["finish_reason"]) == (0, 0, "stop")


def test_a_cached_prefix_skips_only_the_restored_prompt_tokens(eng):
    """generation.rs:2146-2167: prompt [0, 1, 2] with two tokens restored runs one forward of the token 2 at position 2."""
    model = eng.Model.fake(vocab=8, block_tokens=2, prefix_capacity_tokens=64)
    e = eng.Engine(model, max_active_sequences=1, scheduler_token_budget=8, prefill_token_quantum=8)
    first = e.submit([eng.Request([0, 1, 2], 1)])[0]
    e.run()
    second = e.submit([eng.Request([0, 1, 2], 1)])[0]
    e.run()
    m = e.metrics(second)
    assert (m["prompt_tokens"], m["cached_prompt_tokens"]) == (3, 2)
    assert m["prompt_tokens"] - m["cached_prompt_tokens"] == 1          # processed_prompt_tokens
    assert e.trace()[-1] == [(second, 2, 1)]
    assert list(e.result(second)["tokens"]) == list(e.result(first)["tokens"])


def test_one_token_is_legal_at_full_context_and_two_are_not(eng):
    """generation.rs:2230-2266: a prompt that fills the context may still sample one token (its logits need no new cache
    slot); a second token would need one."""
    model, e, rid = one(eng, [0, 1], 1, dict(vocab=8, max_context=2))
    m = e.metrics(rid)
    assert e.result(rid)["state"] == "done" and (m["generated_tokens"], m["decode_steps"]) == (1, 0)
    model, e, rid = one(eng, [0, 1], 2, dict(vocab=8, max_context=2))
    r = e.result(rid)
    assert r["state"] == "failed" and r["kind"] == "invalid_request" and "maximum context length is 2 tokens" in r["message"]
    assert e.trace() == []


def test_the_final_visible_token_finishes_in_the_same_quantum(eng):
    """generation.rs:2404-2445: two new tokens take the first-token forward and one decode; the step that emits the second
    token is terminal (no further forward), the session is handed back empty."""
    model, e, rid = one(eng, [0], 2, dict(vocab=8))
    m = e.metrics(rid)
    assert (m["generated_tokens"], m["decode_steps"], m["finish_reason"]) == (2, 1, "length")
    assert len(e.trace()) == 2 and e.pending() == 0
    assert e.step() == 0 and len(e.trace()) == 2
    assert model.pool_stats()["live_blocks"] == 0


def test_a_zero_budget_request_finishes_without_model_work(eng):
    """generation.rs:2449-2475: max_new_tokens 0 ends with reason Length, no forward, nothing cached."""
    model, e, rid = one(eng, [0], 0, dict(vocab=8))
    m = e.metrics(rid)
    assert e.result(rid)["state"] == "done" and e.trace() == []
    assert (m["generated_tokens"], m["decode_steps"], m["finish_reason"]) == (0, 0, "length")
    assert m["prefill_ms"] == 0.0 and model.pool_stats()["live_blocks"] == 0


def test_the_token_budget_chunks_prefill_without_sampling_intermediate_logits(eng):
    """generation.rs:2517-2585 and 2586-2639 (blocking_quantum_chunks_prefill_and_matches_one_shot_generation): intermediate
    chunks advance the cursor and sample nothing; only the chunk that ends the prompt samples, and the result equals the
    one-shot run."""
    _, chunked, a = one(eng, [1, 2, 3, 4, 5, 6, 7], 3, engine_kw=dict(scheduler_token_budget=3, prefill_token_quantum=3))
    _, whole, b = one(eng, [1, 2, 3, 4, 5, 6, 7], 3)
    assert [t[0][1:] for t in chunked.trace()] == [(0, 3), (3, 3), (6, 1), (7, 1), (8, 1)]
    assert [chunked.tick_info(k)["kind"] for k in range(3)] == ["suffix_prefill", "suffix_prefill", "first_token"]
    assert list(chunked.result(a)["tokens"]) == list(whole.result(b)["tokens"])
    assert chunked.stats()["prefill_tokens"] == 7 and chunked.stats()["decode_tokens"] == 2


def test_generated_penalties_are_sequence_local_across_interleaved_steps(eng):
    """generation.rs:2694-2756: every forward returns the logits [2, 1, 0, -1]; with a presence penalty of 1.5 a sequence
    produces 0, 1, 0 - and so do two sequences stepping in the same batch, and a fresh one afterwards: the penalty counts
    only the sequence's own generated tokens, never the prompt and never a neighbour's."""
    model = eng.Model.fake(vocab=8)
    model.script(logits_row=[2.0, 1.0, 0.0, -1.0])
    e = eng.Engine(model, max_active_sequences=2, scheduler_token_budget=8, prefill_token_quantum=4)
    a, b = e.submit([eng.Request([0], 3, presence_penalty=1.5), eng.Request([0], 3, presence_penalty=1.5)])
    e.run()
    assert all(len(t) == 2 for t in e.trace())            # the two sequences shared every forward
    assert list(e.result(a)["tokens"]) == [0, 1, 0] == list(e.result(b)["tokens"])
    c = e.submit([eng.Request([0], 3, presence_penalty=1.5)])[0]
    e.run()
    assert list(e.result(c)["tokens"]) == [0, 1, 0]
    plain = e.submit([eng.Request([0], 3)])[0]
    e.run()
    assert list(e.result(plain)["tokens"]) == [0, 0, 0]


def test_two_sequences_interleave_without_crossing_sessions(eng):
    """generation.rs:2784-2859: two requests that take turns under a one-token budget end with the tokens each would have
    produced alone."""
    model = eng.Model.fake(vocab=16)
    e = eng.Engine(model, max_active_sequences=2, scheduler_token_budget=1, prefill_token_quantum=1)
    a, b = e.submit([eng.Request([1, 2, 3], 3), eng.Request([4, 5], 4)])
    e.run()
    assert all(len(t) == 1 for t in e.trace())
    _, ea, ra = one(eng, [1, 2, 3], 3)
    _, eb, rb = one(eng, [4, 5], 4)
    assert list(e.result(a)["tokens"]) == list(ea.result(ra)["tokens"])
    assert list(e.result(b)["tokens"]) == list(eb.result(rb)["tokens"])


def test_resumable_steps_run_one_forward_per_quantum_and_hide_the_stop_token(eng):
    """resumable_steps_match_blocking_generation_and_one_forward_per_quantum (generation.rs:2312-2403): prompt [0, 0], up to
    four tokens, stop tokens honoured: three forwards - the prompt, then each visible token at positions 2 and 3 - and the
    third samples the stop token, which is never visible: two tokens, two decode steps, reason Stop."""
    # the fake answers (0 at position 1) -> 2, (2 at position 2) -> 7, (7 at position 3) -> 1, the stop token
    model, e, rid = one(eng, [0, 0], 4, dict(vocab=8), stop_ids=[1], ignore_stop_tokens=False)
    assert e.trace() == [[(rid, 0, 2)], [(rid, 2, 1)], [(rid, 3, 1)]]
    assert list(e.result(rid)["tokens"]) == [2, 7]
    m = e.metrics(rid)
    assert (m["prompt_tokens"], m["generated_tokens"], m["decode_steps"], m["finish_reason"]) == (2, 2, 2, "stop")
    assert model.pool_stats()["live_blocks"] == 0
