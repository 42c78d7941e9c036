"""Every entry of tests/golden/reference_known_answers.json (known answers transcribed from the reference's own tests) against
the oracle and, where no GPU is needed, the product's host library."""
import importlib
import json
from pathlib import Path

import numpy as np
import pytest

GOLDEN = json.loads((Path(__file__).parent / "golden" / "reference_known_answers.json").read_text())


@pytest.fixture(scope="module")
def ops(mk):
    return importlib.import_module("macllm_infer_b200.ops")


def test_every_entry_names_its_source():
    for name, entry in GOLDEN.items():
        if not name.startswith("_"):
            assert ".rs:" in entry["source"], name


def test_prefix_hash(mk):
    from oracle import kv
    pkv = importlib.import_module("macllm_infer_b200.kv")
    g = GOLDEN["prefix_hash_golden"]
    want = bytes.fromhex(g["digest_hex"])
    assert kv.endpoint_digest(g["tokens"], g["endpoint"], g["block_tokens"]) == want
    first = pkv.block_digests(g["block_tokens"], g["tokens"])[0]          # the product's chained digest of the one full block
    assert kv.hash_block(first, g["block_tokens"], 1, g["tokens"][4:]) == want


def test_block_formats_and_unpermutation(ops, orc):
    q4, q8 = GOLDEN["q4_0_block"], GOLDEN["q8_0_block"]
    raw = np.array(q4["bytes"], np.uint8)
    want = np.array(q4["weights"], np.float32)
    assert np.array_equal(orc.dequant(2, raw, 1, 32)[0], want) and np.array_equal(ops.decode_rows(2, raw, 1, 32)[0], want)
    raw = np.array(q8["bytes"], np.uint8)
    assert np.array_equal(orc.dequant(8, raw, 1, 32)[0], np.array(q8["signed"], np.float32) * np.float32(q8["scale"]))
    u = GOLDEN["llama_qk_unpermute"]
    rows = np.arange(u["rows"], dtype=np.float32)
    assert list(ops.unpermute_qk_rows(rows.view(np.uint8), u["rows"], u["heads"]).view(np.float32)) == u["order"]


def test_recurrent_steps(orc):
    g = GOLDEN["gated_delta_step"]
    out, state = orc.gated_delta_recurrence(np.array([[g["query"]]]), np.array([[g["key"]]]), np.array([[g["value"]]]), np.array([[g["decay"]]]),
                                            np.array([[g["beta"]]]), np.array(g["state"], np.float32).reshape(1, 1, 2, 2))
    assert np.max(np.abs(state.reshape(-1) - np.array(g["next_state"], np.float32))) <= g["tolerance"]
    assert np.max(np.abs(out.reshape(-1) - np.array(g["output"], np.float32))) <= g["tolerance"]
    c = GOLDEN["short_convolution"]
    x = np.array(c["input_rows"], np.float32)
    out, tail = orc.short_conv(np.concatenate([x, x, x], axis=1), np.array(c["kernel"], np.float32), np.zeros((1, 2, 2), np.float32))
    assert np.array_equal(out, np.array(c["output"], np.float32)) and np.array_equal(tail[0], np.array(c["tail"], np.float32))


def test_gqa_head_mapping(orc):
    g = GOLDEN["gqa_head_mapping"]
    keys, values = np.array(g["keys"], np.float32), np.array(g["values"], np.float32)
    k_pool, v_pool = np.zeros((1, 1, 2, 2, 1), np.float32), np.zeros((1, 1, 2, 2, 1), np.float32)
    for p in range(2):
        k_pool[0, 0, :, p], v_pool[0, 0, :, p] = keys[p], values[p]
    got = orc.paged_attention(np.ones((1, 4), np.float32), k_pool, v_pool, [0], [0], [1], [1], q_heads=4, kv_heads=2, d=1, block_tokens=2,
                              layers=1, layer=0, scale=1.0, softcap=0.0, mode=2).reshape(4)
    w0, w1 = g["weights"]
    want = [w0 * 1.0 + w1 * 10.0] * 2 + [-w1 - w0 * 10.0] * 2
    assert np.max(np.abs(got - np.array(want, np.float32))) <= g["tolerance"]


def test_schedules(mk):
    eng = importlib.import_module("macllm_infer_b200.engine")
    g = GOLDEN["scheduler_round_robin"]
    e = eng.Engine(eng.Model.fake(vocab=32), max_active_sequences=3, scheduler_token_budget=g["budget"], prefill_token_quantum=g["quantum"])
    e.submit([eng.Request(p, 1) for p in g["prompts"]])
    for _ in range(3):
        e.step()
    assert [[l[0] for l in t] for t in e.trace()] == g["lanes_per_tick"]
    b = GOLDEN["blocked_middle_slot"]
    e = eng.Engine(eng.Model.fake(vocab=32), max_active_sequences=3, scheduler_token_budget=3, prefill_token_quantum=1)
    e.submit([eng.Request([p], 3, event_capacity=c, event_send_timeout_ms=1000.0) for p, c in zip((1, 2, 3), (8, 1, 8))])
    for _ in range(3):
        e.step(0.0)
    assert [[l[0] for l in t] for t in e.trace()] == b["lanes_per_tick"]
    assert [list(l) for l in e.trace()[2]] == b["third_tick"]
