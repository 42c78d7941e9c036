"""The host-side plans of the two TMA matmuls (no GPU): how a launch is cut into tiles, K shares and partial-sum slots.
Invariants the consumer kernels rely on, and the plans of the benchmark's shapes (SmolLM3-3B: hidden 2048, q|k|v 3072,
gate|up 22016, FFN 11008)."""
import importlib

import numpy as np
import pytest

SMS = 148


@pytest.fixture(scope="module")
def env(mk):
    return importlib.import_module("macllm_infer_b200.ops"), importlib.import_module("macllm_infer_b200._capi")


def test_f16_gemm_plans_of_the_benchmark_shapes(env):
    ops, capi = env
    qkv = ops.matmul_plan(capi.PATH_HALF, 3072, 2048, 64)
    assert (qkv["bn"], qkv["row_tiles"], qkv["splits"]) == (64, 24, 6)           # 144 CTAs of one 64-lane decode tick
    down = ops.matmul_plan(capi.PATH_HALF, 2048, 11008, 64)
    assert (down["row_tiles"], down["splits"], down["kb_per_split"]) == (16, 9, 20)
    gate_up = ops.matmul_plan(capi.PATH_HALF, 22016, 2048, 2048)
    assert (gate_up["bn"], gate_up["n_tiles"], gate_up["splits"]) == (256, 8, 1)  # wide ticks never share K
    assert ops.matmul_plan(capi.PATH_HALF, 3072, 2048, 2048)["bn"] == 128         # 2.6 rounds of 128 beat 1.3 rounds of 256
    head = ops.matmul_plan(capi.PATH_HALF, 128256, 2048, 64)
    assert head["splits"] == 1                                                    # enough row tiles already


@pytest.mark.parametrize("rows,cols", [(256, 2048), (2048, 2048), (3072, 2048), (2048, 11008), (22016, 2048), (12288, 4096), (1152, 768)])
@pytest.mark.parametrize("T", [2, 9, 33, 64, 65, 128, 512, 2048])
def test_f16_gemm_plan_invariants(env, rows, cols, T):
    ops, capi = env
    p = ops.matmul_plan(capi.PATH_HALF, rows, cols, T)
    assert p["bn"] in (64, 128, 256) and p["bn"] * p["n_tiles"] >= T > p["bn"] * (p["n_tiles"] - 1)
    assert p["row_tiles"] == -(-rows // 128)
    kb = cols // 64
    assert 1 <= p["splits"] <= 16 and p["kb_per_split"] * p["splits"] >= kb > p["kb_per_split"] * (p["splits"] - 1)
    if p["splits"] > 1:
        assert p["kb_per_split"] >= 4 and p["partial_floats"] == p["splits"] * T * rows <= (16 << 20) // 4
    else:
        assert p["partial_floats"] == 0
    assert ops.matmul_plan(capi.PATH_HALF, rows, cols, T, max_splits=1)["splits"] == 1


@pytest.mark.parametrize("rows,cols", [(2560, 2048), (2048, 2048), (22016, 2048), (2048, 11008), (1000, 11008), (128, 256), (128256, 2048)])
@pytest.mark.parametrize("T", [2, 17, 33, 64])
def test_streamed_matmul_plan_invariants(env, rows, cols, T):
    ops, capi = env
    p = ops.matmul_plan(capi.PATH_STREAM, rows, cols, T)
    nb = cols // 256
    assert p["row_tiles"] == -(-rows // 128) and p["tiles_per_group"] in (1, 2, 4)
    assert p["groups"] == -(-p["row_tiles"] // p["tiles_per_group"]) and p["items"] == p["groups"] * nb
    assert 1 <= p["ctas"] <= min(SMS, p["items"])   # at most one persistent CTA per SM
    assert 1 <= p["slots"] <= 16 and p["bn"] >= T and p["bn"] in (16, 32, 64)
    assert p["partial_floats"] == (p["slots"] * T * rows if p["slots"] > 1 else 0)
    assert p["partial_floats"] * 4 <= 24 << 20
    if p["slots"] == 1:
        assert p["ctas"] <= p["groups"]             # whole groups: every result is complete in one CTA
    whole = ops.matmul_plan(capi.PATH_STREAM, rows, cols, T, max_splits=1)
    assert whole["slots"] == 1 and whole["ctas"] == min(SMS, whole["groups"])


def test_streamed_matmul_plans_of_the_benchmark_shapes(env):
    ops, capi = env
    gate_up = ops.matmul_plan(capi.PATH_STREAM, 22016, 2048, 64)
    assert (gate_up["ctas"], gate_up["tiles_per_group"], gate_up["slots"]) == (148, 2, 3)   # 4.6 items of two units per CTA
    down = ops.matmul_plan(capi.PATH_STREAM, 2048, 11008, 64)
    assert (down["ctas"], down["tiles_per_group"]) == (148, 1) and down["slots"] <= 11
    head = ops.matmul_plan(capi.PATH_STREAM, 128256, 2048, 64)
    assert head["slots"] == 1 and head["ctas"] == 148                                          # 32 MB per slot: never cut


def test_plans_refuse_what_the_kernels_do_not_cover(env):
    ops, capi = env
    with pytest.raises(capi.MkError):
        ops.matmul_plan(capi.PATH_STREAM, 2048, 2048, 65)
    with pytest.raises(capi.MkError):
        ops.matmul_plan(capi.PATH_HALF, 2048, 100, 64)
    with pytest.raises(capi.MkError):
        ops.matmul_plan(capi.PATH_GEMV, 2048, 2048, 4)
