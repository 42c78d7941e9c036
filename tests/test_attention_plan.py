"""The host-side plan of a tick's attention work (no GPU): which one-token lanes have their keys shared out over several
CTAs.  The rules come from measurements on B200: a share costs a partial write, a counter and a merge, so it must be
worth at least 512 keys; with few lanes, histories are cut until about two CTAs per SM are in flight; once lanes x KV
heads give every SM a CTA, only a history more than twice the mean is cut."""
import importlib

import numpy as np
import pytest


@pytest.fixture(scope="module")
def ops(mk):
    return importlib.import_module("macllm_infer_b200.ops")


def test_short_histories_are_never_shared(ops):
    shares, tiles, bound = ops.attention_plan([17, 80, 200, 333], [1, 1, 1, 1], 32, 4)
    assert shares.tolist() == [1, 1, 1, 1] and tiles == 0 and bound >= 4


def test_few_lanes_with_long_histories_are_cut_into_balanced_shares(ops):
    ctx = [8191, 4095, 600, 100]
    shares, _, bound = ops.attention_plan(ctx, [1] * 4, 16, 4)
    assert shares[0] > shares[1] > 1 and shares[3] == 1
    assert shares.max() <= 16 and shares.sum() <= bound
    keys_per_share = [(c + 1) / s for c, s in zip(ctx, shares)]
    assert min(keys_per_share[:2]) >= 512


def test_lanes_that_fill_the_gpu_are_left_whole(ops):
    rng = np.random.default_rng(0)
    ctx = rng.integers(160, 1153, 64)
    shares, _, _ = ops.attention_plan(ctx, [1] * 64, 16, 4)
    assert shares.tolist() == [1] * 64


def test_one_long_history_among_many_short_ones_is_cut(ops):
    ctx = [300] * 63 + [8192]
    shares, _, bound = ops.attention_plan(ctx, [1] * 64, 16, 4)
    assert shares[:63].tolist() == [1] * 63 and 4 <= shares[63] <= 16
    assert shares.sum() <= bound


def test_prefill_lanes_become_query_tiles(ops):
    shares, tiles, _ = ops.attention_plan([0, 100, 40], [512, 1, 33], 16, 4)
    assert shares.tolist() == [0, 1, 0]
    assert tiles == 512 // 16 + (33 + 15) // 16   # 16 query rows x 4 heads per tile of four warps


def test_bad_arguments_are_refused(ops):
    capi = importlib.import_module("macllm_infer_b200._capi")
    with pytest.raises(capi.MkError):
        ops.attention_plan([1], [1], 6, 4)
