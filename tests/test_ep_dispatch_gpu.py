"""The dispatch / return exchange of expert parallelism with data-parallel lanes, checked by itself: the kernels of all
ranks run on one device, stage by stage on one stream, so every flag a kernel waits for was published by an earlier launch
(kernels that wait on one another are never in flight together).  `row * (expert + 1)` stands in for the expert matmuls,
which makes a misplaced row visible as a wrong factor."""
import importlib

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def make_case(rng, ranks, local_experts, hidden, cap, empty_rank=-1):
    experts = ranks * local_experts
    rows = rng.standard_normal((ranks, cap, hidden)).astype(np.float16)
    offsets = np.zeros((ranks, experts + 1), dtype=np.int32)
    for r in range(ranks):
        if r == empty_rank:
            continue
        n = int(rng.integers(cap // 2, cap + 1))
        counts = rng.multinomial(n, rng.dirichlet(np.full(experts, 0.3)))  # skewed: some experts get nothing
        offsets[r, 1:] = np.cumsum(counts)
    return rows, offsets


def expected(rows, offsets, local_experts):
    ranks, cap, hidden = rows.shape
    experts = offsets.shape[1] - 1
    res = np.zeros((ranks, cap, hidden), dtype=np.float32)
    ranges = np.zeros((ranks, local_experts + 1), dtype=np.int32)
    for r in range(ranks):
        for e in range(experts):
            lo, hi = offsets[r, e], offsets[r, e + 1]
            res[r, lo:hi] = rows[r, lo:hi].astype(np.float32) * np.float32(e + 1)
            ranges[e // local_experts, e % local_experts + 1] += hi - lo
    return res, np.cumsum(ranges, axis=1, dtype=np.int32)


@pytest.mark.parametrize("ranks,local_experts,hidden,cap", [(1, 8, 64, 96), (2, 4, 128, 160), (4, 16, 256, 200), (8, 3, 64, 50)])
def test_rows_reach_their_experts_and_come_back_in_place(mk, ranks, local_experts, hidden, cap):
    ops = importlib.import_module("macllm_infer_b200.ops")
    rng = np.random.default_rng(ranks * 100 + local_experts)
    rows, offsets = make_case(rng, ranks, local_experts, hidden, cap, empty_rank=ranks - 1 if ranks > 2 else -1)
    want, want_ranges = expected(rows, offsets, local_experts)
    for exchanges in (1, 3):  # three in a row: both buffers of the double-buffered areas, and the first one again
        got, ranges, status = ops.ep_exchange_emulated(rows, offsets, local_experts, exchanges=exchanges)
        assert not status.any(), [hex(int(s)) for s in status]
        assert np.array_equal(ranges, want_ranges)
        for r in range(ranks):
            n = offsets[r, -1]
            assert np.array_equal(got[r, :n], want[r, :n]), (r, exchanges)


def test_a_rank_that_never_sends_ends_the_waits_with_a_status(mk):
    """Nothing sets the silent rank's flags: the other ranks' waits give up after their limit (2 ms here), name the peer in
    the status word and publish empty row ranges, and the device stays usable."""
    ops = importlib.import_module("macllm_infer_b200.ops")
    rng = np.random.default_rng(9)
    rows, offsets = make_case(rng, 3, 4, 64, 40)
    _, ranges, status = ops.ep_exchange_emulated(rows, offsets, 4, silent_rank=1, wait_ns=2_000_000)
    assert int(status[0]) == 0x4550000 | 1 and int(status[2]) == 0x4550000 | 1 and int(status[1]) == 0
    assert not ranges[0].any() and not ranges[2].any()
    # the same device runs the next exchange normally
    got, _, status = ops.ep_exchange_emulated(rows, offsets, 4)
    want, _ = expected(rows, offsets, 4)
    assert not status.any()
    assert all(np.array_equal(got[r, :offsets[r, -1]], want[r, :offsets[r, -1]]) for r in range(3))
