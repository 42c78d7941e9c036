"""Paged-KV pool parity: the reference's own known-answer cases (crates/macllm-kv/src/cache.rs tests)
run against BOTH the oracle restatement and the product's host library, then a randomised differential
between the two.  CPU only."""
import random

import pytest

from kvadapters import OraclePool, ProductPool

IMPLS = {"oracle": OraclePool, "product": ProductPool}


@pytest.fixture(params=list(IMPLS))
def Pool(request, mk):
    return IMPLS[request.param]


def sub(stats, *keys):
    return tuple(stats[k] for k in keys)


def test_compact_page_table_of_two_lanes(Pool):
    """cache.rs:4898-4977: pool(block_tokens 2, slab_blocks 2, max 4), lanes of 3 and 1 tokens."""
    pool = Pool(2, 2, 4)
    first, second = pool.new_table(), pool.new_table()
    pages, offsets, counts, lens = pool.page_table([first, second], [3, 1])
    assert [list(p) for p in pages] == [[0, 0], [0, 1], [1, 0]]
    assert list(offsets) == [0, 2] and list(counts) == [2, 1] and list(lens) == [3, 1]


def test_shared_full_prefix_appends_on_a_fresh_page(Pool):
    """cache.rs:4585-4630."""
    pool = Pool(4, 2, 2)
    source = pool.new_table()
    assert pool.append([source], [4]) == []
    pool.complete(pool.submitted())
    source_id = source.blocks()[0]
    fork = source.fork_prefix(4)
    assert pool.append([fork], [1]) == []          # no copy-on-write: the shared page is full
    assert source.blocks() == [source_id]
    assert fork.blocks()[0] == source_id and fork.blocks()[1] != source_id
    assert sub(pool.stats(), "live_blocks", "live_references", "shared_blocks") == (2, 3, 1)


def test_shared_partial_prefix_copies_on_write(Pool):
    """cache.rs:4632-4693."""
    pool = Pool(4, 2, 2)
    source = pool.new_table()
    pool.append([source], [4])
    pool.complete(pool.submitted())
    source_id = source.blocks()[0]
    fork = source.fork_prefix(2)
    cows = pool.append([fork], [1])
    assert len(cows) == 1 and cows[0][0] == source_id[0] and cows[0][2] == 2
    assert source.blocks() == [source_id]
    assert fork.blocks()[0] != source_id and fork.blocks()[0][0] == cows[0][1]
    assert sub(pool.stats(), "live_blocks", "live_references", "shared_blocks") == (2, 2, 0)


def test_batch_cows_two_lanes_sharing_one_partial_tail(Pool):
    """cache.rs:4695-4747."""
    pool = Pool(4, 3, 3)
    source = pool.new_table()
    pool.append([source], [2])
    pool.complete(pool.submitted())
    source_id = source.blocks()[0]
    first, second = source.fork_prefix(2), source.fork_prefix(2)
    assert pool.stats()["live_references"] == 3
    cows = pool.append([first, second], [1, 1])
    assert [c[0] for c in cows] == [source_id[0]] * 2 and [c[2] for c in cows] == [2, 2]
    assert source.blocks() == [source_id]
    assert first.blocks()[0] != source_id and second.blocks()[0] != source_id and first.blocks()[0] != second.blocks()[0]
    assert sub(pool.stats(), "live_blocks", "live_references", "shared_blocks") == (3, 3, 0)


def test_exhaustion_mutates_nothing(Pool):
    """cache.rs:4802-4830, 5130-5156: a batch that does not fit leaves stats and epochs untouched."""
    pool = Pool(2, 2, 3)
    a, b = pool.new_table(), pool.new_table()
    assert pool.append([a], [4]) == []
    before = pool.stats()
    assert pool.append([a, b], [1, 4]) is None
    assert pool.stats() == before
    assert len(a) == 4 and len(b) == 0


def test_clear_retires_until_completion_then_reuses_with_new_generation(Pool):
    """cache.rs:5404-5449."""
    pool = Pool(2, 2, 2)
    t = pool.new_table()
    pool.append([t], [3])
    first_ids = t.blocks()
    epoch = pool.submitted()
    t.clear()                                        # device work of `epoch` may still read the pages
    assert sub(pool.stats(), "retired_blocks", "free_blocks", "live_blocks") == (2, 0, 0)
    u = pool.new_table()
    assert pool.append([u], [1]) is None            # nothing is free while the pages are quarantined
    pool.complete(epoch)
    assert sub(pool.stats(), "retired_blocks", "free_blocks") == (0, 2)
    assert pool.append([u], [1]) == []
    (slot, gen), = u.blocks()
    assert slot == first_ids[0][0] and gen == first_ids[0][1] + 1


def test_fork_retains_pages_until_last_owner_releases(Pool):
    """cache.rs:4443-4474."""
    pool = Pool(2, 4, 4)
    source = pool.new_table()
    pool.append([source], [4])
    pool.complete(pool.submitted())
    fork = source.fork_prefix(3)
    assert sub(pool.stats(), "live_blocks", "live_references", "shared_blocks") == (2, 4, 2)
    source.clear()
    assert sub(pool.stats(), "live_blocks", "live_references", "shared_blocks", "free_blocks") == (2, 2, 0, 2)
    fork.clear()
    assert sub(pool.stats(), "live_blocks", "free_blocks") == (0, 4)


def test_zero_growth_batch_still_takes_an_epoch(Pool):
    """cache.rs:5010-5043: appending into a partial page reserves nothing but opens a transaction."""
    pool = Pool(4, 2, 2)
    t = pool.new_table()
    pool.append([t], [1])
    e1 = pool.submitted()
    pool.complete(e1)
    assert pool.append([t], [2]) == []
    assert pool.submitted() == e1 + 1
    assert len(t.blocks()) == 1 and len(t) == 3


def test_randomised_differential_oracle_vs_product(mk):
    """Same random operation sequence on both implementations: block ids (slot, generation), stats,
    copy-on-write plans and exhaustion decisions must agree at every step."""
    for seed in range(6):
        rng = random.Random(seed)
        bt, slab, mx = rng.choice([(2, 2, 9), (4, 3, 12), (16, 8, 24)])
        pools = [OraclePool(bt, slab, mx), ProductPool(bt, slab, mx)]
        tables = [[], []]
        for step in range(300):
            op = rng.random()
            n_tab = len(tables[0])
            if op < 0.15 or n_tab == 0:
                for i, p in enumerate(pools):
                    tables[i].append(p.new_table())
            elif op < 0.55:
                k = rng.randint(1, min(3, n_tab))
                idx = rng.sample(range(n_tab), k)
                ns = [rng.randint(1, 2 * bt + 1) for _ in idx]
                commit = rng.random() < 0.85
                outs = [p.append([tables[i][j] for j in idx], ns, commit) for i, p in enumerate(pools)]
                assert outs[0] == outs[1], (seed, step)
            elif op < 0.7:
                j = rng.randrange(n_tab)
                length = len(tables[0][j])
                if length:
                    n = rng.randint(0, length)
                    for i in range(2):
                        tables[i].append(tables[i][j].fork_prefix(n))
            elif op < 0.85:
                j = rng.randrange(n_tab)
                for i in range(2):
                    tables[i][j].clear()
            else:
                e = pools[0].submitted()
                for p in pools:
                    p.complete(e)
            assert pools[0].stats() == pools[1].stats(), (seed, step)
            for a, b in zip(tables[0], tables[1]):
                assert a.blocks() == b.blocks() and len(a) == len(b), (seed, step)
        for i in range(2):
            for t in tables[i]:
                t.free()


# ---- further known answers of the reference's pool tests (cache.rs; pool(layers, heads, dim, block_tokens, slab_blocks,
# max_blocks) there = Pool(block_tokens, slab_blocks, max_blocks) here)

def test_partial_tail_cow_rollback_quarantines_only_the_replacement(Pool):
    """cache.rs:4750-4799: a fork that shares a partial tail reserves a replacement page, the forward touches it and
    fails: source and fork keep the shared page, only the replacement waits for its epoch."""
    pool = Pool(4, 2, 2)
    source = pool.new_table()
    pool.append([source], [4])
    pool.complete(pool.submitted())
    source_id = source.blocks()[0]
    fork = source.fork_prefix(2)
    failed = pool.append_touch_rollback([fork], [1])
    assert source.blocks() == [source_id] and fork.blocks() == [source_id]
    assert len(source) == 4 and len(fork) == 2
    assert sub(pool.stats(), "live_blocks", "live_references", "shared_blocks", "retired_blocks", "free_blocks") == (1, 2, 1, 1, 0)
    pool.complete(failed)
    assert sub(pool.stats(), "live_blocks", "free_blocks", "retired_blocks") == (1, 1, 0)


def test_second_lane_exhaustion_is_atomic(Pool):
    """cache.rs:5130-5155: two lanes that together need three blocks of a two-block pool: nothing is taken."""
    pool = Pool(2, 1, 2)
    first, second = pool.new_table(), pool.new_table()
    before = pool.stats()
    assert pool.append([first, second], [2, 3]) is None
    assert pool.stats() == before
    assert len(first) == 0 and first.blocks() == [] and len(second) == 0 and second.blocks() == []


def test_exhaustion_does_not_publish_an_epoch(Pool):
    """cache.rs:5334-5355."""
    pool = Pool(2, 1, 1)
    owner, waiter = pool.new_table(), pool.new_table()
    pool.append([owner], [1])
    before = pool.stats()
    assert before["submitted_epoch"] == pool.submitted() == 1
    assert pool.append([waiter], [1]) is None
    assert pool.stats() == before and len(waiter) == 0 and waiter.blocks() == []


def test_two_lanes_commit_in_one_epoch(Pool):
    """cache.rs:4832-4896: one reservation, one epoch, both tables advance."""
    pool = Pool(2, 2, 4)
    first, second = pool.new_table(), pool.new_table()
    assert pool.append([first, second], [3, 1]) == []
    assert pool.submitted() == 1 and len(first) == 3 and len(second) == 1
    assert len(first.blocks()) == 2 and len(second.blocks()) == 1
    assert sub(pool.stats(), "live_blocks", "live_references", "reserved_blocks") == (3, 3, 0)


def test_partial_tail_rollback_stays_private_and_retry_reuses_the_page(Pool):
    """cache.rs:5226-5296: growth inside the table's own partial page needs no new block; a failed attempt leaves the table
    as it was, retires nothing, and still publishes its epoch; the retry lands on the same page."""
    pool = Pool(4, 1, 1)
    table = pool.new_table()
    pool.append([table], [2])
    pool.complete(pool.submitted())
    page = table.blocks()
    failed = pool.append_touch_rollback([table], [1])
    assert len(table) == 2 and table.blocks() == page
    s = pool.stats()
    assert sub(s, "live_blocks", "retired_blocks") == (1, 0) and s["submitted_epoch"] == failed
    assert pool.append([table], [1]) == []
    assert len(table) == 3 and table.blocks() == page


def test_touched_history_is_quarantined_when_the_table_is_cleared_after_a_failed_forward(Pool):
    """cache.rs:5045-5070: the failed forward read the table's history; clearing the table afterwards may not hand those
    pages out before the failed epoch completes."""
    pool = Pool(2, 2, 2)
    table = pool.new_table()
    pool.append([table], [3])
    pool.complete(pool.submitted())
    failed = pool.append_touch_rollback([table], [1])
    table.clear()
    assert sub(pool.stats(), "free_blocks", "live_blocks", "retired_blocks") == (0, 0, 2)
    pool.complete(failed)
    assert pool.stats()["free_blocks"] == 2


def test_a_table_twice_in_one_batch_is_refused_without_pool_mutation(Pool):
    """cache.rs:5186-5200."""
    pool = Pool(2, 1, 2)
    table = pool.new_table()
    before = pool.stats()
    with pytest.raises(Exception):
        pool.append([table, table], [1, 1])
    assert pool.stats() == before and len(table) == 0
    assert pool.append([table], [1]) == []          # the table is not left locked


def test_pool_serialises_reservations_in_epoch_order(mk):
    """cache.rs:5104-5127: while one reservation is open a second one is refused and no device completion can be
    published; the next reservation takes the next epoch.  Oracle pool directly; product through the model-level ABI
    (mk_reserve_batch / mk_reservation_drop on the host-only model), where a reservation stays open between calls."""
    import ctypes as C
    import importlib
    from oracle import kv
    p = kv.Pool(2, 2, 2)
    t1, t2 = kv.Table(p), kv.Table(p)
    r1 = p.reserve_batch([t1], [1])
    with pytest.raises(kv.Invalid, match="transaction 1 is still active"):
        p.reserve_batch([t2], [1])
    with pytest.raises(kv.Invalid, match="cannot publish device completion"):
        p.mark_completed_through(r1.epoch)
    assert p.stats()["submitted_epoch"] == r1.epoch == 1
    r1.rollback()
    r2 = p.reserve_batch([t2], [1])
    assert r2.epoch == 2
    r2.rollback()

    eng = importlib.import_module("macllm_infer_b200.engine")
    capi = importlib.import_module("macllm_infer_b200._capi")
    m = eng.Model.fake(vocab=8, block_tokens=2, slab_blocks=2, kv_capacity_tokens=4)
    s1, s2 = m.new_session(), m.new_session()
    lanes1, keep1 = m._lanes([(s1, [1], 0)])
    lanes2, keep2 = m._lanes([(s2, [1], 0)])
    first, second = C.c_void_p(), C.c_void_p()
    assert capi.lib().mk_reserve_batch(m._h, lanes1, 1, C.byref(first)) == 0
    assert capi.lib().mk_reserve_batch(m._h, lanes2, 1, C.byref(second)) < 0
    assert "transaction 1 is still active" in capi.lib().mk_last_error().decode()
    assert m.pool_stats()["submitted_epoch"] == 1
    assert capi.lib().mk_reservation_drop(first) == 0
    assert capi.lib().mk_reserve_batch(m._h, lanes2, 1, C.byref(second)) == 0
    assert m.pool_stats()["submitted_epoch"] == 2
    assert capi.lib().mk_reservation_drop(second) == 0
    s = m.pool_stats()
    assert (s["reserved_blocks"], s["free_blocks"], s["live_blocks"]) == (0, 2, 0)
    del keep1, keep2


def test_attach_prefix_failures_leave_ownership_unchanged(mk):
    """cache.rs:4476-4526: a prefix cannot come from another pool, be longer than its source, or land in a table that
    already owns pages; every refusal leaves the tables and the pool's counters as they were."""
    import importlib
    from oracle import kv
    pkv = importlib.import_module("macllm_infer_b200.kv")
    capi = importlib.import_module("macllm_infer_b200._capi")

    # oracle
    pool = kv.Pool(2, 2, 2)
    source = kv.Table(pool)
    r = pool.reserve_batch([source], [3])
    r.mark_all_used()
    r.commit()
    pool.mark_completed_through(pool.submitted_epoch)
    before = pool.stats()
    foreign = kv.Table(kv.Pool(2, 1, 1))
    too_long, small = kv.Table(pool), kv.Table(pool, limit=2)
    occupied = source.fork_prefix(1)
    shared = pool.stats()
    for table, n in ((foreign, 2), (too_long, 4), (small, 3), (occupied, 1)):
        kept = (table.logical_len, list(table.blocks))
        with pytest.raises(kv.Invalid):
            table.attach_prefix(source, n)
        assert (table.logical_len, list(table.blocks)) == kept
    assert pool.stats() == shared and shared["live_references"] == before["live_references"] + 1

    # product
    ppool = pkv.KvPool(2, 2, 2)
    psource = ppool.new_table()
    ppool.append_batch([psource], [3])
    ppool.complete_epoch(ppool.submitted_epoch())
    pbefore = ppool.stats()
    assert pbefore == before
    pforeign = pkv.KvPool(2, 1, 1).new_table()
    ptoo_long = ppool.new_table()
    poccupied = psource.fork_prefix(1)
    pshared = ppool.stats()
    assert pshared == shared
    for table, n in ((pforeign, 2), (ptoo_long, 4), (poccupied, 1)):
        kept = (len(table), table.blocks())
        with pytest.raises(capi.MkError):
            table.attach_prefix(psource, n)
        assert (len(table), table.blocks()) == kept
    assert ppool.stats() == pshared


def test_pool_rejects_invalid_and_overflowing_geometry(Pool):
    """cache.rs:3940-3951 (PagedKvPoolConfig::new, cache.rs:126-147): each of the three sizes must be positive and the block
    count must fit the 32-bit slot half of a generational block id."""
    for args, what in (((0, 1, 1), "block_tokens"), ((1, 0, 1), "slab_blocks"), ((1, 1, 0), "max_blocks")):
        with pytest.raises(Exception, match=f"invalid paged KV config: {what} must be positive"):
            Pool(*args)
    with pytest.raises(Exception, match="block-ID range"):
        Pool(1, 1, 0xFFFFFFFF + 1)
    Pool(1, 1, 0xFFFFFFFF)      # the largest legal pool is only a number until blocks are taken


def test_occupancy_across_refcount_cow_and_rollback(Pool):
    """cache.rs:3964-4054 (pool of block_tokens 2, slab_blocks 2, max 4): the occupancy figures after a commit, two forks, a
    cleared fork, a copy-on-write append, a touched rollback on a third fork, its epoch's completion, and the release of
    everything."""
    pool = Pool(2, 2, 4)
    source = pool.new_table()
    assert pool.append([source], [3]) == []
    assert sub(pool.stats(), "live_references", "reserved_blocks") == (2, 0)
    pool.complete(pool.submitted())
    first_fork, second_fork = source.fork_prefix(3), source.fork_prefix(3)
    assert sub(pool.stats(), "live_blocks", "live_references", "shared_blocks") == (2, 6, 2)
    first_fork.clear()
    assert sub(pool.stats(), "live_references", "shared_blocks") == (4, 2)
    cows = pool.append([second_fork], [1])                 # the shared half-full tail is replaced, not written
    assert len(cows) == 1 and cows[0][2] == 1
    cow_epoch = pool.submitted()
    assert sub(pool.stats(), "reserved_blocks", "live_blocks", "live_references", "shared_blocks") == (0, 3, 4, 1)
    rolled_back_fork = source.fork_prefix(3)
    failed_epoch = pool.append_touch_rollback([rolled_back_fork], [1])
    assert sub(pool.stats(), "reserved_blocks", "live_blocks", "live_references", "shared_blocks", "retired_blocks") == (0, 3, 6, 2, 1)
    pool.complete(failed_epoch)
    assert pool.stats()["retired_blocks"] == 0
    for t in (source, second_fork, rolled_back_fork):
        t.clear()
    st = pool.stats()
    assert sub(st, "live_blocks", "live_references", "shared_blocks") == (0, 0, 0)
    assert st["free_blocks"] == st["allocated_blocks"] and st["completed_epoch"] >= cow_epoch
