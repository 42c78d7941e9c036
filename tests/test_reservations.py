"""The model boundary's reservation rules on the host-only model, through the C ABI (mk_reserve_batch,
mk_forward_batch_reserved, mk_reservation_drop, mk_session_clear): the known answers of the reference's decoder and pool tests
for reservations that outlive a call (src/decoder.rs:9142-9223,9439-9523; crates/macllm-kv/src/cache.rs:5157-5224).  No GPU."""
import ctypes as C
import importlib

import pytest


@pytest.fixture(scope="module")
def eng(mk):
    return importlib.import_module("macllm_infer_b200.engine")


@pytest.fixture(scope="module")
def capi(mk):
    return importlib.import_module("macllm_infer_b200._capi")


def reserve(capi, model, lanes):
    arr, keep = model._lanes(lanes)
    r = C.c_void_p()
    st = capi.lib().mk_reserve_batch(model._h, arr, len(lanes), C.byref(r))
    return st, r, (arr, keep)


def last_error(capi):
    return capi.lib().mk_last_error().decode()


def test_a_reservation_refuses_swapped_lanes_and_unlocks_the_tables(eng, capi):
    """decoder.rs:9142-9190: a reservation made for (first, second) is handed to a forward of (second, first): refused with the
    reference's wording, both sessions stay empty, and - the reservation being consumed and rolled back - the same two lanes in
    order run as an ordinary forward afterwards."""
    model = eng.Model.fake(vocab=32)
    first, second = model.new_session(), model.new_session()
    st, r, _ = reserve(capi, model, [(first, [1], 0), (second, [2], 0)])
    assert st == 0
    swapped, keep = model._lanes([(second, [2], 0), (first, [1], 0)])
    st = capi.lib().mk_forward_batch_reserved(model._h, swapped, 2, r, capi.FWD_WANT_TOKENS)
    assert st != 0 and "paged KV reservation lane 0 does not match session, order, start or token count" in last_error(capi)
    assert len(first) == 0 and len(second) == 0
    assert model.pool_stats()["reserved_blocks"] == 0
    _, tokens = model.forward_batch([(first, [1], 0), (second, [2], 0)], want_logits=False)
    assert list(tokens) == [(31 * 1 + 3) % 32, (31 * 2 + 3) % 32]
    assert len(first) == 1 and len(second) == 1


def test_an_open_reservation_blocks_its_table_until_it_is_dropped(eng, capi):
    """cache.rs:5202-5224: while a reservation is open, clearing the session empties it but a new reservation on it is refused;
    dropping the open one rolls it back (nothing reserved, the block free again) and unlocks the table."""
    model = eng.Model.fake(vocab=32, block_tokens=2, slab_blocks=1, kv_capacity_tokens=2)
    s = model.new_session()
    st, r, _ = reserve(capi, model, [(s, [1], 0)])
    assert st == 0 and model.pool_stats()["reserved_blocks"] == 1
    s.clear()
    assert len(s) == 0 and len(s.block_table()[0]) == 0
    st2, _, _ = reserve(capi, model, [(s, [1], 0)])
    assert st2 != 0 and st2 != capi.MK_KV_EXHAUSTED
    assert model.pool_stats()["reserved_blocks"] == 1
    capi.check(capi.lib().mk_reservation_drop(r))
    stats = model.pool_stats()
    assert stats["reserved_blocks"] == 0 and stats["free_blocks"] == stats["allocated_blocks"]
    st3, r3, _ = reserve(capi, model, [(s, [1], 0)])
    assert st3 == 0
    capi.check(capi.lib().mk_reservation_drop(r3))


def test_a_completed_clear_releases_a_single_block_pool_for_a_peer(eng, capi):
    """decoder.rs:9191-9223: a pool of one 16-token block. The first session takes it; the second is told how little is free (the
    boundary's wording, src/architecture.rs:938-950) and stays empty; once the first session is cleared the block is free and
    the second session runs."""
    model = eng.Model.fake(vocab=32, block_tokens=16, slab_blocks=1, kv_capacity_tokens=16)
    first, second = model.new_session(), model.new_session()
    model.forward_batch([(first, [1], 0)])
    assert model.pool_stats()["live_blocks"] == 1
    with pytest.raises(capi.KvExhausted, match=r"KV cache requires 1 additional blocks, but only 0 of 1 are free \(0 retired, 16 tokens/block\)"):
        model.forward_batch([(second, [2], 0)])
    assert len(second) == 0
    first.clear()
    stats = model.pool_stats()
    assert stats["live_blocks"] == 0 and stats["free_blocks"] == 1
    model.forward_batch([(second, [2], 0)])
    assert len(second) == 1


def test_a_session_of_another_model_is_refused_without_mutating_it(eng, capi):
    """decoder.rs:9498-9523."""
    model, other = eng.Model.fake(vocab=32), eng.Model.fake(vocab=32)
    foreign = other.new_session()
    other.forward_batch([(foreign, [1, 2], 0)])
    table = [list(map(int, part)) for part in foreign.block_table()]
    st, _, _ = reserve(capi, model, [(foreign, [3], 2)])
    assert st != 0 and st != capi.MK_KV_EXHAUSTED and "decoder session belongs to a different model instance" in last_error(capi)
    assert len(foreign) == 2 and [list(map(int, part)) for part in foreign.block_table()] == table
    assert model.pool_stats()["allocated_blocks"] == 0


def test_interleaved_sessions_are_independent_and_closing_one_does_not_touch_its_peer(eng, capi):
    """decoder.rs:9459-9497: two sessions advance in turns; closing one gives its pages back and leaves the other's table and
    next token as they were."""
    model = eng.Model.fake(vocab=32, block_tokens=2)
    a, b = model.new_session(), model.new_session()
    model.forward_batch([(a, [1, 2, 3], 0)])
    model.forward_batch([(b, [4], 0)])
    model.forward_batch([(a, [5], 3)])
    before = [list(map(int, part)) for part in b.block_table()]
    live = model.pool_stats()["live_blocks"]
    a.close()
    assert model.pool_stats()["live_blocks"] == live - 2
    assert [list(map(int, part)) for part in b.block_table()] == before and len(b) == 1
    _, tokens = model.forward_batch([(b, [6], 1)], want_logits=False)
    assert list(tokens) == [(31 * 6 + 7 * 1 + 3) % 32]


def test_clearing_a_session_is_a_no_op_while_its_reservation_is_open(eng, capi):
    """PagedKvBlockTable::clear returns at once while a reservation is in flight (cache.rs:1840-1852) and the session keeps its
    length in step with its table (decoder.rs:3804-3818): nothing is lost from under a forward that was already planned."""
    model = eng.Model.fake(vocab=32, block_tokens=2)
    s = model.new_session()
    model.forward_batch([(s, [1, 2, 3], 0)])
    table = [list(map(int, part)) for part in s.block_table()]
    st, r, _ = reserve(capi, model, [(s, [4], 3)])
    assert st == 0
    s.clear()
    assert len(s) == 3 and [list(map(int, part)) for part in s.block_table()] == table
    capi.check(capi.lib().mk_reservation_drop(r))
    s.clear()
    assert len(s) == 0 and len(s.block_table()[0]) == 0
    assert model.pool_stats()["live_blocks"] == 0


def test_prefill_then_decode_advances_the_cache(eng, capi):
    """prefill_then_decode_advances_cache (decoder.rs:8906-8930): a token outside the vocabulary is refused before anything is
    cached; three prompt tokens, then one more at position 3; the same token at position 0 again is refused; clear empties."""
    model = eng.Model.fake(vocab=32)
    s = model.new_session()
    with pytest.raises(capi.MkError, match="outside the model vocabulary"):
        model.forward_batch([(s, [32], 0)])
    assert len(s) == 0
    logits, _ = model.forward_batch([(s, [1, 2, 3], 0)])
    assert logits.shape == (1, 32) and len(s) == 3
    model.forward_batch([(s, [4], 3)])
    assert len(s) == 4
    with pytest.raises(capi.MkError, match="start_pos 0 does not match decoder sequence length 4"):
        model.forward_batch([(s, [4], 0)])
    assert len(s) == 4
    s.clear()
    assert len(s) == 0
