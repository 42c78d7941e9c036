"""Exact-token prefix cache parity: the reference's known answers (crates/macllm-kv/src/prefix_cache.rs
tests) against the oracle restatement and the product's host library, plus a randomised differential."""
import hashlib
import importlib
import random

import pytest

GOLDEN = bytes([234, 223, 154, 217, 54, 25, 155, 93, 168, 35, 250, 114, 218, 228, 3, 17, 159, 115, 165, 90, 62, 133, 54, 226,
                28, 250, 17, 165, 115, 7, 250, 146])


@pytest.fixture(scope="module")
def pkv(mk):
    return importlib.import_module("macllm_infer_b200.kv")


def test_sha256_known_answers(pkv):
    for msg in (b"", b"abc", b"abcdbcdecdefdefgefghfghighijhijkijkljklmklmnlmnomnopnopq", bytes(range(256)) * 5):
        assert pkv.sha256(msg) == hashlib.sha256(msg).digest()
    assert pkv.sha256(b"abc").hex() == "ba7816bf8f01cfea414140de5dae2223b00361a396177a9cb410ff61f20015ad"


def test_hash_has_the_reference_golden_value():
    """prefix_cache.rs:1010-1018: hash_endpoint([0x01020304, 5, 6, 7, 8], 4)."""
    from oracle import kv
    assert kv.endpoint_digest([0x01020304, 5, 6, 7, 8], 5, 4) == GOLDEN


def test_product_block_digests_chain_like_the_oracle(pkv):
    from oracle import kv
    toks = [0x01020304, 5, 6, 7, 8, 9, 10, 11, 12]
    assert pkv.block_digests(4, toks) == kv.full_block_digests(toks, 4)
    # the golden endpoint is a partial block chained on the first full block
    first = pkv.block_digests(4, toks)[0]
    assert kv.hash_block(first, 4, 1, [8]) == GOLDEN


class OracleCache:
    def __init__(self, bt, cap):
        from oracle import kv
        self.c = kv.PrefixCache(bt, cap)

    def insert(self, tokens, value, cost):
        ev = self.c.insert(tokens, value, cost)
        return None if ev is None else list(ev)

    def lookup(self, tokens):
        return self.c.lookup_aligned_common_prefix(tokens, len(tokens))

    def evict(self):
        return self.c.evict_lru()

    def stats(self):
        return self.c.stats()

    def lookup_exact(self, tokens, limit=None):
        return self.c.lookup(tokens, limit)

    def lookup_aligned(self, tokens, limit=None):
        hit = self.c.lookup_aligned_common_prefix(tokens, limit)
        if hit is None:
            return None
        owner = next(e for e in self.c.entries.values() if e.snapshot == hit[1])
        return hit[0], len(owner.tokens), hit[1]

    def set_max_cost(self, cost):
        return self.c.set_max_cost(cost)

    def force_collisions(self):
        self.c.force_collisions()


class ProductCache:
    def __init__(self, bt, cap):
        self.kv = importlib.import_module("macllm_infer_b200.kv")
        self.capi = importlib.import_module("macllm_infer_b200._capi")
        self.c = self.kv.PrefixCache(bt, cap)

    def insert(self, tokens, value, cost):
        try:
            return self.c.insert(tokens, value, cost)
        except self.capi.MkError:
            return None

    def lookup(self, tokens):
        return self.c.lookup(tokens)

    def evict(self):
        return self.c.evict_lru()

    def stats(self):
        return self.c.stats()

    def lookup_exact(self, tokens, limit=None):
        return self.c.lookup_exact(tokens, limit)

    def lookup_aligned(self, tokens, limit=None):
        return self.c.lookup_aligned(tokens, limit)

    def set_max_cost(self, cost):
        return self.c.set_max_cost(cost)

    def force_collisions(self):
        self.c.force_collisions()


@pytest.fixture(params=["oracle", "product"])
def Cache(request, mk):
    return {"oracle": OracleCache, "product": ProductCache}[request.param]


def test_aligned_lookup_reuses_a_long_snapshot_before_a_divergent_suffix(Cache):
    """prefix_cache.rs:773-792."""
    c = Cache(4, 20)
    c.insert(list(range(1, 13)), 7, 7)
    assert c.lookup([1, 2, 3, 4, 5, 6, 99, 100]) == (4, 7)
    assert c.lookup([1, 2, 3, 4, 5, 6, 7, 8, 9, 77, 78]) == (8, 7)


def test_aligned_lookup_strict_bounds(Cache):
    """prefix_cache.rs:795-821."""
    c = Cache(4, 20)
    c.insert(list(range(1, 13)), 1, 1)
    assert c.lookup([1, 2, 3, 4, 5, 6]) == (4, 1)
    assert c.lookup([1, 2, 3, 4]) is None          # an aligned endpoint equal to the prompt is not reusable
    assert c.lookup([0, 1, 2, 3, 4, 5, 6]) is None  # a substring is not a prefix
    s = c.stats()
    assert (s["hits"], s["misses"], s["matched_tokens"]) == (1, 2, 4)


def test_aligned_block_indexes_follow_replacement_and_lru_eviction(Cache):
    """prefix_cache.rs:932-957."""
    c = Cache(4, 2)
    c.insert([1] * 5, 10, 1)
    c.insert([2] * 5, 20, 1)
    assert c.lookup([1, 1, 1, 1, 9]) == (4, 10)
    assert c.insert([3] * 5, 30, 1) == [20]         # LRU is "second": "first" was just touched
    assert c.lookup([2, 2, 2, 2, 9]) is None
    assert c.insert([1] * 5, 11, 1) == []           # replacement is not an eviction
    assert c.lookup([1, 1, 1, 1, 9]) == (4, 11)
    assert c.evict() == 30
    assert c.lookup([3, 3, 3, 3, 9]) is None
    assert c.stats()["evictions"] == 2


def test_insert_evicts_lru_until_the_budget_fits_and_rejects_oversize(Cache):
    """prefix_cache.rs:915-929,181-195."""
    c = Cache(1, 5)
    c.insert([1, 7], 1, 2)
    c.insert([2, 7], 2, 2)
    assert c.lookup([1, 7, 0]) == (2, 1)
    assert c.insert([3, 7], 3, 3) == [2]
    s = c.stats()
    assert (s["entries"], s["cached_blocks"], s["evictions"]) == (2, 5, 1)
    assert c.insert([4, 7], 4, 6) is None           # cost above the budget
    assert c.stats()["entries"] == 2


def test_most_recently_used_enclosing_snapshot_wins(Cache):
    """prefix_cache.rs:341-351."""
    c = Cache(2, 10)
    c.insert([1, 2, 3, 4, 5, 6], 100, 1)
    c.insert([1, 2, 3, 4, 9, 9], 200, 1)
    assert c.lookup([1, 2, 3, 4, 0]) == (4, 200)
    assert c.lookup([1, 2, 3, 4, 5, 6, 0]) == (6, 100)
    assert c.lookup([1, 2, 3, 4, 0]) == (4, 100)   # the last hit made 100 the most recent


def test_randomised_differential(mk):
    for seed in range(5):
        rng = random.Random(seed)
        bt = rng.choice([2, 4, 16])
        a, b = OracleCache(bt, 12), ProductCache(bt, 12)
        stems = [[rng.randrange(5) for _ in range(rng.randint(1, 6 * bt))] for _ in range(6)]
        for step in range(400):
            stem = rng.choice(stems)
            toks = stem[: rng.randint(1, len(stem))] + [rng.randrange(5) for _ in range(rng.randint(0, 3))]
            op = rng.random()
            if op < 0.4:
                cost = rng.randint(0, 5)
                assert a.insert(toks, step, cost) == b.insert(toks, step, cost), (seed, step)
            elif op < 0.9:
                assert a.lookup(toks) == b.lookup(toks), (seed, step)
            else:
                assert a.evict() == b.evict(), (seed, step)
            assert a.stats() == b.stats(), (seed, step)


def test_two_snapshots_with_different_first_blocks_are_told_apart(Cache):
    """prefix_cache.rs:824-846 (there with every block digest forced to collide; here the digests differ, the answers are
    the same): the aligned common prefix of each prompt is found under its own snapshot, a third prompt matches neither."""
    c = Cache(4, 20)
    c.insert([1, 2, 3, 4, 5, 6, 7, 8, 10], 1, 1)
    c.insert([9, 8, 7, 6, 5, 4, 3, 2, 10], 2, 1)
    assert c.lookup([1, 2, 3, 4, 5, 6, 7, 8, 99]) == (8, 1)
    assert c.lookup([9, 8, 7, 6, 5, 4, 3, 2, 99]) == (8, 2)
    assert c.lookup([4, 4, 4, 4, 4, 4, 4, 4, 0]) is None


def test_refused_insertions_leave_the_cache_empty(Cache):
    """prefix_cache.rs:686-702: an empty prefix and a cost above the budget are refused."""
    c = Cache(4, 3)
    assert c.insert([], 0, 0) is None
    assert c.insert([1], 0, 4) is None
    s = c.stats()
    assert (s["entries"], s["cached_blocks"], s["evictions"]) == (0, 0, 0)


def test_endpoint_digest_is_independent_of_how_the_prefix_is_cut(pkv):
    """prefix_cache.rs:1001-1008: the digest of the first n tokens is the chain of the full blocks and one partial block,
    whichever way the prompt was walked; the product's chained block digests are that chain's full-block links."""
    from oracle import kv
    tokens = [10, 20, 30, 40, 50, 60, 70]
    full = kv.full_block_digests(tokens, 4)
    assert pkv.block_digests(4, tokens) == full
    for n in range(1, len(tokens) + 1):
        whole, rest = divmod(n, 4)
        chained = (b"\0" * 32 if whole == 0 else full[whole - 1]) if rest else None
        want = full[whole - 1] if rest == 0 else kv.hash_block(chained, 4, whole, tokens[4 * whole:n])
        assert kv.endpoint_digest(tokens, n, 4) == want, n


def test_hit_refreshes_lru_and_explicit_eviction_returns_the_oldest(Cache):
    """prefix_cache.rs:898-913 (there through the exact-endpoint lookup; one-token blocks make the aligned lookup ask the
    same question): the hit on "one" makes "two" the oldest."""
    c = Cache(1, 10)
    c.insert([1], 1, 1)
    c.insert([2], 2, 2)
    c.insert([3], 3, 3)
    assert c.lookup([1, 9]) == (1, 1)
    assert c.evict() == 2
    s = c.stats()
    assert (s["evictions"], s["entries"], s["cached_blocks"]) == (1, 2, 4)


def test_stats_count_each_lookup_once_and_accumulate_matched_tokens(Cache):
    """prefix_cache.rs:975-999, asked through the aligned lookup: the two-token match is served by the most recently used
    snapshot that encloses it (prefix_cache.rs:341-351), which is "three" after the first hit; the counters are the reference's."""
    c = Cache(1, 10)
    c.insert([1, 2], 2, 1)
    c.insert([1, 2, 3], 3, 1)
    assert c.lookup([1, 2, 3, 4]) == (3, 3)
    assert c.lookup([1, 2, 9]) == (2, 3)
    assert c.lookup([8, 8, 8]) is None
    s = c.stats()
    assert (s["hits"], s["misses"], s["matched_tokens"], s["entries"], s["cached_blocks"], s["evictions"]) == (2, 1, 5, 2, 2, 0)


def test_empty_and_tiny_prompts_are_misses(Cache):
    """prefix_cache.rs:1020-1030: an empty prompt and a prompt no longer than the stored prefix (at least one token must be
    left to compute) miss, and each miss is counted."""
    c = Cache(1, 10)
    c.insert([1], 1, 1)
    assert c.lookup([]) is None
    assert c.lookup([1]) is None
    assert c.lookup([2, 1]) is None
    assert c.stats()["misses"] == 3 and c.stats()["hits"] == 0


# ---- the exact-endpoint lookup (prefix_cache.rs:250-304), the lookup of models whose state restores only where it was saved ----

def test_returns_the_longest_exact_prefix_from_absolute_zero(Cache):
    """prefix_cache.rs:723-739."""
    c = Cache(4, 10)
    c.insert([1, 2], 2, 1)
    c.insert([1, 2, 3], 3, 1)
    c.insert([1, 2, 3, 4], 4, 1)
    assert c.lookup_exact([1, 2, 3, 4, 9], 5) == (4, 4)
    assert c.lookup_exact([0, 1, 2, 3, 4, 9], 6) is None        # a matching substring is not a prefix


def test_excludes_the_prompt_and_maximum_limit_endpoints(Cache):
    """prefix_cache.rs:741-758."""
    c = Cache(4, 10)
    c.insert([1, 2, 3], 3, 1)
    c.insert([1, 2, 3, 4], 4, 1)
    assert c.lookup_exact([1, 2, 3, 4]) == (3, 3)               # the full prompt endpoint stays uncached
    assert c.lookup_exact([1, 2, 3, 4, 5], 4) == (3, 3)         # the supplied maximum is exclusive too
    assert c.lookup_exact([1, 2, 3], 3) is None


def test_backs_off_from_a_candidate_that_fails_exact_verification(Cache):
    """prefix_cache.rs:760-770."""
    c = Cache(4, 10)
    c.insert([7, 8], 1, 1)
    c.insert([7, 8, 9, 10], 2, 1)
    assert c.lookup_exact([7, 8, 99, 10, 11], 5) == (2, 1)


def test_aligned_lookup_handles_shorter_prompts_and_strict_bounds(Cache):
    """prefix_cache.rs:795-821, with the maximum-token bound."""
    c = Cache(4, 20)
    c.insert(list(range(1, 13)), 7, 1)
    assert c.lookup_aligned([1, 2, 3, 4, 5, 6], 6) == (4, 12, 7)     # a shorter prompt may fork an enclosing snapshot
    assert c.lookup_aligned([1, 2, 3, 4, 5, 6], 4) is None           # the bound is exclusive
    assert c.lookup_aligned([1, 2, 3, 4]) is None                    # an aligned endpoint equal to the prompt is not reusable
    assert c.lookup_aligned([0, 1, 2, 3, 4, 5, 6], 7) is None        # a substring is not a prefix


def test_exact_tokens_defeat_injected_digest_collisions(Cache):
    """prefix_cache.rs:824-865: with every digest forced to the same value the answers still come from the tokens."""
    c = Cache(4, 20)
    c.force_collisions()
    c.insert([1, 2, 3, 4, 5, 6, 7, 8, 10], 1, 1)
    c.insert([9, 8, 7, 6, 5, 4, 3, 2, 10], 2, 1)
    assert c.lookup_aligned([1, 2, 3, 4, 5, 6, 7, 8, 99], 9) == (8, 9, 1)
    assert c.lookup_aligned([9, 8, 7, 6, 5, 4, 3, 2, 99], 9) == (8, 9, 2)
    assert c.lookup_aligned([4, 4, 4, 4, 4, 4, 4, 4, 0], 9) is None
    c = Cache(4, 10)
    c.force_collisions()
    c.insert([1, 2, 3], 1, 1)
    c.insert([9, 8, 7], 2, 1)
    assert c.lookup_exact([1, 2, 3, 4], 4) == (3, 1)
    assert c.lookup_exact([9, 8, 7, 6], 4) == (3, 2)
    assert c.lookup_exact([5, 5, 5, 0], 4) is None


def test_replacement_is_exact_even_inside_a_collision_bucket(Cache):
    """prefix_cache.rs:866-896: the same tokens replace their own entry and nothing else; a replacement is not an eviction."""
    c = Cache(4, 10)
    c.force_collisions()
    c.insert([1, 2], 1, 2)
    c.insert([8, 9], 2, 2)
    assert c.insert([1, 2], 3, 3) == []
    s = c.stats()
    assert (s["entries"], s["cached_blocks"], s["evictions"]) == (2, 5, 0)
    assert c.lookup_exact([1, 2, 3], 3) == (2, 3)
    assert c.lookup_exact([8, 9, 0], 3) == (2, 2)


def test_shrinking_budget_and_zero_cost_entries_are_supported(Cache):
    """prefix_cache.rs:959-973."""
    c = Cache(4, 10)
    c.insert([1], 1, 4)
    c.insert([2], 2, 3)
    c.insert([3], 3, 0)
    assert len(c.set_max_cost(3)) == 1
    s = c.stats()
    assert (s["cached_blocks"], s["entries"]) == (3, 2)
    assert len(c.set_max_cost(0)) == 1
    s = c.stats()
    assert (s["cached_blocks"], s["entries"]) == (0, 1)
    assert c.lookup_exact([3, 0], 2) == (1, 3)


def test_empty_and_tiny_bounds_are_misses_on_the_exact_lookup(Cache):
    """prefix_cache.rs:1020-1030 as written there."""
    c = Cache(4, 10)
    c.insert([1], 1, 1)
    assert c.lookup_exact([], 100) is None
    assert c.lookup_exact([1, 2], 0) is None
    assert c.lookup_exact([1, 2], 1) is None
    assert c.stats()["misses"] == 3
