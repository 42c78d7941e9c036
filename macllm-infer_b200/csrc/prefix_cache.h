// Exact-token prefix index: a cost-bounded LRU of snapshots keyed by token prefixes, found through
// chained SHA-256 block digests and always confirmed by an exact token comparison.
// Restates crates/macllm-kv/src/prefix_cache.rs of the reference (TokenPrefixCache :123-547, digest
// format :556-654).
#pragma once
#include "sha256.h"
#include <algorithm>
#include <array>
#include <cstdint>
#include <deque>
#include <map>
#include <optional>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace mk {

using PrefixDigest = std::array<uint8_t, 32>;

struct PrefixDigestHash {
    size_t operator()(const PrefixDigest& d) const {
        size_t h;
        memcpy(&h, d.data(), sizeof h);
        return h;
    }
};

// SHA256(domain || u32le(1) || u32le(block_tokens) || u32le(block_index) || u32le(valid_len) ||
//        previous_digest || u32le tokens...), first previous digest = 32 zero bytes  (:563-586).
inline PrefixDigest prefix_hash_block(const PrefixDigest& previous, uint32_t block_tokens, uint32_t block_index,
                                      const uint32_t* tokens, uint32_t n) {
    static const char domain[] = "macllm-infer/token-prefix";  // plus the terminating NUL
    Sha256 h;
    h.update(domain, sizeof domain);
    h.update_u32le(1);
    h.update_u32le(block_tokens);
    h.update_u32le(block_index);
    h.update_u32le(n);
    h.update(previous.data(), 32);
    for (uint32_t i = 0; i < n; ++i) h.update_u32le(tokens[i]);
    return h.finish();
}

// Digest chain over the full blocks of a prompt, plus partial endpoints on demand (:609-654).
class PromptHashPlan {
public:
    PromptHashPlan(const uint32_t* prompt, size_t maximum_endpoint, size_t block_tokens)
        : prompt_(prompt), bt_(block_tokens) {
        size_t full = maximum_endpoint / block_tokens;
        chains_.reserve(full + 1);
        chains_.push_back(PrefixDigest{});
        for (size_t b = 0; b < full; ++b)
            chains_.push_back(prefix_hash_block(chains_.back(), (uint32_t)bt_, (uint32_t)b, prompt + b * bt_, (uint32_t)bt_));
    }
    PrefixDigest endpoint(size_t token_count) const {
        size_t full = token_count / bt_, rem = token_count % bt_;
        if (rem == 0) return chains_[full];
        return prefix_hash_block(chains_[full], (uint32_t)bt_, (uint32_t)full, prompt_ + full * bt_, (uint32_t)rem);
    }

private:
    const uint32_t* prompt_;
    size_t bt_;
    std::vector<PrefixDigest> chains_;
};

struct PrefixCacheStats {
    uint64_t hits = 0, misses = 0, matched_tokens = 0, evictions = 0, insertions = 0;
    size_t entries = 0, cost = 0, max_cost = 0;
};

template <typename T>
class TokenPrefixCache {
public:
    struct Hit {
        size_t matched_tokens;
        T* snapshot;
        size_t snapshot_tokens;
        size_t cost;
    };
    struct Evicted {
        std::vector<uint32_t> tokens;
        T snapshot;
        size_t cost;
    };

    TokenPrefixCache(size_t block_tokens, size_t max_cost) : bt_(block_tokens), max_cost_(max_cost) {  // :149-175
        if (block_tokens == 0) throw std::runtime_error("prefix-cache block size must be positive");
        if (block_tokens > (size_t)UINT32_MAX) throw std::runtime_error("prefix-cache block size " + std::to_string(block_tokens) + " does not fit the 32-bit hash domain");
    }

    // Every digest of the index becomes the same value: hits must then come from the exact token comparison alone
    // (force_collisions_for_tests of the reference, used by its collision cases :824-897).
    void force_collisions_for_tests() {
        if (!entries_.empty()) throw std::runtime_error("collisions can only be forced on an empty prefix cache");
        forced_ = true;
    }

    // set_max_cost (:395-409): the new budget evicts least recently used snapshots until the cache fits; returns how many.
    size_t set_max_cost(size_t max_cost, std::vector<Evicted>* evicted = nullptr) {
        max_cost_ = max_cost;
        size_t count = 0;
        while (resident_cost_ > max_cost_) {
            auto ev = evict_lru();
            if (!ev) break;
            ++count;
            if (evicted) evicted->push_back(std::move(*ev));
        }
        return count;
    }

    size_t block_tokens() const { return bt_; }
    size_t max_cost() const { return max_cost_; }
    size_t len() const { return entries_.size(); }

    // insert (:181-249): replaces an identical key without counting an eviction, evicts LRU entries
    // until the new cost fits, becomes most recently used.  Returns false when cost > budget or the
    // prefix is empty.  Evicted snapshots are appended to `evicted` when given.
    bool insert(std::vector<uint32_t> tokens, T snapshot, size_t cost, std::vector<Evicted>* evicted = nullptr) {
        if (tokens.empty() || cost > max_cost_) return false;
        PromptHashPlan plan(tokens.data(), tokens.size(), bt_);
        PrefixDigest digest = index(plan.endpoint(tokens.size()));
        std::vector<PrefixDigest> block_digests;
        for (size_t b = 1; b <= tokens.size() / bt_; ++b) block_digests.push_back(index(plan.endpoint(b * bt_)));
        if (auto existing = exact_entry_id(digest, tokens)) remove_entry(*existing, false);
        size_t target_old = max_cost_ - cost;
        while (resident_cost_ > target_old) {
            auto ev = evict_lru();
            if (!ev) break;
            if (evicted) evicted->push_back(std::move(*ev));
        }
        uint64_t id = next_id_++;
        resident_cost_ += cost;
        by_digest_[digest].push_back(id);
        for (size_t b = 0; b < block_digests.size(); ++b) {
            size_t count = (b + 1) * bt_;
            by_block_digest_[block_digests[b]].push_back(BlockEndpoint{id, count});
            ++block_lengths_[count];
        }
        ++lengths_[tokens.size()];
        lru_.push_back(id);
        Entry e{std::move(tokens), std::move(snapshot), cost, digest, std::move(block_digests)};
        entries_.emplace(id, std::move(e));
        ++insertions_;
        return true;
    }

    // lookup (:258-304): longest exact stored prefix strictly shorter than the prompt.
    std::optional<Hit> lookup(const uint32_t* prompt, size_t n, size_t exclusive_max) {
        size_t limit = std::min(n, exclusive_max);
        std::vector<size_t> candidates;
        for (auto it = lengths_.begin(); it != lengths_.end() && it->first < limit; ++it) candidates.push_back(it->first);
        if (candidates.empty()) { ++misses_; return std::nullopt; }
        PromptHashPlan plan(prompt, candidates.back(), bt_);
        for (auto it = candidates.rbegin(); it != candidates.rend(); ++it) {
            size_t length = *it;
            auto bucket = by_digest_.find(index(plan.endpoint(length)));
            if (bucket == by_digest_.end()) continue;
            for (uint64_t id : bucket->second) {
                auto e = entries_.find(id);
                if (e == entries_.end()) continue;
                if (e->second.tokens.size() == length && std::equal(e->second.tokens.begin(), e->second.tokens.end(), prompt))
                    return finish_hit(id, length);
            }
        }
        ++misses_;
        return std::nullopt;
    }

    // lookup_aligned_common_prefix (:316-359): longest block-aligned common prefix inside any stored
    // snapshot, strictly shorter than the prompt; among enclosing entries the most recently used wins.
    std::optional<Hit> lookup_aligned_common_prefix(const uint32_t* prompt, size_t n, size_t exclusive_max) {
        size_t limit = std::min(n, exclusive_max);
        std::vector<size_t> candidates;
        for (auto it = block_lengths_.begin(); it != block_lengths_.end() && it->first < limit; ++it)
            candidates.push_back(it->first);
        if (candidates.empty()) { ++misses_; return std::nullopt; }
        PromptHashPlan plan(prompt, candidates.back(), bt_);
        for (auto it = candidates.rbegin(); it != candidates.rend(); ++it) {
            size_t matched = *it;
            auto bucket = by_block_digest_.find(index(plan.endpoint(matched)));
            if (bucket == by_block_digest_.end()) continue;
            for (auto l = lru_.rbegin(); l != lru_.rend(); ++l) {
                uint64_t id = *l;
                bool listed = false;
                for (const BlockEndpoint& ep : bucket->second)
                    if (ep.entry_id == id && ep.token_count == matched) { listed = true; break; }
                if (!listed) continue;
                auto e = entries_.find(id);
                if (e == entries_.end() || e->second.tokens.size() < matched) continue;
                if (!std::equal(prompt, prompt + matched, e->second.tokens.begin())) continue;
                return finish_hit(id, matched);
            }
        }
        ++misses_;
        return std::nullopt;
    }

    std::optional<Evicted> evict_lru() {  // :385-393
        if (lru_.empty()) return std::nullopt;
        return remove_entry(lru_.front(), true);
    }

    PrefixCacheStats stats() const {
        PrefixCacheStats s;
        s.hits = hits_;
        s.misses = misses_;
        s.matched_tokens = matched_tokens_;
        s.evictions = evictions_;
        s.insertions = insertions_;
        s.entries = entries_.size();
        s.cost = resident_cost_;
        s.max_cost = max_cost_;
        return s;
    }

private:
    struct Entry {
        std::vector<uint32_t> tokens;
        T snapshot;
        size_t cost;
        PrefixDigest digest;
        std::vector<PrefixDigest> block_digests;
    };
    struct BlockEndpoint {
        uint64_t entry_id;
        size_t token_count;
    };

    PrefixDigest index(const PrefixDigest& d) const { return forced_ ? PrefixDigest{} : d; }

    std::optional<uint64_t> exact_entry_id(const PrefixDigest& digest, const std::vector<uint32_t>& tokens) const {
        auto bucket = by_digest_.find(digest);
        if (bucket == by_digest_.end()) return std::nullopt;
        for (uint64_t id : bucket->second) {
            auto e = entries_.find(id);
            if (e != entries_.end() && e->second.tokens == tokens) return id;
        }
        return std::nullopt;
    }

    Hit finish_hit(uint64_t id, size_t matched) {  // :361-379
        ++hits_;
        matched_tokens_ += matched;
        for (auto it = lru_.begin(); it != lru_.end(); ++it)
            if (*it == id) { lru_.erase(it); break; }
        lru_.push_back(id);
        Entry& e = entries_.at(id);
        return Hit{matched, &e.snapshot, e.tokens.size(), e.cost};
    }

    std::optional<Evicted> remove_entry(uint64_t id, bool count_eviction) {  // :463-527
        auto it = entries_.find(id);
        if (it == entries_.end()) return std::nullopt;
        Entry e = std::move(it->second);
        entries_.erase(it);
        resident_cost_ -= e.cost;
        auto bucket = by_digest_.find(e.digest);
        if (bucket != by_digest_.end()) {
            auto& v = bucket->second;
            v.erase(std::remove(v.begin(), v.end(), id), v.end());
            if (v.empty()) by_digest_.erase(bucket);
        }
        for (size_t b = 0; b < e.block_digests.size(); ++b) {
            size_t count = (b + 1) * bt_;
            auto bb = by_block_digest_.find(e.block_digests[b]);
            if (bb != by_block_digest_.end()) {
                auto& v = bb->second;
                v.erase(std::remove_if(v.begin(), v.end(),
                                       [&](const BlockEndpoint& ep) { return ep.entry_id == id && ep.token_count == count; }),
                        v.end());
                if (v.empty()) by_block_digest_.erase(bb);
            }
            auto bl = block_lengths_.find(count);
            if (bl != block_lengths_.end() && --bl->second == 0) block_lengths_.erase(bl);
        }
        auto ln = lengths_.find(e.tokens.size());
        if (ln != lengths_.end() && --ln->second == 0) lengths_.erase(ln);
        for (auto l = lru_.begin(); l != lru_.end(); ++l)
            if (*l == id) { lru_.erase(l); break; }
        if (count_eviction) ++evictions_;
        return Evicted{std::move(e.tokens), std::move(e.snapshot), e.cost};
    }

    size_t bt_, max_cost_, resident_cost_ = 0;
    uint64_t next_id_ = 0;
    std::unordered_map<uint64_t, Entry> entries_;
    std::unordered_map<PrefixDigest, std::vector<uint64_t>, PrefixDigestHash> by_digest_;
    std::unordered_map<PrefixDigest, std::vector<BlockEndpoint>, PrefixDigestHash> by_block_digest_;
    std::map<size_t, size_t> lengths_, block_lengths_;
    std::deque<uint64_t> lru_;
    uint64_t hits_ = 0, misses_ = 0, matched_tokens_ = 0, evictions_ = 0, insertions_ = 0;
    bool forced_ = false;
};

}  // namespace mk
