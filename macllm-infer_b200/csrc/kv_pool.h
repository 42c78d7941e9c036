// Host bookkeeping of the paged KV pool: generational block slots, refcounts, copy-on-write
// reservations and the epoch protocol that keeps a page from being recycled while device work may
// still read it.  Restates crates/macllm-kv/src/cache.rs of the reference (PagedKvPool :588-1370,
// PagedKvBlockTable :1434-1865, SharedPagedKvPool::reserve_batch :2216-2445,
// PagedKvBatchReservation :2453-3005).  No device memory is touched here: the K/V arena lives in the
// model and is indexed by the slot numbers this class hands out.
#pragma once
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace mk {

struct KvPoolExhausted : std::runtime_error {
    int64_t requested, free_blocks, unallocated;
    KvPoolExhausted(int64_t req, int64_t fr, int64_t un)
        : std::runtime_error("paged KV pool exhausted: requested " + std::to_string(req) + " blocks, " + std::to_string(fr) +
                             " free and " + std::to_string(un) + " unallocated"),
          requested(req), free_blocks(fr), unallocated(un) {}
    // the same condition with the wording of the model boundary (KvCacheExhausted, src/architecture.rs:928-953)
    KvPoolExhausted(int64_t req, int64_t fr, int64_t un, const std::string& boundary_message)
        : std::runtime_error(boundary_message), requested(req), free_blocks(fr), unallocated(un) {}
};

struct KvBlockId {
    uint32_t slot = 0;
    uint64_t generation = 0;
    bool operator==(const KvBlockId& o) const { return slot == o.slot && generation == o.generation; }
};

struct KvPoolStats {
    int64_t block_tokens = 0, slab_blocks = 0, max_blocks = 0;
    int64_t allocated_blocks = 0, free_blocks = 0, reserved_blocks = 0, live_blocks = 0, live_references = 0,
            shared_blocks = 0, retired_blocks = 0, slabs = 0;
    uint64_t submitted_epoch = 0, completed_epoch = 0;
};

class KvTable;
class KvReservation;

class KvPool : public std::enable_shared_from_this<KvPool> {
public:
    KvPool(int block_tokens, int slab_blocks, int64_t max_blocks);

    int block_tokens() const { return block_tokens_; }
    int slab_blocks() const { return slab_blocks_; }
    int64_t max_blocks() const { return max_blocks_; }
    KvPoolStats stats() const;
    bool transaction_active() const { return active_transaction_ != 0; }

    // SharedPagedKvPool::reserve_batch: one transaction and one epoch for an ordered lane batch.
    // Throws KvPoolExhausted before anything is mutated.
    std::unique_ptr<KvReservation> reserve_batch(const std::vector<KvTable*>& tables, const std::vector<int64_t>& new_tokens);

    // mark_completed_through: device work up to `epoch` finished; retired pages become free.
    void mark_completed_through(uint64_t epoch);
    uint64_t submitted_epoch() const { return submitted_epoch_; }
    uint64_t completed_epoch() const { return completed_epoch_; }

    // slot -> (slab, offset in slab)
    int slab_of(uint32_t slot) const { return (int)(slot / (uint32_t)slab_blocks_); }
    int slab_offset_of(uint32_t slot) const { return (int)(slot % (uint32_t)slab_blocks_); }

private:
    friend class KvTable;
    friend class KvReservation;
    enum class State : uint8_t { Free, Reserved, Live, Retired };
    struct Slot {
        uint64_t generation = 0;
        State state = State::Free;
        uint64_t transaction = 0;  // Reserved
        int64_t references = 0;    // Live
        uint64_t until = 0;        // Retired
        uint64_t last_use = 0;
    };

    int64_t occupied() const { return reserved_ + live_ + retired_; }
    int64_t free_blocks() const { return (int64_t)slots_.size() - occupied(); }
    void ensure_free_blocks(int64_t requested);
    void begin_transaction(uint64_t& transaction, uint64_t& epoch);
    std::vector<KvBlockId> reserve_blocks(int64_t count, uint64_t transaction);
    const Slot& slot(const KvBlockId& id) const;
    Slot& slot_mut(const KvBlockId& id);
    void validate_owned(const KvBlockId& id, uint64_t transaction) const;
    int64_t live_references(const KvBlockId& id) const;
    void retain_live(const std::vector<KvBlockId>& ids);
    void release_live(const std::vector<KvBlockId>& ids);
    void mark_use(const std::vector<KvBlockId>& ids, uint64_t transaction, uint64_t epoch);
    void commit_reserved_replacing(const std::vector<KvBlockId>& ids, const std::vector<KvBlockId>& superseded, uint64_t transaction);
    void rollback_reserved(const std::vector<KvBlockId>& ids, uint64_t transaction);

    int block_tokens_, slab_blocks_;
    int64_t max_blocks_;
    std::vector<Slot> slots_;
    int64_t slabs_ = 0;
    int64_t reserved_ = 0, live_ = 0, live_refs_ = 0, shared_ = 0, retired_ = 0;
    uint64_t next_transaction_ = 0, active_transaction_ = 0;
    uint64_t submitted_epoch_ = 0, completed_epoch_ = 0;
};

// PagedKvBlockTable: one sequence's ordered list of blocks.
class KvTable {
public:
    KvTable(std::shared_ptr<KvPool> pool, int64_t limit);
    ~KvTable();
    KvTable(const KvTable&) = delete;
    KvTable& operator=(const KvTable&) = delete;

    int64_t logical_len() const { return logical_len_; }
    int64_t owned_blocks() const { return (int64_t)blocks_.size(); }
    const std::vector<KvBlockId>& blocks() const { return blocks_; }
    int64_t limit() const { return limit_; }
    bool in_flight() const { return in_flight_ != 0; }
    const std::shared_ptr<KvPool>& pool() const { return pool_; }

    void attach_prefix(const KvTable& source, int64_t logical_len);
    std::unique_ptr<KvTable> fork_prefix(int64_t logical_len) const;
    // Returns false (and changes nothing) while a reservation holds the table.
    bool clear();

private:
    friend class KvPool;
    friend class KvReservation;
    std::shared_ptr<KvPool> pool_;
    std::vector<KvBlockId> blocks_;
    int64_t logical_len_ = 0;
    int64_t limit_;
    uint64_t in_flight_ = 0;
};

struct KvCowCopy {
    uint32_t src_slot, dst_slot;
    int32_t rows;
};

// PagedKvBatchReservation: rolls back on destruction unless committed.
class KvReservation {
public:
    ~KvReservation();
    uint64_t epoch() const { return epoch_; }
    size_t lane_count() const { return lanes_.size(); }
    int64_t lane_old_len(size_t lane) const { return lanes_.at(lane).old_len; }
    int64_t lane_new_len(size_t lane) const { return lanes_.at(lane).new_len; }
    const std::vector<KvBlockId>& lane_blocks(size_t lane) const { return lanes_.at(lane).provisional; }
    KvTable* lane_table(size_t lane) const { return lanes_.at(lane).table; }
    // Copy-on-write page copies the device must perform before the first write of this batch.
    const std::vector<KvCowCopy>& cow_copies() const { return cows_; }
    // build_attention_batch: records every referenced page as used in this epoch and returns the
    // compact page table: rows (compact slab index in order of first appearance, block in slab).
    void mark_all_used();
    void page_table(std::vector<uint32_t>& pages, std::vector<int32_t>& lane_offsets, std::vector<int32_t>& lane_counts,
                    std::vector<int32_t>& lane_lens);
    // commit: Reserved -> Live(1), superseded copy-on-write sources lose one reference, tables take
    // their provisional blocks.
    uint64_t commit();
    void rollback();

private:
    friend class KvPool;
    struct Lane {
        KvTable* table;
        int64_t old_len, new_len, new_tokens;
        int64_t growth_blocks, reserved_blocks;
        std::vector<KvBlockId> provisional;
        bool cow = false;
        size_t cow_index = 0;
        KvBlockId cow_source;
        int32_t cow_valid = 0;
    };
    KvReservation() = default;
    std::shared_ptr<KvPool> pool_;
    uint64_t transaction_ = 0, epoch_ = 0;
    std::vector<Lane> lanes_;
    std::vector<KvBlockId> reserved_, superseded_;
    std::vector<KvCowCopy> cows_;
    bool finalized_ = false;
};

}  // namespace mk
