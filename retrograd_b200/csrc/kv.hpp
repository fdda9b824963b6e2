// Host-side bookkeeping of the paged KV cache: per-slot block tables over a pool of
// fixed-size blocks with reference counts.
//
// This realises the sequence-memory contract of the reference's engine
// (crates/retrograd-ffi/runtime/include/retro_lora_train.h:2481-2487,2721-2762;
// crates/retrograd-ffi/runtime/src/retro_gen_core.cpp:2779-2937): seq_cp between slots is a
// metadata-only operation (blocks are shared, the boundary block is copied on the first write),
// seq_rm of a whole sequence or of a head/tail range always works, seq_pos reports the resident
// span, and `cells_used` stays the LOGICAL sum of spans even though shared blocks are stored once.
// Every change to a table entry is queued as a (flat index, block) patch for the device copy of
// the tables, and every copy-on-write as a (src, dst) block pair.
#pragma once

#include <algorithm>
#include <cstdint>
#include <vector>

namespace rb200 {

struct KvSlot {
    int32_t pos_min = -1;
    int32_t pos_max = -1;
    std::vector<int32_t> blocks;   // indexed by pos / block_tokens, -1 = none
    bool empty() const { return pos_min < 0; }
};

class KvManager {
public:
    KvManager(uint32_t n_slots, uint32_t n_blocks, uint32_t block_tokens, uint32_t max_blocks_per_slot)
        : block_tokens_(block_tokens), max_blocks_(max_blocks_per_slot), refcount_(n_blocks, 0), slots_(n_slots) {
        free_.reserve(n_blocks);
        for (int32_t b = (int32_t)n_blocks - 1; b >= 0; --b) free_.push_back(b);
    }

    uint32_t block_tokens() const { return block_tokens_; }
    uint32_t max_blocks() const { return max_blocks_; }
    uint32_t n_blocks() const { return (uint32_t)refcount_.size(); }
    uint32_t blocks_used() const { return (uint32_t)(refcount_.size() - free_.size()); }
    const KvSlot & slot(int32_t s) const { return slots_[s]; }
    uint32_t n_slots() const { return (uint32_t)slots_.size(); }

    std::vector<int32_t> & patches() { return patches_; }
    std::vector<int32_t> & copies() { return copies_; }

    uint64_t cells_used() const {
        uint64_t used = 0;
        for (const KvSlot & s : slots_) if (!s.empty()) used += (uint64_t)(s.pos_max - s.pos_min + 1);
        return used;
    }

    // Transaction over one step: begin(), reserve() per row, then commit() or rollback().
    void begin() { undo_.clear(); txn_patches_ = patches_.size(); txn_copies_ = copies_.size(); }

    enum Reserve { OK, GAP, FULL };

    // Makes positions [pos0, pos0 + n) of `slot` writable by this step.
    Reserve reserve(int32_t s, int32_t pos0, int32_t n) {
        KvSlot & sl = slots_[s];
        if (!sl.empty() && pos0 > sl.pos_max + 1) return GAP;
        undo_.push_back({UNDO_SPAN, s, sl.pos_min, sl.pos_max});
        const int32_t b0 = pos0 / (int32_t)block_tokens_, b1 = (pos0 + n - 1) / (int32_t)block_tokens_;
        if ((int32_t)sl.blocks.size() <= b1) {
            undo_.push_back({UNDO_RESIZE, s, (int32_t)sl.blocks.size(), 0});
            sl.blocks.resize(b1 + 1, -1);
        }
        for (int32_t bi = b0; bi <= b1; ++bi) {
            const int32_t cur = sl.blocks[bi];
            if (cur >= 0 && refcount_[cur] == 1) continue;
            if (free_.empty()) return FULL;
            const int32_t fresh = free_.back();
            free_.pop_back();
            refcount_[fresh] = 1;
            undo_.push_back({UNDO_ALLOC, s, bi, cur});
            if (cur >= 0) {
                // shared block: copy on write
                --refcount_[cur];
                copies_.push_back(cur);
                copies_.push_back(fresh);
            }
            sl.blocks[bi] = fresh;
            patches_.push_back(s * (int32_t)max_blocks_ + bi);
            patches_.push_back(fresh);
        }
        if (sl.empty()) sl.pos_min = pos0;
        sl.pos_min = std::min(sl.pos_min, pos0);
        sl.pos_max = std::max(sl.pos_max, pos0 + n - 1);
        return OK;
    }

    void rollback() {
        for (size_t i = undo_.size(); i-- > 0;) {
            const Undo & u = undo_[i];
            KvSlot & sl = slots_[u.slot];
            switch (u.kind) {
                case UNDO_SPAN: sl.pos_min = u.a; sl.pos_max = u.b; break;
                case UNDO_RESIZE: sl.blocks.resize(u.a); break;
                case UNDO_ALLOC: {
                    const int32_t fresh = sl.blocks[u.a];
                    refcount_[fresh] = 0;
                    free_.push_back(fresh);
                    sl.blocks[u.a] = u.b;
                    if (u.b >= 0) ++refcount_[u.b];
                    break;
                }
            }
        }
        undo_.clear();
        patches_.resize(txn_patches_);
        copies_.resize(txn_copies_);
    }

    void commit() { undo_.clear(); }

    // [p0, p1), negative = open. Returns false for a range that would leave a hole.
    bool seq_rm(int32_t s, int32_t p0, int32_t p1) {
        KvSlot & sl = slots_[s];
        if (sl.empty()) return true;
        if (p0 < 0) p0 = 0;
        if (p1 < 0) p1 = sl.pos_max + 1;
        if (p0 >= p1 || p0 > sl.pos_max || p1 <= sl.pos_min) return true;
        const int32_t B = (int32_t)block_tokens_;
        if (p0 <= sl.pos_min && p1 > sl.pos_max) {
            for (int32_t & b : sl.blocks) release(b);
            sl = KvSlot{};
            return true;
        }
        if (p1 > sl.pos_max) {           // tail
            const int32_t keep_last = (p0 - 1) / B;
            for (int32_t bi = keep_last + 1; bi < (int32_t)sl.blocks.size(); ++bi) release(sl.blocks[bi]);
            sl.blocks.resize(keep_last + 1);
            sl.pos_max = p0 - 1;
            return true;
        }
        if (p0 <= sl.pos_min) {          // head
            for (int32_t bi = 0; bi < p1 / B; ++bi) release(sl.blocks[bi]);
            sl.pos_min = p1;
            return true;
        }
        return false;
    }

    enum Copy { COPIED, NOTHING, DST_NOT_EMPTY };

    Copy seq_cp(int32_t src, int32_t dst, int32_t p0, int32_t p1) {
        if (src == dst) return NOTHING;
        const KvSlot & from = slots_[src];
        KvSlot & to = slots_[dst];
        if (from.empty()) return NOTHING;
        if (p0 < 0) p0 = 0;
        if (p1 < 0) p1 = from.pos_max + 1;
        p0 = std::max(p0, from.pos_min);
        p1 = std::min(p1, from.pos_max + 1);
        if (p0 >= p1) return NOTHING;
        if (!to.empty()) return DST_NOT_EMPTY;
        const int32_t B = (int32_t)block_tokens_;
        const int32_t b0 = p0 / B, b1 = (p1 - 1) / B;
        to.blocks.assign(b1 + 1, -1);
        for (int32_t bi = b0; bi <= b1; ++bi) {
            const int32_t blk = from.blocks[bi];
            to.blocks[bi] = blk;
            ++refcount_[blk];
            patches_.push_back(dst * (int32_t)max_blocks_ + bi);
            patches_.push_back(blk);
        }
        to.pos_min = p0;
        to.pos_max = p1 - 1;
        return COPIED;
    }

    void clear_all() {
        for (KvSlot & sl : slots_) {
            for (int32_t & b : sl.blocks) release(b);
            sl = KvSlot{};
        }
    }

private:
    enum UndoKind { UNDO_SPAN, UNDO_RESIZE, UNDO_ALLOC };
    struct Undo {
        UndoKind kind;
        int32_t slot;
        int32_t a;
        int32_t b;
    };

    void release(int32_t & b) {
        if (b < 0) return;
        if (--refcount_[b] == 0) free_.push_back(b);
        b = -1;
    }

    uint32_t block_tokens_;
    uint32_t max_blocks_;
    std::vector<uint32_t> refcount_;
    std::vector<int32_t> free_;
    std::vector<KvSlot> slots_;
    std::vector<int32_t> patches_;
    std::vector<int32_t> copies_;
    std::vector<Undo> undo_;
    size_t txn_patches_ = 0, txn_copies_ = 0;
};

} // namespace rb200
