// Host-only checks of the paged-KV bookkeeping (retrograd_b200/csrc/kv.hpp): block sharing on
// seq_cp, copy-on-write of the boundary block, logical cells_used, transactional reservation.
#include "../../retrograd_b200/csrc/kv.hpp"

#include <cstdio>
#include <cstdlib>

using namespace rb200;

#define CHECK(cond)                                                                  \
    do {                                                                             \
        if (!(cond)) {                                                               \
            std::fprintf(stderr, "CHECK failed at line %d: %s\n", __LINE__, #cond);  \
            std::exit(1);                                                            \
        }                                                                            \
    } while (0)

int main() {
    // 4 slots, 8 blocks of 16 cells, up to 6 blocks per slot
    KvManager kv(4, 8, 16, 6);
    kv.begin();
    CHECK(kv.reserve(0, 0, 20) == KvManager::OK);
    kv.commit();
    CHECK(kv.slot(0).pos_min == 0 && kv.slot(0).pos_max == 19);
    CHECK(kv.blocks_used() == 2 && kv.cells_used() == 20);
    CHECK(kv.patches().size() == 4 && kv.copies().empty());
    kv.patches().clear();

    // a gap is refused and changes nothing
    kv.begin();
    CHECK(kv.reserve(0, 25, 1) == KvManager::GAP);
    kv.rollback();
    CHECK(kv.slot(0).pos_max == 19);

    // metadata-only copy of a mid-block prefix: blocks shared, logical cells counted twice
    CHECK(kv.seq_cp(0, 1, 0, 18) == KvManager::COPIED);
    CHECK(kv.slot(1).pos_min == 0 && kv.slot(1).pos_max == 17);
    CHECK(kv.blocks_used() == 2 && kv.cells_used() == 38);
    CHECK(kv.slot(1).blocks[0] == kv.slot(0).blocks[0] && kv.slot(1).blocks[1] == kv.slot(0).blocks[1]);
    CHECK(kv.seq_cp(0, 1, 0, 5) == KvManager::DST_NOT_EMPTY);
    kv.patches().clear();

    // the first write into the shared boundary block copies it
    kv.begin();
    CHECK(kv.reserve(1, 18, 1) == KvManager::OK);
    kv.commit();
    CHECK(kv.copies().size() == 2 && kv.copies()[0] == kv.slot(0).blocks[1] && kv.copies()[1] == kv.slot(1).blocks[1]);
    CHECK(kv.slot(1).blocks[1] != kv.slot(0).blocks[1] && kv.slot(1).blocks[0] == kv.slot(0).blocks[0]);
    CHECK(kv.blocks_used() == 3);
    kv.copies().clear();
    kv.patches().clear();
    // the source now owns its boundary block alone: no second copy
    kv.begin();
    CHECK(kv.reserve(0, 20, 1) == KvManager::OK);
    kv.commit();
    CHECK(kv.copies().empty() && kv.blocks_used() == 3);

    // a step that does not fit rolls back every row of it
    kv.begin();
    CHECK(kv.reserve(2, 0, 64) == KvManager::OK);     // 4 blocks -> 7 used
    CHECK(kv.reserve(3, 0, 40) == KvManager::FULL);   // needs 3, one left
    kv.rollback();
    CHECK(kv.blocks_used() == 3 && kv.slot(2).empty() && kv.slot(3).empty());
    CHECK(kv.patches().empty());

    // removals: tail, head, hole, whole
    CHECK(kv.seq_rm(0, 17, -1) && kv.slot(0).pos_max == 16);
    CHECK(!kv.seq_rm(0, 3, 9));
    CHECK(kv.seq_rm(0, -1, 16) && kv.slot(0).pos_min == 16);   // drops block 0 of slot 0 (still held by slot 1)
    CHECK(kv.blocks_used() == 3);
    CHECK(kv.seq_rm(1, -1, -1) && kv.slot(1).empty());
    CHECK(kv.blocks_used() == 1);
    CHECK(kv.seq_rm(0, -1, -1) && kv.blocks_used() == 0 && kv.cells_used() == 0);

    // an empty slot accepts any first position
    kv.begin();
    CHECK(kv.reserve(3, 37, 3) == KvManager::OK);
    kv.commit();
    CHECK(kv.slot(3).pos_min == 37 && kv.slot(3).pos_max == 39 && kv.blocks_used() == 1);
    std::puts("ok");
    return 0;
}
