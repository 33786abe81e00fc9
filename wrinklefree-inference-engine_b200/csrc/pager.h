// Host-side page and slot bookkeeping for paged per-sequence caches: a LIFO free list that hands pages out 0, 1, 2, ... (the hand-out order of
// the reference's KVCacheManager, tests/test_kv_cache_cpp.py:44-70), one block-table row per sequence slot, and a free list of the slots
// themselves (a slot also names a sequence's fixed-size recurrent state).  Pages and slots that are given back are handed out again first.
#pragma once
#include <stdint.h>
#include <vector>

namespace wf {

struct PageTable {
    int max_pages = 0, page_size = 1, slots = 0, max_blocks = 0;
    std::vector<int32_t> free_pages;   // back() is handed out next
    std::vector<int32_t> free_slots;
    std::vector<int32_t> table;        // [slots][max_blocks], -1 = no page
    std::vector<int32_t> held;         // [slots] blocks in use
    std::vector<uint8_t> live;         // [slots]
    bool dirty = true;                 // the table changed since the owner last copied it to the device

    void init(int max_pages_, int page_size_, int slots_, int max_blocks_) {
        max_pages = max_pages_; page_size = page_size_; slots = slots_; max_blocks = max_blocks_;
        table.assign((size_t)slots * max_blocks, -1);
        held.assign(slots, 0);
        live.assign(slots, 0);
        reset();
    }
    void reset() {
        free_pages.clear();
        for (int p = max_pages - 1; p >= 0; --p) free_pages.push_back(p);
        free_slots.clear();
        for (int s = slots - 1; s >= 0; --s) free_slots.push_back(s);
        std::fill(table.begin(), table.end(), -1);
        std::fill(held.begin(), held.end(), 0);
        std::fill(live.begin(), live.end(), 0);
        dirty = true;
    }
    int32_t* row(int slot) { return table.data() + (size_t)slot * max_blocks; }
    int blocks_for(int tokens) const { return (tokens + page_size - 1) / page_size; }
    // pages for tokens [0, tokens) of a slot; false (and nothing allocated) when the pool or the row cannot hold them
    bool ensure(int slot, int tokens) {
        const int need = blocks_for(tokens);
        if (need > max_blocks) return false;
        if (need - held[slot] > (int)free_pages.size()) return false;
        for (int b = held[slot]; b < need; ++b) {
            row(slot)[b] = free_pages.back();
            free_pages.pop_back();
            dirty = true;
        }
        if (need > held[slot]) held[slot] = need;
        return true;
    }
    // give back the pages beyond tokens
    void truncate(int slot, int tokens) {
        const int need = blocks_for(tokens);
        for (int b = held[slot] - 1; b >= need; --b) {
            free_pages.push_back(row(slot)[b]);
            row(slot)[b] = -1;
            dirty = true;
        }
        if (need < held[slot]) held[slot] = need;
    }
    int acquire_slot() {
        if (free_slots.empty()) return -1;
        const int s = free_slots.back();
        free_slots.pop_back();
        live[s] = 1;
        return s;
    }
    void release_slot(int slot) {
        if (slot < 0 || slot >= slots || !live[slot]) return;
        truncate(slot, 0);
        live[slot] = 0;
        free_slots.push_back(slot);
    }
};

}  // namespace wf
