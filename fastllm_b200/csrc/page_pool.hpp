// Host-side allocator of cache pages: a fixed pool shared by sequence slots, pages handed out on demand and given back when a
// slot's sequence ends.  Plain C++ (no CUDA): the device page table is a mirror the owner uploads after `grow`.
#pragma once
#include <stdexcept>
#include <vector>

namespace fl {

class PagePool {
public:
    PagePool() = default;
    PagePool(int pages, int slots, int pages_per_slot, int page_tokens)
        : pages_(pages), per_slot_(pages_per_slot), page_tokens_(page_tokens), table_((size_t)slots * pages_per_slot, -1),
          held_(slots, 0) {
        free_.reserve(pages);
        for (int p = pages - 1; p >= 0; --p) free_.push_back(p);      // lowest page first
    }
    int pages_total() const { return pages_; }
    int pages_free() const { return (int)free_.size(); }
    int pages_per_slot() const { return per_slot_; }
    int held(int slot) const { return held_[slot]; }
    const int* row(int slot) const { return table_.data() + (size_t)slot * per_slot_; }
    // pages a slot would have to take to hold `tokens` tokens
    int missing(int slot, int tokens) const {
        const int need = (tokens + page_tokens_ - 1) / page_tokens_;
        return need > held_[slot] ? need - held_[slot] : 0;
    }
    // make the slot hold `tokens` tokens; returns false (and changes nothing) if the pool or the slot's row is too small
    bool grow(int slot, int tokens) {
        const int need = (tokens + page_tokens_ - 1) / page_tokens_;
        if (need > per_slot_ || need - held_[slot] > (int)free_.size()) return false;
        while (held_[slot] < need) {
            table_[(size_t)slot * per_slot_ + held_[slot]++] = free_.back();
            free_.pop_back();
        }
        return true;
    }
    // the slot's sequence is over: its pages return to the pool (last taken = first reused)
    void release(int slot) {
        for (int i = 0; i < held_[slot]; ++i) {
            free_.push_back(table_[(size_t)slot * per_slot_ + i]);
            table_[(size_t)slot * per_slot_ + i] = -1;
        }
        held_[slot] = 0;
    }

private:
    int pages_ = 0, per_slot_ = 0, page_tokens_ = 64;
    std::vector<int> table_, held_, free_;
};

}  // namespace fl
