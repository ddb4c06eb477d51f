#include "cache/pages.h"

#include <algorithm>
#include <set>

namespace llm {

PagePool::PagePool(int n_pages) : n_pages_(n_pages), held_((size_t)std::max(n_pages, 0), 0) {
  if (n_pages < 1) LLM_THROW(Cache, "a cache needs at least one page");
  for (int p = n_pages - 1; p >= 0; --p) free_.push_back(p);
}

std::vector<int> PagePool::take(int n) {
  if (n < 0) LLM_THROW(Cache, "cannot take %d pages", n);
  if (n > (int)free_.size())
    LLM_THROW(Cache, "the cache is full: %d pages wanted, %d of %d free", n, (int)free_.size(), n_pages_);
  std::vector<int> out;
  out.reserve((size_t)n);
  for (int i = 0; i < n; ++i) {
    out.push_back(free_.back());
    free_.pop_back();
    held_[(size_t)out.back()] = 1;
  }
  return out;
}

void PagePool::give_back(const std::vector<int> &pages) {
  std::set<int> seen;
  for (int p : pages) {
    if (p < 0 || p >= n_pages_) LLM_THROW(Cache, "page %d does not exist (pool of %d)", p, n_pages_);
    if (!held_[(size_t)p]) LLM_THROW(Cache, "page %d is freed twice", p);
    if (!seen.insert(p).second) LLM_THROW(Cache, "a page is named twice in one release");
  }
  for (int p : pages) {
    held_[(size_t)p] = 0;
    free_.push_back(p);
  }
}

void PagePool::check() const {
  std::set<int> free_set(free_.begin(), free_.end());
  if (free_set.size() != free_.size()) LLM_THROW(Cache, "a page is on the free list twice");
  for (int p = 0; p < n_pages_; ++p) {
    const bool is_free = free_set.count(p) != 0;
    if (is_free == (held_[(size_t)p] != 0))
      LLM_THROW(Cache, "page %d is %s", p, is_free ? "both free and held" : "lost");
  }
}

SlotTable::SlotTable(int n_slots) : n_slots_(n_slots), held_((size_t)std::max(n_slots, 0), 0) {
  if (n_slots < 1) LLM_THROW(Cache, "a cache needs at least one slot");
  for (int s = n_slots - 1; s >= 0; --s) free_.push_back(s);
}

int SlotTable::take() {
  if (free_.empty()) LLM_THROW(Cache, "no free slot: all %d sequences slots are in use", n_slots_);
  const int s = free_.back();
  free_.pop_back();
  held_[(size_t)s] = 1;
  return s;
}

void SlotTable::give_back(int slot) {
  if (slot < 0 || slot >= n_slots_) LLM_THROW(Cache, "slot %d does not exist (%d slots)", slot, n_slots_);
  if (!held_[(size_t)slot]) LLM_THROW(Cache, "slot %d is freed twice or was never taken", slot);
  held_[(size_t)slot] = 0;
  free_.insert(std::upper_bound(free_.begin(), free_.end(), slot, std::greater<int>()), slot);
}

std::vector<int> SlotTable::held() const {
  std::vector<int> out;
  for (int s = 0; s < n_slots_; ++s)
    if (held_[(size_t)s]) out.push_back(s);
  return out;
}

}  // namespace llm
