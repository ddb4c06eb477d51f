// Bookkeeping of the cache on the host: pages of tokens and slots of sequences.
//
// The reference's cache is a dictionary of tensors that grows by allocate-and-copy at every step
// and holds one rectangular batch (src/libllm/kv_cache.cc:27-67, src/libllm/llama.cc:203-212).
// Here storage is allocated once and handed out in pages of `page_size` tokens; a sequence owns a
// slot and a list of pages per cache group, and gives all of it back when it ends.
#pragma once
#include <vector>

#include "util/error.h"

namespace llm {

// Free list of page numbers with checks against loss and double use.
class PagePool {
 public:
  explicit PagePool(int n_pages);
  int n_pages() const { return n_pages_; }
  int available() const { return (int)free_.size(); }
  int in_use() const { return n_pages_ - (int)free_.size(); }
  std::vector<int> take(int n);                    // n pages, or Error(Cache) with nothing taken
  void give_back(const std::vector<int> &pages);   // all of them, or Error(Cache) with nothing changed
  void check() const;                              // every page is either free or held, none both or neither

 private:
  int n_pages_;
  std::vector<int> free_;
  std::vector<char> held_;
};

// Slots of sequences: lowest free slot first, so slots are used again at once.
class SlotTable {
 public:
  explicit SlotTable(int n_slots);
  int n_slots() const { return n_slots_; }
  int available() const { return (int)free_.size(); }
  int take();
  void give_back(int slot);
  bool is_held(int slot) const { return slot >= 0 && slot < n_slots_ && held_[slot]; }
  std::vector<int> held() const;

 private:
  int n_slots_;
  std::vector<int> free_;       // kept sorted, highest first
  std::vector<char> held_;
};

}  // namespace llm
