// The cache: keys and values per layer run in pages, a slot per sequence, and beside it
// fixed-size state per sequence.
//
// Layer runs whose mixers have the same CacheNeed (kind, heads, widths of keys and values,
// window) form a group with storage and a page pool of its own: K of shape
// [runs, pages, kv_heads, page_size, k_dim] and V likewise with v_dim (no V when v_dim is 0).
// A sequence holds, per group, a list mapping its logical pages (position / page_size) to pool
// pages; a "window" group gives pages back as soon as every position in them has left the
// window.  The reference keeps one growing tensor pair per layer for one rectangular batch
// (src/libllm/kv_cache.h:31-59, src/libllm/llama.cc:188-212).
#pragma once
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "cache/pages.h"
#include "parts/part.h"

namespace llm {

struct CacheGroup {
  CacheNeed need;
  std::vector<int> runs;                 // schedule entries that own storage here
  std::unique_ptr<PagePool> pool;
  DeviceBuffer k, v;
  size_t k_run_bytes = 0, v_run_bytes = 0;
};

struct SequenceRecord {
  int slot = 0;
  int length = 0;
  std::vector<std::vector<int>> pages;   // per group: logical page -> pool page, -1 released
};

struct RunState {                        // the state tensors of one schedule entry
  std::vector<StateNeed> needs;
  std::vector<DeviceBuffer> buffers;     // [slots, *shape] each
};

class KVCache {
 public:
  // run_needs[i]: what schedule entry i wants cached (has[i] false: nothing of its own).
  // capacity_tokens: tokens all live sequences may hold together, each sequence's count rounded
  // up to whole pages.  With `allocate` false only the bookkeeping exists (no device is touched).
  KVCache(const std::vector<CacheNeed> &run_needs, const std::vector<char> &has,
          const std::vector<std::vector<StateNeed>> &run_states, int64_t capacity_tokens, DType dtype, int page_size = 64,
          int max_slots = 0, bool allocate = true);

  int page_size() const { return page_size_; }
  int n_pages() const { return n_pages_; }
  DType dtype() const { return dtype_; }
  const std::vector<CacheGroup> &groups() const { return groups_; }
  // entry -> (group, index in the group), or (-1, -1)
  const std::vector<std::pair<int, int>> &run_group() const { return run_group_; }
  const SlotTable &slots() const { return *slots_; }
  const std::map<int, SequenceRecord> &sequences() const { return sequences_; }

  int open(cudaStream_t stream = nullptr);
  void close(int slot);
  int length(int slot) const { return record(slot).length; }
  // Pages for every sequence of `growth` (slot, new length).  Either all are granted or
  // Error(Cache) is thrown and nothing has changed.
  void reserve(const std::vector<std::pair<int, int>> &growth);
  // The sequence now holds new_len tokens; window groups drop pages no later query can see (a
  // query at position p >= new_len sees keys > p - window).
  void commit(int slot, int new_len);
  // int32 [slots.size(), width] into `out`; unused entries are 0 (never read: positions beyond a
  // sequence's length are never asked for) and released ones -1.
  void page_table(int group, const std::vector<int> &slots, int width, int *out) const;
  int pages_needed(int slot) const;

  // What schedule entry `entry` sees: its own storage, or that of `source` (>= 0).
  bool layer_cache(int entry, int source, const std::vector<const int *> &tables, int table_width, LayerCache *out) const;
  StateView state_view(int entry) const;
  const std::vector<RunState> &states() const { return states_; }

  // Host bookkeeping is consistent: no page lost, held twice or freed twice.
  void check() const;
  Json info() const;

 private:
  const SequenceRecord &record(int slot) const;
  SequenceRecord &record(int slot);
  int page_size_, n_pages_;
  DType dtype_;
  bool allocated_;
  std::vector<CacheGroup> groups_;
  std::vector<std::pair<int, int>> run_group_;
  std::unique_ptr<SlotTable> slots_;
  std::map<int, SequenceRecord> sequences_;
  std::vector<RunState> states_;
};

}  // namespace llm
