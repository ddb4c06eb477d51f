#include "cache/kv_cache.h"

#include <algorithm>
#include <set>

namespace llm {

static int64_t numel(const std::vector<int64_t> &shape) {
  int64_t n = 1;
  for (auto s : shape) n *= s;
  return n;
}

KVCache::KVCache(const std::vector<CacheNeed> &run_needs, const std::vector<char> &has,
                 const std::vector<std::vector<StateNeed>> &run_states, int64_t capacity_tokens, DType dtype, int page_size,
                 int max_slots, bool allocate)
    : page_size_(page_size), dtype_(dtype), allocated_(allocate) {
  if (page_size < 1 || capacity_tokens < 1) LLM_THROW(Cache, "cache capacity and page size must be positive");
  n_pages_ = (int)((capacity_tokens + page_size - 1) / page_size);
  for (size_t i = 0; i < run_needs.size(); ++i) {
    if (!has[i]) {
      run_group_.push_back({-1, -1});
      continue;
    }
    int g = -1;
    for (size_t j = 0; j < groups_.size(); ++j)
      if (groups_[j].need == run_needs[i]) g = (int)j;
    if (g < 0) {
      g = (int)groups_.size();
      groups_.emplace_back();
      groups_.back().need = run_needs[i];
      groups_.back().pool.reset(new PagePool(n_pages_));
    }
    run_group_.push_back({g, (int)groups_[(size_t)g].runs.size()});
    groups_[(size_t)g].runs.push_back((int)i);
  }
  if (allocate) {
    for (auto &grp : groups_) {
      const size_t per_token = (size_t)grp.need.n_kv_heads * dtype_size(dtype);
      grp.k_run_bytes = (size_t)n_pages_ * page_size * per_token * (size_t)grp.need.k_dim;
      grp.v_run_bytes = (size_t)n_pages_ * page_size * per_token * (size_t)grp.need.v_dim;
      grp.k.allocate(grp.k_run_bytes * grp.runs.size(), true);
      if (grp.v_run_bytes) grp.v.allocate(grp.v_run_bytes * grp.runs.size(), true);
    }
  }
  slots_.reset(new SlotTable(max_slots > 0 ? max_slots : n_pages_));
  for (const auto &needs : run_states) {
    states_.emplace_back();
    states_.back().needs = needs;
    if (allocate)
      for (const auto &n : needs)
        states_.back().buffers.emplace_back((size_t)slots_->n_slots() * (size_t)numel(n.shape) * dtype_size(n.dtype), true);
  }
}

const SequenceRecord &KVCache::record(int slot) const {
  auto it = sequences_.find(slot);
  if (it == sequences_.end()) LLM_THROW(Cache, "slot %d is not open", slot);
  return it->second;
}
SequenceRecord &KVCache::record(int slot) {
  auto it = sequences_.find(slot);
  if (it == sequences_.end()) LLM_THROW(Cache, "slot %d is not open", slot);
  return it->second;
}

int KVCache::open(cudaStream_t stream) {
  const int slot = slots_->take();
  SequenceRecord rec;
  rec.slot = slot;
  rec.pages.resize(groups_.size());
  sequences_[slot] = rec;
  if (allocated_)
    for (auto &st : states_)
      for (size_t i = 0; i < st.needs.size(); ++i) {
        const size_t row = (size_t)numel(st.needs[i].shape) * dtype_size(st.needs[i].dtype);
        LLM_CUDA(cudaMemsetAsync((char *)st.buffers[i].get() + row * (size_t)slot, 0, row, stream));
      }
  return slot;
}

void KVCache::close(int slot) {
  auto it = sequences_.find(slot);
  if (it == sequences_.end()) LLM_THROW(Cache, "slot %d is not open (closed twice?)", slot);
  for (size_t g = 0; g < groups_.size(); ++g) {
    std::vector<int> pages;
    for (int p : it->second.pages[g])
      if (p >= 0) pages.push_back(p);
    groups_[g].pool->give_back(pages);
  }
  sequences_.erase(it);
  slots_->give_back(slot);
}

void KVCache::reserve(const std::vector<std::pair<int, int>> &growth) {
  struct Taken {
    int slot, group;
    size_t count;
    std::vector<int> pages;
  };
  std::vector<Taken> taken;
  try {
    for (const auto &gr : growth) {
      SequenceRecord &rec = record(gr.first);
      if (gr.second < rec.length)
        LLM_THROW(Cache, "slot %d: a sequence cannot shrink (%d -> %d)", gr.first, rec.length, gr.second);
      const int want = (gr.second + page_size_ - 1) / page_size_;
      for (size_t g = 0; g < groups_.size(); ++g) {
        const int missing = want - (int)rec.pages[g].size();
        if (missing > 0) {
          std::vector<int> pages = groups_[g].pool->take(missing);
          rec.pages[g].insert(rec.pages[g].end(), pages.begin(), pages.end());
          taken.push_back({gr.first, (int)g, pages.size(), std::move(pages)});
        }
      }
    }
  } catch (const Error &) {
    for (auto it = taken.rbegin(); it != taken.rend(); ++it) {
      SequenceRecord &rec = sequences_[it->slot];
      rec.pages[(size_t)it->group].resize(rec.pages[(size_t)it->group].size() - it->count);
      groups_[(size_t)it->group].pool->give_back(it->pages);
    }
    throw;
  }
}

void KVCache::commit(int slot, int new_len) {
  SequenceRecord &rec = record(slot);
  rec.length = new_len;
  for (size_t g = 0; g < groups_.size(); ++g) {
    const CacheNeed &need = groups_[g].need;
    if (need.kind != "window" || need.window <= 0) continue;
    const int first_needed = std::max(0, new_len - need.window + 1);
    std::vector<int> drop;
    const int upto = std::min(first_needed / page_size_, (int)rec.pages[g].size());
    for (int lp = 0; lp < upto; ++lp)
      if (rec.pages[g][(size_t)lp] >= 0) {
        drop.push_back(rec.pages[g][(size_t)lp]);
        rec.pages[g][(size_t)lp] = -1;
      }
    if (!drop.empty()) groups_[g].pool->give_back(drop);
  }
}

void KVCache::page_table(int group, const std::vector<int> &slots, int width, int *out) const {
  std::fill(out, out + slots.size() * (size_t)width, 0);
  for (size_t i = 0; i < slots.size(); ++i) {
    const auto &pages = record(slots[i]).pages[(size_t)group];
    if ((int)pages.size() > width)
      LLM_THROW(Cache, "slot %d holds %d pages, the step's table has %d", slots[i], (int)pages.size(), width);
    std::copy(pages.begin(), pages.end(), out + i * (size_t)width);
  }
}

int KVCache::pages_needed(int slot) const {
  int n = 0;
  for (const auto &p : record(slot).pages) n = std::max(n, (int)p.size());
  return n;
}

bool KVCache::layer_cache(int entry, int source, const std::vector<const int *> &tables, int table_width, LayerCache *out) const {
  const int owner = source >= 0 ? source : entry;
  const auto rg = run_group_[(size_t)owner];
  if (rg.first < 0) return false;
  const CacheGroup &grp = groups_[(size_t)rg.first];
  out->k = grp.k ? (char *)grp.k.get() + grp.k_run_bytes * (size_t)rg.second : nullptr;
  out->v = grp.v ? (char *)grp.v.get() + grp.v_run_bytes * (size_t)rg.second : nullptr;
  out->n_pages = n_pages_;
  out->page_table = tables[(size_t)rg.first];
  out->table_width = table_width;
  out->page_size = page_size_;
  out->writes = source < 0;
  out->group = rg.first;
  out->dtype = dtype_;
  out->need = grp.need;
  return true;
}

StateView KVCache::state_view(int entry) const {
  StateView view;
  const RunState &st = states_[(size_t)entry];
  for (size_t i = 0; i < st.needs.size(); ++i) {
    StateTensor t;
    t.name = st.needs[i].name;
    t.data = i < st.buffers.size() ? st.buffers[i].get() : nullptr;
    t.shape = st.needs[i].shape;
    t.dtype = st.needs[i].dtype;
    t.n_slots = slots_->n_slots();
    view.push_back(t);
  }
  return view;
}

void KVCache::check() const {
  for (size_t g = 0; g < groups_.size(); ++g) {
    groups_[g].pool->check();
    std::vector<int> held;
    for (const auto &kv : sequences_)
      for (int p : kv.second.pages[g])
        if (p >= 0) held.push_back(p);
    std::set<int> uniq(held.begin(), held.end());
    if (uniq.size() != held.size()) LLM_THROW(Cache, "group %zu: a page belongs to two sequences", g);
    if ((int)held.size() != groups_[g].pool->in_use())
      LLM_THROW(Cache, "group %zu: %d pages are held, sequences own %zu", g, groups_[g].pool->in_use(), held.size());
  }
  std::vector<int> open_slots;
  for (const auto &kv : sequences_) open_slots.push_back(kv.first);
  if (open_slots != slots_->held()) LLM_THROW(Cache, "open sequences and held slots differ");
}

Json KVCache::info() const {
  Json j = Json::object();
  j.set("page_size", page_size_);
  j.set("n_pages", n_pages_);
  j.set("n_slots", slots_->n_slots());
  j.set("slots_available", slots_->available());
  Json gs = Json::array();
  for (const auto &grp : groups_) {
    Json g = Json::object();
    g.set("kind", grp.need.kind);
    g.set("n_kv_heads", grp.need.n_kv_heads);
    g.set("k_dim", grp.need.k_dim);
    g.set("v_dim", grp.need.v_dim);
    g.set("window", grp.need.window > 0 ? Json(grp.need.window) : Json());
    g.set("runs", Json::list(grp.runs));
    g.set("pages_in_use", grp.pool->in_use());
    g.set("pages_available", grp.pool->available());
    g.set("k_address", (int64_t)(uintptr_t)grp.k.get());
    g.set("v_address", (int64_t)(uintptr_t)grp.v.get());
    gs.push(g);
  }
  j.set("groups", gs);
  Json rg = Json::array();
  for (const auto &p : run_group_) {
    if (p.first < 0) {
      rg.push(Json());
    } else {
      Json pair = Json::array();
      pair.push(p.first);
      pair.push(p.second);
      rg.push(pair);
    }
  }
  j.set("run_group", rg);
  Json seqs = Json::object();
  for (const auto &kv : sequences_) {
    Json s = Json::object();
    s.set("length", kv.second.length);
    Json pages = Json::array();
    for (const auto &p : kv.second.pages) pages.push(Json::list(p));
    s.set("pages", pages);
    seqs.set(std::to_string(kv.first), s);
  }
  j.set("sequences", seqs);
  Json st = Json::array();
  for (const auto &rs : states_) {
    Json o = Json::object();
    for (size_t i = 0; i < rs.needs.size(); ++i) {
      Json e = Json::object();
      e.set("shape", Json::list(rs.needs[i].shape));
      e.set("dtype", dtype_name(rs.needs[i].dtype));
      e.set("address", (int64_t)(uintptr_t)(i < rs.buffers.size() ? rs.buffers[i].get() : nullptr));
      o.set(rs.needs[i].name, e);
    }
    st.push(o);
  }
  j.set("state", st);
  return j;
}

}  // namespace llm
