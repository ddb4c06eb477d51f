#include "engine/step.h"

#include <algorithm>
#include <cstring>
#include <numeric>
#include <set>

#include "csrc/kernels.h"
#include "parts/chain.h"
#include "parts/linear.h"

namespace llm {

void SamplingParams::validate() const {
  if (temperature < 0) LLM_THROW(InvalidArg, "temperature must not be negative");
  if (top_k < 0 || top_k > 1024) LLM_THROW(InvalidArg, "top_k must lie in 0..1024 (0: the whole vocabulary)");
  if (!(top_p > 0)) LLM_THROW(InvalidArg, "top_p must be positive");
  if (top_k == 0 && top_p < 1.0f && temperature > 0) LLM_THROW(InvalidArg, "top_p below 1 needs a top_k");
}

bool Engine::GraphKey::operator<(const GraphKey &o) const {
  if (batch != o.batch) return batch < o.batch;
  if (width != o.width) return width < o.width;
  if (sampled != o.sampled) return sampled < o.sampled;
  if (!sampled) return false;
  return sampling < o.sampling;
}

// ---------------------------------------------------------------- the step's integer arrays
// Host staging (pinned) and device copy of one step's descriptor: tokens, the sequence and
// position of each token, each sequence's start, past length and slot, the wanted rows, the
// uniform numbers, the rows of fed tokens, and a page table per cache group.
class Engine::Descriptor {
 public:
  enum Field { Tokens, TokSeq, TokPos, SeqStart, SeqPast, SeqSlot, Want, Uniforms, Fed, Tables };

  Descriptor() { LLM_CUDA(cudaEventCreateWithFlags(&copied_, cudaEventDisableTiming)); }
  ~Descriptor() { cudaEventDestroy(copied_); }

  void shape(int T, int B, int W, const std::vector<int> &widths) {
    wait_host_free();
    n_tokens = T;
    n_seqs = B;
    n_want = W;
    this->widths = widths;
    sizes_ = {T, T, T, B + 1, B, B, W, std::max(B, W), T};
    for (int w : widths) sizes_.push_back(B * w);
    offsets_.assign(1, 0);
    for (int s : sizes_) offsets_.push_back(offsets_.back() + (size_t)((s + 3) / 4 * 4));
    const size_t bytes = offsets_.back() * sizeof(int);
    if (bytes > host_.bytes()) {
      // the device copy may still be read by kernels of an earlier step
      LLM_CUDA(cudaDeviceSynchronize());
      const size_t grown = std::max(bytes, host_.bytes() * 2);
      host_.allocate(grown);
      dev_.allocate(grown);
    }
    memset(host_.get(), 0, bytes);
  }
  size_t words() const { return offsets_.back(); }
  int *host(int field) { return host_.as<int>() + offsets_[(size_t)field]; }
  int *dev(int field) { return dev_.as<int>() + offsets_[(size_t)field]; }
  int *host_base() { return host_.as<int>(); }
  int *dev_base() { return dev_.as<int>(); }
  int size(int field) const { return sizes_[(size_t)field]; }

  void wait_host_free() {
    if (pending_) {
      LLM_CUDA(cudaEventSynchronize(copied_));
      pending_ = false;
    }
  }
  void upload(cudaStream_t s) {
    LLM_CUDA(cudaMemcpyAsync(dev_.get(), host_.get(), words() * sizeof(int), cudaMemcpyHostToDevice, s));
    in_flight(s);
  }
  // What was launched up to here reads the host staging (a copy, or a graph that copies by
  // itself): the staging is free again when that has run.
  void in_flight(cudaStream_t s) {
    LLM_CUDA(cudaEventRecord(copied_, s));
    pending_ = true;
  }
  cudaEvent_t event() const { return copied_; }

  int n_tokens = 0, n_seqs = 0, n_want = 0;
  std::vector<int> widths;

 private:
  PinnedBuffer host_;
  DeviceBuffer dev_;
  cudaEvent_t copied_ = nullptr;
  bool pending_ = false;
  std::vector<int> sizes_;
  std::vector<size_t> offsets_;
};

// A captured step of B sequences bringing one token each, page tables `width` wide.  The graph
// holds its own copies (descriptor in, tokens out), so a step is one launch.
struct Engine::DecodeGraph {
  int batch = 0, width = 0;
  bool sampled = false;
  SamplingParams sampling;
  Descriptor desc;
  Arena arena{(size_t)16 << 20};
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  Act logits;
  PinnedBuffer host_tokens;          // batch tokens, then the status word
  ~DecodeGraph() {
    if (exec) cudaGraphExecDestroy(exec);
    if (graph) cudaGraphDestroy(graph);
  }
};

// ---------------------------------------------------------------- construction
Engine::Engine(std::unique_ptr<Model> model, const Options &options) : model_(std::move(model)), opt_(options) {
  if (!model_->loaded()) LLM_THROW(InvalidArg, "an engine needs a model with its weights loaded");
  if (opt_.max_tokens < 1) LLM_THROW(InvalidArg, "max_tokens must be positive");
  if (opt_.page_size != model_->page_size()) LLM_THROW(InvalidArg, "the model was built for pages of %d tokens", model_->page_size());
  make_current();
  LLM_CUDA(cudaDeviceGetAttribute(&sm_count_, cudaDevAttrMultiProcessorCount, opt_.device));
  const int64_t n_pages = (opt_.max_tokens + opt_.page_size - 1) / opt_.page_size;
  max_seq_len_ = model_->max_positions();
  if (opt_.max_seq_len > 0) max_seq_len_ = std::min(max_seq_len_, opt_.max_seq_len);
  max_seq_len_ = std::min(max_seq_len_, n_pages * opt_.page_size);
  opt_.max_step_tokens = std::max(1, opt_.max_step_tokens);
  std::vector<CacheNeed> needs;
  std::vector<char> has;
  model_->cache_needs(&needs, &has);
  cache_.reset(new KVCache(needs, has, model_->state_needs(), opt_.max_tokens, model_->dtype(), opt_.page_size, opt_.max_slots));
  LLM_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
  status_.allocate(sizeof(int), true);
  counters_.allocate((sizeof(int) << 18) + 64 * sizeof(int), true);      // the last 64 are the chained kernel's
  // The tokens the last sampling step drew, kept on the device: the next step can take them from
  // here (StepItem::fed_row) while the host is still reading them back.
  last_capacity_ = std::max(opt_.max_step_tokens, 1024);
  last_tokens_.allocate(sizeof(int) * (size_t)last_capacity_, true);
  for (int i = 0; i < 4; ++i) eager_desc_.emplace_back(new Descriptor());
  token_ring_.resize(4);
  for (auto &t : token_ring_) {
    t.buf.allocate(sizeof(int) * ((size_t)last_capacity_ + 1));
    LLM_CUDA(cudaEventCreateWithFlags(&t.done, cudaEventDisableTiming));
  }
  status_host_.allocate(sizeof(int));
}

Engine::~Engine() {
  cudaSetDevice(opt_.device);
  if (stream_) cudaStreamSynchronize(stream_);
  for (auto &g : graphs_) g.clear();
  for (auto &t : token_ring_)
    if (t.done) cudaEventDestroy(t.done);
  if (stream_) cudaStreamDestroy(stream_);
}

void Engine::make_current() const { LLM_CUDA(cudaSetDevice(opt_.device)); }

int Engine::open_sequence() {
  make_current();
  return cache_->open(stream_);
}
void Engine::close_sequence(int slot) { cache_->close(slot); }
void Engine::synchronize() {
  make_current();
  LLM_CUDA(cudaStreamSynchronize(stream_));
}

long long Engine::chain_launches() const { return chain_launches_ + (chain_ ? chain_->launches() : 0); }

void Engine::raise_status(int code) {
  cudaMemsetAsync(status_.get(), 0, sizeof(int), stream_);
  cudaMemsetAsync(counters_.get(), 0, counters_.bytes(), stream_);      // a kernel that gave up may have left its counts
  LLM_THROW(Extension, "a tensor-core kernel gave up waiting on a barrier (code %d: 1 loader, 2-3 issue, 4-6 epilogue, 7-8 a job of a "
                       "chain, 9 a probe); "
                       "the step's results are not valid", code);
}

void Engine::check_status() {
  make_current();
  LLM_CUDA(cudaMemcpyAsync(status_host_.get(), status_.get(), sizeof(int), cudaMemcpyDeviceToHost, stream_));
  LLM_CUDA(cudaStreamSynchronize(stream_));
  const int code = *status_host_.as<int>();
  if (code) raise_status(code);
}

// ---------------------------------------------------------------- checks
void Engine::validate(const std::vector<StepItem> &items) const {
  std::set<int> seen;
  const int64_t V = vocab();
  for (const auto &it : items) {
    if (!seen.insert(it.slot).second) LLM_THROW(InvalidArg, "slot %d appears twice in one step", it.slot);
    const int n = (int)it.tokens.size();
    if (n == 0) LLM_THROW(InvalidArg, "slot %d: a sequence in a step brings at least one token", it.slot);
    const int past = cache_->length(it.slot);     // throws if the slot is not open
    if ((int64_t)past + n > max_seq_len_)
      LLM_THROW(InvalidArg, "slot %d: %d + %d tokens exceed the longest sequence this engine holds (%lld)", it.slot, past, n,
                (long long)max_seq_len_);
    if (it.fed_row >= 0) {
      if (n != 1 || it.fed_row >= last_capacity_)
        LLM_THROW(InvalidArg, "slot %d: a fed token is one token from a row of the last step", it.slot);
    } else {
      for (int t : it.tokens)
        if (t < 0 || t >= V) LLM_THROW(InvalidArg, "slot %d: token id %d outside the vocabulary (%lld)", it.slot, t, (long long)V);
    }
    for (int w : it.want)
      if (w < 0 || w >= n) LLM_THROW(InvalidArg, "slot %d: wanted place %d outside the %d tokens given", it.slot, w, n);
  }
}

// ---------------------------------------------------------------- descriptor
void Engine::fill(Descriptor &d, const std::vector<Piece> &pieces, const std::vector<StepItem> &items,
                  const std::vector<int> &want_rows, const float *uniforms, int n_uniforms) {
  int *tokens = d.host(Descriptor::Tokens), *tok_seq = d.host(Descriptor::TokSeq), *tok_pos = d.host(Descriptor::TokPos);
  int *seq_start = d.host(Descriptor::SeqStart), *seq_past = d.host(Descriptor::SeqPast), *seq_slot = d.host(Descriptor::SeqSlot);
  int *fed = d.host(Descriptor::Fed);
  int o = 0;
  std::vector<int> slots;
  for (size_t b = 0; b < pieces.size(); ++b) {
    const Piece &p = pieces[b];
    const StepItem &it = items[(size_t)p.index];
    if (it.fed_row >= 0) {
      tokens[o] = 0;
      fed[o] = it.fed_row;
    } else {
      for (int i = 0; i < p.count; ++i) {
        tokens[o + i] = it.tokens[(size_t)(p.start + i)];
        fed[o + i] = -1;
      }
    }
    for (int i = 0; i < p.count; ++i) {
      tok_seq[o + i] = (int)b;
      tok_pos[o + i] = p.past + p.start + i;
    }
    seq_start[b] = o;
    seq_past[b] = p.past + p.start;
    seq_slot[b] = p.slot;
    slots.push_back(p.slot);
    o += p.count;
  }
  seq_start[pieces.size()] = o;
  std::copy(want_rows.begin(), want_rows.end(), d.host(Descriptor::Want));
  if (uniforms) memcpy(d.host(Descriptor::Uniforms), uniforms, sizeof(float) * (size_t)n_uniforms);
  for (size_t g = 0; g < d.widths.size(); ++g) cache_->page_table((int)g, slots, d.widths[g], d.host(Descriptor::Tables + (int)g));
}

StepContext Engine::context(Descriptor &d, const std::vector<Piece> &pieces, int n_want, bool decode_only, int max_kv_len,
                            Arena *arena, std::vector<const int *> *tables) {
  StepContext ctx;
  ctx.dtype = model_->dtype();
  ctx.stream = stream_;
  ctx.n_tokens = d.n_tokens;
  ctx.n_seqs = (int)pieces.size();
  ctx.n_want = n_want;
  ctx.tokens = d.dev(Descriptor::Tokens);
  ctx.tok_seq = d.dev(Descriptor::TokSeq);
  ctx.tok_pos = d.dev(Descriptor::TokPos);
  ctx.seq_start = d.dev(Descriptor::SeqStart);
  ctx.seq_past = d.dev(Descriptor::SeqPast);
  ctx.seq_slot = d.dev(Descriptor::SeqSlot);
  ctx.want_rows = d.dev(Descriptor::Want);
  int max_q = 0;
  for (const auto &p : pieces) {
    ctx.q_lens.push_back(p.count);
    ctx.past_lens.push_back(p.past + p.start);
    ctx.slots.push_back(p.slot);
    max_q = std::max(max_q, p.count);
  }
  ctx.max_q_len = max_q;
  ctx.max_kv_len = max_kv_len;
  ctx.decode_only = decode_only;
  ctx.arena = arena;
  ctx.tc_status = status_.as<int>();
  ctx.zero_counters = counters_.as<int>();
  ctx.n_zero_counters = 1 << 18;
  ctx.sm_count = sm_count_;
  // Steps of single tokens in bfloat16 queue their products and norms and launch them together.
  ctx.chain = nullptr;
  if (decode_only && ctx.dtype == DType::BF16 && fast_switches().gemm_tc && fast_switches().gemm_chain &&
      kernels::available("gemm_chain") && d.n_tokens <= kernels::gemm_chain_max_tokens()) {
    if (chain_) chain_launches_ += chain_->launches();
    chain_.reset(new Chain(counters_.as<int>() + (1 << 18), status_.as<int>()));
    ctx.chain = chain_.get();
  }
  tables->clear();
  for (size_t g = 0; g < d.widths.size(); ++g) tables->push_back(d.dev(Descriptor::Tables + (int)g));
  return ctx;
}

void Engine::sample(const Act &logits, const SamplingParams &s, const float *uniforms_dev, int *out) {
  if (s.greedy()) kernels::argmax((const float *)logits.data, logits.ld, (int)logits.rows, (int)logits.cols, out, stream_);
  else kernels::sample((const float *)logits.data, logits.ld, (int)logits.rows, (int)logits.cols, s.temperature, s.top_k, s.top_p,
                       uniforms_dev, out, stream_);
}

// ---------------------------------------------------------------- the step
StepResult Engine::step(const std::vector<StepItem> &items, const SamplingParams *sampling, const float *uniforms) {
  make_current();
  if (items.empty()) LLM_THROW(InvalidArg, "a step needs at least one sequence");
  validate(items);
  if (sampling) sampling->validate();
  // Pages first: either the whole step fits the cache or nothing changes.
  std::vector<std::pair<int, int>> growth;
  bool decode_only = true;
  for (const auto &it : items) {
    growth.push_back({it.slot, cache_->length(it.slot) + (int)it.tokens.size()});
    decode_only = decode_only && it.tokens.size() == 1;
  }
  cache_->reserve(growth);
  StepResult out;
  if (decode_only && opt_.use_graphs && model_->capturable() && (int)items.size() <= opt_.max_step_tokens)
    out = run_decode_graph(items, sampling, uniforms);
  else
    out = run_eager(items, sampling, uniforms);
  ++steps_run_;
  return out;
}

void Engine::read_logits(const StepResult &r, float *host) {
  make_current();
  if (r.n_rows > 0 && r.logits)
    LLM_CUDA(cudaMemcpyAsync(host, r.logits, sizeof(float) * (size_t)r.n_rows * (size_t)vocab(), cudaMemcpyDeviceToHost, stream_));
  check_status();
}

void Engine::read_tokens(const StepResult &r, int *host) {
  make_current();
  if (r.n_rows > 0 && r.tokens) LLM_CUDA(cudaMemcpyAsync(host, r.tokens, sizeof(int) * (size_t)r.n_rows, cudaMemcpyDeviceToHost, stream_));
  check_status();
}

// ---------------------------------------------------------------- eager path (prompts, mixed steps)
StepResult Engine::run_eager(const std::vector<StepItem> &items, const SamplingParams *sampling, const float *uniforms) {
  // Pieces: the step's tokens in launch sequences of at most max_step_tokens, cut inside a prompt
  // where need be.
  std::vector<std::vector<Piece>> chunks(1);
  int room = opt_.max_step_tokens;
  for (size_t i = 0; i < items.size(); ++i) {
    const int past = cache_->length(items[i].slot);
    const int n = (int)items[i].tokens.size();
    int start = 0;
    while (start < n) {
      if (room == 0) {
        chunks.emplace_back();
        room = opt_.max_step_tokens;
      }
      const int c = std::min(room, n - start);
      chunks.back().push_back({(int)i, items[i].slot, start, c, past});
      start += c;
      room -= c;
    }
  }
  std::vector<int> want_base(items.size() + 1, 0);
  for (size_t i = 0; i < items.size(); ++i) want_base[i + 1] = want_base[i] + (int)items[i].want.size();
  const int W = want_base.back();
  const int64_t V = vocab();
  scratch_.compact();
  layer_scratch_[0].compact();
  layer_scratch_[1].compact();
  results_.compact();
  results_.reset();
  float *all_logits = W ? results_.alloc_n<float>((size_t)W * (size_t)V) : nullptr;
  int *all_tokens = (sampling && W) ? results_.alloc_n<int>((size_t)W) : nullptr;

  for (const auto &pieces : chunks) {
    int T = 0;
    for (const auto &p : pieces) T += p.count;
    // wanted rows of this launch sequence, with the place each has in the step's result
    std::vector<int> want_rows, global;
    std::vector<float> uni;
    int o = 0, max_kv = 0, need_pages = 0;
    for (const auto &p : pieces) {
      const StepItem &it = items[(size_t)p.index];
      for (size_t j = 0; j < it.want.size(); ++j) {
        const int w = it.want[j];
        if (w >= p.start && w < p.start + p.count) {
          want_rows.push_back(o + w - p.start);
          global.push_back(want_base[(size_t)p.index] + (int)j);
          uni.push_back(uniforms ? uniforms[(size_t)global.back()] : 0.f);
        }
      }
      o += p.count;
      max_kv = std::max(max_kv, p.past + p.start + p.count);
      // every page the slot holds: the step's pages were all taken before its first launch sequence
      need_pages = std::max(need_pages, cache_->pages_needed(p.slot));
    }
    const int width = std::max(8, (need_pages + 7) / 8 * 8);
    Descriptor &d = *eager_desc_[eager_turn_];
    eager_turn_ = (eager_turn_ + 1) % eager_desc_.size();
    d.shape(T, (int)pieces.size(), (int)want_rows.size(), std::vector<int>(cache_->groups().size(), width));
    fill(d, pieces, items, want_rows, uni.data(), (int)uni.size());
    d.upload(stream_);
    last_h2d_ = (long long)(d.words() * sizeof(int));
    last_d2h_ = 0;
    bool all_single = true;
    for (const auto &p : pieces) all_single = all_single && p.count == 1;
    std::vector<const int *> tables;
    scratch_.reset();
    StepContext ctx = context(d, pieces, (int)want_rows.size(), all_single, max_kv, &scratch_, &tables);
    ctx.layer_arenas[0] = &layer_scratch_[0];
    ctx.layer_arenas[1] = &layer_scratch_[1];
    Act logits = model_->forward(ctx, *cache_, tables, width, last_tokens_.as<int>(), d.dev(Descriptor::Fed));
    int *chunk_tokens = nullptr;
    if (sampling && !want_rows.empty()) {
      chunk_tokens = scratch_.alloc_n<int>(want_rows.size());
      sample(logits, *sampling, (const float *)d.dev(Descriptor::Uniforms), chunk_tokens);
    }
    // into the step's result, in runs of rows that are neighbours there too
    for (size_t a = 0; a < global.size();) {
      size_t b = a + 1;
      while (b < global.size() && global[b] == global[b - 1] + 1) ++b;
      LLM_CUDA(cudaMemcpyAsync(all_logits + (size_t)global[a] * (size_t)V, (const float *)logits.data + a * (size_t)V,
                               sizeof(float) * (b - a) * (size_t)V, cudaMemcpyDeviceToDevice, stream_));
      if (chunk_tokens)
        LLM_CUDA(cudaMemcpyAsync(all_tokens + global[a], chunk_tokens + a, sizeof(int) * (b - a), cudaMemcpyDeviceToDevice, stream_));
      a = b;
    }
    for (const auto &p : pieces) cache_->commit(p.slot, p.past + p.start + p.count);
  }
  StepResult r;
  r.logits = all_logits;
  r.n_rows = W;
  r.tokens = all_tokens;
  return r;
}

// ---------------------------------------------------------------- graph path (one token each)
Act Engine::graph_body(DecodeGraph &g) {
  Descriptor &d = g.desc;
  kernels::copy_words(d.host_base(), d.dev_base(), (int)d.words(), stream_);
  // stand-in pieces: the launches depend on the step's shape alone
  std::vector<Piece> pieces;
  for (int i = 0; i < g.batch; ++i) pieces.push_back({i, 0, 0, 1, 0});
  std::vector<const int *> tables;
  g.arena.reset();
  StepContext ctx = context(d, pieces, g.batch, true, g.width * opt_.page_size, &g.arena, &tables);
  ctx.captured = true;
  Act logits = model_->forward(ctx, *cache_, tables, g.width, last_tokens_.as<int>(), d.dev(Descriptor::Fed));
  if (g.sampled) {
    sample(logits, g.sampling, (const float *)d.dev(Descriptor::Uniforms), last_tokens_.as<int>());
    kernels::gather_words(last_tokens_.as<int>(), g.batch, status_.as<int>(), 1, g.host_tokens.as<int>(), stream_);
  }
  return logits;
}

StepResult Engine::run_decode_graph(const std::vector<StepItem> &items, const SamplingParams *sampling, const float *uniforms) {
  const int B = (int)items.size();
  std::vector<Piece> pieces;
  int need_pages = 1;
  for (int i = 0; i < B; ++i) {
    const int past = cache_->length(items[(size_t)i].slot);
    pieces.push_back({i, items[(size_t)i].slot, 0, 1, past});
    need_pages = std::max(need_pages, (past + 1 + opt_.page_size - 1) / opt_.page_size);
  }
  int width = 8;
  while (width < need_pages) width *= 2;
  GraphKey key{B, width, sampling != nullptr, sampling ? *sampling : SamplingParams()};
  // Each shape has two graphs taken in turn: while one step runs, the next one's descriptor is
  // written into the other graph's staging, and a step's tokens are read while the other runs.
  int &turn = graph_turn_[key];
  auto &table = graphs_[turn];
  turn ^= 1;
  std::unique_ptr<DecodeGraph> &slot = table[key];
  const bool fresh = !slot;
  if (fresh) {
    slot.reset(new DecodeGraph());
    slot->batch = B;
    slot->width = width;
    slot->sampled = sampling != nullptr;
    if (sampling) slot->sampling = *sampling;
    slot->desc.shape(B, B, B, std::vector<int>(cache_->groups().size(), width));
    if (sampling) slot->host_tokens.allocate(sizeof(int) * ((size_t)B + 1));
  }
  DecodeGraph &g = *slot;
  // Logits are computed for every sequence; the wanted ones are picked afterwards.
  std::vector<int> rows, all_rows((size_t)B);
  std::iota(all_rows.begin(), all_rows.end(), 0);
  std::vector<float> uni((size_t)B, 0.f);
  int k = 0;
  for (int i = 0; i < B; ++i)
    if (!items[(size_t)i].want.empty()) {
      rows.push_back(i);
      if (sampling && uniforms) uni[(size_t)i] = uniforms[k];
      ++k;
    }
  g.desc.wait_host_free();
  fill(g.desc, pieces, items, all_rows, uni.data(), B);
  if (fresh) {
    // First use: the step runs once outside capture (which also sets kernel attributes and sizes
    // the arena) and its results are this call's results; then the same launches are captured,
    // which executes nothing.  The step must not run twice: a mixer with state of its own would
    // advance twice.
    bool capturing = false;
    try {
      g.logits = graph_body(g);
      LLM_CUDA(cudaStreamSynchronize(stream_));
      g.arena.set_frozen(true);
      LLM_CUDA(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal));
      capturing = true;
      const Act again = graph_body(g);
      capturing = false;
      LLM_CUDA(cudaStreamEndCapture(stream_, &g.graph));
      LLM_CUDA(cudaGraphInstantiate(&g.exec, g.graph, 0));
      if (again.data != g.logits.data)
        LLM_THROW(Extension, "a captured step put its logits elsewhere than its first run (a part allocates differently from run to run)");
    } catch (...) {
      if (capturing) {
        cudaGraph_t broken = nullptr;
        cudaStreamEndCapture(stream_, &broken);
        if (broken) cudaGraphDestroy(broken);
        cudaGetLastError();
      }
      table.erase(key);
      throw;
    }
    ++graphs_captured_;
  } else {
    LLM_CUDA(cudaGraphLaunch(g.exec, stream_));
    ++graph_replays_;
  }
  g.desc.in_flight(stream_);         // the staging is free, and the tokens are out, when this launch is done
  last_h2d_ = (long long)(g.desc.words() * sizeof(int));
  last_d2h_ = g.sampled ? (long long)sizeof(int) * (B + 1) : 0;
  last_graph_ = &g;
  for (const auto &p : pieces) cache_->commit(p.slot, p.past + 1);
  StepResult r;
  const int64_t V = vocab();
  if ((int)rows.size() == B) {
    r.logits = (const float *)g.logits.data;
    r.tokens = sampling ? last_tokens_.as<int>() : nullptr;
    r.n_rows = B;
    return r;
  }
  // some sequences want nothing: the others' rows, gathered
  results_.reset();
  float *picked = rows.empty() ? nullptr : results_.alloc_n<float>(rows.size() * (size_t)V);
  int *picked_tokens = (sampling && !rows.empty()) ? results_.alloc_n<int>(rows.size()) : nullptr;
  for (size_t i = 0; i < rows.size(); ++i) {
    LLM_CUDA(cudaMemcpyAsync(picked + i * (size_t)V, (const float *)g.logits.data + (size_t)rows[i] * (size_t)V, sizeof(float) * (size_t)V,
                             cudaMemcpyDeviceToDevice, stream_));
    if (picked_tokens)
      LLM_CUDA(cudaMemcpyAsync(picked_tokens + i, last_tokens_.as<int>() + rows[i], sizeof(int), cudaMemcpyDeviceToDevice, stream_));
  }
  r.logits = picked;
  r.tokens = picked_tokens;
  r.n_rows = (int)rows.size();
  return r;
}

// ---------------------------------------------------------------- sampled steps whose tokens come later
PendingTokens Engine::step_tokens(const std::vector<StepItem> &items, const SamplingParams &sampling, const float *uniforms) {
  for (const auto &it : items)
    if (it.want.size() != 1) LLM_THROW(InvalidArg, "step_tokens: every item wants exactly one place");
  const int n = (int)items.size();
  if (n > last_capacity_) LLM_THROW(InvalidArg, "step_tokens: %d sequences, at most %d are taken", n, last_capacity_);
  last_graph_ = nullptr;
  StepResult r = step(items, &sampling, uniforms);
  PendingTokens p;
  p.engine_ = this;
  p.n_ = n;
  if (last_graph_ && last_graph_->sampled && r.tokens == last_tokens_.as<int>()) {
    // the graph has copied them out itself; its buffer is read before the graph runs again
    p.host_ = last_graph_->host_tokens.as<int>();
    p.done_ = last_graph_->desc.event();
    return p;
  }
  if (r.tokens != last_tokens_.as<int>())
    LLM_CUDA(cudaMemcpyAsync(last_tokens_.get(), r.tokens, sizeof(int) * (size_t)n, cudaMemcpyDeviceToDevice, stream_));
  HostTokens &h = token_ring_[token_turn_];
  token_turn_ = (token_turn_ + 1) % token_ring_.size();
  LLM_CUDA(cudaEventSynchronize(h.done));          // its last reader is long gone; this only orders the reuse
  LLM_CUDA(cudaMemcpyAsync(h.buf.get(), last_tokens_.get(), sizeof(int) * (size_t)n, cudaMemcpyDeviceToHost, stream_));
  LLM_CUDA(cudaMemcpyAsync(h.buf.as<int>() + n, status_.get(), sizeof(int), cudaMemcpyDeviceToHost, stream_));
  LLM_CUDA(cudaEventRecord(h.done, stream_));
  p.host_ = h.buf.as<int>();
  p.done_ = h.done;
  return p;
}

std::vector<int> PendingTokens::result() {
  if (!engine_) LLM_THROW(InvalidArg, "no step is pending");
  engine_->make_current();
  LLM_CUDA(cudaEventSynchronize(done_));
  const int code = host_[n_];
  if (code) engine_->raise_status(code);
  return std::vector<int>(host_, host_ + n_);
}

}  // namespace llm
