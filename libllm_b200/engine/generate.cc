#include "engine/generate.h"

#include <map>

#include "sampling/rng.h"

namespace llm {

std::vector<std::vector<int>> plan_batches(const std::vector<int> &prompt_lengths, const std::vector<int> &max_new_tokens,
                                           int64_t capacity_tokens, int max_batch, int page_size, int64_t max_seq_len) {
  std::vector<std::vector<int>> batches(1);
  int64_t used = 0;
  for (size_t i = 0; i < prompt_lengths.size(); ++i) {
    const int n = prompt_lengths[i], m = max_new_tokens[i];
    if (n < 1) LLM_THROW(InvalidArg, "request %zu: a prompt needs at least one token", i);
    if (m < 0) LLM_THROW(InvalidArg, "request %zu: max_new_tokens must not be negative", i);
    const int64_t total = (int64_t)n + m;
    if (max_seq_len > 0 && total > max_seq_len)
      LLM_THROW(InvalidArg, "request %zu: %d prompt + %d new tokens exceed the longest sequence (%lld)", i, n, m, (long long)max_seq_len);
    const int64_t need = (total + page_size - 1) / page_size * page_size;
    if (need > capacity_tokens)
      LLM_THROW(Cache, "request %zu needs room for %lld tokens, the cache holds %lld", i, (long long)need, (long long)capacity_tokens);
    if (!batches.back().empty() && (used + need > capacity_tokens || (int)batches.back().size() >= max_batch)) {
      batches.emplace_back();
      used = 0;
    }
    batches.back().push_back((int)i);
    used += need;
  }
  if (batches.back().empty()) batches.pop_back();
  return batches;
}

StopDecision should_stop(int token, int n_generated, int max_new_tokens, const std::set<int> &stop_tokens) {
  if (stop_tokens.count(token)) return {true, false};
  return {n_generated + 1 >= max_new_tokens, true};
}

std::vector<std::vector<int>> generate(Engine &engine, const std::vector<std::vector<int>> &prompts,
                                       const std::vector<int> &max_new_tokens, const GenerateOptions &opt) {
  const size_t n = prompts.size();
  std::vector<int> limits;
  if (max_new_tokens.size() == 1) limits.assign(n, max_new_tokens[0]);
  else limits = max_new_tokens;
  if (limits.size() != n) LLM_THROW(InvalidArg, "max_new_tokens: one number, or one per prompt");
  std::set<int> stops;
  if (opt.use_model_stop_tokens) stops.insert(engine.model().spec().stop_tokens.begin(), engine.model().spec().stop_tokens.end());
  else stops.insert(opt.stop_tokens.begin(), opt.stop_tokens.end());
  opt.sampling.validate();
  std::vector<std::vector<int>> out(n);
  std::vector<int> lengths;
  for (const auto &p : prompts) lengths.push_back((int)p.size());
  const int page = engine.cache().page_size();
  const int64_t capacity = (int64_t)engine.cache().n_pages() * page;
  const auto batches = plan_batches(lengths, limits, capacity, opt.max_batch, page, engine.max_seq_len());

  for (const auto &batch : batches) {
    std::vector<int> live;
    for (int i : batch)
      if (limits[(size_t)i] > 0) live.push_back(i);
    if (live.empty()) continue;
    std::map<int, int> slots, produced;
    try {
      for (int i : live) {
        slots[i] = engine.open_sequence();
        produced[i] = 0;
      }
      // The step that is running on the device: (request ids in row order, pending tokens).  While
      // the host waits for its tokens, the next step is already queued behind it with every
      // sequence that can still go on; it takes its tokens from the device.  A sequence that turns
      // out to have ended (a stop token) has then run one step too many: its result is dropped and
      // its slot is given back, nothing else sees it.
      std::vector<StepItem> items;
      std::vector<float> uni;
      for (int i : live) {
        StepItem it;
        it.slot = slots[i];
        it.tokens = prompts[(size_t)i];
        it.want = {(int)prompts[(size_t)i].size() - 1};
        items.push_back(std::move(it));
        uni.push_back(uniform(opt.seed, (uint64_t)i, 0));
      }
      std::vector<int> ids = live;
      PendingTokens pending = engine.step_tokens(items, opt.sampling, uni.data());
      std::set<int> ended;
      bool running = true;
      while (running) {
        // queue the next step: the sequences of this one that have not reached their count
        std::vector<int> next_ids;
        PendingTokens next_pending;
        items.clear();
        uni.clear();
        for (size_t row = 0; row < ids.size(); ++row) {
          const int i = ids[row];
          if (ended.count(i) || produced[i] + 1 >= limits[(size_t)i]) continue;
          StepItem it;
          it.slot = slots[i];
          it.tokens = {0};
          it.want = {0};
          it.fed_row = (int)row;
          items.push_back(std::move(it));
          uni.push_back(uniform(opt.seed, (uint64_t)i, (uint64_t)produced[i] + 1));
          next_ids.push_back(i);
        }
        if (!items.empty()) next_pending = engine.step_tokens(items, opt.sampling, uni.data());
        // now this step's tokens (the one device-to-host read of the step)
        const std::vector<int> tokens = pending.result();
        for (size_t row = 0; row < ids.size(); ++row) {
          const int i = ids[row];
          if (ended.count(i)) continue;                 // it ran one step beyond its end
          const StopDecision d = should_stop(tokens[row], produced[i], limits[(size_t)i], stops);
          if (d.emit) {
            out[(size_t)i].push_back(tokens[row]);
            ++produced[i];
            if (opt.on_token) opt.on_token(i, tokens[row]);
          }
          if (d.ends) {
            ended.insert(i);
            engine.close_sequence(slots[i]);
            slots.erase(i);
          }
        }
        running = next_pending.valid();
        ids = next_ids;
        pending = next_pending;
      }
    } catch (...) {
      for (auto &kv : slots) {
        try {
          engine.close_sequence(kv.second);
        } catch (...) {
        }
      }
      throw;
    }
    for (auto &kv : slots) engine.close_sequence(kv.second);
  }
  return out;
}

// ---------------------------------------------------------------- one prompt, token by token
Completion::Completion(Engine &engine, std::vector<int> prompt, int max_new_tokens, const SamplingParams &sampling, uint64_t seed,
                       const std::set<int> &stop_tokens)
    : engine_(engine), prompt_(std::move(prompt)), sampling_(sampling), seed_(seed), stops_(stop_tokens) {
  if (prompt_.empty()) LLM_THROW(InvalidArg, "a prompt needs at least one token");
  sampling_.validate();
  const int64_t room = engine.max_seq_len() - (int64_t)prompt_.size();
  if (room < 0)
    LLM_THROW(InvalidArg, "the prompt of %zu tokens exceeds the longest sequence (%lld)", prompt_.size(), (long long)engine.max_seq_len());
  limit_ = (int)std::max<int64_t>(0, std::min<int64_t>(max_new_tokens, room));
}

Completion::~Completion() { finish(); }

void Completion::finish() {
  if (slot_ >= 0) {
    try {
      if (running_.valid()) running_.result();      // let a step that is under way end before its pages go back
    } catch (...) {
    }
    try {
      engine_.close_sequence(slot_);
    } catch (...) {
    }
    slot_ = -1;
  }
  ended_ = true;
}

bool Completion::next(int *token) {
  if (ended_ || limit_ <= 0) {
    finish();
    return false;
  }
  if (!started_) {
    started_ = true;
    slot_ = engine_.open_sequence();
    StepItem it;
    it.slot = slot_;
    it.tokens = prompt_;
    it.want = {(int)prompt_.size() - 1};
    const float u = uniform(seed_, 0, 0);
    running_ = engine_.step_tokens({it}, sampling_, &u);
  }
  // queue the step after this one before reading this one's token
  PendingTokens current = running_;
  running_ = PendingTokens();
  if (produced_ + 1 < limit_) {
    StepItem it;
    it.slot = slot_;
    it.tokens = {0};
    it.want = {0};
    it.fed_row = 0;
    const float u = uniform(seed_, 0, (uint64_t)produced_ + 1);
    running_ = engine_.step_tokens({it}, sampling_, &u);
  }
  const int tok = current.result()[0];
  const StopDecision d = should_stop(tok, produced_, limit_, stops_);
  if (d.emit) {
    *token = tok;
    ++produced_;
  }
  if (d.ends) finish();
  return d.emit;
}

}  // namespace llm
