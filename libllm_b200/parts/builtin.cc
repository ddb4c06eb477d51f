// The parts the library brings: RMSNorm, rotary position encoding, grouped-query attention over
// the paged cache, the dense SwiGLU feed-forward and the pre-norm block.
#include <cmath>

#include "config/config.h"
#include "csrc/kernels.h"
#include "parts/chain.h"
#include "parts/linear.h"
#include "parts/part.h"
#include "util/log.h"

namespace llm {

namespace {

ConfigReader reader_of(const Json &spec, const char *what) { return ConfigReader(spec, std::string(what) + " description"); }

// ---------------------------------------------------------------- RMSNorm
// y = x * w / sqrt(mean(x^2) + eps), sums and scaling in 32-bit (src/flint/cpu/normalizations.cc:52-64,
// src/flint/cuda/rms_norm.cu:59-75).  Before the norm the stream's pending addition is applied in
// 32-bit: the reference's separate residual add (src/libllm/llama.cc:252-266).
class RMSNorm : public Norm {
 public:
  RMSNorm(const Json &spec, const BuildEnv &env) : Norm(spec, env) {
    ConfigReader r = reader_of(spec, "rmsnorm");
    size_ = r.integer("size");
    eps_ = r.number("eps");
    name_ = r.string("weight");
  }
  std::vector<TensorNeed> tensor_needs() const override { return {{name_, {size_}, TensorRole::Vector, false}}; }
  void load(const Loader &l) override { weight_ = l.fetch(tensor_needs()[0]); }
  std::vector<std::string> kernel_families() const override { return {"elementwise"}; }
  Act forward(StepContext &ctx, ResidualStream &stream, const int *rows, int n_rows) override {
    const int64_t n = rows ? n_rows : stream.rows;
    Act out = ctx.arena->act(ctx.dtype, n, size_);
    if (ctx.chain && ctx.dtype == DType::BF16 &&
        ctx.chain->add_norm(stream.resid, stream.pending.data ? &stream.pending : nullptr, weight_.buf.as<float>(), (float)eps_,
                            out.data, rows, (int)n, (int)size_, ctx.stream)) {
      if (!rows) stream.pending = Act();
      return out;
    }
    flush_chain(ctx);
    kernels::add_rmsnorm(stream.resid, stream.pending.data ? &stream.pending : nullptr, weight_.buf.as<float>(), (float)eps_,
                         out.data, ctx.dtype, rows, (int)n, (int)size_, ctx.stream);
    if (!rows) stream.pending = Act();
    return out;
  }

 private:
  int64_t size_;
  double eps_;
  std::string name_;
  Weight weight_;
};

// ---------------------------------------------------------------- rotary position encoding
// f_i = theta^(-2i/d) for i < d/2.  With llama3 scaling a frequency whose wavelength 2*pi/f is
// shorter than original/high_freq_factor is kept, one longer than original/low_freq_factor is
// divided by `factor`, and between them the two are blended linearly in original/wavelength.  The
// reference takes the finished cos/sin table from the checkpoint's own rotary module
// (tools/llama_exporter.py:54-62).
}  // namespace

std::vector<double> rotary_frequencies(int64_t rotary_dim, double theta, const Json &scaling) {
  std::vector<double> freqs;
  for (int64_t i = 0; i < rotary_dim / 2; ++i) freqs.push_back(std::pow(theta, -2.0 * (double)i / (double)rotary_dim));
  if (scaling.is_null()) return freqs;
  ConfigReader r(scaling, "rope description: scaling");
  const std::string type = r.string_or("rope_type", "llama3");
  if (type != "llama3") LLM_THROW(Config, "rope scaling '%s' is not supported", type.c_str());
  const double orig = (double)r.integer("original_max_position_embeddings");
  const double lo = r.number("low_freq_factor"), hi = r.number("high_freq_factor"), factor = r.number("factor");
  for (auto &f : freqs) {
    const double wavelen = 2.0 * M_PI / f;
    if (wavelen < orig / hi) continue;
    if (wavelen > orig / lo) {
      f = f / factor;
    } else {
      const double s = (orig / wavelen - lo) / (hi - lo);
      f = (1.0 - s) * f / factor + s * f;
    }
  }
  return freqs;
}

namespace {

// Holds table[p] = (cos(p*f_0..), sin(p*f_0..)), [positions, rotary_dim] in 32-bit, computed in
// 64-bit and rounded once; it stands for the reference's stored `rope` tensor
// (src/libllm/llama.cc:282-283).  The rotation pairs channel i with i + rotary_dim/2
// (src/libllm/llama.cc:151-176).  Parts with the same description share one table.
class RotaryEmbedding : public PositionEncoding {
 public:
  RotaryEmbedding(const Json &spec, const BuildEnv &env) : PositionEncoding(spec, env) {
    ConfigReader r = reader_of(spec, "rope");
    head_dim_ = r.integer("head_dim");
    rotary_dim_ = r.integer_or("rotary_dim", head_dim_);
    theta_ = r.number_or("theta", 10000.0);
    if (rotary_dim_ % 2 || rotary_dim_ > head_dim_ || rotary_dim_ <= 0)
      LLM_THROW(Config, "rotary width %lld does not fit head size %lld", (long long)rotary_dim_, (long long)head_dim_);
    rotary_frequencies(rotary_dim_, theta_, spec.get("scaling"));     // checks the scaling's keys
  }
  std::vector<std::string> kernel_families() const override { return {"rope"}; }
  void load(const Loader &) override {
    const std::string key = "rope:" + spec_.dump() + ":" + std::to_string(env_.max_positions);
    if (env_.shared) {
      auto it = env_.shared->find(key);
      if (it != env_.shared->end()) {
        table_ = it->second;
        return;
      }
    }
    const std::vector<double> freqs = rotary_frequencies(rotary_dim_, theta_, spec_.get("scaling"));
    const int64_t half = rotary_dim_ / 2, P = env_.max_positions;
    std::vector<float> host((size_t)(P * rotary_dim_));
    for (int64_t p = 0; p < P; ++p)
      for (int64_t i = 0; i < half; ++i) {
        const double a = (double)p * freqs[(size_t)i];
        host[(size_t)(p * rotary_dim_ + i)] = (float)std::cos(a);
        host[(size_t)(p * rotary_dim_ + half + i)] = (float)std::sin(a);
      }
    table_ = std::make_shared<Weight>();
    table_->dtype = DType::F32;
    table_->rows = P;
    table_->cols = rotary_dim_;
    table_->buf.allocate(host.size() * sizeof(float));
    LLM_CUDA(cudaMemcpy(table_->buf.get(), host.data(), host.size() * sizeof(float), cudaMemcpyHostToDevice));
    if (env_.shared) (*env_.shared)[key] = table_;
  }
  void rotate_and_store(StepContext &ctx, const Act &qkv, const Act &q_out, const QkvLayout &l, LayerCache &cache) override {
    kernels::rope_cache_write(qkv, q_out, l.n_heads, l.n_kv_heads, l.head_dim, table_->buf.as<float>(), (int)table_->rows,
                              (int)rotary_dim_, ctx.tok_seq, ctx.tok_pos, cache.page_table, cache.table_width, cache.k, cache.v,
                              cache.page_size, cache.writes, ctx.stream);
  }
  const float *half_split_table(int *rows, int *rotary_dim) const override {
    if (!table_) return nullptr;
    *rows = (int)table_->rows;
    *rotary_dim = (int)rotary_dim_;
    return table_->buf.as<float>();
  }

 private:
  int64_t head_dim_, rotary_dim_;
  double theta_;
  std::shared_ptr<Weight> table_;
};

// ---------------------------------------------------------------- attention
// q, k, v from one stacked product, rotation of q and k, append to the cache,
// softmax(q k^T / sqrt(d)) v per head with a causal mask, output projection
// (src/libllm/llama.cc:178-225).  The stacked matrix is [Wq; Wk; Wv] as the reference's exporter
// builds it (tools/llama_exporter.py:64-71), made here when the weights are loaded.  The position
// part owns the rotation; without one, queries and keys are used as they come.
class Attention : public Mixer {
 public:
  Attention(const Json &spec, const BuildEnv &env) : Mixer(spec, env) {
    ConfigReader r = reader_of(spec, "attention");
    hidden_ = r.integer("hidden");
    n_heads_ = (int)r.integer("n_heads");
    n_kv_ = (int)r.integer_or("n_kv_heads", n_heads_);
    d_ = (int)r.integer("head_dim");
    window_ = (int)r.integer_or("window", 0, 0);
    bias_ = r.boolean_or("bias", false);
    scale_ = (float)r.number_or("scale", 1.0 / std::sqrt((double)d_));
    q_name_ = r.string("q");
    k_name_ = r.string("k");
    v_name_ = r.string("v");
    o_name_ = r.string("o");
    if (n_heads_ % n_kv_) LLM_THROW(Config, "attention: %d heads are not a multiple of %d groups", n_heads_, n_kv_);
    if (d_ % 16 || d_ < 16 || d_ > 256)
      LLM_THROW(Unsupported, "attention: head size %d is not supported (multiples of 16 from 16 to 256)", d_);
    if (r.integer_or("v_head_dim", d_) != d_)
      LLM_THROW(Unsupported, "attention: values of another width than the keys (%lld against %d) are not built",
                (long long)r.integer("v_head_dim"), d_);
    if (!spec.get("position").is_null()) position_ = build_as<PositionEncoding>("position", spec.get("position"), env);
    q_width_ = (int64_t)n_heads_ * d_;
    kv_width_ = (int64_t)n_kv_ * d_;
  }

  std::vector<TensorNeed> tensor_needs() const override {
    std::vector<TensorNeed> needs = {{q_name_, {q_width_, hidden_}}, {k_name_, {kv_width_, hidden_}}, {v_name_, {kv_width_, hidden_}},
                                     {o_name_, {hidden_, q_width_}}};
    if (bias_)
      for (const auto &p : {std::make_pair(q_name_, q_width_), std::make_pair(k_name_, kv_width_), std::make_pair(v_name_, kv_width_)}) {
        std::string n = p.first;
        const std::string suffix = "weight";
        if (n.size() >= suffix.size() && n.compare(n.size() - suffix.size(), suffix.size(), suffix) == 0) n.resize(n.size() - suffix.size());
        needs.push_back({n + "bias", {p.second}, TensorRole::Vector, false});
      }
    if (position_)
      for (auto &n : position_->tensor_needs()) needs.push_back(n);
    return needs;
  }

  void load(const Loader &l) override {
    const std::vector<TensorNeed> needs = tensor_needs();
    const size_t es = dtype_size(l.engine);
    w_qkv_.dtype = l.engine;
    w_qkv_.rows = q_width_ + 2 * kv_width_;
    w_qkv_.cols = hidden_;
    w_qkv_.buf.allocate((size_t)w_qkv_.rows * (size_t)hidden_ * es);
    char *p = (char *)w_qkv_.buf.get();
    l.fetch_into(needs[0], l.engine, p);
    l.fetch_into(needs[1], l.engine, p + (size_t)q_width_ * hidden_ * es);
    l.fetch_into(needs[2], l.engine, p + (size_t)(q_width_ + kv_width_) * hidden_ * es);
    w_o_ = l.fetch(needs[3]);
    if (bias_) {
      b_qkv_.dtype = DType::F32;
      b_qkv_.rows = 1;
      b_qkv_.cols = w_qkv_.rows;
      b_qkv_.buf.allocate((size_t)w_qkv_.rows * 4);
      float *b = b_qkv_.buf.as<float>();
      l.fetch_into(needs[4], DType::F32, b);
      l.fetch_into(needs[5], DType::F32, b + q_width_);
      l.fetch_into(needs[6], DType::F32, b + q_width_ + kv_width_);
      if (l.engine == DType::BF16) {
        static bool said = false;
        if (!said) {
          said = true;
          log_warning("attention with a bias: its q|k|v product runs on the CUDA cores in bfloat16 too (the tensor-core "
                      "product has no bias term)");
        }
      }
    }
    if (position_) position_->load(l);
  }

  std::vector<std::string> kernel_families() const override {
    std::vector<std::string> fams = product_families(env_.dtype);
    fams.push_back("rope");
    fams.push_back("attention_generic");
    if (env_.dtype != DType::BF16) return fams;
    const FastSwitches &f = fast_switches();
    const int group = n_heads_ / n_kv_;
    const bool tiled = env_.page_size == 64 && d_ % 16 == 0 && d_ >= 16 && d_ <= 128;
    if (f.prefill_attention_tc && env_.page_size == 64 && (d_ == 64 || d_ == 128)) fams.push_back("attention_prefill_tc");
    else if (f.prefill_attention && tiled) fams.push_back("attention_prefill");
    if (f.decode_attention_tc && tiled && group <= 16 && !bias_ && position_) fams.push_back("attention_decode_tc");
    else if (f.decode_attention && (d_ == 16 || d_ == 32 || d_ == 64 || d_ == 128) &&
             (group == 1 || group == 2 || group == 3 || group == 4 || group == 8))
      fams.push_back("attention_decode");
    return fams;
  }

  bool wants_cache() const override { return true; }
  CacheNeed cache_need() const override {
    CacheNeed n;
    n.kind = window_ > 0 ? "window" : "full";
    n.n_kv_heads = n_kv_;
    n.k_dim = n.v_dim = d_;
    n.window = window_;
    return n;
  }

  Act forward(StepContext &ctx, const Act &x, LayerCache *cache, StateView *) override {
    if (!cache) LLM_THROW(InvalidArg, "attention: the run has no cache to attend over");
    const FastSwitches &f = fast_switches();
    const int group = n_heads_ / n_kv_;
    // The products hand over 32-bit results: q and k are rounded to the engine's type once, after
    // the rotation, and the residual addition gets an unrounded term.
    int table_rows = 0, rot_dim = 0;
    const float *table = position_ ? position_->half_split_table(&table_rows, &rot_dim) : nullptr;
    const bool fused = table && !bias_ && ctx.decode_only && f.decode_attention_tc && ctx.dtype == DType::BF16 &&
                       kernels::available("attention_decode_tc") && kernels::attention_decode_tc_supported(d_, cache->page_size, group);
    Act qkv = linear(ctx, x, w_qkv_, bias_ ? b_qkv_.buf.as<float>() : nullptr, DType::F32, fused);
    flush_chain(ctx);
    if (fused) {
      const int max_len = std::max(ctx.max_kv_len, 1);
      const int pairs = std::max(1, ctx.n_seqs * n_kv_);
      const int slots = ctx.sm_count * kernels::attention_decode_tc_ctas_per_sm(d_);
      // As many key splits as fill the GPU once (all CTAs resident together), each of at least a
      // page at the longest length.  The kernel cuts every sequence's own length into that many
      // runs, so the number depends on the batch and the bound on the length, not on the lengths.
      const int n_splits = std::max(1, std::min(slots / pairs, std::max(1, max_len / cache->page_size)));
      Act out = ctx.arena->act(DType::BF16, ctx.n_tokens, q_width_);
      float *ws_o = nullptr, *ws_ml = nullptr;
      int *counters = nullptr;
      if (n_splits > 1) {
        ws_o = ctx.arena->alloc_n<float>((size_t)ctx.n_seqs * n_heads_ * n_splits * d_);
        ws_ml = ctx.arena->alloc_n<float>((size_t)ctx.n_seqs * n_heads_ * n_splits * 2);
        if (pairs > ctx.n_zero_counters)
          LLM_THROW(Unsupported, "fused decode attention: %d (sequence, kv head) pairs in one step, %d are provided for", pairs,
                    ctx.n_zero_counters);
        counters = ctx.zero_counters;
      }
      kernels::attention_decode_tc(qkv, table, table_rows, rot_dim, ctx.tok_pos, cache->page_table, cache->table_width, cache->k,
                                   cache->v, cache->writes, ctx.n_seqs, n_heads_, n_kv_, d_, cache->page_size, 0, max_len, n_splits,
                                   window_, scale_, ws_o, ws_ml, counters, out, ctx.stream);
      return linear(ctx, out, w_o_, nullptr, DType::F32, true);
    }
    Act q = ctx.arena->act(ctx.dtype, ctx.n_tokens, q_width_);
    const QkvLayout layout{n_heads_, n_kv_, d_};
    if (position_) {
      position_->rotate_and_store(ctx, qkv, q, layout, *cache);
    } else {
      kernels::rope_cache_write(qkv, q, n_heads_, n_kv_, d_, nullptr, 0, 0, ctx.tok_seq, ctx.tok_pos, cache->page_table,
                                cache->table_width, cache->k, cache->v, cache->page_size, cache->writes, ctx.stream);
    }
    Act out = ctx.arena->act(ctx.dtype, ctx.n_tokens, q_width_);
    bool done = false;
    if (ctx.dtype == DType::BF16) {
      if (ctx.decode_only && f.decode_attention && kernels::available("attention_decode") &&
          kernels::attention_decode_supported(d_, group)) {
        // enough CTAs to fill the GPU about eight times over at the longest length, runs of at
        // least two pages; the same for every step of a captured graph
        const int max_len = std::max(ctx.max_kv_len, 1);
        const int pairs = std::max(1, ctx.n_seqs * n_kv_);
        const int want = std::max(1, (8 * ctx.sm_count + pairs - 1) / pairs);
        const int most = std::max(1, max_len / (2 * cache->page_size));
        int n_splits = std::max(1, std::min(want, most));
        int chunk = (max_len + n_splits - 1) / n_splits;
        chunk = (chunk + cache->page_size - 1) / cache->page_size * cache->page_size;
        n_splits = std::max(1, (max_len + chunk - 1) / chunk);
        float *ws_o = nullptr, *ws_ml = nullptr;
        if (n_splits > 1) {
          ws_o = ctx.arena->alloc_n<float>((size_t)ctx.n_seqs * n_heads_ * n_splits * d_);
          ws_ml = ctx.arena->alloc_n<float>((size_t)ctx.n_seqs * n_heads_ * n_splits * 2);
        }
        kernels::attention_decode(q, out, cache->k, cache->v, ctx.tok_pos, cache->page_table, cache->table_width, n_heads_, n_kv_,
                                  d_, cache->page_size, chunk, n_splits, window_, scale_, ws_o, ws_ml, ctx.stream);
        done = true;
      } else if (f.prefill_attention_tc && (d_ == 64 || d_ == 128) && kernels::available("attention_prefill_tc") &&
                 kernels::attention_prefill_tc_supported(d_, cache->page_size)) {
        kernels::attention_prefill_tc(q, out, cache->k, cache->v, cache->n_pages, ctx.seq_start, ctx.seq_past, cache->page_table,
                                      cache->table_width, ctx.n_seqs, ctx.max_q_len, n_heads_, n_kv_, d_, cache->page_size, window_,
                                      scale_, ctx.tc_status, ctx.stream);
        done = true;
      } else if (f.prefill_attention && kernels::available("attention_prefill") &&
                 kernels::attention_prefill_supported(d_, cache->page_size)) {
        kernels::attention_prefill(q, out, cache->k, cache->v, ctx.seq_start, ctx.seq_past, cache->page_table, cache->table_width,
                                   ctx.n_seqs, ctx.max_q_len, n_heads_, n_kv_, d_, cache->page_size, window_, scale_, ctx.stream);
        done = true;
      }
    }
    if (!done)
      kernels::attention_generic(q, out, cache->k, cache->v, ctx.tok_seq, ctx.tok_pos, cache->page_table, cache->table_width,
                                 n_heads_, n_kv_, d_, cache->page_size, window_, scale_, ctx.stream);
    return linear(ctx, out, w_o_, nullptr, DType::F32, true);
  }

 private:
  int64_t hidden_, q_width_, kv_width_;
  int n_heads_, n_kv_, d_, window_;
  bool bias_;
  float scale_;
  std::string q_name_, k_name_, v_name_, o_name_;
  std::unique_ptr<PositionEncoding> position_;
  Weight w_qkv_, w_o_, b_qkv_;
};

// ---------------------------------------------------------------- SwiGLU
// down(silu(gate(x)) * up(x)), no biases (src/libllm/llama.cc:81-98).  Gate and up are one
// stacked product, gate rows first (tools/llama_exporter.py:73-77); the activation a/(1+exp(-a))
// times up is computed in 32-bit (src/flint/cuda/swiglu.cu:44-49).
class SwiGLU : public FeedForward {
 public:
  SwiGLU(const Json &spec, const BuildEnv &env) : FeedForward(spec, env) {
    ConfigReader r = reader_of(spec, "swiglu");
    hidden_ = r.integer("hidden");
    inter_ = r.integer("intermediate");
    gate_ = r.string("gate");
    up_ = r.string("up");
    down_ = r.string("down");
  }
  std::vector<TensorNeed> tensor_needs() const override {
    return {{gate_, {inter_, hidden_}}, {up_, {inter_, hidden_}}, {down_, {hidden_, inter_}}};
  }
  void load(const Loader &l) override {
    const auto needs = tensor_needs();
    const size_t es = dtype_size(l.engine);
    w_gate_up_.dtype = l.engine;
    w_gate_up_.rows = 2 * inter_;
    w_gate_up_.cols = hidden_;
    w_gate_up_.buf.allocate((size_t)(2 * inter_ * hidden_) * es);
    l.fetch_into(needs[0], l.engine, w_gate_up_.buf.get());
    l.fetch_into(needs[1], l.engine, (char *)w_gate_up_.buf.get() + (size_t)(inter_ * hidden_) * es);
    w_down_ = l.fetch(needs[2]);
  }
  std::vector<std::string> kernel_families() const override {
    std::vector<std::string> fams = product_families(env_.dtype);
    fams.push_back("elementwise");
    return fams;
  }
  Act forward(StepContext &ctx, const Act &x) override {
    const FastSwitches &f = fast_switches();
    Act m;
    if (x.dtype == DType::BF16) {
      m = small_batch_linear(ctx, x, w_gate_up_, ctx.dtype, true, false);
      // silu(gate) * up of a prompt step in one launch of the tcgen05 product (two accumulators per
      // tile), where that beats the library product followed by a SwiGLU pass: measured at 2,048
      // tokens, 129 us against 146 us at K = 2,048, but 403 us against 379 us at K = 4,096.
      if (!m.data && f.gemm_tc && x.rows >= f.fused_gate_up_tokens && x.cols <= f.fused_gate_up_max_k &&
          kernels::gemm_tc_supported(x, w_gate_up_)) {
        m = ctx.arena->act(ctx.dtype, x.rows, inter_);
        flush_chain(ctx);
        kernels::gemm_tc(x, w_gate_up_, m, true, ctx.tc_status, ctx.stream);
      }
    }
    if (!m.data) {
      Act gu = linear(ctx, x, w_gate_up_, nullptr, DType::F32);
      flush_chain(ctx);
      m = ctx.arena->act(ctx.dtype, x.rows, inter_);
      kernels::swiglu(gu, m.data, ctx.dtype, ctx.stream);
    }
    return linear(ctx, m, w_down_, nullptr, DType::F32, true);
  }

 private:
  int64_t hidden_, inter_;
  std::string gate_, up_, down_;
  Weight w_gate_up_, w_down_;
};

// ---------------------------------------------------------------- pre-norm block
// h = x + mixer(norm1(x)); out = h + ff(norm2(h)) (src/libllm/llama.cc:251-267).  Each addition is
// left pending on the stream and applied, in 32-bit, by the next norm.
class PreNormBlock : public Block {
 public:
  PreNormBlock(const Json &spec, const BuildEnv &env) : Block(spec, env) {
    ConfigReader r = reader_of(spec, "prenorm block");
    mixer_norm_ = build_as<Norm>("norm", r.object("mixer_norm"), env);
    mixer_ = build_as<Mixer>("mixer", r.object("mixer"), env);
    ff_norm_ = build_as<Norm>("norm", r.object("ff_norm"), env);
    ff_ = build_as<FeedForward>("feed_forward", r.object("ff"), env);
  }
  std::vector<Part *> parts() const { return {mixer_norm_.get(), mixer_.get(), ff_norm_.get(), ff_.get()}; }
  Mixer *mixer_part() override { return mixer_.get(); }
  std::vector<TensorNeed> tensor_needs() const override {
    std::vector<TensorNeed> out;
    for (Part *p : parts())
      for (auto &n : p->tensor_needs()) out.push_back(n);
    return out;
  }
  void load(const Loader &l) override {
    for (Part *p : parts()) p->load(l);
  }
  std::vector<std::string> kernel_families() const override {
    std::vector<std::string> out;
    for (Part *p : parts())
      for (auto &f : p->kernel_families()) out.push_back(f);
    return out;
  }
  bool capturable() const override {
    for (Part *p : parts())
      if (!p->capturable()) return false;
    return true;
  }
  void forward(StepContext &ctx, ResidualStream &stream, LayerCache *cache, StateView *state) override {
    // After a norm the stream holds everything added so far, so a part may add its result to it
    // directly (StepContext::residual_sink); what it returns otherwise stays pending for the next norm.
    auto sink = [&](bool on) {
      ctx.residual_sink = on ? stream.resid : nullptr;
      ctx.sink_rows = stream.rows;
      ctx.sink_cols = stream.hidden;
    };
    Act h = mixer_norm_->forward(ctx, stream);
    sink(true);
    Act r = mixer_->forward(ctx, h, cache, state);
    sink(false);
    stream.pending = r.data == (void *)stream.resid ? Act() : r;
    if (ctx.nothing_read_after) {       // no logits wanted from this step: the stream is read by nobody
      flush_chain(ctx);
      stream.pending = Act();
      return;
    }
    if (ctx.rows_read_after && ctx.n_rows_read_after < stream.rows && !stream.picked) {
      // the last layer of a prompt step: the feed-forward of the wanted rows alone
      flush_chain(ctx);
      const int64_t n = ctx.n_rows_read_after;
      float *few = ctx.arena->alloc_n<float>((size_t)(n * stream.hidden));
      kernels::gather_rows_add(stream.resid, stream.pending.data ? &stream.pending : nullptr, ctx.rows_read_after, (int)n, few,
                               (int)stream.hidden, ctx.stream);
      stream.resid = few;
      stream.rows = n;
      stream.pending = Act();
      stream.picked = true;
    }
    h = ff_norm_->forward(ctx, stream);
    sink(true);
    r = ff_->forward(ctx, h);
    sink(false);
    stream.pending = r.data == (void *)stream.resid ? Act() : r;
  }

 private:
  std::unique_ptr<Norm> mixer_norm_, ff_norm_;
  std::unique_ptr<Mixer> mixer_;
  std::unique_ptr<FeedForward> ff_;
};

template <typename T>
PartFactory factory_of() {
  return [](const Json &spec, const BuildEnv &env) { return std::unique_ptr<Part>(new T(spec, env)); };
}

}  // namespace

void register_part_raw(const std::string &category, const std::string &kind, PartFactory factory);   // parts/part.cc

void register_builtin_parts() {
  register_part_raw("norm", "rmsnorm", factory_of<RMSNorm>());
  register_part_raw("position", "rope", factory_of<RotaryEmbedding>());
  register_part_raw("mixer", "attention", factory_of<Attention>());
  register_part_raw("feed_forward", "swiglu", factory_of<SwiGLU>());
  register_part_raw("block", "prenorm", factory_of<PreNormBlock>());
}

}  // namespace llm
