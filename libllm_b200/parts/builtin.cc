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
// src/flint/cuda/rms_norm.cu:59-75).  With `weight_offset` c the stored weight is applied as (c + w).  Before the norm the stream's pending addition is applied in
// 32-bit: the reference's separate residual add (src/libllm/llama.cc:252-266).
class RMSNorm : public Norm {
 public:
  RMSNorm(const Json &spec, const BuildEnv &env) : Norm(spec, env) {
    ConfigReader r = reader_of(spec, "rmsnorm");
    size_ = r.integer("size");
    eps_ = r.number("eps");
    name_ = r.string("weight");
    offset_ = r.number_or("weight_offset", 0.0, false);
  }
  std::vector<TensorNeed> tensor_needs() const override { return {{name_, {size_}, TensorRole::Vector, false}}; }
  void load(const Loader &l) override {
    weight_ = l.fetch(tensor_needs()[0]);
    // a weight stored around nought and applied as (offset + w): added once, in 32-bit, to the 32-bit copy
    if (offset_ != 0.0) kernels::add_scalar(weight_.buf.as<float>(), size_, (float)offset_, nullptr);
  }
  std::vector<std::string> kernel_families() const override { return {"elementwise"}; }
  bool rms_params(const float **weight, float *eps) const override {
    *weight = weight_.buf.as<float>();
    *eps = (float)eps_;
    return true;
  }
  Act forward(StepContext &ctx, ResidualStream &stream, const int *rows, int n_rows) override {
    if (stream.streams > 1 || stream.pending_mix)
      LLM_THROW(InvalidArg, "rmsnorm: the residual stream has %d copies (or a result waiting to move them); the block that keeps them joins them first", stream.streams);
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
  double eps_, offset_ = 0.0;
  std::string name_;
  Weight weight_;
};

// ---------------------------------------------------------------- layer norm
// y = (x - mean) / sqrt(var + eps) * w + b, var the mean of the squared deviations, everything in
// 32-bit; `bias` may be left out.  The stream's pending addition is applied first, as in RMSNorm.
class LayerNorm : public Norm {
 public:
  LayerNorm(const Json &spec, const BuildEnv &env) : Norm(spec, env) {
    ConfigReader r = reader_of(spec, "layernorm");
    size_ = r.integer("size");
    eps_ = r.number("eps");
    name_ = r.string("weight");
    bias_name_ = r.string_or("bias", "");
  }
  std::vector<TensorNeed> tensor_needs() const override {
    std::vector<TensorNeed> needs = {{name_, {size_}, TensorRole::Vector, false}};
    if (!bias_name_.empty()) needs.push_back({bias_name_, {size_}, TensorRole::Vector, false});
    return needs;
  }
  void load(const Loader &l) override {
    const auto needs = tensor_needs();
    weight_ = l.fetch(needs[0]);
    if (needs.size() > 1) bias_ = l.fetch(needs[1]);
  }
  std::vector<std::string> kernel_families() const override { return {"elementwise"}; }
  Act forward(StepContext &ctx, ResidualStream &stream, const int *rows, int n_rows) override {
    const int64_t n = rows ? n_rows : stream.rows;
    Act out = ctx.arena->act(ctx.dtype, n, size_);
    flush_chain(ctx);
    kernels::add_layernorm(stream.resid, stream.pending.data ? &stream.pending : nullptr, weight_.buf.as<float>(),
                           bias_name_.empty() ? nullptr : bias_.buf.as<float>(), (float)eps_, out.data, ctx.dtype, rows, (int)n,
                           (int)size_, ctx.stream);
    if (!rows) stream.pending = Act();
    return out;
  }
  bool forward_conv(StepContext &ctx, ResidualStream &stream, const TimeConv &conv, Act *out) override {
    if (!ctx.decode_only || conv.taps < 2 || conv.taps > 8 || !conv.state || stream.rows != ctx.n_seqs) return false;
    // the fused kernel keeps the row in registers, four values to a load
    const Act &pend = stream.pending;
    if (size_ % 4 || size_ > 8192 || (pend.data && (pend.dtype != DType::F32 || pend.parts > 8 || pend.part_stride % 4))) return false;
    *out = ctx.arena->act(ctx.dtype, stream.rows, size_);
    flush_chain(ctx);
    kernels::add_layernorm_conv(stream.resid, stream.pending.data ? &stream.pending : nullptr, weight_.buf.as<float>(),
                                bias_name_.empty() ? nullptr : bias_.buf.as<float>(), (float)eps_, out->data, ctx.dtype, (int)stream.rows,
                                (int)size_, conv.weight, conv.state, ctx.seq_slot, conv.taps, ctx.stream);
    stream.pending = Act();
    return true;
  }

 private:
  int64_t size_;
  double eps_;
  std::string name_, bias_name_;
  Weight weight_, bias_;
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
  if (type == "yarn") {
    // Frequencies whose wavelength is short against the original length stay, long ones are divided by
    // `factor`, with a linear ramp over the pair index between the pairs that turn beta_fast and beta_slow
    // times within the original length: pair(t) = d ln(original / (2 pi t)) / (2 ln theta).
    const double orig = r.number("original_max_position_embeddings"), factor = r.number("factor");
    const double fast = r.number("beta_fast"), slow = r.number("beta_slow");
    r.number_or("magnitude", 1.0);                       // on the table's cosines and sines; applied where the table is made
    auto pair_of = [&](double turns) { return (double)rotary_dim * std::log(orig / (2.0 * M_PI * turns)) / (2.0 * std::log(theta)); };
    const double lo = std::max(std::floor(pair_of(fast)), 0.0), hi = std::min(std::ceil(pair_of(slow)), (double)rotary_dim - 1.0);
    for (size_t i = 0; i < freqs.size(); ++i) {
      const double ramp = std::min(std::max(((double)i - lo) / std::max(hi - lo, 0.001), 0.0), 1.0);
      freqs[i] = freqs[i] / factor * ramp + freqs[i] * (1.0 - ramp);
    }
    return freqs;
  }
  if (type != "llama3") LLM_THROW(Config, "rope scaling '%s' is not supported (llama3, yarn)", type.c_str());
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
    const std::string pairing = r.string_or("pairing", "half");
    if (pairing != "half" && pairing != "interleaved") r.fail("'pairing' must be \"half\" (channel i with i + rotary_dim/2) or \"interleaved\" (2i with 2i + 1)");
    interleaved_ = pairing == "interleaved";
    const Json &sc = spec.get("scaling");
    if (sc.is_object() && sc.has("magnitude") && sc.get("magnitude").is_number()) magnitude_ = sc.get("magnitude").as_number();
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
        host[(size_t)(p * rotary_dim_ + i)] = (float)(std::cos(a) * magnitude_);
        host[(size_t)(p * rotary_dim_ + half + i)] = (float)(std::sin(a) * magnitude_);
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
    if (interleaved_) {
      kernels::rope_pairs_place(qkv, q_out, l.n_heads, l.n_kv_heads, l.head_dim, l.head_dim, nullptr, false, table_->buf.as<float>(),
                                (int)table_->rows, (int)rotary_dim_, ctx.tok_seq, ctx.tok_pos, cache.page_table, cache.table_width,
                                cache.k, cache.v, cache.page_size, cache.writes, ctx.stream);
      return;
    }
    kernels::rope_cache_write(qkv, q_out, l.n_heads, l.n_kv_heads, l.head_dim, table_->buf.as<float>(), (int)table_->rows,
                              (int)rotary_dim_, ctx.tok_seq, ctx.tok_pos, cache.page_table, cache.table_width, cache.k, cache.v,
                              cache.page_size, cache.writes, ctx.stream);
  }
  const float *half_split_table(int *rows, int *rotary_dim) const override {
    if (!table_ || interleaved_) return nullptr;
    *rows = (int)table_->rows;
    *rotary_dim = (int)rotary_dim_;
    return table_->buf.as<float>();
  }
  const float *pair_table(int *rows, int *rotary_dim, bool *interleaved) const override {
    if (!table_) return nullptr;
    *rows = (int)table_->rows;
    *rotary_dim = (int)rotary_dim_;
    *interleaved = interleaved_;
    return table_->buf.as<float>();
  }

 private:
  int64_t head_dim_, rotary_dim_;
  double theta_, magnitude_ = 1.0;
  bool interleaved_ = false;
  std::shared_ptr<Weight> table_;
};

// ---------------------------------------------------------------- attention
// q, k, v from one stacked product, rotation of q and k, append to the cache,
// softmax(q k^T / sqrt(d)) v per head with a causal mask, output projection
// (src/libllm/llama.cc:178-225).  The stacked matrix is [Wq; Wk; Wv] as the reference's exporter
// builds it (tools/llama_exporter.py:64-71), made here when the weights are loaded.  The position
// part owns the rotation; without one, queries and keys are used as they come.
//
// Options beyond the reference's attention, each a key of the description:
//   v_head_dim   values (and the heads' results) of another width than queries and keys
//   qk_norm      {q, k, eps}: an RMS norm over the whole q projection and the whole k projection
//                (weights of n_heads * head_dim and n_kv_heads * head_dim values) before the rotation
//   block        a query sees only the keys of its own block of `block` positions, counted from
//                position 0 of the sequence (a chunked mask); the cache gives earlier pages back
//   head_gate    a matrix [n_heads, hidden]: head h's result is multiplied by sigmoid(gate x)_h
//                before the output projection; its rows ride at the end of the stacked product
//   out_gate     a matrix [n_heads * v_head_dim, hidden]: the same per channel of the concatenated heads
//   sink         with `window`: the first `sink` positions of a sequence stay visible to every later query
//                (at their true positions); the cache holds on to their pages
//   v_norm       {eps}: every value head is divided by its root mean square over its channels before it
//                is cached (no weight)
//   values       "keys": there is no value matrix; a position's value is its key as projected (bias added), before
//                the rotation.  Needs a rotation in neighbouring pairs (position.pairing "interleaved"), whose
//                placement kernel also adds the biases (32-bit)
//   head_norm    {eps}: AFTER the rotation every query head and every key head is divided by its root mean square over
//                its head_dim channels, sqrt(mean + eps), without a weight (a rotation of pairs (i, i + rotary_dim/2) or none)
//   null_key     a number s0: every query also sees one key whose score is s0 and which has no value, so that
//                p_j = exp(s_j) / (exp(s0) + sum exp(s_j)); with 0 the softmax has one added to its denominator
//   q_bias, k_bias, v_bias   names of the biases (default: the matrix's name with "weight" replaced by "bias").
//                Without a rotation the biases are added where q, k and v are placed (32-bit), so that the
//                product itself runs on the tensor cores like any other
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
    scale_ = (float)r.number_or("scale", 1.0 / std::sqrt((double)d_), false);
    q_name_ = r.string("q");
    k_name_ = r.string("k");
    values_from_keys_ = r.string_or("values", "own") == "keys";
    v_name_ = values_from_keys_ ? std::string() : r.string("v");
    o_name_ = r.string("o");
    if (n_heads_ % n_kv_) LLM_THROW(Config, "attention: %d heads are not a multiple of %d groups", n_heads_, n_kv_);
    dv_ = (int)r.integer_or("v_head_dim", d_);
    if (d_ > 256 || dv_ > 256) LLM_THROW(Unsupported, "attention: head sizes %d / %d are not supported (up to 256)", d_, dv_);
    block_ = (int)r.integer_or("block", 0, 0);
    if (r.present("qk_norm")) {
      ConfigReader n(r.object("qk_norm"), "attention description: qk_norm");
      q_norm_name_ = n.string("q");
      k_norm_name_ = n.string("k");
      qk_eps_ = (float)n.number("eps");
    }
    gate_name_ = r.string_or("head_gate", "");
    const std::string out_gate = r.string_or("out_gate", "");
    if (!out_gate.empty()) {
      if (!gate_name_.empty()) LLM_THROW(Config, "attention: a gate per head or per channel, not both");
      gate_name_ = out_gate;
      gate_per_channel_ = true;
    }
    sink_ = (int)r.integer_or("sink", 0, 0);
    if (sink_ > 0 && (window_ == 0 || block_ > 0)) LLM_THROW(Config, "attention: kept first positions ('sink') go with a window");
    if (r.present("v_norm")) v_eps_ = (float)ConfigReader(r.object("v_norm"), "attention description: v_norm").number("eps", false);
    if (r.present("head_norm")) head_eps_ = (float)ConfigReader(r.object("head_norm"), "attention description: head_norm").number("eps", false);
    if (r.present("null_key")) null_score_ = (float)r.number("null_key", false);
    if (!spec.get("position").is_null()) position_ = build_as<PositionEncoding>("position", spec.get("position"), env);
    const Json &pos_spec = spec.get("position");
    pairs_place_ = position_ && pos_spec.is_object() && pos_spec.has("pairing") && pos_spec.get("pairing").is_string() &&
                   pos_spec.get("pairing").as_string() == "interleaved" && q_norm_name_.empty();
    place_adds_bias_ = (!position_ && q_norm_name_.empty()) || pairs_place_;
    if (head_eps_ >= 0.f && (pairs_place_ || !q_norm_name_.empty() || bias_ || v_eps_ >= 0.f || values_from_keys_))
      LLM_THROW(Unsupported, "attention: a norm per head after the rotation goes with a rotation of pairs (i, i + rotary_dim/2) or none, and with no other norm or bias");
    if (head_eps_ >= 0.f) place_adds_bias_ = false;
    if (values_from_keys_ && (!pairs_place_ || dv_ != d_ || !gate_name_.empty() || v_eps_ >= 0.f))
      LLM_THROW(Unsupported, "attention: values that are the keys go with a rotation in neighbouring pairs, values as wide as keys, no gate and no value norm");
    if (v_eps_ >= 0.f && !place_adds_bias_) LLM_THROW(Unsupported, "attention: a value norm together with a rotation or a q/k norm is not built");
    if (bias_ && !place_adds_bias_ && (!gate_name_.empty() || !q_norm_name_.empty()))
      LLM_THROW(Unsupported, "attention: a bias together with a rotation and a gate or a q/k norm is not built");
    for (const char *key : {"q_bias", "k_bias", "v_bias"}) bias_names_.push_back(r.string_or(key, ""));
    q_width_ = (int64_t)n_heads_ * d_;
    kv_width_ = (int64_t)n_kv_ * d_;
    v_width_ = values_from_keys_ ? 0 : (int64_t)n_kv_ * dv_;
    o_width_ = (int64_t)n_heads_ * dv_;
    gate_offset_ = q_width_ + kv_width_ + v_width_;
    // rows of the stacked matrix: a multiple of 8, so that rows of the 32-bit product start on 32 bytes
    gate_rows_ = gate_name_.empty() ? 0 : gate_per_channel_ ? o_width_ : (int64_t)n_heads_;
    stacked_rows_ = (gate_offset_ + gate_rows_ + 7) / 8 * 8;
    // the tiled attention kernels take heads whose values are as wide as their keys, in multiples of 16
    plain_ = dv_ == d_ && d_ % 16 == 0 && d_ >= 16 && scale_ > 0.f;
  }

  std::vector<TensorNeed> tensor_needs() const override {
    std::vector<TensorNeed> needs = {{q_name_, {q_width_, hidden_}}, {k_name_, {kv_width_, hidden_}}};
    if (!values_from_keys_) needs.push_back({v_name_, {v_width_, hidden_}});
    needs.push_back({o_name_, {hidden_, o_width_}});
    if (bias_) {
      size_t which = 0;
      for (const auto &p : {std::make_pair(q_name_, q_width_), std::make_pair(k_name_, kv_width_), std::make_pair(v_name_, v_width_)}) {
        if (p.first.empty()) continue;                 // no value matrix
        std::string n = p.first;
        const std::string suffix = "weight";
        if (n.size() >= suffix.size() && n.compare(n.size() - suffix.size(), suffix.size(), suffix) == 0) n.resize(n.size() - suffix.size());
        const std::string given = which < bias_names_.size() ? bias_names_[which] : "";
        needs.push_back({given.empty() ? n + "bias" : given, {p.second}, TensorRole::Vector, false});
        ++which;
      }
    }
    if (!q_norm_name_.empty()) {
      needs.push_back({q_norm_name_, {q_width_}, TensorRole::Vector, false});
      needs.push_back({k_norm_name_, {kv_width_}, TensorRole::Vector, false});
    }
    if (!gate_name_.empty()) needs.push_back({gate_name_, {gate_rows_, hidden_}});
    if (position_)
      for (auto &n : position_->tensor_needs()) needs.push_back(n);
    return needs;
  }

  void load(const Loader &l) override {
    const std::vector<TensorNeed> needs = tensor_needs();
    const size_t es = dtype_size(l.engine);
    w_qkv_.dtype = l.engine;
    w_qkv_.rows = stacked_rows_;
    w_qkv_.cols = hidden_;
    w_qkv_.buf.allocate((size_t)w_qkv_.rows * (size_t)hidden_ * es, true);
    char *p = (char *)w_qkv_.buf.get();
    l.fetch_into(needs[0], l.engine, p);
    l.fetch_into(needs[1], l.engine, p + (size_t)q_width_ * hidden_ * es);
    const size_t nv = values_from_keys_ ? 0 : 1;      // matrices and biases of the values
    if (nv) l.fetch_into(needs[2], l.engine, p + (size_t)(q_width_ + kv_width_) * hidden_ * es);
    w_o_ = l.fetch(needs[2 + nv]);
    const size_t first_bias = 3 + nv;
    size_t next = bias_ ? first_bias + 2 + nv : first_bias;
    if (!q_norm_name_.empty()) {
      q_norm_ = l.fetch(needs[next]);
      k_norm_ = l.fetch(needs[next + 1]);
      next += 2;
    }
    if (!gate_name_.empty()) l.fetch_into(needs[next], l.engine, p + (size_t)gate_offset_ * hidden_ * es);
    if (bias_) {
      b_qkv_.dtype = DType::F32;
      b_qkv_.rows = 1;
      b_qkv_.cols = w_qkv_.rows;
      b_qkv_.buf.allocate((size_t)w_qkv_.rows * 4, true);
      float *b = b_qkv_.buf.as<float>();
      l.fetch_into(needs[first_bias], DType::F32, b);
      l.fetch_into(needs[first_bias + 1], DType::F32, b + q_width_);
      if (nv) l.fetch_into(needs[first_bias + 2], DType::F32, b + q_width_ + kv_width_);
      if (l.engine == DType::BF16 && !place_adds_bias_) {
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
    if (!plain_) return fams;
    if (!gate_name_.empty()) fams.push_back("elementwise");
    const bool tiled = env_.page_size == 64 && d_ % 16 == 0 && d_ >= 16 && d_ <= 128;
    if (f.prefill_attention_tc && env_.page_size == 64 && (d_ == 64 || d_ == 128)) fams.push_back("attention_prefill_tc");
    else if (f.prefill_attention && tiled) fams.push_back("attention_prefill");
    if (f.decode_attention_tc && tiled && group <= 16 && !bias_ && position_ && gate_name_.empty() && q_norm_name_.empty() &&
        head_eps_ < 0.f && !(null_score_ > kernels::NO_NULL_KEY))
      fams.push_back("attention_decode_tc");
    else if (f.decode_attention && (d_ == 16 || d_ == 32 || d_ == 64 || d_ == 128) &&
             (group == 1 || group == 2 || group == 3 || group == 4 || group == 8))
      fams.push_back("attention_decode");
    return fams;
  }

  bool wants_cache() const override { return true; }
  CacheNeed cache_need() const override {
    CacheNeed n;
    // a mask of both kinds keeps everything: neither rule alone says which pages are done with
    n.kind = window_ > 0 && block_ > 0 ? "full" : window_ > 0 ? "window" : block_ > 0 ? "block" : "full";
    n.n_kv_heads = n_kv_;
    n.k_dim = d_;
    n.v_dim = dv_;
    n.window = n.kind == "window" ? window_ : 0;
    n.block = n.kind == "block" ? block_ : 0;
    n.sink = n.kind == "window" ? sink_ : 0;
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
    const bool has_gate = !gate_name_.empty();
    const float *gate = nullptr;
    const bool has_null = null_score_ > kernels::NO_NULL_KEY;
    const bool fused = plain_ && !has_gate && q_norm_name_.empty() && head_eps_ < 0.f && !has_null && table && !bias_ && ctx.decode_only && f.decode_attention_tc && ctx.dtype == DType::BF16 &&
                       kernels::available("attention_decode_tc") && kernels::attention_decode_tc_supported(d_, cache->page_size, group);
    Act qkv = linear(ctx, x, w_qkv_, bias_ && !place_adds_bias_ ? b_qkv_.buf.as<float>() : nullptr, DType::F32, fused);
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
                                   window_, block_, scale_, ws_o, ws_ml, counters, out, ctx.stream);
      return linear(ctx, out, w_o_, nullptr, DType::F32, true);
    }
    Act q = ctx.arena->act(ctx.dtype, ctx.n_tokens, q_width_);
    const QkvLayout layout{n_heads_, n_kv_, d_};
    if (has_gate) gate = (const float *)qkv.data + gate_offset_;
    if (pairs_place_) {
      int rows = 0, rot = 0;
      bool interleaved = false;
      const float *pairs = position_->pair_table(&rows, &rot, &interleaved);
      if (!pairs || !interleaved) LLM_THROW(Unsupported, "attention: the position part has no table of neighbouring pairs");
      kernels::rope_pairs_place(qkv, q, n_heads_, n_kv_, d_, dv_, bias_ ? b_qkv_.buf.as<float>() : nullptr, values_from_keys_, pairs, rows,
                                rot, ctx.tok_seq, ctx.tok_pos, cache->page_table, cache->table_width, cache->k, cache->v,
                                cache->page_size, cache->writes, ctx.stream);
    } else if (place_adds_bias_ && (bias_ || v_eps_ >= 0.f)) {
      kernels::kv_place(qkv, q, n_heads_, n_kv_, d_, dv_, bias_ ? b_qkv_.buf.as<float>() : nullptr, v_eps_, ctx.tok_seq, ctx.tok_pos,
                        cache->page_table, cache->table_width, cache->k, cache->v, cache->page_size, cache->writes, ctx.stream);
    } else if (head_eps_ >= 0.f) {
      if (position_ && !table) LLM_THROW(Unsupported, "attention: a norm per head needs a position part with a half-split table (or none)");
      kernels::rope_headnorm_place(qkv, q, n_heads_, n_kv_, d_, dv_, head_eps_, table, table_rows, rot_dim, ctx.tok_seq, ctx.tok_pos,
                                   cache->page_table, cache->table_width, cache->k, cache->v, cache->page_size, cache->writes, ctx.stream);
    } else if (!q_norm_name_.empty() || dv_ != d_) {
      if (position_ && !table)
        LLM_THROW(Unsupported, "attention: a q/k norm or values of another width need a position part with a half-split table (or none)");
      kernels::qk_place(qkv, q, n_heads_, n_kv_, d_, dv_, q_norm_.buf.as<float>(), k_norm_.buf.as<float>(), qk_eps_, table, table_rows,
                        rot_dim, ctx.tok_seq, ctx.tok_pos, cache->page_table, cache->table_width, cache->k, cache->v,
                        cache->page_size, cache->writes, ctx.stream);
    } else if (position_) {
      position_->rotate_and_store(ctx, qkv, q, layout, *cache);
    } else {
      kernels::rope_cache_write(qkv, q, n_heads_, n_kv_, d_, nullptr, 0, 0, ctx.tok_seq, ctx.tok_pos, cache->page_table,
                                cache->table_width, cache->k, cache->v, cache->page_size, cache->writes, ctx.stream);
    }
    Act out = ctx.arena->act(ctx.dtype, ctx.n_tokens, o_width_);
    bool done = false;
    // a gate per channel is applied behind the attention kernel, whichever it is
    const float *channel_gate = gate_per_channel_ ? gate : nullptr;
    if (gate_per_channel_) gate = nullptr;
    if (ctx.dtype == DType::BF16 && plain_) {
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
                                  d_, cache->page_size, chunk, n_splits, window_, block_, scale_, ws_o, ws_ml,
                                  channel_gate ? channel_gate : gate, qkv.ld, ctx.stream, sink_, channel_gate != nullptr, null_score_);
        gate = nullptr;                 // applied
        channel_gate = nullptr;
        done = true;
      } else if (f.prefill_attention_tc && (d_ == 64 || d_ == 128) && kernels::available("attention_prefill_tc") &&
                 kernels::attention_prefill_tc_supported(d_, cache->page_size)) {
        kernels::attention_prefill_tc(q, out, cache->k, cache->v, cache->n_pages, ctx.seq_start, ctx.seq_past, cache->page_table,
                                      cache->table_width, ctx.n_seqs, ctx.max_q_len, n_heads_, n_kv_, d_, cache->page_size, window_,
                                      block_, scale_, ctx.tc_status, ctx.stream, sink_, null_score_);
        done = true;
      } else if (f.prefill_attention && kernels::available("attention_prefill") &&
                 kernels::attention_prefill_supported(d_, cache->page_size)) {
        kernels::attention_prefill(q, out, cache->k, cache->v, ctx.seq_start, ctx.seq_past, cache->page_table, cache->table_width,
                                   ctx.n_seqs, ctx.max_q_len, n_heads_, n_kv_, d_, cache->page_size, window_, block_, scale_, ctx.stream,
                                   sink_, null_score_);
        done = true;
      }
      if (done && gate) kernels::head_gate(out, gate, qkv.ld, n_heads_, dv_, ctx.stream);
    }
    if (!done)
      kernels::attention_generic(q, out, cache->k, cache->v, ctx.tok_seq, ctx.tok_pos, cache->page_table, cache->table_width,
                                 n_heads_, n_kv_, d_, dv_, cache->page_size, window_, block_, scale_, gate, qkv.ld, ctx.stream, sink_, 0,
                                 null_score_);
    if (channel_gate) kernels::head_gate(out, channel_gate, qkv.ld, n_heads_ * dv_, 1, ctx.stream);
    return linear(ctx, out, w_o_, nullptr, DType::F32, true);
  }

 private:
  int64_t hidden_, q_width_, kv_width_, v_width_, o_width_, gate_offset_, stacked_rows_;
  int64_t gate_rows_ = 0;
  int n_heads_, n_kv_, d_, dv_, window_, block_, sink_ = 0;
  bool bias_, plain_, gate_per_channel_ = false, place_adds_bias_ = false, values_from_keys_ = false, pairs_place_ = false;
  float scale_, qk_eps_ = 0.f, v_eps_ = -1.f, head_eps_ = -1.f, null_score_ = kernels::NO_NULL_KEY;
  std::vector<std::string> bias_names_;
  std::string q_name_, k_name_, v_name_, o_name_, q_norm_name_, k_norm_name_, gate_name_;
  std::unique_ptr<PositionEncoding> position_;
  Weight w_qkv_, w_o_, b_qkv_, q_norm_, k_norm_;
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
// left pending on the stream and applied, in 32-bit, by the next norm.  Options:
//   mixer_conv  {taps, weight}: what the mixer reads, n = norm1(x), becomes n + conv(n), a causal
//               convolution over time on each channel (weight [hidden, taps], the last tap on the
//               token itself, zeros before the sequence's start); the last taps - 1 rows of n are
//               state of the run, per sequence, in the engine's type
//   ff, ff_norm may be null: the block is the mixer alone
//   mixer_scale, ff_scale  names of vectors [hidden]: a sublayer's result is multiplied by its vector,
//               channel by channel, before it is added to the stream (32-bit, in the pass that adds it)
const char *const CONV_STATE = "mixer_conv.inputs";
class PreNormBlock : public Block {
 public:
  PreNormBlock(const Json &spec, const BuildEnv &env) : Block(spec, env) {
    ConfigReader r = reader_of(spec, "prenorm block");
    mixer_norm_ = build_as<Norm>("norm", r.object("mixer_norm"), env);
    mixer_ = build_as<Mixer>("mixer", r.object("mixer"), env);
    if (r.present("ff")) {
      ff_norm_ = build_as<Norm>("norm", r.object("ff_norm"), env);
      ff_ = build_as<FeedForward>("feed_forward", r.object("ff"), env);
    }
    if (r.present("mixer_conv")) {
      ConfigReader c(r.object("mixer_conv"), "prenorm block: mixer_conv");
      taps_ = (int)c.integer("taps");
      conv_name_ = c.string("weight");
      hidden_ = c.integer("hidden");
      if (taps_ > 8) LLM_THROW(Unsupported, "prenorm block: a convolution of %d taps is not supported (up to 8)", taps_);
    }
    mixer_scale_name_ = r.string_or("mixer_scale", "");
    ff_scale_name_ = ff_ ? r.string_or("ff_scale", "") : "";
    if (!mixer_scale_name_.empty() || !ff_scale_name_.empty()) hidden_ = r.integer("hidden");
  }
  std::vector<Part *> parts() const {
    std::vector<Part *> p = {mixer_norm_.get(), mixer_.get()};
    if (ff_) {
      p.push_back(ff_norm_.get());
      p.push_back(ff_.get());
    }
    return p;
  }
  Mixer *mixer_part() override { return mixer_.get(); }
  std::vector<StateNeed> state_need() override {
    std::vector<StateNeed> needs;
    if (taps_ > 1) needs.push_back({CONV_STATE, {(int64_t)taps_ - 1, hidden_}, env_.dtype});
    for (auto &n : mixer_->state_need()) needs.push_back(n);
    return needs;
  }
  std::vector<TensorNeed> tensor_needs() const override {
    std::vector<TensorNeed> out;
    for (Part *p : parts())
      for (auto &n : p->tensor_needs()) out.push_back(n);
    if (taps_ > 0) out.push_back({conv_name_, {hidden_, (int64_t)taps_}, TensorRole::Vector, false});
    if (!mixer_scale_name_.empty()) out.push_back({mixer_scale_name_, {hidden_}, TensorRole::Vector, false});
    if (!ff_scale_name_.empty()) out.push_back({ff_scale_name_, {hidden_}, TensorRole::Vector, false});
    return out;
  }
  void load(const Loader &l) override {
    for (Part *p : parts()) p->load(l);
    if (taps_ > 0) conv_ = l.fetch({conv_name_, {hidden_, (int64_t)taps_}, TensorRole::Vector, false});
    if (!mixer_scale_name_.empty()) mixer_scale_ = l.fetch({mixer_scale_name_, {hidden_}, TensorRole::Vector, false});
    if (!ff_scale_name_.empty()) ff_scale_ = l.fetch({ff_scale_name_, {hidden_}, TensorRole::Vector, false});
  }
  std::vector<std::string> kernel_families() const override {
    std::vector<std::string> out;
    for (Part *p : parts())
      for (auto &f : p->kernel_families()) out.push_back(f);
    if (taps_ > 0) out.push_back("recurrent");
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
    Act h;
    StateView mixer_state;
    if (taps_ > 0) {
      void *conv_state = nullptr;
      if (state)
        for (const auto &t : *state) {
          if (t.name == CONV_STATE) conv_state = t.data;
          else mixer_state.push_back(t);
        }
      if (taps_ > 1 && !conv_state) LLM_THROW(InvalidArg, "prenorm block: the run has no state for its convolution");
      TimeConv conv;
      conv.weight = conv_.buf.as<float>();
      conv.state = conv_state;
      conv.taps = taps_;
      // a step of single tokens: the norm runs the convolution in its own launch where it can
      if (!mixer_norm_->forward_conv(ctx, stream, conv, &h)) {
        h = mixer_norm_->forward(ctx, stream);
        flush_chain(ctx);
        Act mixed = ctx.arena->act(ctx.dtype, h.rows, h.cols);
        kernels::causal_conv(h, mixed, conv.weight, conv.state, ctx.tok_seq, ctx.tok_pos, ctx.seq_start, ctx.seq_past, ctx.seq_slot,
                             ctx.n_seqs, taps_, ctx.decode_only, ctx.stream);
        h = mixed;
      }
      state = mixer_state.empty() ? nullptr : &mixer_state;
    } else {
      h = mixer_norm_->forward(ctx, stream);
    }
    // a result that is scaled before it is added cannot be added by the product that makes it
    const float *mixer_scale = mixer_scale_name_.empty() ? nullptr : mixer_scale_.buf.as<float>();
    const float *ff_scale = ff_scale_name_.empty() ? nullptr : ff_scale_.buf.as<float>();
    sink(mixer_scale == nullptr);
    Act r = mixer_->forward(ctx, h, cache, state);
    sink(false);
    stream.pending = r.data == (void *)stream.resid ? Act() : scaled(r, mixer_scale);
    if (ctx.nothing_read_after) {       // no logits wanted from this step: the stream is read by nobody
      flush_chain(ctx);
      stream.pending = Act();
      return;
    }
    if (!ff_) return;
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
    sink(ff_scale == nullptr);
    r = ff_->forward(ctx, h);
    sink(false);
    stream.pending = r.data == (void *)stream.resid ? Act() : scaled(r, ff_scale);
  }

 private:
  static Act scaled(Act r, const float *scale) {
    if (!scale) return r;
    if (r.col_scale) LLM_THROW(Unsupported, "prenorm block: a sublayer's result carries a scale of its own beside the block's");
    r.col_scale = scale;
    return r;
  }
  std::unique_ptr<Norm> mixer_norm_, ff_norm_;
  std::unique_ptr<Mixer> mixer_;
  std::unique_ptr<FeedForward> ff_;
  int taps_ = 0;
  int64_t hidden_ = 0;
  std::string conv_name_, mixer_scale_name_, ff_scale_name_;
  Weight conv_, mixer_scale_, ff_scale_;
};

// ---------------------------------------------------------------- pre-norm block over several residual streams
// The model carries `streams` copies x_0 .. x_{S-1} of the residual stream, all equal to the token's row at the start
// ("hyper-connections").  Sublayer q (the mixer, then the feed-forward) has a vector `in` [S], a vector `out` [S]
// and a matrix `mix` [S, S] indexed [from, to]:
//   u = sum_s in[s] x_s;   y = sublayer(norm(u));   x_t <- sum_s mix[s, t] x_s + out[t] y   (all t at once, from the old x)
// With in = out = (1), mix = (1) and one stream this is the pre-norm block.  A sublayer's result stays pending on the
// stream with its `mix` and `out`; the next pass over the rows (the next sublayer's join and norm, or the model's
// sum of the copies before its last norm) applies it, so a sublayer costs one pass over the S copies: read, move, join,
// norm (csrc/elementwise.cu: hyper_mix_norm).  Everything between the sublayers is 32-bit.  The feed-forward may be
// absent.  In the last layer of a step that wants few rows, the feed-forward runs for those rows alone.  With one
// stream the three tensors may be missing from the files: they count as 1.
class HyperBlock : public Block {
 public:
  HyperBlock(const Json &spec, const BuildEnv &env) : Block(spec, env) {
    ConfigReader r = reader_of(spec, "hyper block");
    streams_ = (int)r.integer("streams");
    hidden_ = r.integer("hidden");
    if (streams_ > 16) LLM_THROW(Unsupported, "hyper block: %d residual streams are not supported (up to 16)", streams_);
    mixer_norm_ = build_as<Norm>("norm", r.object("mixer_norm"), env);
    mixer_ = build_as<Mixer>("mixer", r.object("mixer"), env);
    for (const char *k : {"mixer_in", "mixer_out", "mixer_mix"}) names_.push_back(r.string(k));
    if (r.present("ff")) {
      ff_norm_ = build_as<Norm>("norm", r.object("ff_norm"), env);
      ff_ = build_as<FeedForward>("feed_forward", r.object("ff"), env);
      for (const char *k : {"ff_in", "ff_out", "ff_mix"}) names_.push_back(r.string(k));
    }
  }
  int streams() const override { return streams_; }
  std::vector<Part *> parts() const {
    std::vector<Part *> p = {mixer_norm_.get(), mixer_.get()};
    if (ff_) {
      p.push_back(ff_norm_.get());
      p.push_back(ff_.get());
    }
    return p;
  }
  Mixer *mixer_part() override { return mixer_.get(); }
  std::vector<TensorNeed> own_needs() const {
    std::vector<TensorNeed> out;
    // drawn weights: `in` and the columns of `mix` average the copies, so that drawn models keep their scale
    for (size_t i = 0; i < names_.size(); ++i)
      out.push_back({names_[i], i % 3 == 2 ? std::vector<int64_t>{streams_, streams_} : std::vector<int64_t>{streams_}, TensorRole::Vector,
                     streams_ == 1, i % 3 == 1 ? 1.f : 1.f / (float)streams_});
    return out;
  }
  std::vector<TensorNeed> tensor_needs() const override {
    std::vector<TensorNeed> out;
    for (Part *p : parts())
      for (auto &n : p->tensor_needs()) out.push_back(n);
    for (auto &n : own_needs()) out.push_back(n);
    return out;
  }
  void load(const Loader &l) override {
    for (Part *p : parts()) p->load(l);
    joins_.clear();
    for (auto &n : own_needs()) {
      if (!n.optional || l.has(n.name)) {
        joins_.push_back(l.fetch(n));
        continue;
      }
      // one stream whose joining tensors are not stored: in = out = mix = 1, the plain residual sum
      Weight one;
      one.dtype = DType::F32;
      one.rows = one.cols = 1;
      one.buf.allocate(sizeof(float));
      const float v = 1.f;
      LLM_CUDA(cudaMemcpy(one.buf.get(), &v, sizeof(float), cudaMemcpyHostToDevice));
      joins_.push_back(std::move(one));
    }
  }
  std::vector<std::string> kernel_families() const override {
    std::vector<std::string> out = {"elementwise"};
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
    if (stream.streams != streams_ || stream.hidden != hidden_)
      LLM_THROW(InvalidArg, "hyper block: built for %d streams of %lld channels, given %d of %lld", streams_, (long long)hidden_,
                stream.streams, (long long)stream.hidden);
    ctx.residual_sink = nullptr;            // a result moves every copy: no product can add it as it stores
    Act h = join(ctx, stream, *mixer_norm_, joins_[0], nullptr, 0);
    Act r = mixer_->forward(ctx, h, cache, state);
    leave(stream, r, 1);
    if (ctx.nothing_read_after) {           // no logits wanted from this step: the stream is read by nobody
      flush_chain(ctx);
      stream.pending = Act();
      return;
    }
    if (!ff_) return;
    const bool few = ctx.rows_read_after && ctx.n_rows_read_after < stream.rows && !stream.picked;
    h = join(ctx, stream, *ff_norm_, joins_[3], few ? ctx.rows_read_after : nullptr, few ? ctx.n_rows_read_after : 0);
    r = ff_->forward(ctx, h);
    leave(stream, r, 4);
  }

 private:
  // Applies what is pending, joins the copies with `in`, norms; with `rows` the stream goes on with those rows alone.
  Act join(StepContext &ctx, ResidualStream &stream, Norm &norm, const Weight &in, const int *rows, int n_rows) {
    flush_chain(ctx);
    const int64_t n = rows ? n_rows : stream.rows, H = stream.hidden;
    float *x_out = stream.resid;
    int64_t out_stride = stream.stream_stride;
    if (rows) {
      x_out = ctx.arena->alloc_n<float>((size_t)streams_ * (size_t)(n * H));
      out_stride = n * H;
    }
    const Act *delta = stream.pending.data ? &stream.pending : nullptr;
    const int64_t in_stride = stream.spread ? stream.stream_stride : 0;
    const float *w = nullptr;
    float eps = 0.f;
    Act h;
    if (norm.rms_params(&w, &eps)) {
      h = ctx.arena->act(ctx.dtype, n, H);
      kernels::hyper_mix_norm(stream.resid, in_stride, x_out, out_stride, streams_, delta, stream.pending_mix, stream.pending_out,
                              in.buf.as<float>(), w, eps, h.data, ctx.dtype, rows, (int)n, (int)H, ctx.stream);
    } else {
      // any other norm: the joined rows in 32-bit, then the norm's own pass over them
      float *u = ctx.arena->alloc_n<float>((size_t)(n * H));
      kernels::hyper_mix_norm(stream.resid, in_stride, x_out, out_stride, streams_, delta, stream.pending_mix, stream.pending_out,
                              in.buf.as<float>(), nullptr, 0.f, u, DType::F32, rows, (int)n, (int)H, ctx.stream);
      ResidualStream one;
      one.resid = u;
      one.rows = n;
      one.hidden = H;
      h = norm.forward(ctx, one);
    }
    stream.resid = x_out;
    stream.stream_stride = out_stride;
    stream.rows = n;
    stream.spread = true;
    stream.pending = Act();
    stream.pending_mix = stream.pending_out = nullptr;
    if (rows) stream.picked = true;
    return h;
  }
  void leave(ResidualStream &stream, const Act &r, size_t first) {
    if (r.dtype != DType::F32 || r.rows != stream.rows || r.cols != stream.hidden || r.ld != stream.hidden)
      LLM_THROW(Unsupported, "hyper block: a sublayer hands over dense 32-bit rows");
    stream.pending = r;
    stream.pending_out = joins_[first].buf.as<float>();
    stream.pending_mix = joins_[first + 1].buf.as<float>();
  }
  int streams_ = 1;
  int64_t hidden_ = 0;
  std::unique_ptr<Norm> mixer_norm_, ff_norm_;
  std::unique_ptr<Mixer> mixer_;
  std::unique_ptr<FeedForward> ff_;
  std::vector<std::string> names_;        // in, out, mix of the mixer, then of the feed-forward
  std::vector<Weight> joins_;
};

// ---------------------------------------------------------------- parallel block
// out = x + mixer(h) + ff(h) with h = norm(x): one norm, and both sublayers read its output.  The
// feed-forward may be absent.  The mixer's result is added to the stream (by its own last product
// where that can add as it stores, else by an addition pass) before the feed-forward's is left
// pending for the next norm, since the stream carries one pending addition.
class ParallelBlock : public Block {
 public:
  ParallelBlock(const Json &spec, const BuildEnv &env) : Block(spec, env) {
    ConfigReader r = reader_of(spec, "parallel block");
    norm_ = build_as<Norm>("norm", r.object("norm"), env);
    mixer_ = build_as<Mixer>("mixer", r.object("mixer"), env);
    if (r.present("ff")) ff_ = build_as<FeedForward>("feed_forward", r.object("ff"), env);
  }
  std::vector<Part *> parts() const {
    std::vector<Part *> p = {norm_.get(), mixer_.get()};
    if (ff_) p.push_back(ff_.get());
    return p;
  }
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
    std::vector<std::string> out = {"elementwise"};
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
    auto sink = [&](bool on) {
      ctx.residual_sink = on ? stream.resid : nullptr;
      ctx.sink_rows = stream.rows;
      ctx.sink_cols = stream.hidden;
    };
    Act h = norm_->forward(ctx, stream);
    // the last layer of a prompt step: the feed-forward of the wanted rows alone, from their norms
    const bool few = ff_ && ctx.rows_read_after && ctx.n_rows_read_after < stream.rows && !stream.picked;
    Act h_few;
    if (few) h_few = norm_->forward(ctx, stream, ctx.rows_read_after, ctx.n_rows_read_after);
    // Steps of few tokens, whose products hand back partial products: room in which the mixer's and the
    // feed-forward's parts lie one behind the other, so that the next norm adds them all in one pass.
    constexpr int POOL_PARTS = 16;
    const bool pooled = ff_ && !few && ctx.dtype == DType::BF16 && stream.rows <= fast_switches().tc_tokens && !ctx.chain;
    if (pooled) {
      ctx.parts_pool = ctx.arena->alloc_n<float>((size_t)POOL_PARTS * (size_t)(stream.rows * stream.hidden));
      ctx.parts_cap = POOL_PARTS;
      ctx.parts_used = 0;
      ctx.parts_rows = stream.rows;
      ctx.parts_cols = stream.hidden;
    }
    float *const pool = ctx.parts_pool;
    sink(true);
    Act r = mixer_->forward(ctx, h, cache, state);
    sink(false);
    stream.pending = r.data == (void *)stream.resid ? Act() : r;
    const int mixer_parts = ctx.parts_used;
    const bool mixer_pooled = pooled && r.data == (void *)pool && r.parts == mixer_parts;
    if (!mixer_pooled) ctx.parts_pool = nullptr;
    if (ctx.nothing_read_after) {       // no logits wanted from this step: the stream is read by nobody
      flush_chain(ctx);
      stream.pending = Act();
      ctx.parts_pool = nullptr;
      return;
    }
    if (!ff_) return;
    if (mixer_pooled) {
      sink(true);
      Act f = ff_->forward(ctx, h);
      sink(false);
      ctx.parts_pool = nullptr;
      if (f.data == (void *)(pool + (size_t)mixer_parts * (size_t)r.part_stride) && f.parts == ctx.parts_used - mixer_parts) {
        r.parts = ctx.parts_used;             // the mixer's parts, then the feed-forward's
        stream.pending = r;
        return;
      }
      // the feed-forward put its result elsewhere: the mixer's parts are added first, then its own stay pending
      flush_chain(ctx);
      kernels::add_rmsnorm(stream.resid, &stream.pending, nullptr, 0.f, nullptr, ctx.dtype, nullptr, (int)stream.rows,
                           (int)stream.hidden, ctx.stream);
      stream.pending = f.data == (void *)stream.resid ? Act() : f;
      return;
    }
    if (few) {
      flush_chain(ctx);
      const int64_t n = ctx.n_rows_read_after;
      float *rows = ctx.arena->alloc_n<float>((size_t)(n * stream.hidden));
      kernels::gather_rows_add(stream.resid, stream.pending.data ? &stream.pending : nullptr, ctx.rows_read_after, (int)n, rows,
                               (int)stream.hidden, ctx.stream);
      stream.resid = rows;
      stream.rows = n;
      stream.pending = Act();
      stream.picked = true;
      h = h_few;
    } else if (stream.pending.data) {
      flush_chain(ctx);
      kernels::add_rmsnorm(stream.resid, &stream.pending, nullptr, 0.f, nullptr, ctx.dtype, nullptr, (int)stream.rows,
                           (int)stream.hidden, ctx.stream);
      stream.pending = Act();
    }
    sink(true);
    r = ff_->forward(ctx, h);
    sink(false);
    stream.pending = r.data == (void *)stream.resid ? Act() : r;
  }

 private:
  std::unique_ptr<Norm> norm_;
  std::unique_ptr<Mixer> mixer_;
  std::unique_ptr<FeedForward> ff_;
};

template <typename T>
PartFactory factory_of() {
  return [](const Json &spec, const BuildEnv &env) { return std::unique_ptr<Part>(new T(spec, env)); };
}

}  // namespace

void register_part_raw(const std::string &category, const std::string &kind, PartFactory factory);   // parts/part.cc

void register_feed_forward_parts();   // parts/feed_forward.cc
void register_recurrent_parts();      // parts/recurrent.cc
void register_latent_parts();         // parts/latent.cc

void register_builtin_parts() {
  register_part_raw("block", "parallel", factory_of<ParallelBlock>());
  register_feed_forward_parts();
  register_recurrent_parts();
  register_latent_parts();
  register_part_raw("norm", "rmsnorm", factory_of<RMSNorm>());
  register_part_raw("norm", "layernorm", factory_of<LayerNorm>());
  register_part_raw("position", "rope", factory_of<RotaryEmbedding>());
  register_part_raw("mixer", "attention", factory_of<Attention>());
  register_part_raw("feed_forward", "swiglu", factory_of<SwiGLU>());
  register_part_raw("block", "prenorm", factory_of<PreNormBlock>());
  register_part_raw("block", "hyper", factory_of<HyperBlock>());
}

}  // namespace llm
