// Mixers that carry a fixed-size state from token to token instead of keys and values.
//
// "general_delta": the generalized delta rule.  Per head, with h the mixer's input and d channels:
//   r = W_r h, k = W_k h, v = W_v h
//   decay    w = exp(-decay_scale * sigmoid(w0 + W_2 tanh(W_1 h)))     per key channel (W_1 of low rank)
//   removal  a = sigmoid(W_a h + a_bias)                               per key channel
//   unit key u = k / sqrt(sum(k^2) + key_eps)
//   state    S <- diag(w) S - (a * u)(u^T S) + k v^T                   both terms read the old S
//   result   o = S^T r, divided by its root mean square over the head (eps), times `norm`
//            (a weight over all heads' channels), times sigmoid(W_g h), then W_o.
// The state (heads x d x d, 32-bit) starts at zero and belongs to the run and the sequence.  All
// projections of h are one stacked product [r; k; v; g; a; W_1] with a 32-bit result; everything
// from there to the state is 32-bit (csrc/recurrent.cu).  The reference has no such mixer.
#include <cmath>

#include "config/config.h"
#include "csrc/kernels.h"
#include "parts/chain.h"
#include "parts/linear.h"
#include "parts/part.h"

namespace llm {

namespace {

class GeneralDelta : public Mixer {
 public:
  GeneralDelta(const Json &spec, const BuildEnv &env) : Mixer(spec, env) {
    ConfigReader r(spec, "general_delta description");
    hidden_ = r.integer("hidden");
    n_heads_ = (int)r.integer("n_heads");
    d_ = (int)r.integer("head_dim");
    if (d_ > 256) LLM_THROW(Unsupported, "general_delta: heads of %d channels are not supported (up to 256)", d_);
    rank_ = r.integer_or("decay_rank", -1);          // -1: the size W_1 is stored with
    eps_ = (float)r.number("eps");
    decay_scale_ = (float)r.number_or("decay_scale", std::exp(-0.5));
    key_eps_ = (float)r.number_or("key_eps", 1e-6);
    for (const char *key : {"r", "k", "v", "g", "a", "a_bias", "w1", "w2", "w0", "norm", "o"}) names_.push_back(r.string(key));
    width_ = (int64_t)n_heads_ * d_;
  }
  enum { R, K, V, G, A, A_BIAS, W1, W2, W0, NORM, O };

  std::vector<TensorNeed> tensor_needs() const override {
    std::vector<TensorNeed> needs;
    for (int i : {R, K, V, G, A}) needs.push_back({names_[(size_t)i], {width_, hidden_}});
    needs.push_back({names_[A_BIAS], {width_}, TensorRole::Vector, false});
    needs.push_back({names_[W1], {rank_, hidden_}});
    needs.push_back({names_[W2], {width_, rank_}, TensorRole::Vector, false});
    needs.push_back({names_[W0], {width_}, TensorRole::Vector, false});
    needs.push_back({names_[NORM], {width_}, TensorRole::Vector, false});
    needs.push_back({names_[O], {hidden_, width_}});
    return needs;
  }

  void load(const Loader &l) override {
    if (rank_ < 0) {
      const std::vector<int64_t> stored = l.shape_of(names_[W1]);
      rank_ = stored.size() == 2 ? stored[0] : DRAWN_FREE_SIZE;
    }
    const std::vector<TensorNeed> needs = tensor_needs();
    const size_t es = dtype_size(l.engine);
    // rows of the stacked matrix in multiples of 8, so that rows of the 32-bit product start on 32 bytes
    w_in_.dtype = l.engine;
    w_in_.rows = (5 * width_ + rank_ + 7) / 8 * 8;
    w_in_.cols = hidden_;
    w_in_.buf.allocate((size_t)w_in_.rows * (size_t)hidden_ * es, true);
    for (int i = 0; i < 5; ++i) l.fetch_into(needs[(size_t)i], l.engine, (char *)w_in_.buf.get() + (size_t)i * width_ * hidden_ * es);
    l.fetch_into(needs[6], l.engine, (char *)w_in_.buf.get() + (size_t)5 * width_ * hidden_ * es);
    a_bias_ = l.fetch(needs[5]);
    w2_ = l.fetch(needs[7]);
    w0_ = l.fetch(needs[8]);
    norm_ = l.fetch(needs[9]);
    w_o_ = l.fetch(needs[10]);
  }

  std::vector<std::string> kernel_families() const override {
    std::vector<std::string> fams = product_families(env_.dtype);
    fams.push_back("recurrent");
    return fams;
  }

  std::vector<StateNeed> state_need() const override { return {{"general_delta.S", {(int64_t)n_heads_, (int64_t)d_, (int64_t)d_}, DType::F32}}; }

  Act forward(StepContext &ctx, const Act &x, LayerCache *, StateView *state) override {
    float *S = nullptr;
    if (state)
      for (const auto &t : *state)
        if (t.name == "general_delta.S") S = (float *)t.data;
    if (!S) LLM_THROW(InvalidArg, "general_delta: the run has no state");
    Act proj = linear(ctx, x, w_in_, nullptr, DType::F32);
    flush_chain(ctx);
    const int T = ctx.n_tokens;
    const int W = (int)width_;
    if (ctx.decode_only && T == ctx.n_seqs && kernels::delta_step_supported(d_)) {
      // a step of single tokens: the vectors, the state's step, the norm and the gate in one launch
      Act y = ctx.arena->act(ctx.dtype, T, width_);
      kernels::delta_step(proj, 0, W, 2 * W, 3 * W, 4 * W, 5 * W, (int)rank_, w2_.buf.as<float>(), w0_.buf.as<float>(),
                          a_bias_.buf.as<float>(), decay_scale_, key_eps_, norm_.buf.as<float>(), eps_, S, y, ctx.seq_slot, n_heads_, d_,
                          ctx.stream);
      return linear(ctx, y, w_o_, nullptr, DType::F32, true);
    }
    float *prep = ctx.arena->alloc_n<float>((size_t)T * (size_t)width_ * 3);
    Act o = ctx.arena->act(DType::F32, T, width_);
    kernels::delta_rule(proj, 0, W, 2 * W, 4 * W, 5 * W, (int)rank_, w2_.buf.as<float>(), w0_.buf.as<float>(), a_bias_.buf.as<float>(),
                        decay_scale_, key_eps_, prep, S, o, ctx.seq_start, ctx.seq_slot, ctx.n_seqs, n_heads_, d_, ctx.stream);
    Act y = ctx.arena->act(ctx.dtype, T, width_);
    kernels::head_norm_gate(o, norm_.buf.as<float>(), (const float *)proj.data + 3 * W, proj.ld, eps_, n_heads_, d_, y, ctx.stream);
    return linear(ctx, y, w_o_, nullptr, DType::F32, true);
  }

 private:
  int64_t hidden_, width_, rank_;
  int n_heads_, d_;
  float eps_, decay_scale_, key_eps_;
  std::vector<std::string> names_;
  Weight w_in_, w_o_, a_bias_, w2_, w0_, norm_;
};

// "channel_delta": the gated delta rule with a decay per head and key channel.  With h the mixer's input, H heads,
// G key heads of d channels (head i reads key head i / (H / G)), values of dv channels:
//   q = W_q h, k = W_k h (G x d), v = W_v h (H x dv); each passes a short causal convolution over time per channel
//   (`taps` taps, the last one the token's own, zeros before the sequence's start) and silu;
//   q and k become unit vectors per key head, x / sqrt(sum x^2 + key_eps), q also times d^(-1/2);
//   beta = sigmoid(W_b h) per head;  g = exp(-exp(A_log[head]) * softplus(W_a2 (W_a1 h) + dt_bias)) per head and key channel;
//   S <- diag(g) S;  e = beta (v - S^T k);  S <- S + k e^T;  o = S^T q   (the read-out sees the token's own write);
//   o / rms(o over the head, eps) * norm (dv values that the heads share) * sigmoid(W_g2 (W_g1 h)), then W_o.
// State per run and sequence, zero at the start: S (heads x dv x d, 32-bit; a value column's key rows together) and the
// last taps - 1 rows of the three projections (32-bit, as the stacked product left them).  All products of h are one
// stacked product [q; k; v; b; a1; g1] with a 32-bit result; everything from there to the norm's result is 32-bit
// (csrc/recurrent.cu: the convolution, channel_delta_prepare, the scan of general_delta with its vectors renamed,
// head_norm_gate).  The ranks of the two low-rank inputs are the sizes a1 and g1 are stored with.
class ChannelDelta : public Mixer {
 public:
  ChannelDelta(const Json &spec, const BuildEnv &env) : Mixer(spec, env) {
    ConfigReader r(spec, "channel_delta description");
    hidden_ = r.integer("hidden");
    n_heads_ = (int)r.integer("n_heads");
    n_kv_ = (int)r.integer_or("n_kv_heads", n_heads_);
    d_ = (int)r.integer("head_dim");
    dv_ = (int)r.integer_or("v_head_dim", d_);
    taps_ = (int)r.integer_or("taps", 1);
    eps_ = (float)r.number("eps");
    key_eps_ = (float)r.number_or("key_eps", 1e-6);
    rank_a_ = r.integer_or("decay_rank", -1);         // -1: the sizes a1 and g1 are stored with
    rank_g_ = r.integer_or("gate_rank", -1);
    if (n_heads_ % n_kv_) r.fail("'n_heads' must be a multiple of 'n_kv_heads'");
    if (d_ > 256) LLM_THROW(Unsupported, "channel_delta: heads of %d key channels are not supported (up to 256)", d_);
    if (taps_ < 1 || taps_ > 8) LLM_THROW(Unsupported, "channel_delta: a convolution of %d taps is not supported (1 to 8)", taps_);
    for (const char *key : {"q", "k", "v", "b", "a1", "g1", "q_conv", "k_conv", "v_conv", "a2", "dt_bias", "A_log", "g2", "norm", "o"})
      names_.push_back(r.string(key));
    qk_width_ = (int64_t)n_kv_ * d_;
    k_width_ = (int64_t)n_heads_ * d_;
    v_width_ = (int64_t)n_heads_ * dv_;
    conv_width_ = 2 * qk_width_ + v_width_;
    row_ld_ = (conv_width_ + 2 * k_width_ + 3) / 4 * 4;
  }
  enum { Q, K, V, B, A1, G1, Q_CONV, K_CONV, V_CONV, A2, DT_BIAS, A_LOG, G2, NORM, O };

  std::vector<TensorNeed> tensor_needs() const override {
    std::vector<TensorNeed> needs;
    needs.push_back({names_[Q], {qk_width_, hidden_}});
    needs.push_back({names_[K], {qk_width_, hidden_}});
    needs.push_back({names_[V], {v_width_, hidden_}});
    needs.push_back({names_[B], {(int64_t)n_heads_, hidden_}});
    needs.push_back({names_[A1], {rank_a_, hidden_}});
    needs.push_back({names_[G1], {rank_g_, hidden_}});
    needs.push_back({names_[Q_CONV], {qk_width_, (int64_t)taps_}, TensorRole::Vector, false});
    needs.push_back({names_[K_CONV], {qk_width_, (int64_t)taps_}, TensorRole::Vector, false});
    needs.push_back({names_[V_CONV], {v_width_, (int64_t)taps_}, TensorRole::Vector, false});
    needs.push_back({names_[A2], {k_width_, rank_a_}, TensorRole::Vector, false});
    needs.push_back({names_[DT_BIAS], {k_width_}, TensorRole::Vector, false});
    needs.push_back({names_[A_LOG], {(int64_t)n_heads_}, TensorRole::Vector, false});
    needs.push_back({names_[G2], {v_width_, rank_g_}, TensorRole::Vector, false});
    needs.push_back({names_[NORM], {(int64_t)dv_}, TensorRole::Vector, false});
    needs.push_back({names_[O], {hidden_, v_width_}});
    return needs;
  }

  void load(const Loader &l) override {
    auto stored_rank = [&](int64_t &rank, const std::string &name) {
      if (rank >= 0) return;
      const std::vector<int64_t> stored = l.shape_of(name);
      rank = stored.size() == 2 ? stored[0] : DRAWN_FREE_SIZE;
    };
    stored_rank(rank_a_, names_[A1]);
    stored_rank(rank_g_, names_[G1]);
    const std::vector<TensorNeed> needs = tensor_needs();
    const size_t es = dtype_size(l.engine);
    off_b_ = conv_width_;
    off_a1_ = off_b_ + n_heads_;
    off_g1_ = off_a1_ + rank_a_;
    // rows of the stacked matrix in multiples of 8, so that rows of the 32-bit product start on 32 bytes
    w_in_.dtype = l.engine;
    w_in_.rows = (off_g1_ + rank_g_ + 7) / 8 * 8;
    w_in_.cols = hidden_;
    w_in_.buf.allocate((size_t)w_in_.rows * (size_t)hidden_ * es, true);
    const int64_t at[6] = {0, qk_width_, 2 * qk_width_, off_b_, off_a1_, off_g1_};
    for (int i = 0; i < 6; ++i) l.fetch_into(needs[(size_t)i], l.engine, (char *)w_in_.buf.get() + (size_t)at[i] * hidden_ * es);
    // the three convolutions' weights one behind the other, as their channels lie in a row of the product
    conv_.dtype = DType::F32;
    conv_.rows = conv_width_;
    conv_.cols = taps_;
    conv_.buf.allocate((size_t)conv_width_ * taps_ * sizeof(float), true);
    l.fetch_into(needs[Q_CONV], DType::F32, conv_.buf.as<float>());
    l.fetch_into(needs[K_CONV], DType::F32, conv_.buf.as<float>() + qk_width_ * taps_);
    l.fetch_into(needs[V_CONV], DType::F32, conv_.buf.as<float>() + 2 * qk_width_ * taps_);
    a2_ = l.fetch(needs[A2]);
    dt_bias_ = l.fetch(needs[DT_BIAS]);
    a_log_ = l.fetch(needs[A_LOG]);
    g2_ = l.fetch(needs[G2]);
    // the heads share the norm's weight: one copy per head, as the norm kernel reads it
    norm_.dtype = DType::F32;
    norm_.rows = 1;
    norm_.cols = v_width_;
    norm_.buf.allocate((size_t)v_width_ * sizeof(float), true);
    for (int h = 0; h < n_heads_; ++h) l.fetch_into(needs[NORM], DType::F32, norm_.buf.as<float>() + (size_t)h * dv_);
    w_o_ = l.fetch(needs[O]);
  }

  std::vector<std::string> kernel_families() const override {
    std::vector<std::string> fams = product_families(env_.dtype);
    fams.push_back("recurrent");
    return fams;
  }

  std::vector<StateNeed> state_need() const override {
    std::vector<StateNeed> needs = {{"channel_delta.S", {(int64_t)n_heads_, (int64_t)dv_, (int64_t)d_}, DType::F32}};
    if (taps_ > 1) needs.push_back({"channel_delta.inputs", {(int64_t)taps_ - 1, conv_width_}, DType::F32});
    return needs;
  }

  Act forward(StepContext &ctx, const Act &x, LayerCache *, StateView *state) override {
    float *S = nullptr;
    void *inputs = nullptr;
    if (state)
      for (const auto &t : *state) {
        if (t.name == "channel_delta.S") S = (float *)t.data;
        if (t.name == "channel_delta.inputs") inputs = t.data;
      }
    if (!S || (taps_ > 1 && !inputs)) LLM_THROW(InvalidArg, "channel_delta: the run has no state");
    Act proj = linear(ctx, x, w_in_, nullptr, DType::F32);
    flush_chain(ctx);
    const int T = ctx.n_tokens;
    // a row of `cv`: the convolved q | k | v, then room for every head's query and the key it learns
    Act cv = ctx.arena->act(DType::F32, T, row_ld_);
    Act conv_in = proj, conv_out = cv;
    conv_in.cols = conv_out.cols = conv_width_;
    kernels::causal_conv(conv_in, conv_out, conv_.buf.as<float>(), inputs, ctx.tok_seq, ctx.tok_pos, ctx.seq_start, ctx.seq_past,
                         ctx.seq_slot, ctx.n_seqs, taps_, ctx.decode_only, ctx.stream, true);
    float *prep = ctx.arena->alloc_n<float>((size_t)T * (size_t)k_width_ * 3);
    float *gate = ctx.arena->alloc_n<float>((size_t)T * (size_t)v_width_);
    kernels::channel_delta_prepare(cv, proj, (int)off_b_, (int)off_a1_, (int)rank_a_, (int)off_g1_, (int)rank_g_, a2_.buf.as<float>(),
                                   dt_bias_.buf.as<float>(), a_log_.buf.as<float>(), g2_.buf.as<float>(), key_eps_, prep, gate, n_heads_,
                                   n_kv_, d_, dv_, ctx.stream);
    Act o = ctx.arena->act(DType::F32, T, v_width_);
    kernels::delta_scan(cv, (int)conv_width_, (int)(conv_width_ + k_width_), (int)(2 * qk_width_), prep, S, o, ctx.seq_start, ctx.seq_slot,
                        ctx.n_seqs, n_heads_, d_, dv_, ctx.stream);
    Act y = ctx.arena->act(ctx.dtype, T, v_width_);
    kernels::head_norm_gate(o, norm_.buf.as<float>(), gate, v_width_, eps_, n_heads_, dv_, y, ctx.stream);
    return linear(ctx, y, w_o_, nullptr, DType::F32, true);
  }

 private:
  int64_t hidden_, qk_width_, k_width_, v_width_, conv_width_, row_ld_, rank_a_, rank_g_;
  int64_t off_b_ = 0, off_a1_ = 0, off_g1_ = 0;
  int n_heads_, n_kv_, d_, dv_, taps_;
  float eps_, key_eps_;
  std::vector<std::string> names_;
  Weight w_in_, conv_, a2_, dt_bias_, a_log_, g2_, norm_, w_o_;
};

}  // namespace

void register_part_raw(const std::string &category, const std::string &kind, PartFactory factory);   // parts/part.cc

void register_recurrent_parts() {
  register_part_raw("mixer", "general_delta",
                    [](const Json &spec, const BuildEnv &env) { return std::unique_ptr<Part>(new GeneralDelta(spec, env)); });
  register_part_raw("mixer", "channel_delta",
                    [](const Json &spec, const BuildEnv &env) { return std::unique_ptr<Part>(new ChannelDelta(spec, env)); });
}

}  // namespace llm
