// Feed-forwards beyond the reference's SwiGLU: the two-matrix form with a choice of activation, and
// the routed form (mixture of experts) over it.
#include <algorithm>

#include "config/config.h"
#include "csrc/kernels.h"
#include "parts/chain.h"
#include "parts/linear.h"
#include "parts/part.h"

namespace llm {

namespace {

int activation_code(const std::string &name, const ConfigReader &r) {
  if (name == "gelu") return kernels::GeluErf;          // 0.5 z (1 + erf(z / sqrt 2))
  if (name == "gelu_tanh") return kernels::GeluTanh;    // 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
  if (name == "silu") return kernels::Silu;
  if (name == "relu2") return kernels::Relu2;           // max(z, 0)^2
  r.fail("activation '" + name + "' is not known (gelu, gelu_tanh, silu, relu2)");
}

// ---------------------------------------------------------------- up, activation, down
// down(act(up x)), no biases; the activation in 32-bit on the product's 32-bit result.
class Mlp : public FeedForward {
 public:
  Mlp(const Json &spec, const BuildEnv &env) : FeedForward(spec, env) {
    ConfigReader r(spec, "mlp description");
    hidden_ = r.integer("hidden");
    inter_ = r.integer("intermediate");
    act_ = activation_code(r.string_or("activation", "gelu"), r);
    up_ = r.string("up");
    down_ = r.string("down");
  }
  std::vector<TensorNeed> tensor_needs() const override { return {{up_, {inter_, hidden_}}, {down_, {hidden_, inter_}}}; }
  void load(const Loader &l) override {
    const auto needs = tensor_needs();
    w_up_ = l.fetch(needs[0]);
    w_down_ = l.fetch(needs[1]);
  }
  std::vector<std::string> kernel_families() const override {
    std::vector<std::string> fams = product_families(env_.dtype);
    fams.push_back("moe");
    return fams;
  }
  Act forward(StepContext &ctx, const Act &x) override {
    Act u = linear(ctx, x, w_up_, nullptr, DType::F32);
    flush_chain(ctx);
    Act m = ctx.arena->act(ctx.dtype, x.rows, inter_);
    kernels::activation(u, m, act_, ctx.stream);
    return linear(ctx, m, w_down_, nullptr, DType::F32, true);
  }

 private:
  int64_t hidden_, inter_;
  int act_;
  std::string up_, down_;
  Weight w_up_, w_down_;
};

// ---------------------------------------------------------------- routed experts
// Router logits z = W_router x (a product with 32-bit accumulation and a 32-bit result), scores
// sigmoid(z) or softmax(z), the `top` largest chosen; their scores, as they are or divided by
// their sum (`renormalize`), weigh the experts.  `weight_on` "input": the output is the sum of
// expert(w x); "output": of w expert(x).  Experts are two-matrix feed-forwards whose tensors are
// named by a pattern with "{}" for the expert's number; they lie stacked on the device,
// [experts, ff, hidden] and [experts, hidden, ff].  A `shared` feed-forward (any description) runs
// for every token and is added.  With `expert.gate` (a third pattern) an expert is down(act(gate x) * up x); its
// gate and up rows lie interleaved in one stacked matrix [experts, 2 ff, hidden] and the weight goes on the
// output.  The result is [parts, T, hidden]: a part per choice, then the
// shared one's, which the stream adds in that order.
// Further keys, all optional: `correction`, a vector over the experts that is added to the scores for the CHOICE
// only (the weights use the scores as they are); `groups` {count, keep, top}: the experts form `count` equal groups
// of neighbours, a group's score is the sum of its `top` (2) largest corrected scores, and only experts of the `keep`
// best groups can be chosen; `norm_eps`, added to the sum that `renormalize` divides by; `route_scale`, a factor on
// the weights; `shared_gate`, a matrix [1, hidden]: the shared feed-forward's result is multiplied by sigmoid(gate x),
// one number per token (its row rides behind the router's rows in one stacked product).
class RoutedFeedForward : public FeedForward {
 public:
  RoutedFeedForward(const Json &spec, const BuildEnv &env) : FeedForward(spec, env) {
    ConfigReader r(spec, "moe description");
    hidden_ = r.integer("hidden");
    experts_ = (int)r.integer("experts");
    top_ = (int)r.integer("top");
    if (top_ > experts_) r.fail("'top' exceeds 'experts'");
    const std::string score = r.string_or("score", "softmax");
    if (score != "sigmoid" && score != "softmax") r.fail("'score' must be \"sigmoid\" or \"softmax\"");
    score_ = score == "softmax" ? 1 : 0;
    renormalize_ = r.boolean_or("renormalize", false);
    const std::string on = r.string_or("weight_on", "output");
    if (on != "input" && on != "output") r.fail("'weight_on' must be \"input\" or \"output\"");
    weight_on_output_ = on == "output";
    router_ = r.string("router");
    ConfigReader e(r.object("expert"), "moe description: expert");
    inter_ = e.integer("intermediate");
    act_ = activation_code(e.string_or("activation", "gelu"), e);
    up_ = e.string("up");
    down_ = e.string("down");
    gate_ = e.string_or("gate", "");
    if (up_.find("{}") == std::string::npos || down_.find("{}") == std::string::npos ||
        (!gate_.empty() && gate_.find("{}") == std::string::npos))
      e.fail("'up', 'down' and 'gate' are patterns with \"{}\" for the expert's number");
    if (!gate_.empty() && !weight_on_output_) e.fail("gated experts take their weight on the output");
    if (r.present("shared")) shared_ = build_as<FeedForward>("feed_forward", r.object("shared"), env);
    correction_ = r.string_or("correction", "");
    if (r.present("groups")) {
      ConfigReader g(r.object("groups"), "moe description: groups");
      groups_ = (int)g.integer("count");
      keep_ = (int)g.integer("keep");
      group_top_ = (int)g.integer_or("top", 2);
      if (experts_ % groups_) g.fail("'count' must divide the number of experts");
      if (keep_ > groups_) g.fail("'keep' exceeds 'count'");
      if ((int64_t)keep_ * (experts_ / groups_) < top_) g.fail("the kept groups hold fewer experts than 'top'");
    }
    norm_eps_ = (float)r.number_or("norm_eps", 0.0, false);
    route_scale_ = (float)r.number_or("route_scale", 1.0, false);
    shared_gate_ = r.string_or("shared_gate", "");
    if (!shared_gate_.empty() && !shared_) r.fail("'shared_gate' goes with a 'shared' feed-forward");
    grouped_route_ = !correction_.empty() || groups_ > 1 || norm_eps_ != 0.f || route_scale_ != 1.f;
    router_rows_ = shared_gate_.empty() ? experts_ : (experts_ + 1 + 7) / 8 * 8;
  }
  static std::string numbered(const std::string &pattern, int e) {
    std::string s = pattern;
    s.replace(s.find("{}"), 2, std::to_string(e));
    return s;
  }
  std::vector<TensorNeed> tensor_needs() const override {
    std::vector<TensorNeed> needs = {{router_, {(int64_t)experts_, hidden_}}};
    for (int e = 0; e < experts_; ++e) {
      needs.push_back({numbered(up_, e), {inter_, hidden_}});
      needs.push_back({numbered(down_, e), {hidden_, inter_}});
      if (!gate_.empty()) needs.push_back({numbered(gate_, e), {inter_, hidden_}});
    }
    if (shared_)
      for (auto &n : shared_->tensor_needs()) needs.push_back(n);
    if (!correction_.empty()) needs.push_back({correction_, {(int64_t)experts_}, TensorRole::Vector, false});
    if (!shared_gate_.empty()) needs.push_back({shared_gate_, {1, hidden_}});
    return needs;
  }
  void load(const Loader &l) override {
    const auto needs = tensor_needs();
    if (shared_gate_.empty()) {
      w_router_ = l.fetch(needs[0]);
    } else {
      // [router; the shared feed-forward's gate; zeros up to a multiple of 8 rows]
      const size_t row_bytes = (size_t)hidden_ * dtype_size(l.engine);
      w_router_.dtype = l.engine;
      w_router_.rows = router_rows_;
      w_router_.cols = hidden_;
      w_router_.buf.allocate((size_t)router_rows_ * row_bytes, true);
      l.fetch_into(needs[0], l.engine, w_router_.buf.get());
      l.fetch_into(needs.back(), l.engine, (char *)w_router_.buf.get() + (size_t)experts_ * row_bytes);
    }
    if (!correction_.empty()) w_correction_ = l.fetch(needs[needs.size() - (shared_gate_.empty() ? 1 : 2)]);
    const size_t es = dtype_size(l.engine), one = (size_t)(inter_ * hidden_) * es;
    const bool gated = !gate_.empty();
    const size_t per = gated ? 3 : 2, row = (size_t)hidden_ * es;
    w_up_.allocate(one * (size_t)experts_ * (gated ? 2 : 1));
    w_down_.allocate(one * (size_t)experts_);
    DeviceBuffer staged;
    if (gated) staged.allocate(one);
    for (int e = 0; e < experts_; ++e) {
      l.fetch_into(needs[2 + per * (size_t)e], l.engine, (char *)w_down_.get() + one * (size_t)e);
      if (!gated) {
        l.fetch_into(needs[1 + per * (size_t)e], l.engine, (char *)w_up_.get() + one * (size_t)e);
        continue;
      }
      // row 2n: the gate's row n; row 2n + 1: the up row n
      char *dst = (char *)w_up_.get() + 2 * one * (size_t)e;
      for (int half = 0; half < 2; ++half) {
        l.fetch_into(needs[(half == 0 ? 3 : 1) + per * (size_t)e], l.engine, staged.get());
        LLM_CUDA(cudaMemcpy2D(dst + (size_t)half * row, 2 * row, staged.get(), row, row, (size_t)inter_, cudaMemcpyDeviceToDevice));
      }
    }
    if (shared_) shared_->load(l);
  }
  std::vector<std::string> kernel_families() const override {
    std::vector<std::string> fams = product_families(env_.dtype);
    fams.push_back("moe");
    if (env_.dtype == DType::BF16 && fast_switches().moe_tc && hidden_ % 8 == 0 && inter_ % 8 == 0) fams.push_back("moe_tc");
    if (shared_)
      for (auto &f : shared_->kernel_families()) fams.push_back(f);
    return fams;
  }
  bool capturable() const override { return !shared_ || shared_->capturable(); }

  Act forward(StepContext &ctx, const Act &x) override {
    const int64_t T = x.rows;
    // the shared expert first: its last product may add to the residual stream as it stores
    Act s;
    float *const sink = ctx.residual_sink;
    if (!shared_gate_.empty()) ctx.residual_sink = nullptr;   // a gated result cannot be added by the product that makes it
    if (shared_) s = shared_->forward(ctx, x);
    const bool s_own = s.data && s.data != (void *)sink;
    ctx.residual_sink = nullptr;                     // what follows returns its own buffers
    Act z = linear(ctx, x, w_router_, nullptr, DType::F32);
    ctx.residual_sink = sink;
    flush_chain(ctx);
    const int n_rows = (int)T * top_;
    int *chosen = ctx.arena->alloc_n<int>((size_t)n_rows);
    float *weight = ctx.arena->alloc_n<float>((size_t)n_rows);
    if (grouped_route_)
      kernels::moe_route_grouped(z, experts_, top_, score_, correction_.empty() ? nullptr : w_correction_.buf.as<float>(), groups_, keep_,
                                 group_top_, renormalize_, norm_eps_, route_scale_, chosen, weight, ctx.stream);
    else
      kernels::moe_route(z, experts_, top_, score_, renormalize_, chosen, weight, ctx.stream);
    Act out = ctx.arena->act(DType::F32, T, hidden_, top_ + (s_own ? s.parts : 0));
    const bool aligned = x.dtype == DType::BF16 && x.ld % 8 == 0 && (uintptr_t)x.data % 16 == 0;
    if (aligned && fast_switches().moe_tc && kernels::available("moe_tc") && kernels::moe_tc_supported((int)hidden_, (int)inter_)) {
      const int tile = kernels::moe_tc_tile_rows(n_rows);
      int *offsets = ctx.arena->alloc_n<int>((size_t)experts_ + 1);
      int *perm = ctx.arena->alloc_n<int>((size_t)n_rows);
      int *tiles = ctx.arena->alloc_n<int>(1 + 2 * ((size_t)std::min(experts_, n_rows) + (size_t)(n_rows / tile)));
      void *xs = ctx.arena->alloc((size_t)n_rows * (size_t)hidden_ * 2);
      void *mid = ctx.arena->alloc((size_t)n_rows * (size_t)inter_ * 2);
      kernels::moe_sort(chosen, n_rows, experts_, tile, offsets, perm, tiles, ctx.stream);
      kernels::moe_tc(x, w_up_.get(), w_down_.get(), offsets, perm, tiles, weight, experts_, top_, (int)hidden_, (int)inter_, act_,
                      weight_on_output_, xs, mid, (float *)out.data, ctx.tc_status, ctx.stream, !gate_.empty());
    } else if (aligned && kernels::moe_grouped_supported((int)hidden_, (int)inter_)) {
      const int tile = kernels::moe_tile_rows();
      int *offsets = ctx.arena->alloc_n<int>((size_t)experts_ + 1);
      int *perm = ctx.arena->alloc_n<int>((size_t)n_rows);
      int *tiles = ctx.arena->alloc_n<int>(1 + 2 * ((size_t)std::min(experts_, n_rows) + (size_t)(n_rows / tile)));
      void *mid = ctx.arena->alloc((size_t)n_rows * (size_t)inter_ * 2);
      kernels::moe_sort(chosen, n_rows, experts_, tile, offsets, perm, tiles, ctx.stream);
      kernels::moe_grouped(x, w_up_.get(), w_down_.get(), offsets, perm, tiles, weight, experts_, top_, (int)hidden_, (int)inter_,
                           act_, weight_on_output_, mid, (float *)out.data, ctx.stream, !gate_.empty());
    } else {
      kernels::moe_rows(x, w_up_.get(), w_down_.get(), chosen, weight, top_, (int)hidden_, (int)inter_, act_, weight_on_output_,
                        (float *)out.data, ctx.stream, !gate_.empty());
    }
    if (s_own) {
      if (s.dtype != DType::F32 || s.rows != T || s.cols != hidden_ || s.ld != hidden_)
        LLM_THROW(Unsupported, "moe: the shared feed-forward must hand over dense 32-bit rows");
      if (!shared_gate_.empty())
        kernels::row_gate((const float *)s.data, s.part_stride, (float *)out.data + (size_t)top_ * (size_t)out.part_stride,
                          out.part_stride, s.parts, (const float *)z.data + experts_, z.ld, (int)T, (int)hidden_, ctx.stream);
      for (int p = 0; p < s.parts && shared_gate_.empty(); ++p)
        LLM_CUDA(cudaMemcpyAsync((float *)out.data + (size_t)(top_ + p) * (size_t)out.part_stride,
                                 (const float *)s.data + (size_t)p * (size_t)s.part_stride, sizeof(float) * (size_t)(T * hidden_),
                                 cudaMemcpyDeviceToDevice, ctx.stream));
    }
    return out;
  }

 private:
  int64_t hidden_, inter_;
  int experts_, top_, score_, act_;
  bool renormalize_, weight_on_output_, grouped_route_ = false;
  int groups_ = 1, keep_ = 1, group_top_ = 2, router_rows_ = 0;
  float norm_eps_ = 0.f, route_scale_ = 1.f;
  std::string router_, up_, down_, gate_, correction_, shared_gate_;
  Weight w_router_, w_correction_;
  DeviceBuffer w_up_, w_down_;
  std::unique_ptr<FeedForward> shared_;
};

// ---------------------------------------------------------------- clamped gated unit
// down(g * sigmoid(slope g) * (u + up_shift)) with g = min(gate x, limit), u = clamp(up x, -limit, limit).
// Gate and up are one stacked product with a 32-bit result; their biases (optional) are added where the
// unit is computed, in 32-bit, so that the product runs on the tensor cores like any other; the down
// matrix's bias (optional) rides with the result and is added, in 32-bit, by the pass that adds the
// result to the residual stream (Act::col_bias).  `limit` 0: no bounds.
class ClampedGlu : public FeedForward {
 public:
  ClampedGlu(const Json &spec, const BuildEnv &env) : FeedForward(spec, env) {
    ConfigReader r(spec, "clamped_glu description");
    hidden_ = r.integer("hidden");
    inter_ = r.integer("intermediate");
    limit_ = (float)r.number_or("limit", 0.0, false);
    slope_ = (float)r.number_or("slope", 1.0, false);
    up_shift_ = (float)r.number_or("up_shift", 0.0, false);
    if (limit_ < 0.f) r.fail("'limit' must not be negative");
    gate_ = r.string("gate");
    up_ = r.string("up");
    down_ = r.string("down");
    gate_bias_ = r.string_or("gate_bias", "");
    up_bias_ = r.string_or("up_bias", "");
    down_bias_ = r.string_or("down_bias", "");
    if (gate_bias_.empty() != up_bias_.empty()) r.fail("'gate_bias' and 'up_bias' come together");
  }
  std::vector<TensorNeed> tensor_needs() const override {
    std::vector<TensorNeed> needs = {{gate_, {inter_, hidden_}}, {up_, {inter_, hidden_}}, {down_, {hidden_, inter_}}};
    if (!gate_bias_.empty()) {
      needs.push_back({gate_bias_, {inter_}, TensorRole::Vector, false});
      needs.push_back({up_bias_, {inter_}, TensorRole::Vector, false});
    }
    if (!down_bias_.empty()) needs.push_back({down_bias_, {hidden_}, TensorRole::Vector, false});
    return needs;
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
    size_t next = 3;
    if (!gate_bias_.empty()) {
      b_gate_up_.dtype = DType::F32;
      b_gate_up_.rows = 1;
      b_gate_up_.cols = 2 * inter_;
      b_gate_up_.buf.allocate((size_t)(2 * inter_) * sizeof(float));
      l.fetch_into(needs[next], DType::F32, b_gate_up_.buf.get());
      l.fetch_into(needs[next + 1], DType::F32, b_gate_up_.buf.as<float>() + inter_);
      next += 2;
    }
    if (!down_bias_.empty()) b_down_ = l.fetch(needs[next]);
  }
  std::vector<std::string> kernel_families() const override {
    std::vector<std::string> fams = product_families(env_.dtype);
    fams.push_back("elementwise");
    return fams;
  }
  Act forward(StepContext &ctx, const Act &x) override {
    Act gu = linear(ctx, x, w_gate_up_, nullptr, DType::F32);
    flush_chain(ctx);
    Act m = ctx.arena->act(ctx.dtype, x.rows, inter_);
    kernels::clamped_glu(gu, gate_bias_.empty() ? nullptr : b_gate_up_.buf.as<float>(), m, limit_, slope_, up_shift_, ctx.stream);
    if (down_bias_.empty()) return linear(ctx, m, w_down_, nullptr, DType::F32, true);
    // with a bias the product cannot add to the stream as it stores: the bias goes with the result
    float *const sink = ctx.residual_sink;
    ctx.residual_sink = nullptr;
    Act y = linear(ctx, m, w_down_, nullptr, DType::F32, true);
    ctx.residual_sink = sink;
    y.col_bias = b_down_.buf.as<float>();
    return y;
  }

 private:
  int64_t hidden_, inter_;
  float limit_, slope_, up_shift_;
  std::string gate_, up_, down_, gate_bias_, up_bias_, down_bias_;
  Weight w_gate_up_, w_down_, b_gate_up_, b_down_;
};

template <typename T>
PartFactory factory_of() {
  return [](const Json &spec, const BuildEnv &env) { return std::unique_ptr<Part>(new T(spec, env)); };
}

}  // namespace

void register_part_raw(const std::string &category, const std::string &kind, PartFactory factory);   // parts/part.cc

void register_feed_forward_parts() {
  register_part_raw("feed_forward", "mlp", factory_of<Mlp>());
  register_part_raw("feed_forward", "moe", factory_of<RoutedFeedForward>());
  register_part_raw("feed_forward", "clamped_glu", factory_of<ClampedGlu>());
}

}  // namespace llm
