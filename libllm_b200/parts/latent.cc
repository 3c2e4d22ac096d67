// "latent_attention": attention whose keys and values are functions of one cached vector per position.
//
// With h the mixer's input, H heads of `head_dim` unrotated and `rot_dim` rotated query/key channels, values of
// `v_head_dim`, latents of `q_rank` and `kv_rank` channels:
//   c_q = rms(W_dq h) * q_norm,   q = W_uq c_q, head by head [head_dim unrotated | rot_dim rotated]
//   [c' | k_r'] = W_dkv h,        c = rms(c') * kv_norm,   k_r = rotated k_r' (one part that all heads share)
//   head: k = [W_uk c | k_r], v = W_uv c, score = (q . k) * scale, causal softmax, then W_o on the heads.
// Only [c | k_r] is cached: one row of kv_rank + rot_dim channels per position (cache need: one key head of
// that width, no value storage).  The products with W_uk and W_uv are moved to the query's side and behind the
// weighted sum (csrc/latent.cu says how), so a step reads the cached rows once per head and never expands them.
// A run that the schedule gives another run's cache (ScheduleEntry::cache_from) has no W_dkv of its own: it
// reads the rows that run appended, with its own W_uk, W_uv and queries.  With `window` w a query at position p sees the
// rows of positions p - w + 1 .. p only, and the cache gives earlier pages back.  The rotation is the position part's
// (either pairing; its table carries whatever the scaling puts on cosines and sines); `scale` is the
// description's.  The reference has no such mixer (its attention: src/libllm/llama.cc:178-225).
#include <algorithm>
#include <cmath>

#include "config/config.h"
#include "csrc/kernels.h"
#include "parts/chain.h"
#include "parts/linear.h"
#include "parts/part.h"

namespace llm {

namespace {

class LatentAttention : public Mixer {
 public:
  LatentAttention(const Json &spec, const BuildEnv &env) : Mixer(spec, env) {
    ConfigReader r(spec, "latent_attention description");
    hidden_ = r.integer("hidden");
    n_heads_ = (int)r.integer("n_heads");
    d_ = (int)r.integer("head_dim");
    rot_ = (int)r.integer("rot_dim", 0);
    dv_ = (int)r.integer_or("v_head_dim", d_);
    kv_rank_ = (int)r.integer("kv_rank");
    q_rank_ = (int)r.integer("q_rank");
    scale_ = (float)r.number_or("scale", 1.0 / std::sqrt((double)(d_ + rot_)), false);
    eps_ = (float)r.number("eps");
    window_ = (int)r.integer_or("window", 0, 0);
    q_down_ = r.string("q_down");
    q_norm_ = r.string("q_norm");
    q_up_ = r.string("q_up");
    kv_down_ = r.string_or("kv_down", "");
    kv_norm_ = r.string_or("kv_norm", "");
    if (kv_down_.empty() != kv_norm_.empty()) r.fail("'kv_down' and 'kv_norm' come together");
    k_up_ = r.string("k_up");
    v_up_ = r.string("v_up");
    o_ = r.string("o");
    if (rot_ % 2) r.fail("'rot_dim' must be even");
    if (kv_rank_ + rot_ > 1024 || kv_rank_ > 1024)
      LLM_THROW(Unsupported, "latent_attention: cached rows of %d channels are not supported (up to 1024)", kv_rank_ + rot_);
    if (rot_ > 0) {
      if (spec.get("position").is_null()) r.fail("rotated channels need a 'position' part");
      position_ = build_as<PositionEncoding>("position", spec.get("position"), env);
    }
    down_rows_ = ((int64_t)q_rank_ + (own_latent() ? kv_rank_ + rot_ : 0) + 7) / 8 * 8;
  }
  bool own_latent() const { return !kv_down_.empty(); }

  std::vector<TensorNeed> tensor_needs() const override {
    std::vector<TensorNeed> needs = {{q_down_, {(int64_t)q_rank_, hidden_}},
                                     {q_norm_, {(int64_t)q_rank_}, TensorRole::Vector, false},
                                     {q_up_, {(int64_t)n_heads_ * (d_ + rot_), (int64_t)q_rank_}},
                                     {k_up_, {(int64_t)n_heads_ * d_, (int64_t)kv_rank_}},
                                     {v_up_, {(int64_t)n_heads_ * dv_, (int64_t)kv_rank_}},
                                     {o_, {hidden_, (int64_t)n_heads_ * dv_}}};
    if (own_latent()) {
      needs.push_back({kv_down_, {(int64_t)kv_rank_ + rot_, hidden_}});
      needs.push_back({kv_norm_, {(int64_t)kv_rank_}, TensorRole::Vector, false});
    }
    if (position_)
      for (auto &n : position_->tensor_needs()) needs.push_back(n);
    return needs;
  }

  void load(const Loader &l) override {
    const std::vector<TensorNeed> needs = tensor_needs();
    const size_t es = dtype_size(l.engine);
    // both latents' projections are one stacked product [W_dq; W_dkv] with a 32-bit result
    w_down_.dtype = l.engine;
    w_down_.rows = down_rows_;
    w_down_.cols = hidden_;
    w_down_.buf.allocate((size_t)down_rows_ * (size_t)hidden_ * es, true);
    l.fetch_into(needs[0], l.engine, w_down_.buf.get());
    w_q_norm_ = l.fetch(needs[1]);
    w_uq_ = l.fetch(needs[2]);
    w_uk_ = l.fetch(needs[3]);
    w_uv_ = l.fetch(needs[4]);
    w_o_ = l.fetch(needs[5]);
    if (l.engine == DType::BF16) {
      // [W_uk; W_uv] stacked, for prompt steps that materialise the heads' keys and values in one product
      const int64_t k_rows = (int64_t)n_heads_ * d_, v_rows = (int64_t)n_heads_ * dv_;
      w_ukv_.dtype = l.engine;
      w_ukv_.rows = (k_rows + v_rows + 7) / 8 * 8;
      w_ukv_.cols = kv_rank_;
      w_ukv_.buf.allocate((size_t)w_ukv_.rows * (size_t)kv_rank_ * es, true);
      l.fetch_into(needs[3], l.engine, w_ukv_.buf.get());
      l.fetch_into(needs[4], l.engine, (char *)w_ukv_.buf.get() + (size_t)k_rows * kv_rank_ * es);
    }
    if (own_latent()) {
      l.fetch_into(needs[6], l.engine, (char *)w_down_.buf.get() + (size_t)q_rank_ * hidden_ * es);
      w_kv_norm_ = l.fetch(needs[7]);
    }
    if (position_) position_->load(l);
  }

  std::vector<std::string> kernel_families() const override {
    std::vector<std::string> fams = product_families(env_.dtype);
    fams.push_back("latent");
    if (env_.dtype == DType::BF16) fams.push_back("latent_tc");
    fams.push_back("attention_generic");
    return fams;
  }

  bool wants_cache() const override { return true; }
  CacheNeed cache_need() const override {
    CacheNeed n;
    n.kind = window_ > 0 ? "window" : "full";    // pages that have left every later query's window go back to the pool
    n.window = window_;
    n.n_kv_heads = 1;
    n.k_dim = kv_rank_ + rot_;
    n.v_dim = 0;                                       // the values are functions of the key rows
    return n;
  }

  Act forward(StepContext &ctx, const Act &x, LayerCache *cache, StateView *) override {
    if (!cache) LLM_THROW(InvalidArg, "latent_attention: the run has no cache to attend over");
    if (cache->need.n_kv_heads != 1 || cache->need.k_dim != kv_rank_ + rot_)
      LLM_THROW(Config, "latent_attention: the cache holds rows of %d x %d channels, this run reads rows of %d", cache->need.n_kv_heads,
                cache->need.k_dim, kv_rank_ + rot_);
    if (own_latent() != cache->writes)
      LLM_THROW(Config, own_latent() ? "latent_attention: a run with a latent projection of its own was given another run's cache"
                                     : "latent_attention: a run without a latent projection needs another run's cache");
    int table_rows = 0, rot = 0;
    bool interleaved = false;
    const float *table = nullptr;
    if (position_) {
      table = position_->pair_table(&table_rows, &rot, &interleaved);
      if (!table || rot != rot_) LLM_THROW(Unsupported, "latent_attention: the position part has no table of %d rotated channels", rot_);
    }
    const int T = ctx.n_tokens;
    const int row = kv_rank_ + rot_;
    Act proj = linear(ctx, x, w_down_, nullptr, DType::F32);
    flush_chain(ctx);
    Act cq = ctx.arena->act(ctx.dtype, T, q_rank_);
    kernels::latent_place(proj, 0, q_rank_, w_q_norm_.buf.as<float>(), cq, own_latent() ? q_rank_ : -1, kv_rank_, rot_,
                          own_latent() ? w_kv_norm_.buf.as<float>() : nullptr, eps_, table, table_rows, interleaved, ctx.tok_seq,
                          ctx.tok_pos, cache->page_table, cache->table_width, cache->k, cache->page_size, ctx.stream);
    const bool tc = ctx.dtype == DType::BF16 && kernels::available("latent_tc");
    bool from_start = !ctx.decode_only && !ctx.captured && (int)ctx.past_lens.size() == ctx.n_seqs;
    for (int past : ctx.past_lens) from_start = from_start && past == 0;
    Act heads = ctx.arena->act(ctx.dtype, T, (int64_t)n_heads_ * dv_);
    if (tc && from_start && w_ukv_.buf.get() && kernels::latent_prefill_supported(d_, rot_, dv_)) {
      // every sequence brings its first tokens: the heads' keys and values of the step's own rows are one product
      // over the rows as the cache holds them, and the attention is the flash form over those
      Act c = ctx.arena->act(ctx.dtype, T, kv_rank_);
      Act kr = ctx.arena->act(ctx.dtype, T, std::max(rot_, 8));
      kr.cols = kr.ld = rot_;
      kernels::latent_rows(cache->k, cache->page_size, row, kv_rank_, ctx.tok_seq, ctx.tok_pos, cache->page_table, cache->table_width, T,
                           c, kr, ctx.stream);
      Act q = linear(ctx, cq, w_uq_, nullptr, DType::F32);
      Act kv = linear(ctx, c, w_ukv_, nullptr, ctx.dtype);
      flush_chain(ctx);
      Act qb = ctx.arena->act(ctx.dtype, T, (int64_t)n_heads_ * (d_ + rot_));
      kernels::latent_rotate_q(q, qb, n_heads_, d_, rot_, table, table_rows, interleaved, ctx.tok_pos, ctx.stream);
      kernels::latent_prefill(qb, kv, kr, heads, ctx.seq_start, ctx.n_seqs, ctx.max_q_len, n_heads_, d_, rot_, dv_, scale_, ctx.stream,
                              window_);
      return linear(ctx, heads, w_o_, nullptr, DType::F32, true);
    }
    Act q = linear(ctx, cq, w_uq_, nullptr, DType::F32);
    flush_chain(ctx);
    Act qa = ctx.arena->act(ctx.dtype, T, (int64_t)n_heads_ * row);
    kernels::latent_absorb(q, w_uk_.buf.get(), qa, n_heads_, d_, rot_, kv_rank_, table, table_rows, interleaved, ctx.tok_pos, ctx.stream);
    Act mixed = ctx.arena->act(ctx.dtype, T, (int64_t)n_heads_ * kv_rank_);
    if (tc && kernels::latent_decode_supported(kv_rank_, rot_)) {
      // all heads of a token over the cached rows.  A run's partial result is heads x kv_rank 32-bit sums, as many
      // bytes as some tens of cached rows, so a run takes at least 256 keys; within that, enough runs to give
      // every multiprocessor a CTA.  The same for every step of a captured graph.
      const int max_len = window_ > 0 ? std::min(std::max(ctx.max_kv_len, 1), window_ + 63) : std::max(ctx.max_kv_len, 1);
      const int ctas = std::max(1, T * ((n_heads_ + 31) / 32));
      const int want = std::max(1, (ctx.sm_count + ctas - 1) / ctas);
      const int most = std::max(1, max_len / (window_ > 0 ? 128 : 256));      // under a window a token has few keys: shorter runs, more CTAs
      const int n_splits = std::max(1, std::min(std::min(want, most), 64));
      float *ws = nullptr;
      if (n_splits > 1) ws = ctx.arena->alloc_n<float>(kernels::latent_decode_floats(T, n_heads_, kv_rank_, n_splits));
      kernels::latent_decode(qa, cache->k, cache->page_size, ctx.tok_seq, ctx.tok_pos, cache->page_table, cache->table_width, n_heads_,
                             kv_rank_, rot_, n_splits, scale_, mixed, ws, ctx.stream, window_);
    } else {
      kernels::attention_generic(qa, mixed, cache->k, cache->k, ctx.tok_seq, ctx.tok_pos, cache->page_table, cache->table_width, n_heads_,
                                 1, row, kv_rank_, cache->page_size, window_, 0, scale_, nullptr, 0, ctx.stream, 0, row);
    }
    kernels::latent_expand(mixed, w_uv_.buf.get(), heads, n_heads_, kv_rank_, dv_, ctx.stream);
    return linear(ctx, heads, w_o_, nullptr, DType::F32, true);
  }

 private:
  int64_t hidden_, down_rows_;
  int n_heads_, d_, rot_, dv_, kv_rank_, q_rank_, window_ = 0;
  float scale_, eps_;
  std::string q_down_, q_norm_, q_up_, kv_down_, kv_norm_, k_up_, v_up_, o_;
  std::unique_ptr<PositionEncoding> position_;
  Weight w_down_, w_q_norm_, w_uq_, w_uk_, w_uv_, w_ukv_, w_o_, w_kv_norm_;
};

}  // namespace

void register_part_raw(const std::string &category, const std::string &kind, PartFactory factory);   // parts/part.cc

void register_latent_parts() {
  register_part_raw("mixer", "latent_attention",
                    [](const Json &spec, const BuildEnv &env) { return std::unique_ptr<Part>(new LatentAttention(spec, env)); });
}

}  // namespace llm
