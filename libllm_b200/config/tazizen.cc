// The Tazizen decoder: its configuration and its description as parts.
//
// config.json (`architecture`: "Tazizen") lists the layers one by one; every size and constant is read from it.
// The stream starts as the token's row ("embed").  With `streams` S the model carries S copies of the residual
// stream and every sublayer is joined to them by three small tensors ("l<i>.hc<q>.in" [S], ".out" [S], ".mix"
// [S, S]; q = 1 the mixer, 2 the feed-forward; block kind "hyper"); without the key a layer is the plain pre-norm
// block.  Norms are RMS norms whose weight is stored around nought and applied as (1 + w) ("l<i>.norm1",
// "l<i>.norm2", "final.norm").  A layer names
//   type   "attention": grouped-query attention, a rotation of the first rot.dims channels of every head in
//          pairs (i, i + dims/2) with optional YaRN scaling, after it every query and key head divided by its
//          root mean square (no weight), a score scale of its own, a sliding window (mask.size), a softmax with
//          one added to its denominator (a key of score 0 without a value), a sigmoid gate per channel on the
//          concatenated heads (".g"), computed from the mixer's input;
//          "latent_attention": queries through a normed latent of q_rank channels, keys and values through a
//          normed latent of kv_rank channels plus one rotated key part of rot_dim channels that all heads share
//          (parts/latent.cc), a sliding window, the ordinary softmax;
//   mlp    null, or {kind "moe"}: experts down(silu(gate h) * up h) chosen by sigmoid scores plus a correction,
//          among the best groups of experts, weighted by their scores over their sum times router.scale, plus a
//          shared expert times sigmoid(sg h) (parts/feed_forward.cc).
// `loop` {start, stop, times}: layers start .. stop-1 run `times` times in a row with the same weights, each pass
// with a cache of its own.  Last: the norm over the sum of the copies, then logits = head x.
#include <cmath>

#include "config/config.h"

namespace llm {

namespace {

// What a model of this design can hold when the engine names no shorter bound: the configuration itself has no
// longest sequence.
const int64_t TAZIZEN_MAX_POSITIONS = 1 << 20;
// The design's constants.
const double ROUTE_NORM_EPS = 1e-20;    // weights: s / (sum of the chosen s + this)
const int64_t GROUP_TOP = 2;            // a group's score: the sum of its two largest corrected scores
const double NULL_KEY_SCORE = 0.0;      // the softmax's extra key: exp(0) = 1 joins the denominator

Json parse_rot(const Json &raw, const std::string &where, int64_t head_dim) {
  ConfigReader r(raw, where);
  Json rot = Json::object();
  const int64_t dims = r.integer("dims");
  if (dims % 2 || dims > head_dim) r.fail("'dims' must be even and at most the rotated head's size");
  rot.set("dims", dims);
  rot.set("base", r.number("base"));
  if (r.present("scaling")) {
    ConfigReader s(r.object("scaling"), where + ".scaling");
    Json sc = Json::object();
    sc.set("factor", s.number("factor"));
    sc.set("original", s.number("original"));
    sc.set("fast", s.number("fast"));
    sc.set("slow", s.number("slow"));
    rot.set("scaling", sc);
  } else {
    rot.set("scaling", Json());
  }
  return rot;
}

Json parse_mask(const ConfigReader &r, const std::string &where) {
  Json mask = Json::object();
  mask.set("size", r.present("mask") ? Json(ConfigReader(r.object("mask"), where + ".mask").integer("size")) : Json());
  return mask;
}

Json parse_mixer(const Json &layer, const std::string &where) {
  ConfigReader lr(layer, where);
  const std::string type = lr.string("type");
  ConfigReader r(lr.object("mixer"), where + ": mixer");
  Json m = Json::object();
  const int64_t heads = r.integer("heads"), dim = r.integer("dim");
  m.set("heads", heads);
  m.set("dim", dim);
  if (type == "attention") {
    const int64_t kv = r.integer_or("kv_heads", heads);
    if (heads % kv) r.fail("'heads' must be a multiple of 'kv_heads'");
    m.set("kv_heads", kv);
    m.set("vdim", r.integer_or("vdim", dim));
    m.set("scale", r.number_or("scale", 1.0 / std::sqrt((double)dim), false));
    m.set("rot", r.present("rot") ? parse_rot(r.object("rot"), where + ": mixer.rot", dim) : Json());
  } else if (type == "latent_attention") {
    const int64_t rot_dim = r.integer("rot_dim", 0);
    m.set("rot_dim", rot_dim);
    m.set("vdim", r.integer_or("vdim", dim));
    m.set("kv_rank", r.integer("kv_rank"));
    m.set("q_rank", r.integer("q_rank"));
    m.set("scale", r.number_or("scale", 1.0 / std::sqrt((double)(dim + rot_dim)), false));
    if (rot_dim > 0) {
      Json rot = parse_rot(r.object("rot"), where + ": mixer.rot", rot_dim);
      if (rot.get("dims").as_int() != rot_dim) r.fail("'rot.dims' must equal 'rot_dim'");
      m.set("rot", rot);
    } else {
      m.set("rot", Json());
    }
  } else {
    lr.fail("mixer type '" + type + "' is not known (attention, latent_attention)");
  }
  m.set("mask", parse_mask(r, where + ": mixer"));
  return m;
}

Json parse_mlp(const Json &raw, const std::string &where) {
  if (raw.is_null()) return Json();
  if (!raw.is_object()) LLM_THROW(Config, "%s: 'mlp' must be an object or null", where.c_str());
  ConfigReader r(raw, where + ": mlp");
  const std::string kind = r.string_or("kind", "moe");
  if (kind != "moe") r.fail("feed-forward kind '" + kind + "' is not known (moe)");
  Json m = Json::object();
  m.set("kind", kind);
  Json expert = Json::object();
  expert.set("ff", ConfigReader(r.object("expert"), where + ": mlp.expert").integer("ff"));
  m.set("expert", expert);
  ConfigReader ro(r.object("router"), where + ": mlp.router");
  Json router = Json::object();
  const int64_t experts = ro.integer("experts"), top = ro.integer("top");
  if (top > experts) ro.fail("'top' exceeds 'experts'");
  router.set("experts", experts);
  router.set("top", top);
  router.set("scale", ro.number_or("scale", 1.0, false));
  if (ro.present("groups")) {
    ConfigReader g(ro.object("groups"), where + ": mlp.router.groups");
    Json groups = Json::object();
    const int64_t count = g.integer("count"), keep = g.integer("keep");
    if (experts % count) g.fail("'count' must divide 'experts'");
    if (keep > count) g.fail("'keep' exceeds 'count'");
    if (keep * (experts / count) < top) g.fail("the kept groups hold fewer experts than 'top'");
    groups.set("count", count);
    groups.set("keep", keep);
    router.set("groups", groups);
  } else {
    router.set("groups", Json());
  }
  m.set("router", router);
  if (r.present("shared")) {
    Json shared = Json::object();
    shared.set("ff", ConfigReader(r.object("shared"), where + ": mlp.shared").integer("ff"));
    m.set("shared", shared);
  } else {
    m.set("shared", Json());
  }
  return m;
}

// config.json as read -> normal form: the same layout with every optional key present.
Json parse_tazizen(const Json &data) {
  const std::string where = "config.json";
  ConfigReader r(data, where);
  Json c = Json::object();
  c.set("architecture", "Tazizen");
  c.set("vocab", r.integer("vocab"));
  c.set("width", r.integer("width"));
  Json norm = Json::object();
  norm.set("eps", ConfigReader(r.object("norm"), where + ": norm").number("eps"));
  c.set("norm", norm);
  c.set("streams", r.present("streams") ? Json(r.integer("streams")) : Json());
  const Json &layers = data.get("layers");
  if (!layers.is_array() || layers.size() == 0) r.fail("'layers' must be a list with at least one layer");
  Json ls = Json::array();
  for (size_t i = 0; i < layers.size(); ++i) {
    const std::string lw = where + ": layers[" + std::to_string(i) + "]";
    const Json &l = layers.at(i);
    if (!l.is_object()) LLM_THROW(Config, "%s must be an object", lw.c_str());
    Json o = Json::object();
    o.set("type", ConfigReader(l, lw).string("type"));
    o.set("mixer", parse_mixer(l, lw));
    o.set("mlp", parse_mlp(l.get("mlp"), lw));
    ls.push(o);
  }
  c.set("layers", ls);
  const int64_t n = (int64_t)layers.size();
  Json loop = Json::object();
  if (r.present("loop")) {
    ConfigReader lp(r.object("loop"), where + ": loop");
    const int64_t start = lp.integer("start", 0), stop = lp.integer("stop", 0), times = lp.integer_or("times", 1, 0);
    if (start > stop || stop > n) lp.fail("'start' <= 'stop' <= the number of layers");
    loop.set("start", start);
    loop.set("stop", stop);
    loop.set("times", times);
  } else {
    loop.set("start", (int64_t)0);
    loop.set("stop", (int64_t)0);
    loop.set("times", (int64_t)1);
  }
  c.set("loop", loop);
  return c;
}

Json rope_description(const Json &rot, int64_t head_dim) {
  Json p = Json::object();
  p.set("kind", "rope");
  p.set("head_dim", head_dim);
  p.set("rotary_dim", rot.get("dims"));
  p.set("theta", rot.get("base"));
  p.set("pairing", "half");                         // channel i goes with channel i + dims/2
  const Json &sc = rot.get("scaling");
  if (sc.is_null()) {
    p.set("scaling", Json());
  } else {
    Json y = Json::object();
    y.set("rope_type", "yarn");
    y.set("factor", sc.get("factor"));
    y.set("original_max_position_embeddings", sc.get("original"));
    y.set("beta_fast", sc.get("fast"));
    y.set("beta_slow", sc.get("slow"));
    y.set("magnitude", 0.1 * std::log(sc.get("factor").as_number()) + 1.0);   // on cosines and sines alike
    p.set("scaling", y);
  }
  return p;
}

ModelSpec describe_tazizen(const Json &c) {
  const int64_t width = c.get("width").as_int();
  const double eps = c.get("norm").get("eps").as_number();
  auto norm = [&](const std::string &weight) {
    Json n = Json::object();
    n.set("kind", "rmsnorm");
    n.set("size", width);
    n.set("eps", eps);
    n.set("weight", weight);
    n.set("weight_offset", 1.0);                     // stored around nought, applied as 1 + w
    return n;
  };
  auto gated_unit = [&](const std::string &prefix, const Json &ff) {
    Json f = Json::object();
    f.set("kind", "swiglu");
    f.set("hidden", width);
    f.set("intermediate", ff);
    f.set("gate", prefix + "gate");
    f.set("up", prefix + "up");
    f.set("down", prefix + "down");
    return f;
  };
  ModelSpec s;
  s.name = "Tazizen";
  s.vocab_size = c.get("vocab").as_int();
  s.hidden = width;
  s.embedding = "embed";
  s.head = "head";
  s.max_positions = TAZIZEN_MAX_POSITIONS;
  const bool hyper = !c.get("streams").is_null();
  s.streams = hyper ? (int)c.get("streams").as_int() : 1;
  const Json &layers = c.get("layers");
  for (size_t i = 0; i < layers.size(); ++i) {
    const Json &l = layers.at(i);
    const Json &m = l.get("mixer");
    const std::string type = l.get("type").as_string();
    const std::string p = "l" + std::to_string(i) + ".", x = p + "mix.";
    const Json &window = m.get("mask").get("size");
    Json mixer = Json::object();
    if (type == "attention") {
      mixer.set("kind", "attention");
      mixer.set("hidden", width);
      mixer.set("n_heads", m.get("heads"));
      mixer.set("n_kv_heads", m.get("kv_heads"));
      mixer.set("head_dim", m.get("dim"));
      mixer.set("v_head_dim", m.get("vdim"));
      mixer.set("scale", m.get("scale"));
      mixer.set("position", m.get("rot").is_null() ? Json() : rope_description(m.get("rot"), m.get("dim").as_int()));
      Json hn = Json::object();
      hn.set("eps", eps);
      mixer.set("head_norm", hn);                    // after the rotation, per head, no weight
      mixer.set("null_key", NULL_KEY_SCORE);
      if (!window.is_null()) mixer.set("window", window);
      mixer.set("out_gate", x + "g");
      mixer.set("q", x + "q");
      mixer.set("k", x + "k");
      mixer.set("v", x + "v");
      mixer.set("o", x + "o");
    } else {
      mixer.set("kind", "latent_attention");
      mixer.set("hidden", width);
      mixer.set("n_heads", m.get("heads"));
      mixer.set("head_dim", m.get("dim"));
      mixer.set("rot_dim", m.get("rot_dim"));
      mixer.set("v_head_dim", m.get("vdim"));
      mixer.set("kv_rank", m.get("kv_rank"));
      mixer.set("q_rank", m.get("q_rank"));
      mixer.set("scale", m.get("scale"));
      mixer.set("eps", eps);
      if (!window.is_null()) mixer.set("window", window);
      mixer.set("position", m.get("rot").is_null() ? Json() : rope_description(m.get("rot"), m.get("rot_dim").as_int()));
      mixer.set("q_down", x + "dq");
      mixer.set("q_norm", x + "dq.norm");
      mixer.set("q_up", x + "uq");
      mixer.set("kv_down", x + "dkv");
      mixer.set("kv_norm", x + "dkv.norm");
      mixer.set("k_up", x + "uk");
      mixer.set("v_up", x + "uv");
      mixer.set("o", x + "o");
    }
    Json ff;
    const Json &f = l.get("mlp");
    if (!f.is_null()) {
      const Json &ro = f.get("router");
      ff = Json::object();
      ff.set("kind", "moe");
      ff.set("hidden", width);
      ff.set("experts", ro.get("experts"));
      ff.set("top", ro.get("top"));
      ff.set("score", "sigmoid");
      ff.set("renormalize", true);
      ff.set("norm_eps", ROUTE_NORM_EPS);
      ff.set("route_scale", ro.get("scale"));
      ff.set("weight_on", "output");
      ff.set("router", p + "mlp.router");
      ff.set("correction", p + "mlp.correction");
      if (!ro.get("groups").is_null()) {
        Json g = Json::object();
        g.set("count", ro.get("groups").get("count"));
        g.set("keep", ro.get("groups").get("keep"));
        g.set("top", GROUP_TOP);
        ff.set("groups", g);
      }
      Json e = Json::object();
      e.set("intermediate", f.get("expert").get("ff"));
      e.set("activation", "silu");
      e.set("gate", p + "mlp.e{}.gate");
      e.set("up", p + "mlp.e{}.up");
      e.set("down", p + "mlp.e{}.down");
      ff.set("expert", e);
      if (!f.get("shared").is_null()) {
        ff.set("shared", gated_unit(p + "mlp.shared.", f.get("shared").get("ff")));
        ff.set("shared_gate", p + "mlp.shared.sg");
      }
    }
    Json block = Json::object();
    block.set("kind", hyper ? "hyper" : "prenorm");
    block.set("hidden", width);
    block.set("mixer_norm", norm(p + "norm1"));
    block.set("mixer", mixer);
    block.set("ff_norm", ff.is_null() ? Json() : norm(p + "norm2"));
    block.set("ff", ff);
    if (hyper) {
      block.set("streams", (int64_t)s.streams);
      block.set("mixer_in", p + "hc1.in");
      block.set("mixer_out", p + "hc1.out");
      block.set("mixer_mix", p + "hc1.mix");
      if (!ff.is_null()) {
        block.set("ff_in", p + "hc2.in");
        block.set("ff_out", p + "hc2.out");
        block.set("ff_mix", p + "hc2.mix");
      }
    }
    s.layers.push_back(block);
  }
  // the order of runs: the layers before the loop, the looped ones `times` times, the rest
  const Json &loop = c.get("loop");
  const int64_t n = (int64_t)layers.size(), start = loop.get("start").as_int(), stop = loop.get("stop").as_int(),
                times = loop.get("times").as_int();
  for (int64_t i = 0; i < start; ++i) s.schedule.push_back({(int)i, -1, ""});
  for (int64_t t = 0; t < times; ++t)
    for (int64_t i = start; i < stop; ++i) s.schedule.push_back({(int)i, -1, ""});
  for (int64_t i = stop; i < n; ++i) s.schedule.push_back({(int)i, -1, ""});
  s.final_norm = norm("final.norm");
  return s;
}

}  // namespace

void register_architecture_unlocked(Architecture arch);   // config/config.cc

void register_tazizen_architecture() {
  Architecture a;
  a.name = "Tazizen";
  a.parse = parse_tazizen;
  a.describe = describe_tazizen;
  register_architecture_unlocked(std::move(a));
}

}  // namespace llm
