// The Sobezen decoder: its configuration and its description as parts.
//
// config.json (`architecture`: "Sobezen") lists the layers one by one; every size and constant is
// read from it, and the ranks of the low-rank inputs of a channel_delta mixer from the stored
// tensors.  The stream starts as embedding.scale times the token's row ("embed").  Every layer is
// a pre-norm block with RMS norms ("l<i>.norm1", "l<i>.norm2") whose sublayers' results are
// multiplied, channel by channel, by a vector before they are added ("l<i>.ls1", "l<i>.ls2"):
//   x += ls1 * mixer(norm1 x), x += ls2 * ff(norm2 x).
// A layer names
//   type   "attention": grouped-query attention whose values are its keys as projected (before
//          the rotation; there is no value matrix), biases on q and k, a rotation of the first
//          rot.dims channels of each head in pairs (2i, 2i + 1), a score scale of its own;
//          "latent_attention": queries through a normed latent of q_rank channels, keys and
//          values through a normed latent of kv_rank channels plus one rotated key part of
//          rot_dim channels that all heads share; only those two are cached; YaRN scaling of the
//          rotation; with `kv_from` the layer reads another layer's cache and has no latent
//          projection of its own (parts/latent.cc);
//          "channel_delta": the gated delta rule with a decay per key channel, short causal
//          convolutions on q, k and v, and low-rank inputs for decay and gate (parts/recurrent.cc);
//   mlp    null, or {kind "dense", ff, limit}: down(g * sigmoid(1.702 g) * (u + 1)) with
//          g = min(gate h, limit), u = clamp(up h, -limit, limit), biases on all three matrices.
// Then the last RMS norm ("final.norm"), the output matrix ("head") and logits times logit_scale.
#include <cmath>

#include "config/config.h"

namespace llm {

namespace {

// What a model of this design can hold when the engine names no shorter bound: the configuration
// itself has no longest sequence.
const int64_t SOBEZEN_MAX_POSITIONS = 1 << 20;

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

Json parse_mixer(const Json &layer, const std::string &where, size_t index, const Json &all) {
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
    const int64_t vdim = r.integer_or("vdim", dim);
    if (vdim != dim) r.fail("the values are the keys: 'vdim' must equal 'dim'");
    m.set("vdim", vdim);
    m.set("scale", r.number("scale", false));
    m.set("rot", parse_rot(r.object("rot"), where + ": mixer.rot", dim));
  } else if (type == "latent_attention") {
    const int64_t rot_dim = r.integer("rot_dim");
    m.set("rot_dim", rot_dim);
    m.set("vdim", r.integer("vdim"));
    m.set("kv_rank", r.integer("kv_rank"));
    m.set("q_rank", r.integer("q_rank"));
    m.set("scale", r.number("scale", false));
    Json rot = parse_rot(r.object("rot"), where + ": mixer.rot", rot_dim);
    if (rot.get("dims").as_int() != rot_dim) r.fail("'rot.dims' must equal 'rot_dim'");
    m.set("rot", rot);
    if (r.present("kv_from")) {
      const int64_t from = r.integer("kv_from", 0);
      if (from >= (int64_t)index) r.fail("'kv_from' must name an earlier layer");
      const Json &src = all.at((size_t)from);
      ConfigReader sr(src, where + ": the layer 'kv_from' names");
      if (sr.string("type") != "latent_attention") r.fail("'kv_from' must name a latent_attention layer");
      ConfigReader sm(sr.object("mixer"), where + ": the mixer 'kv_from' names");
      if (sm.present("kv_from")) r.fail("'kv_from' must name a layer with a latent projection of its own");
      if (sm.integer("kv_rank") != m.get("kv_rank").as_int() || sm.integer("rot_dim") != rot_dim)
        r.fail("the layer 'kv_from' names has another 'kv_rank' or 'rot_dim'");
      m.set("kv_from", from);
    } else {
      m.set("kv_from", Json());
    }
  } else if (type == "channel_delta") {
    const int64_t kv = r.integer_or("kv_heads", heads);
    if (heads % kv) r.fail("'heads' must be a multiple of 'kv_heads'");
    m.set("kv_heads", kv);
    m.set("vdim", r.integer_or("vdim", dim));
    m.set("conv", r.integer("conv"));
  } else {
    lr.fail("mixer type '" + type + "' is not known (attention, latent_attention, channel_delta)");
  }
  return m;
}

Json parse_mlp(const Json &raw, const std::string &where) {
  if (raw.is_null()) return Json();
  if (!raw.is_object()) LLM_THROW(Config, "%s: 'mlp' must be an object or null", where.c_str());
  ConfigReader r(raw, where + ": mlp");
  const std::string kind = r.string("kind");
  if (kind != "dense") r.fail("feed-forward kind '" + kind + "' is not known (dense)");
  Json m = Json::object();
  m.set("kind", kind);
  m.set("ff", r.integer("ff"));
  m.set("limit", r.number("limit"));
  return m;
}

// config.json as read -> normal form: the same layout with every optional key present.
Json parse_sobezen(const Json &data) {
  const std::string where = "config.json";
  ConfigReader r(data, where);
  Json c = Json::object();
  c.set("architecture", "Sobezen");
  c.set("vocab", r.integer("vocab"));
  c.set("width", r.integer("width"));
  Json norm = Json::object();
  norm.set("eps", ConfigReader(r.object("norm"), where + ": norm").number("eps"));
  c.set("norm", norm);
  Json emb = Json::object();
  emb.set("scale", r.present("embedding") ? ConfigReader(r.object("embedding"), where + ": embedding").number_or("scale", 1.0, false) : 1.0);
  c.set("embedding", emb);
  c.set("logit_scale", r.number_or("logit_scale", 1.0, false));
  const Json &layers = data.get("layers");
  if (!layers.is_array() || layers.size() == 0) r.fail("'layers' must be a list with at least one layer");
  Json ls = Json::array();
  for (size_t i = 0; i < layers.size(); ++i) {
    const std::string lw = where + ": layers[" + std::to_string(i) + "]";
    const Json &l = layers.at(i);
    if (!l.is_object()) LLM_THROW(Config, "%s must be an object", lw.c_str());
    Json o = Json::object();
    o.set("type", ConfigReader(l, lw).string("type"));
    o.set("mixer", parse_mixer(l, lw, i, layers));
    o.set("mlp", parse_mlp(l.get("mlp"), lw));
    ls.push(o);
  }
  c.set("layers", ls);
  return c;
}

Json rope_description(const Json &rot, int64_t head_dim) {
  Json p = Json::object();
  p.set("kind", "rope");
  p.set("head_dim", head_dim);
  p.set("rotary_dim", rot.get("dims"));
  p.set("theta", rot.get("base"));
  p.set("pairing", "interleaved");                  // channel 2i goes with channel 2i + 1
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

ModelSpec describe_sobezen(const Json &c) {
  const int64_t width = c.get("width").as_int();
  const double eps = c.get("norm").get("eps").as_number();
  auto norm = [&](const std::string &weight) {
    Json n = Json::object();
    n.set("kind", "rmsnorm");
    n.set("size", width);
    n.set("eps", eps);
    n.set("weight", weight);
    return n;
  };
  ModelSpec s;
  s.name = "Sobezen";
  s.vocab_size = c.get("vocab").as_int();
  s.hidden = width;
  s.embedding = "embed";
  s.head = "head";
  s.max_positions = SOBEZEN_MAX_POSITIONS;
  s.embedding_scale = c.get("embedding").get("scale").as_number();
  s.logit_scale = c.get("logit_scale").as_number();
  const Json &layers = c.get("layers");
  for (size_t i = 0; i < layers.size(); ++i) {
    const Json &l = layers.at(i);
    const Json &m = l.get("mixer");
    const std::string type = l.get("type").as_string();
    const std::string p = "l" + std::to_string(i) + ".", x = p + "mix.";
    Json mixer = Json::object();
    int cache_from = -1;
    if (type == "attention") {
      mixer.set("kind", "attention");
      mixer.set("hidden", width);
      mixer.set("n_heads", m.get("heads"));
      mixer.set("n_kv_heads", m.get("kv_heads"));
      mixer.set("head_dim", m.get("dim"));
      mixer.set("scale", m.get("scale"));
      mixer.set("position", rope_description(m.get("rot"), m.get("dim").as_int()));
      mixer.set("values", "keys");                   // v = k as projected, before the rotation
      mixer.set("bias", true);
      mixer.set("q_bias", x + "q.b");
      mixer.set("k_bias", x + "k.b");
      mixer.set("q", x + "q");
      mixer.set("k", x + "k");
      mixer.set("o", x + "o");
    } else if (type == "latent_attention") {
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
      mixer.set("position", rope_description(m.get("rot"), m.get("rot_dim").as_int()));
      mixer.set("q_down", x + "dq");
      mixer.set("q_norm", x + "dq.norm");
      mixer.set("q_up", x + "uq");
      if (m.get("kv_from").is_null()) {
        mixer.set("kv_down", x + "dkv");
        mixer.set("kv_norm", x + "dkv.norm");
      } else {
        cache_from = (int)m.get("kv_from").as_int();  // layers run once each, in order: entry j is layer j
      }
      mixer.set("k_up", x + "uk");
      mixer.set("v_up", x + "uv");
      mixer.set("o", x + "o");
    } else {
      mixer.set("kind", "channel_delta");
      mixer.set("hidden", width);
      mixer.set("n_heads", m.get("heads"));
      mixer.set("n_kv_heads", m.get("kv_heads"));
      mixer.set("head_dim", m.get("dim"));
      mixer.set("v_head_dim", m.get("vdim"));
      mixer.set("taps", m.get("conv"));
      mixer.set("eps", eps);
      mixer.set("key_eps", 1e-6);                    // the design's constant: unit vectors x / sqrt(sum x^2 + 1e-6)
      for (const char *t : {"q", "k", "v", "b", "A_log", "norm", "a1", "a2", "dt_bias", "g1", "g2", "o"}) mixer.set(t, x + t);
      mixer.set("q_conv", x + "q.conv");
      mixer.set("k_conv", x + "k.conv");
      mixer.set("v_conv", x + "v.conv");
    }
    Json ff;
    const Json &f = l.get("mlp");
    if (!f.is_null()) {
      ff = Json::object();
      ff.set("kind", "clamped_glu");
      ff.set("hidden", width);
      ff.set("intermediate", f.get("ff"));
      ff.set("limit", f.get("limit"));
      ff.set("slope", 1.702);                        // the design's constants: g * sigmoid(1.702 g) * (u + 1)
      ff.set("up_shift", 1.0);
      ff.set("gate", p + "mlp.gate");
      ff.set("up", p + "mlp.up");
      ff.set("down", p + "mlp.down");
      ff.set("gate_bias", p + "mlp.gate.b");
      ff.set("up_bias", p + "mlp.up.b");
      ff.set("down_bias", p + "mlp.down.b");
    }
    Json block = Json::object();
    block.set("kind", "prenorm");
    block.set("mixer_norm", norm(p + "norm1"));
    block.set("mixer", mixer);
    block.set("mixer_scale", p + "ls1");
    block.set("ff_norm", ff.is_null() ? Json() : norm(p + "norm2"));
    block.set("ff", ff);
    if (!ff.is_null()) block.set("ff_scale", p + "ls2");
    block.set("hidden", width);
    s.layers.push_back(block);
    s.schedule.push_back({(int)i, cache_from, ""});
  }
  s.final_norm = norm("final.norm");
  return s;
}

}  // namespace

void register_architecture_unlocked(Architecture arch);   // config/config.cc

void register_sobezen_architecture() {
  Architecture a;
  a.name = "Sobezen";
  a.parse = parse_sobezen;
  a.describe = describe_sobezen;
  register_architecture_unlocked(std::move(a));
}

}  // namespace llm
