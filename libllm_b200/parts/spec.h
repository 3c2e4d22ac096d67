// The description of a model as data: which parts each layer is made of, with every size and
// constant as a field, the order in which layers run, and the names of their tensors.
//
// An architecture (libllm_b200/config/llama.cc) turns its configuration into one ModelSpec; the
// generic model (libllm_b200/engine/model.cc) builds the part that each description names through
// the part registry (libllm_b200/parts/part.h).  A part's description is a JSON object whose
// "kind" selects the class; the other keys are that class's own and are read, with checks, by
// its constructor.  A description knows nothing about the model it is used in.  The reference
// builds its one architecture in code (src/libllm/llama.cc:111-141, 231-249, 273-292); the keys
// here are the arguments of those build functions.
//
//   norm "rmsnorm":        size, eps, weight (tensor name)
//   norm "layernorm":      size, eps, weight, bias (tensor names; bias optional)
//   mixer "general_delta": hidden, n_heads, head_dim, eps, decay_rank, decay_scale, key_eps, tensor names (parts/recurrent.cc)
//   position "rope":       head_dim, rotary_dim, theta, scaling (null or the llama3 parameters)
//   mixer "attention":     hidden, n_heads, n_kv_heads, head_dim, v_head_dim (default head_dim),
//                          position (a position description or null), window (null: all keys),
//                          scale (null: 1/sqrt(head_dim)), bias, q, k, v, o (tensor names)
//   feed_forward "swiglu": hidden, intermediate, gate, up, down (tensor names)
//   mixer "attention" also: v_head_dim, qk_norm {q, k, eps}, block (mask), head_gate (parts/builtin.cc)
//   feed_forward "mlp":    hidden, intermediate, activation (gelu, gelu_tanh, silu), up, down
//   feed_forward "moe":    hidden, experts, top, score, renormalize, weight_on, router, expert {..}, shared
//   block "prenorm":       mixer_norm, mixer, ff_norm, ff (descriptions; ff and ff_norm may be null), mixer_conv {taps, weight, hidden}
//   block "parallel":      norm, mixer, ff (a description or null): x + mixer(norm x) + ff(norm x)
//   block "hyper":         the pre-norm block over several copies of the residual stream (parts/builtin.cc)
#pragma once
#include <string>
#include <vector>

#include "util/json.h"

namespace llm {

// One run of a layer.  `layer` indexes ModelSpec::layers; the same layer may be named by several
// entries (its weights are then used twice, each run with a cache of its own).  `cache_from`
// names an earlier entry whose cache this run reads instead of keeping one: it appends nothing.
// `input_mix` names a matrix [hidden, 2 * hidden]: right before this run the residual stream x
// becomes W [x; x0], x0 being the token rows as they entered the first layer (a model that runs some
// of its layers several times feeds the tokens to every pass this way).
struct ScheduleEntry {
  int layer = 0;
  int cache_from = -1;
  std::string input_mix;
};

struct ModelSpec {
  std::string name;
  int64_t vocab_size = 0;
  int64_t hidden = 0;
  std::string embedding;                  // tensor name of the token table
  std::string position_table;             // [max_positions, hidden]: a learned vector per position, added to the token's row; empty: none
  std::vector<Json> layers;               // block descriptions
  std::vector<ScheduleEntry> schedule;
  Json final_norm;
  std::string head;                       // output matrix; empty: the token table
  int64_t max_positions = 0;
  std::vector<int> stop_tokens;
  double embedding_scale = 1.0;           // token rows are multiplied by this before the first layer
  double logit_scale = 1.0;               // logits are multiplied by this ...
  double logit_softcap = 0.0;             // ... and, if positive, bounded: cap * tanh(logit / cap)
  // Copies of the residual stream the model carries (blocks of kind "hyper").  All start as the token's row; the last
  // norm reads their sum.
  int streams = 1;
  // Tensors that may lie in the files without any part asking for them ('*' matches any run of
  // characters).  Other unexpected tensors are reported as a warning, not an error.
  std::vector<std::string> ignore_tensors;

  Json to_json() const;
  static ModelSpec from_json(const Json &j);
};

}  // namespace llm
