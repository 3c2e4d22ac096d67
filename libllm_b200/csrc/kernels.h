// The host library's view of the kernel libraries: one C++ function per exported kernel.
//
// Each family of kernels (libllm_b200/csrc/*.cu) is a shared library of its own, built by
// libllm_b200/csrc/build.py for sm_100a when something first needs it.  The host library opens a
// family when one of its functions is first called and turns a non-zero status into an llm::Error
// that carries the family's own message.  There is no fallback: a family that is not built, or
// that cannot be loaded, is an error that says so.
#pragma once
#include <cuda_runtime.h>

#include <string>
#include <vector>

#include "util/device.h"

namespace llm {
namespace kernels {

// Where a family's library lies.  Set by whoever built them (the Python package after
// csrc/build.py ran); otherwise the file `kernels.manifest` (lines "family path") in the folder
// named by LIBLLM_B200_KERNEL_DIR, or else in the folder of this library itself, is read.
void set_library(const std::string &family, const std::string &path);
bool available(const std::string &family);
void *symbol(const std::string &family, const std::string &name);
std::vector<std::string> loaded_libraries();

// ---- elementwise
void embedding(DType table_dtype, const void *table, const int *tokens, const int *fed_tokens, const int *fed_rows,
               float *out, int n_tokens, int hidden, int vocab, cudaStream_t s, const void *pos_table = nullptr, int pos_rows = 0,
               const int *tok_pos = nullptr);   // pos_table [pos_rows, hidden] in the table's type: a learned vector per position, added
void copy_words(const int *src, int *dst, int n, cudaStream_t s);
void gather_words(const int *src1, int n1, const int *src2, int n2, int *dst, cudaStream_t s);
void add_rmsnorm(float *resid, const Act *delta, const float *weight, float eps, void *out, DType out_dtype,
                 const int *rows, int n_rows, int hidden, cudaStream_t s);
// Several residual streams [n_streams][rows][hidden] (in_stride / out_stride floats apart; in_stride 0: all equal to x_in):
// applies the pending result `delta` (x_t <- sum_s mix[s, t] x_s + outw[t] y), then u = sum_s inw[s] x_s (inw null: the plain
// sum) and out = rmsnorm(u) * norm_w, or u itself in 32-bit when norm_w is null.  With `rows`, x_out and out hold those rows only.
void hyper_mix_norm(const float *x_in, long long in_stride, float *x_out, long long out_stride, int n_streams, const Act *delta,
                    const float *mix, const float *outw, const float *inw, const float *norm_w, float eps, void *out, DType out_dtype,
                    const int *rows, int n_rows, int hidden, cudaStream_t s);
void add_scalar(float *x, long long n, float value, cudaStream_t s);
// The same pass with a layer norm: (v - mean) / sqrt(var + eps) * weight + bias (bias may be null).
void add_layernorm(float *resid, const Act *delta, const float *weight, const float *bias, float eps, void *out, DType out_dtype,
                   const int *rows, int n_rows, int hidden, cudaStream_t s);
// A step of single tokens: the layer norm of every row, then out = h + conv(h) over time with the taps - 1 rows of
// state[seq_slot[row]] (in out's type), which move on by one.
void add_layernorm_conv(float *resid, const Act *delta, const float *weight, const float *bias, float eps, void *out, DType out_dtype,
                        int n_rows, int hidden, const float *conv_w, void *state, const int *seq_slot, int taps, cudaStream_t s);
// out[i] = resid[rows[i]] + delta's parts at that row (32-bit)
void gather_rows_add(const float *resid, const Act *delta, const int *rows, int n_rows, float *out, int hidden, cudaStream_t s);
void swiglu(const Act &gu, void *out, DType out_dtype, cudaStream_t s);
// gu [T, 2 I] (gate | up), bias [2 I] or null; out [T, I] = g * sigmoid(slope g) * (u + up_shift), g and u bounded by limit
void clamped_glu(const Act &gu, const float *bias, const Act &out, float limit, float slope, float up_shift, cudaStream_t s);
// out[t] = [resid[t] + delta's parts at t | other[t]] in out's type, [rows, 2 * hidden]
void concat_stream(const float *resid, const Act *delta, const float *other, const Act &out, int hidden, cudaStream_t s);
void scale_rows(float *x, long long n, float scale, cudaStream_t s);
void logit_transform(float *logits, long long n, float scale, float softcap, cudaStream_t s);
void random_fill(void *out, DType dtype, long long n, unsigned long long seed, int law, float a, float b, cudaStream_t s);
// ---- products
void gemm_plain(const Act &x, const Weight &w, const float *bias, const Act &out, cudaStream_t s);
bool gemm_tc_supported(const Act &x, const Weight &w);
int gemm_tc_suggest_parts(int M, int N, int K);
void gemm_tc(const Act &x, const Weight &w, const Act &out, bool swiglu, int *status, cudaStream_t s);
void gemm_tc_wait_probe(long long limit_ns, int *status, cudaStream_t s);
// One job of a chain of products and norms run as one launch (csrc/gemm_chain.cu, which has the
// same structure under the name llm_chain_job).
struct ChainJob {
  int kind;                 // 0 product, 1 SwiGLU product, 2 add + RMSNorm
  int dep0, dep1;           // jobs of the chain that must be complete first; -1: none
  const void *x;
  long long ldx;
  const void *w;
  void *out;
  long long ldo;
  int M, N, K, k_parts;
  long long part_stride;
  float *resid;
  const float *delta;
  int delta_parts;
  long long delta_stride;
  const float *weight;
  float eps;
  const int *rows;
  int n_rows, hidden;
};
int gemm_chain_max_jobs();
int gemm_chain_max_tokens();
int gemm_chain_max_hidden();
int gemm_chain_counters();
void gemm_chain(const ChainJob *jobs, int n_jobs, int *counters, int *status, cudaStream_t s);
bool gemv_supported(const Act &x, const Weight &w);
int gemv_suggest_parts(int M, int N, int K);
void gemv_bf16(const Act &x, const Weight &w, const Act &out, bool swiglu, cudaStream_t s);
// ---- rotation and cache append
void rope_cache_write(const Act &qkv, const Act &q_out, int n_heads, int n_kv, int d, const float *table, int table_rows,
                      int rot_dim, const int *tok_seq, const int *tok_pos, const int *page_table, int pt_stride,
                      void *kcache, void *vcache, int page_size, bool write_cache, cudaStream_t s);
// The same for rows [q | k | v (n_kv * dv) | ...] with an RMS norm over all of q and all of k before the
// rotation (weights of n_heads * d and n_kv * d values; null: none) and values of width dv.
void qk_place(const Act &qkv, const Act &q_out, int n_heads, int n_kv, int d, int dv, const float *q_norm, const float *k_norm,
              float eps, const float *table, int table_rows, int rot_dim, const int *tok_seq, const int *tok_pos,
              const int *page_table, int pt_stride, void *kcache, void *vcache, int page_size, bool write_cache, cudaStream_t s);
// Rows [q | k | v (n_kv * dv) | ...]: rotation of the first rot_dim channels of each q and k head (pairs i, i + rot_dim/2), THEN
// every q and k head divided by its root mean square over d (sqrt(mean + eps), no weight; eps < 0: no norm), q -> q_out,
// k and v appended to the cache.
void rope_headnorm_place(const Act &qkv, const Act &q_out, int n_heads, int n_kv, int d, int dv, float eps, const float *table,
                         int table_rows, int rot_dim, const int *tok_seq, const int *tok_pos, const int *page_table, int pt_stride,
                         void *kcache, void *vcache, int page_size, bool write_cache, cudaStream_t s);
// Rows [q | k | v | ...] without a rotation: adds `bias` (one 32-bit value per stacked row; null: none), divides each
// value head by its root mean square when v_eps >= 0, writes q and appends k, v to the cache.
// rows [q | k | v] (no v part with values_from_keys: the value cache gets the key as projected); bias over the row's columns
// or null; rotation of the first rot_dim channels of each q and k head in pairs (2i, 2i + 1), table [positions, rot_dim]
void rope_pairs_place(const Act &qkv, const Act &q_out, int n_heads, int n_kv, int d, int dv, const float *bias, bool values_from_keys,
                      const float *table, int table_rows, int rot_dim, const int *tok_seq, const int *tok_pos, const int *page_table,
                      int pt_stride, void *kcache, void *vcache, int page_size, bool write_cache, cudaStream_t s);
void kv_place(const Act &qkv, const Act &q_out, int n_heads, int n_kv, int d, int dv, const float *bias, float v_eps,
              const int *tok_seq, const int *tok_pos, const int *page_table, int pt_stride, void *kcache, void *vcache,
              int page_size, bool write_cache, cudaStream_t s);
// ---- attention
constexpr float NO_NULL_KEY = -__builtin_huge_valf();
// Masks: `window` > 0, a query sees the last `window` keys; `block` > 0, only keys of its own block
// of `block` positions counted from 0; `sink` > 0 (with a window): the first `sink` positions stay visible.  `gate` (32-bit, one value per token and head, row stride
// gate_stride; null: none): the head's result is multiplied by sigmoid(gate).
void attention_generic(const Act &q, const Act &out, const void *kc, const void *vc, const int *tok_seq, const int *tok_pos,
                       const int *page_table, int pt_stride, int n_heads, int n_kv, int d, int dv, int page_size, int window,
                       int block, float scale, const float *gate, long long gate_stride, cudaStream_t s, int sink = 0, int v_ld = 0,
                       float null_score = NO_NULL_KEY);
// v_ld > 0: value rows lie v_ld channels apart (the values are the first dv channels of the key rows when vc is kc).
// null_score: every query also sees one key of that score that has no value (exp(null_score) joins the softmax's
// denominator); NO_NULL_KEY: none.
// ---- latent attention (csrc/latent.cu): attention over one cached row [c | k_r] per position that every head reads
// proj rows (32-bit) hold the query latent at off_q and, with off_kv >= 0, the key/value latent and the shared key part;
// cq_out = rms(query latent) * q_weight; the token's cache row = [rms(first kv_rank) * kv_weight | rotated last rot].
void latent_place(const Act &proj, int off_q, int q_rank, const float *q_weight, const Act &cq_out, int off_kv, int kv_rank, int rot,
                  const float *kv_weight, float eps, const float *table, int table_rows, bool interleaved, const int *tok_seq,
                  const int *tok_pos, const int *page_table, int pt_stride, void *cache, int page_size, cudaStream_t s);
// q [T, heads * (d + rot)] 32-bit -> out [T, heads * (kv_rank + rot)]: [w_uk_h^T q_h[:d] | rotated q_h[d:]]
void latent_absorb(const Act &q, const void *w_uk, const Act &out, int n_heads, int d, int rot, int kv_rank, const float *table,
                   int table_rows, bool interleaved, const int *tok_pos, cudaStream_t s);
// x [T, heads * kv_rank] -> out [T, heads * dv]: out_h = w_uv_h x_h
void latent_expand(const Act &x, const void *w_uv, const Act &out, int n_heads, int kv_rank, int dv, cudaStream_t s);
// ---- latent attention on the tensor cores (csrc/latent_tc.cu), bfloat16
// The cached rows of the step's tokens, whoever appended them: c_out [T, kv_rank], kr_out [T, row - kv_rank].
void latent_rows(const void *cache, int page_size, int row, int kv_rank, const int *tok_seq, const int *tok_pos, const int *page_table,
                 int pt_stride, int n_tokens, const Act &c_out, const Act &kr_out, cudaStream_t s);
// q [T, heads * (d + rot)] 32-bit -> out, the same layout in bfloat16 with each head's last rot channels rotated
void latent_rotate_q(const Act &q, const Act &out, int n_heads, int d, int rot, const float *table, int table_rows, bool interleaved,
                     const int *tok_pos, cudaStream_t s);
bool latent_prefill_supported(int d, int rot, int dv);
// Sequences that start at their first token, heads materialised: kv [T, heads * d | heads * dv], kr [T, rot] rotated.
void latent_prefill(const Act &q, const Act &kv, const Act &kr, const Act &out, const int *seq_start, int n_seqs, int max_q_len,
                    int n_heads, int d, int rot, int dv, float scale, cudaStream_t s, int window = 0);
bool latent_decode_supported(int kv_rank, int rot);
size_t latent_decode_floats(int n_tokens, int n_heads, int kv_rank, int n_splits);
// qa [T, heads * (kv_rank + rot)] (latent_absorb) over the cached rows -> out [T, heads * kv_rank]; ws: latent_decode_floats
void latent_decode(const Act &qa, const void *cache, int page_size, const int *tok_seq, const int *tok_pos, const int *page_table,
                   int pt_stride, int n_heads, int kv_rank, int rot, int n_splits, float scale, const Act &out, float *ws, cudaStream_t s,
                   int window = 0);
bool attention_decode_supported(int d, int group);
void attention_decode(const Act &q, const Act &out, const void *kc, const void *vc, const int *tok_pos, const int *page_table,
                      int pt_stride, int n_heads, int n_kv, int d, int page_size, int chunk, int n_splits, int window,
                      int block, float scale, float *ws_o, float *ws_ml, const float *gate, long long gate_stride,
                      cudaStream_t s, int sink = 0, bool gate_per_channel = false, float null_score = NO_NULL_KEY);
bool attention_decode_tc_supported(int d, int page_size, int group);
int attention_decode_tc_ctas_per_sm(int d);
void attention_decode_tc(const Act &qkv, const float *table, int table_rows, int rot_dim, const int *tok_pos,
                         const int *page_table, int pt_stride, void *kc, void *vc, bool write_cache, int n_seqs, int n_heads,
                         int n_kv, int d, int page_size, int chunk, int max_len, int n_splits, int window, int block,
                         float scale, float *ws_o, float *ws_ml, int *counters, const Act &out, cudaStream_t s);
bool attention_prefill_supported(int d, int page_size);
void attention_prefill(const Act &q, const Act &out, const void *kc, const void *vc, const int *seq_start, const int *seq_past,
                       const int *page_table, int pt_stride, int n_seqs, int max_q_len, int n_heads, int n_kv, int d,
                       int page_size, int window, int block, float scale, cudaStream_t s, int sink = 0, float null_score = NO_NULL_KEY);
bool attention_prefill_tc_supported(int d, int page_size);
void attention_prefill_tc(const Act &q, const Act &out, const void *kc, const void *vc, long long n_pages, const int *seq_start,
                          const int *seq_past, const int *page_table, int pt_stride, int n_seqs, int max_q_len, int n_heads,
                          int n_kv, int d, int page_size, int window, int block, float scale, int *status, cudaStream_t s,
                          int sink = 0, float null_score = NO_NULL_KEY);
// out[t, h, :] *= sigmoid(gate[t * gate_stride + h]) for heads of width dv
void head_gate(const Act &out, const float *gate, long long gate_stride, int n_heads, int dv, cudaStream_t s);
// ---- routed feed-forward (csrc/moe.cu)
enum Activation { GeluErf = 0, GeluTanh = 1, Silu = 2, Relu2 = 3 };
void activation(const Act &in, const Act &out, int act, cudaStream_t s);
// logits [T, E] 32-bit -> chosen [T * top], weight [T * top]; score 0 sigmoid, 1 softmax
void moe_route(const Act &logits, int n_experts, int top, int score, bool renormalize, int *chosen, float *weight, cudaStream_t s);
// The choice on s + correction (null: none) among the experts of the `keep` best of n_groups groups (a group's score: the sum of
// its group_top largest corrected scores); weights s, with `renormalize` s / (sum + norm_eps), times route_scale.
void moe_route_grouped(const Act &logits, int n_experts, int top, int score, const float *correction, int n_groups, int keep,
                       int group_top, bool renormalize, float norm_eps, float route_scale, int *chosen, float *weight, cudaStream_t s);
// out[p, t, :] = x[p, t, :] * sigmoid(gate[t * gate_stride]) for n_parts parts, 32-bit rows
void row_gate(const float *x, long long x_stride, float *out, long long out_stride, int n_parts, const float *gate,
              long long gate_stride, int n_rows, int cols, cudaStream_t s);
int moe_tile_rows();
void moe_sort(const int *chosen, int n_rows, int n_experts, int tile_rows, int *offsets, int *perm, int *tiles, cudaStream_t s);
// x [T, width]; up [E, ff, width], down [E, width, ff] in x's type; out [top, T, width] 32-bit.  `gated`: up is
// [E, 2 ff, width], an expert's gate and up rows interleaved, and the expert is down(act(gate x) * up x).
void moe_rows(const Act &x, const void *up, const void *down, const int *chosen, const float *weight, int top, int width, int ff,
              int act, bool weight_on_output, float *out, cudaStream_t s, bool gated = false);
bool moe_grouped_supported(int width, int ff);
void moe_grouped(const Act &x, const void *up, const void *down, const int *offsets, const int *perm, const int *tiles,
                 const float *weight, int n_experts, int top, int width, int ff, int act, bool weight_on_output, void *mid,
                 float *out, cudaStream_t s, bool gated = false);
// The same on tcgen05 (csrc/moe_tc.cu): the table of tiles must have moe_tc_tile_rows(rows) rows to a tile;
// xs [T * top, width] receives the tokens' rows in sorted order.
bool moe_tc_supported(int width, int ff);
int moe_tc_tile_rows(int n_rows);
void moe_tc(const Act &x, const void *up, const void *down, const int *offsets, const int *perm, const int *tiles,
            const float *weight, int n_experts, int top, int width, int ff, int act, bool weight_on_output, void *xs, void *mid,
            float *out, int *status, cudaStream_t s, bool gated = false);
// ---- state carried from token to token (csrc/recurrent.cu)
// out = h + conv(h) over time per channel, weight [width, taps] 32-bit; state [slots, taps - 1, width] in h's type.
// With silu_alone: out = silu(conv(h)), the short convolution of a projection.
void causal_conv(const Act &h, const Act &out, const float *weight, void *state, const int *tok_seq, const int *tok_pos,
                 const int *seq_start, const int *seq_past, const int *seq_slot, int n_seqs, int taps, bool single_tokens,
                 cudaStream_t s, bool silu_alone = false);
// The delta rule's recurrence alone: rows (32-bit) hold r, k (heads x d) and v (heads x dv) at their offsets, prep
// [tokens, heads, 3, d] the decay w, the removal b and the direction u; state [slots, heads, dv, d]; out [tokens, heads * dv].
void delta_scan(const Act &rows, int off_r, int off_k, int off_v, const float *prep, float *state, const Act &out, const int *seq_start,
                const int *seq_slot, int n_seqs, int n_heads, int d, int dv, cudaStream_t s);
// The gated delta rule's vectors from the convolved projections (csrc/recurrent.cu says which).
void channel_delta_prepare(const Act &cv, const Act &proj, int off_b, int off_a1, int rank_a, int off_g1, int rank_g, const float *a2,
                           const float *dt_bias, const float *a_log, const float *g2, float key_eps, float *prep, float *gate,
                           int n_heads, int n_kv, int d, int dv, cudaStream_t s);
// The generalized delta rule over the 32-bit rows `proj` (offsets of r, k, v, the removal logits and the low-rank decay
// input within a row); prep: scratch [tokens, heads, 3, d] floats; state [slots, heads, d, d] floats; out [tokens, heads * d].
void delta_rule(const Act &proj, int off_r, int off_k, int off_v, int off_a, int off_x1, int rank, const float *w2, const float *w0,
                const float *a_bias, float decay_scale, float key_eps, float *prep, float *state, const Act &out,
                const int *seq_start, const int *seq_slot, int n_seqs, int n_heads, int d, cudaStream_t s);
// A step of single tokens (row b = sequence b): the same, with the norm over each head, its weight and the gate
// (logits at off_g of the rows) behind it, in one launch; out [sequences, heads * d] in the engine's type.
bool delta_step_supported(int d);
void delta_step(const Act &proj, int off_r, int off_k, int off_v, int off_g, int off_a, int off_x1, int rank, const float *w2,
                const float *w0, const float *a_bias, float decay_scale, float key_eps, const float *norm_w, float eps, float *state,
                const Act &out, const int *seq_slot, int n_heads, int d, cudaStream_t s);
// out[t, h, :] = x / rms(x over the head; eps < 0: no norm) * weight (null: none) * sigmoid(gate) (null: none)
void head_norm_gate(const Act &x, const float *weight, const float *gate, long long gate_stride, float eps, int n_heads, int dv,
                    const Act &out, cudaStream_t s);
// ---- sampling
void argmax(const float *logits, long long stride, int n_rows, int vocab, int *out, cudaStream_t s);
void sample(const float *logits, long long stride, int n_rows, int vocab, float temperature, int top_k, float top_p,
            const float *uniforms, int *out, cudaStream_t s);

// Kernel launches issued through this file since the process started (graph replays not counted).
long long launches();

}  // namespace kernels
}  // namespace llm
