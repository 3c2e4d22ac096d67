#include "csrc/kernels.h"

#include <dirent.h>
#include <dlfcn.h>

#include <atomic>
#include <cstdlib>
#include <fstream>
#include <map>
#include <mutex>
#include <sstream>

namespace llm {
namespace kernels {

namespace {
struct Family {
  std::string path;
  void *handle = nullptr;
  const char *(*last_error)() = nullptr;
};
std::map<std::string, Family> &families() {
  static std::map<std::string, Family> f;
  return f;
}
std::mutex &lock() {
  static std::mutex m;
  return m;
}
std::atomic<long long> g_launches{0};
bool g_manifest_read = false;

std::string own_folder() {
  Dl_info info;
  if (dladdr((void *)&own_folder, &info) && info.dli_fname) {
    std::string p = info.dli_fname;
    const size_t slash = p.rfind('/');
    return slash == std::string::npos ? "." : p.substr(0, slash);
  }
  return ".";
}

void read_manifest_locked() {
  if (g_manifest_read) return;
  g_manifest_read = true;
  const char *env = getenv("LIBLLM_B200_KERNEL_DIR");
  const std::string dir = env && *env ? env : own_folder();
  std::ifstream f(dir + "/kernels.manifest");
  std::string line;
  while (std::getline(f, line)) {
    std::istringstream ls(line);
    std::string fam, path;
    if (!(ls >> fam)) continue;
    std::getline(ls, path);
    const size_t b = path.find_first_not_of(" \t");
    if (b == std::string::npos) continue;
    path = path.substr(b);
    if (path[0] != '/') path = dir + "/" + path;
    if (!families().count(fam)) families()[fam].path = path;
  }
}

Family &open_family(const std::string &name) {
  std::lock_guard<std::mutex> g(lock());
  read_manifest_locked();
  auto it = families().find(name);
  if (it == families().end() || it->second.path.empty())
    LLM_THROW(Extension, "the kernel library '%s' is not built (run `python -m libllm_b200.csrc.build %s`); there is no fallback",
              name.c_str(), name.c_str());
  Family &f = it->second;
  if (!f.handle) {
    f.handle = dlopen(f.path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!f.handle) LLM_THROW(Extension, "cannot load %s: %s", f.path.c_str(), dlerror());
    f.last_error = (const char *(*)())dlsym(f.handle, ("llm_" + name + "_last_error").c_str());
  }
  return f;
}

[[noreturn]] void fail(const std::string &family, const char *fn, int status) {
  Family &f = open_family(family);
  const std::string msg = f.last_error ? f.last_error() : "";
  if (status == STATUS_INVALID_ARG) throw Error(ErrorKind::Unsupported, msg);
  LLM_THROW(Extension, "%s failed (status %#x): %s", fn, status, msg.c_str());
}

template <typename Fn>
Fn resolve(const char *family, const char *name) {
  return (Fn)symbol(family, name);
}

#define LLM_KERNEL(family, name, ...)                                           \
  using name##_fn_t = int (*)(__VA_ARGS__);                                     \
  static name##_fn_t name##_fn() {                                              \
    static name##_fn_t f = resolve<name##_fn_t>(family, #name);                 \
    return f;                                                                   \
  }
#define LLM_CALL(family, name, ...)                                             \
  do {                                                                          \
    g_launches.fetch_add(1, std::memory_order_relaxed);                         \
    const int st_ = name##_fn()(__VA_ARGS__);                                   \
    if (st_ != 0) fail(family, #name, st_);                                     \
  } while (0)

inline int code(DType t) { return (int)t; }
}  // namespace

void set_library(const std::string &family, const std::string &path) {
  std::lock_guard<std::mutex> g(lock());
  Family &f = families()[family];
  if (f.handle && f.path != path)
    LLM_THROW(Extension, "the kernel library '%s' is loaded from %s already", family.c_str(), f.path.c_str());
  f.path = path;
}

bool available(const std::string &family) {
  std::lock_guard<std::mutex> g(lock());
  read_manifest_locked();
  auto it = families().find(family);
  return it != families().end() && !it->second.path.empty();
}

void *symbol(const std::string &family, const std::string &name) {
  Family &f = open_family(family);
  void *p = dlsym(f.handle, name.c_str());
  if (!p) LLM_THROW(Extension, "%s does not export %s (a stale build?)", f.path.c_str(), name.c_str());
  return p;
}

std::vector<std::string> loaded_libraries() {
  std::lock_guard<std::mutex> g(lock());
  std::vector<std::string> out;
  for (const auto &kv : families())
    if (kv.second.handle) out.push_back(kv.second.path);
  return out;
}

long long launches() { return g_launches.load(); }

// ---------------------------------------------------------------- elementwise
LLM_KERNEL("elementwise", llm_embedding_pos, int, const void *, const int *, const int *, const int *, float *, int, int, int,
           const void *, int, const int *, cudaStream_t)
LLM_KERNEL("elementwise", llm_add_layernorm, float *, const void *, int, int, long long, const float *, const float *, float, void *,
           int, const int *, int, int, cudaStream_t)
LLM_KERNEL("elementwise", llm_copy_words, const int *, int *, int, cudaStream_t)
LLM_KERNEL("elementwise", llm_gather_words, const int *, int, const int *, int, int *, cudaStream_t)
LLM_KERNEL("elementwise", llm_add_rmsnorm_scaled, float *, const void *, int, int, long long, const float *, float, void *, int,
           const int *, int, int, const float *, const float *, cudaStream_t)
LLM_KERNEL("elementwise", llm_gather_rows_add_scaled, const float *, const void *, int, int, long long, const int *, int, float *, int,
           const float *, const float *, cudaStream_t)
LLM_KERNEL("elementwise", llm_clamped_glu, int, int, const void *, long long, const float *, void *, int, int, float, float, float,
           cudaStream_t)
LLM_KERNEL("elementwise", llm_swiglu, int, int, const void *, void *, int, int, cudaStream_t)
LLM_KERNEL("elementwise", llm_scale_rows, float *, long long, float, cudaStream_t)
LLM_KERNEL("elementwise", llm_logit_transform, float *, long long, float, float, cudaStream_t)
LLM_KERNEL("elementwise", llm_random_fill, void *, int, long long, unsigned long long, int, float, float, cudaStream_t)

void embedding(DType dt, const void *table, const int *tokens, const int *fed_tokens, const int *fed_rows, float *out,
               int n, int hidden, int vocab, cudaStream_t s, const void *pos_table, int pos_rows, const int *tok_pos) {
  LLM_CALL("elementwise", llm_embedding_pos, code(dt), table, tokens, fed_rows ? fed_tokens : nullptr, fed_rows, out, n, hidden, vocab,
           pos_table, pos_rows, tok_pos, s);
}
void add_layernorm(float *resid, const Act *delta, const float *weight, const float *bias, float eps, void *out, DType out_dtype,
                   const int *rows, int n_rows, int hidden, cudaStream_t s) {
  if (delta && (delta->col_scale || delta->col_bias))
    LLM_THROW(Unsupported, "add_layernorm: a pending addition with a scale or a bias over its columns is taken by the RMS norm's pass only");
  const bool has = delta && delta->data;
  LLM_CALL("elementwise", llm_add_layernorm, resid, has ? delta->data : nullptr, has ? code(delta->dtype) : 0,
           has ? delta->parts : 0, has ? (long long)delta->part_stride : 0, weight, bias, eps, out, code(out_dtype), rows, n_rows,
           hidden, s);
}
void copy_words(const int *src, int *dst, int n, cudaStream_t s) { LLM_CALL("elementwise", llm_copy_words, src, dst, n, s); }
void gather_words(const int *src1, int n1, const int *src2, int n2, int *dst, cudaStream_t s) {
  LLM_CALL("elementwise", llm_gather_words, src1, n1, src2, n2, dst, s);
}
LLM_KERNEL("elementwise", llm_hyper_mix_norm, const float *, long long, float *, long long, int, const float *, int, long long,
           const float *, const float *, const float *, const float *, const float *, const float *, float, void *, int, const int *, int,
           int, cudaStream_t)
LLM_KERNEL("elementwise", llm_add_scalar, float *, long long, float, cudaStream_t)
void hyper_mix_norm(const float *x_in, long long in_stride, float *x_out, long long out_stride, int n_streams, const Act *delta,
                    const float *mix, const float *outw, const float *inw, const float *norm_w, float eps, void *out, DType out_dtype,
                    const int *rows, int n_rows, int hidden, cudaStream_t s) {
  const bool has = delta && delta->data;
  if (has && delta->dtype != DType::F32) LLM_THROW(InvalidArg, "hyper_mix_norm: a pending result is 32-bit");
  LLM_CALL("elementwise", llm_hyper_mix_norm, x_in, in_stride, x_out, out_stride, n_streams, has ? (const float *)delta->data : nullptr,
           has ? delta->parts : 0, has ? (long long)delta->part_stride : 0, has ? delta->col_scale : nullptr,
           has ? delta->col_bias : nullptr, mix, outw, inw, norm_w, eps, out, code(out_dtype), rows, n_rows, hidden, s);
}
void add_scalar(float *x, long long n, float value, cudaStream_t s) { LLM_CALL("elementwise", llm_add_scalar, x, n, value, s); }
void add_rmsnorm(float *resid, const Act *delta, const float *weight, float eps, void *out, DType out_dtype, const int *rows,
                 int n_rows, int hidden, cudaStream_t s) {
  const bool has = delta && delta->data;
  LLM_CALL("elementwise", llm_add_rmsnorm_scaled, resid, has ? delta->data : nullptr, has ? code(delta->dtype) : 0,
           has ? delta->parts : 0, has ? (long long)delta->part_stride : 0, weight, eps, out, code(out_dtype), rows, n_rows,
           hidden, has ? delta->col_scale : nullptr, has ? delta->col_bias : nullptr, s);
}
LLM_KERNEL("elementwise", llm_add_layernorm_conv, float *, const void *, int, int, long long, const float *, const float *, float, void *,
           int, int, int, const float *, void *, const int *, int, cudaStream_t)
void add_layernorm_conv(float *resid, const Act *delta, const float *weight, const float *bias, float eps, void *out, DType out_dtype,
                        int n_rows, int hidden, const float *conv_w, void *state, const int *seq_slot, int taps, cudaStream_t s) {
  if (delta && (delta->col_scale || delta->col_bias))
    LLM_THROW(Unsupported, "add_layernorm_conv: a pending addition with a scale or a bias over its columns is taken by the RMS norm's pass only");
  const bool has = delta && delta->data;
  LLM_CALL("elementwise", llm_add_layernorm_conv, resid, has ? delta->data : nullptr, has ? code(delta->dtype) : 0,
           has ? delta->parts : 0, has ? (long long)delta->part_stride : 0, weight, bias, eps, out, code(out_dtype), n_rows, hidden,
           conv_w, state, seq_slot, taps, s);
}
void gather_rows_add(const float *resid, const Act *delta, const int *rows, int n_rows, float *out, int hidden, cudaStream_t s) {
  const bool has = delta && delta->data;
  LLM_CALL("elementwise", llm_gather_rows_add_scaled, resid, has ? delta->data : nullptr, has ? code(delta->dtype) : 0,
           has ? delta->parts : 0, has ? (long long)delta->part_stride : 0, rows, n_rows, out, hidden, has ? delta->col_scale : nullptr,
           has ? delta->col_bias : nullptr, s);
}
void clamped_glu(const Act &gu, const float *bias, const Act &out, float limit, float slope, float up_shift, cudaStream_t s) {
  LLM_CALL("elementwise", llm_clamped_glu, code(gu.dtype), code(out.dtype), gu.data, (long long)gu.ld, bias, out.data, (int)gu.rows,
           (int)out.cols, limit, slope, up_shift, s);
}
LLM_KERNEL("elementwise", llm_concat_stream, const float *, const float *, int, long long, const float *, void *, int, int, int,
           cudaStream_t)
void concat_stream(const float *resid, const Act *delta, const float *other, const Act &out, int hidden, cudaStream_t s) {
  if (delta && (delta->col_scale || delta->col_bias))
    LLM_THROW(Unsupported, "concat_stream: a pending addition with a scale or a bias over its columns is taken by the RMS norm's pass only");
  const bool has = delta && delta->data;
  if (has && delta->dtype != DType::F32) LLM_THROW(InvalidArg, "concat_stream: a pending addition is 32-bit");
  LLM_CALL("elementwise", llm_concat_stream, resid, has ? (const float *)delta->data : nullptr, has ? delta->parts : 0,
           has ? (long long)delta->part_stride : 0, other, out.data, code(out.dtype), (int)out.rows, hidden, s);
}
void swiglu(const Act &gu, void *out, DType out_dtype, cudaStream_t s) {
  LLM_CALL("elementwise", llm_swiglu, code(gu.dtype), code(out_dtype), gu.data, out, (int)gu.rows, (int)(gu.cols / 2), s);
}
void scale_rows(float *x, long long n, float scale, cudaStream_t s) { LLM_CALL("elementwise", llm_scale_rows, x, n, scale, s); }
void logit_transform(float *logits, long long n, float scale, float softcap, cudaStream_t s) {
  LLM_CALL("elementwise", llm_logit_transform, logits, n, scale, softcap, s);
}
void random_fill(void *out, DType dtype, long long n, unsigned long long seed, int law, float a, float b, cudaStream_t s) {
  LLM_CALL("elementwise", llm_random_fill, out, code(dtype), n, seed, law, a, b, s);
}

// ---------------------------------------------------------------- products
LLM_KERNEL("gemm_plain", llm_gemm_plain, int, int, const void *, long long, const void *, long long, const float *, void *,
           long long, int, int, int, cudaStream_t)
LLM_KERNEL("gemm_tc", llm_gemm_tc, const void *, long long, const void *, void *, long long, int, int, int, int, int, int,
           long long, int *, cudaStream_t)
LLM_KERNEL("gemv", llm_gemv_bf16, const void *, long long, const void *, void *, long long, int, int, int, int, int, int,
           long long, cudaStream_t)

void gemm_plain(const Act &x, const Weight &w, const float *bias, const Act &out, cudaStream_t s) {
  LLM_CALL("gemm_plain", llm_gemm_plain, code(x.dtype), code(out.dtype), x.data, (long long)x.ld, w.data(), (long long)w.cols,
           bias, out.data, (long long)out.ld, (int)x.rows, (int)w.rows, (int)x.cols, s);
}
bool gemm_tc_supported(const Act &x, const Weight &w) {
  return x.dtype == DType::BF16 && w.dtype == DType::BF16 && x.rows > 0 && x.cols % 8 == 0 && (x.rows == 1 || x.ld % 8 == 0) &&
         (uintptr_t)x.data % 16 == 0 && (uintptr_t)w.data() % 16 == 0;
}
int gemm_tc_suggest_parts(int M, int N, int K) {
  static auto f = resolve<int (*)(int, int, int)>("gemm_tc", "llm_gemm_tc_suggest_parts");
  return f(M, N, K);
}
void gemm_tc(const Act &x, const Weight &w, const Act &out, bool swiglu, int *status, cudaStream_t s) {
  LLM_CALL("gemm_tc", llm_gemm_tc, x.data, (long long)(x.rows > 1 ? x.ld : x.cols), w.data(), out.data,
           (long long)(x.rows > 1 ? out.ld : out.cols), code(out.dtype), (int)x.rows, (int)w.rows, (int)x.cols, swiglu ? 1 : 0,
           out.parts, (long long)out.part_stride, status, s);
}
LLM_KERNEL("gemm_tc", llm_gemm_tc_wait_probe, long long, int *, cudaStream_t)
void gemm_tc_wait_probe(long long limit_ns, int *status, cudaStream_t s) { LLM_CALL("gemm_tc", llm_gemm_tc_wait_probe, limit_ns, status, s); }
LLM_KERNEL("gemm_chain", llm_gemm_chain, const ChainJob *, int, int *, int *, cudaStream_t)
static int chain_limit(const char *name) {
  return resolve<int (*)()>("gemm_chain", name)();
}
int gemm_chain_max_jobs() {
  static const int v = chain_limit("llm_gemm_chain_max_jobs");
  return v;
}
int gemm_chain_max_tokens() {
  static const int v = chain_limit("llm_gemm_chain_max_tokens");
  return v;
}
int gemm_chain_max_hidden() {
  static const int v = chain_limit("llm_gemm_chain_max_hidden");
  return v;
}
int gemm_chain_counters() {
  static const int v = chain_limit("llm_gemm_chain_counters");
  return v;
}
void gemm_chain(const ChainJob *jobs, int n_jobs, int *counters, int *status, cudaStream_t s) {
  LLM_CALL("gemm_chain", llm_gemm_chain, jobs, n_jobs, counters, status, s);
}
bool gemv_supported(const Act &x, const Weight &w) {
  return x.dtype == DType::BF16 && w.dtype == DType::BF16 && x.rows > 0 && x.rows <= 64 && x.cols % 8 == 0 && x.ld % 8 == 0 &&
         (uintptr_t)x.data % 16 == 0 && (uintptr_t)w.data() % 16 == 0;
}
int gemv_suggest_parts(int M, int N, int K) {
  static auto f = resolve<int (*)(int, int, int)>("gemv", "llm_gemv_suggest_parts");
  return f(M, N, K);
}
void gemv_bf16(const Act &x, const Weight &w, const Act &out, bool swiglu, cudaStream_t s) {
  LLM_CALL("gemv", llm_gemv_bf16, x.data, (long long)(x.rows > 1 ? x.ld : x.cols), w.data(), out.data,
           (long long)(x.rows > 1 ? out.ld : out.cols), code(out.dtype), (int)x.rows, (int)w.rows, (int)x.cols, swiglu ? 1 : 0,
           out.parts, (long long)out.part_stride, s);
}

// ---------------------------------------------------------------- rotation and cache append
LLM_KERNEL("rope", llm_rope_cache_write, int, int, const void *, long long, void *, long long, int, int, int, int, const float *,
           int, int, const int *, const int *, const int *, int, void *, void *, int, int, cudaStream_t)

void rope_cache_write(const Act &qkv, const Act &q_out, int n_heads, int n_kv, int d, const float *table, int table_rows,
                      int rot_dim, const int *tok_seq, const int *tok_pos, const int *page_table, int pt_stride, void *kcache,
                      void *vcache, int page_size, bool write_cache, cudaStream_t s) {
  LLM_CALL("rope", llm_rope_cache_write, code(qkv.dtype), code(q_out.dtype), qkv.data, (long long)qkv.ld, q_out.data,
           (long long)q_out.ld, (int)qkv.rows, n_heads, n_kv, d, table, table_rows, rot_dim, tok_seq, tok_pos, page_table,
           pt_stride, kcache, vcache, page_size, write_cache ? 1 : 0, s);
}

LLM_KERNEL("rope", llm_rope_headnorm_place, int, int, const void *, long long, void *, long long, int, int, int, int, int, float,
           const float *, int, int, const int *, const int *, const int *, int, void *, void *, int, int, cudaStream_t)
void rope_headnorm_place(const Act &qkv, const Act &q_out, int n_heads, int n_kv, int d, int dv, float eps, const float *table,
                         int table_rows, int rot_dim, const int *tok_seq, const int *tok_pos, const int *page_table, int pt_stride,
                         void *kcache, void *vcache, int page_size, bool write_cache, cudaStream_t s) {
  LLM_CALL("rope", llm_rope_headnorm_place, code(qkv.dtype), code(q_out.dtype), qkv.data, (long long)qkv.ld, q_out.data,
           (long long)q_out.ld, (int)qkv.rows, n_heads, n_kv, d, dv, eps, table, table_rows, rot_dim, tok_seq, tok_pos, page_table,
           pt_stride, kcache, vcache, page_size, write_cache ? 1 : 0, s);
}
LLM_KERNEL("rope", llm_qk_place, int, int, const void *, long long, void *, long long, int, int, int, int, int, const float *,
           const float *, float, const float *, int, int, const int *, const int *, const int *, int, void *, void *, int, int,
           cudaStream_t)
void qk_place(const Act &qkv, const Act &q_out, int n_heads, int n_kv, int d, int dv, const float *q_norm, const float *k_norm,
              float eps, const float *table, int table_rows, int rot_dim, const int *tok_seq, const int *tok_pos,
              const int *page_table, int pt_stride, void *kcache, void *vcache, int page_size, bool write_cache, cudaStream_t s) {
  LLM_CALL("rope", llm_qk_place, code(qkv.dtype), code(q_out.dtype), qkv.data, (long long)qkv.ld, q_out.data, (long long)q_out.ld,
           (int)qkv.rows, n_heads, n_kv, d, dv, q_norm, k_norm, eps, table, table_rows, rot_dim, tok_seq, tok_pos, page_table,
           pt_stride, kcache, vcache, page_size, write_cache ? 1 : 0, s);
}

LLM_KERNEL("rope", llm_kv_place, int, int, const void *, long long, void *, long long, int, int, int, int, int, const float *, float,
           const int *, const int *, const int *, int, void *, void *, int, int, cudaStream_t)
void kv_place(const Act &qkv, const Act &q_out, int n_heads, int n_kv, int d, int dv, const float *bias, float v_eps,
              const int *tok_seq, const int *tok_pos, const int *page_table, int pt_stride, void *kcache, void *vcache,
              int page_size, bool write_cache, cudaStream_t s) {
  LLM_CALL("rope", llm_kv_place, code(qkv.dtype), code(q_out.dtype), qkv.data, (long long)qkv.ld, q_out.data, (long long)q_out.ld,
           (int)qkv.rows, n_heads, n_kv, d, dv, bias, v_eps, tok_seq, tok_pos, page_table, pt_stride, kcache, vcache, page_size,
           write_cache ? 1 : 0, s);
}

LLM_KERNEL("rope", llm_rope_pairs_place, int, int, const void *, long long, void *, long long, int, int, int, int, int, const float *, int,
           const float *, int, int, const int *, const int *, const int *, int, void *, void *, int, int, cudaStream_t)
void rope_pairs_place(const Act &qkv, const Act &q_out, int n_heads, int n_kv, int d, int dv, const float *bias, bool values_from_keys,
                      const float *table, int table_rows, int rot_dim, const int *tok_seq, const int *tok_pos, const int *page_table,
                      int pt_stride, void *kcache, void *vcache, int page_size, bool write_cache, cudaStream_t s) {
  LLM_CALL("rope", llm_rope_pairs_place, code(qkv.dtype), code(q_out.dtype), qkv.data, (long long)qkv.ld, q_out.data, (long long)q_out.ld,
           (int)qkv.rows, n_heads, n_kv, d, dv, bias, values_from_keys ? 1 : 0, table, table_rows, rot_dim, tok_seq, tok_pos, page_table,
           pt_stride, kcache, vcache, page_size, write_cache ? 1 : 0, s);
}

// ---------------------------------------------------------------- attention
LLM_KERNEL("attention_generic", llm_attention_generic_ld, int, const void *, long long, void *, long long, const void *, const void *,
           const int *, const int *, const int *, int, int, int, int, int, int, int, int, int, int, int, float, const float *, long long,
           float, cudaStream_t)
LLM_KERNEL("attention_decode", llm_attention_decode_null, const void *, long long, void *, long long, const void *, const void *,
           const int *, const int *, int, int, int, int, int, int, int, int, int, int, int, float, float *, float *, const float *,
           long long, int, float, cudaStream_t)
LLM_KERNEL("attention_decode_tc", llm_attention_decode_tc, const float *, long long, int, long long, const float *, int, int,
           const int *, const int *, int, void *, void *, int, int, int, int, int, int, int, int, int, int, int, float, float *,
           float *, int *, void *, long long, cudaStream_t)
LLM_KERNEL("attention_prefill", llm_attention_prefill_null, const void *, long long, void *, long long, const void *, const void *,
           const int *, const int *, const int *, int, int, int, int, int, int, int, int, int, int, float, float, cudaStream_t)
LLM_KERNEL("elementwise", llm_head_gate, void *, int, long long, const float *, long long, int, int, int, cudaStream_t)
void head_gate(const Act &out, const float *gate, long long gate_stride, int n_heads, int dv, cudaStream_t s) {
  LLM_CALL("elementwise", llm_head_gate, out.data, code(out.dtype), (long long)out.ld, gate, gate_stride, (int)out.rows, n_heads, dv, s);
}
LLM_KERNEL("attention_prefill_tc", llm_attention_prefill_tc_null, const void *, long long, long long, void *, long long, const void *,
           const void *, long long, const int *, const int *, const int *, int, int, int, int, int, int, int, int, int, int, float, float,
           int, int *, cudaStream_t)

void attention_generic(const Act &q, const Act &out, const void *kc, const void *vc, const int *tok_seq, const int *tok_pos,
                       const int *page_table, int pt_stride, int n_heads, int n_kv, int d, int dv, int page_size, int window,
                       int block, float scale, const float *gate, long long gate_stride, cudaStream_t s, int sink, int v_ld,
                       float null_score) {
  LLM_CALL("attention_generic", llm_attention_generic_ld, code(q.dtype), q.data, (long long)q.ld, out.data, (long long)out.ld, kc, vc,
           tok_seq, tok_pos, page_table, pt_stride, (int)q.rows, n_heads, n_kv, d, dv, v_ld > 0 ? v_ld : dv, page_size, window, block,
           sink, scale, gate, gate_stride, null_score, s);
}

// ---------------------------------------------------------------- latent attention
LLM_KERNEL("latent", llm_latent_place, int, const float *, long long, int, int, int, const float *, void *, long long, int, int, int,
           const float *, float, const float *, int, int, const int *, const int *, const int *, int, void *, int, cudaStream_t)
LLM_KERNEL("latent", llm_latent_absorb, int, const float *, long long, const void *, void *, long long, int, int, int, int, int,
           const float *, int, int, const int *, cudaStream_t)
LLM_KERNEL("latent", llm_latent_expand, int, const void *, long long, const void *, void *, long long, int, int, int, int, cudaStream_t)
void latent_place(const Act &proj, int off_q, int q_rank, const float *q_weight, const Act &cq_out, int off_kv, int kv_rank, int rot,
                  const float *kv_weight, float eps, const float *table, int table_rows, bool interleaved, const int *tok_seq,
                  const int *tok_pos, const int *page_table, int pt_stride, void *cache, int page_size, cudaStream_t s) {
  if (proj.dtype != DType::F32) LLM_THROW(InvalidArg, "latent_place: the latents' projections are 32-bit");
  LLM_CALL("latent", llm_latent_place, code(cq_out.dtype), (const float *)proj.data, (long long)proj.ld, (int)proj.rows, off_q, q_rank,
           q_weight, cq_out.data, (long long)cq_out.ld, off_kv, kv_rank, rot, kv_weight, eps, table, table_rows, interleaved ? 1 : 0,
           tok_seq, tok_pos, page_table, pt_stride, cache, page_size, s);
}
void latent_absorb(const Act &q, const void *w_uk, const Act &out, int n_heads, int d, int rot, int kv_rank, const float *table,
                   int table_rows, bool interleaved, const int *tok_pos, cudaStream_t s) {
  if (q.dtype != DType::F32) LLM_THROW(InvalidArg, "latent_absorb: the queries are 32-bit");
  LLM_CALL("latent", llm_latent_absorb, code(out.dtype), (const float *)q.data, (long long)q.ld, w_uk, out.data, (long long)out.ld,
           (int)q.rows, n_heads, d, rot, kv_rank, table, table_rows, interleaved ? 1 : 0, tok_pos, s);
}
void latent_expand(const Act &x, const void *w_uv, const Act &out, int n_heads, int kv_rank, int dv, cudaStream_t s) {
  if (x.dtype != out.dtype) LLM_THROW(InvalidArg, "latent_expand: input and output have one type");
  LLM_CALL("latent", llm_latent_expand, code(x.dtype), x.data, (long long)x.ld, w_uv, out.data, (long long)out.ld, (int)x.rows, n_heads,
           kv_rank, dv, s);
}
LLM_KERNEL("latent_tc", llm_latent_rows, const void *, int, int, int, const int *, const int *, const int *, int, int, void *, void *,
           cudaStream_t)
LLM_KERNEL("latent_tc", llm_latent_rotate_q, const float *, long long, void *, long long, int, int, int, int, const float *, int, int,
           const int *, cudaStream_t)
LLM_KERNEL("latent_tc", llm_latent_prefill, const void *, long long, const void *, long long, const void *, void *, long long, const int *,
           int, int, int, int, int, int, float, int, cudaStream_t)
LLM_KERNEL("latent_tc", llm_latent_decode, const void *, long long, const void *, int, const int *, const int *, const int *, int, int,
           int, int, int, int, float, void *, long long, float *, int, cudaStream_t)
void latent_rows(const void *cache, int page_size, int row, int kv_rank, const int *tok_seq, const int *tok_pos, const int *page_table,
                 int pt_stride, int n_tokens, const Act &c_out, const Act &kr_out, cudaStream_t s) {
  if (c_out.dtype != DType::BF16 || c_out.ld != kv_rank || (row > kv_rank && (kr_out.dtype != DType::BF16 || kr_out.ld != row - kv_rank)))
    LLM_THROW(InvalidArg, "latent_rows: dense bfloat16 results");
  LLM_CALL("latent_tc", llm_latent_rows, cache, page_size, row, kv_rank, tok_seq, tok_pos, page_table, pt_stride, n_tokens, c_out.data,
           kr_out.data, s);
}
void latent_rotate_q(const Act &q, const Act &out, int n_heads, int d, int rot, const float *table, int table_rows, bool interleaved,
                     const int *tok_pos, cudaStream_t s) {
  if (q.dtype != DType::F32 || out.dtype != DType::BF16) LLM_THROW(InvalidArg, "latent_rotate_q: 32-bit queries, a bfloat16 result");
  LLM_CALL("latent_tc", llm_latent_rotate_q, (const float *)q.data, (long long)q.ld, out.data, (long long)out.ld, (int)q.rows, n_heads, d,
           rot, table, table_rows, interleaved ? 1 : 0, tok_pos, s);
}
bool latent_prefill_supported(int d, int rot, int dv) {
  static auto f = resolve<int (*)(int, int, int)>("latent_tc", "llm_latent_prefill_supports");
  return f(d, rot, dv) != 0;
}
void latent_prefill(const Act &q, const Act &kv, const Act &kr, const Act &out, const int *seq_start, int n_seqs, int max_q_len,
                    int n_heads, int d, int rot, int dv, float scale, cudaStream_t s, int window) {
  if (q.dtype != DType::BF16 || kv.dtype != DType::BF16 || out.dtype != DType::BF16 || (rot > 0 && (kr.dtype != DType::BF16 || kr.ld != rot)))
    LLM_THROW(InvalidArg, "latent_prefill: bfloat16 operands");
  LLM_CALL("latent_tc", llm_latent_prefill, q.data, (long long)q.ld, kv.data, (long long)kv.ld, kr.data, out.data, (long long)out.ld,
           seq_start, n_seqs, max_q_len, n_heads, d, rot, dv, scale, window, s);
}
bool latent_decode_supported(int kv_rank, int rot) {
  static auto f = resolve<int (*)(int, int)>("latent_tc", "llm_latent_decode_supports");
  return f(kv_rank, rot) != 0;
}
size_t latent_decode_floats(int n_tokens, int n_heads, int kv_rank, int n_splits) {
  return n_splits <= 1 ? 0 : (size_t)n_tokens * n_heads * n_splits * ((size_t)kv_rank + 2);
}
void latent_decode(const Act &qa, const void *cache, int page_size, const int *tok_seq, const int *tok_pos, const int *page_table,
                   int pt_stride, int n_heads, int kv_rank, int rot, int n_splits, float scale, const Act &out, float *ws, cudaStream_t s,
                   int window) {
  if (qa.dtype != DType::BF16 || out.dtype != DType::BF16) LLM_THROW(InvalidArg, "latent_decode: bfloat16 operands");
  LLM_CALL("latent_tc", llm_latent_decode, qa.data, (long long)qa.ld, cache, page_size, tok_seq, tok_pos, page_table, pt_stride,
           (int)qa.rows, n_heads, kv_rank, rot, n_splits, scale, out.data, (long long)out.ld, ws, window, s);
}
bool attention_decode_supported(int d, int group) {
  static auto f = resolve<int (*)(int, int)>("attention_decode", "llm_attention_decode_supports");
  return f(d, group) != 0;
}
void attention_decode(const Act &q, const Act &out, const void *kc, const void *vc, const int *tok_pos, const int *page_table,
                      int pt_stride, int n_heads, int n_kv, int d, int page_size, int chunk, int n_splits, int window,
                      int block, float scale, float *ws_o, float *ws_ml, const float *gate, long long gate_stride,
                      cudaStream_t s, int sink, bool gate_per_channel, float null_score) {
  const int B = (int)q.rows;
  LLM_CALL("attention_decode", llm_attention_decode_null, q.data, (long long)(B > 1 ? q.ld : q.cols), out.data,
           (long long)(B > 1 ? out.ld : out.cols), kc, vc, tok_pos, page_table, pt_stride, B, n_heads, n_kv, d, page_size, chunk,
           n_splits, window, block, sink, scale, ws_o, ws_ml, gate, gate_stride, gate_per_channel ? 1 : 0, null_score, s);
}
bool attention_decode_tc_supported(int d, int page_size, int group) {
  static auto f = resolve<int (*)(int, int, int)>("attention_decode_tc", "llm_attention_decode_tc_supports");
  return f(d, page_size, group) != 0;
}
int attention_decode_tc_ctas_per_sm(int d) {
  static auto f = resolve<int (*)(int)>("attention_decode_tc", "llm_attention_decode_tc_ctas_per_sm");
  return f(d);
}
void attention_decode_tc(const Act &qkv, const float *table, int table_rows, int rot_dim, const int *tok_pos,
                         const int *page_table, int pt_stride, void *kc, void *vc, bool write_cache, int n_seqs, int n_heads,
                         int n_kv, int d, int page_size, int chunk, int max_len, int n_splits, int window, int block,
                         float scale, float *ws_o, float *ws_ml, int *counters, const Act &out, cudaStream_t s) {
  LLM_CALL("attention_decode_tc", llm_attention_decode_tc, (const float *)qkv.data, (long long)(n_seqs > 1 ? qkv.ld : qkv.cols),
           qkv.parts, (long long)qkv.part_stride, table, table_rows, rot_dim, tok_pos, page_table, pt_stride, kc, vc,
           write_cache ? 1 : 0, n_seqs, n_heads, n_kv, d, page_size, chunk, max_len, n_splits, window, block, scale, ws_o, ws_ml,
           counters, out.data, (long long)(n_seqs > 1 ? out.ld : out.cols), s);
}
bool attention_prefill_supported(int d, int page_size) {
  static auto f = resolve<int (*)(int, int)>("attention_prefill", "llm_attention_prefill_supports");
  return f(d, page_size) != 0;
}
void attention_prefill(const Act &q, const Act &out, const void *kc, const void *vc, const int *seq_start, const int *seq_past,
                       const int *page_table, int pt_stride, int n_seqs, int max_q_len, int n_heads, int n_kv, int d,
                       int page_size, int window, int block, float scale, cudaStream_t s, int sink, float null_score) {
  LLM_CALL("attention_prefill", llm_attention_prefill_null, q.data, (long long)q.ld, out.data, (long long)out.ld, kc, vc, seq_start,
           seq_past, page_table, pt_stride, n_seqs, max_q_len, n_heads, n_kv, d, page_size, window, block, sink, scale, null_score, s);
}
bool attention_prefill_tc_supported(int d, int page_size) {
  static auto f = resolve<int (*)(int, int)>("attention_prefill_tc", "llm_attention_prefill_tc_supports");
  return f(d, page_size) != 0;
}
void attention_prefill_tc(const Act &q, const Act &out, const void *kc, const void *vc, long long n_pages, const int *seq_start,
                          const int *seq_past, const int *page_table, int pt_stride, int n_seqs, int max_q_len, int n_heads,
                          int n_kv, int d, int page_size, int window, int block, float scale, int *status, cudaStream_t s,
                          int sink, float null_score) {
  LLM_CALL("attention_prefill_tc", llm_attention_prefill_tc_null, q.data, (long long)q.ld, (long long)q.rows, out.data,
           (long long)out.ld, kc, vc, n_pages, seq_start, seq_past, page_table, pt_stride, n_seqs, max_q_len, n_heads, n_kv, d,
           page_size, window, block, sink, scale, null_score, 0, status, s);
}

// ---------------------------------------------------------------- routed feed-forward
LLM_KERNEL("moe", llm_activation, int, int, const void *, void *, long long, int, cudaStream_t)
LLM_KERNEL("moe", llm_moe_route, const float *, long long, int, int, int, int, int, int *, float *, cudaStream_t)
LLM_KERNEL("moe", llm_moe_route_grouped, const float *, long long, int, int, int, int, const float *, int, int, int, int, float, float,
           int *, float *, cudaStream_t)
LLM_KERNEL("moe", llm_row_gate, const float *, long long, float *, long long, int, const float *, long long, int, int, cudaStream_t)
void moe_route_grouped(const Act &logits, int n_experts, int top, int score, const float *correction, int n_groups, int keep,
                       int group_top, bool renormalize, float norm_eps, float route_scale, int *chosen, float *weight, cudaStream_t s) {
  LLM_CALL("moe", llm_moe_route_grouped, (const float *)logits.data, (long long)logits.ld, (int)logits.rows, n_experts, top, score,
           correction, n_groups, keep, group_top, renormalize ? 1 : 0, norm_eps, route_scale, chosen, weight, s);
}
void row_gate(const float *x, long long x_stride, float *out, long long out_stride, int n_parts, const float *gate,
              long long gate_stride, int n_rows, int cols, cudaStream_t s) {
  LLM_CALL("moe", llm_row_gate, x, x_stride, out, out_stride, n_parts, gate, gate_stride, n_rows, cols, s);
}
LLM_KERNEL("moe", llm_moe_sort, const int *, int, int, int, int *, int *, int *, cudaStream_t)
LLM_KERNEL("moe", llm_moe_rows, int, const void *, long long, const void *, const void *, const int *, const float *, int, int, int,
           int, int, int, int, float *, cudaStream_t)
LLM_KERNEL("moe", llm_moe_grouped, const void *, long long, const void *, const void *, const int *, const int *, const int *,
           const float *, int, int, int, int, int, int, int, int, void *, float *, cudaStream_t)
void activation(const Act &in, const Act &out, int act, cudaStream_t s) {
  if (in.ld != in.cols || out.ld != out.cols) LLM_THROW(InvalidArg, "activation: rows must be dense");
  LLM_CALL("moe", llm_activation, code(in.dtype), code(out.dtype), in.data, out.data, (long long)(in.rows * in.cols), act, s);
}
void moe_route(const Act &logits, int n_experts, int top, int score, bool renormalize, int *chosen, float *weight, cudaStream_t s) {
  LLM_CALL("moe", llm_moe_route, (const float *)logits.data, (long long)logits.ld, (int)logits.rows, n_experts, top, score,
           renormalize ? 1 : 0, chosen, weight, s);
}
int moe_tile_rows() {
  static auto f = resolve<int (*)()>("moe", "llm_moe_tile_rows");
  return f();
}
void moe_sort(const int *chosen, int n_rows, int n_experts, int tile_rows, int *offsets, int *perm, int *tiles, cudaStream_t s) {
  LLM_CALL("moe", llm_moe_sort, chosen, n_rows, n_experts, tile_rows, offsets, perm, tiles, s);
}
LLM_KERNEL("moe", llm_moe_gather, const void *, long long, const int *, int, int, int, void *, cudaStream_t)
LLM_KERNEL("moe_tc", llm_moe_tc, const void *, const void *, const void *, const int *, const int *, const int *, const float *, int,
           int, int, int, int, int, int, int, void *, float *, int *, cudaStream_t)
bool moe_tc_supported(int width, int ff) {
  static auto f = resolve<int (*)(int, int)>("moe_tc", "llm_moe_tc_supports");
  return f(width, ff) != 0;
}
int moe_tc_tile_rows(int n_rows) {
  static auto f = resolve<int (*)(int)>("moe_tc", "llm_moe_tc_tile_rows");
  return f(n_rows);
}
void moe_tc(const Act &x, const void *up, const void *down, const int *offsets, const int *perm, const int *tiles,
            const float *weight, int n_experts, int top, int width, int ff, int act, bool weight_on_output, void *xs, void *mid,
            float *out, int *status, cudaStream_t s, bool gated) {
  const int n_rows = (int)x.rows * top;
  LLM_CALL("moe", llm_moe_gather, x.data, (long long)x.ld, perm, n_rows, top, width, xs, s);
  LLM_CALL("moe_tc", llm_moe_tc, xs, up, down, offsets, perm, tiles, weight, (int)x.rows, n_experts, top, width, ff, act,
           weight_on_output ? 1 : 0, gated ? 1 : 0, mid, out, status, s);
}
void moe_rows(const Act &x, const void *up, const void *down, const int *chosen, const float *weight, int top, int width, int ff,
              int act, bool weight_on_output, float *out, cudaStream_t s, bool gated) {
  LLM_CALL("moe", llm_moe_rows, code(x.dtype), x.data, (long long)x.ld, up, down, chosen, weight, (int)x.rows, top, width, ff, act,
           weight_on_output ? 1 : 0, gated ? 1 : 0, out, s);
}
bool moe_grouped_supported(int width, int ff) {
  static auto f = resolve<int (*)(int, int)>("moe", "llm_moe_grouped_supports");
  return f(width, ff) != 0;
}
void moe_grouped(const Act &x, const void *up, const void *down, const int *offsets, const int *perm, const int *tiles,
                 const float *weight, int n_experts, int top, int width, int ff, int act, bool weight_on_output, void *mid,
                 float *out, cudaStream_t s, bool gated) {
  LLM_CALL("moe", llm_moe_grouped, x.data, (long long)x.ld, up, down, offsets, perm, tiles, weight, (int)x.rows, n_experts, top,
           width, ff, act, weight_on_output ? 1 : 0, gated ? 1 : 0, mid, out, s);
}

// ---------------------------------------------------------------- state carried from token to token
LLM_KERNEL("recurrent", llm_causal_conv_mode, int, const void *, long long, void *, long long, const float *, void *, const int *,
           const int *, const int *, const int *, const int *, int, int, int, int, int, int, cudaStream_t)
LLM_KERNEL("recurrent", llm_delta_scan, const float *, long long, int, int, int, const float *, float *, float *, long long, const int *,
           const int *, int, int, int, int, int, cudaStream_t)
LLM_KERNEL("recurrent", llm_channel_delta_prepare, float *, long long, const float *, long long, int, int, int, int, int, const float *,
           const float *, const float *, const float *, float, float *, float *, int, int, int, int, int, cudaStream_t)
LLM_KERNEL("recurrent", llm_delta_rule, const float *, long long, int, int, int, int, int, int, const float *, const float *,
           const float *, float, float, float *, float *, float *, long long, const int *, const int *, int, int, int, int, cudaStream_t)
LLM_KERNEL("recurrent", llm_head_norm_gate, const float *, long long, const float *, const float *, long long, float, int, int, int,
           void *, int, long long, cudaStream_t)
void causal_conv(const Act &h, const Act &out, const float *weight, void *state, const int *tok_seq, const int *tok_pos,
                 const int *seq_start, const int *seq_past, const int *seq_slot, int n_seqs, int taps, bool single_tokens,
                 cudaStream_t s, bool silu_alone) {
  if (h.dtype != out.dtype) LLM_THROW(InvalidArg, "causal_conv: input and output have one type");
  LLM_CALL("recurrent", llm_causal_conv_mode, code(h.dtype), h.data, (long long)h.ld, out.data, (long long)out.ld, weight, state, tok_seq,
           tok_pos, seq_start, seq_past, seq_slot, (int)h.rows, n_seqs, (int)h.cols, taps, single_tokens ? 1 : 0, silu_alone ? 1 : 0, s);
}
void delta_scan(const Act &rows, int off_r, int off_k, int off_v, const float *prep, float *state, const Act &out, const int *seq_start,
                const int *seq_slot, int n_seqs, int n_heads, int d, int dv, cudaStream_t s) {
  if (rows.dtype != DType::F32 || out.dtype != DType::F32) LLM_THROW(InvalidArg, "delta_scan: vectors and results are 32-bit");
  LLM_CALL("recurrent", llm_delta_scan, (const float *)rows.data, (long long)rows.ld, off_r, off_k, off_v, prep, state, (float *)out.data,
           (long long)out.ld, seq_start, seq_slot, (int)rows.rows, n_seqs, n_heads, d, dv, s);
}
void channel_delta_prepare(const Act &cv, const Act &proj, int off_b, int off_a1, int rank_a, int off_g1, int rank_g, const float *a2,
                           const float *dt_bias, const float *a_log, const float *g2, float key_eps, float *prep, float *gate,
                           int n_heads, int n_kv, int d, int dv, cudaStream_t s) {
  if (cv.dtype != DType::F32 || proj.dtype != DType::F32) LLM_THROW(InvalidArg, "channel_delta_prepare: projections are 32-bit");
  LLM_CALL("recurrent", llm_channel_delta_prepare, (float *)cv.data, (long long)cv.ld, (const float *)proj.data, (long long)proj.ld, off_b,
           off_a1, rank_a, off_g1, rank_g, a2, dt_bias, a_log, g2, key_eps, prep, gate, (int)proj.rows, n_heads, n_kv, d, dv, s);
}
void delta_rule(const Act &proj, int off_r, int off_k, int off_v, int off_a, int off_x1, int rank, const float *w2, const float *w0,
                const float *a_bias, float decay_scale, float key_eps, float *prep, float *state, const Act &out,
                const int *seq_start, const int *seq_slot, int n_seqs, int n_heads, int d, cudaStream_t s) {
  if (proj.dtype != DType::F32 || out.dtype != DType::F32) LLM_THROW(InvalidArg, "delta_rule: projections and results are 32-bit");
  LLM_CALL("recurrent", llm_delta_rule, (const float *)proj.data, (long long)proj.ld, off_r, off_k, off_v, off_a, off_x1, rank, w2, w0,
           a_bias, decay_scale, key_eps, prep, state, (float *)out.data, (long long)out.ld, seq_start, seq_slot, (int)proj.rows,
           n_seqs, n_heads, d, s);
}
LLM_KERNEL("recurrent", llm_delta_step, const float *, long long, int, int, int, int, int, int, int, const float *, const float *,
           const float *, float, float, const float *, float, float *, void *, int, long long, const int *, int, int, int, cudaStream_t)
bool delta_step_supported(int d) {
  static auto f = resolve<int (*)(int)>("recurrent", "llm_delta_step_supports");
  return f(d) != 0;
}
void delta_step(const Act &proj, int off_r, int off_k, int off_v, int off_g, int off_a, int off_x1, int rank, const float *w2,
                const float *w0, const float *a_bias, float decay_scale, float key_eps, const float *norm_w, float eps, float *state,
                const Act &out, const int *seq_slot, int n_heads, int d, cudaStream_t s) {
  if (proj.dtype != DType::F32) LLM_THROW(InvalidArg, "delta_step: projections are 32-bit");
  LLM_CALL("recurrent", llm_delta_step, (const float *)proj.data, (long long)proj.ld, off_r, off_k, off_v, off_g, off_a, off_x1, rank,
           w2, w0, a_bias, decay_scale, key_eps, norm_w, eps, state, out.data, code(out.dtype), (long long)out.ld, seq_slot,
           (int)proj.rows, n_heads, d, s);
}
void head_norm_gate(const Act &x, const float *weight, const float *gate, long long gate_stride, float eps, int n_heads, int dv,
                    const Act &out, cudaStream_t s) {
  if (x.dtype != DType::F32) LLM_THROW(InvalidArg, "head_norm_gate: the heads' results are 32-bit");
  LLM_CALL("recurrent", llm_head_norm_gate, (const float *)x.data, (long long)x.ld, weight, gate, gate_stride, eps, (int)x.rows,
           n_heads, dv, out.data, code(out.dtype), (long long)out.ld, s);
}

// ---------------------------------------------------------------- sampling
LLM_KERNEL("sampling", llm_argmax, const float *, long long, int, int, int *, cudaStream_t)
LLM_KERNEL("sampling", llm_sample, const float *, long long, int, int, float, int, float, const float *, int *, cudaStream_t)

void argmax(const float *logits, long long stride, int n_rows, int vocab, int *out, cudaStream_t s) {
  LLM_CALL("sampling", llm_argmax, logits, stride, n_rows, vocab, out, s);
}
void sample(const float *logits, long long stride, int n_rows, int vocab, float temperature, int top_k, float top_p,
            const float *uniforms, int *out, cudaStream_t s) {
  LLM_CALL("sampling", llm_sample, logits, stride, n_rows, vocab, temperature, top_k, top_p, uniforms, out, s);
}

}  // namespace kernels
}  // namespace llm
