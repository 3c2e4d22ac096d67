// Causal grouped-query attention over the paged cache, any head size up to 1,024 (values may
// have another width than keys, or be the first channels of the key rows themselves: v_ld), any number of heads and groups; optional sliding window,
// optional block mask (a query sees only keys of its own block of `block` positions, blocks
// counted from position 0), optionally the first `sink` positions of the sequence kept visible
// beyond the window (at their true positions), optional gate per (token, head) on the result (multiplied by
// sigmoid(gate)); element type float or bfloat16, arithmetic in 32-bit.  One warp serves one (token, head): lanes take 32 keys at a time
// for the scores, then 32 channels at a time for the weighted sum, with a running
// maximum and sum (the online form of softmax, src/flint/cpu/softmax.cc:31-60).
//
// This is the attention of the true 32-bit path and of head sizes the fast bfloat16
// kernels do not take.  It serves prompts and single tokens alike: the keys of the
// step's own tokens are already in the cache when it runs, and the token at position p
// reads keys 0..p (or the last `window` of them), which is the bottom-right aligned
// causal mask of the reference (src/flint/operators.cc:119-124).  Head h reads
// key/value head h / (heads / kv_heads) (src/flint/operators.cc:43-56); scores are
// scaled by 1/sqrt(d) (src/flint/operators.cc:115-117).
//
// A token's result depends only on its own sequence: the order of additions is fixed by
// the position, not by the batch.
#include "common.cuh"
#include <math.h>

LLM_DEFINE_LAST_ERROR(llm_attention_generic_last_error)

constexpr int WARPS = 4;
constexpr int MAX_D_SMALL = 256, MAX_D_LARGE = 1024;

__device__ __forceinline__ float dot_row(const float *q, const float *k, int d, bool vec) {
  float acc = 0.f;
  if (!vec) {
    for (int c = 0; c < d; ++c) acc = fmaf(q[c], k[c], acc);
    return acc;
  }
  for (int c = 0; c < d; c += 4) {
    const float4 v = *reinterpret_cast<const float4 *>(k + c);
    acc = fmaf(q[c], v.x, acc);
    acc = fmaf(q[c + 1], v.y, acc);
    acc = fmaf(q[c + 2], v.z, acc);
    acc = fmaf(q[c + 3], v.w, acc);
  }
  return acc;
}
__device__ __forceinline__ float dot_row(const float *q, const __nv_bfloat16 *k, int d, bool vec) {
  float acc = 0.f;
  if (!vec) {
    for (int c = 0; c < d; ++c) acc = fmaf(q[c], __bfloat162float(k[c]), acc);
    return acc;
  }
  for (int c = 0; c < d; c += 8) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(k + c);
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      acc = fmaf(q[c + 2 * i], f.x, acc);
      acc = fmaf(q[c + 2 * i + 1], f.y, acc);
    }
  }
  return acc;
}

template <typename T, int MAX_D>
__global__ void __launch_bounds__(WARPS * 32)
attention_generic_kernel(const T *__restrict__ q, long long q_stride, T *__restrict__ out,
                         long long out_stride, const T *__restrict__ kcache,
                         const T *__restrict__ vcache, const int *__restrict__ tok_seq,
                         const int *__restrict__ tok_pos, const int *__restrict__ page_table,
                         int pt_stride, int n_tokens, int n_heads, int n_kv, int d, int dv, int page_size,
                         int window, int block, int sink, float scale, const float *__restrict__ gate,
                         long long gate_stride, int vec, int v_ld, float null_score) {
  __shared__ __align__(16) float q_s[WARPS][MAX_D];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long w = (long long)blockIdx.x * WARPS + warp;
  const int token = (int)(w / n_heads), h = (int)(w % n_heads);
  if (token >= n_tokens) return;
  const int p = tok_pos[token];
  const int *pt = page_table + (size_t)tok_seq[token] * pt_stride;
  const int kvh = h / (n_heads / n_kv);
  const T *qrow = q + (size_t)token * q_stride + (size_t)h * d;
  for (int c = lane; c < d; c += 32) q_s[warp][c] = to_float(qrow[c]);
  __syncwarp();

  int kstart = window > 0 ? max(0, p - window + 1) : 0;
  if (block > 0) kstart = max(kstart, p / block * block);
  float m = -INFINITY, l = 0.f;
  float acc[MAX_D / 32];
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) acc[i] = 0.f;

  // two runs of keys: the kept first positions that lie before the window, then the window
  const int sink_end = (window > 0 && block == 0) ? min(sink, kstart) : 0;
  for (int run = sink_end > 0 ? 0 : 1; run < 2; ++run) {
    const int k0 = run == 0 ? 0 : kstart, k1 = run == 0 ? sink_end : p + 1;
    for (int kb = k0; kb < k1; kb += 32) {
      const int j = kb + lane;
      const bool valid = j < k1;
      float s = -INFINITY;
      if (valid) {
        const int page = pt[j / page_size];
        const T *krow = kcache + (((size_t)page * n_kv + kvh) * page_size + (j % page_size)) * d;
        s = dot_row(q_s[warp], krow, d, vec != 0) * scale;
      }
      const float m_new = fmaxf(m, warp_max(s));          // finite: lane 0 always holds a key
      const float pj = valid ? expf(s - m_new) : 0.f;
      const float alpha = expf(m - m_new);                // 0 on the first block (m = -inf)
      l = l * alpha + warp_sum(pj);
#pragma unroll
      for (int i = 0; i < MAX_D / 32; ++i) acc[i] *= alpha;
      const int nvalid = min(32, k1 - kb);
      for (int jj = 0; jj < nvalid; ++jj) {
        const float pv = __shfl_sync(0xffffffffu, pj, jj);
        const int key = kb + jj;
        const int page = pt[key / page_size];
        const T *vrow = vcache + (((size_t)page * n_kv + kvh) * page_size + (key % page_size)) * v_ld;
#pragma unroll
        for (int i = 0; i < MAX_D / 32; ++i) {
          const int c = lane + 32 * i;
          if (c < dv) acc[i] = fmaf(pv, to_float(vrow[c]), acc[i]);
        }
      }
      m = m_new;
    }
  }
  T *orow = out + (size_t)token * out_stride + (size_t)h * dv;
  if (null_score > -INFINITY) {     // one more key whose score is null_score and whose value is nought
    const float m_new = fmaxf(m, null_score), alpha = expf(m - m_new);
    l = l * alpha + expf(null_score - m_new);
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) acc[i] *= alpha;
  }
  float inv = 1.f / l;
  if (gate) inv *= 1.f / (1.f + expf(-gate[(size_t)token * gate_stride + h]));
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) {
    const int c = lane + 32 * i;
    if (c < dv) orow[c] = from_float<T>(acc[i] * inv);
  }
}

// v_ld: channels between two value rows of the value storage (dv for a storage of its own; the key rows' width
// when the values are the first dv channels of the keys and vcache is kcache).
LLM_EXPORT int llm_attention_generic_ld(int dtype, const void *q, long long q_stride, void *out,
                                        long long out_stride, const void *kcache, const void *vcache,
                                        const int *tok_seq, const int *tok_pos, const int *page_table,
                                        int pt_stride, int n_tokens, int n_heads, int n_kv, int d, int dv, int v_ld,
                                        int page_size, int window, int block, int sink, float scale, const float *gate,
                                        long long gate_stride, float null_score, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv > 0 && n_heads % n_kv == 0, "attention: bad head counts %d/%d", n_heads, n_kv);
  LLM_REQUIRE(d > 0 && d <= MAX_D_LARGE && dv > 0 && dv <= MAX_D_LARGE, "attention: head sizes %d / %d are not supported (up to %d)", d, dv,
              MAX_D_LARGE);
  LLM_REQUIRE(v_ld >= dv, "attention: value rows of %d channels in a storage of %d a row", dv, v_ld);
  LLM_REQUIRE(window >= 0 && block >= 0 && sink >= 0, "attention: bad window, block or number of kept first positions");
  LLM_REQUIRE(sink == 0 || block == 0, "attention: kept first positions go with a window, not with a block mask");
  // 16-byte loads of key rows where rows start on such a boundary
  const int vec = (dtype == LLM_F32 ? d % 4 == 0 : d % 8 == 0) && (uintptr_t)kcache % 16 == 0;
  const long long warps = (long long)n_tokens * n_heads;
  const long long blocks = (warps + WARPS - 1) / WARPS;
  LLM_REQUIRE(blocks < 2147483647LL, "attention: too many tokens for one launch");
  const bool small = d <= MAX_D_SMALL && dv <= MAX_D_SMALL;
#define GENERIC_GO(T, MAXD)                                                                                              \
  attention_generic_kernel<T, MAXD><<<(unsigned)blocks, WARPS * 32, 0, stream>>>(                                          \
      (const T *)q, q_stride, (T *)out, out_stride, (const T *)kcache, (const T *)vcache, tok_seq, tok_pos, page_table, pt_stride, \
      n_tokens, n_heads, n_kv, d, dv, page_size, window, block, sink, scale, gate, gate_stride, vec, v_ld, null_score)
  if (dtype == LLM_F32 && small) GENERIC_GO(float, MAX_D_SMALL);
  else if (dtype == LLM_F32) GENERIC_GO(float, MAX_D_LARGE);
  else if (dtype == LLM_BF16 && small) GENERIC_GO(__nv_bfloat16, MAX_D_SMALL);
  else if (dtype == LLM_BF16) GENERIC_GO(__nv_bfloat16, MAX_D_LARGE);
  else LLM_FAIL("attention: unknown dtype %d", dtype);
#undef GENERIC_GO
  LLM_CHECK_LAUNCH("attention_generic");
  return LLM_OK;
}

LLM_EXPORT int llm_attention_generic(int dtype, const void *q, long long q_stride, void *out,
                                     long long out_stride, const void *kcache, const void *vcache,
                                     const int *tok_seq, const int *tok_pos, const int *page_table,
                                     int pt_stride, int n_tokens, int n_heads, int n_kv, int d, int dv,
                                     int page_size, int window, int block, int sink, float scale, const float *gate,
                                     long long gate_stride, cudaStream_t stream) {
  return llm_attention_generic_ld(dtype, q, q_stride, out, out_stride, kcache, vcache, tok_seq, tok_pos, page_table, pt_stride,
                                  n_tokens, n_heads, n_kv, d, dv, dv, page_size, window, block, sink, scale, gate, gate_stride, -INFINITY, stream);
}
