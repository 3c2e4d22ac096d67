// Kernels of latent attention: keys and values of all heads are functions of one cached vector
// per position, c (kv_rank channels, RMS-normed), plus one rotated key part (rot_dim channels)
// that all heads share.  A head's unrotated key is W_uk c and its value W_uv c, so
//   score = q_n . (W_uk c) + q_r . k_r = (W_uk^T q_n) . c + q_r . k_r
//   head  = sum_j p_j W_uv c_j        = W_uv (sum_j p_j c_j)
// and attention runs over the cached rows [c | k_r] themselves, as one key/value head that every
// query head reads: the query is [W_uk^T q_n | q_r] (kv_rank + rot_dim channels), the values are
// the first kv_rank channels of the key rows, and the head's result is expanded by W_uv after.
// Here: the placement of a step's tokens (both latents' norms, the rotation, the append to the
// cache), the queries' absorption of W_uk, and the expansion of the heads' results by W_uv.  The
// attention itself is attention_generic.cu (value rows with the key rows' stride).  No
// counterpart in the reference, whose one mixer caches keys and values per head
// (src/libllm/llama.cc:178-225).
//
// 32-bit: norms (sums over the product's 32-bit result), rotation, every accumulation.
#include "common.cuh"
#include <math.h>
#include <algorithm>

LLM_DEFINE_LAST_ERROR(llm_latent_last_error)

// One pair of a rotation table row: cs = [cosines (rot/2) | sines (rot/2)]; pair i is channels (2i, 2i + 1) when
// interleaved, (i, i + rot/2) otherwise.  (u, v) -> (u cos - v sin, v cos + u sin).
__device__ __forceinline__ void rotate_pair(const float *x, const float *cs, int rot, int i, int interleaved, int *ca, int *cb, float *ra,
                                            float *rb) {
  const int half = rot / 2;
  const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
  const float u = x[a], v = x[b], c = cs[i], s = cs[half + i];
  *ca = a, *cb = b;
  *ra = u * c - v * s;
  *rb = v * c + u * s;
}

// ---------------------------------------------------------------- placement
// proj rows (32-bit): the query latent (q_rank values at off_q) and, when the run has a latent projection of
// its own (off_kv >= 0), kv_rank + rot_dim values at off_kv.  cq_out = rms(query latent) * q_weight in the
// engine's type; cache row of the token = [rms(first kv_rank) * kv_weight | rotated last rot_dim].
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS)
latent_place_kernel(const float *__restrict__ proj, long long ld, int off_q, int q_rank, const float *__restrict__ q_weight,
                    T *__restrict__ cq_out, long long ldq, int off_kv, int kv_rank, int rot, const float *__restrict__ kv_weight,
                    float eps, const float *__restrict__ table, int table_rows, int interleaved, const int *__restrict__ tok_seq,
                    const int *__restrict__ tok_pos, const int *__restrict__ page_table, int pt_stride, T *__restrict__ cache,
                    int page_size) {
  __shared__ float scratch[THREADS / 32 + 1];
  grid_dependents_launch();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const float *row = proj + (size_t)t * ld;
  {
    float ss = 0.f;
    for (int c = threadIdx.x; c < q_rank; c += THREADS) ss = fmaf(row[off_q + c], row[off_q + c], ss);
    const float inv = rsqrtf(block_sum<THREADS>(ss, scratch) / (float)q_rank + eps);
    for (int c = threadIdx.x; c < q_rank; c += THREADS) cq_out[(size_t)t * ldq + c] = from_float<T>(row[off_q + c] * inv * q_weight[c]);
  }
  if (off_kv < 0) return;
  const int pos = tok_pos[t];
  const int page = page_table[(size_t)tok_seq[t] * pt_stride + pos / page_size];
  T *dst = cache + ((size_t)page * page_size + (pos % page_size)) * (size_t)(kv_rank + rot);
  const float *kv = row + off_kv;
  float ss = 0.f;
  for (int c = threadIdx.x; c < kv_rank; c += THREADS) ss = fmaf(kv[c], kv[c], ss);
  const float inv = rsqrtf(block_sum<THREADS>(ss, scratch) / (float)kv_rank + eps);
  for (int c = threadIdx.x; c < kv_rank; c += THREADS) dst[c] = from_float<T>(kv[c] * inv * kv_weight[c]);
  const float *cs = table + (size_t)(pos < table_rows ? pos : table_rows - 1) * rot;
  for (int i = threadIdx.x; i < rot / 2; i += THREADS) {
    int a, b;
    float ra, rb;
    rotate_pair(kv + kv_rank, cs, rot, i, interleaved, &a, &b, &ra, &rb);
    dst[kv_rank + a] = from_float<T>(ra);
    dst[kv_rank + b] = from_float<T>(rb);
  }
}

LLM_EXPORT int llm_latent_place(int dtype, const float *proj, long long ld, int n_tokens, int off_q, int q_rank, const float *q_weight,
                                void *cq_out, long long ldq, int off_kv, int kv_rank, int rot, const float *kv_weight, float eps,
                                const float *table, int table_rows, int interleaved, const int *tok_seq, const int *tok_pos,
                                const int *page_table, int pt_stride, void *cache, int page_size, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && q_rank > 0 && off_q >= 0 && q_weight && cq_out, "latent_place: bad sizes");
  if (off_kv >= 0)
    LLM_REQUIRE(kv_rank > 0 && rot >= 0 && rot % 2 == 0 && kv_weight && cache && page_table && (rot == 0 || (table && table_rows > 0)),
                "latent_place: bad sizes of the key/value latent");
  constexpr int THREADS = 256;
  if (dtype == LLM_F32)
    llm_launch(latent_place_kernel<float, THREADS>, dim3(n_tokens), dim3(THREADS), 0, stream, proj, ld, off_q, q_rank, q_weight,
               (float *)cq_out, ldq, off_kv, kv_rank, rot, kv_weight, eps, table, table_rows, interleaved, tok_seq, tok_pos, page_table,
               pt_stride, (float *)cache, page_size);
  else if (dtype == LLM_BF16)
    llm_launch(latent_place_kernel<__nv_bfloat16, THREADS>, dim3(n_tokens), dim3(THREADS), 0, stream, proj, ld, off_q, q_rank, q_weight,
               (__nv_bfloat16 *)cq_out, ldq, off_kv, kv_rank, rot, kv_weight, eps, table, table_rows, interleaved, tok_seq, tok_pos,
               page_table, pt_stride, (__nv_bfloat16 *)cache, page_size);
  else LLM_FAIL("latent_place: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("latent_place");
  return LLM_OK;
}

// ---------------------------------------------------------------- the queries take in W_uk
// q rows (32-bit) [heads, d + rot]: out[t, h] = [sum_i q[t, h, i] * w_uk[h * d + i, :] (kv_rank) | rotated q[t, h, d:] (rot)]
// in the engine's type.  A CTA takes one head and TT tokens: the tokens' unrotated parts lie in shared memory, a
// thread owns output channels and walks the head's d rows of w_uk (its neighbours read the neighbouring channels);
// the channels are shared out over blockIdx.z so that a step of few tokens still fills the device.
constexpr int LAT_TT = 16;
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS)
latent_absorb_kernel(const float *__restrict__ q, long long ldq, const T *__restrict__ w_uk, T *__restrict__ out, long long ldo,
                     int n_tokens, int d, int rot, int kv_rank, const float *__restrict__ table, int table_rows, int interleaved,
                     const int *__restrict__ tok_pos) {
  extern __shared__ float qs[];                        // [LAT_TT][d]
  grid_dependents_launch();
  grid_dependency_wait();
  const int t0 = blockIdx.x * LAT_TT, h = blockIdx.y;
  const int nt = min(LAT_TT, n_tokens - t0);
  for (int i = threadIdx.x; i < LAT_TT * d; i += THREADS) {
    const int t = i / d, c = i - t * d;
    qs[i] = t < nt ? q[(size_t)(t0 + t) * ldq + (size_t)h * (d + rot) + c] : 0.f;
  }
  __syncthreads();
  const T *w = w_uk + (size_t)h * d * kv_rank;
  for (int c = blockIdx.z * THREADS + threadIdx.x; c < kv_rank; c += THREADS * gridDim.z) {
    float acc[LAT_TT];
#pragma unroll
    for (int t = 0; t < LAT_TT; ++t) acc[t] = 0.f;
#pragma unroll 16
    for (int i = 0; i < d; ++i) {
      const float wv = to_float(w[(size_t)i * kv_rank + c]);
#pragma unroll
      for (int t = 0; t < LAT_TT; ++t) acc[t] = fmaf(qs[t * d + i], wv, acc[t]);
    }
#pragma unroll
    for (int t = 0; t < LAT_TT; ++t)
      if (t < nt) out[(size_t)(t0 + t) * ldo + (size_t)h * (kv_rank + rot) + c] = from_float<T>(acc[t]);
  }
  const int half = rot / 2;
  if (blockIdx.z != 0) return;
  for (int i = threadIdx.x; i < nt * half; i += THREADS) {
    const int t = i / half, pr = i - t * half;
    const int pos = tok_pos[t0 + t];
    const float *cs = table + (size_t)(pos < table_rows ? pos : table_rows - 1) * rot;
    int a, b;
    float ra, rb;
    rotate_pair(q + (size_t)(t0 + t) * ldq + (size_t)h * (d + rot) + d, cs, rot, pr, interleaved, &a, &b, &ra, &rb);
    T *dst = out + (size_t)(t0 + t) * ldo + (size_t)h * (kv_rank + rot) + kv_rank;
    dst[a] = from_float<T>(ra);
    dst[b] = from_float<T>(rb);
  }
}

LLM_EXPORT int llm_latent_absorb(int dtype, const float *q, long long ldq, const void *w_uk, void *out, long long ldo, int n_tokens,
                                 int n_heads, int d, int rot, int kv_rank, const float *table, int table_rows, int interleaved,
                                 const int *tok_pos, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_heads > 0 && n_heads <= 65535 && d > 0 && kv_rank > 0 && rot >= 0 && rot % 2 == 0, "latent_absorb: bad sizes");
  LLM_REQUIRE(rot == 0 || (table && table_rows > 0), "latent_absorb: a rotation needs its table");
  constexpr int THREADS = 128;
  const size_t smem = (size_t)LAT_TT * d * sizeof(float);
  LLM_REQUIRE(smem <= 96 * 1024, "latent_absorb: heads of %d channels are not supported", d);
  const dim3 grid((n_tokens + LAT_TT - 1) / LAT_TT, n_heads, (kv_rank + THREADS - 1) / THREADS);
  if (dtype == LLM_F32) {
    LLM_CHECK_CUDA(llm_allow_smem(latent_absorb_kernel<float, THREADS>, smem), "latent_absorb attribute");
    llm_launch(latent_absorb_kernel<float, THREADS>, grid, dim3(THREADS), smem, stream, q, ldq, (const float *)w_uk, (float *)out, ldo,
               n_tokens, d, rot, kv_rank, table, table_rows, interleaved, tok_pos);
  } else if (dtype == LLM_BF16) {
    LLM_CHECK_CUDA(llm_allow_smem(latent_absorb_kernel<__nv_bfloat16, THREADS>, smem), "latent_absorb attribute");
    llm_launch(latent_absorb_kernel<__nv_bfloat16, THREADS>, grid, dim3(THREADS), smem, stream, q, ldq, (const __nv_bfloat16 *)w_uk,
               (__nv_bfloat16 *)out, ldo, n_tokens, d, rot, kv_rank, table, table_rows, interleaved, tok_pos);
  } else LLM_FAIL("latent_absorb: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("latent_absorb");
  return LLM_OK;
}

// ---------------------------------------------------------------- the heads' results are expanded by W_uv
// x [tokens, heads, kv_rank] (the weighted sums of cached latents), w_uv [heads * dv, kv_rank]:
// out[t, h, j] = sum_c x[t, h, c] * w_uv[h * dv + j, c].  A CTA takes one head and TT tokens; a warp owns output
// channels, its lanes walk a row of w_uv together (in lane order, then the shuffle tree); blockIdx.z shares the
// output channels out, eight to a CTA.
constexpr int LAT_ET = 8;
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS)
latent_expand_kernel(const T *__restrict__ x, long long ldx, const T *__restrict__ w_uv, T *__restrict__ out, long long ldo, int n_tokens,
                     int kv_rank, int dv) {
  extern __shared__ float xs[];                        // [LAT_ET][kv_rank]
  grid_dependents_launch();
  grid_dependency_wait();
  const int t0 = blockIdx.x * LAT_ET, h = blockIdx.y;
  const int nt = min(LAT_ET, n_tokens - t0);
  for (int i = threadIdx.x; i < LAT_ET * kv_rank; i += THREADS) {
    const int t = i / kv_rank, c = i - t * kv_rank;
    xs[i] = t < nt ? to_float(x[(size_t)(t0 + t) * ldx + (size_t)h * kv_rank + c]) : 0.f;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int j = blockIdx.z * (THREADS / 32) + warp; j < dv; j += THREADS / 32 * gridDim.z) {
    const T *w = w_uv + ((size_t)h * dv + j) * kv_rank;
    float acc[LAT_ET];
#pragma unroll
    for (int t = 0; t < LAT_ET; ++t) acc[t] = 0.f;
    for (int c = lane; c < kv_rank; c += 32) {
      const float wv = to_float(w[c]);
#pragma unroll
      for (int t = 0; t < LAT_ET; ++t) acc[t] = fmaf(xs[t * kv_rank + c], wv, acc[t]);
    }
#pragma unroll
    for (int t = 0; t < LAT_ET; ++t) {
      const float s = warp_sum(acc[t]);
      if (lane == 0 && t < nt) out[(size_t)(t0 + t) * ldo + (size_t)h * dv + j] = from_float<T>(s);
    }
  }
}

LLM_EXPORT int llm_latent_expand(int dtype, const void *x, long long ldx, const void *w_uv, void *out, long long ldo, int n_tokens,
                                 int n_heads, int kv_rank, int dv, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_heads > 0 && n_heads <= 65535 && kv_rank > 0 && dv > 0, "latent_expand: bad sizes");
  constexpr int THREADS = 256;
  const size_t smem = (size_t)LAT_ET * kv_rank * sizeof(float);
  LLM_REQUIRE(smem <= 96 * 1024, "latent_expand: a latent of %d channels is not supported", kv_rank);
  const dim3 grid((n_tokens + LAT_ET - 1) / LAT_ET, n_heads, std::min(64, (dv + THREADS / 32 - 1) / (THREADS / 32)));
  if (dtype == LLM_F32) {
    LLM_CHECK_CUDA(llm_allow_smem(latent_expand_kernel<float, THREADS>, smem), "latent_expand attribute");
    llm_launch(latent_expand_kernel<float, THREADS>, grid, dim3(THREADS), smem, stream, (const float *)x, ldx, (const float *)w_uv,
               (float *)out, ldo, n_tokens, kv_rank, dv);
  } else if (dtype == LLM_BF16) {
    LLM_CHECK_CUDA(llm_allow_smem(latent_expand_kernel<__nv_bfloat16, THREADS>, smem), "latent_expand attribute");
    llm_launch(latent_expand_kernel<__nv_bfloat16, THREADS>, grid, dim3(THREADS), smem, stream, (const __nv_bfloat16 *)x, ldx,
               (const __nv_bfloat16 *)w_uv, (__nv_bfloat16 *)out, ldo, n_tokens, kv_rank, dv);
  } else LLM_FAIL("latent_expand: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("latent_expand");
  return LLM_OK;
}
