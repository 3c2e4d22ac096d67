// Kernels of mixers that carry fixed-size state from token to token: a short causal convolution
// over time on each channel, and the generalized delta rule (a matrix of state per head that
// decays per key channel, forgets along the current unit key and learns the outer product of key
// and value), with the norm and gate that follow it.  No counterpart in the reference, whose one
// mixer is attention (src/libllm/llama.cc:178-225).
//
// Everything that enters the recurrence is 32-bit: the projections arrive as the 32-bit results of
// their products, decays, removal rates, unit keys and the state itself are float.  A sequence's
// result depends on nothing but its own tokens and state: one thread owns one column of one head's
// state (or a fixed share of its rows), sums run in a fixed order, and no sum crosses sequences.
#include "common.cuh"
#include <math.h>

LLM_DEFINE_LAST_ERROR(llm_recurrent_last_error)

// ---------------------------------------------------------------- causal convolution over time
// out_t = h_t + sum_j w[c, j] * h_(t - taps + 1 + j), zeros before the sequence's start.  The last
// taps - 1 inputs of every sequence are its state, state[slot][i][c] for the position
// length - (taps - 1) + i.  Rows whose window lies inside the step are computed by CTAs that own a
// run of rows (blockIdx.y < n_chunks); the first taps - 1 rows of each sequence, which need the
// state, by a CTA of their sequence (blockIdx.y - n_chunks), whose threads read the old state of
// their channel into registers before they write the new one: no other thread reads it.
constexpr int CONV_MAX_TAPS = 8;
constexpr int CONV_THREADS = 128;

template <int N>
__device__ __forceinline__ float pick(const float (&a)[N], int idx) {
  float r = 0.f;
#pragma unroll
  for (int k = 0; k < N; ++k)
    if (k == idx) r = a[k];
  return r;
}

// vals[j] = h at position p - taps + 1 + j; the same order of operations wherever a row is computed.
// mode 0: the input plus its convolution; mode 1: silu of the convolution alone (a projection's short convolution).
__device__ __forceinline__ float conv_row(const float (&w)[CONV_MAX_TAPS], const float (&vals)[CONV_MAX_TAPS], int taps, int mode) {
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; ++j)
    if (j < taps) s = fmaf(w[j], vals[j], s);
  if (mode == 1) return s / (1.f + expf(-s));
  return pick(vals, taps - 1) + s;
}

// V channels to a thread: 1, or as many as 16 bytes hold where rows allow such loads.
template <typename T, int V>
struct ConvVec {
  float x[V];
};
template <typename T, int V>
__device__ __forceinline__ ConvVec<T, V> conv_load(const T *p) {
  ConvVec<T, V> r;
  if (V == 1) {
    r.x[0] = to_float(p[0]);
  } else if (sizeof(T) == 4) {
    const float4 v = *reinterpret_cast<const float4 *>(p);
    r.x[0] = v.x, r.x[1] = v.y, r.x[2] = v.z, r.x[3] = v.w;
  } else {
    const uint4 raw = *reinterpret_cast<const uint4 *>(p);
    const __nv_bfloat162 *h2 = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
    for (int i = 0; i < V / 2; ++i) {
      const float2 f = __bfloat1622float2(h2[i]);
      r.x[2 * i] = f.x, r.x[2 * i + 1] = f.y;
    }
  }
  return r;
}
template <typename T, int V>
__device__ __forceinline__ void conv_store(T *p, const ConvVec<T, V> &r) {
  if (V == 1) {
    p[0] = from_float<T>(r.x[0]);
  } else if (sizeof(T) == 4) {
    *reinterpret_cast<float4 *>(p) = make_float4(r.x[0], r.x[1], r.x[2], r.x[3]);
  } else {
    uint4 raw;
    __nv_bfloat162 *h2 = reinterpret_cast<__nv_bfloat162 *>(&raw);
#pragma unroll
    for (int i = 0; i < V / 2; ++i) h2[i] = __floats2bfloat162_rn(r.x[2 * i], r.x[2 * i + 1]);
    *reinterpret_cast<uint4 *>(p) = raw;
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(CONV_THREADS)
causal_conv_kernel(const T *__restrict__ h, long long ldh, T *__restrict__ out, long long ldo, const float *__restrict__ weight,
                   T *__restrict__ state, const int *__restrict__ tok_seq, const int *__restrict__ tok_pos,
                   const int *__restrict__ seq_start, const int *__restrict__ seq_past, const int *__restrict__ seq_slot,
                   int n_tokens, int width, int taps, int n_chunks, int chunk_rows, int mode) {
  using Vec = ConvVec<T, V>;
  grid_dependents_launch();
  const int c = (blockIdx.x * CONV_THREADS + threadIdx.x) * V;
  float w[V][CONV_MAX_TAPS];
#pragma unroll
  for (int v = 0; v < V; ++v)
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) w[v][j] = (c + v < width && j < taps) ? weight[(size_t)(c + v) * taps + j] : 0.f;
  grid_dependency_wait();
  if (c >= width) return;
  const int keep = taps - 1;
  Vec vals[CONV_MAX_TAPS];
  auto row_out = [&]() {                              // the same order of operations wherever a row is computed
    Vec r;
#pragma unroll
    for (int v = 0; v < V; ++v) {
      float column[CONV_MAX_TAPS];
#pragma unroll
      for (int j = 0; j < CONV_MAX_TAPS; ++j) column[j] = vals[j].x[v];
      r.x[v] = conv_row(w[v], column, taps, mode);
    }
    return r;
  };
  if ((int)blockIdx.y < n_chunks) {
    const int r0 = blockIdx.y * chunk_rows, r1 = min(n_tokens, r0 + chunk_rows);
    // which rows are this CTA's: asked for all rows at once, so that their loads do not wait for one another
    unsigned mine = 0;
    for (int row = r0; row < r1; ++row) mine |= (tok_pos[row] - seq_past[tok_seq[row]] >= keep ? 1u : 0u) << (row - r0);
    for (int row = r0; row < r1; ++row) {
      if (!((mine >> (row - r0)) & 1u)) continue;               // the sequence's own CTA computes it
#pragma unroll
      for (int j = 0; j < CONV_MAX_TAPS; ++j)
        if (j < taps) vals[j] = conv_load<T, V>(h + (size_t)(row - keep + j) * ldh + c);
      conv_store<T, V>(out + (size_t)row * ldo + c, row_out());
    }
    return;
  }
  const int b = blockIdx.y - n_chunks;
  const int start = seq_start[b], n = seq_start[b + 1] - start;
  T *st = state + (size_t)seq_slot[b] * keep * width + c;
  Vec old[CONV_MAX_TAPS - 1];
#pragma unroll
  for (int i = 0; i < CONV_MAX_TAPS - 1; ++i)
    if (i < keep) old[i] = conv_load<T, V>(st + (size_t)i * width);
  // position (relative to the sequence's length before the step) -> input
  auto at = [&](int rel) {
    if (rel >= 0) return conv_load<T, V>(h + (size_t)(start + rel) * ldh + c);
    Vec r = old[0];
#pragma unroll
    for (int i = 1; i < CONV_MAX_TAPS - 1; ++i)
      if (i == keep + rel) r = old[i];
    return r;
  };
  for (int i = 0; i < min(n, keep); ++i) {
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j)
      if (j < taps) vals[j] = at(i - keep + j);
    conv_store<T, V>(out + (size_t)(start + i) * ldo + c, row_out());
  }
  for (int i = 0; i < keep; ++i) conv_store<T, V>(st + (size_t)i * width, at(n - keep + i));
}

LLM_EXPORT int llm_causal_conv_mode(int dtype, const void *h, long long ldh, void *out, long long ldo, const float *weight, void *state,
                                    const int *tok_seq, const int *tok_pos, const int *seq_start, const int *seq_past,
                                    const int *seq_slot, int n_tokens, int n_seqs, int width, int taps, int single_tokens, int mode,
                                    cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(mode == 0 || mode == 1, "causal_conv: mode %d is not known (0: input plus convolution, 1: silu of the convolution)", mode);
  LLM_REQUIRE(n_tokens > 0 && n_seqs > 0 && width > 0, "causal_conv: bad sizes");
  LLM_REQUIRE(taps >= 1 && taps <= CONV_MAX_TAPS, "causal_conv: %d taps are not supported (1 to %d)", taps, CONV_MAX_TAPS);
  LLM_REQUIRE(taps == 1 || state != nullptr, "causal_conv: a convolution of %d taps needs its state", taps);
  const int chunk_rows = 16;                          // at most 32 (a bit per row)
  // a step of single tokens has no row whose window lies inside the step (but for one tap)
  const int n_chunks = single_tokens && taps > 1 ? 0 : (n_tokens + chunk_rows - 1) / chunk_rows;
  const int n_own = taps > 1 ? n_seqs : 0;
  if (n_chunks + n_own == 0) return LLM_OK;
  LLM_REQUIRE(n_chunks + n_own <= 65535, "causal_conv: too many rows for one launch");
  // 16 bytes of channels to a thread where every row starts on such a boundary
  const int per = dtype == LLM_F32 ? 4 : 8;
  const bool vec = width % per == 0 && ldh % per == 0 && ldo % per == 0 && (uintptr_t)h % 16 == 0 && (uintptr_t)out % 16 == 0 &&
                   (uintptr_t)state % 16 == 0;
  const int v = vec ? per : 1;
  const dim3 grid((width + CONV_THREADS * v - 1) / (CONV_THREADS * v), n_chunks + n_own);
#define CONV_GO(T, V)                                                                                                       \
  llm_launch(causal_conv_kernel<T, V>, grid, dim3(CONV_THREADS), 0, stream, (const T *)h, ldh, (T *)out, ldo, weight, (T *)state, \
             tok_seq, tok_pos, seq_start, seq_past, seq_slot, n_tokens, width, taps, n_chunks, chunk_rows, mode)
  if (dtype == LLM_F32 && vec) CONV_GO(float, 4);
  else if (dtype == LLM_F32) CONV_GO(float, 1);
  else if (dtype == LLM_BF16 && vec) CONV_GO(__nv_bfloat16, 8);
  else if (dtype == LLM_BF16) CONV_GO(__nv_bfloat16, 1);
  else LLM_FAIL("causal_conv: unknown dtype %d", dtype);
#undef CONV_GO
  LLM_CHECK_LAUNCH("causal_conv");
  return LLM_OK;
}

LLM_EXPORT int llm_causal_conv(int dtype, const void *h, long long ldh, void *out, long long ldo, const float *weight, void *state,
                               const int *tok_seq, const int *tok_pos, const int *seq_start, const int *seq_past,
                               const int *seq_slot, int n_tokens, int n_seqs, int width, int taps, int single_tokens,
                               cudaStream_t stream) {
  return llm_causal_conv_mode(dtype, h, ldh, out, ldo, weight, state, tok_seq, tok_pos, seq_start, seq_past, seq_slot, n_tokens, n_seqs,
                              width, taps, single_tokens, 0, stream);
}

// ---------------------------------------------------------------- the delta rule: what each token brings
// From a token's projections (32-bit rows of the stacked product: r, k, v, ..., the removal
// logits and the low-rank decay input) to the vectors of the recurrence, per head and key channel:
//   decay   w = exp(-decay_scale * sigmoid(w0 + W2 tanh(x1)))       x1 = the low-rank projection
//   unit    u = k / sqrt(sum(k^2) + key_eps)
//   removal b = sigmoid(a + a_bias) * u
// prep [tokens, heads, 3, d]: w, b, u.  A CTA takes one head and a run of tokens, a warp one token
// at a time: the head's rows of W2 ([d, rank], each row padded by one value so that the lanes'
// reads fall on different banks) lie in shared memory when they fit, tanh(x1) is taken once per
// token and warp.  Sums over the head run in lane order then the shuffle tree, whatever the launch.
constexpr int DP_WARPS = 4;
constexpr int DP_TOKENS = 32;                        // tokens of a CTA

__global__ void __launch_bounds__(DP_WARPS * 32)
delta_prepare_kernel(const float *__restrict__ proj, long long ld, int off_k, int off_a, int off_x1, int rank,
                     const float *__restrict__ w2, const float *__restrict__ w0, const float *__restrict__ a_bias,
                     float decay_scale, float key_eps, int n_tokens, int n_heads, int d, int w2_shared,
                     float *__restrict__ prep) {
  extern __shared__ float dp_smem[];                 // tanh(x1) [warps][rank], then W2's rows of the head [d][rank + 1]
  grid_dependents_launch();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int hd = blockIdx.y;
  float *th = dp_smem + warp * rank;
  float *w2s = dp_smem + DP_WARPS * rank;
  const float *w2h = w2 + (size_t)hd * d * rank;
  if (w2_shared)                                     // weights: nothing of the step is read yet
    for (int i = threadIdx.x; i < d * rank; i += DP_WARPS * 32) w2s[(i / rank) * (rank + 1) + i % rank] = w2h[i];
  grid_dependency_wait();
  __syncthreads();
  const int t1 = min(n_tokens, (int)(blockIdx.x + 1) * DP_TOKENS);
  for (int t = blockIdx.x * DP_TOKENS + warp; t < t1; t += DP_WARPS) {
    const float *row = proj + (size_t)t * ld;
    const float *k = row + off_k + (size_t)hd * d;
    __syncwarp();
    for (int q = lane; q < rank; q += 32) th[q] = tanhf(row[off_x1 + q]);
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) ss = fmaf(k[i], k[i], ss);
    ss = warp_sum(ss);
    __syncwarp();
    const float inv = 1.f / sqrtf(ss + key_eps);
    float *o = prep + ((size_t)t * n_heads + hd) * 3 * d;
    for (int i0 = 0; i0 < d; i0 += 128) {             // four channels of a lane at a time: four chains of sums, not one
      float z[4];
      int chs[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int i = i0 + lane + 32 * c;
        chs[c] = i < d ? i : -1;
        z[c] = i < d ? w0[hd * d + i] : 0.f;
      }
      if (w2_shared) {
        for (int q = 0; q < rank; ++q) {
          const float tq = th[q];
#pragma unroll
          for (int c = 0; c < 4; ++c)
            if (chs[c] >= 0) z[c] = fmaf(w2s[chs[c] * (rank + 1) + q], tq, z[c]);
        }
      } else {
        for (int q = 0; q < rank; ++q) {
          const float tq = th[q];
#pragma unroll
          for (int c = 0; c < 4; ++c)
            if (chs[c] >= 0) z[c] = fmaf(w2h[(size_t)chs[c] * rank + q], tq, z[c]);
        }
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int i = chs[c];
        if (i < 0) continue;
        const int ch = hd * d + i;
        const float u = k[i] * inv;
        const float a = 1.f / (1.f + expf(-(row[off_a + ch] + a_bias[ch])));
        o[i] = expf(-decay_scale / (1.f + expf(-z[c])));
        o[d + i] = a * u;
        o[2 * d + i] = u;
      }
    }
  }
}

// ---------------------------------------------------------------- the delta rule: the recurrence
// Per head, state S [d keys x d values]:  S <- diag(w) S - b (u^T S) + k v^T  (both terms read the
// old S), then o = S^T r.  A column of S never meets another column, so LANES neighbouring lanes,
// each with d / LANES of its rows in registers, own column j for the whole step and walk the
// sequence's tokens in order.  The tokens' vectors (w, b, u from the preparation, k and r from the
// product's rows, the CTA's columns of v) come through a ring of 8 or 16 tokens in shared memory,
// filled by a third warp's asynchronous copies that run that many tokens ahead of the arithmetic (what a token
// needs was written by the kernels just before and may come from DRAM), so that a token costs its arithmetic and a
// share of a barrier, not a trip to memory.  (Issued by the warps of the recurrence themselves, the copies and their
// address arithmetic cost a scan of 2,048 tokens 0.3 ms of its 0.86.)  Sums run over four partial sums in
// a fixed order, then the lanes' shuffle tree.  state[slot][head][j][i] (a column's rows together).
constexpr int DR_THREADS = 64;
constexpr int DR_STAGES_MAX = 16;                   // tokens of the ring: 16 where they fit 48 KB of shared memory, else 8

__device__ __forceinline__ void cp_async4(void *smem, const void *gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async16_cg(void *smem, const void *gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit_group() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// One token of one column: this thread's share S[ROWS] of the column, the token's vectors w, b, u, k, r (each
// VLEN floats on; `vecs` points at this thread's share of w, 16-byte aligned), the column's value v.  Returns the
// column's read-out S^T r, summed over the LANES lanes of the column.  Sums run over four partial sums in a
// fixed order, then the lanes' shuffle tree: the same wherever a token is computed.
template <int ROWS, int LANES>
__device__ __forceinline__ float delta_token(float (&S)[ROWS], const float *vecs, int VLEN, float v) {
  const float4 *w4 = reinterpret_cast<const float4 *>(vecs), *b4 = reinterpret_cast<const float4 *>(vecs + VLEN);
  const float4 *u4 = reinterpret_cast<const float4 *>(vecs + 2 * VLEN), *k4 = reinterpret_cast<const float4 *>(vecs + 3 * VLEN);
  const float4 *r4 = reinterpret_cast<const float4 *>(vecs + 4 * VLEN);
  float p4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int i = 0; i < ROWS / 4; ++i) {
    const float4 uu = u4[i];
    p4[0] = fmaf(uu.x, S[4 * i], p4[0]);
    p4[1] = fmaf(uu.y, S[4 * i + 1], p4[1]);
    p4[2] = fmaf(uu.z, S[4 * i + 2], p4[2]);
    p4[3] = fmaf(uu.w, S[4 * i + 3], p4[3]);
  }
  float us = (p4[0] + p4[1]) + (p4[2] + p4[3]);
  // what does not wait for u^T S is taken while its shuffles are on their way: e = w S + k v, then S = e - b (u^T S)
  float e[ROWS];
#pragma unroll
  for (int i = 0; i < ROWS / 4; ++i) {
    const float4 ww = w4[i], kk = k4[i];
    e[4 * i] = fmaf(ww.x, S[4 * i], kk.x * v);
    e[4 * i + 1] = fmaf(ww.y, S[4 * i + 1], kk.y * v);
    e[4 * i + 2] = fmaf(ww.z, S[4 * i + 2], kk.z * v);
    e[4 * i + 3] = fmaf(ww.w, S[4 * i + 3], kk.w * v);
  }
#pragma unroll
  for (int o = 1; o < LANES; o <<= 1) us += __shfl_xor_sync(0xffffffffu, us, o);
  float a4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int i = 0; i < ROWS / 4; ++i) {
    const float4 bq = b4[i], rr = r4[i];
    S[4 * i] = fmaf(-bq.x, us, e[4 * i]);
    S[4 * i + 1] = fmaf(-bq.y, us, e[4 * i + 1]);
    S[4 * i + 2] = fmaf(-bq.z, us, e[4 * i + 2]);
    S[4 * i + 3] = fmaf(-bq.w, us, e[4 * i + 3]);
    a4[0] = fmaf(S[4 * i], rr.x, a4[0]);
    a4[1] = fmaf(S[4 * i + 1], rr.y, a4[1]);
    a4[2] = fmaf(S[4 * i + 2], rr.z, a4[2]);
    a4[3] = fmaf(S[4 * i + 3], rr.w, a4[3]);
  }
  float acc = (a4[0] + a4[1]) + (a4[2] + a4[3]);
#pragma unroll
  for (int o = 1; o < LANES; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  return acc;
}

template <int DMAX, int LANES, bool VEC>
__global__ void __launch_bounds__(DR_THREADS + 32)
delta_rule_kernel(const float *__restrict__ proj, long long ld, int off_r, int off_k, int off_v,
                  const float *__restrict__ prep, float *__restrict__ state, float *__restrict__ out, long long ldo,
                  const int *__restrict__ seq_start, const int *__restrict__ seq_slot, int n_heads, int d, int dv) {
  constexpr int ROWS = DMAX / LANES;                 // rows of a column held by one thread
  constexpr int COLS = DR_THREADS / LANES;           // columns of a CTA
  constexpr int PAD = ROWS + 4;                      // a lane's share of a vector, padded: the lanes' loads fall on different banks
  constexpr int VLEN = LANES * PAD;
  constexpr int SLOT = 5 * VLEN + COLS;              // floats of one token in the ring: w, b, u, k, r, then the CTA's columns of v
  constexpr int UNIT = VEC ? 4 : 1;                  // floats to a copy
  constexpr int PER = (5 * DMAX / UNIT + COLS / UNIT + 31) / 32;   // copies of a loader lane per token
  constexpr int DR_STAGES = DR_STAGES_MAX * SLOT * 4 <= 48 * 1024 ? DR_STAGES_MAX : DR_STAGES_MAX / 2;
  // Tokens go through the ring in groups of G: a group of copies is G tokens, DR_STAGES / G - 1 groups are in flight, and
  // a barrier stands before every group (its copies have arrived for everyone, and everyone is done with the group whose
  // place the next copies take).
  constexpr int G = DR_STAGES / 4;
  constexpr int GROUPS = DR_STAGES / G;
  __shared__ __align__(16) float ring[DR_STAGES][SLOT];
  grid_dependency_wait();
  const int b = blockIdx.x, hd = blockIdx.y;
  const int tid = threadIdx.x;
  const int j0 = blockIdx.z * COLS;
  const int start = seq_start[b], n = seq_start[b + 1] - start;
  const int n_groups = (n + G - 1) / G;
  // rows beyond d of a lane's share are never copied: they stay zero, and so do the state's rows there
  for (int i = tid; i < DR_STAGES * SLOT; i += DR_THREADS + 32) (&ring[0][0])[i] = 0.f;
  __syncthreads();

  if (tid >= DR_THREADS) {
    // ------------------------------------------------------------ the loader warp
    // Its lanes' copies of a token, worked out once: where from (an offset into the token's prepared vectors, or into
    // its row of the product, marked by bit 30) and where to (element i of a vector lies at (i / ROWS) * PAD + i % ROWS).
    const int lane = tid - DR_THREADS;
    int from[PER], to[PER];
    const int per_vec = d / UNIT, n_v = (min(COLS, dv - j0) + UNIT - 1) / UNIT;
#pragma unroll
    for (int e = 0; e < PER; ++e) {
      const int idx = lane + e * 32;
      from[e] = to[e] = -1;
      if (idx < 5 * per_vec) {
        const int which = idx / per_vec, i = (idx - which * per_vec) * UNIT;
        from[e] = which < 3 ? which * d + i : ((which == 3 ? off_k : off_r) + hd * d + i) | (1 << 30);
        to[e] = which * VLEN + (i / ROWS) * PAD + i % ROWS;
      } else if (idx - 5 * per_vec < n_v) {
        const int i = (idx - 5 * per_vec) * UNIT;
        from[e] = (off_v + hd * dv + j0 + i) | (1 << 30);
        to[e] = 5 * VLEN + i;
      }
    }
    auto fetch_group = [&](int p) {
      for (int t = G * p; t < min(n, G * p + G); ++t) {
        float *dst = ring[t % DR_STAGES];
        const float *row = proj + (size_t)(start + t) * ld;
        const float *pr = prep + ((size_t)(start + t) * n_heads + hd) * 3 * d;
#pragma unroll
        for (int e = 0; e < PER; ++e)
          if (to[e] >= 0) {
            const float *src = (from[e] & (1 << 30)) ? row + (from[e] & ~(1 << 30)) : pr + from[e];
            if (VEC) cp_async16_cg(dst + to[e], src);
            else cp_async4(dst + to[e], src);
          }
      }
      cp_async_commit_group();
    };
    for (int p = 0; p < GROUPS - 1; ++p) fetch_group(p);
    for (int p = 0; p < n_groups; ++p) {
      cp_async_wait_group<GROUPS - 2>();              // group p has arrived
      __syncthreads();                                // the other warps may read it; they are done with group p - 1
      fetch_group(p + GROUPS - 1);                    // ... whose place these copies take
    }
    cp_async_wait_group<0>();
    return;
  }

  // -------------------------------------------------------------- the two warps of the recurrence
  const int sub = tid % LANES, col = tid / LANES;
  const int j = j0 + col;
  const bool live = j < dv;
  float S[ROWS];
  float *sp = state + (((size_t)seq_slot[b] * n_heads + hd) * dv + (live ? j : 0)) * d + sub * ROWS;
#pragma unroll
  for (int i = 0; i < ROWS; ++i) S[i] = (live && sub * ROWS + i < d) ? sp[i] : 0.f;
  auto token = [&](int t) {
    const float *slot = ring[t % DR_STAGES];
    const float acc = delta_token<ROWS, LANES>(S, slot + sub * PAD, VLEN, slot[5 * VLEN + col]);
    if (live && sub == 0) out[(size_t)(start + t) * ldo + (size_t)hd * dv + j] = acc;
  };
  for (int p = 0; p < n_groups; ++p) {
    __syncthreads();
    if (G * p + G <= n) {
#pragma unroll
      for (int g = 0; g < G; ++g) token(G * p + g);
    } else {
      for (int t = G * p; t < n; ++t) token(t);
    }
  }
  // Only now may the next kernel's CTAs come onto the SMs: this kernel runs for as long as its longest sequence
  // with few warps to a CTA, and a dependent let in at the start would sit beside them in its wait for all that time.
  grid_dependents_launch();
  if (live)
#pragma unroll
    for (int i = 0; i < ROWS; ++i)
      if (sub * ROWS + i < d) sp[i] = S[i];
}

static int launch_delta_scan(const float *proj, long long ld, int off_r, int off_k, int off_v, const float *prep, float *state,
                             float *out, long long ldo, const int *seq_start, const int *seq_slot, int n_seqs, int n_heads, int d,
                             int dv, cudaStream_t stream) {
  // 16-byte copies where every vector starts on such a boundary
  const bool vec16 = d % 4 == 0 && dv % 4 == 0 && ld % 4 == 0 && off_r % 4 == 0 && off_k % 4 == 0 && off_v % 4 == 0 && (uintptr_t)proj % 16 == 0 &&
                     (uintptr_t)prep % 16 == 0;
  // Launched without the overlap attribute: the kernel before it (the preparation) is wide and short, this one narrow and
  // long; let in beside it, its CTAs took their places on the SMs early and a prompt step of 2,048 tokens took 9.8 ms
  // instead of 5.9 (measured).
#define DR_GO2(DMAX, LANES, VEC)                                                                                        \
  llm_launch_after(delta_rule_kernel<DMAX, LANES, VEC>, dim3(n_seqs, n_heads, (dv + DR_THREADS / LANES - 1) / (DR_THREADS / LANES)), \
                   dim3(DR_THREADS + 32), 0, stream, proj, ld, off_r, off_k, off_v, (const float *)prep, state, out, ldo, seq_start, \
                   seq_slot, n_heads, d, dv)
#define DR_GO(DMAX, LANES)              \
  do {                                  \
    if (vec16) DR_GO2(DMAX, LANES, true); \
    else DR_GO2(DMAX, LANES, false);    \
  } while (0)
  if (d <= 32) DR_GO(32, 2);
  else if (d <= 64) DR_GO(64, 4);
  else if (d <= 128) DR_GO(128, 4);
  else DR_GO(256, 8);
#undef DR_GO2
#undef DR_GO
  LLM_CHECK_LAUNCH("delta_rule");
  return LLM_OK;
}

LLM_EXPORT int llm_delta_rule(const float *proj, long long ld, int off_r, int off_k, int off_v, int off_a, int off_x1, int rank,
                              const float *w2, const float *w0, const float *a_bias, float decay_scale, float key_eps,
                              float *prep, float *state, float *out, long long ldo, const int *seq_start, const int *seq_slot,
                              int n_tokens, int n_seqs, int n_heads, int d, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_seqs > 0 && n_heads > 0 && d > 0 && rank > 0, "delta_rule: bad sizes");
  LLM_REQUIRE(d <= 256, "delta_rule: heads of %d channels are not supported (up to 256)", d);
  LLM_REQUIRE(n_heads <= 65535 && n_seqs < 2147483647, "delta_rule: too many heads or sequences");
  {
    const size_t with_w2 = ((size_t)DP_WARPS * rank + (size_t)d * (rank + 1)) * sizeof(float);
    const int w2_shared = with_w2 <= 96 * 1024;
    const size_t smem = w2_shared ? with_w2 : (size_t)DP_WARPS * rank * sizeof(float);
    LLM_REQUIRE(smem <= 96 * 1024, "delta_rule: a decay input of rank %d is not supported", rank);
    LLM_CHECK_CUDA(llm_allow_smem(delta_prepare_kernel, smem), "delta_prepare attribute");
    llm_launch(delta_prepare_kernel, dim3((unsigned)((n_tokens + DP_TOKENS - 1) / DP_TOKENS), n_heads), dim3(DP_WARPS * 32), smem, stream,
               proj, ld, off_k, off_a, off_x1, rank, w2, w0, a_bias, decay_scale, key_eps, n_tokens, n_heads, d, w2_shared, prep);
    LLM_CHECK_LAUNCH("delta_prepare");
  }
  return launch_delta_scan(proj, ld, off_r, off_k, off_v, prep, state, out, ldo, seq_start, seq_slot, n_seqs, n_heads, d, d, stream);
}

// The recurrence alone, for a mixer that prepares the tokens' vectors itself: rows `proj` (32-bit) hold r and k
// (heads x d each) and v (heads x dv), `prep` [tokens, heads, 3, d] holds w, b, u; state [slots, heads, dv, d].
LLM_EXPORT int llm_delta_scan(const float *proj, long long ld, int off_r, int off_k, int off_v, const float *prep, float *state,
                              float *out, long long ldo, const int *seq_start, const int *seq_slot, int n_tokens, int n_seqs,
                              int n_heads, int d, int dv, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_seqs > 0 && n_heads > 0 && d > 0 && dv > 0, "delta_scan: bad sizes");
  LLM_REQUIRE(d <= 256, "delta_scan: heads of %d key channels are not supported (up to 256)", d);
  LLM_REQUIRE(n_heads <= 65535 && n_seqs < 2147483647, "delta_scan: too many heads or sequences");
  return launch_delta_scan(proj, ld, off_r, off_k, off_v, prep, state, out, ldo, seq_start, seq_slot, n_seqs, n_heads, d, dv, stream);
}

// ---------------------------------------------------------------- the delta rule: a step of single tokens
// Everything between the stacked product and the output projection in one launch, a CTA per (sequence, head):
// the token's vectors (as delta_prepare_kernel makes them), the state's step (delta_token, the scan's own
// arithmetic, with all of the head's columns in this CTA), the norm over the head, its weight and the gate.
template <int DMAX, int LANES, typename TO>
__global__ void __launch_bounds__(DMAX *LANES)
delta_step_kernel(const float *__restrict__ proj, long long ld, int off_r, int off_k, int off_v, int off_g, int off_a, int off_x1,
                  int rank, const float *__restrict__ w2, const float *__restrict__ w0, const float *__restrict__ a_bias,
                  float decay_scale, float key_eps, const float *__restrict__ norm_w, float eps, float *__restrict__ state,
                  TO *__restrict__ out, long long ldo, const int *__restrict__ seq_slot, int n_heads, int d, int w2_shared) {
  constexpr int ROWS = DMAX / LANES, PAD = ROWS + 4, VLEN = LANES * PAD, THREADS = DMAX * LANES;
  __shared__ __align__(16) float vecs[5 * VLEN];
  __shared__ float vals[DMAX], outs[DMAX], red[2];
  extern __shared__ float th[];                       // tanh of the low-rank input, `rank` floats; then W2's rows of the head, [d][rank + 1]
  grid_dependents_launch();
  const int b = blockIdx.x, hd = blockIdx.y;
  const int tid = threadIdx.x, sub = tid % LANES, col = tid / LANES, lane = tid & 31, warp = tid >> 5;
  const bool live = col < d;
  for (int i = tid; i < 5 * VLEN; i += THREADS) vecs[i] = 0.f;
  float *w2s = th + rank;
  if (w2_shared) {                                    // weights: on their way before the step's own data is waited for
    const float *w2h = w2 + (size_t)hd * d * rank;
    for (int i = tid; i < d * rank; i += THREADS) w2s[(i / rank) * (rank + 1) + i % rank] = w2h[i];
  }
  grid_dependency_wait();
  const float *row = proj + (size_t)b * ld;
  const float *k = row + off_k + (size_t)hd * d;
  // this thread's share of its column of the state: on its way while the vectors are made
  float S[ROWS];
  float *sp = state + (((size_t)seq_slot[b] * n_heads + hd) * d + (live ? col : 0)) * d + sub * ROWS;
#pragma unroll
  for (int i = 0; i < ROWS; ++i) S[i] = (live && sub * ROWS + i < d) ? sp[i] : 0.f;
  for (int q = tid; q < rank; q += THREADS) th[q] = tanhf(row[off_x1 + q]);
  if (warp == 0) {                                    // the key's length: lane order, then the shuffle tree
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) ss = fmaf(k[i], k[i], ss);
    ss = warp_sum(ss);
    if (lane == 0) red[0] = 1.f / sqrtf(ss + key_eps);
  }
  __syncthreads();
  if (tid < d) {
    const int i = tid, ch = hd * d + i;
    float z = w0[ch];
    const float *w2r = w2_shared ? w2s + i * (rank + 1) : w2 + (size_t)ch * rank;
    for (int q = 0; q < rank; ++q) z = fmaf(w2r[q], th[q], z);
    const float u = k[i] * red[0];
    const float a = 1.f / (1.f + expf(-(row[off_a + ch] + a_bias[ch])));
    const int at = (i / ROWS) * PAD + i % ROWS;
    vecs[at] = expf(-decay_scale / (1.f + expf(-z)));
    vecs[VLEN + at] = a * u;
    vecs[2 * VLEN + at] = u;
    vecs[3 * VLEN + at] = k[i];
    vecs[4 * VLEN + at] = row[off_r + ch];
    vals[i] = row[off_v + ch];
  }
  __syncthreads();
  const float acc = delta_token<ROWS, LANES>(S, vecs + sub * PAD, VLEN, live ? vals[col] : 0.f);
  if (live) {
#pragma unroll
    for (int i = 0; i < ROWS; ++i)
      if (sub * ROWS + i < d) sp[i] = S[i];
    if (sub == 0) outs[col] = acc;
  }
  __syncthreads();
  if (warp == 0) {
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) ss = fmaf(outs[i], outs[i], ss);
    ss = warp_sum(ss);
    if (lane == 0) red[1] = 1.f / sqrtf(ss / (float)d + eps);
  }
  __syncthreads();
  if (tid < d) {
    const int ch = hd * d + tid;
    const float g = row[off_g + ch];
    out[(size_t)b * ldo + ch] = from_float<TO>(outs[tid] * red[1] * norm_w[ch] / (1.f + expf(-g)));
  }
}

// 1 if a step of single tokens with heads of d channels has a kernel of its own.
LLM_EXPORT int llm_delta_step_supports(int d) { return d <= 128; }

LLM_EXPORT int llm_delta_step(const float *proj, long long ld, int off_r, int off_k, int off_v, int off_g, int off_a, int off_x1,
                              int rank, const float *w2, const float *w0, const float *a_bias, float decay_scale, float key_eps,
                              const float *norm_w, float eps, float *state, void *out, int out_dtype, long long ldo,
                              const int *seq_slot, int n_seqs, int n_heads, int d, cudaStream_t stream) {
  if (n_seqs == 0) return LLM_OK;
  LLM_REQUIRE(n_seqs > 0 && n_heads > 0 && d > 0 && rank > 0 && llm_delta_step_supports(d), "delta_step: bad sizes");
  LLM_REQUIRE(n_heads <= 65535, "delta_step: too many heads");
  const size_t with_w2 = ((size_t)rank + (size_t)d * (rank + 1)) * sizeof(float);
  const int w2_shared = with_w2 <= 64 * 1024;
  const size_t smem = w2_shared ? with_w2 : (size_t)rank * sizeof(float);
  LLM_REQUIRE(smem <= 64 * 1024, "delta_step: a decay input of rank %d is not supported", rank);
#define DS_GO(DMAX, LANES, TO)                                                                                          \
  do {                                                                                                                  \
    LLM_CHECK_CUDA(llm_allow_smem(delta_step_kernel<DMAX, LANES, TO>, smem), "delta_step attribute");                   \
    llm_launch(delta_step_kernel<DMAX, LANES, TO>, dim3(n_seqs, n_heads), dim3(DMAX * LANES), smem, stream, proj, ld, off_r, off_k, \
               off_v, off_g, off_a, off_x1, rank, w2, w0, a_bias, decay_scale, key_eps, norm_w, eps, state, (TO *)out, ldo, seq_slot, \
               n_heads, d, w2_shared);                                                                                  \
  } while (0)
#define DS_SIZES(TO)                     \
  do {                                   \
    if (d <= 32) DS_GO(32, 2, TO);       \
    else if (d <= 64) DS_GO(64, 4, TO);  \
    else DS_GO(128, 4, TO);              \
  } while (0)
  if (out_dtype == LLM_F32) DS_SIZES(float);
  else if (out_dtype == LLM_BF16) DS_SIZES(__nv_bfloat16);
  else LLM_FAIL("delta_step: unknown dtype %d", out_dtype);
#undef DS_SIZES
#undef DS_GO
  LLM_CHECK_LAUNCH("delta_step");
  return LLM_OK;
}

// ---------------------------------------------------------------- norm per head, weight, gate
// out[t, h, :] = x[t, h, :] / sqrt(mean(x[t, h, :]^2) + eps) * weight[h, :] * sigmoid(gate[t, h, :])
// eps < 0: no norm; weight null: none; gate null: none (gate: 32-bit logits, row stride gate_stride).
// One warp per (token, head).
template <typename T, bool VEC>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float *__restrict__ x, long long ldx, const float *__restrict__ weight, const float *__restrict__ gate,
                      long long gate_stride, float eps, int n_tokens, int n_heads, int dv, T *__restrict__ out, long long ldo) {
  grid_dependents_launch();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= (long long)n_tokens * n_heads) return;
  const int t = (int)(item / n_heads), hd = (int)(item - (long long)t * n_heads);
  const float *xr = x + (size_t)t * ldx + (size_t)hd * dv;
  const float *wr = weight ? weight + (size_t)hd * dv : nullptr;
  const float *gr = gate ? gate + (size_t)t * gate_stride + (size_t)hd * dv : nullptr;
  T *orow = out + (size_t)t * ldo + (size_t)hd * dv;
  if (VEC) {                                          // four channels to a lane: widths in multiples of 4, rows on 16 bytes
    float4 v[2];                                      // heads of up to 256 channels
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int i = (lane + 32 * r) * 4;
      v[r] = i < dv ? ld4(xr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      ss = fmaf(v[r].x, v[r].x, ss);
      ss = fmaf(v[r].y, v[r].y, ss);
      ss = fmaf(v[r].z, v[r].z, ss);
      ss = fmaf(v[r].w, v[r].w, ss);
    }
    // the weight's and the gate's loads are on their way while the sum is taken
    float4 w4[2], g4[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int i = (lane + 32 * r) * 4;
      w4[r] = (wr && i < dv) ? ld4(wr + i) : make_float4(1.f, 1.f, 1.f, 1.f);
      g4[r] = (gr && i < dv) ? ld4(gr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float inv = 1.f;
    if (eps >= 0.f) inv = 1.f / sqrtf(warp_sum(ss) / (float)dv + eps);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int i = (lane + 32 * r) * 4;
      if (i >= dv) continue;
      float4 y = make_float4(v[r].x * inv * w4[r].x, v[r].y * inv * w4[r].y, v[r].z * inv * w4[r].z, v[r].w * inv * w4[r].w);
      if (gr)
        y = make_float4(y.x / (1.f + expf(-g4[r].x)), y.y / (1.f + expf(-g4[r].y)), y.z / (1.f + expf(-g4[r].z)),
                        y.w / (1.f + expf(-g4[r].w)));
      st4(orow + i, y);
    }
    return;
  }
  float inv = 1.f;
  if (eps >= 0.f) {
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) ss = fmaf(xr[i], xr[i], ss);
    ss = warp_sum(ss);
    inv = 1.f / sqrtf(ss / (float)dv + eps);
  }
  for (int i = lane; i < dv; i += 32) {
    float v = xr[i] * inv;
    if (wr) v *= wr[i];
    if (gr) v *= 1.f / (1.f + expf(-gr[i]));
    orow[i] = from_float<T>(v);
  }
}

LLM_EXPORT int llm_head_norm_gate(const float *x, long long ldx, const float *weight, const float *gate, long long gate_stride,
                                  float eps, int n_tokens, int n_heads, int dv, void *out, int out_dtype, long long ldo,
                                  cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_heads > 0 && dv > 0 && x && out, "head_norm_gate: bad arguments");
  const long long items = (long long)n_tokens * n_heads;
  const dim3 grid((unsigned)((items + 3) / 4));
  const bool vec = dv % 4 == 0 && dv <= 256 && ldx % 4 == 0 && ldo % 4 == 0 && gate_stride % 4 == 0 && (uintptr_t)x % 16 == 0 &&
                   (uintptr_t)weight % 16 == 0 && (uintptr_t)gate % 16 == 0 && (uintptr_t)out % 16 == 0;
#define HNG_GO(T, VEC)                                                                                                  \
  llm_launch(head_norm_gate_kernel<T, VEC>, grid, dim3(128), 0, stream, x, ldx, weight, gate, gate_stride, eps, n_tokens, n_heads, dv, \
             (T *)out, ldo)
  if (out_dtype == LLM_F32 && vec) HNG_GO(float, true);
  else if (out_dtype == LLM_F32) HNG_GO(float, false);
  else if (out_dtype == LLM_BF16 && vec) HNG_GO(__nv_bfloat16, true);
  else if (out_dtype == LLM_BF16) HNG_GO(__nv_bfloat16, false);
  else LLM_FAIL("head_norm_gate: unknown dtype %d", out_dtype);
#undef HNG_GO
  LLM_CHECK_LAUNCH("head_norm_gate");
  return LLM_OK;
}

// ---------------------------------------------------------------- the gated delta rule with a decay per key channel
// Per head, state S [d keys x dv values], in this order:
//   S <- diag(g) S;  e = beta (v - S^T k);  S <- S + k e^T;  o = S^T q.
// With w = g, u = g * k (so that u^T S_old = k^T diag(g) S_old), b = beta k and the key that is learned beta k, this is
//   S <- diag(w) S - b (u^T S) + (beta k) v^T     (both terms read the old S),
// the recurrence of delta_rule_kernel.  This kernel makes a token's vectors from the convolved projections:
//   rows `cv` (32-bit) [q (kv_heads x d) | k (kv_heads x d) | v (heads x dv) | room for r (heads x d) | room for k (heads x d)],
//   q and k made unit vectors per kv head (x / sqrt(sum x^2 + key_eps)), q also times d^(-1/2); head h reads kv head
//   h / (heads / kv_heads);  beta = sigmoid(proj[off_b + h]);
//   g = exp(-exp(a_log[h]) * softplus(a2 x1 + dt_bias)), x1 = proj[off_a1 ...] (rank_a values), a2 [heads * d, rank_a];
//   prep [tokens, heads, 3, d] = w, b, u;  r and beta k into their room of the row;
//   gate [tokens, heads * dv] = g2 x2, x2 = proj[off_g1 ...] (rank_g values), g2 [heads * dv, rank_g]  (logits; the sigmoid is the
//   norm kernel's).
// A CTA takes CD_TT tokens and CD_THREADS channels (blockIdx.y counts the runs of channels): a row of a2 or g2 is read
// once for the CTA's tokens.  Every sum runs in the same order (lanes, then the shuffle tree; the ranks ascending)
// whatever the batch and the grouping.
constexpr int CD_THREADS = 256;
constexpr int CD_TT = 4;
__device__ __forceinline__ float softplus32(float x) { return x > 20.f ? x : log1pf(expf(x)); }

__global__ void __launch_bounds__(CD_THREADS)
channel_delta_prepare_kernel(float *__restrict__ cv, long long ldc, const float *__restrict__ proj, long long ld, int off_b, int off_a1,
                             int rank_a, int off_g1, int rank_g, const float *__restrict__ a2, const float *__restrict__ dt_bias,
                             const float *__restrict__ a_log, const float *__restrict__ g2, float key_eps, float *__restrict__ prep,
                             float *__restrict__ gate, int n_tokens, int n_heads, int n_kv, int d, int dv) {
  extern __shared__ float cd_sm[];                     // x1 [TT][rank_a] | x2 [TT][rank_g] | inv_q [TT][n_kv] | inv_k [TT][n_kv]
  float *x1 = cd_sm, *x2 = x1 + CD_TT * rank_a, *inv_q = x2 + CD_TT * rank_g, *inv_k = inv_q + CD_TT * n_kv;
  grid_dependents_launch();
  grid_dependency_wait();
  const int t0 = blockIdx.x * CD_TT, nt = min(CD_TT, n_tokens - t0);
  for (int i = threadIdx.x; i < CD_TT * rank_a; i += CD_THREADS) {
    const int tt = i / rank_a;
    x1[i] = tt < nt ? proj[(size_t)(t0 + tt) * ld + off_a1 + (i - tt * rank_a)] : 0.f;
  }
  for (int i = threadIdx.x; i < CD_TT * rank_g; i += CD_THREADS) {
    const int tt = i / rank_g;
    x2[i] = tt < nt ? proj[(size_t)(t0 + tt) * ld + off_g1 + (i - tt * rank_g)] : 0.f;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int item = warp; item < nt * 2 * n_kv; item += CD_THREADS / 32) {   // per token: q heads, then k heads
    const int tt = item / (2 * n_kv), which = item - tt * 2 * n_kv;
    const float *x = cv + (size_t)(t0 + tt) * ldc + (size_t)which * d;
    float ss = 0.f;
    for (int c = lane; c < d; c += 32) ss = fmaf(x[c], x[c], ss);
    ss = warp_sum(ss);
    if (lane == 0) {
      if (which < n_kv) inv_q[tt * n_kv + which] = rsqrtf(ss + key_eps) * rsqrtf((float)d);
      else inv_k[tt * n_kv + which - n_kv] = rsqrtf(ss + key_eps);
    }
  }
  __syncthreads();
  const int group = n_heads / n_kv;
  const int off_v = 2 * n_kv * d, off_r = off_v + n_heads * dv, off_k = off_r + n_heads * d;
  const int i = blockIdx.y * CD_THREADS + threadIdx.x;
  if (i < n_heads * d) {
    const int h = i / d, c = i - h * d, g = h / group;
    const float *a = a2 + (size_t)i * rank_a;
    float s[CD_TT];
#pragma unroll
    for (int tt = 0; tt < CD_TT; ++tt) s[tt] = 0.f;
    for (int j = 0; j < rank_a; ++j) {
      const float av = a[j];
#pragma unroll
      for (int tt = 0; tt < CD_TT; ++tt) s[tt] = fmaf(av, x1[tt * rank_a + j], s[tt]);
    }
    const float rate = -expf(a_log[h]), bias = dt_bias[i];
#pragma unroll
    for (int tt = 0; tt < CD_TT; ++tt) {
      if (tt < nt) {
        float *row = cv + (size_t)(t0 + tt) * ldc;
        const float q = row[g * d + c] * inv_q[tt * n_kv + g];
        const float k = row[(n_kv + g) * d + c] * inv_k[tt * n_kv + g];
        const float beta = 1.f / (1.f + expf(-proj[(size_t)(t0 + tt) * ld + off_b + h]));
        const float w = expf(rate * softplus32(s[tt] + bias));
        float *p = prep + ((size_t)(t0 + tt) * n_heads + h) * 3 * d;
        p[c] = w;
        p[d + c] = beta * k;
        p[2 * d + c] = w * k;
        row[off_r + i] = q;
        row[off_k + i] = beta * k;
      }
    }
  }
  if (i < n_heads * dv) {
    const float *a = g2 + (size_t)i * rank_g;
    float s[CD_TT];
#pragma unroll
    for (int tt = 0; tt < CD_TT; ++tt) s[tt] = 0.f;
    for (int j = 0; j < rank_g; ++j) {
      const float av = a[j];
#pragma unroll
      for (int tt = 0; tt < CD_TT; ++tt) s[tt] = fmaf(av, x2[tt * rank_g + j], s[tt]);
    }
#pragma unroll
    for (int tt = 0; tt < CD_TT; ++tt)
      if (tt < nt) gate[(size_t)(t0 + tt) * n_heads * dv + i] = s[tt];
  }
}

LLM_EXPORT int llm_channel_delta_prepare(float *cv, long long ldc, const float *proj, long long ld, int off_b, int off_a1, int rank_a,
                                         int off_g1, int rank_g, const float *a2, const float *dt_bias, const float *a_log,
                                         const float *g2, float key_eps, float *prep, float *gate, int n_tokens, int n_heads, int n_kv,
                                         int d, int dv, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv > 0 && n_heads % n_kv == 0 && d > 0 && dv > 0 && rank_a > 0 && rank_g > 0,
              "channel_delta_prepare: bad sizes");
  LLM_REQUIRE(ldc >= 2LL * n_kv * d + (long long)n_heads * dv + 2LL * n_heads * d, "channel_delta_prepare: rows too short");
  const size_t smem = (size_t)CD_TT * (rank_a + rank_g + 2 * n_kv) * sizeof(float);
  LLM_REQUIRE(smem <= 96 * 1024, "channel_delta_prepare: low-rank inputs of %d and %d values are not supported", rank_a, rank_g);
  LLM_CHECK_CUDA(llm_allow_smem(channel_delta_prepare_kernel, smem), "channel_delta_prepare attribute");
  const int widest = n_heads * (d > dv ? d : dv);
  llm_launch(channel_delta_prepare_kernel, dim3((n_tokens + CD_TT - 1) / CD_TT, (widest + CD_THREADS - 1) / CD_THREADS), dim3(CD_THREADS), smem,
             stream, cv, ldc, proj, ld, off_b, off_a1, rank_a, off_g1, rank_g, a2, dt_bias, a_log, g2, key_eps, prep, gate, n_tokens, n_heads,
             n_kv, d, dv);
  LLM_CHECK_LAUNCH("channel_delta_prepare");
  return LLM_OK;
}
