// Embedding gather, residual-add + RMSNorm, and SwiGLU.  Element type T is float (the
// true 32-bit path) or bfloat16; all arithmetic is in 32-bit.
//
// Reference counterparts: lookup (src/flint/cuda/lookup.cu:30-43), rmsNorm
// (src/flint/cuda/rms_norm.cu:31-84) followed by a separate add
// (src/flint/cuda/binary.cu:48-88), swiglu (src/flint/cuda/swiglu.cu:29-59).  Here the
// residual stream is kept in 32-bit and the add is part of the norm kernel, so one
// pass over the row does what three launches do there.
#include "common.cuh"

LLM_DEFINE_LAST_ERROR(llm_elementwise_last_error)

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embedding_kernel(const T *__restrict__ table, const int *__restrict__ tokens,
                                 const int *__restrict__ fed_tokens, const int *__restrict__ fed_rows,
                                 float *__restrict__ out, int hidden, int vocab, const T *__restrict__ pos_table,
                                 int pos_rows, const int *__restrict__ tok_pos) {
  grid_dependents_launch();
  grid_dependency_wait();
  const int t = blockIdx.x;
  // A token either comes with the step (tokens[t]) or is the one the previous step sampled for
  // row fed_rows[t] of its batch, still on the device (fed_tokens): the host can then start this
  // step before it has read that token back.
  int id = tokens[t];
  if (fed_rows != nullptr && fed_rows[t] >= 0) id = fed_tokens[fed_rows[t]];
  // Token ids are checked on the host before they are uploaded; ids that the sampler
  // wrote on the device are below the vocabulary size by construction.  The clamp keeps
  // the read inside the table whatever happens.
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const T *row = table + (size_t)id * hidden;
  float *o = out + (size_t)t * hidden;
  if (pos_table == nullptr) {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_float(row[i]);
    return;
  }
  // a learned vector per position is added to the token's row (32-bit sum of the two stored values)
  int p = tok_pos[t];
  p = p < 0 ? 0 : (p >= pos_rows ? pos_rows - 1 : p);      // the host refuses sequences longer than the table
  const T *prow = pos_table + (size_t)p * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_float(row[i]) + to_float(prow[i]);
}

// pos_table [pos_rows, hidden] in the table's type with the tokens' positions tok_pos, or null: no position vectors.
LLM_EXPORT int llm_embedding_pos(int dtype, const void *table, const int *tokens, const int *fed_tokens,
                                 const int *fed_rows, float *out, int n_tokens, int hidden, int vocab,
                                 const void *pos_table, int pos_rows, const int *tok_pos, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && hidden > 0 && vocab > 0, "embedding: bad sizes");
  LLM_REQUIRE(pos_table == nullptr || (pos_rows > 0 && tok_pos != nullptr), "embedding: position vectors come with the positions");
  LLM_REQUIRE((fed_tokens == nullptr) == (fed_rows == nullptr), "embedding: fed tokens come with their rows");
  int threads = hidden >= 1024 ? 256 : 128;
  // A step's first kernel after its descriptor has arrived, and launched so that it starts only
  // when that is complete: the kernels after it read positions and page tables from the descriptor
  // before they wait for their own predecessors, which is safe because none of them can start before
  // this one has.  (Inside a single-token step's graph the descriptor comes by a kernel just before
  // this one; with an overlapping launch here, a later kernel could in rare runs read the positions
  // of the step before last.)
  if (dtype == LLM_F32)
    llm_launch_after(embedding_kernel<float>, n_tokens, threads, 0, stream, (const float *)table, tokens, fed_tokens, fed_rows, out, hidden, vocab,
                     (const float *)pos_table, pos_rows, tok_pos);
  else if (dtype == LLM_BF16)
    llm_launch_after(embedding_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, (const __nv_bfloat16 *)table, tokens, fed_tokens, fed_rows, out, hidden, vocab,
                     (const __nv_bfloat16 *)pos_table, pos_rows, tok_pos);
  else
    LLM_FAIL("embedding: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("embedding");
  return LLM_OK;
}

LLM_EXPORT int llm_embedding(int dtype, const void *table, const int *tokens, const int *fed_tokens,
                             const int *fed_rows, float *out, int n_tokens, int hidden, int vocab,
                             cudaStream_t stream) {
  return llm_embedding_pos(dtype, table, tokens, fed_tokens, fed_rows, out, n_tokens, hidden, vocab, nullptr, 0, nullptr, stream);
}

// ---------------------------------------------------------------- small copies as kernels
// n 32-bit words from src to dst, either of which may be pinned host memory (which the device
// reaches by the same address).  A step's descriptor comes in and its tokens go out this way inside
// the step's graph: a copy of the copy engine there costs 8 to 15 us of hand-over on either side,
// a kernel two or three.
// The kernels behind it may start only when the words are written: later kernels of a step read
// the descriptor before they wait for their predecessors.
__global__ void copy_words_kernel(const int *__restrict__ src, int *__restrict__ dst, int n) {
  grid_dependency_wait();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) dst[i] = src[i];
  __threadfence();
  grid_dependents_launch();
}

LLM_EXPORT int llm_copy_words(const int *src, int *dst, int n, cudaStream_t stream) {
  if (n == 0) return LLM_OK;
  LLM_REQUIRE(n > 0 && src != nullptr && dst != nullptr, "copy_words: bad arguments");
  const int blocks = n <= 1024 ? 1 : (n + 1023) / 1024 > 64 ? 64 : (n + 1023) / 1024;
  llm_launch(copy_words_kernel, blocks, n < 256 ? 64 : 256, 0, stream, src, dst, n);
  LLM_CHECK_LAUNCH("copy_words");
  return LLM_OK;
}

// n1 words from src1 followed by n2 words from src2, to dst (which may be pinned host memory): a
// step's sampled tokens and the status word of its tensor-core kernels leave the device together.
__global__ void gather_words_kernel(const int *__restrict__ src1, int n1, const int *__restrict__ src2, int n2,
                                    int *__restrict__ dst) {
  grid_dependency_wait();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n1 + n2; i += gridDim.x * blockDim.x)
    dst[i] = i < n1 ? src1[i] : src2[i - n1];
  __threadfence_system();
  grid_dependents_launch();
}

LLM_EXPORT int llm_gather_words(const int *src1, int n1, const int *src2, int n2, int *dst, cudaStream_t stream) {
  if (n1 + n2 == 0) return LLM_OK;
  LLM_REQUIRE(n1 >= 0 && n2 >= 0 && dst != nullptr && (n1 == 0 || src1) && (n2 == 0 || src2), "gather_words: bad arguments");
  const int n = n1 + n2;
  const int blocks = n <= 1024 ? 1 : (n + 1023) / 1024 > 64 ? 64 : (n + 1023) / 1024;
  llm_launch(gather_words_kernel, blocks, n < 256 ? 64 : 256, 0, stream, src1, n1, src2, n2, dst);
  LLM_CHECK_LAUNCH("gather_words");
  return LLM_OK;
}

// ---------------------------------------------------------------- add + rmsnorm
// For each output row i (source row r = rows ? rows[i] : i):
//   v = resid[r] + sum_p delta[p][r]      (32-bit; parts added in index order)
//       with col_scale / col_bias (vectors over the columns, either may be null):
//       v = resid[r] + (sum_p delta[p][r] + col_bias) * col_scale
//   if (!rows) resid[r] = v               (the residual stream moves on)
//   out[i] = v * w * rsqrt(mean(v^2) + eps)   (skipped when out is null)
template <typename TD, typename TO, int THREADS>
__global__ void add_rmsnorm_kernel(float *__restrict__ resid, const TD *__restrict__ delta,
                                   int n_parts, size_t part_stride, const float *__restrict__ weight,
                                   float eps, TO *__restrict__ out, const int *__restrict__ rows,
                                   int hidden, const float *__restrict__ col_scale,
                                   const float *__restrict__ col_bias) {
  extern __shared__ float row_buf[];   // hidden floats
  __shared__ float scratch[THREADS / 32 + 1];
  grid_dependents_launch();
  grid_dependency_wait();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float *x = resid + (size_t)r * hidden;
  float ss = 0.f;
  for (int c = threadIdx.x; c < hidden; c += THREADS) {
    float v = x[c];
    if (col_scale || col_bias) {
      float d = 0.f;
      for (int p = 0; p < n_parts; ++p) d += to_float(delta[p * part_stride + (size_t)r * hidden + c]);
      if (col_bias) d += col_bias[c];
      if (col_scale) d *= col_scale[c];
      if (n_parts > 0) v += d;
    } else {
      for (int p = 0; p < n_parts; ++p) v += to_float(delta[p * part_stride + (size_t)r * hidden + c]);
    }
    row_buf[c] = v;
    if (!rows && n_parts > 0) x[c] = v;
    ss += v * v;
  }
  if (!out) return;
  const float total = block_sum<THREADS>(ss, scratch);
  const float inv = rsqrtf(total / (float)hidden + eps);
  TO *o = out + (size_t)i * hidden;
  for (int c = threadIdx.x; c < hidden; c += THREADS) o[c] = from_float<TO>(row_buf[c] * weight[c] * inv);
}

// The same for rows whose width is a multiple of 4 and at most 4 * VPT * THREADS, with up
// to MAXP parts: every thread issues all its loads (the row, every part, the weight) before
// it uses one, so the kernel waits for memory once and not once per part.  The values,
// the order of the additions and the order of the sum of squares within a thread differ
// from the general kernel's only in which thread owns which columns; like it, a row's
// result does not depend on the other rows of the launch.
template <typename TD, typename TO, int THREADS, int VPT, int MAXP>
__global__ void __launch_bounds__(THREADS)
add_rmsnorm_vec_kernel(float *__restrict__ resid, const TD *__restrict__ delta, int n_parts,
                       size_t part_stride, const float *__restrict__ weight, float eps,
                       TO *__restrict__ out, const int *__restrict__ rows, int hidden,
                       const float *__restrict__ col_scale, const float *__restrict__ col_bias) {
  __shared__ float scratch[THREADS / 32 + 1];
  grid_dependents_launch();
  const int i = blockIdx.x;
  const int n4 = hidden / 4;
  const bool scaled = col_scale || col_bias;
  float4 v[VPT], w[VPT], d[VPT][MAXP], cs[VPT], cb[VPT];
  if (out) {                             // the norm's weight does not depend on the kernel before
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int c4 = threadIdx.x + j * THREADS;
      if (c4 < n4) w[j] = ld4(weight + 4 * c4);
    }
  }
  if (scaled) {                          // weights too
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int c4 = threadIdx.x + j * THREADS;
      cs[j] = (col_scale && c4 < n4) ? ld4(col_scale + 4 * c4) : make_float4(1.f, 1.f, 1.f, 1.f);
      cb[j] = (col_bias && c4 < n4) ? ld4(col_bias + 4 * c4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  grid_dependency_wait();
  const int r = rows ? rows[i] : i;
  float *x = resid + (size_t)r * hidden;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int c4 = threadIdx.x + j * THREADS;
    if (c4 < n4) {
      v[j] = ld4(x + 4 * c4);
#pragma unroll
      for (int p = 0; p < MAXP; ++p)
        if (p < n_parts) d[j][p] = ld4(delta + p * part_stride + (size_t)r * hidden + 4 * c4);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int c4 = threadIdx.x + j * THREADS;
    if (c4 < n4) {
      if (scaled && n_parts > 0) {         // the parts' sum first, then bias and scale, then the stream
        float4 t = d[j][0];
#pragma unroll
        for (int p = 1; p < MAXP; ++p)
          if (p < n_parts) {
            t.x += d[j][p].x;
            t.y += d[j][p].y;
            t.z += d[j][p].z;
            t.w += d[j][p].w;
          }
        v[j].x += (t.x + cb[j].x) * cs[j].x;
        v[j].y += (t.y + cb[j].y) * cs[j].y;
        v[j].z += (t.z + cb[j].z) * cs[j].z;
        v[j].w += (t.w + cb[j].w) * cs[j].w;
      } else {
#pragma unroll
        for (int p = 0; p < MAXP; ++p)
          if (p < n_parts) {
            v[j].x += d[j][p].x;
            v[j].y += d[j][p].y;
            v[j].z += d[j][p].z;
            v[j].w += d[j][p].w;
          }
      }
      if (!rows && n_parts > 0) st4(x + 4 * c4, v[j]);
      ss += v[j].x * v[j].x;
      ss += v[j].y * v[j].y;
      ss += v[j].z * v[j].z;
      ss += v[j].w * v[j].w;
    }
  }
  if (!out) return;
  const float total = block_sum<THREADS>(ss, scratch);
  const float inv = rsqrtf(total / (float)hidden + eps);
  TO *o = out + (size_t)i * hidden;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int c4 = threadIdx.x + j * THREADS;
    if (c4 < n4)
      st4(o + 4 * c4, make_float4(v[j].x * w[j].x * inv, v[j].y * w[j].y * inv, v[j].z * w[j].z * inv,
                                  v[j].w * w[j].w * inv));
  }
}

template <typename TD, typename TO>
static int launch_add_rmsnorm(float *resid, const void *delta, int n_parts, size_t part_stride,
                              const float *weight, float eps, void *out, const int *rows, int n_rows,
                              int hidden, cudaStream_t stream, const float *col_scale = nullptr,
                              const float *col_bias = nullptr) {
  constexpr int THREADS = 256;
  constexpr int VPT = 4;
  const bool aligned = hidden % 4 == 0 && (uintptr_t)resid % 16 == 0 && (uintptr_t)delta % 16 == 0 &&
                       (uintptr_t)weight % 16 == 0 && (uintptr_t)out % 16 == 0 && part_stride % 4 == 0 &&
                       (uintptr_t)col_scale % 16 == 0 && (uintptr_t)col_bias % 16 == 0;
  if (aligned && hidden <= 4 * VPT * THREADS && n_parts <= 16) {
    // one instantiation per bound on the parts: registers for eight parts cost a prompt step
    // (one part, thousands of rows) a third of its speed
    // A thread per four columns where the row allows it (up to 4,096 columns): with many parts the
    // loads of a row are in flight from more warps at once.
#define ADDNORM_GO2(T_, V_, MAXP)                                                                        \
  llm_launch(add_rmsnorm_vec_kernel<TD, TO, T_, V_, MAXP>, n_rows, T_, 0, stream, resid,                 \
             (const TD *)delta, n_parts, part_stride, weight, eps, (TO *)out, rows, hidden, col_scale,   \
             col_bias)
#define ADDNORM_GO(MAXP)                                                                                 \
  do {                                                                                                   \
    if (hidden <= 2048) ADDNORM_GO2(512, 1, MAXP);                                                       \
    else if (hidden <= 4096) ADDNORM_GO2(1024, 1, MAXP);                                                 \
    else ADDNORM_GO2(THREADS, VPT, MAXP);                                                                \
  } while (0)
    if (n_parts <= 1) ADDNORM_GO(1);
    else if (n_parts <= 4) ADDNORM_GO(4);
    else if (n_parts <= 8) ADDNORM_GO(8);
    else ADDNORM_GO(16);                   // a mixer's and a feed-forward's parts together (a parallel block)
#undef ADDNORM_GO
#undef ADDNORM_GO2
    LLM_CHECK_LAUNCH("add_rmsnorm");
    return LLM_OK;
  }
  size_t smem = (size_t)hidden * sizeof(float);
  auto kern = add_rmsnorm_kernel<TD, TO, THREADS>;
  if (smem > 48 * 1024) {
    LLM_REQUIRE(smem <= 200 * 1024, "add_rmsnorm: a row of %d values does not fit shared memory", hidden);
    LLM_CHECK_CUDA(llm_allow_smem(kern, smem), "add_rmsnorm attribute");
  }
  llm_launch(kern, n_rows, THREADS, smem, stream, resid, (const TD *)delta, n_parts, part_stride, weight, eps,
             (TO *)out, rows, hidden, col_scale, col_bias);
  LLM_CHECK_LAUNCH("add_rmsnorm");
  return LLM_OK;
}

// With a scale and a bias over the columns (either may be null) on what is added.
// delta_dtype: type of delta; out_dtype: type of out.  delta may be null (n_parts 0),
// out may be null (add only), rows may be null (all rows, residual written back).
LLM_EXPORT int llm_add_rmsnorm_scaled(float *resid, const void *delta, int delta_dtype, int n_parts,
                               long long part_stride, const float *weight, float eps, void *out,
                               int out_dtype, const int *rows, int n_rows, int hidden,
                               const float *col_scale, const float *col_bias, cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE(n_rows > 0 && hidden > 0 && n_parts >= 0, "add_rmsnorm: bad sizes");
  LLM_REQUIRE(out == nullptr || weight != nullptr, "add_rmsnorm: a norm needs its weight");
  if (!delta) n_parts = 0;
  if (delta_dtype == LLM_F32 && out_dtype == LLM_F32)
    return launch_add_rmsnorm<float, float>(resid, delta, n_parts, part_stride, weight, eps, out, rows, n_rows, hidden, stream, col_scale, col_bias);
  if (delta_dtype == LLM_F32 && out_dtype == LLM_BF16)
    return launch_add_rmsnorm<float, __nv_bfloat16>(resid, delta, n_parts, part_stride, weight, eps, out, rows, n_rows, hidden, stream, col_scale, col_bias);
  if (delta_dtype == LLM_BF16 && out_dtype == LLM_BF16)
    return launch_add_rmsnorm<__nv_bfloat16, __nv_bfloat16>(resid, delta, n_parts, part_stride, weight, eps, out, rows, n_rows, hidden, stream, col_scale, col_bias);
  if (delta_dtype == LLM_BF16 && out_dtype == LLM_F32)
    return launch_add_rmsnorm<__nv_bfloat16, float>(resid, delta, n_parts, part_stride, weight, eps, out, rows, n_rows, hidden, stream, col_scale, col_bias);
  LLM_FAIL("add_rmsnorm: unknown dtypes %d, %d", delta_dtype, out_dtype);
}

// ---------------------------------------------------------------- add + layer norm
LLM_EXPORT int llm_add_rmsnorm(float *resid, const void *delta, int delta_dtype, int n_parts,
                               long long part_stride, const float *weight, float eps, void *out,
                               int out_dtype, const int *rows, int n_rows, int hidden,
                               cudaStream_t stream) {
  return llm_add_rmsnorm_scaled(resid, delta, delta_dtype, n_parts, part_stride, weight, eps, out, out_dtype, rows, n_rows,
                                hidden, nullptr, nullptr, stream);
}

// As add_rmsnorm, with the norm  out = (v - mean) / sqrt(var + eps) * w + b,  var the mean of the
// squared deviations (two passes over the row, which is kept in shared memory; sums in 32-bit in
// the block's fixed order).
template <typename TD, typename TO, int THREADS>
__global__ void __launch_bounds__(THREADS)
add_layernorm_kernel(float *__restrict__ resid, const TD *__restrict__ delta, int n_parts, size_t part_stride,
                     const float *__restrict__ weight, const float *__restrict__ bias, float eps, TO *__restrict__ out,
                     const int *__restrict__ rows, int hidden) {
  extern __shared__ float row_buf[];   // hidden floats
  __shared__ float scratch[THREADS / 32 + 1];
  grid_dependents_launch();
  grid_dependency_wait();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float *x = resid + (size_t)r * hidden;
  float sum = 0.f;
  for (int c = threadIdx.x; c < hidden; c += THREADS) {
    float v = x[c];
    for (int p = 0; p < n_parts; ++p) v += to_float(delta[p * part_stride + (size_t)r * hidden + c]);
    row_buf[c] = v;
    if (!rows && n_parts > 0) x[c] = v;
    sum += v;
  }
  if (!out) return;
  const float mean = block_sum<THREADS>(sum, scratch) / (float)hidden;
  float ss = 0.f;
  for (int c = threadIdx.x; c < hidden; c += THREADS) {
    const float dv = row_buf[c] - mean;
    ss = fmaf(dv, dv, ss);
  }
  const float var = block_sum<THREADS>(ss, scratch) / (float)hidden;
  const float inv = 1.f / sqrtf(var + eps);
  TO *o = out + (size_t)i * hidden;
  for (int c = threadIdx.x; c < hidden; c += THREADS)
    o[c] = from_float<TO>((row_buf[c] - mean) * inv * weight[c] + (bias ? bias[c] : 0.f));
}

// The same with the row in registers, four values to a load (widths that are multiples of 4, up to 8,192; up
// to MAXP parts, whose loads are all issued before any is used).  The sums' order within a thread differs from
// the general kernel's only in which thread owns which columns; a row's result does not depend on the launch.
template <typename TD, typename TO, int THREADS, int VPT, int MAXP>
__global__ void __launch_bounds__(THREADS)
add_layernorm_vec_kernel(float *__restrict__ resid, const TD *__restrict__ delta, int n_parts, size_t part_stride,
                         const float *__restrict__ weight, const float *__restrict__ bias, float eps, TO *__restrict__ out,
                         const int *__restrict__ rows, int hidden) {
  __shared__ float scratch[THREADS / 32 + 1];
  grid_dependents_launch();
  const int i = blockIdx.x;
  const int n4 = hidden / 4;
  float4 v[VPT], w[VPT], b[VPT], d[VPT][MAXP];
  if (out) {                             // the norm's weight and bias do not depend on the kernel before
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int c4 = threadIdx.x + j * THREADS;
      if (c4 < n4) {
        w[j] = ld4(weight + 4 * c4);
        b[j] = bias ? ld4(bias + 4 * c4) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
  }
  grid_dependency_wait();
  const int r = rows ? rows[i] : i;
  float *x = resid + (size_t)r * hidden;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int c4 = threadIdx.x + j * THREADS;
    if (c4 < n4) {
      v[j] = ld4(x + 4 * c4);
#pragma unroll
      for (int p = 0; p < MAXP; ++p)
        if (p < n_parts) d[j][p] = ld4(delta + p * part_stride + (size_t)r * hidden + 4 * c4);
    }
  }
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int c4 = threadIdx.x + j * THREADS;
    if (c4 < n4) {
#pragma unroll
      for (int p = 0; p < MAXP; ++p)
        if (p < n_parts) {
          v[j].x += d[j][p].x;
          v[j].y += d[j][p].y;
          v[j].z += d[j][p].z;
          v[j].w += d[j][p].w;
        }
      if (!rows && n_parts > 0) st4(x + 4 * c4, v[j]);
      sum += v[j].x;
      sum += v[j].y;
      sum += v[j].z;
      sum += v[j].w;
    }
  }
  if (!out) return;
  const float mean = block_sum<THREADS>(sum, scratch) / (float)hidden;
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int c4 = threadIdx.x + j * THREADS;
    if (c4 < n4) {
      v[j] = make_float4(v[j].x - mean, v[j].y - mean, v[j].z - mean, v[j].w - mean);
      ss = fmaf(v[j].x, v[j].x, ss);
      ss = fmaf(v[j].y, v[j].y, ss);
      ss = fmaf(v[j].z, v[j].z, ss);
      ss = fmaf(v[j].w, v[j].w, ss);
    }
  }
  const float var = block_sum<THREADS>(ss, scratch) / (float)hidden;
  const float inv = 1.f / sqrtf(var + eps);
  TO *o = out + (size_t)i * hidden;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int c4 = threadIdx.x + j * THREADS;
    if (c4 < n4)
      st4(o + 4 * c4, make_float4(v[j].x * inv * w[j].x + b[j].x, v[j].y * inv * w[j].y + b[j].y, v[j].z * inv * w[j].z + b[j].z,
                                  v[j].w * inv * w[j].w + b[j].w));
  }
}

template <typename TD, typename TO>
static int launch_add_layernorm(float *resid, const void *delta, int n_parts, size_t part_stride, const float *weight,
                                const float *bias, float eps, void *out, const int *rows, int n_rows, int hidden,
                                cudaStream_t stream) {
  const bool aligned = hidden % 4 == 0 && (uintptr_t)resid % 16 == 0 && (uintptr_t)delta % 16 == 0 && (uintptr_t)weight % 16 == 0 &&
                       (uintptr_t)bias % 16 == 0 && (uintptr_t)out % 16 == 0 && part_stride % 4 == 0;
  if (aligned && hidden <= 8192 && n_parts <= 16) {
#define ADDLN_GO(T_, V_, MAXP)                                                                            \
  llm_launch(add_layernorm_vec_kernel<TD, TO, T_, V_, MAXP>, n_rows, T_, 0, stream, resid, (const TD *)delta, n_parts, part_stride, \
             weight, bias, eps, (TO *)out, rows, hidden)
#define ADDLN_SIZE(MAXP)                                    \
  do {                                                      \
    if (hidden <= 512) ADDLN_GO(128, 1, MAXP);              \
    else if (hidden <= 2048) ADDLN_GO(512, 1, MAXP);        \
    else if (hidden <= 4096) ADDLN_GO(1024, 1, MAXP);       \
    else ADDLN_GO(1024, 2, MAXP);                           \
  } while (0)
    // one instantiation per bound on the parts (a prompt step has one part and thousands of rows)
    if (n_parts <= 1) ADDLN_SIZE(1);
    else if (n_parts <= 4) ADDLN_SIZE(4);
    else if (n_parts <= 8) ADDLN_SIZE(8);
    else ADDLN_SIZE(16);
#undef ADDLN_SIZE
#undef ADDLN_GO
    LLM_CHECK_LAUNCH("add_layernorm");
    return LLM_OK;
  }
  const size_t smem = (size_t)hidden * sizeof(float);
  LLM_REQUIRE(smem <= 200 * 1024, "add_layernorm: a row of %d values does not fit shared memory", hidden);
  if (hidden <= 1024) {
    auto kern = add_layernorm_kernel<TD, TO, 128>;
    llm_launch(kern, n_rows, 128, smem, stream, resid, (const TD *)delta, n_parts, part_stride, weight, bias, eps, (TO *)out, rows, hidden);
  } else {
    auto kern = add_layernorm_kernel<TD, TO, 512>;
    if (smem > 48 * 1024) LLM_CHECK_CUDA(llm_allow_smem(kern, smem), "add_layernorm attribute");
    llm_launch(kern, n_rows, 512, smem, stream, resid, (const TD *)delta, n_parts, part_stride, weight, bias, eps, (TO *)out, rows, hidden);
  }
  LLM_CHECK_LAUNCH("add_layernorm");
  return LLM_OK;
}

LLM_EXPORT int llm_add_layernorm(float *resid, const void *delta, int delta_dtype, int n_parts, long long part_stride,
                                 const float *weight, const float *bias, float eps, void *out, int out_dtype, const int *rows,
                                 int n_rows, int hidden, cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE(n_rows > 0 && hidden > 0 && n_parts >= 0, "add_layernorm: bad sizes");
  LLM_REQUIRE(out == nullptr || weight != nullptr, "add_layernorm: a norm needs its weight");
  if (!delta) n_parts = 0;
  if (delta_dtype == LLM_F32 && out_dtype == LLM_F32)
    return launch_add_layernorm<float, float>(resid, delta, n_parts, part_stride, weight, bias, eps, out, rows, n_rows, hidden, stream);
  if (delta_dtype == LLM_F32 && out_dtype == LLM_BF16)
    return launch_add_layernorm<float, __nv_bfloat16>(resid, delta, n_parts, part_stride, weight, bias, eps, out, rows, n_rows, hidden, stream);
  if (delta_dtype == LLM_BF16 && out_dtype == LLM_BF16)
    return launch_add_layernorm<__nv_bfloat16, __nv_bfloat16>(resid, delta, n_parts, part_stride, weight, bias, eps, out, rows, n_rows, hidden, stream);
  if (delta_dtype == LLM_BF16 && out_dtype == LLM_F32)
    return launch_add_layernorm<__nv_bfloat16, float>(resid, delta, n_parts, part_stride, weight, bias, eps, out, rows, n_rows, hidden, stream);
  LLM_FAIL("add_layernorm: unknown dtypes %d, %d", delta_dtype, out_dtype);
}

// Layer norm of a step of single tokens followed by the convolution over time that the mixer's input goes
// through (parts/builtin.cc: prenorm block, mixer_conv): row i is sequence i's one token, the taps - 1 rows before
// it are the sequence's state[slot][0 .. taps - 2] (in out's type), which moves on by one row.  The normalised row
// is rounded to out's type before the convolution reads it, as it is where the two are separate kernels, so that a
// token's result is the same whether it came with a prompt or alone.  A thread reads and writes the state of its
// own channels only.
template <typename TD, typename TO, int THREADS, int VPT, int MAXP>
__global__ void __launch_bounds__(THREADS)
add_layernorm_conv_kernel(float *__restrict__ resid, const TD *__restrict__ delta, int n_parts, size_t part_stride,
                          const float *__restrict__ weight, const float *__restrict__ bias, float eps, TO *__restrict__ out,
                          int hidden, const float *__restrict__ conv_w, TO *__restrict__ state, const int *__restrict__ seq_slot,
                          int taps) {
  constexpr int MAX_KEEP = 7;            // taps - 1 of the longest convolution
  __shared__ float scratch[THREADS / 32 + 1];
  grid_dependents_launch();
  const int i = blockIdx.x;
  const int n4 = hidden / 4, keep = taps - 1;
  float4 v[VPT], w[VPT], b[VPT], d[VPT][MAXP];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {        // the norm's weight and bias do not depend on the kernel before
    const int c4 = threadIdx.x + j * THREADS;
    if (c4 < n4) {
      w[j] = ld4(weight + 4 * c4);
      b[j] = bias ? ld4(bias + 4 * c4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  grid_dependency_wait();
  float *x = resid + (size_t)i * hidden;
  TO *st = state + (size_t)seq_slot[i] * keep * hidden;
  float4 old[VPT][MAX_KEEP];             // the sequence's earlier rows: on their way while the norm is taken
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int c4 = threadIdx.x + j * THREADS;
    if (c4 < n4) {
      v[j] = ld4(x + 4 * c4);
#pragma unroll
      for (int p = 0; p < MAXP; ++p)
        if (p < n_parts) d[j][p] = ld4(delta + p * part_stride + (size_t)i * hidden + 4 * c4);
#pragma unroll
      for (int t = 0; t < MAX_KEEP; ++t)
        if (t < keep) old[j][t] = ld4(st + (size_t)t * hidden + 4 * c4);
    }
  }
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int c4 = threadIdx.x + j * THREADS;
    if (c4 < n4) {
#pragma unroll
      for (int p = 0; p < MAXP; ++p)
        if (p < n_parts) {
          v[j].x += d[j][p].x;
          v[j].y += d[j][p].y;
          v[j].z += d[j][p].z;
          v[j].w += d[j][p].w;
        }
      if (n_parts > 0) st4(x + 4 * c4, v[j]);
      sum += v[j].x;
      sum += v[j].y;
      sum += v[j].z;
      sum += v[j].w;
    }
  }
  const float mean = block_sum<THREADS>(sum, scratch) / (float)hidden;
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int c4 = threadIdx.x + j * THREADS;
    if (c4 < n4) {
      v[j] = make_float4(v[j].x - mean, v[j].y - mean, v[j].z - mean, v[j].w - mean);
      ss = fmaf(v[j].x, v[j].x, ss);
      ss = fmaf(v[j].y, v[j].y, ss);
      ss = fmaf(v[j].z, v[j].z, ss);
      ss = fmaf(v[j].w, v[j].w, ss);
    }
  }
  const float var = block_sum<THREADS>(ss, scratch) / (float)hidden;
  const float inv = 1.f / sqrtf(var + eps);
  TO *o = out + (size_t)i * hidden;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int c4 = threadIdx.x + j * THREADS;
    if (c4 >= n4) continue;
    float h[4] = {v[j].x * inv * w[j].x + b[j].x, v[j].y * inv * w[j].y + b[j].y, v[j].z * inv * w[j].z + b[j].z,
                  v[j].w * inv * w[j].w + b[j].w};
    float res[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      h[e] = to_float(from_float<TO>(h[e]));      // the convolution reads the row as it is stored
      const float *cw = conv_w + (size_t)(4 * c4 + e) * taps;
      // the same order of operations as the convolution's own kernel: taps in order, then the token itself
      float s = 0.f;
#pragma unroll
      for (int t = 0; t < MAX_KEEP; ++t)
        if (t < keep) s = fmaf(cw[t], e == 0 ? old[j][t].x : e == 1 ? old[j][t].y : e == 2 ? old[j][t].z : old[j][t].w, s);
      s = fmaf(cw[keep], h[e], s);
      res[e] = h[e] + s;
    }
#pragma unroll
    for (int t = 1; t < MAX_KEEP; ++t)
      if (t < keep) st4(st + (size_t)(t - 1) * hidden + 4 * c4, old[j][t]);
    st4(st + (size_t)(keep - 1) * hidden + 4 * c4, make_float4(h[0], h[1], h[2], h[3]));
    st4(o + 4 * c4, make_float4(res[0], res[1], res[2], res[3]));
  }
}

// 1 if the fused kernel takes rows of this width with this many parts pending (else: the norm, then the convolution).
LLM_EXPORT int llm_add_layernorm_conv_supports(int hidden, int n_parts, int taps) {
  return hidden % 4 == 0 && hidden <= 8192 && n_parts <= 8 && taps >= 2 && taps <= 8;
}

LLM_EXPORT int llm_add_layernorm_conv(float *resid, const void *delta, int delta_dtype, int n_parts, long long part_stride,
                                      const float *weight, const float *bias, float eps, void *out, int out_dtype, int n_rows,
                                      int hidden, const float *conv_w, void *state, const int *seq_slot, int taps,
                                      cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE(n_rows > 0 && hidden > 0 && n_parts >= 0 && out && weight && conv_w && state && seq_slot, "add_layernorm_conv: bad arguments");
  if (!delta) n_parts = 0;
  LLM_REQUIRE(llm_add_layernorm_conv_supports(hidden, n_parts, taps), "add_layernorm_conv: rows of %d values with %d parts and %d taps are not taken",
              hidden, n_parts, taps);
  LLM_REQUIRE((uintptr_t)resid % 16 == 0 && (uintptr_t)delta % 16 == 0 && (uintptr_t)weight % 16 == 0 && (uintptr_t)bias % 16 == 0 &&
                  (uintptr_t)out % 16 == 0 && (uintptr_t)state % 16 == 0 && part_stride % 4 == 0,
              "add_layernorm_conv: rows must be 16-byte aligned");
#define ADDLNC_GO(TD, TO, T_, V_, MAXP)                                                                                 \
  llm_launch(add_layernorm_conv_kernel<TD, TO, T_, V_, MAXP>, n_rows, T_, 0, stream, resid, (const TD *)delta, n_parts, (size_t)part_stride, \
             weight, bias, eps, (TO *)out, hidden, conv_w, (TO *)state, seq_slot, taps)
#define ADDLNC_SIZE(TD, TO, MAXP)                                \
  do {                                                           \
    if (hidden <= 512) ADDLNC_GO(TD, TO, 128, 1, MAXP);          \
    else if (hidden <= 2048) ADDLNC_GO(TD, TO, 512, 1, MAXP);    \
    else if (hidden <= 4096) ADDLNC_GO(TD, TO, 1024, 1, MAXP);   \
    else ADDLNC_GO(TD, TO, 1024, 2, MAXP);                       \
  } while (0)
#define ADDLNC_PARTS(TD, TO)                  \
  do {                                        \
    if (n_parts <= 1) ADDLNC_SIZE(TD, TO, 1); \
    else if (n_parts <= 4) ADDLNC_SIZE(TD, TO, 4); \
    else ADDLNC_SIZE(TD, TO, 8);              \
  } while (0)
  if (delta_dtype == LLM_F32 && out_dtype == LLM_F32) ADDLNC_PARTS(float, float);
  else if (delta_dtype == LLM_F32 && out_dtype == LLM_BF16) ADDLNC_PARTS(float, __nv_bfloat16);
  else LLM_FAIL("add_layernorm_conv: unsupported dtypes %d, %d", delta_dtype, out_dtype);
#undef ADDLNC_PARTS
#undef ADDLNC_SIZE
#undef ADDLNC_GO
  LLM_CHECK_LAUNCH("add_layernorm_conv");
  return LLM_OK;
}

// ---------------------------------------------------------------- rows of the stream picked out
// out[i] = resid[rows[i]] + sum_p delta[p][rows[i]] (32-bit, parts in index order): the residual
// stream of the rows that anything still reads, when the others are done with.
template <typename TD>
__global__ void gather_rows_add_kernel(const float *__restrict__ resid, const TD *__restrict__ delta, int n_parts,
                                       size_t part_stride, const int *__restrict__ rows, float *__restrict__ out, int hidden,
                                       const float *__restrict__ col_scale, const float *__restrict__ col_bias) {
  grid_dependents_launch();
  grid_dependency_wait();
  const int i = blockIdx.x;
  const size_t r = (size_t)rows[i];
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = resid[r * hidden + c];
    if (col_scale || col_bias) {
      float d = 0.f;
      for (int p = 0; p < n_parts; ++p) d += to_float(delta[p * part_stride + r * hidden + c]);
      if (col_bias) d += col_bias[c];
      if (col_scale) d *= col_scale[c];
      if (n_parts > 0) v += d;
    } else {
      for (int p = 0; p < n_parts; ++p) v += to_float(delta[p * part_stride + r * hidden + c]);
    }
    out[(size_t)i * hidden + c] = v;
  }
}

LLM_EXPORT int llm_gather_rows_add_scaled(const float *resid, const void *delta, int delta_dtype, int n_parts, long long part_stride,
                                          const int *rows, int n_rows, float *out, int hidden, const float *col_scale,
                                          const float *col_bias, cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE(n_rows > 0 && hidden > 0 && n_parts >= 0 && rows != nullptr && out != nullptr, "gather_rows_add: bad arguments");
  if (!delta) n_parts = 0;
  if (delta_dtype == LLM_BF16 && n_parts > 0)
    LLM_CHECK_CUDA(llm_launch(gather_rows_add_kernel<__nv_bfloat16>, dim3(n_rows), dim3(256), 0, stream, resid, (const __nv_bfloat16 *)delta,
                              n_parts, (size_t)part_stride, rows, out, hidden, col_scale, col_bias), "gather_rows_add launch");
  else
    LLM_CHECK_CUDA(llm_launch(gather_rows_add_kernel<float>, dim3(n_rows), dim3(256), 0, stream, resid, (const float *)delta, n_parts,
                              (size_t)part_stride, rows, out, hidden, col_scale, col_bias), "gather_rows_add launch");
  return LLM_OK;
}

LLM_EXPORT int llm_gather_rows_add(const float *resid, const void *delta, int delta_dtype, int n_parts, long long part_stride,
                                   const int *rows, int n_rows, float *out, int hidden, cudaStream_t stream) {
  return llm_gather_rows_add_scaled(resid, delta, delta_dtype, n_parts, part_stride, rows, n_rows, out, hidden, nullptr, nullptr, stream);
}

// ---------------------------------------------------------------- swiglu
// out[t, i] = silu(gu[t, i]) * gu[t, inter + i], silu(a) = a / (1 + exp(-a)).  TI is the
// type of the stacked gate|up product (32-bit when the product gives that), T of out.
template <typename TI, typename T>
__global__ void swiglu_kernel(const TI *__restrict__ gu, T *__restrict__ out, int inter, size_t total) {
  grid_dependents_launch();
  grid_dependency_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / inter;
    const int i = (int)(idx - t * inter);
    const float g = to_float(gu[t * 2 * inter + i]);
    const float u = to_float(gu[t * 2 * inter + inter + i]);
    out[idx] = from_float<T>(g / (1.f + expf(-g)) * u);
  }
}

// Four values per thread (widths that are a multiple of 4, 16-byte aligned rows).
template <typename TI, typename T>
__global__ void swiglu_vec_kernel(const TI *__restrict__ gu, T *__restrict__ out, int inter4, size_t total4) {
  grid_dependents_launch();
  grid_dependency_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total4;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / inter4;
    const int i = (int)(idx - t * inter4) * 4;
    const TI *row = gu + t * 8 * (size_t)inter4;
    const float4 g = ld4(row + i), u = ld4(row + 4 * (size_t)inter4 + i);
    st4(out + idx * 4, make_float4(g.x / (1.f + expf(-g.x)) * u.x, g.y / (1.f + expf(-g.y)) * u.y,
                                   g.z / (1.f + expf(-g.z)) * u.z, g.w / (1.f + expf(-g.w)) * u.w));
  }
}

LLM_EXPORT int llm_swiglu(int in_dtype, int dtype, const void *gu, void *out, int n_tokens, int inter,
                          cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && inter > 0, "swiglu: bad sizes");
  const int threads = 256;
  const bool vec = inter % 4 == 0 && (uintptr_t)gu % 16 == 0 && (uintptr_t)out % 16 == 0;
  const size_t total = vec ? (size_t)n_tokens * (inter / 4) : (size_t)n_tokens * inter;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > (size_t)sm_count() * 32) blocks = (size_t)sm_count() * 32;
#define SWIGLU_GO(TI, T)                                                                                     \
  do {                                                                                                       \
    if (vec)                                                                                                 \
      llm_launch(swiglu_vec_kernel<TI, T>, (unsigned)blocks, threads, 0, stream, (const TI *)gu, (T *)out, inter / 4, total); \
    else                                                                                                     \
      llm_launch(swiglu_kernel<TI, T>, (unsigned)blocks, threads, 0, stream, (const TI *)gu, (T *)out, inter, total); \
  } while (0)
  if (in_dtype == LLM_F32 && dtype == LLM_F32) SWIGLU_GO(float, float);
  else if (in_dtype == LLM_F32 && dtype == LLM_BF16) SWIGLU_GO(float, __nv_bfloat16);
  else if (in_dtype == LLM_BF16 && dtype == LLM_BF16) SWIGLU_GO(__nv_bfloat16, __nv_bfloat16);
  else LLM_FAIL("swiglu: unsupported dtypes in %d out %d", in_dtype, dtype);
#undef SWIGLU_GO
  LLM_CHECK_LAUNCH("swiglu");
  return LLM_OK;
}

// ---------------------------------------------------------------- clamped gated unit
// Rows [gate (inter) | up (inter)] of a stacked product (32-bit or bfloat16), biases of 2 * inter 32-bit
// values (null: none) added here, in 32-bit, so that the product runs without them:
//   g = min(gate + b_g, limit), u = clamp(up + b_u, -limit, limit), out = g * sigmoid(slope * g) * (u + up_shift).
// limit <= 0: no bounds.
__device__ __forceinline__ float clamped_glu_one(float g, float u, float limit, float slope, float up_shift) {
  if (limit > 0.f) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
  }
  return g / (1.f + expf(-slope * g)) * (u + up_shift);
}

template <typename TI, typename T>
__global__ void clamped_glu_kernel(const TI *__restrict__ gu, long long ld, const float *__restrict__ bias, T *__restrict__ out,
                                   int inter, size_t total, float limit, float slope, float up_shift) {
  grid_dependents_launch();
  grid_dependency_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / inter;
    const int i = (int)(idx - t * inter);
    const float g = to_float(gu[t * ld + i]) + (bias ? bias[i] : 0.f);
    const float u = to_float(gu[t * ld + inter + i]) + (bias ? bias[inter + i] : 0.f);
    out[idx] = from_float<T>(clamped_glu_one(g, u, limit, slope, up_shift));
  }
}

// Four values per thread (widths that are a multiple of 4, 16-byte aligned rows).
template <typename TI, typename T>
__global__ void clamped_glu_vec_kernel(const TI *__restrict__ gu, long long ld, const float *__restrict__ bias, T *__restrict__ out,
                                       int inter4, size_t total4, float limit, float slope, float up_shift) {
  grid_dependents_launch();
  grid_dependency_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total4; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / inter4;
    const int i = (int)(idx - t * inter4) * 4;
    const TI *row = gu + t * ld;
    float4 g = ld4(row + i), u = ld4(row + 4 * (size_t)inter4 + i);
    if (bias) {
      const float4 bg = ld4(bias + i), bu = ld4(bias + 4 * (size_t)inter4 + i);
      g = make_float4(g.x + bg.x, g.y + bg.y, g.z + bg.z, g.w + bg.w);
      u = make_float4(u.x + bu.x, u.y + bu.y, u.z + bu.z, u.w + bu.w);
    }
    st4(out + idx * 4, make_float4(clamped_glu_one(g.x, u.x, limit, slope, up_shift), clamped_glu_one(g.y, u.y, limit, slope, up_shift),
                                   clamped_glu_one(g.z, u.z, limit, slope, up_shift), clamped_glu_one(g.w, u.w, limit, slope, up_shift)));
  }
}

LLM_EXPORT int llm_clamped_glu(int in_dtype, int dtype, const void *gu, long long ld, const float *bias, void *out, int n_tokens,
                               int inter, float limit, float slope, float up_shift, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && inter > 0 && ld >= 2LL * inter, "clamped_glu: bad sizes");
  const int threads = 256;
  const bool vec = inter % 4 == 0 && ld % 8 == 0 && (uintptr_t)gu % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)bias % 16 == 0;
  const size_t total = vec ? (size_t)n_tokens * (inter / 4) : (size_t)n_tokens * inter;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > (size_t)sm_count() * 32) blocks = (size_t)sm_count() * 32;
#define CGLU_GO(TI, T)                                                                                                   \
  do {                                                                                                                   \
    if (vec)                                                                                                             \
      llm_launch(clamped_glu_vec_kernel<TI, T>, (unsigned)blocks, threads, 0, stream, (const TI *)gu, ld, bias, (T *)out, inter / 4, \
                 total, limit, slope, up_shift);                                                                         \
    else                                                                                                                 \
      llm_launch(clamped_glu_kernel<TI, T>, (unsigned)blocks, threads, 0, stream, (const TI *)gu, ld, bias, (T *)out, inter, total, \
                 limit, slope, up_shift);                                                                                \
  } while (0)
  if (in_dtype == LLM_F32 && dtype == LLM_F32) CGLU_GO(float, float);
  else if (in_dtype == LLM_F32 && dtype == LLM_BF16) CGLU_GO(float, __nv_bfloat16);
  else if (in_dtype == LLM_BF16 && dtype == LLM_BF16) CGLU_GO(__nv_bfloat16, __nv_bfloat16);
  else LLM_FAIL("clamped_glu: unsupported dtypes in %d out %d", in_dtype, dtype);
#undef CGLU_GO
  LLM_CHECK_LAUNCH("clamped_glu");
  return LLM_OK;
}

// ---------------------------------------------------------------- scaling of rows and logits
// x *= scale over n values: the token rows of an architecture that scales its embedding.
__global__ void scale_rows_kernel(float *__restrict__ x, long long n, float scale) {
  grid_dependents_launch();
  grid_dependency_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    x[i] *= scale;
}

LLM_EXPORT int llm_scale_rows(float *x, long long n, float scale, cudaStream_t stream) {
  if (n == 0) return LLM_OK;
  LLM_REQUIRE(n > 0 && x != nullptr, "scale_rows: bad arguments");
  long long blocks = (n + 255) / 256;
  if (blocks > (long long)sm_count() * 16) blocks = (long long)sm_count() * 16;
  llm_launch(scale_rows_kernel, (unsigned)blocks, 256, 0, stream, x, n, scale);
  LLM_CHECK_LAUNCH("scale_rows");
  return LLM_OK;
}

// logit = logit * scale, then, with a positive cap, cap * tanh(logit / cap), in 32-bit.
__global__ void logit_transform_kernel(float *__restrict__ x, long long n, float scale, float cap) {
  grid_dependents_launch();
  grid_dependency_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float v = x[i] * scale;
    if (cap > 0.f) v = cap * tanhf(v / cap);
    x[i] = v;
  }
}

LLM_EXPORT int llm_logit_transform(float *x, long long n, float scale, float cap, cudaStream_t stream) {
  if (n == 0) return LLM_OK;
  LLM_REQUIRE(n > 0 && x != nullptr, "logit_transform: bad arguments");
  long long blocks = (n + 255) / 256;
  if (blocks > (long long)sm_count() * 16) blocks = (long long)sm_count() * 16;
  llm_launch(logit_transform_kernel, (unsigned)blocks, 256, 0, stream, x, n, scale, cap);
  LLM_CHECK_LAUNCH("logit_transform");
  return LLM_OK;
}

// ---------------------------------------------------------------- random weights on the device
// Element i is a pure function of (seed, i): two SplitMix64 outputs give two uniform numbers;
// law 0 turns them into a normal number with mean a and deviation b (Box-Muller), law 1 into a
// uniform number in [a, b).  The random-weights mode of a benchmark fills its tensors here
// instead of drawing a billion numbers on the host.
__device__ __forceinline__ unsigned long long splitmix64(unsigned long long z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

template <typename T>
__global__ void random_fill_kernel(T *__restrict__ out, long long n, unsigned long long seed, int law, float a, float b) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const unsigned long long h1 = splitmix64(seed ^ splitmix64((unsigned long long)i));
    const unsigned long long h2 = splitmix64(h1);
    const float u1 = ((float)(h1 >> 40) + 1.0f) * (1.0f / 16777216.0f);      // (0, 1]
    const float u2 = (float)(h2 >> 40) * (1.0f / 16777216.0f);               // [0, 1)
    float v;
    if (law == 0) v = a + b * sqrtf(-2.0f * logf(u1)) * cosf(6.283185307179586f * u2);
    else v = a + (b - a) * u2;
    out[i] = from_float<T>(v);
  }
}

LLM_EXPORT int llm_random_fill(void *out, int dtype, long long n, unsigned long long seed, int law, float a, float b,
                               cudaStream_t stream) {
  if (n == 0) return LLM_OK;
  LLM_REQUIRE(n > 0 && out != nullptr && (law == 0 || law == 1), "random_fill: bad arguments");
  long long blocks = (n + 255) / 256;
  if (blocks > (long long)sm_count() * 32) blocks = (long long)sm_count() * 32;
  if (dtype == LLM_F32) random_fill_kernel<float><<<(unsigned)blocks, 256, 0, stream>>>((float *)out, n, seed, law, a, b);
  else if (dtype == LLM_BF16) random_fill_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>((__nv_bfloat16 *)out, n, seed, law, a, b);
  else LLM_FAIL("random_fill: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("random_fill");
  return LLM_OK;
}

// ---------------------------------------------------------------- the stream beside another tensor
// out[t] = [resid[t] + sum_p delta[p][t] | other[t]], two rows of `hidden` values side by side in
// the type of out: the input of a projection that mixes the residual stream with a second tensor
// of the same shape (the token rows, for a model that feeds them to every pass of a loop).
template <typename TO>
__global__ void concat_stream_kernel(const float *__restrict__ resid, const float *__restrict__ delta, int n_parts,
                                     size_t part_stride, const float *__restrict__ other, TO *__restrict__ out,
                                     int hidden, size_t total) {
  grid_dependents_launch();
  grid_dependency_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / hidden;
    const int c = (int)(idx - t * hidden);
    float v = resid[idx];
    for (int p = 0; p < n_parts; ++p) v += delta[p * part_stride + idx];
    out[t * 2 * hidden + c] = from_float<TO>(v);
    out[t * 2 * hidden + hidden + c] = from_float<TO>(other[idx]);
  }
}

LLM_EXPORT int llm_concat_stream(const float *resid, const float *delta, int n_parts, long long part_stride,
                                 const float *other, void *out, int out_dtype, int n_rows, int hidden,
                                 cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE(n_rows > 0 && hidden > 0 && resid && other && out && n_parts >= 0, "concat_stream: bad arguments");
  if (!delta) n_parts = 0;
  const size_t total = (size_t)n_rows * hidden;
  size_t blocks = (total + 255) / 256;
  if (blocks > (size_t)sm_count() * 32) blocks = (size_t)sm_count() * 32;
  if (out_dtype == LLM_F32)
    llm_launch(concat_stream_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, resid, delta, n_parts,
               (size_t)part_stride, other, (float *)out, hidden, total);
  else if (out_dtype == LLM_BF16)
    llm_launch(concat_stream_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, stream, resid, delta, n_parts,
               (size_t)part_stride, other, (__nv_bfloat16 *)out, hidden, total);
  else LLM_FAIL("concat_stream: unknown dtype %d", out_dtype);
  LLM_CHECK_LAUNCH("concat_stream");
  return LLM_OK;
}

// ---------------------------------------------------------------- a gate per head
// x[t, h * dv + c] *= sigmoid(gate[t * gate_stride + h]): the output gate of an attention whose
// kernel does not apply it itself.  The gate is 32-bit (a column block of the stacked product).
template <typename T>
__global__ void head_gate_kernel(T *__restrict__ x, long long ld, const float *__restrict__ gate, long long gate_stride,
                                 int n_heads, int dv, size_t total) {
  grid_dependents_launch();
  grid_dependency_wait();
  const int width = n_heads * dv;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / width;
    const int c = (int)(idx - t * width);
    const float g = 1.f / (1.f + expf(-gate[t * gate_stride + c / dv]));
    T *p = x + t * ld + c;
    *p = from_float<T>(to_float(*p) * g);
  }
}

// Four channels to a thread (head widths that are a multiple of 4, 8-byte aligned rows).
template <typename T>
__global__ void head_gate_vec_kernel(T *__restrict__ x, long long ld, const float *__restrict__ gate, long long gate_stride,
                                     int n_heads, int dv4, size_t total4) {
  grid_dependents_launch();
  grid_dependency_wait();
  const int width4 = n_heads * dv4;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total4; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / width4;
    const int c4 = (int)(idx - t * width4);
    const float g = 1.f / (1.f + expf(-gate[t * gate_stride + c4 / dv4]));
    T *p = x + t * ld + 4 * c4;
    const float4 v = ld4(p);
    st4(p, make_float4(v.x * g, v.y * g, v.z * g, v.w * g));
  }
}

// A gate per channel: x[t, c] *= sigmoid(gate[t * gate_stride + c]), four channels to a thread.
template <typename T>
__global__ void channel_gate_vec_kernel(T *__restrict__ x, long long ld, const float *__restrict__ gate, long long gate_stride,
                                        int width4, size_t total4) {
  grid_dependents_launch();
  grid_dependency_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total4; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / width4;
    const int c = (int)(idx - t * width4) * 4;
    const float4 g = ld4(gate + t * gate_stride + c);
    T *p = x + t * ld + c;
    const float4 v = ld4(p);
    st4(p, make_float4(v.x / (1.f + expf(-g.x)), v.y / (1.f + expf(-g.y)), v.z / (1.f + expf(-g.z)), v.w / (1.f + expf(-g.w))));
  }
}

LLM_EXPORT int llm_head_gate(void *x, int dtype, long long ld, const float *gate, long long gate_stride, int n_tokens,
                             int n_heads, int dv, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_heads > 0 && dv > 0 && x && gate, "head_gate: bad arguments");
  if (dv == 1 && n_heads % 4 == 0 && ld % 4 == 0 && gate_stride % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)gate % 16 == 0) {
    // heads of one channel: a gate per channel
    const size_t total4 = (size_t)n_tokens * (n_heads / 4);
    size_t blocks4 = (total4 + 255) / 256;
    if (blocks4 > (size_t)sm_count() * 32) blocks4 = (size_t)sm_count() * 32;
    if (dtype == LLM_F32)
      llm_launch(channel_gate_vec_kernel<float>, dim3((unsigned)blocks4), dim3(256), 0, stream, (float *)x, ld, gate, gate_stride,
                 n_heads / 4, total4);
    else if (dtype == LLM_BF16)
      llm_launch(channel_gate_vec_kernel<__nv_bfloat16>, dim3((unsigned)blocks4), dim3(256), 0, stream, (__nv_bfloat16 *)x, ld, gate,
                 gate_stride, n_heads / 4, total4);
    else LLM_FAIL("head_gate: unknown dtype %d", dtype);
    LLM_CHECK_LAUNCH("head_gate");
    return LLM_OK;
  }
  if (dv % 4 == 0 && ld % 4 == 0 && (uintptr_t)x % 16 == 0) {
    const size_t total4 = (size_t)n_tokens * n_heads * (dv / 4);
    size_t blocks4 = (total4 + 255) / 256;
    if (blocks4 > (size_t)sm_count() * 32) blocks4 = (size_t)sm_count() * 32;
    if (dtype == LLM_F32)
      llm_launch(head_gate_vec_kernel<float>, dim3((unsigned)blocks4), dim3(256), 0, stream, (float *)x, ld, gate, gate_stride,
                 n_heads, dv / 4, total4);
    else if (dtype == LLM_BF16)
      llm_launch(head_gate_vec_kernel<__nv_bfloat16>, dim3((unsigned)blocks4), dim3(256), 0, stream, (__nv_bfloat16 *)x, ld, gate,
                 gate_stride, n_heads, dv / 4, total4);
    else LLM_FAIL("head_gate: unknown dtype %d", dtype);
    LLM_CHECK_LAUNCH("head_gate");
    return LLM_OK;
  }
  const size_t total = (size_t)n_tokens * n_heads * dv;
  size_t blocks = (total + 255) / 256;
  if (blocks > (size_t)sm_count() * 32) blocks = (size_t)sm_count() * 32;
  if (dtype == LLM_F32)
    llm_launch(head_gate_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, (float *)x, ld, gate, gate_stride, n_heads, dv, total);
  else if (dtype == LLM_BF16)
    llm_launch(head_gate_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, stream, (__nv_bfloat16 *)x, ld, gate,
               gate_stride, n_heads, dv, total);
  else LLM_FAIL("head_gate: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("head_gate");
  return LLM_OK;
}

// ---------------------------------------------------------------- several residual streams
// A model that carries S copies x_0 .. x_{S-1} of the residual stream ("hyper-connections") joins a
// sublayer to them with three small tensors: what the sublayer reads is u = sum_s a[s] x_s, and its
// result y moves every stream at once, from the old ones: x_t <- sum_s M[s, t] x_s + o[t] y.  One CTA
// per row does, in this order and all in 32-bit:
//   1. the pending move of the sublayer before (delta != null: y = (sum of delta's parts + col_bias) *
//      col_scale with matrix `mix` [S, S] indexed [from, to] and vector `outw` [S]); the new streams are
//      stored (x_out; in place when x_out is x_in and rows is null)
//   2. u = sum_s inw[s] x_s, or the plain sum of the streams when inw is null
//   3. out = u / sqrt(mean(u^2) + eps) * norm_w in out's type, or u itself (32-bit) when norm_w is null.
// in_stride 0: the S streams are all equal to the one at x_in (a model's first layer).  With `rows`, output
// row i is source row rows[i] and x_out holds the n_rows chosen rows only (out_stride apart per stream).
// A row's result depends on that row alone; every sum has a fixed order.
constexpr int HYPER_MAX_STREAMS = 16;
template <typename TO, int THREADS, int VEC, int MAXS>       // MAXS >= S: how many copies the unrolled loops provide for
__global__ void __launch_bounds__(THREADS)
hyper_mix_norm_kernel(const float *__restrict__ x_in, long long in_stride, float *__restrict__ x_out, long long out_stride, int S,
                      const float *__restrict__ delta, int n_parts, size_t part_stride, const float *__restrict__ col_scale,
                      const float *__restrict__ col_bias, const float *__restrict__ mix, const float *__restrict__ outw,
                      const float *__restrict__ inw, const float *__restrict__ norm_w, float eps, TO *__restrict__ out,
                      const int *__restrict__ rows, int hidden) {
  extern __shared__ float row_buf[];   // hidden floats
  __shared__ float scratch[THREADS / 32 + 1];
  __shared__ float s_mix[MAXS * MAXS], s_out[MAXS], s_in[MAXS];
  grid_dependents_launch();
  if (threadIdx.x < S * S) s_mix[threadIdx.x] = delta ? mix[threadIdx.x] : 0.f;       // weights: written when the model was loaded
  if (threadIdx.x < S) {
    s_out[threadIdx.x] = delta ? outw[threadIdx.x] : 0.f;
    s_in[threadIdx.x] = inw ? inw[threadIdx.x] : 1.f;
  }
  grid_dependency_wait();
  __syncthreads();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  const bool store = x_out != nullptr && (delta != nullptr || x_out != x_in || rows != nullptr || in_stride == 0);
  float ss = 0.f;
  for (int c = threadIdx.x * VEC; c < hidden; c += THREADS * VEC) {
    float xs[MAXS][VEC];
#pragma unroll
    for (int s = 0; s < MAXS; ++s)
      if (s < S) {
        const float *p = x_in + (size_t)s * in_stride + (size_t)r * hidden + c;
        if (VEC == 4) {
          const float4 v = *reinterpret_cast<const float4 *>(p);
          xs[s][0] = v.x, xs[s][1 % VEC] = v.y, xs[s][2 % VEC] = v.z, xs[s][3 % VEC] = v.w;
        } else {
          xs[s][0] = *p;
        }
      }
    float y[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) y[k] = 0.f;
    if (delta) {
      for (int p = 0; p < n_parts; ++p) {
        const float *dp = delta + p * part_stride + (size_t)r * hidden + c;
        if (VEC == 4) {
          const float4 v = *reinterpret_cast<const float4 *>(dp);
          y[0] += v.x, y[1 % VEC] += v.y, y[2 % VEC] += v.z, y[3 % VEC] += v.w;
        } else {
          y[0] += *dp;
        }
      }
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        if (col_bias) y[k] += col_bias[c + k];
        if (col_scale) y[k] *= col_scale[c + k];
      }
    }
    float u[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) u[k] = 0.f;
#pragma unroll
    for (int t = 0; t < MAXS; ++t)
      if (t < S) {
        float nv[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          if (delta) {
            float a = 0.f;
#pragma unroll
            for (int s = 0; s < MAXS; ++s)
              if (s < S) a = fmaf(s_mix[s * S + t], xs[s][k], a);
            nv[k] = fmaf(s_out[t], y[k], a);
          } else {
            nv[k] = xs[t][k];
          }
          u[k] = fmaf(s_in[t], nv[k], u[k]);
        }
        if (store) {
          float *q = x_out + (size_t)t * out_stride + (size_t)i * hidden + c;
          if (VEC == 4) *reinterpret_cast<float4 *>(q) = make_float4(nv[0], nv[1 % VEC], nv[2 % VEC], nv[3 % VEC]);
          else *q = nv[0];
        }
      }
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      row_buf[c + k] = u[k];
      ss = fmaf(u[k], u[k], ss);
    }
  }
  if (!out) return;
  if (!norm_w) {
    __syncthreads();
    for (int c = threadIdx.x; c < hidden; c += THREADS) out[(size_t)i * hidden + c] = from_float<TO>(row_buf[c]);
    return;
  }
  const float total = block_sum<THREADS>(ss, scratch);
  const float inv = rsqrtf(total / (float)hidden + eps);
  TO *o = out + (size_t)i * hidden;
  for (int c = threadIdx.x; c < hidden; c += THREADS) o[c] = from_float<TO>(row_buf[c] * inv * norm_w[c]);
}

template <typename TO>
static int launch_hyper(const float *x_in, long long in_stride, float *x_out, long long out_stride, int S, const float *delta,
                        int n_parts, size_t part_stride, const float *col_scale, const float *col_bias, const float *mix,
                        const float *outw, const float *inw, const float *norm_w, float eps, TO *out, const int *rows, int n_rows,
                        int hidden, cudaStream_t stream) {
  const size_t smem = (size_t)hidden * sizeof(float);
  LLM_REQUIRE(smem <= 200 * 1024, "hyper_mix_norm: a row of %d values does not fit shared memory", hidden);
  const bool vec = hidden % 4 == 0 && in_stride % 4 == 0 && out_stride % 4 == 0 && part_stride % 4 == 0 && (uintptr_t)x_in % 16 == 0 &&
                   (uintptr_t)x_out % 16 == 0 && (uintptr_t)delta % 16 == 0;
#define HYPER_GO(THREADS, VEC, MAXS)                                                                                               \
  do {                                                                                                                             \
    auto kern = hyper_mix_norm_kernel<TO, THREADS, VEC, MAXS>;                                                                     \
    LLM_CHECK_CUDA(llm_allow_smem(kern, smem), "hyper_mix_norm attribute");                                                       \
    llm_launch(kern, dim3(n_rows), dim3(THREADS), smem, stream, x_in, in_stride, x_out, out_stride, S, delta, n_parts, part_stride, \
               col_scale, col_bias, mix, outw, inw, norm_w, eps, out, rows, hidden);                                               \
  } while (0)
  // wide rows: 512 threads, so that a row of 2,048 values is one round of loads per thread; up to four copies (the
  // usual case) keep the unrolled loops short
  if (S <= 4) {
    if (vec && hidden >= 2048) HYPER_GO(512, 4, 4);
    else if (vec) HYPER_GO(256, 4, 4);
    else HYPER_GO(256, 1, 4);
  } else if (S <= 8) {
    if (vec) HYPER_GO(256, 4, 8);
    else HYPER_GO(256, 1, 8);
  } else {
    if (vec) HYPER_GO(256, 4, 16);
    else HYPER_GO(256, 1, 16);
  }
#undef HYPER_GO
  LLM_CHECK_LAUNCH("hyper_mix_norm");
  return LLM_OK;
}

LLM_EXPORT int llm_hyper_mix_norm(const float *x_in, long long in_stride, float *x_out, long long out_stride, int n_streams,
                                  const float *delta, int n_parts, long long part_stride, const float *col_scale,
                                  const float *col_bias, const float *mix, const float *outw, const float *inw, const float *norm_w,
                                  float eps, void *out, int out_dtype, const int *rows, int n_rows, int hidden, cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE(n_rows > 0 && hidden > 0 && n_streams >= 1 && n_streams <= HYPER_MAX_STREAMS, "hyper_mix_norm: %d streams of %d x %d (up to %d streams)",
              n_streams, n_rows, hidden, HYPER_MAX_STREAMS);
  LLM_REQUIRE(x_in != nullptr && (delta == nullptr || (mix != nullptr && outw != nullptr && n_parts > 0)), "hyper_mix_norm: a pending result needs its matrix and vector");
  LLM_REQUIRE(norm_w == nullptr || out != nullptr, "hyper_mix_norm: a norm needs a place for its result");
  if (out_dtype == LLM_BF16 && norm_w)
    return launch_hyper<__nv_bfloat16>(x_in, in_stride, x_out, out_stride, n_streams, delta, n_parts, (size_t)part_stride, col_scale, col_bias,
                                       mix, outw, inw, norm_w, eps, (__nv_bfloat16 *)out, rows, n_rows, hidden, stream);
  LLM_REQUIRE(out_dtype == LLM_F32 || out == nullptr, "hyper_mix_norm: the streams' sum is 32-bit");
  return launch_hyper<float>(x_in, in_stride, x_out, out_stride, n_streams, delta, n_parts, (size_t)part_stride, col_scale, col_bias, mix, outw,
                             inw, norm_w, eps, (float *)out, rows, n_rows, hidden, stream);
}

// x[i] += value: a stored norm weight w that is applied as (offset + w).
__global__ void add_scalar_kernel(float *__restrict__ x, long long n, float value) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) x[i] += value;
}
LLM_EXPORT int llm_add_scalar(float *x, long long n, float value, cudaStream_t stream) {
  if (n <= 0) return LLM_OK;
  const long long blocks = (n + 255) / 256;
  add_scalar_kernel<<<(unsigned)(blocks > 1024 ? 1024 : blocks), 256, 0, stream>>>(x, n, value);
  LLM_CHECK_LAUNCH("add_scalar");
  return LLM_OK;
}
