// Rotary position encoding of q and k and the append of k and v to the paged cache,
// in one pass over the stacked q|k|v rows of a step.
//
// The reference rotates with about fourteen elementwise launches per layer
// (src/libllm/llama.cc:151-176) and appends by re-allocating and copying the whole
// cache (src/libllm/llama.cc:203-212, src/flint/functional.cc:126-144).  The rotation
// pairs element i with i + d/2 (src/libllm/llama.cc:151-164):
//   out[i]       = x[i] * cos - x[i + d/2] * sin
//   out[i + d/2] = x[i + d/2] * cos + x[i] * sin
// cos and sin come from a 32-bit table [positions, d] (d/2 cosines, then d/2 sines) that
// is computed in 64-bit on the host side; the arithmetic here is 32-bit, rounded once.
//
// Cache layout per layer: [pages, kv_heads, page_size, d]; a token at position p of a
// sequence lies in page page_table[seq][p / page_size] at row p % page_size.
#include "common.cuh"

LLM_DEFINE_LAST_ERROR(llm_rope_last_error)

// TI: type of the stacked q|k|v rows (the product's output, 32-bit when the product can
// give that, so that q and k are rounded once, after the rotation); T: type of the
// rotated queries and of the cache.
template <typename TI, typename T>
__global__ void rope_cache_write_kernel(const TI *__restrict__ qkv, long long row_stride,
                                        T *__restrict__ q_out, long long q_stride, int n_heads,
                                        int n_kv, int d, const float *__restrict__ table,
                                        int table_rows, int rot_dim, const int *__restrict__ tok_seq,
                                        const int *__restrict__ tok_pos, const int *__restrict__ page_table,
                                        int pt_stride, T *__restrict__ kcache, T *__restrict__ vcache,
                                        int page_size) {
  grid_dependents_launch();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const int slot = blockIdx.y;                 // 0..n_heads-1: q, then k heads, then v heads
  const int pos = tok_pos[t];
  const TI *row = qkv + (size_t)t * row_stride + (size_t)slot * d;
  const int half = rot_dim / 2;
  const bool is_v = slot >= n_heads + n_kv;
  const bool is_k = !is_v && slot >= n_heads;
  T *dst;
  if (is_k || is_v) {
    const int kvh = is_k ? slot - n_heads : slot - n_heads - n_kv;
    const int page = page_table[(size_t)tok_seq[t] * pt_stride + pos / page_size];
    T *base = is_k ? kcache : vcache;
    dst = base + (((size_t)page * n_kv + kvh) * page_size + (pos % page_size)) * d;
  } else {
    dst = q_out + (size_t)t * q_stride + (size_t)slot * d;
  }
  if (is_v) {
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = from_float<T>(to_float(row[i]));
    return;
  }
  const int p = pos < table_rows ? pos : table_rows - 1;   // the host refuses longer sequences
  const float *cs = table + (size_t)p * rot_dim;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float c = cs[i], s = cs[half + i];
    const float a = to_float(row[i]), b = to_float(row[i + half]);
    dst[i] = from_float<T>(a * c - b * s);
    dst[i + half] = from_float<T>(b * c + a * s);
  }
  // Channels beyond the rotated ones (rot_dim < d) pass through unchanged.
  for (int i = rot_dim + threadIdx.x; i < d; i += blockDim.x) dst[i] = from_float<T>(to_float(row[i]));
}

// The same with four channel pairs per thread and one CTA per token, for head sizes that are
// a multiple of 8 and rotate all of their channels: 16-byte loads, and the position and the
// page are looked up once per token.
template <typename TI, typename T>
__global__ void __launch_bounds__(256)
rope_cache_write_vec_kernel(const TI *__restrict__ qkv, long long row_stride, T *__restrict__ q_out,
                            long long q_stride, int n_heads, int n_kv, int d, const float *__restrict__ table,
                            int table_rows, const int *__restrict__ tok_seq, const int *__restrict__ tok_pos,
                            const int *__restrict__ page_table, int pt_stride, T *__restrict__ kcache,
                            T *__restrict__ vcache, int page_size, int n_slots) {
  grid_dependents_launch();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  const int half = d / 2, groups = half / 4;
  size_t cache_row = 0;
  if (n_slots > n_heads) {
    const int page = page_table[(size_t)tok_seq[t] * pt_stride + pos / page_size];
    cache_row = (size_t)page * n_kv * page_size + (pos % page_size);
  }
  const float *cs = table + (size_t)(pos < table_rows ? pos : table_rows - 1) * d;
  for (int item = threadIdx.x; item < n_slots * groups; item += blockDim.x) {
    const int slot = item / groups, j = (item % groups) * 4;
    const TI *row = qkv + (size_t)t * row_stride + (size_t)slot * d;
    const float4 a = ld4(row + j), b = ld4(row + j + half);
    const bool is_v = slot >= n_heads + n_kv;
    T *dst;
    if (slot < n_heads) {
      dst = q_out + (size_t)t * q_stride + (size_t)slot * d;
    } else {
      const int kvh = is_v ? slot - n_heads - n_kv : slot - n_heads;
      dst = (is_v ? vcache : kcache) + (cache_row + (size_t)kvh * page_size) * d;
    }
    if (is_v) {
      st4(dst + j, a);
      st4(dst + j + half, b);
    } else {
      const float4 c = ld4(cs + j), s = ld4(cs + half + j);
      st4(dst + j, make_float4(a.x * c.x - b.x * s.x, a.y * c.y - b.y * s.y, a.z * c.z - b.z * s.z, a.w * c.w - b.w * s.w));
      st4(dst + j + half, make_float4(b.x * c.x + a.x * s.x, b.y * c.y + a.y * s.y, b.z * c.z + a.z * s.z, b.w * c.w + a.w * s.w));
    }
  }
}

// in_dtype: type of qkv; dtype: type of q_out and of the cache.  With write_cache == 0
// only the query heads are processed (the layer reads another layer's keys and values).
LLM_EXPORT int llm_rope_cache_write(int in_dtype, int dtype, const void *qkv, long long row_stride,
                                    void *q_out, long long q_stride, int n_tokens, int n_heads,
                                    int n_kv, int d, const float *table, int table_rows, int rot_dim,
                                    const int *tok_seq, const int *tok_pos, const int *page_table,
                                    int pt_stride, void *kcache, void *vcache, int page_size,
                                    int write_cache, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv > 0 && d > 0, "rope: bad sizes");
  // rot_dim 0: nothing is rotated (a mixer without a position encoding); queries pass through and
  // keys and values are appended as they are
  LLM_REQUIRE(rot_dim % 2 == 0 && rot_dim <= d && rot_dim >= 0 && (rot_dim == 0 || table != nullptr),
              "rope: rotated width %d does not fit head size %d", rot_dim, d);
  LLM_REQUIRE(n_heads + 2 * n_kv <= 65535, "rope: too many heads for one launch");
  const int n_slots = write_cache ? n_heads + 2 * n_kv : n_heads;
  const bool vec = d % 8 == 0 && rot_dim == d && row_stride % 4 == 0 && q_stride % 4 == 0 &&
                   (uintptr_t)qkv % 16 == 0 && (uintptr_t)q_out % 16 == 0 && (uintptr_t)table % 16 == 0 &&
                   (uintptr_t)kcache % 16 == 0 && (uintptr_t)vcache % 16 == 0;
  if (vec) {
    const int items = n_slots * (d / 8);
    const int vthreads = items >= 256 ? 256 : (items + 31) / 32 * 32;
#define ROPE_VEC(TI, T)                                                                                  \
  llm_launch(rope_cache_write_vec_kernel<TI, T>, dim3(n_tokens), dim3(vthreads), 0, stream, (const TI *)qkv, \
             row_stride, (T *)q_out, q_stride, n_heads, n_kv, d, table, table_rows, tok_seq, tok_pos,    \
             page_table, pt_stride, (T *)kcache, (T *)vcache, page_size, n_slots)
    if (in_dtype == LLM_F32 && dtype == LLM_F32) ROPE_VEC(float, float);
    else if (in_dtype == LLM_F32 && dtype == LLM_BF16) ROPE_VEC(float, __nv_bfloat16);
    else if (in_dtype == LLM_BF16 && dtype == LLM_BF16) ROPE_VEC(__nv_bfloat16, __nv_bfloat16);
    else LLM_FAIL("rope: unsupported dtypes in %d out %d", in_dtype, dtype);
#undef ROPE_VEC
    LLM_CHECK_LAUNCH("rope_cache_write");
    return LLM_OK;
  }
  dim3 grid(n_tokens, n_slots);
  int threads = d / 2 >= 64 ? 64 : 32;
#define ROPE_LAUNCH(TI, T)                                                                              \
  llm_launch(rope_cache_write_kernel<TI, T>, grid, dim3(threads), 0, stream,                           \
      (const TI *)qkv, row_stride, (T *)q_out, q_stride, n_heads, n_kv, d, table, table_rows, rot_dim,  \
      tok_seq, tok_pos, page_table, pt_stride, (T *)kcache, (T *)vcache, page_size)
  if (in_dtype == LLM_F32 && dtype == LLM_F32) ROPE_LAUNCH(float, float);
  else if (in_dtype == LLM_F32 && dtype == LLM_BF16) ROPE_LAUNCH(float, __nv_bfloat16);
  else if (in_dtype == LLM_BF16 && dtype == LLM_BF16) ROPE_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else LLM_FAIL("rope: unsupported dtypes in %d out %d", in_dtype, dtype);
#undef ROPE_LAUNCH
  LLM_CHECK_LAUNCH("rope_cache_write");
  return LLM_OK;
}

// ---------------------------------------------------------------- norm of the whole projection + rotation + append
// For mixers that normalise their queries and keys before the rotation, and for values of another
// width than the keys.  A row of the stacked product is [q: n_heads * d | k: n_kv * d | v: n_kv * dv |
// anything else]; one CTA serves one token:
//   q <- q / sqrt(mean(q^2) + eps) * q_norm   over all n_heads * d channels at once (likewise k)
//   rotation of the first rot_dim channels of every q and k head (pairs i, i + rot_dim/2)
//   q -> q_out, k and v -> the token's row of the paged cache ([pages, kv_heads, page_size, d or dv]).
// Norm weights may be null (no norm) and rot_dim 0 (no rotation).  Sums, factors and angles are
// 32-bit; a sum's order is fixed by the thread count, not by the batch.
template <typename TI, typename T>
__global__ void __launch_bounds__(256)
qk_place_kernel(const TI *__restrict__ qkv, long long row_stride, T *__restrict__ q_out, long long q_stride,
                int n_heads, int n_kv, int d, int dv, const float *__restrict__ q_norm,
                const float *__restrict__ k_norm, float eps, const float *__restrict__ table, int table_rows,
                int rot_dim, const int *__restrict__ tok_seq, const int *__restrict__ tok_pos,
                const int *__restrict__ page_table, int pt_stride, T *__restrict__ kcache,
                T *__restrict__ vcache, int page_size, int write_cache) {
  __shared__ float scratch[256 / 32 + 1];
  grid_dependents_launch();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  const TI *row = qkv + (size_t)t * row_stride;
  const int qw = n_heads * d, kw = n_kv * d;
  float q_fac = 1.f, k_fac = 1.f;
  if (q_norm) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < qw; c += 256) {
      const float v = to_float(row[c]);
      ss = fmaf(v, v, ss);
    }
    q_fac = 1.f / sqrtf(block_sum<256>(ss, scratch) / (float)qw + eps);
  }
  if (k_norm && write_cache) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < kw; c += 256) {
      const float v = to_float(row[qw + c]);
      ss = fmaf(v, v, ss);
    }
    k_fac = 1.f / sqrtf(block_sum<256>(ss, scratch) / (float)kw + eps);
  }
  size_t cache_row = 0;
  if (write_cache) {
    const int page = page_table[(size_t)tok_seq[t] * pt_stride + pos / page_size];
    cache_row = (size_t)page * n_kv * page_size + (pos % page_size);
  }
  const int half = rot_dim / 2;
  const float *cs = table ? table + (size_t)(pos < table_rows ? pos : table_rows - 1) * rot_dim : nullptr;
  const int per_head = d - half;               // `half` pairs, then the channels that are not rotated
  const int n_rot = (n_heads + (write_cache ? n_kv : 0)) * per_head;
  for (int item = threadIdx.x; item < n_rot; item += 256) {
    const int slot = item / per_head, i = item - slot * per_head;
    const bool is_q = slot < n_heads;
    const TI *src = row + (size_t)slot * d;
    const float *nw = is_q ? (q_norm ? q_norm + (size_t)slot * d : nullptr) : (k_norm ? k_norm + (size_t)(slot - n_heads) * d : nullptr);
    const float fac = is_q ? q_fac : k_fac;
    T *dst = is_q ? q_out + (size_t)t * q_stride + (size_t)slot * d
                  : kcache + (cache_row + (size_t)(slot - n_heads) * page_size) * d;
    if (i < half) {
      float a = to_float(src[i]) * fac, b = to_float(src[i + half]) * fac;
      if (nw) {
        a *= nw[i];
        b *= nw[i + half];
      }
      const float c = cs[i], s = cs[half + i];
      dst[i] = from_float<T>(a * c - b * s);
      dst[i + half] = from_float<T>(b * c + a * s);
    } else {
      const int ch = i + half;
      float a = to_float(src[ch]) * fac;
      if (nw) a *= nw[ch];
      dst[ch] = from_float<T>(a);
    }
  }
  if (write_cache) {
    const TI *vsrc = row + qw + kw;
    for (int item = threadIdx.x; item < n_kv * dv; item += 256) {
      const int kvh = item / dv, ch = item - kvh * dv;
      vcache[(cache_row + (size_t)kvh * page_size) * dv + ch] = from_float<T>(to_float(vsrc[item]));
    }
  }
}

// The same four channels (or channel pairs) to a thread, for widths that are multiples of 4 (the
// rotated width of 8) and 16-byte aligned rows: both sums of squares go through one reduction.
template <typename TI, typename T>
__global__ void __launch_bounds__(256)
qk_place_vec_kernel(const TI *__restrict__ qkv, long long row_stride, T *__restrict__ q_out, long long q_stride,
                    int n_heads, int n_kv, int d, int dv, const float *__restrict__ q_norm,
                    const float *__restrict__ k_norm, float eps, const float *__restrict__ table, int table_rows,
                    int rot_dim, const int *__restrict__ tok_seq, const int *__restrict__ tok_pos,
                    const int *__restrict__ page_table, int pt_stride, T *__restrict__ kcache,
                    T *__restrict__ vcache, int page_size, int write_cache) {
  __shared__ float sq[256 / 32 + 1], sk[256 / 32 + 1];
  grid_dependents_launch();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  const TI *row = qkv + (size_t)t * row_stride;
  const int qw = n_heads * d, kw = n_kv * d;
  float q_fac = 1.f, k_fac = 1.f;
  if (q_norm) {
    float ssq = 0.f, ssk = 0.f;
    for (int c = threadIdx.x * 4; c < qw; c += 1024) {
      const float4 v = ld4(row + c);
      ssq = fmaf(v.x, v.x, ssq);
      ssq = fmaf(v.y, v.y, ssq);
      ssq = fmaf(v.z, v.z, ssq);
      ssq = fmaf(v.w, v.w, ssq);
    }
    if (write_cache)
      for (int c = threadIdx.x * 4; c < kw; c += 1024) {
        const float4 v = ld4(row + qw + c);
        ssk = fmaf(v.x, v.x, ssk);
        ssk = fmaf(v.y, v.y, ssk);
        ssk = fmaf(v.z, v.z, ssk);
        ssk = fmaf(v.w, v.w, ssk);
      }
    // warps first, then the warp totals in warp order (a fixed order of additions)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    ssq = warp_sum(ssq);
    ssk = warp_sum(ssk);
    if (lane == 0) {
      sq[warp] = ssq;
      sk[warp] = ssk;
    }
    __syncthreads();
    if (warp == 0) {
      float a = lane < 8 ? sq[lane] : 0.f, b = lane < 8 ? sk[lane] : 0.f;
      a = warp_sum(a);
      b = warp_sum(b);
      if (lane == 0) {
        sq[8] = a;
        sk[8] = b;
      }
    }
    __syncthreads();
    q_fac = 1.f / sqrtf(sq[8] / (float)qw + eps);
    k_fac = 1.f / sqrtf(sk[8] / (float)kw + eps);
  }
  size_t cache_row = 0;
  if (write_cache) {
    const int page = page_table[(size_t)tok_seq[t] * pt_stride + pos / page_size];
    cache_row = (size_t)page * n_kv * page_size + (pos % page_size);
  }
  const int half = rot_dim / 2;
  const float *cs = table ? table + (size_t)(pos < table_rows ? pos : table_rows - 1) * rot_dim : nullptr;
  const int per_head = (d - half) / 4;          // groups of four: `half / 4` of pairs, then channels that are not rotated
  const int n_rot = (n_heads + (write_cache ? n_kv : 0)) * per_head;
  for (int item = threadIdx.x; item < n_rot; item += 256) {
    const int slot = item / per_head, i = (item - slot * per_head) * 4;
    const bool is_q = slot < n_heads;
    const TI *src = row + (size_t)slot * d;
    const float *nw = is_q ? (q_norm ? q_norm + (size_t)slot * d : nullptr) : (k_norm ? k_norm + (size_t)(slot - n_heads) * d : nullptr);
    const float fac = is_q ? q_fac : k_fac;
    T *dst = is_q ? q_out + (size_t)t * q_stride + (size_t)slot * d
                  : kcache + (cache_row + (size_t)(slot - n_heads) * page_size) * d;
    if (i < half) {
      float4 a = ld4(src + i), b = ld4(src + i + half);
      a = make_float4(a.x * fac, a.y * fac, a.z * fac, a.w * fac);
      b = make_float4(b.x * fac, b.y * fac, b.z * fac, b.w * fac);
      if (nw) {
        const float4 wa = ld4(nw + i), wb = ld4(nw + i + half);
        a = make_float4(a.x * wa.x, a.y * wa.y, a.z * wa.z, a.w * wa.w);
        b = make_float4(b.x * wb.x, b.y * wb.y, b.z * wb.z, b.w * wb.w);
      }
      const float4 c = ld4(cs + i), s = ld4(cs + half + i);
      st4(dst + i, make_float4(a.x * c.x - b.x * s.x, a.y * c.y - b.y * s.y, a.z * c.z - b.z * s.z, a.w * c.w - b.w * s.w));
      st4(dst + i + half, make_float4(b.x * c.x + a.x * s.x, b.y * c.y + a.y * s.y, b.z * c.z + a.z * s.z, b.w * c.w + a.w * s.w));
    } else {
      const int ch = i + half;
      float4 a = ld4(src + ch);
      a = make_float4(a.x * fac, a.y * fac, a.z * fac, a.w * fac);
      if (nw) {
        const float4 wa = ld4(nw + ch);
        a = make_float4(a.x * wa.x, a.y * wa.y, a.z * wa.z, a.w * wa.w);
      }
      st4(dst + ch, a);
    }
  }
  if (write_cache) {
    const TI *vsrc = row + qw + kw;
    const int dv4 = dv / 4;
    for (int item = threadIdx.x; item < n_kv * dv4; item += 256) {
      const int kvh = item / dv4, ch = (item - kvh * dv4) * 4;
      st4(vcache + (cache_row + (size_t)kvh * page_size) * dv + ch, ld4(vsrc + (size_t)kvh * dv + ch));
    }
  }
}

LLM_EXPORT int llm_qk_place(int in_dtype, int dtype, const void *qkv, long long row_stride, void *q_out,
                            long long q_stride, int n_tokens, int n_heads, int n_kv, int d, int dv,
                            const float *q_norm, const float *k_norm, float eps, const float *table,
                            int table_rows, int rot_dim, const int *tok_seq, const int *tok_pos,
                            const int *page_table, int pt_stride, void *kcache, void *vcache, int page_size,
                            int write_cache, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv > 0 && d > 0 && dv > 0, "qk_place: bad sizes");
  LLM_REQUIRE(rot_dim % 2 == 0 && rot_dim <= d && rot_dim >= 0 && (rot_dim == 0 || table != nullptr),
              "qk_place: rotated width %d does not fit head size %d", rot_dim, d);
  LLM_REQUIRE(row_stride >= (long long)n_heads * d + (long long)n_kv * (d + dv), "qk_place: the stacked rows are too short");
  LLM_REQUIRE((q_norm == nullptr) == (k_norm == nullptr), "qk_place: the norm has weights for both q and k or for neither");
  const bool vec = d % 4 == 0 && dv % 4 == 0 && rot_dim % 8 == 0 && row_stride % 4 == 0 && q_stride % 4 == 0 &&
                   (uintptr_t)qkv % 16 == 0 && (uintptr_t)q_out % 16 == 0 && (uintptr_t)table % 16 == 0 &&
                   (uintptr_t)kcache % 16 == 0 && (uintptr_t)vcache % 16 == 0 && (uintptr_t)q_norm % 16 == 0 &&
                   (uintptr_t)k_norm % 16 == 0 && ((long long)n_heads * d) % 4 == 0;
#define QK_PLACE(TI, T)                                                                                          \
  llm_launch(vec ? qk_place_vec_kernel<TI, T> : qk_place_kernel<TI, T>, dim3(n_tokens), dim3(256), 0, stream, (const TI *)qkv, row_stride, (T *)q_out, \
             q_stride, n_heads, n_kv, d, dv, q_norm, k_norm, eps, table, table_rows, rot_dim, tok_seq, tok_pos,  \
             page_table, pt_stride, (T *)kcache, (T *)vcache, page_size, write_cache)
  if (in_dtype == LLM_F32 && dtype == LLM_F32) QK_PLACE(float, float);
  else if (in_dtype == LLM_F32 && dtype == LLM_BF16) QK_PLACE(float, __nv_bfloat16);
  else if (in_dtype == LLM_BF16 && dtype == LLM_BF16) QK_PLACE(__nv_bfloat16, __nv_bfloat16);
  else LLM_FAIL("qk_place: unsupported dtypes in %d out %d", in_dtype, dtype);
#undef QK_PLACE
  LLM_CHECK_LAUNCH("qk_place");
  return LLM_OK;
}

// ---------------------------------------------------------------- placing without rotation: bias, value norm
// Rows [q | k | v (n_kv * dv) | ...] of a stacked product whose matrix has biases and whose
// attention uses no rotation: the bias (32-bit, one value per stacked row of the matrix; null:
// none) is added here, in 32-bit, so that the product itself can run without one; each value head
// is divided by its root mean square over dv, sqrt(mean(v^2) + v_eps), when v_eps >= 0 (no
// weight), and is cached so.  q goes to q_out, k and v to the cache.  A CTA a token; a warp takes
// a value head at a time (sum in lane order, then the shuffle tree).
template <typename TI, typename T, bool VEC>
__global__ void __launch_bounds__(256)
kv_place_kernel(const TI *__restrict__ qkv, long long row_stride, T *__restrict__ q_out, long long q_stride, int n_heads,
                int n_kv, int d, int dv, const float *__restrict__ bias, float v_eps, const int *__restrict__ tok_seq,
                const int *__restrict__ tok_pos, const int *__restrict__ page_table, int pt_stride, T *__restrict__ kcache,
                T *__restrict__ vcache, int page_size, int write_cache) {
  grid_dependents_launch();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const TI *row = qkv + (size_t)t * row_stride;
  const int qw = n_heads * d, kw = n_kv * d;
  auto add4 = [](float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); };
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  if (VEC) {
    for (int c = threadIdx.x * 4; c < qw; c += 1024) st4(q_out + (size_t)t * q_stride + c, add4(ld4(row + c), bias ? ld4(bias + c) : zero4));
  } else {
    for (int c = threadIdx.x; c < qw; c += 256)
      q_out[(size_t)t * q_stride + c] = from_float<T>(to_float(row[c]) + (bias ? bias[c] : 0.f));
  }
  if (!write_cache) return;
  const int pos = tok_pos[t];
  const int page = page_table[(size_t)tok_seq[t] * pt_stride + pos / page_size];
  const size_t cache_row = (size_t)page * n_kv * page_size + (pos % page_size);
  if (VEC) {
    for (int c = threadIdx.x * 4; c < kw; c += 1024) {
      const int kvh = c / d, ch = c - kvh * d;
      st4(kcache + (cache_row + (size_t)kvh * page_size) * d + ch, add4(ld4(row + qw + c), bias ? ld4(bias + qw + c) : zero4));
    }
  } else {
    for (int c = threadIdx.x; c < kw; c += 256) {
      const int kvh = c / d, ch = c - kvh * d;
      kcache[(cache_row + (size_t)kvh * page_size) * d + ch] = from_float<T>(to_float(row[qw + c]) + (bias ? bias[qw + c] : 0.f));
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int kvh = warp; kvh < n_kv; kvh += 8) {
    const TI *v = row + qw + kw + (size_t)kvh * dv;
    const float *vb = bias ? bias + qw + kw + (size_t)kvh * dv : nullptr;
    T *dst = vcache + (cache_row + (size_t)kvh * page_size) * dv;
    if (VEC) {                                        // four channels to a lane, heads of up to 256 channels
      float4 x[2];
      float ss = 0.f;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int i = (lane + 32 * r) * 4;
        x[r] = i < dv ? add4(ld4(v + i), vb ? ld4(vb + i) : zero4) : zero4;
        ss = fmaf(x[r].x, x[r].x, ss);
        ss = fmaf(x[r].y, x[r].y, ss);
        ss = fmaf(x[r].z, x[r].z, ss);
        ss = fmaf(x[r].w, x[r].w, ss);
      }
      const float inv = v_eps >= 0.f ? 1.f / sqrtf(warp_sum(ss) / (float)dv + v_eps) : 1.f;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int i = (lane + 32 * r) * 4;
        if (i < dv) st4(dst + i, make_float4(x[r].x * inv, x[r].y * inv, x[r].z * inv, x[r].w * inv));
      }
      continue;
    }
    float inv = 1.f;
    if (v_eps >= 0.f) {
      float ss = 0.f;
      for (int i = lane; i < dv; i += 32) {
        const float x = to_float(v[i]) + (vb ? vb[i] : 0.f);
        ss = fmaf(x, x, ss);
      }
      ss = warp_sum(ss);
      inv = 1.f / sqrtf(ss / (float)dv + v_eps);
    }
    for (int i = lane; i < dv; i += 32) dst[i] = from_float<T>((to_float(v[i]) + (vb ? vb[i] : 0.f)) * inv);
  }
}

LLM_EXPORT int llm_kv_place(int in_dtype, int dtype, const void *qkv, long long row_stride, void *q_out, long long q_stride,
                            int n_tokens, int n_heads, int n_kv, int d, int dv, const float *bias, float v_eps,
                            const int *tok_seq, const int *tok_pos, const int *page_table, int pt_stride, void *kcache,
                            void *vcache, int page_size, int write_cache, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv > 0 && d > 0 && dv > 0, "kv_place: bad sizes");
  LLM_REQUIRE(row_stride >= (long long)n_heads * d + (long long)n_kv * (d + dv), "kv_place: the stacked rows are too short");
  // four channels to a thread where widths are multiples of 4 and rows start on 16 bytes
  const bool vec = d % 4 == 0 && dv % 4 == 0 && dv <= 256 && row_stride % 4 == 0 && q_stride % 4 == 0 && (uintptr_t)qkv % 16 == 0 &&
                   (uintptr_t)q_out % 16 == 0 && (uintptr_t)bias % 16 == 0 && (uintptr_t)kcache % 16 == 0 && (uintptr_t)vcache % 16 == 0;
#define KV_PLACE(TI, T)                                                                                                  \
  if (vec)                                                                                                               \
    llm_launch(kv_place_kernel<TI, T, true>, dim3(n_tokens), dim3(256), 0, stream, (const TI *)qkv, row_stride, (T *)q_out, q_stride, \
               n_heads, n_kv, d, dv, bias, v_eps, tok_seq, tok_pos, page_table, pt_stride, (T *)kcache, (T *)vcache, page_size, \
               write_cache);                                                                                             \
  else                                                                                                                   \
    llm_launch(kv_place_kernel<TI, T, false>, dim3(n_tokens), dim3(256), 0, stream, (const TI *)qkv, row_stride, (T *)q_out, q_stride, \
             n_heads, n_kv, d, dv, bias, v_eps, tok_seq, tok_pos, page_table, pt_stride, (T *)kcache, (T *)vcache, page_size, \
             write_cache)
  if (in_dtype == LLM_F32 && dtype == LLM_F32) { KV_PLACE(float, float); }
  else if (in_dtype == LLM_F32 && dtype == LLM_BF16) { KV_PLACE(float, __nv_bfloat16); }
  else if (in_dtype == LLM_BF16 && dtype == LLM_BF16) { KV_PLACE(__nv_bfloat16, __nv_bfloat16); }
  else LLM_FAIL("kv_place: unsupported dtypes in %d out %d", in_dtype, dtype);
#undef KV_PLACE
  LLM_CHECK_LAUNCH("kv_place");
  return LLM_OK;
}

// ---------------------------------------------------------------- rotation in neighbouring pairs, bias, values from keys
// Rows [q: n_heads * d | k: n_kv * d | v: n_kv * dv] of a stacked product.  `bias` (32-bit, one value per
// column of the row; null: none) is added first, in 32-bit.  The first rot_dim channels of every q and k
// head are rotated in pairs (2i, 2i + 1) by the angle of pair i, whose cosine is table[p][i] and whose
// sine is table[p][rot_dim/2 + i]:  (u, v) -> (u cos - v sin, v cos + u sin); the other channels pass.
// q goes to q_out, k to the token's row of the paged key cache.  With values_from_keys the rows have no v
// part and the value cache gets the key as projected (bias added, not rotated), so dv = d; otherwise v is
// copied.  One CTA a token, two neighbouring channels to a thread at a time.
template <typename TI, typename T>
__global__ void __launch_bounds__(256)
rope_pairs_place_kernel(const TI *__restrict__ qkv, long long row_stride, T *__restrict__ q_out, long long q_stride, int n_heads,
                        int n_kv, int d, int dv, const float *__restrict__ bias, int values_from_keys,
                        const float *__restrict__ table, int table_rows, int rot_dim, const int *__restrict__ tok_seq,
                        const int *__restrict__ tok_pos, const int *__restrict__ page_table, int pt_stride, T *__restrict__ kcache,
                        T *__restrict__ vcache, int page_size, int write_cache) {
  grid_dependents_launch();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const TI *row = qkv + (size_t)t * row_stride;
  const int pos = tok_pos[t];
  size_t cache_row = 0;
  if (write_cache) {
    const int page = page_table[(size_t)tok_seq[t] * pt_stride + pos / page_size];
    cache_row = (size_t)page * n_kv * page_size + (pos % page_size);
  }
  const int half = rot_dim / 2;
  const float *cs = rot_dim > 0 ? table + (size_t)(pos < table_rows ? pos : table_rows - 1) * rot_dim : nullptr;
  const int units = (d + 1) / 2;                     // two channels each; the last one may hold a single channel
  const int n_slots = n_heads + (write_cache ? n_kv : 0);
  for (int item = threadIdx.x; item < n_slots * units; item += 256) {
    const int slot = item / units, u = item - slot * units;
    const int c0 = 2 * u, col = slot * d + c0;
    const bool two = c0 + 1 < d;
    const float a = to_float(row[col]) + (bias ? bias[col] : 0.f);
    const float b = two ? to_float(row[col + 1]) + (bias ? bias[col + 1] : 0.f) : 0.f;
    float ra = a, rb = b;
    if (c0 + 1 < rot_dim) {
      const float c = cs[u], sn = cs[half + u];
      ra = a * c - b * sn;
      rb = b * c + a * sn;
    }
    if (slot < n_heads) {
      T *dst = q_out + (size_t)t * q_stride + col;
      dst[0] = from_float<T>(ra);
      if (two) dst[1] = from_float<T>(rb);
    } else {
      const int kvh = slot - n_heads;
      T *dst = kcache + (cache_row + (size_t)kvh * page_size) * d + c0;
      dst[0] = from_float<T>(ra);
      if (two) dst[1] = from_float<T>(rb);
      if (values_from_keys) {
        T *vd = vcache + (cache_row + (size_t)kvh * page_size) * d + c0;
        vd[0] = from_float<T>(a);
        if (two) vd[1] = from_float<T>(b);
      }
    }
  }
  if (write_cache && !values_from_keys) {
    const int v0 = (n_heads + n_kv) * d;
    for (int c = threadIdx.x; c < n_kv * dv; c += 256) {
      const int kvh = c / dv, ch = c - kvh * dv;
      vcache[(cache_row + (size_t)kvh * page_size) * dv + ch] = from_float<T>(to_float(row[v0 + c]) + (bias ? bias[v0 + c] : 0.f));
    }
  }
}

LLM_EXPORT int llm_rope_pairs_place(int in_dtype, int dtype, const void *qkv, long long row_stride, void *q_out, long long q_stride,
                                    int n_tokens, int n_heads, int n_kv, int d, int dv, const float *bias, int values_from_keys,
                                    const float *table, int table_rows, int rot_dim, const int *tok_seq, const int *tok_pos,
                                    const int *page_table, int pt_stride, void *kcache, void *vcache, int page_size, int write_cache,
                                    cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv > 0 && d > 0 && dv > 0, "rope_pairs_place: bad sizes");
  LLM_REQUIRE(rot_dim >= 0 && rot_dim % 2 == 0 && rot_dim <= d && (rot_dim == 0 || (table != nullptr && table_rows > 0)),
              "rope_pairs_place: rotated width %d does not fit head size %d", rot_dim, d);
  LLM_REQUIRE(!values_from_keys || dv == d, "rope_pairs_place: values that are the keys have the keys' width");
  LLM_REQUIRE(row_stride >= (long long)(n_heads + n_kv) * d + (values_from_keys ? 0LL : (long long)n_kv * dv),
              "rope_pairs_place: the stacked rows are too short");
#define PAIRS_PLACE(TI, T)                                                                                               \
  llm_launch(rope_pairs_place_kernel<TI, T>, dim3(n_tokens), dim3(256), 0, stream, (const TI *)qkv, row_stride, (T *)q_out, q_stride, \
             n_heads, n_kv, d, dv, bias, values_from_keys, table, table_rows, rot_dim, tok_seq, tok_pos, page_table, pt_stride, \
             (T *)kcache, (T *)vcache, page_size, write_cache)
  if (in_dtype == LLM_F32 && dtype == LLM_F32) PAIRS_PLACE(float, float);
  else if (in_dtype == LLM_F32 && dtype == LLM_BF16) PAIRS_PLACE(float, __nv_bfloat16);
  else if (in_dtype == LLM_BF16 && dtype == LLM_BF16) PAIRS_PLACE(__nv_bfloat16, __nv_bfloat16);
  else LLM_FAIL("rope_pairs_place: unsupported dtypes in %d out %d", in_dtype, dtype);
#undef PAIRS_PLACE
  LLM_CHECK_LAUNCH("rope_pairs_place");
  return LLM_OK;
}

// ---------------------------------------------------------------- rotation, then a unit norm per head, + append
// For mixers that divide every query and key head by its root mean square AFTER the rotation (no weight):
//   rotation of the first rot_dim channels of every q and k head (pairs i, i + rot_dim/2; the table's row may
//   carry a factor on cosines and sines alike), then head <- head / sqrt(mean(head^2) + eps) over its d channels
//   (eps < 0: no norm), q -> q_out, k and v -> the token's row of the paged cache; values of width dv as they are.
// A row of the stacked product is [q: n_heads * d | k: n_kv * d | v: n_kv * dv | anything else].  One CTA per
// token, a few lanes per head; a head's channels stay in registers between the rotation and the norm
// (d - rot_dim/2 <= 512).  Angles come from the table (computed in 64-bit, rounded once); sums and factors are 32-bit and
// a head's sum has a fixed order.
// LANES lanes share a head (8, 16 or 32: the fewer, the more heads a warp has in flight at once), ITEMS items each; an
// item is V consecutive pairs (or unrotated channels): V = 4 where the widths are multiples of 4 and rows lie on 16 bytes.
template <typename TI, typename T, int LANES, int ITEMS, int V>
__global__ void __launch_bounds__(256)
rope_headnorm_place_kernel(const TI *__restrict__ qkv, long long row_stride, T *__restrict__ q_out, long long q_stride, int n_heads,
                           int n_kv, int d, int dv, float eps, const float *__restrict__ table, int table_rows, int rot_dim,
                           const int *__restrict__ tok_seq, const int *__restrict__ tok_pos, const int *__restrict__ page_table,
                           int pt_stride, T *__restrict__ kcache, T *__restrict__ vcache, int page_size, int write_cache) {
  grid_dependents_launch();
  grid_dependency_wait();
  constexpr int PER_WARP = 32 / LANES;
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane % LANES, group = lane / LANES;
  const int pos = tok_pos[t];
  const TI *row = qkv + (size_t)t * row_stride;
  const int qw = n_heads * d, kw = n_kv * d;
  size_t cache_row = 0;
  if (write_cache) {
    const int page = page_table[(size_t)tok_seq[t] * pt_stride + pos / page_size];
    cache_row = (size_t)page * n_kv * page_size + (pos % page_size);
  }
  const int half = rot_dim / 2;
  const float *cs = table ? table + (size_t)(pos < table_rows ? pos : table_rows - 1) * rot_dim : nullptr;
  const int per_head = d - half;               // `half` pairs, then the channels that are not rotated
  const int n_slots = n_heads + (write_cache ? n_kv : 0);
  // every lane of a warp goes through the same number of rounds: the shuffles below are the whole warp's
  for (int base = warp * PER_WARP; base < n_slots; base += 8 * PER_WARP) {
    const int slot = base + group;
    const bool live = slot < n_slots;
    const bool is_q = slot < n_heads;
    const TI *src = row + (size_t)(live ? slot : 0) * d;
    float a[ITEMS][V], b[ITEMS][V];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const int i = (sub + LANES * k) * V;
#pragma unroll
      for (int e = 0; e < V; ++e) a[k][e] = b[k][e] = 0.f;
      if (live && i < per_head) {
        if (i < half) {
          float u[V], v[V], c[V], sn[V];
          if (V == 4) {
            const float4 u4 = ld4(src + i), v4 = ld4(src + i + half), c4 = ld4(cs + i), s4 = ld4(cs + half + i);
            u[0] = u4.x, u[1 % V] = u4.y, u[2 % V] = u4.z, u[3 % V] = u4.w;
            v[0] = v4.x, v[1 % V] = v4.y, v[2 % V] = v4.z, v[3 % V] = v4.w;
            c[0] = c4.x, c[1 % V] = c4.y, c[2 % V] = c4.z, c[3 % V] = c4.w;
            sn[0] = s4.x, sn[1 % V] = s4.y, sn[2 % V] = s4.z, sn[3 % V] = s4.w;
          } else {
            u[0] = to_float(src[i]), v[0] = to_float(src[i + half]), c[0] = cs[i], sn[0] = cs[half + i];
          }
#pragma unroll
          for (int e = 0; e < V; ++e) {
            a[k][e] = u[e] * c[e] - v[e] * sn[e];
            b[k][e] = v[e] * c[e] + u[e] * sn[e];
          }
        } else {
          if (V == 4) {
            const float4 u4 = ld4(src + i + half);
            a[k][0] = u4.x, a[k][1 % V] = u4.y, a[k][2 % V] = u4.z, a[k][3 % V] = u4.w;
          } else {
            a[k][0] = to_float(src[i + half]);
          }
        }
#pragma unroll
        for (int e = 0; e < V; ++e) {
          ss = fmaf(a[k][e], a[k][e], ss);
          ss = fmaf(b[k][e], b[k][e], ss);
        }
      }
    }
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float fac = eps >= 0.f ? 1.f / sqrtf(ss / (float)d + eps) : 1.f;
    if (!live) continue;
    T *dst = is_q ? q_out + (size_t)t * q_stride + (size_t)slot * d : kcache + (cache_row + (size_t)(slot - n_heads) * page_size) * d;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const int i = (sub + LANES * k) * V;
      if (i < per_head) {
        if (V == 4) {
          st4(dst + (i < half ? i : i + half), make_float4(a[k][0] * fac, a[k][1 % V] * fac, a[k][2 % V] * fac, a[k][3 % V] * fac));
          if (i < half) st4(dst + i + half, make_float4(b[k][0] * fac, b[k][1 % V] * fac, b[k][2 % V] * fac, b[k][3 % V] * fac));
        } else if (i < half) {
          dst[i] = from_float<T>(a[k][0] * fac);
          dst[i + half] = from_float<T>(b[k][0] * fac);
        } else {
          dst[i + half] = from_float<T>(a[k][0] * fac);
        }
      }
    }
  }
  if (write_cache) {
    const TI *vsrc = row + qw + kw;
    if (V == 4) {
      const int dv4 = dv / 4;
      for (int item = threadIdx.x; item < n_kv * dv4; item += 256) {
        const int kvh = item / dv4, ch = (item - kvh * dv4) * 4;
        st4(vcache + (cache_row + (size_t)kvh * page_size) * dv + ch, ld4(vsrc + (size_t)kvh * dv + ch));
      }
    } else {
      for (int item = threadIdx.x; item < n_kv * dv; item += 256) {
        const int kvh = item / dv, ch = item - kvh * dv;
        vcache[(cache_row + (size_t)kvh * page_size) * dv + ch] = from_float<T>(to_float(vsrc[item]));
      }
    }
  }
}

LLM_EXPORT int llm_rope_headnorm_place(int in_dtype, int dtype, const void *qkv, long long row_stride, void *q_out, long long q_stride,
                                       int n_tokens, int n_heads, int n_kv, int d, int dv, float eps, const float *table, int table_rows,
                                       int rot_dim, const int *tok_seq, const int *tok_pos, const int *page_table, int pt_stride,
                                       void *kcache, void *vcache, int page_size, int write_cache, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv > 0 && d > 0 && dv > 0, "rope_headnorm_place: bad sizes");
  LLM_REQUIRE(rot_dim % 2 == 0 && rot_dim <= d && rot_dim >= 0 && (rot_dim == 0 || table != nullptr),
              "rope_headnorm_place: rotated width %d does not fit head size %d", rot_dim, d);
  const int per_head = d - rot_dim / 2;
  LLM_REQUIRE(per_head <= 32 * 16, "rope_headnorm_place: heads of %d channels are not supported", d);
  LLM_REQUIRE(row_stride >= (long long)n_heads * d + (long long)n_kv * (d + dv), "rope_headnorm_place: the stacked rows are too short");
  // four channels to a load where every width is a multiple of 4 and every row starts on 16 bytes
  const bool vec = d % 4 == 0 && dv % 4 == 0 && rot_dim % 8 == 0 && row_stride % 4 == 0 && q_stride % 4 == 0 && (uintptr_t)qkv % 16 == 0 &&
                   (uintptr_t)q_out % 16 == 0 && (uintptr_t)table % 16 == 0 && (uintptr_t)kcache % 16 == 0 && (uintptr_t)vcache % 16 == 0 &&
                   ((long long)n_heads * d) % 4 == 0 && ((long long)n_kv * d) % 4 == 0;
#define HN_GO(TI, T, LANES, ITEMS, V)                                                                                            \
  llm_launch(rope_headnorm_place_kernel<TI, T, LANES, ITEMS, V>, dim3(n_tokens), dim3(256), 0, stream, (const TI *)qkv, row_stride, \
             (T *)q_out, q_stride, n_heads, n_kv, d, dv, eps, table, table_rows, rot_dim, tok_seq, tok_pos, page_table,            \
             pt_stride, (T *)kcache, (T *)vcache, page_size, write_cache)
#define HN_PLACE(TI, T)                                                \
  do {                                                                 \
    if (vec && per_head <= 64) HN_GO(TI, T, 8, 2, 4);                  \
    else if (vec && per_head <= 128) HN_GO(TI, T, 16, 2, 4);           \
    else if (vec) HN_GO(TI, T, 32, 4, 4);                              \
    else if (per_head <= 64) HN_GO(TI, T, 8, 8, 1);                    \
    else if (per_head <= 128) HN_GO(TI, T, 16, 8, 1);                  \
    else HN_GO(TI, T, 32, 16, 1);                                      \
  } while (0)
  if (in_dtype == LLM_F32 && dtype == LLM_F32) HN_PLACE(float, float);
  else if (in_dtype == LLM_F32 && dtype == LLM_BF16) HN_PLACE(float, __nv_bfloat16);
  else if (in_dtype == LLM_BF16 && dtype == LLM_BF16) HN_PLACE(__nv_bfloat16, __nv_bfloat16);
  else LLM_FAIL("rope_headnorm_place: unsupported dtypes in %d out %d", in_dtype, dtype);
#undef HN_GO
#undef HN_PLACE
  LLM_CHECK_LAUNCH("rope_headnorm_place");
  return LLM_OK;
}
