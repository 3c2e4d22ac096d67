// Routed feed-forward (mixture of experts): choice of experts, grouping of (token, choice) rows
// by expert, and the experts' two products.
//
// A token's router logits z [experts] (a product, computed elsewhere in 32-bit) give scores
// sigmoid(z) or softmax(z); the `top` largest are chosen (the lower index on equal scores) and the
// chosen scores, optionally divided by their sum, are the weights.  Row r = token * top + choice.
//
// The experts are small two-matrix feed-forwards without biases, down(act(up(x))); the weight of a
// row multiplies either the expert's input or its output.  Since up has no bias, up(w x) = w up(x),
// so "input" is applied to the 32-bit result of the first product, before the activation, and
// "output" after it (down is linear too); neither rounds a scaled input to 16 bits.
// Gated experts, down(act(gate(x)) * up(x)): `up` then holds both matrices of an expert, rows
// interleaved ([experts, 2 ff, width]: row 2n of gate, row 2n + 1 of up), so that a tile of the first
// product holds a feature's two halves side by side; the weight goes on the output.
//
// Two forms of the products:
//  * moe_rows_kernel: one CTA per row, both products on the CUDA cores in 32-bit arithmetic
//    (float or bfloat16 operands).  The true 32-bit path, and widths the tiled form does not take.
//  * moe_grouped_kernel: rows sorted by expert (moe_sort_kernel) and multiplied tile by tile with
//    mma.sync m16n8k16 (bfloat16 operands, 32-bit accumulation): 64 rows x 128 weight rows per
//    CTA, K in steps of 32 through a three-stage cp.async ring.  The first product gathers its
//    rows from the tokens, scales, applies the activation and stores bfloat16 in sorted order; the
//    second reads those and scatters its 32-bit rows to out[choice][token].
// A row's result does not depend on which other rows the step has: each output element is one
// accumulator with a fixed order over K, and the results of a token's choices are kept apart
// ([top, tokens, width]) for the consumer to add in order.
#include "common.cuh"
#include "mma_tiles.cuh"
#include <math.h>

LLM_DEFINE_LAST_ERROR(llm_moe_last_error)

enum { ACT_GELU_ERF = 0, ACT_GELU_TANH = 1, ACT_SILU = 2, ACT_RELU2 = 3 };

__device__ __forceinline__ float activate(float z, int kind) {
  if (kind == ACT_GELU_ERF) return 0.5f * z * (1.f + erff(z * 0.70710678118654752f));
  if (kind == ACT_GELU_TANH) return 0.5f * z * (1.f + tanhf(0.79788456080286536f * (z + 0.044715f * z * z * z)));
  if (kind == ACT_RELU2) return z > 0.f ? z * z : 0.f;     // the square of max(z, 0)
  return z / (1.f + expf(-z));
}

// ---------------------------------------------------------------- choice of experts
// One warp per token.  score_kind 0: sigmoid, 1: softmax over all experts.
__global__ void moe_route_kernel(const float *__restrict__ logits, long long ld, int n_tokens, int n_experts, int top,
                                 int score_kind, int renormalize, int *__restrict__ chosen, float *__restrict__ weight) {
  grid_dependents_launch();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= n_tokens) return;
  const float *z = logits + (size_t)t * ld;
  float zmax = -INFINITY, denom = 1.f;
  if (score_kind == 1) {
    for (int e = lane; e < n_experts; e += 32) zmax = fmaxf(zmax, z[e]);
    zmax = warp_max(zmax);
    float s = 0.f;
    for (int e = lane; e < n_experts; e += 32) s += expf(z[e] - zmax);
    denom = warp_sum(s);
  }
  float total = 0.f;
  unsigned long long taken_lo = 0ull;           // bit i: this lane's expert lane + 32 i is taken
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane, i = 0; e < n_experts; e += 32, ++i) {
      if (i < 64 && ((taken_lo >> i) & 1ull)) continue;
      const float v = z[e];
      if (v > best) {
        best = v;
        best_e = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
    if ((best_e & 31) == lane) taken_lo |= 1ull << (best_e >> 5);
    const float s = score_kind == 1 ? expf(best - zmax) / denom : 1.f / (1.f + expf(-best));
    total += s;
    if (lane == 0) {
      chosen[(size_t)t * top + j] = best_e;
      weight[(size_t)t * top + j] = s;
    }
  }
  if (renormalize) {
    __syncwarp();
    for (int j = lane; j < top; j += 32) weight[(size_t)t * top + j] /= total;
  }
}

LLM_EXPORT int llm_moe_route(const float *logits, long long ld, int n_tokens, int n_experts, int top, int score_kind,
                             int renormalize, int *chosen, float *weight, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_experts > 0 && top > 0 && top <= n_experts, "moe_route: %d of %d experts", top, n_experts);
  LLM_REQUIRE(n_experts <= 2048, "moe_route: at most 2048 experts (%d)", n_experts);
  LLM_REQUIRE(score_kind == 0 || score_kind == 1, "moe_route: unknown score %d", score_kind);
  const int warps = 4;
  llm_launch(moe_route_kernel, dim3((n_tokens + warps - 1) / warps), dim3(warps * 32), 0, stream, logits, ld, n_tokens, n_experts,
             top, score_kind, renormalize, chosen, weight);
  LLM_CHECK_LAUNCH("moe_route");
  return LLM_OK;
}

// ---------------------------------------------------------------- choice among the best groups, by corrected scores
// One warp per token.  Scores s = sigmoid(z) (score_kind 0) or softmax(z) (1).  The CHOICE is made on c = s +
// correction (a vector over the experts; null: c = s); the WEIGHTS are the chosen experts' s.  With n_groups > 1
// the experts form n_groups equal groups of neighbours, a group's score is the sum of its `group_top` largest c,
// and only experts of the `keep` best groups can be chosen: the others' c count as minus infinity (c may be
// negative, so nought would not do).  Weights: s, or with `renormalize` s / (sum of the chosen s + norm_eps), then
// times route_scale.  Ties go to the lower index.  Everything is 32-bit; a token's result depends on its row alone.
__global__ void moe_route_grouped_kernel(const float *__restrict__ logits, long long ld, int n_tokens, int n_experts, int top,
                                         int score_kind, const float *__restrict__ correction, int n_groups, int keep,
                                         int group_top, int renormalize, float norm_eps, float route_scale,
                                         int *__restrict__ chosen, float *__restrict__ weight) {
  extern __shared__ float route_sh[];            // per warp: c [E], group scores [n_groups]
  grid_dependents_launch();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= n_tokens) return;
  float *c = route_sh + (size_t)warp * (n_experts + n_groups), *gs = c + n_experts;
  const float *z = logits + (size_t)t * ld;
  float zmax = -INFINITY, denom = 1.f;
  if (score_kind == 1) {
    for (int e = lane; e < n_experts; e += 32) zmax = fmaxf(zmax, z[e]);
    zmax = warp_max(zmax);
    float s = 0.f;
    for (int e = lane; e < n_experts; e += 32) s += expf(z[e] - zmax);
    denom = warp_sum(s);
  }
  auto score_of = [&](int e) { return score_kind == 1 ? expf(z[e] - zmax) / denom : 1.f / (1.f + expf(-z[e])); };
  for (int e = lane; e < n_experts; e += 32) c[e] = score_of(e) + (correction ? correction[e] : 0.f);
  __syncwarp();
  if (n_groups > 1) {
    const int per = n_experts / n_groups;
    for (int g = lane; g < n_groups; g += 32) {
      // the sum of the group's group_top largest: each pass takes the largest below (value, index) of the pass before
      float sum = 0.f, last_v = INFINITY;
      int last_e = -1;
      for (int k = 0; k < group_top && k < per; ++k) {
        float best = -INFINITY;
        int best_e = -1;
        for (int e = g * per; e < (g + 1) * per; ++e) {
          const float v = c[e];
          const bool after = v < last_v || (v == last_v && e > last_e);
          if (after && (best_e < 0 || v > best)) {
            best = v;
            best_e = e;
          }
        }
        sum += best;
        last_v = best;
        last_e = best_e;
      }
      gs[g] = sum;
    }
    __syncwarp();
    // the `keep` best groups, one after another; a kept group's score becomes +infinity as its mark
    for (int k = 0; k < keep; ++k) {
      float best = -INFINITY;
      int best_g = 0x7fffffff;
      for (int g = lane; g < n_groups; g += 32) {
        const float v = gs[g];
        if (v != INFINITY && (best_g == 0x7fffffff || v > best)) {
          best = v;
          best_g = g;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int og = __shfl_xor_sync(0xffffffffu, best_g, o);
        if (og != 0x7fffffff && (best_g == 0x7fffffff || ob > best || (ob == best && og < best_g))) {
          best = ob;
          best_g = og;
        }
      }
      __syncwarp();
      if (lane == 0 && best_g != 0x7fffffff) gs[best_g] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < n_experts; e += 32)
      if (gs[e / per] != INFINITY) c[e] = -INFINITY;
    __syncwarp();
  }
  float total = 0.f;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane; e < n_experts; e += 32) {
      const float v = c[e];
      if (v != -INFINITY && (best_e == 0x7fffffff || v > best)) {
        best = v;
        best_e = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (oe != 0x7fffffff && (best_e == 0x7fffffff || ob > best || (ob == best && oe < best_e))) {
        best = ob;
        best_e = oe;
      }
    }
    __syncwarp();
    if (best_e == 0x7fffffff) best_e = 0;          // fewer experts may be chosen than `top`: refused by the caller
    const float s = score_of(best_e);
    total += s;
    if (lane == 0) {
      c[best_e] = -INFINITY;
      chosen[(size_t)t * top + j] = best_e;
      weight[(size_t)t * top + j] = s;
    }
    __syncwarp();
  }
  for (int j = lane; j < top; j += 32) {
    float w = weight[(size_t)t * top + j];
    if (renormalize) w = w / (total + norm_eps);
    weight[(size_t)t * top + j] = w * route_scale;
  }
}

LLM_EXPORT int llm_moe_route_grouped(const float *logits, long long ld, int n_tokens, int n_experts, int top, int score_kind,
                                     const float *correction, int n_groups, int keep, int group_top, int renormalize, float norm_eps,
                                     float route_scale, int *chosen, float *weight, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_experts > 0 && top > 0 && top <= n_experts, "moe_route: %d of %d experts", top, n_experts);
  LLM_REQUIRE(n_experts <= 2048, "moe_route: at most 2048 experts (%d)", n_experts);
  LLM_REQUIRE(score_kind == 0 || score_kind == 1, "moe_route: unknown score %d", score_kind);
  LLM_REQUIRE(n_groups >= 1 && n_experts % n_groups == 0 && keep >= 1 && keep <= n_groups && group_top >= 1,
              "moe_route: %d experts in %d groups of which %d are kept", n_experts, n_groups, keep);
  LLM_REQUIRE(n_groups == 1 || (long long)keep * (n_experts / n_groups) >= top, "moe_route: %d kept groups of %d experts hold fewer than the %d to choose",
              keep, n_experts / n_groups, top);
  const int warps = 4;
  const size_t smem = (size_t)warps * (size_t)(n_experts + n_groups) * sizeof(float);
  llm_launch(moe_route_grouped_kernel, dim3((n_tokens + warps - 1) / warps), dim3(warps * 32), smem, stream, logits, ld, n_tokens,
             n_experts, top, score_kind, correction, n_groups, keep, group_top, renormalize, norm_eps, route_scale, chosen, weight);
  LLM_CHECK_LAUNCH("moe_route_grouped");
  return LLM_OK;
}

// out[p, t, :] = x[p, t, :] * sigmoid(gate[t * gate_stride]) for every part p (32-bit rows; parts x_stride and out_stride
// floats apart): a feed-forward's result, whole or in partial products, weighed by one number per token.
__global__ void row_gate_kernel(const float *__restrict__ x, long long x_stride, float *__restrict__ out, long long out_stride,
                                const float *__restrict__ gate, long long gate_stride, int cols, long long total) {
  grid_dependents_launch();
  grid_dependency_wait();
  const float *xp = x + (size_t)blockIdx.y * x_stride;
  float *op = out + (size_t)blockIdx.y * out_stride;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / cols;
    op[i] = xp[i] * (1.f / (1.f + expf(-gate[t * gate_stride])));
  }
}
LLM_EXPORT int llm_row_gate(const float *x, long long x_stride, float *out, long long out_stride, int n_parts, const float *gate,
                            long long gate_stride, int n_rows, int cols, cudaStream_t stream) {
  if (n_rows == 0 || cols == 0 || n_parts == 0) return LLM_OK;
  LLM_REQUIRE(n_rows > 0 && cols > 0 && n_parts > 0 && n_parts <= 65535 && x && out && gate, "row_gate: bad arguments");
  const long long total = (long long)n_rows * cols;
  long long blocks = (total + 255) / 256;
  if (blocks > (long long)sm_count() * 16) blocks = (long long)sm_count() * 16;
  llm_launch(row_gate_kernel, dim3((unsigned)blocks, (unsigned)n_parts), dim3(256), 0, stream, x, x_stride, out, out_stride, gate,
             gate_stride, cols, total);
  LLM_CHECK_LAUNCH("row_gate");
  return LLM_OK;
}

// ---------------------------------------------------------------- rows by expert
// One CTA.  offsets[e] .. offsets[e + 1]: the sorted places of expert e's rows; perm[place] = row;
// tiles[0] = number of row tiles, then (expert, first place) per tile of at most `tile_rows` rows of
// one expert.  Which place a row gets within its expert depends on the order the threads arrive
// in; no result depends on it.
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int *__restrict__ chosen, int n_rows, int n_experts, int tile_rows, int *__restrict__ offsets,
                int *__restrict__ perm, int *__restrict__ tiles) {
  extern __shared__ int sh[];                  // counts [E], cursor [E]
  int *counts = sh, *cursor = sh + n_experts;
  grid_dependents_launch();
  grid_dependency_wait();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int r = threadIdx.x; r < n_rows; r += blockDim.x) atomicAdd(&counts[chosen[r]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0, n_tiles = 0;
    for (int e = 0; e < n_experts; ++e) {
      cursor[e] = o;
      offsets[e] = o;
      for (int r0 = 0; r0 < counts[e]; r0 += tile_rows) {
        tiles[1 + 2 * n_tiles] = e;
        tiles[2 + 2 * n_tiles] = o + r0;
        ++n_tiles;
      }
      o += counts[e];
    }
    offsets[n_experts] = o;
    tiles[0] = n_tiles;
  }
  __syncthreads();
  for (int r = threadIdx.x; r < n_rows; r += blockDim.x) perm[atomicAdd(&cursor[chosen[r]], 1)] = r;
}

LLM_EXPORT int llm_moe_sort(const int *chosen, int n_rows, int n_experts, int tile_rows, int *offsets, int *perm, int *tiles,
                            cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE(n_rows > 0 && n_experts > 0 && n_experts <= 4096 && tile_rows > 0, "moe_sort: bad sizes");
  llm_launch(moe_sort_kernel, dim3(1), dim3(1024), (size_t)n_experts * 2 * sizeof(int), stream, chosen, n_rows, n_experts,
             tile_rows, offsets, perm, tiles);
  LLM_CHECK_LAUNCH("moe_sort");
  return LLM_OK;
}
LLM_EXPORT int llm_moe_tile_rows() { return 64; }

// ---------------------------------------------------------------- both products, a CTA per row
template <typename T>
__device__ __forceinline__ float dot_cols(const T *__restrict__ w, const float *__restrict__ x, int n, int lane) {
  float acc = 0.f;
  for (int c = lane; c < n; c += 32) acc = fmaf(to_float(w[c]), x[c], acc);
  return warp_sum(acc);
}

// x [tokens, width]; up [experts, ff, width]; down [experts, width, ff]; out [top, tokens, width] 32-bit.
// weight_on 0: input, 1: output.
template <typename T>
__global__ void __launch_bounds__(256)
moe_rows_kernel(const T *__restrict__ x, long long ldx, const T *__restrict__ up, const T *__restrict__ down,
                const int *__restrict__ chosen, const float *__restrict__ weight, int n_tokens, int top, int width, int ff,
                int act, int weight_on, int gated, float *__restrict__ out) {
  extern __shared__ float shf[];               // x row [width], hidden [ff]
  float *xs = shf, *hs = shf + width;
  grid_dependents_launch();
  grid_dependency_wait();
  const int r = blockIdx.x, t = r / top, j = r - t * top;
  const int e = chosen[r];
  const float w = weight[r];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int c = threadIdx.x; c < width; c += 256) xs[c] = to_float(x[(size_t)t * ldx + c]);
  __syncthreads();
  const T *wu = up + (size_t)e * ff * width * (gated ? 2 : 1);
  for (int n = warp; n < ff; n += 8) {
    if (gated) {
      const float g = dot_cols(wu + (size_t)(2 * n) * width, xs, width, lane);
      const float u = dot_cols(wu + (size_t)(2 * n + 1) * width, xs, width, lane);
      if (lane == 0) hs[n] = w * (activate(g, act) * u);
      continue;
    }
    const float v = dot_cols(wu + (size_t)n * width, xs, width, lane);
    if (lane == 0) hs[n] = weight_on == 0 ? activate(w * v, act) : w * activate(v, act);
  }
  __syncthreads();
  const T *wd = down + (size_t)e * width * ff;
  float *o = out + ((size_t)j * n_tokens + t) * width;
  for (int m = warp; m < width; m += 8) {
    const float v = dot_cols(wd + (size_t)m * ff, hs, ff, lane);
    if (lane == 0) o[m] = v;
  }
}

LLM_EXPORT int llm_moe_rows(int dtype, const void *x, long long ldx, const void *up, const void *down, const int *chosen,
                            const float *weight, int n_tokens, int top, int width, int ff, int act, int weight_on, int gated,
                            float *out, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && top > 0 && width > 0 && ff > 0, "moe_rows: bad sizes");
  LLM_REQUIRE(!gated || weight_on == 1, "moe_rows: gated experts take their weight on the output");
  const size_t smem = (size_t)(width + ff) * sizeof(float);
  LLM_REQUIRE(smem <= 200 * 1024, "moe_rows: rows of %d + %d values do not fit shared memory", width, ff);
  if (dtype == LLM_F32) {
    LLM_CHECK_CUDA(llm_allow_smem(moe_rows_kernel<float>, smem), "moe_rows attribute");
    llm_launch(moe_rows_kernel<float>, dim3(n_tokens * top), dim3(256), smem, stream, (const float *)x, ldx, (const float *)up,
               (const float *)down, chosen, weight, n_tokens, top, width, ff, act, weight_on, gated, out);
  } else {
    LLM_CHECK_CUDA(llm_allow_smem(moe_rows_kernel<__nv_bfloat16>, smem), "moe_rows attribute");
    llm_launch(moe_rows_kernel<__nv_bfloat16>, dim3(n_tokens * top), dim3(256), smem, stream, (const __nv_bfloat16 *)x, ldx,
               (const __nv_bfloat16 *)up, (const __nv_bfloat16 *)down, chosen, weight, n_tokens, top, width, ff, act, weight_on, gated, out);
  }
  LLM_CHECK_LAUNCH("moe_rows");
  return LLM_OK;
}

// ---------------------------------------------------------------- the products by expert on mma.sync
constexpr int GM = 64, GN = 128, GK = 32, GSTAGES = 3, GPAD = 8;
constexpr int GLD = GK + GPAD;                 // 40 values = 80 bytes a row: ldmatrix without bank conflicts

// C[place, n] = sum_k A[arow(place), k] * W[expert][n, k] for the places of one tile.
// second == 0: A = x, arow = perm[place] / top; C -> mid[place, n] = bfloat16(act and weight applied).
// second == 1: A = mid, arow = place;           C -> out[perm % top][perm / top][n], 32-bit.
__global__ void __launch_bounds__(256)
moe_grouped_kernel(const __nv_bfloat16 *__restrict__ A, long long lda, const __nv_bfloat16 *__restrict__ W, int N, int K,
                   const int *__restrict__ offsets, const int *__restrict__ perm, const int *__restrict__ tiles,
                   const float *__restrict__ weight, int n_tokens, int top, int act, int weight_on, int second, int gated,
                   __nv_bfloat16 *__restrict__ mid, float *__restrict__ out) {
  __shared__ __align__(16) __nv_bfloat16 As[GSTAGES][GM][GLD];
  __shared__ __align__(16) __nv_bfloat16 Bs[GSTAGES][GN][GLD];
  __shared__ int row_src[GM], row_id[GM];
  grid_dependents_launch();
  grid_dependency_wait();
  if ((int)blockIdx.x >= tiles[0]) return;
  const int expert = tiles[1 + 2 * blockIdx.x], place0 = tiles[2 + 2 * blockIdx.x];
  const int n_rows = min(GM, offsets[expert + 1] - place0);
  const int n0 = blockIdx.y * GN;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < GM) {
    const int id = tid < n_rows ? perm[place0 + tid] : -1;
    row_id[tid] = id;
    row_src[tid] = id < 0 ? -1 : (second ? place0 + tid : id / top);
  }
  __syncthreads();
  const __nv_bfloat16 *Wb = W + (size_t)expert * N * K;
  const int k_steps = (K + GK - 1) / GK;

  auto load = [&](int stage, int ks) {
    const int k0 = ks * GK;
    // A: 64 rows x 4 pieces of 8 values; B: 128 rows x 4 pieces
    {
      const int r = tid >> 2, piece = tid & 3, k = k0 + piece * 8;
      const int src = row_src[r];
      const bool ok = src >= 0 && k < K;
      cp_async16(&As[stage][r][piece * 8], ok ? A + (size_t)src * lda + k : A, ok);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int item = tid + i * 256, r = item >> 2, piece = item & 3, k = k0 + piece * 8;
      const bool ok = n0 + r < N && k < K;
      cp_async16(&Bs[stage][r][piece * 8], ok ? Wb + (size_t)(n0 + r) * K + k : Wb, ok);
    }
  };

  // warp grid 2 (rows) x 4 (columns): a warp owns 32 rows x 32 columns = 2 x 4 mma tiles
  const int wm = warp >> 2, wn = warp & 3;
  float acc[2][4][4];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[a][b][c] = 0.f;

  for (int s = 0; s < GSTAGES - 1; ++s) {
    if (s < k_steps) load(s, s);
    cp_async_commit();
  }
  for (int ks = 0; ks < k_steps; ++ks) {
    cp_async_wait<GSTAGES - 2>();
    __syncthreads();
    const int nxt = ks + GSTAGES - 1;
    if (nxt < k_steps) load(nxt % GSTAGES, nxt);
    cp_async_commit();
    const int st = ks % GSTAGES;
#pragma unroll
    for (int kk = 0; kk < GK; kk += 16) {
      unsigned af[2][4], bf[2][4];
#pragma unroll
      for (int a = 0; a < 2; ++a)
        ldmatrix_x4(af[a], &As[st][wm * 32 + a * 16 + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
      for (int b = 0; b < 2; ++b)        // 16 weight rows at a time: matrices (n 0-7, k lo), (n 0-7, k hi), (n 8-15, k lo), (n 8-15, k hi)
        ldmatrix_x4(bf[b], &Bs[st][wn * 32 + b * 16 + (lane & 7) + ((lane >> 4) << 3)][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) mma16816(acc[a][b], af[a], bf[b >> 1][(b & 1) * 2], bf[b >> 1][(b & 1) * 2 + 1]);
    }
  }
  cp_async_wait<0>();

  const int g = lane >> 2, tq = lane & 3;
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = wm * 32 + a * 16 + g + half * 8;
      const int id = row_id[r];
      if (id < 0) continue;
      const float w = weight[id];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int n = n0 + wn * 32 + b * 8 + tq * 2;
        const float v0 = acc[a][b][half * 2], v1 = acc[a][b][half * 2 + 1];
        if (!second && gated) {
          // columns n (even: the gate's row of feature n / 2) and n + 1 (the up row of the same feature)
          if (n + 1 < N) mid[(size_t)(place0 + r) * (N / 2) + n / 2] = __float2bfloat16_rn(w * (activate(v0, act) * v1));
        } else if (!second) {
          __nv_bfloat16 *dst = mid + (size_t)(place0 + r) * N;
          const float y0 = weight_on == 0 ? activate(w * v0, act) : w * activate(v0, act);
          const float y1 = weight_on == 0 ? activate(w * v1, act) : w * activate(v1, act);
          if (n < N) dst[n] = __float2bfloat16_rn(y0);
          if (n + 1 < N) dst[n + 1] = __float2bfloat16_rn(y1);
        } else {
          float *dst = out + ((size_t)(id % top) * n_tokens + id / top) * N;
          if (n < N) dst[n] = v0;
          if (n + 1 < N) dst[n + 1] = v1;
        }
      }
    }
}

// x [tokens, width] bfloat16; mid [tokens * top, ff] bfloat16 scratch; out [top, tokens, width] 32-bit.
LLM_EXPORT int llm_moe_grouped(const void *x, long long ldx, const void *up, const void *down, const int *offsets, const int *perm,
                               const int *tiles, const float *weight, int n_tokens, int n_experts, int top, int width, int ff,
                               int act, int weight_on, int gated, void *mid, float *out, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && top > 0 && width > 0 && ff > 0 && n_experts > 0, "moe_grouped: bad sizes");
  LLM_REQUIRE(!gated || weight_on == 1, "moe_grouped: gated experts take their weight on the output");
  LLM_REQUIRE(width % 8 == 0 && ff % 8 == 0 && ldx % 8 == 0, "moe_grouped: widths %d / %d must be multiples of 8", width, ff);
  LLM_REQUIRE((uintptr_t)x % 16 == 0 && (uintptr_t)up % 16 == 0 && (uintptr_t)down % 16 == 0 && (uintptr_t)mid % 16 == 0,
              "moe_grouped: operands must be 16-byte aligned");
  const int n_rows = n_tokens * top;
  const int max_tiles = min(n_experts, n_rows) + n_rows / GM;
  const int n_first = gated ? 2 * ff : ff;
  llm_launch(moe_grouped_kernel, dim3(max_tiles, (n_first + GN - 1) / GN), dim3(256), 0, stream, (const __nv_bfloat16 *)x, ldx,
             (const __nv_bfloat16 *)up, n_first, width, offsets, perm, tiles, weight, n_tokens, top, act, weight_on, 0, gated,
             (__nv_bfloat16 *)mid, (float *)nullptr);
  LLM_CHECK_LAUNCH("moe_grouped (first product)");
  llm_launch(moe_grouped_kernel, dim3(max_tiles, (width + GN - 1) / GN), dim3(256), 0, stream, (const __nv_bfloat16 *)mid,
             (long long)ff, (const __nv_bfloat16 *)down, width, ff, offsets, perm, tiles, weight, n_tokens, top, act, weight_on, 1, 0,
             (__nv_bfloat16 *)nullptr, out);
  LLM_CHECK_LAUNCH("moe_grouped (second product)");
  return LLM_OK;
}
LLM_EXPORT int llm_moe_grouped_supports(int width, int ff) { return width % 8 == 0 && ff % 8 == 0; }

// ---------------------------------------------------------------- an activation over rows
template <typename TI, typename T>
__global__ void activation_kernel(const TI *__restrict__ in, T *__restrict__ out, size_t n, int act) {
  grid_dependents_launch();
  grid_dependency_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_float<T>(activate(to_float(in[i]), act));
}

// Four values to a thread (counts that are multiples of 4, 16-byte aligned).
template <typename TI, typename T>
__global__ void activation_vec_kernel(const TI *__restrict__ in, T *__restrict__ out, size_t n4, int act) {
  grid_dependents_launch();
  grid_dependency_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    const float4 v = ld4(in + 4 * i);
    st4(out + 4 * i, make_float4(activate(v.x, act), activate(v.y, act), activate(v.z, act), activate(v.w, act)));
  }
}

LLM_EXPORT int llm_activation(int in_dtype, int dtype, const void *in, void *out, long long n, int act, cudaStream_t stream) {
  if (n == 0) return LLM_OK;
  LLM_REQUIRE(n > 0 && act >= 0 && act <= 3, "activation: bad arguments");
  if (n % 4 == 0 && (uintptr_t)in % 16 == 0 && (uintptr_t)out % 16 == 0 && (in_dtype == LLM_F32 || dtype == LLM_BF16)) {
    const size_t n4 = (size_t)n / 4;
    size_t blocks4 = (n4 + 255) / 256;
    if (blocks4 > (size_t)sm_count() * 32) blocks4 = (size_t)sm_count() * 32;
    if (in_dtype == LLM_F32 && dtype == LLM_F32)
      llm_launch(activation_vec_kernel<float, float>, dim3((unsigned)blocks4), dim3(256), 0, stream, (const float *)in, (float *)out, n4, act);
    else if (in_dtype == LLM_F32 && dtype == LLM_BF16)
      llm_launch(activation_vec_kernel<float, __nv_bfloat16>, dim3((unsigned)blocks4), dim3(256), 0, stream, (const float *)in,
                 (__nv_bfloat16 *)out, n4, act);
    else
      llm_launch(activation_vec_kernel<__nv_bfloat16, __nv_bfloat16>, dim3((unsigned)blocks4), dim3(256), 0, stream,
                 (const __nv_bfloat16 *)in, (__nv_bfloat16 *)out, n4, act);
    LLM_CHECK_LAUNCH("activation");
    return LLM_OK;
  }
  size_t blocks = ((size_t)n + 255) / 256;
  if (blocks > (size_t)sm_count() * 32) blocks = (size_t)sm_count() * 32;
  if (in_dtype == LLM_F32 && dtype == LLM_F32)
    llm_launch(activation_kernel<float, float>, dim3((unsigned)blocks), dim3(256), 0, stream, (const float *)in, (float *)out, (size_t)n, act);
  else if (in_dtype == LLM_F32 && dtype == LLM_BF16)
    llm_launch(activation_kernel<float, __nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, stream, (const float *)in,
               (__nv_bfloat16 *)out, (size_t)n, act);
  else if (in_dtype == LLM_BF16 && dtype == LLM_BF16)
    llm_launch(activation_kernel<__nv_bfloat16, __nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, stream,
               (const __nv_bfloat16 *)in, (__nv_bfloat16 *)out, (size_t)n, act);
  else LLM_FAIL("activation: unsupported dtypes in %d out %d", in_dtype, dtype);
  LLM_CHECK_LAUNCH("activation");
  return LLM_OK;
}

// ---------------------------------------------------------------- the tokens' rows in sorted order
// xs[place] = x[perm[place] / top], 16 bytes to a thread: the operand of the tensor-memory form of the first
// product (csrc/moe_tc.cu), whose loads want the rows of a tile one behind the other.
__global__ void moe_gather_kernel(const uint4 *__restrict__ x, long long ldx16, const int *__restrict__ perm, int top,
                                  int width16, size_t total, uint4 *__restrict__ xs) {
  grid_dependents_launch();
  grid_dependency_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t place = idx / width16;
    const int c = (int)(idx - place * width16);
    xs[idx] = x[(size_t)(perm[place] / top) * ldx16 + c];
  }
}

LLM_EXPORT int llm_moe_gather(const void *x, long long ldx, const int *perm, int n_rows, int top, int width, void *xs,
                              cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE(n_rows > 0 && top > 0 && width % 8 == 0 && ldx % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)xs % 16 == 0,
              "moe_gather: rows of bfloat16 in multiples of 8, 16-byte aligned");
  const size_t total = (size_t)n_rows * (width / 8);
  size_t blocks = (total + 255) / 256;
  if (blocks > (size_t)sm_count() * 32) blocks = (size_t)sm_count() * 32;
  llm_launch_after(moe_gather_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, (const uint4 *)x, ldx / 8, perm, top, width / 8, total,
             (uint4 *)xs);
  LLM_CHECK_LAUNCH("moe_gather");
  return LLM_OK;
}
