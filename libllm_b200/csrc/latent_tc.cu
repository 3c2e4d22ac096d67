// Latent attention on the tensor cores (bfloat16 operands, 32-bit accumulation, mma.sync m16n8k16).
//
// A position's cached row is [c | k_r]: the normed latent (kv_rank channels) and the rotated key part that all
// heads share (rot channels).  Two forms of the same attention, chosen by what the step brings:
//
//  * A step whose sequences all start at their first token (latent_prefill): keys and values of every head are
//    materialised for the step's own rows by one library product, kv = [W_uk; W_uv] c, and the kernel is the
//    flash form over them.  A head's key is [kv's unrotated part for the head | k_r], of d + rot channels, its
//    value kv's part of dv channels; the two sizes differ, so the key tile and the value tile have their own
//    widths.  The products cost heads * (d + rot + dv) per (query, key) pair, the least of the two forms.
//
//  * Every other step, decoding above all (latent_decode): W_uk is taken into the queries and W_uv is applied
//    behind the weighted sum (csrc/latent.cu), so all heads of a token read the same rows: one key/value
//    "head" of kv_rank + rot channels whose values are its first kv_rank channels.  A CTA takes one token and 32
//    heads; the rows go through shared memory once for all of them.  The warps first share out the keys of a
//    tile of 64 for S = Q K^T (16 heads x 16 keys each, over the whole row), leave S in shared memory, and then
//    share out the value channels for O += P C (16 heads x a quarter of the channels each); each redoes the
//    cheap softmax step for its 16 heads.  Long sequences are cut into runs over several CTAs; a second kernel
//    joins the runs' partial results.  The cache is read once per token, not once per head.
//
// 32-bit: scores, maxima, exponentials, sums, the output accumulation and the joining of runs.  The reference
// has no such mixer (its attention: src/libllm/llama.cc:178-225, over src/flint/cuda/flash_attn.cc).
#include "common.cuh"
#include "mma_tiles.cuh"
#include <math.h>

LLM_DEFINE_LAST_ERROR(llm_latent_tc_last_error)

constexpr int LT_BN = 64;                // keys per tile

// ---------------------------------------------------------------- the step's rows, out of the cache
// c_out [T, kv_rank] and kr_out [T, rot] = the cached rows of the step's tokens (whoever appended them).
__global__ void __launch_bounds__(128)
latent_rows_kernel(const __nv_bfloat16 *__restrict__ cache, int page_size, int row, int kv_rank, const int *__restrict__ tok_seq,
                   const int *__restrict__ tok_pos, const int *__restrict__ page_table, int pt_stride,
                   __nv_bfloat16 *__restrict__ c_out, __nv_bfloat16 *__restrict__ kr_out) {
  grid_dependents_launch();
  grid_dependency_wait();
  const int t = blockIdx.x, pos = tok_pos[t];
  const int page = page_table[(size_t)tok_seq[t] * pt_stride + pos / page_size];
  const __nv_bfloat16 *src = cache + ((size_t)page * page_size + pos % page_size) * (size_t)row;
  const int rot = row - kv_rank;
  for (int c = threadIdx.x; c < kv_rank; c += 128) c_out[(size_t)t * kv_rank + c] = src[c];
  for (int c = threadIdx.x; c < rot; c += 128) kr_out[(size_t)t * rot + c] = src[kv_rank + c];
}

LLM_EXPORT int llm_latent_rows(const void *cache, int page_size, int row, int kv_rank, const int *tok_seq, const int *tok_pos,
                               const int *page_table, int pt_stride, int n_tokens, void *c_out, void *kr_out, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && page_size > 0 && kv_rank > 0 && row >= kv_rank && cache && c_out && (row == kv_rank || kr_out),
              "latent_rows: bad sizes");
  llm_launch(latent_rows_kernel, dim3(n_tokens), dim3(128), 0, stream, (const __nv_bfloat16 *)cache, page_size, row, kv_rank, tok_seq,
             tok_pos, page_table, pt_stride, (__nv_bfloat16 *)c_out, (__nv_bfloat16 *)kr_out);
  LLM_CHECK_LAUNCH("latent_rows");
  return LLM_OK;
}

// ---------------------------------------------------------------- the queries' rotation
// q rows (32-bit) [heads, d + rot] -> bfloat16, the last rot channels of each head rotated by the token's
// position.  Table row = [cosines (rot/2) | sines (rot/2)]; pair i is channels (2i, 2i+1) when interleaved, else
// (i, i + rot/2).
__global__ void __launch_bounds__(256)
latent_rotate_q_kernel(const float *__restrict__ q, long long ldq, __nv_bfloat16 *__restrict__ out, long long ldo, int n_heads, int d,
                       int rot, const float *__restrict__ table, int table_rows, int interleaved, const int *__restrict__ tok_pos) {
  grid_dependents_launch();
  grid_dependency_wait();
  const int t = blockIdx.x, dk = d + rot, half = rot / 2;
  const int pos = tok_pos[t];
  const float *cs = rot > 0 ? table + (size_t)(pos < table_rows ? pos : table_rows - 1) * rot : nullptr;
  const float *src = q + (size_t)t * ldq;
  __nv_bfloat16 *dst = out + (size_t)t * ldo;
  for (int i = threadIdx.x; i < n_heads * d; i += 256) {
    const int h = i / d, c = i - h * d;
    dst[(size_t)h * dk + c] = __float2bfloat16(src[(size_t)h * dk + c]);
  }
  for (int i = threadIdx.x; i < n_heads * half; i += 256) {
    const int h = i / half, p = i - h * half;
    const int a = interleaved ? 2 * p : p, b = interleaved ? 2 * p + 1 : p + half;
    const float u = src[(size_t)h * dk + d + a], v = src[(size_t)h * dk + d + b], co = cs[p], si = cs[half + p];
    dst[(size_t)h * dk + d + a] = __float2bfloat16(u * co - v * si);
    dst[(size_t)h * dk + d + b] = __float2bfloat16(v * co + u * si);
  }
}

LLM_EXPORT int llm_latent_rotate_q(const float *q, long long ldq, void *out, long long ldo, int n_tokens, int n_heads, int d, int rot,
                                   const float *table, int table_rows, int interleaved, const int *tok_pos, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_heads > 0 && d >= 0 && rot >= 0 && rot % 2 == 0 && d + rot > 0, "latent_rotate_q: bad sizes");
  LLM_REQUIRE(rot == 0 || (table && table_rows > 0), "latent_rotate_q: a rotation needs its table");
  llm_launch(latent_rotate_q_kernel, dim3(n_tokens), dim3(256), 0, stream, q, ldq, (__nv_bfloat16 *)out, ldo, n_heads, d, rot, table,
             table_rows, interleaved, tok_pos);
  LLM_CHECK_LAUNCH("latent_rotate_q");
  return LLM_OK;
}

// ---------------------------------------------------------------- prompt steps from the first token: materialised heads
// One CTA takes 128 query rows of one head of one sequence, its eight warps 16 rows each; key tiles of 64 rows are
// walked with two tiles in flight, up to the one that holds the CTA's last row; a warp sits out the tiles that lie
// wholly behind its rows.  q [T, heads * (d + rot)] (rotated), kv [T, heads * d | heads * dv], kr [T, rot]
// (rotated), out [T, heads * dv]; sequence b owns rows seq_start[b] .. seq_start[b+1]-1 at positions 0 .. ; with
// `window` > 0 the row at position p sees keys p - window + 1 .. p only.
// Key rows are d + rot channels rounded up to 16 (the rest zeros), value rows DVP >= dv channels (the rest zeros).
constexpr int LP_WARPS = 8;
constexpr int LP_BM = 16 * LP_WARPS;

template <int DVP>
__global__ void __launch_bounds__(LP_WARPS * 32)
latent_prefill_kernel(const __nv_bfloat16 *__restrict__ q, long long ldq, const __nv_bfloat16 *__restrict__ kv, long long ldkv,
                      const __nv_bfloat16 *__restrict__ kr, __nv_bfloat16 *__restrict__ out, long long ldo,
                      const int *__restrict__ seq_start, int n_heads, int d, int rot, int dv, float scale_log2, int window) {
  constexpr int LDV = DVP + 8;
  constexpr int VCH = DVP / 8;
  constexpr int NT = LT_BN / 8;
  constexpr int DT = DVP / 8;
  const int dk = d + rot;
  const int dkp = (dk + 15) / 16 * 16;
  const int ldk = dkp + 8;
  const int kch = dkp / 8;                                   // 16-byte pieces of a key row
  const int KS = dkp / 16;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16 *sQ = reinterpret_cast<__nv_bfloat16 *>(smem_raw);
  __nv_bfloat16 *sK = sQ + LP_BM * ldk;                      // [2][64][ldk]
  __nv_bfloat16 *sV = sK + 2 * LT_BN * ldk;                  // [2][64][LDV]

  grid_dependents_launch();
  grid_dependency_wait();
  const int b = blockIdx.z, h = blockIdx.y;
  const int q0 = seq_start[b], n_q = seq_start[b + 1] - q0;
  const int tile = gridDim.x - 1 - blockIdx.x;               // long tiles first
  const int r0 = tile * LP_BM;
  if (r0 >= n_q) return;
  const int rows = min(LP_BM, n_q - r0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int n_iter = min((n_q + LT_BN - 1) / LT_BN, (r0 + LP_BM) / LT_BN);   // key tiles up to the one with the CTA's last row,
  const int it0 = window > 0 ? max(0, r0 - window + 1) / LT_BN : 0;          // from the one with the first key its first row sees
  const int d8 = d / 8, dk8 = dk / 8, dv8 = dv / 8;
  const size_t v_off = (size_t)n_heads * d + (size_t)h * dv;

  auto load_kv = [&](int kt, int stage) {
    __nv_bfloat16 *tk = sK + stage * LT_BN * ldk, *tv = sV + stage * LT_BN * LDV;
    for (int c = tid; c < LT_BN * kch; c += LP_WARPS * 32) {
      const int r = c / kch, ch = c - r * kch;
      const int j = kt * LT_BN + r;
      const bool ok = j < n_q && ch < dk8;
      const size_t rowi = (size_t)(q0 + (j < n_q ? j : 0));
      const __nv_bfloat16 *src = ch < d8 ? kv + rowi * ldkv + (size_t)h * d + ch * 8
                                         : kr + rowi * rot + (ch < dk8 ? ch - d8 : 0) * 8;
      cp_async16(tk + r * ldk + ch * 8, ok ? src : kv, ok);
    }
    for (int c = tid; c < LT_BN * VCH; c += LP_WARPS * 32) {
      const int r = c / VCH, ch = c - r * VCH;
      const int j = kt * LT_BN + r;
      const bool ok = j < n_q && ch < dv8;
      cp_async16(tv + r * LDV + ch * 8, ok ? kv + (size_t)(q0 + j) * ldkv + v_off + ch * 8 : kv, ok);
    }
  };

  for (int c = tid; c < LP_BM * kch; c += LP_WARPS * 32) {
    const int r = c / kch, ch = c - r * kch;
    const bool ok = r < rows && ch < dk8;
    cp_async16(sQ + r * ldk + ch * 8, ok ? q + (size_t)(q0 + r0 + r) * ldq + (size_t)h * dk + ch * 8 : q, ok);
  }
  load_kv(it0, 0);
  cp_async_commit();

  float o[DT][4];
#pragma unroll
  for (int i = 0; i < DT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int pos0 = r0 + warp * 16 + g, pos1 = pos0 + 8;

  for (int it = it0; it < n_iter; ++it) {
    const int stage = (it - it0) & 1;
    if (it + 1 < n_iter) load_kv(it + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const __nv_bfloat16 *tk = sK + stage * LT_BN * ldk, *tv = sV + stage * LT_BN * LDV;
    const int k0 = it * LT_BN;
    // else: no row of this warp sees a key of the tile (it lies behind the rows, or before the first row's window)
    if (k0 <= r0 + warp * 16 + 15 && (window == 0 || k0 + LT_BN - 1 > r0 + warp * 16 - window)) {

    float s[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[n][j] = 0.f;
#pragma unroll 2
    for (int ks = 0; ks < KS; ++ks) {
      unsigned qf[4];
      ldmatrix_x4(qf, sQ + (warp * 16 + (lane & 15)) * ldk + ks * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int n2 = 0; n2 < NT / 2; ++n2) {
        unsigned kb[4];
        ldmatrix_x4(kb, tk + (n2 * 16 + (lane & 7) + (lane >> 4) * 8) * ldk + ks * 16 + ((lane >> 3) & 1) * 8);
        mma16816(s[2 * n2], qf, kb[0], kb[1]);
        mma16816(s[2 * n2 + 1], qf, kb[2], kb[3]);
      }
    }

    if (k0 + LT_BN - 1 > r0 + warp * 16) {                   // a tile on the diagonal: key j is seen by the row at p when j <= p
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int key = k0 + n * 8 + 2 * t + (j & 1);
          if (key > ((j & 2) ? pos1 : pos0)) s[n][j] = -INFINITY;
        }
    }
    if (window > 0 && k0 <= r0 + warp * 16 + 15 - window) {  // a tile on the window's edge: the row at p sees key j when j > p - window
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int key = k0 + n * 8 + 2 * t + (j & 1);
          if (key <= ((j & 2) ? pos1 : pos0) - window) s[n][j] = -INFINITY;
        }
    }

    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      mx[0] = fmaxf(mx[0], fmaxf(s[n][0], s[n][1]));
      mx[1] = fmaxf(mx[1], fmaxf(s[n][2], s[n][3]));
    }
    float alpha[2], moff[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      moff[r] = m_new == -INFINITY ? 0.f : m_new * scale_log2;
      alpha[r] = m_run[r] == -INFINITY ? 0.f : exp2f(m_run[r] * scale_log2 - moff[r]);
      m_run[r] = m_new;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      s[n][0] = exp2f(fmaf(s[n][0], scale_log2, -moff[0]));
      s[n][1] = exp2f(fmaf(s[n][1], scale_log2, -moff[0]));
      s[n][2] = exp2f(fmaf(s[n][2], scale_log2, -moff[1]));
      s[n][3] = exp2f(fmaf(s[n][3], scale_log2, -moff[1]));
      sum[0] += s[n][0] + s[n][1];
      sum[1] += s[n][2] + s[n][3];
    }
    l_run[0] = l_run[0] * alpha[0] + sum[0];
    l_run[1] = l_run[1] * alpha[1] + sum[1];
#pragma unroll
    for (int i = 0; i < DT; ++i) {
      o[i][0] *= alpha[0];
      o[i][1] *= alpha[0];
      o[i][2] *= alpha[1];
      o[i][3] *= alpha[1];
    }
#pragma unroll
    for (int kk = 0; kk < LT_BN / 16; ++kk) {
      unsigned pa[4];
      pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int d2 = 0; d2 < DT / 2; ++d2) {
        unsigned vb[4];
        ldmatrix_x4_trans(vb, tv + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDV + d2 * 16 + (lane >> 4) * 8);
        mma16816(o[2 * d2], pa, vb[0], vb[1]);
        mma16816(o[2 * d2 + 1], pa, vb[2], vb[3]);
      }
    }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  const int row_a = warp * 16 + g, row_b = row_a + 8;
  const float inv_a = 1.f / l_run[0], inv_b = 1.f / l_run[1];
  __nv_bfloat16 *oa = out + (size_t)(q0 + r0 + row_a) * ldo + (size_t)h * dv + 2 * t;
  __nv_bfloat16 *ob = out + (size_t)(q0 + r0 + row_b) * ldo + (size_t)h * dv + 2 * t;
#pragma unroll
  for (int i = 0; i < DT; ++i) {
    if (i * 8 < dv) {
      if (row_a < rows) *reinterpret_cast<unsigned *>(oa + i * 8) = pack_bf16(o[i][0] * inv_a, o[i][1] * inv_a);
      if (row_b < rows) *reinterpret_cast<unsigned *>(ob + i * 8) = pack_bf16(o[i][2] * inv_b, o[i][3] * inv_b);
    }
  }
}

static size_t latent_prefill_smem(int d, int rot, int dvp) {
  const int dkp = (d + rot + 15) / 16 * 16;
  return ((size_t)(LP_BM + 2 * LT_BN) * (dkp + 8) + (size_t)2 * LT_BN * (dvp + 8)) * sizeof(__nv_bfloat16);
}
static int latent_dvp(int dv) { return dv <= 32 ? 32 : dv <= 64 ? 64 : dv <= 128 ? 128 : dv <= 256 ? 256 : 0; }

// 1 if heads of these sizes have an instantiation (16-byte pieces everywhere, the tiles fit), else 0.
LLM_EXPORT int llm_latent_prefill_supports(int d, int rot, int dv) {
  if (d < 0 || rot < 0 || dv <= 0 || d + rot <= 0 || d % 8 || rot % 8 || dv % 8) return 0;
  const int dvp = latent_dvp(dv);
  return dvp > 0 && latent_prefill_smem(d, rot, dvp) <= (size_t)200 * 1024;
}

template <int DVP>
static int launch_latent_prefill(const void *q, long long ldq, const void *kv, long long ldkv, const void *kr, void *out, long long ldo,
                                 const int *seq_start, int n_seqs, int max_q_len, int n_heads, int d, int rot, int dv, float scale,
                                 int window, cudaStream_t stream) {
  const size_t smem = latent_prefill_smem(d, rot, DVP);
  auto kern = latent_prefill_kernel<DVP>;
  LLM_CHECK_CUDA(llm_allow_smem(kern, smem), "latent_prefill attribute");
  dim3 grid((max_q_len + LP_BM - 1) / LP_BM, n_heads, n_seqs);
  llm_launch(kern, grid, dim3(LP_WARPS * 32), smem, stream, (const __nv_bfloat16 *)q, ldq, (const __nv_bfloat16 *)kv, ldkv,
             (const __nv_bfloat16 *)kr, (__nv_bfloat16 *)out, ldo, seq_start, n_heads, d, rot, dv, scale * 1.4426950408889634f, window);
  LLM_CHECK_LAUNCH("latent_prefill");
  return LLM_OK;
}

LLM_EXPORT int llm_latent_prefill(const void *q, long long ldq, const void *kv, long long ldkv, const void *kr, void *out, long long ldo,
                                  const int *seq_start, int n_seqs, int max_q_len, int n_heads, int d, int rot, int dv, float scale,
                                  int window, cudaStream_t stream) {
  if (n_seqs == 0 || max_q_len == 0) return LLM_OK;
  LLM_REQUIRE(window >= 0, "latent_prefill: bad window");
  LLM_REQUIRE(llm_latent_prefill_supports(d, rot, dv), "latent_prefill: heads of %d + %d key and %d value channels are not supported", d,
              rot, dv);
  LLM_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && n_heads > 0 && n_heads <= 65535 && ldq % 8 == 0 && ldkv % 8 == 0 && ldo % 2 == 0 &&
                  (rot == 0 || kr),
              "latent_prefill: bad sizes");
  switch (latent_dvp(dv)) {
    case 32: return launch_latent_prefill<32>(q, ldq, kv, ldkv, kr, out, ldo, seq_start, n_seqs, max_q_len, n_heads, d, rot, dv, scale, window, stream);
    case 64: return launch_latent_prefill<64>(q, ldq, kv, ldkv, kr, out, ldo, seq_start, n_seqs, max_q_len, n_heads, d, rot, dv, scale, window, stream);
    case 128: return launch_latent_prefill<128>(q, ldq, kv, ldkv, kr, out, ldo, seq_start, n_seqs, max_q_len, n_heads, d, rot, dv, scale, window, stream);
    default: return launch_latent_prefill<256>(q, ldq, kv, ldkv, kr, out, ldo, seq_start, n_seqs, max_q_len, n_heads, d, rot, dv, scale, window, stream);
  }
}

// ---------------------------------------------------------------- every other step: all heads over the cached rows
// qa [T, heads * row] = [W_uk^T q_unrotated | rotated q part] per head (latent_absorb), cache [pages, page_size, row];
// token t of sequence tok_seq[t] sees positions 0 .. tok_pos[t], or with `window` > 0 the last `window` of them.  Result per head: the weighted sum of the rows'
// first kv_rank channels, out [T, heads * kv_rank] (n_splits == 1) or unnormalised partial sums ws_o
// [T, heads, n_splits, kv_rank] with (maximum in the exponent's units, sum) in ws_ml [T, heads, n_splits, 2].
constexpr int LD_WARPS = 8;
constexpr int LD_HT = 32;                // heads per CTA: two groups of 16
constexpr int LD_SS = LT_BN + 8;         // row stride of S in shared memory, floats

static __host__ __device__ inline int latent_rowp(int row) { return (row + 15) / 16 * 16; }

template <int MAXR>                      // kv_rank <= MAXR; a warp owns MAXR / 4 value channels
__global__ void __launch_bounds__(LD_WARPS * 32)
latent_decode_kernel(const __nv_bfloat16 *__restrict__ qa, long long ldq, const __nv_bfloat16 *__restrict__ cache, int page_size,
                     const int *__restrict__ tok_seq, const int *__restrict__ tok_pos, const int *__restrict__ page_table, int pt_stride,
                     int n_heads, int row, int kv_rank, int n_splits, float scale_log2, __nv_bfloat16 *__restrict__ out, long long ldo,
                     float *__restrict__ ws_o, float *__restrict__ ws_ml, int window) {
  constexpr int SL = MAXR / 4;           // value channels of a warp
  constexpr int DT = SL / 8;
  constexpr int NT = LT_BN / 8;
  const int rowp = latent_rowp(row), ldr = rowp + 8, rch = rowp / 8, row8 = row / 8, KS = rowp / 16;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float *sS = reinterpret_cast<float *>(smem_raw);                               // [32][LD_SS]
  __nv_bfloat16 *sQ = reinterpret_cast<__nv_bfloat16 *>(sS + LD_HT * LD_SS);     // [32][ldr]
  __nv_bfloat16 *sK = sQ + LD_HT * ldr;                                          // [2][64][ldr]

  grid_dependents_launch();
  grid_dependency_wait();
  const int split = blockIdx.x, h0 = blockIdx.y * LD_HT, tok = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int hg = warp >> 2, part = warp & 3;       // head group; key quarter in the first product, channel quarter in the second
  const int pos = tok_pos[tok], len = pos + 1;
  const int *pt = page_table + (size_t)tok_seq[tok] * pt_stride;
  const int kstart = window > 0 ? max(0, pos - window + 1) : 0;      // the first key the token sees
  const int tile_first = kstart / LT_BN, tiles = (len + LT_BN - 1) / LT_BN - tile_first;
  const int per = (tiles + n_splits - 1) / n_splits;
  const int kt0 = tile_first + split * per, kt1 = min(tile_first + tiles, kt0 + per);
  const int n_iter = kt1 - kt0;
  const int head_a = h0 + hg * 16 + g, head_b = head_a + 8;

  if (n_iter <= 0) {                                // a run without keys: nothing to join
    if (n_splits > 1 && part == 0 && t == 0) {
      if (head_a < n_heads) {
        float *ml = ws_ml + (((size_t)tok * n_heads + head_a) * n_splits + split) * 2;
        ml[0] = -INFINITY, ml[1] = 0.f;
      }
      if (head_b < n_heads) {
        float *ml = ws_ml + (((size_t)tok * n_heads + head_b) * n_splits + split) * 2;
        ml[0] = -INFINITY, ml[1] = 0.f;
      }
    }
    return;
  }

  auto load_rows = [&](int kt, int stage) {
    __nv_bfloat16 *tk = sK + stage * LT_BN * ldr;
    for (int c = tid; c < LT_BN * rch; c += LD_WARPS * 32) {
      const int r = c / rch, ch = c - r * rch;
      const int j = kt * LT_BN + r;
      const bool ok = j >= kstart && j < len && ch < row8;
      const int jj = j >= kstart && j < len ? j : pos;       // a page before the window may have been given back
      const __nv_bfloat16 *src = cache + ((size_t)pt[jj / page_size] * page_size + jj % page_size) * (size_t)row + (ok ? ch : 0) * 8;
      cp_async16(tk + r * ldr + ch * 8, src, ok);
    }
  };
  for (int c = tid; c < LD_HT * rch; c += LD_WARPS * 32) {
    const int r = c / rch, ch = c - r * rch;
    const bool ok = h0 + r < n_heads && ch < row8;
    cp_async16(sQ + r * ldr + ch * 8, ok ? qa + (size_t)tok * ldq + (size_t)(h0 + r) * row + ch * 8 : qa, ok);
  }
  load_rows(kt0, 0);
  cp_async_commit();

  float o[DT][4];
#pragma unroll
  for (int i = 0; i < DT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  for (int it = 0; it < n_iter; ++it) {
    const int stage = it & 1;
    if (it + 1 < n_iter) load_rows(kt0 + it + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const __nv_bfloat16 *tk = sK + stage * LT_BN * ldr;

    {  // S for heads hg * 16 .. + 15 and keys part * 16 .. + 15 of the tile
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
      for (int ks = 0; ks < KS; ++ks) {
        unsigned qf[4], kb[4];
        ldmatrix_x4(qf, sQ + (hg * 16 + (lane & 15)) * ldr + ks * 16 + (lane >> 4) * 8);
        ldmatrix_x4(kb, tk + (part * 16 + (lane & 7) + (lane >> 4) * 8) * ldr + ks * 16 + ((lane >> 3) & 1) * 8);
        mma16816(s0, qf, kb[0], kb[1]);
        mma16816(s1, qf, kb[2], kb[3]);
      }
      float *ra = sS + (hg * 16 + g) * LD_SS + part * 16 + 2 * t, *rb = ra + 8 * LD_SS;
      *reinterpret_cast<float2 *>(ra) = make_float2(s0[0], s0[1]);
      *reinterpret_cast<float2 *>(rb) = make_float2(s0[2], s0[3]);
      *reinterpret_cast<float2 *>(ra + 8) = make_float2(s1[0], s1[1]);
      *reinterpret_cast<float2 *>(rb + 8) = make_float2(s1[2], s1[3]);
    }
    __syncthreads();

    float s[NT][4];
    const int k0 = (kt0 + it) * LT_BN;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const float2 a = *reinterpret_cast<const float2 *>(sS + (hg * 16 + g) * LD_SS + n * 8 + 2 * t);
      const float2 b = *reinterpret_cast<const float2 *>(sS + (hg * 16 + g + 8) * LD_SS + n * 8 + 2 * t);
      const int key = k0 + n * 8 + 2 * t;
      const bool see0 = key <= pos && key >= kstart, see1 = key + 1 <= pos && key + 1 >= kstart;
      s[n][0] = see0 ? a.x : -INFINITY;
      s[n][1] = see1 ? a.y : -INFINITY;
      s[n][2] = see0 ? b.x : -INFINITY;
      s[n][3] = see1 ? b.y : -INFINITY;
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      mx[0] = fmaxf(mx[0], fmaxf(s[n][0], s[n][1]));
      mx[1] = fmaxf(mx[1], fmaxf(s[n][2], s[n][3]));
    }
    float alpha[2], moff[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      moff[r] = m_new == -INFINITY ? 0.f : m_new * scale_log2;
      alpha[r] = m_run[r] == -INFINITY ? 0.f : exp2f(m_run[r] * scale_log2 - moff[r]);
      m_run[r] = m_new;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      s[n][0] = exp2f(fmaf(s[n][0], scale_log2, -moff[0]));
      s[n][1] = exp2f(fmaf(s[n][1], scale_log2, -moff[0]));
      s[n][2] = exp2f(fmaf(s[n][2], scale_log2, -moff[1]));
      s[n][3] = exp2f(fmaf(s[n][3], scale_log2, -moff[1]));
      sum[0] += s[n][0] + s[n][1];
      sum[1] += s[n][2] + s[n][3];
    }
    l_run[0] = l_run[0] * alpha[0] + sum[0];
    l_run[1] = l_run[1] * alpha[1] + sum[1];
#pragma unroll
    for (int i = 0; i < DT; ++i) {
      o[i][0] *= alpha[0];
      o[i][1] *= alpha[0];
      o[i][2] *= alpha[1];
      o[i][3] *= alpha[1];
    }
#pragma unroll
    for (int kk = 0; kk < LT_BN / 16; ++kk) {
      unsigned pa[4];
      pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int d2 = 0; d2 < DT / 2; ++d2) {
        const int col = part * SL + d2 * 16;
        if (col < kv_rank) {
          unsigned vb[4];
          ldmatrix_x4_trans(vb, tk + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldr + col + (lane >> 4) * 8);
          mma16816(o[2 * d2], pa, vb[0], vb[1]);
          mma16816(o[2 * d2 + 1], pa, vb[2], vb[3]);
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  if (n_splits == 1) {
    const float inv_a = 1.f / l_run[0], inv_b = 1.f / l_run[1];
    __nv_bfloat16 *oa = out + (size_t)tok * ldo + (size_t)head_a * kv_rank + 2 * t;
    __nv_bfloat16 *ob = out + (size_t)tok * ldo + (size_t)head_b * kv_rank + 2 * t;
#pragma unroll
    for (int i = 0; i < DT; ++i) {
      const int col = part * SL + i * 8;
      if (col < kv_rank) {
        if (head_a < n_heads) *reinterpret_cast<unsigned *>(oa + col) = pack_bf16(o[i][0] * inv_a, o[i][1] * inv_a);
        if (head_b < n_heads) *reinterpret_cast<unsigned *>(ob + col) = pack_bf16(o[i][2] * inv_b, o[i][3] * inv_b);
      }
    }
    return;
  }
  float *wa = ws_o + (((size_t)tok * n_heads + head_a) * n_splits + split) * kv_rank + 2 * t;
  float *wb = ws_o + (((size_t)tok * n_heads + head_b) * n_splits + split) * kv_rank + 2 * t;
#pragma unroll
  for (int i = 0; i < DT; ++i) {
    const int col = part * SL + i * 8;
    if (col < kv_rank) {
      if (head_a < n_heads) *reinterpret_cast<float2 *>(wa + col) = make_float2(o[i][0], o[i][1]);
      if (head_b < n_heads) *reinterpret_cast<float2 *>(wb + col) = make_float2(o[i][2], o[i][3]);
    }
  }
  if (part == 0 && t == 0) {
    if (head_a < n_heads) {
      float *ml = ws_ml + (((size_t)tok * n_heads + head_a) * n_splits + split) * 2;
      ml[0] = m_run[0] == -INFINITY ? -INFINITY : m_run[0] * scale_log2, ml[1] = l_run[0];
    }
    if (head_b < n_heads) {
      float *ml = ws_ml + (((size_t)tok * n_heads + head_b) * n_splits + split) * 2;
      ml[0] = m_run[1] == -INFINITY ? -INFINITY : m_run[1] * scale_log2, ml[1] = l_run[1];
    }
  }
}

// out[t, h, :] = sum_s w_s o_s / sum_s w_s l_s with w_s = 2^(m_s - max m): one CTA per (token, head).  The runs'
// weights go through shared memory once, so that the loads of the partial sums are independent of one another.
constexpr int LJ_MAX = 64;               // runs at most
__global__ void __launch_bounds__(128)
latent_join_kernel(const float *__restrict__ ws_o, const float *__restrict__ ws_ml, int n_splits, int kv_rank,
                   __nv_bfloat16 *__restrict__ out, long long ldo, int n_heads) {
  __shared__ float w[LJ_MAX];
  __shared__ float inv_s;
  grid_dependents_launch();
  grid_dependency_wait();
  const int h = blockIdx.x, tok = blockIdx.y;
  const float *ml = ws_ml + ((size_t)tok * n_heads + h) * n_splits * 2;
  const float *po = ws_o + ((size_t)tok * n_heads + h) * n_splits * (size_t)kv_rank;
  if (threadIdx.x < 32) {
    float m = -INFINITY;
    for (int s = threadIdx.x; s < n_splits; s += 32) m = fmaxf(m, ml[2 * s]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    for (int s = threadIdx.x; s < n_splits; s += 32) w[s] = ml[2 * s] == -INFINITY ? 0.f : exp2f(ml[2 * s] - m);
    __syncwarp();
    if (threadIdx.x == 0) {
      float l = 0.f;
      for (int s = 0; s < n_splits; ++s) l = fmaf(w[s], ml[2 * s + 1], l);       // in the order of the runs
      inv_s = 1.f / l;
    }
  }
  __syncthreads();
  const float inv = inv_s;
  for (int c = threadIdx.x; c < kv_rank; c += 128) {
    float acc = 0.f;
#pragma unroll 8
    for (int s = 0; s < n_splits; ++s) {
      const float v = po[(size_t)s * kv_rank + c];
      acc = w[s] != 0.f ? fmaf(w[s], v, acc) : acc;        // a run without keys left nothing there
    }
    out[(size_t)tok * ldo + (size_t)h * kv_rank + c] = __float2bfloat16(acc * inv);
  }
}

static int latent_maxr(int kv_rank) { return kv_rank <= 128 ? 128 : kv_rank <= 256 ? 256 : kv_rank <= 512 ? 512 : 0; }
static size_t latent_decode_smem(int row) {
  return (size_t)LD_HT * LD_SS * sizeof(float) + (size_t)(LD_HT + 2 * LT_BN) * (latent_rowp(row) + 8) * sizeof(__nv_bfloat16);
}

// 1 if rows of these sizes have an instantiation (16-byte pieces, whole value tiles, the tiles fit), else 0.
LLM_EXPORT int llm_latent_decode_supports(int kv_rank, int rot) {
  if (kv_rank <= 0 || rot < 0 || kv_rank % 16 || rot % 8) return 0;
  return latent_maxr(kv_rank) > 0 && latent_decode_smem(kv_rank + rot) <= (size_t)220 * 1024;
}

// Floats of workspace for n_splits > 1: partial sums, then (maximum, sum) pairs.
LLM_EXPORT long long llm_latent_decode_floats_needed(int n_tokens, int n_heads, int kv_rank, int n_splits) {
  return n_splits <= 1 ? 0 : (long long)n_tokens * n_heads * n_splits * (kv_rank + 2);
}

template <int MAXR>
static int launch_latent_decode(const void *qa, long long ldq, const void *cache, int page_size, const int *tok_seq, const int *tok_pos,
                                const int *page_table, int pt_stride, int n_tokens, int n_heads, int row, int kv_rank, int n_splits,
                                float scale, void *out, long long ldo, float *ws_o, float *ws_ml, int window, cudaStream_t stream) {
  const size_t smem = latent_decode_smem(row);
  auto kern = latent_decode_kernel<MAXR>;
  LLM_CHECK_CUDA(llm_allow_smem(kern, smem), "latent_decode attribute");
  dim3 grid(n_splits, (n_heads + LD_HT - 1) / LD_HT, n_tokens);
  llm_launch(kern, grid, dim3(LD_WARPS * 32), smem, stream, (const __nv_bfloat16 *)qa, ldq, (const __nv_bfloat16 *)cache, page_size,
             tok_seq, tok_pos, page_table, pt_stride, n_heads, row, kv_rank, n_splits, scale * 1.4426950408889634f, (__nv_bfloat16 *)out,
             ldo, ws_o, ws_ml, window);
  LLM_CHECK_LAUNCH("latent_decode");
  return LLM_OK;
}

LLM_EXPORT int llm_latent_decode(const void *qa, long long ldq, const void *cache, int page_size, const int *tok_seq, const int *tok_pos,
                                 const int *page_table, int pt_stride, int n_tokens, int n_heads, int kv_rank, int rot, int n_splits,
                                 float scale, void *out, long long ldo, float *ws, int window, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(window >= 0, "latent_decode: bad window");
  LLM_REQUIRE(llm_latent_decode_supports(kv_rank, rot), "latent_decode: rows of %d + %d channels are not supported", kv_rank, rot);
  LLM_REQUIRE(n_tokens > 0 && n_tokens <= 65535 && n_heads > 0 && page_size > 0 && n_splits >= 1 && n_splits <= LJ_MAX && ldq % 8 == 0 && ldo % 2 == 0 &&
                  (n_splits == 1 || ws),
              "latent_decode: bad sizes");
  const int row = kv_rank + rot;
  float *ws_o = ws, *ws_ml = ws ? ws + (size_t)n_tokens * n_heads * n_splits * kv_rank : nullptr;
  int st;
  switch (latent_maxr(kv_rank)) {
    case 128: st = launch_latent_decode<128>(qa, ldq, cache, page_size, tok_seq, tok_pos, page_table, pt_stride, n_tokens, n_heads, row, kv_rank, n_splits, scale, out, ldo, ws_o, ws_ml, window, stream); break;
    case 256: st = launch_latent_decode<256>(qa, ldq, cache, page_size, tok_seq, tok_pos, page_table, pt_stride, n_tokens, n_heads, row, kv_rank, n_splits, scale, out, ldo, ws_o, ws_ml, window, stream); break;
    default: st = launch_latent_decode<512>(qa, ldq, cache, page_size, tok_seq, tok_pos, page_table, pt_stride, n_tokens, n_heads, row, kv_rank, n_splits, scale, out, ldo, ws_o, ws_ml, window, stream); break;
  }
  if (st != LLM_OK || n_splits == 1) return st;
  llm_launch(latent_join_kernel, dim3(n_heads, n_tokens), dim3(128), 0, stream, (const float *)ws_o, (const float *)ws_ml, n_splits, kv_rank,
             (__nv_bfloat16 *)out, ldo, n_heads);
  LLM_CHECK_LAUNCH("latent_join");
  return LLM_OK;
}
