// Attention of the step's query tokens over the paged key/value cache, on the CUDA
// cores, for any head size up to 256 (steps of 2), any number of heads and groups,
// float or bf16 storage.  Serves prefill and decode alike: a query token at
// position p attends to cached positions [max(0, p + 1 - window), p] of its own
// sequence, which the rope/cache-write kernel has filled before this runs.
//
// Formulas (SimonWaldherr/RustyLLM): query head h uses KV head g = h / (H/G)
// (src/model.rs:6034-6198); score_t = (q_h . K[t, g]) / sqrt(head_dim); streaming
// softmax with running (max, denominator, output) in 32-bit (src/model.rs:5807-5869);
// causality by loop bound, window start max(0, pos + 1 - W) (src/model.rs:7239-7243).
//
// One CTA of eight warps per (token, query head).  Keys are taken 32 at a time in position
// order, chunk c of a token's keys by warp c % 8; within a chunk every key's row is read by
// the whole warp (lane l holds dimensions l, l + 32, ...: consecutive lanes, consecutive
// addresses, for keys and values alike) and its score is the warp's sum of the lanes'
// partial products.  At the end the warps' (max, denominator, output) are merged in the order
// of the warps.  Chunks, their warps and every order of summation depend on the token's
// position and the window alone, so the result for a position does not depend on the batch
// or on how the tokens were split into steps - bit for bit.
#include <math.h>

#include "common.cuh"

#define ATT_WARPS 8
#define ATT_MAX_HD 256

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_simt_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ k_pool,
                      const T* __restrict__ v_pool, const int* __restrict__ page_table, int max_pages,
                      const int* __restrict__ slot_of_token, const int* __restrict__ positions,
                      T* __restrict__ out, int ldo, int H, int G, int hd, int vd, float scale, int window) {
  constexpr int NE = ATT_MAX_HD / 32;
  __shared__ float s_acc[ATT_WARPS][ATT_MAX_HD];
  __shared__ float s_max[ATT_WARPS], s_sum[ATT_WARPS];
  const int m = blockIdx.x, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = h / (H / G);
  const int pos = positions[m];
  const int slot = slot_of_token[m];
  const int* pages = page_table + (size_t)slot * max_pages;
  const T* qrow = q + (size_t)m * ldq + (size_t)h * hd;
  float qv[NE];                       // this lane's dimensions of the query, scaled
#pragma unroll
  for (int e = 0; e < NE; ++e) {
    const int d = lane + 32 * e;
    qv[e] = d < hd ? rl_ld(qrow + d) * scale : 0.f;
  }

  const int start = (window > 0 && pos + 1 - window > 0) ? pos + 1 - window : 0;
  float acc[NE];
#pragma unroll
  for (int e = 0; e < NE; ++e) acc[e] = 0.f;
  float run_max = -INFINITY, run_sum = 0.f;
  const size_t head_off = (size_t)g * RL_PAGE * hd, v_head_off = (size_t)g * RL_PAGE * vd;
  const size_t page_stride = (size_t)G * RL_PAGE * hd, v_page_stride = (size_t)G * RL_PAGE * vd;

  for (int t0 = start + 32 * warp; t0 <= pos; t0 += 32 * ATT_WARPS) {
    const int n = min(32, pos - t0 + 1);
    float s = -INFINITY;              // lane j: the score of key t0 + j
    for (int j = 0; j < n; ++j) {
      const int tj = t0 + j;
      const T* krow = k_pool + (size_t)pages[tj / RL_PAGE] * page_stride + head_off + (size_t)(tj % RL_PAGE) * hd;
      float part = 0.f;
#pragma unroll
      for (int e = 0; e < NE; ++e) {
        const int d = lane + 32 * e;
        if (d < hd) part = fmaf(qv[e], rl_ld(krow + d), part);
      }
      const float sj = rl_warp_sum(part);
      if (lane == j) s = sj;
    }
    const float new_max = fmaxf(run_max, rl_warp_max(s));   // finite: key t0 is valid
    const float corr = expf(run_max - new_max);              // exp(-inf) = 0 on the warp's first chunk
    const float p = (lane < n) ? expf(s - new_max) : 0.f;
    run_sum = run_sum * corr + rl_warp_sum(p);
    run_max = new_max;
#pragma unroll
    for (int e = 0; e < NE; ++e) acc[e] *= corr;
    for (int j = 0; j < n; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const int tj = t0 + j;
      const T* vrow = v_pool + (size_t)pages[tj / RL_PAGE] * v_page_stride + v_head_off + (size_t)(tj % RL_PAGE) * vd;
#pragma unroll
      for (int e = 0; e < NE; ++e) {
        const int d = lane + 32 * e;
        if (d < vd) acc[e] = fmaf(pj, rl_ld(vrow + d), acc[e]);
      }
    }
  }
  // ---- the warps' results, merged in the order of the warps (warp 0 always holds keys) ----
  if (lane == 0) { s_max[warp] = run_max; s_sum[warp] = run_sum; }
#pragma unroll
  for (int e = 0; e < NE; ++e) {
    const int d = lane + 32 * e;
    if (d < vd) s_acc[warp][d] = acc[e];
  }
  __syncthreads();
  float M = -INFINITY;
#pragma unroll
  for (int w = 0; w < ATT_WARPS; ++w) M = fmaxf(M, s_max[w]);
  float wgt[ATT_WARPS], L = 0.f;
#pragma unroll
  for (int w = 0; w < ATT_WARPS; ++w) {
    wgt[w] = s_max[w] > -INFINITY ? expf(s_max[w] - M) : 0.f;
    L += s_sum[w] * wgt[w];
  }
  const float inv = 1.0f / L;
  T* orow = out + (size_t)m * ldo + (size_t)h * vd;
  for (int d = threadIdx.x; d < vd; d += ATT_WARPS * 32) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) o += s_acc[w][d] * wgt[w];
    rl_st(orow + d, o * inv);
  }
}

// q: [M, ldq] with head h at columns [h*hd, (h+1)*hd); out: [M, ldo] with head h at columns
// [h*vd, (h+1)*vd).  k_pool: [num_pages, G, RL_PAGE, hd], v_pool: [num_pages, G, RL_PAGE, vd]
// (value heads may be narrower or wider than key heads: the reference keeps value_dim apart
// from head_dim, src/model.rs:33, 67-69), both in the same dtype as q.
extern "C" int rl_attention_simt(const void* q, int ldq, const void* k_pool, const void* v_pool,
                                 int dtype, const int* page_table, int max_pages,
                                 const int* slot_of_token, const int* positions, void* out, int ldo,
                                 int num_tokens, int num_heads, int num_kv_heads, int head_dim, int value_dim,
                                 float scale, int window, cudaStream_t stream) {
  RL_REQUIRE(num_tokens >= 0 && num_heads > 0 && num_kv_heads > 0, "rl_attention_simt: bad sizes");
  RL_REQUIRE(num_heads % num_kv_heads == 0, "rl_attention_simt: %d heads are no multiple of %d KV heads",
             num_heads, num_kv_heads);
  RL_REQUIRE(head_dim > 0 && head_dim <= ATT_MAX_HD && head_dim % 2 == 0,
             "rl_attention_simt: head_dim %d must be even and <= %d", head_dim, ATT_MAX_HD);
  RL_REQUIRE(value_dim > 0 && value_dim <= ATT_MAX_HD, "rl_attention_simt: value_dim %d must lie in (0, %d]", value_dim, ATT_MAX_HD);
  RL_REQUIRE(ldq >= num_heads * head_dim && ldo >= num_heads * value_dim, "rl_attention_simt: row strides too small");
  RL_REQUIRE(window >= 0, "rl_attention_simt: negative window");
  if (num_tokens == 0) return RL_OK;
  dim3 grid(num_tokens, num_heads);
  if (dtype == RL_F32)
    attention_simt_kernel<float><<<grid, ATT_WARPS * 32, 0, stream>>>(
        (const float*)q, ldq, (const float*)k_pool, (const float*)v_pool, page_table, max_pages,
        slot_of_token, positions, (float*)out, ldo, num_heads, num_kv_heads, head_dim, value_dim, scale, window);
  else if (dtype == RL_BF16)
    attention_simt_kernel<__nv_bfloat16><<<grid, ATT_WARPS * 32, 0, stream>>>(
        (const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, page_table,
        max_pages, slot_of_token, positions, (__nv_bfloat16*)out, ldo, num_heads, num_kv_heads, head_dim, value_dim, scale, window);
  else
    RL_REQUIRE(false, "rl_attention_simt: unknown dtype %d", dtype);
  RL_LAUNCH_CHECK("rl_attention_simt");
  return RL_OK;
}
