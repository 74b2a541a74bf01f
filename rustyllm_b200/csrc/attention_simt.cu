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
// One warp per (token, query head).  Keys are taken 32 at a time in position
// order, so the result for a position does not depend on the batch or on how the
// tokens were split into steps.
#include <math.h>

#include "common.cuh"

#define ATT_WARPS 4
#define ATT_MAX_HD 256

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const T* __restrict__ k, int hd);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ q, const float* __restrict__ k, int hd) {
  float s = 0.f;
  for (int d = 0; d < hd; ++d) s = fmaf(q[d], k[d], s);
  return s;
}
template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ q, const __nv_bfloat16* __restrict__ k, int hd) {
  float s = 0.f;
  for (int d = 0; d < hd; d += 2) {
    const float2 kk = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(k + d));
    s = fmaf(q[d], kk.x, s);
    s = fmaf(q[d + 1], kk.y, s);
  }
  return s;
}

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_simt_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ k_pool,
                      const T* __restrict__ v_pool, const int* __restrict__ page_table, int max_pages,
                      const int* __restrict__ slot_of_token, const int* __restrict__ positions,
                      T* __restrict__ out, int ldo, int H, int G, int hd, int vd, float scale, int window) {
  __shared__ float qs[ATT_WARPS][ATT_MAX_HD];
  const int m = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * ATT_WARPS + warp;
  if (h >= H) return;  // whole warp leaves; no block-wide barrier below
  const int g = h / (H / G);
  const int pos = positions[m];
  const int slot = slot_of_token[m];
  const int* pages = page_table + (size_t)slot * max_pages;
  const T* qrow = q + (size_t)m * ldq + (size_t)h * hd;
  for (int d = lane; d < hd; d += 32) qs[warp][d] = rl_ld(qrow + d) * scale;
  __syncwarp();

  const int start = (window > 0 && pos + 1 - window > 0) ? pos + 1 - window : 0;
  constexpr int NE = ATT_MAX_HD / 32;
  float acc[NE];
#pragma unroll
  for (int e = 0; e < NE; ++e) acc[e] = 0.f;
  float run_max = -INFINITY, run_sum = 0.f;
  const size_t head_off = (size_t)g * RL_PAGE * hd, v_head_off = (size_t)g * RL_PAGE * vd;
  const size_t page_stride = (size_t)G * RL_PAGE * hd, v_page_stride = (size_t)G * RL_PAGE * vd;

  for (int t0 = start; t0 <= pos; t0 += 32) {
    const int t = t0 + lane;
    float s = -INFINITY;
    if (t <= pos) {
      const T* krow = k_pool + (size_t)pages[t / RL_PAGE] * page_stride + head_off + (size_t)(t % RL_PAGE) * hd;
      s = dot_row<T>(qs[warp], krow, hd);
    }
    const float new_max = fmaxf(run_max, rl_warp_max(s));   // finite: key t0 is always valid
    const float corr = expf(run_max - new_max);              // exp(-inf) = 0 on the first chunk
    const float p = (t <= pos) ? expf(s - new_max) : 0.f;
    run_sum = run_sum * corr + rl_warp_sum(p);
    run_max = new_max;
#pragma unroll
    for (int e = 0; e < NE; ++e) acc[e] *= corr;
    const int n = min(32, pos - t0 + 1);
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
  const float inv = 1.0f / run_sum;
  T* orow = out + (size_t)m * ldo + (size_t)h * vd;
#pragma unroll
  for (int e = 0; e < NE; ++e) {
    const int d = lane + 32 * e;
    if (d < vd) rl_st(orow + d, acc[e] * inv);
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
  dim3 grid(num_tokens, (num_heads + ATT_WARPS - 1) / ATT_WARPS);
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
