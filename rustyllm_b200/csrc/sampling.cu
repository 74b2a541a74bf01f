// Turning rows of 32-bit logits into token ids on the device: repeat penalty,
// greedy argmax, and temperature sampling with an optional min-p cut.
//
// Semantics (SimonWaldherr/RustyLLM src/sampling.rs):
//   repeat penalty: for each token of the recent window, once per occurrence,
//     l > 0 -> l / p, else l * p; non-finite -> -inf            (321-338)
//   greedy: highest finite logit, the first one wins; none finite -> 0 (341-356)
//   temperature: w_i = exp((l_i - max) / T) with non-finite logits as -inf,
//     r = u * sum(w), answer = first i whose running sum exceeds r, else the last
//     candidate (98-123, 186-211); min-p drops w_i < min_p (the top weight is 1)
//     before the draw (125-148).
// The uniform u in [0, 1) comes from the host's per-sequence generator.  Sums are
// taken in a fixed order (per-thread contiguous segments, then segment totals in
// index order), so a row's answer does not depend on the other rows.
#include <math.h>

#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ float finite_or_neg_inf(float v) { return isfinite(v) ? v : -INFINITY; }

// ------------------------------------------------------------------ repeat penalty
__global__ void repeat_penalty_rows_kernel(float* __restrict__ logits, int rows, int vocab,
                                           const int* __restrict__ recent, const int* __restrict__ recent_len,
                                           int window, float penalty) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  float* l = logits + (size_t)row * vocab;
  const int n = min(recent_len[row], window);
  for (int i = 0; i < n; ++i) {
    const int tok = recent[(size_t)row * window + i];
    if (tok < 0 || tok >= vocab) continue;
    const float v = l[tok];
    l[tok] = !isfinite(v) ? -INFINITY : (v > 0.f ? v / penalty : v * penalty);
  }
}

// recent: [rows, window] token ids, oldest first, of which the first recent_len[row] count.
extern "C" int rl_repeat_penalty(float* logits, int rows, int vocab, const int* recent,
                                 const int* recent_len, int window, float penalty, cudaStream_t stream) {
  RL_REQUIRE(rows >= 0 && vocab > 0 && window > 0, "rl_repeat_penalty: bad sizes");
  RL_REQUIRE(isfinite(penalty) && penalty > 0.f, "rl_repeat_penalty: penalty must be finite and > 0");
  if (rows == 0 || penalty == 1.0f) return RL_OK;
  repeat_penalty_rows_kernel<<<(rows + 63) / 64, 64, 0, stream>>>(logits, rows, vocab, recent, recent_len, window, penalty);
  RL_LAUNCH_CHECK("rl_repeat_penalty");
  return RL_OK;
}

// ------------------------------------------------------------------ greedy
__device__ __forceinline__ void argmax_combine(float& bv, int& bi, float ov, int oi) {
  if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
}

__device__ int block_argmax(const float* __restrict__ l, int vocab, float scale) {
  __shared__ float sv[SAMPLE_THREADS / 32];
  __shared__ int si[SAMPLE_THREADS / 32];
  __shared__ int result;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = finite_or_neg_inf(l[i]) * scale;
    if (v > bv) { bv = v; bi = i; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    argmax_combine(bv, bi, ov, oi);
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) argmax_combine(bv, bi, sv[w], si[w]);
    result = (bi == 0x7fffffff) ? 0 : bi;   // nothing finite: token 0
  }
  __syncthreads();
  return result;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, int vocab, int* __restrict__ out) {
  const int row = blockIdx.x;
  const int r = block_argmax(logits + (size_t)row * vocab, vocab, 1.0f);
  if (threadIdx.x == 0) out[row] = r;
}

extern "C" int rl_argmax(const float* logits, int rows, int vocab, int* out, cudaStream_t stream) {
  RL_REQUIRE(rows >= 0 && vocab > 0, "rl_argmax: bad sizes rows=%d vocab=%d", rows, vocab);
  if (rows == 0) return RL_OK;
  argmax_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(logits, vocab, out);
  RL_LAUNCH_CHECK("rl_argmax");
  return RL_OK;
}

// ------------------------------------------------------------------ temperature
// Per-row temperature: a row with temperature < 1e-6 is answered greedily, as the
// reference does (src/sampling.rs:78-85).
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_temperature_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
                          const float* __restrict__ uniform, const float* __restrict__ min_p,
                          int* __restrict__ out) {
  __shared__ float seg_sum[SAMPLE_THREADS];
  __shared__ float red[SAMPLE_THREADS / 32];
  __shared__ float s_max, s_total;
  __shared__ int s_seg;
  const int row = blockIdx.x;
  const float* l = logits + (size_t)row * vocab;
  const float temp = temperature[row];
  if (temp < 1e-6f) {
    const int r = block_argmax(l, vocab, 1.0f);
    if (threadIdx.x == 0) out[row] = r;
    return;
  }
  const float inv_temp = 1.0f / temp;
  const float cut = min_p ? min_p[row] : 0.f;

  // 1. maximum of the scaled finite logits
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) mx = fmaxf(mx, finite_or_neg_inf(l[i]) * inv_temp);
  mx = rl_warp_max(mx);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = red[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) t = fmaxf(t, red[w]);
    s_max = t;
  }
  __syncthreads();
  mx = s_max;
  if (!(mx > -INFINITY)) {  // nothing finite
    if (threadIdx.x == 0) out[row] = 0;
    return;
  }

  // 2. weights, summed over contiguous per-thread segments
  const int seg = (vocab + blockDim.x - 1) / blockDim.x;
  const int lo = threadIdx.x * seg, hi = min(lo + seg, vocab);
  float mine = 0.f;
  for (int i = lo; i < hi; ++i) {
    const float w = expf(finite_or_neg_inf(l[i]) * inv_temp - mx);
    if (w >= cut) mine += w;
  }
  seg_sum[threadIdx.x] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int t = 0; t < (int)blockDim.x; ++t) total += seg_sum[t];
    s_total = total;
    const float r = uniform[row] * total;
    // first segment whose inclusive running sum exceeds r
    float c = 0.f;
    int chosen = -1;
    for (int t = 0; t < (int)blockDim.x; ++t) {
      const float incl = c + seg_sum[t];
      if (incl > r && seg_sum[t] > 0.f) { chosen = t; break; }
      c = incl;
    }
    s_seg = chosen;
    seg_sum[0] = c;  // exclusive sum in front of the chosen segment (slot 0 is consumed)
  }
  __syncthreads();
  const float total = s_total;
  if (!isfinite(total) || total <= 0.f) {  // src/sampling.rs:112-119: fall back to the best index
    const int r = block_argmax(l, vocab, 1.0f);
    if (threadIdx.x == 0) out[row] = r;
    return;
  }
  const int chosen = s_seg;
  if (chosen < 0) {
    // rounding left r at or above the total: the last kept candidate (src/sampling.rs:210)
    if (threadIdx.x == 0) {
      int last = vocab - 1;  // without a cut the reference answers n - 1 (src/sampling.rs:211)
      for (int i = vocab - 1; cut > 0.f && i >= 0; --i) {
        const float w = expf(finite_or_neg_inf(l[i]) * inv_temp - mx);
        if (w >= cut && w > 0.f) { last = i; break; }
      }
      out[row] = last;
    }
    return;
  }
  if ((int)threadIdx.x == chosen) {
    const float r = uniform[row] * total;
    float c = seg_sum[0];
    int answer = -1, last = lo;
    for (int i = lo; i < hi; ++i) {
      const float w = expf(finite_or_neg_inf(l[i]) * inv_temp - mx);
      if (w >= cut && w > 0.f) {
        last = i;
        c += w;
        if (c > r) { answer = i; break; }
      }
    }
    out[row] = answer >= 0 ? answer : last;
  }
}

// temperature, uniform: [rows]; min_p: [rows] or nullptr.
extern "C" int rl_sample_temperature(const float* logits, int rows, int vocab, const float* temperature,
                                     const float* uniform, const float* min_p, int* out,
                                     cudaStream_t stream) {
  RL_REQUIRE(rows >= 0 && vocab > 0, "rl_sample_temperature: bad sizes rows=%d vocab=%d", rows, vocab);
  if (rows == 0) return RL_OK;
  sample_temperature_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(logits, vocab, temperature, uniform, min_p, out);
  RL_LAUNCH_CHECK("rl_sample_temperature");
  return RL_OK;
}
