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
// taken in a fixed order (each warp a contiguous range of the vocabulary, 32
// neighbouring entries a load; then the ranges' totals in index order), so a row's
// answer does not depend on the other rows.
//
// A row is the work of a thread-block cluster of up to 8 CTAs (8 while the call's rows leave
// room for that, else 4, 2 or 1), each with its share of the vocabulary, so that enough loads
// are in flight to read a row of 128 K logits in a few microseconds; the CTAs exchange their
// maxima and sums through distributed shared memory.  The sums are taken over the same eight
// parts of the row whatever the number of CTAs, so a row's draw is the same in a call of one
// row and of a hundred.  Every path through a kernel passes the same cluster barriers in all CTAs.
#include <math.h>

#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ float finite_or_neg_inf(float v) { return isfinite(v) ? v : -INFINITY; }

// ------------------------------------------------------------------ repeat penalty
// The reference walks the recent tokens in order and pushes a token's logit toward zero once
// for every time it occurs (src/sampling.rs:321-338).  One warp a row: the lane that holds a
// token's first occurrence counts its occurrences and applies the rule that many times to the
// one value it loads, so the row's loads are in flight together instead of one after another
// (64 recent tokens: 33 us as a chain of read-modify-writes, 3 us so).
__global__ void __launch_bounds__(128)
repeat_penalty_rows_kernel(float* __restrict__ logits, int rows, int vocab,
                           const int* __restrict__ recent, const int* __restrict__ recent_len,
                           int window, float penalty) {
  __shared__ int staged[4][256];
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  float* l = logits + (size_t)row * vocab;
  const int* r = recent + (size_t)row * window;
  const int n = min(recent_len[row], window);
  if (n <= 256) {                          // the row's recent tokens once into shared memory
    int* mine = staged[threadIdx.x >> 5];
    for (int i = lane; i < n; i += 32) mine[i] = r[i];
    __syncwarp();
    r = mine;
  }
  for (int i = lane; i < n; i += 32) {
    const int tok = r[i];
    if (tok < 0 || tok >= vocab) continue;
    int times = 1;
    bool first = true;
    for (int j = 0; j < n; ++j) {
      if (j == i || r[j] != tok) continue;
      if (j < i) { first = false; break; }
      ++times;
    }
    if (!first) continue;
    float v = l[tok];
    for (int t = 0; t < times; ++t) v = !isfinite(v) ? -INFINITY : (v > 0.f ? v / penalty : v * penalty);
    l[tok] = v;
  }
}

// recent: [rows, window] token ids, oldest first, of which the first recent_len[row] count.
extern "C" int rl_repeat_penalty(float* logits, int rows, int vocab, const int* recent,
                                 const int* recent_len, int window, float penalty, cudaStream_t stream) {
  RL_REQUIRE(rows >= 0 && vocab > 0 && window > 0, "rl_repeat_penalty: bad sizes");
  RL_REQUIRE(isfinite(penalty) && penalty > 0.f, "rl_repeat_penalty: penalty must be finite and > 0");
  if (rows == 0 || penalty == 1.0f) return RL_OK;
  repeat_penalty_rows_kernel<<<(rows + 3) / 4, 128, 0, stream>>>(logits, rows, vocab, recent, recent_len, window, penalty);
  RL_LAUNCH_CHECK("rl_repeat_penalty");
  return RL_OK;
}

// ------------------------------------------------------------------ cluster helpers
#define SAMPLE_CLUSTER 8      // CTAs a row at most (the launch chooses 1, 2, 4 or 8: sample_cluster_for)

__device__ __forceinline__ uint32_t sample_cluster_size() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t sample_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void sample_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the 32-bit word at `p` (an address in this CTA's shared memory) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t sample_peer_u32(const void* p, uint32_t rank) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  uint32_t ra, v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a), "r"(rank));
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(ra) : "memory");
  return v;
}
// this CTA's share [lo, hi) of a row: whole multiples of 1024 entries, so that each warp's
// part of it starts on a multiple of 32
__device__ __forceinline__ void sample_slice(int vocab, int* lo, int* hi, int* per_warp) {
  const int ncta = (int)sample_cluster_size();
  const int slice = ((vocab + ncta - 1) / ncta + SAMPLE_THREADS - 1) / SAMPLE_THREADS * SAMPLE_THREADS;
  *lo = min((int)sample_cluster_rank() * slice, vocab);
  *hi = min(*lo + slice, vocab);
  *per_warp = slice / (SAMPLE_THREADS / 32);
}

// ------------------------------------------------------------------ greedy
__device__ __forceinline__ void argmax_combine(float& bv, int& bi, float ov, int oi) {
  if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
}

// Highest finite logit of the row, the first one wins; token 0 if none is finite.  Called
// by all threads of all CTAs of the cluster; CTA 0's thread 0 gets the answer (others -1).
// Passes two cluster barriers.
__device__ int cluster_argmax(const float* __restrict__ l, int vocab) {
  __shared__ float sv[SAMPLE_THREADS / 32];
  __shared__ int si[SAMPLE_THREADS / 32];
  __shared__ float cta_v;
  __shared__ int cta_i;
  int lo, hi, per_warp;
  sample_slice(vocab, &lo, &hi, &per_warp);
  float bv = -INFINITY;
  int bi = 0x7fffffff;
#pragma unroll 8
  for (int i = lo + (int)threadIdx.x; i < hi; i += SAMPLE_THREADS) {
    const float v = finite_or_neg_inf(l[i]);
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
    for (int w = 1; w < SAMPLE_THREADS / 32; ++w) argmax_combine(bv, bi, sv[w], si[w]);
    cta_v = bv; cta_i = bi;
  }
  sample_cluster_sync();
  int result = -1;
  if (threadIdx.x == 0 && sample_cluster_rank() == 0) {
    for (uint32_t r = 1; r < sample_cluster_size(); ++r)
      argmax_combine(bv, bi, __uint_as_float(sample_peer_u32(&cta_v, r)), (int)sample_peer_u32(&cta_i, r));
    result = (bi == 0x7fffffff) ? 0 : bi;   // nothing finite: token 0
  }
  sample_cluster_sync();                    // nobody leaves while its shared memory may still be read
  return result;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, int vocab, int* __restrict__ out) {
  const int row = blockIdx.x / (int)sample_cluster_size();
  const int r = cluster_argmax(logits + (size_t)row * vocab, vocab);
  if (r >= 0) out[row] = r;
}

// CTAs a row: eight while they fill no more than half of the SMs, else the most (4, 2, 1) that leave
// every CTA of the launch an SM of its own - a CTA has 1,024 threads, two fit an SM, and 64 rows of
// eight CTAs ran as two waves (temperature sampling of 64 rows of 128,256 logits: 51 us, as two CTAs a
// row 26 us; 256 rows: 173 and 66 us; argmax of 256 rows: 53 and 26 us).  Small vocabularies: one CTA.
static int sample_cluster_for(int rows, int vocab) {
  const int sms = rl_num_sms();
  return vocab < 16384 ? 1 : rows * 16 <= sms ? 8 : rows * 4 <= sms ? 4 : rows * 2 <= sms ? 2 : 1;
}

static cudaError_t sample_launch_cluster(void (*kernel)(const float*, int, int*), int rows, cudaStream_t stream,
                                         const float* logits, int vocab, int* out) {
  const int cl = sample_cluster_for(rows, vocab);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(rows * cl);
  cfg.blockDim = dim3(SAMPLE_THREADS);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cl; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, logits, vocab, out);
}

extern "C" int rl_argmax(const float* logits, int rows, int vocab, int* out, cudaStream_t stream) {
  RL_REQUIRE(rows >= 0 && vocab > 0, "rl_argmax: bad sizes rows=%d vocab=%d", rows, vocab);
  RL_REQUIRE((long long)rows * SAMPLE_CLUSTER <= 0x7fffffffLL, "rl_argmax: too many rows");
  if (rows == 0) return RL_OK;
  cudaError_t e = sample_launch_cluster(argmax_kernel, rows, stream, logits, vocab, out);
  RL_REQUIRE(e == cudaSuccess, "rl_argmax: launch failed: %s", cudaGetErrorString(e));
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
  constexpr int NW = SAMPLE_THREADS / 32;
  // The row is summed in SAMPLE_CLUSTER parts of NW ranges each, whatever the number of CTAs the
  // launch gave it (a CTA takes SAMPLE_CLUSTER / ncta parts in turn): every sum below is the same
  // additions in the same order for 1, 2, 4 and 8 CTAs a row, so a row's draw does not depend on
  // how many rows the call has.
  __shared__ float range_sum[SAMPLE_CLUSTER][NW];
  __shared__ float part_sum[SAMPLE_CLUSTER];
  __shared__ float red[NW];
  __shared__ float cta_max;
  const uint32_t ncta = sample_cluster_size();
  const int row = blockIdx.x / (int)ncta;
  const uint32_t rank = sample_cluster_rank();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* l = logits + (size_t)row * vocab;
  const float temp = temperature[row];
  if (temp < 1e-6f) {
    const int r = cluster_argmax(l, vocab);
    if (r >= 0) out[row] = r;
    return;
  }
  const float inv_temp = 1.0f / temp;
  const float cut = min_p ? min_p[row] : 0.f;
  const int part = ((vocab + SAMPLE_CLUSTER - 1) / SAMPLE_CLUSTER + SAMPLE_THREADS - 1) / SAMPLE_THREADS * SAMPLE_THREADS;
  const int per_warp = part / NW;                 // tokens a range
  const int ppc = SAMPLE_CLUSTER / (int)ncta;     // parts a CTA
  const int lo = min((int)rank * ppc * part, vocab), hi = min(lo + ppc * part, vocab);

  // 1. maximum of the scaled finite logits: this CTA's share, then the cluster's
  float mx = -INFINITY;
#pragma unroll 8
  for (int i = lo + (int)threadIdx.x; i < hi; i += SAMPLE_THREADS) mx = fmaxf(mx, finite_or_neg_inf(l[i]) * inv_temp);
  mx = rl_warp_max(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = red[0];
    for (int w = 1; w < NW; ++w) t = fmaxf(t, red[w]);
    cta_max = t;
  }
  sample_cluster_sync();                                       // barrier 1
  mx = -INFINITY;
  for (uint32_t r = 0; r < ncta; ++r) mx = fmaxf(mx, __uint_as_float(sample_peer_u32(&cta_max, r)));
  if (!(mx > -INFINITY)) {  // nothing finite
    if (threadIdx.x == 0 && rank == 0) out[row] = 0;
    sample_cluster_sync();
    return;
  }

  // 2. weights, summed over one contiguous range of the vocabulary per warp and part
  for (int q = 0; q < ppc; ++q) {
    const int plo = min(lo + q * part, hi);
    const int wlo = min(plo + warp * per_warp, hi), whi = min(min(wlo + per_warp, plo + part), hi);
    float mine = 0.f;
#pragma unroll 8
    for (int i = wlo + lane; i < whi; i += 32) {
      const float w = expf(finite_or_neg_inf(l[i]) * inv_temp - mx);
      if (w >= cut) mine += w;
    }
    for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
    if (lane == 0) range_sum[q][warp] = mine;
  }
  __syncthreads();
  if ((int)threadIdx.x < ppc) {
    float t = 0.f;
    for (int w = 0; w < NW; ++w) t += range_sum[threadIdx.x][w];
    part_sum[threadIdx.x] = t;
  }
  sample_cluster_sync();                                       // barrier 2
  // every thread walks the parts' totals (the same additions in the same order everywhere)
  float totals[SAMPLE_CLUSTER];
  float total = 0.f;
#pragma unroll
  for (int p = 0; p < SAMPLE_CLUSTER; ++p) {
    totals[p] = __uint_as_float(sample_peer_u32(&part_sum[p % ppc], (uint32_t)(p / ppc)));
    total += totals[p];
  }
  sample_cluster_sync();                                       // barrier 3: shared memory of peers is not read below
  if (!isfinite(total) || total <= 0.f) {  // src/sampling.rs:112-119: fall back to the best index
    const int r = cluster_argmax(l, vocab);
    if (r >= 0) out[row] = r;
    return;
  }
  const float r = uniform[row] * total;
  float before = 0.f;       // sum in front of the chosen part
  int chosen_part = -1;
#pragma unroll
  for (int p = 0; p < SAMPLE_CLUSTER; ++p) {
    if (chosen_part < 0) {
      const float incl = before + totals[p];
      if (incl > r && totals[p] > 0.f) chosen_part = p; else before = incl;
    }
  }
  if (chosen_part < 0) {
    // rounding left r at or above the total: the last kept candidate (src/sampling.rs:210)
    if (threadIdx.x == 0 && rank == 0) {
      int last = vocab - 1;  // without a cut the reference answers n - 1 (src/sampling.rs:211)
      for (int i = vocab - 1; cut > 0.f && i >= 0; --i) {
        const float w = expf(finite_or_neg_inf(l[i]) * inv_temp - mx);
        if (w >= cut && w > 0.f) { last = i; break; }
      }
      out[row] = last;
    }
    return;
  }
  if ((int)rank != chosen_part / ppc) return;
  const int q = chosen_part % ppc;
  int chosen = -1;
  for (int w = 0; w < NW; ++w) {
    const float incl = before + range_sum[q][w];
    if (incl > r && range_sum[q][w] > 0.f) { chosen = w; break; }
    before = incl;
  }
  if (chosen < 0) {          // the part's total said "in here", the walk over its ranges "not yet": its last range that kept anything
    for (int w = NW - 1; w >= 0; --w) if (range_sum[q][w] > 0.f) { chosen = w; break; }
    before = -INFINITY;      // the walk below then never passes r and ends at the range's last kept entry
  }
  if (warp != chosen) return;
  // 3. the chosen warp walks its range, 32 entries at a time, to the entry where the
  // running sum passes r
  const int plo = min(lo + q * part, hi);
  const int wlo = min(plo + warp * per_warp, hi), whi = min(min(wlo + per_warp, plo + part), hi);
  float c = before;
  int last_kept = wlo;
  for (int i0 = wlo; i0 < whi; i0 += 32) {
    const int i = i0 + lane;
    float w = i < whi ? expf(finite_or_neg_inf(l[i]) * inv_temp - mx) : 0.f;
    const bool kept = w >= cut && w > 0.f;
    if (!kept) w = 0.f;
    float incl = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const float v = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += v; }
    const unsigned passed = __ballot_sync(0xffffffffu, kept && c + incl > r);
    if (passed) {
      if (lane == 0) out[row] = i0 + __ffs(passed) - 1;
      return;
    }
    const unsigned kept_mask = __ballot_sync(0xffffffffu, kept);
    if (kept_mask) last_kept = i0 + 31 - __clz(kept_mask);
    c += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) out[row] = last_kept;    // rounding in the walk: the range's last kept entry
}

// temperature, uniform: [rows]; min_p: [rows] or nullptr.
extern "C" int rl_sample_temperature(const float* logits, int rows, int vocab, const float* temperature,
                                     const float* uniform, const float* min_p, int* out,
                                     cudaStream_t stream) {
  RL_REQUIRE(rows >= 0 && vocab > 0, "rl_sample_temperature: bad sizes rows=%d vocab=%d", rows, vocab);
  if (rows == 0) return RL_OK;
  const int cl = sample_cluster_for(rows, vocab);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(rows * cl);
  cfg.blockDim = dim3(SAMPLE_THREADS);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cl; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, sample_temperature_kernel, logits, vocab, temperature, uniform, min_p, out);
  RL_REQUIRE(e == cudaSuccess, "rl_sample_temperature: launch failed: %s", cudaGetErrorString(e));
  RL_LAUNCH_CHECK("rl_sample_temperature");
  return RL_OK;
}
