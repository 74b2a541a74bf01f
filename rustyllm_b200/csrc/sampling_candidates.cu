// Sampling from a candidate set on the device: top-k (with optional top-p and min-p
// inside it) and top-p over the whole vocabulary.  One block per row.
//
// Semantics (SimonWaldherr/RustyLLM src/sampling.rs):
//   top-k (215-306): the k largest logits, ties to the lower index (the reference
//     replaces a candidate only on a strictly greater logit), in descending order;
//     w_j = exp((l_j - l_0) / T); min-p keeps the head with w_j >= min_p * w_0 (at
//     least one); top-p keeps the head whose running sum first exceeds
//     top_p * sum(all k); one uniform r = u * kept_sum; the answer is the first
//     candidate whose running sum exceeds r, else the last kept one.  All sums run
//     in float32 over the sorted candidates, as the reference's do.
//   top-p without top-k (151-209): the reference sorts the whole vocabulary.  Here the
//     nucleus is found by a radix selection on the weights' bit patterns with exact
//     (fixed-point) bin sums: the smallest set of highest weights whose sum exceeds
//     top_p * sum(all), ties at the boundary to the lower index; min-p then drops
//     w < min_p.  The draw walks the kept tokens by descending weight like the
//     reference's, by the same selection run to the sum u * kept.  Sums are exact
//     integers (2^-40 of the top weight) where the reference adds float32 in sorted
//     order, so a uniform within float rounding of a boundary may map to the neighbour.
#include <math.h>

#include "common.cuh"

#define CAND_THREADS 1024
#define CAND_MAX_K 1024

__device__ __forceinline__ float cand_finite(float v) { return isfinite(v) ? v : -INFINITY; }
// order-preserving map from float to unsigned
__device__ __forceinline__ uint32_t ord_key(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float ord_value(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k);
}

// ------------------------------------------------------------------ top-k
__global__ void __launch_bounds__(CAND_THREADS)
sample_topk_kernel(const float* __restrict__ logits, int vocab, const int* __restrict__ rows,
                   const float* __restrict__ temperature, const float* __restrict__ uniform,
                   const float* __restrict__ min_p, const int* __restrict__ top_k,
                   const float* __restrict__ top_p, int* __restrict__ out) {
  __shared__ uint32_t hist[256];
  __shared__ uint32_t ckey[CAND_MAX_K];
  __shared__ int cidx[CAND_MAX_K];
  __shared__ int seg_eq[CAND_THREADS];
  __shared__ uint32_t s_prefix;
  __shared__ int s_remaining, s_count;
  const int row = rows[blockIdx.x];
  const float* l = logits + (size_t)row * vocab;
  const int K = min(top_k[blockIdx.x], CAND_MAX_K);
  const int tid = threadIdx.x;

  // 1. radix selection of the K-th largest key, 8 bits a pass
  if (tid == 0) { s_prefix = 0; s_remaining = K; }
  uint32_t mask = 0;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    for (int i = tid; i < vocab; i += CAND_THREADS) {
      const uint32_t key = ord_key(cand_finite(l[i]));
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      int c = 0, chosen = 0;
      for (int b = 255; b >= 0; --b) {
        if (c + (int)hist[b] >= s_remaining) { chosen = b; break; }
        c += (int)hist[b];
      }
      s_remaining -= c;
      s_prefix = prefix | ((uint32_t)chosen << shift);
    }
    mask |= 255u << shift;
    __syncthreads();
  }
  const uint32_t T = s_prefix;
  const int need_eq = s_remaining;          // >= 1: how many keys equal to T belong to the set
  const int count_gt = K - need_eq;

  // 2. gather: keys above T in any order, keys equal to T by ascending index
  if (tid == 0) s_count = 0;
  const int seg = (vocab + CAND_THREADS - 1) / CAND_THREADS;
  const int lo = tid * seg, hi = min(lo + seg, vocab);
  __syncthreads();
  int eq = 0;
  for (int i = lo; i < hi; ++i) {
    const uint32_t key = ord_key(cand_finite(l[i]));
    if (key > T) {
      const int slot = atomicAdd(&s_count, 1);
      ckey[slot] = key; cidx[slot] = i;
    } else if (key == T) {
      ++eq;
    }
  }
  seg_eq[tid] = eq;
  __syncthreads();
  if (tid == 0) {
    int c = 0;
    for (int t = 0; t < CAND_THREADS; ++t) { const int e = seg_eq[t]; seg_eq[t] = c; c += e; }
  }
  __syncthreads();
  int rank = seg_eq[tid];
  for (int i = lo; i < hi && rank < need_eq; ++i) {
    if (ord_key(cand_finite(l[i])) == T) {
      ckey[count_gt + rank] = T; cidx[count_gt + rank] = i;
      ++rank;
    }
  }
  for (int i = K + tid; i < CAND_MAX_K; i += CAND_THREADS) { ckey[i] = 0u; cidx[i] = 0x7fffffff; }
  __syncthreads();

  // 3. bitonic sort: key descending, index ascending
  for (int k = 2; k <= CAND_MAX_K; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      const int partner = tid ^ j;
      if (partner > tid) {
        const uint32_t ka = ckey[tid], kb = ckey[partner];
        const int ia = cidx[tid], ib = cidx[partner];
        const bool a_first = ka > kb || (ka == kb && ia < ib);   // a belongs before b
        const bool ascending_block = (tid & k) == 0;
        if (a_first != ascending_block) {
          ckey[tid] = kb; ckey[partner] = ka; cidx[tid] = ib; cidx[partner] = ia;
        }
      }
      __syncthreads();
    }
  }

  // 4. the reference's sequential procedure over the sorted candidates
  if (tid == 0) {
    const float v0 = ord_value(ckey[0]);
    if (!(v0 > -INFINITY)) { out[row] = 0; return; }       // nothing finite (src/sampling.rs:242-244)
    const float inv_temp = 1.0f / temperature[row];
    float* w = reinterpret_cast<float*>(ckey);             // weights overwrite the keys in place
    float sum = 0.f;
    for (int j = 0; j < K; ++j) {
      const float wj = expf((ord_value(ckey[j]) - v0) * inv_temp);
      w[j] = wj;
      sum += wj;
    }
    if (!isfinite(sum) || sum <= 0.f) { out[row] = cidx[0]; return; }
    int limit = K;
    const float mp = min_p[row];
    if (mp > 0.f) {
      const float thr = mp * w[0];
      limit = K;
      for (int j = 0; j < K; ++j) if (w[j] < thr) { limit = j; break; }
      if (limit < 1) limit = 1;
    }
    int cutoff = limit;
    float kept = 0.f;
    for (int j = 0; j < limit; ++j) kept += w[j];
    const float tp = top_p[blockIdx.x];
    if (tp < 1.0f) {
      float c = 0.f;
      const float thr = tp * sum;
      for (int j = 0; j < limit; ++j) {
        c += w[j];
        if (c > thr) { cutoff = j + 1; kept = c; break; }
      }
    }
    if (!isfinite(kept) || kept <= 0.f) { out[row] = cidx[0]; return; }
    const float r = uniform[row] * kept;
    float c = 0.f;
    int answer = cidx[cutoff - 1];
    for (int j = 0; j < cutoff; ++j) {
      c += w[j];
      if (c > r) { answer = cidx[j]; break; }
    }
    out[row] = answer;
  }
}

// ------------------------------------------------------------------ top-p over the vocabulary
#define FX_ONE 1099511627776.0f   // 2^40: fixed-point scale of a weight in [0, 1]

struct ToppShared {
  unsigned long long hsum[256];
  uint32_t hcnt[256];
  int seg_eq[CAND_THREADS];
  float red[CAND_THREADS / 32];
  unsigned long long total, above, kept;
  uint32_t prefix;
  int need_eq;
  float max;
};

// Walks the vocabulary's weights from the highest down (ties: lower index first) until their
// running sum exceeds thr, without sorting: a radix selection on the weights' bit patterns,
// 8 bits a pass, with exact fixed-point sums per bin.  Leaves in sh.prefix the weight (as
// bits) of the token at which the sum crosses thr, in sh.need_eq which of the tokens of that
// weight it is (1 = the first by index), in sh.above the sum of all greater weights.  If the
// whole sum does not exceed thr, it is the last token of the order.  All threads call it.
__device__ void topp_walk(const float* __restrict__ l, int vocab, float inv_temp, float mx,
                          unsigned long long thr, ToppShared& sh) {
  const int tid = threadIdx.x;
  if (tid == 0) { sh.prefix = 0; sh.above = 0ull; }
  uint32_t mask = 0;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    if (tid < 256) { sh.hsum[tid] = 0ull; sh.hcnt[tid] = 0u; }
    __syncthreads();
    const uint32_t prefix = sh.prefix;
    for (int i = tid; i < vocab; i += CAND_THREADS) {
      const float w = expf(cand_finite(l[i]) * inv_temp - mx);
      const uint32_t key = __float_as_uint(w);      // w >= 0: bit order is value order
      if ((key & mask) == prefix) {
        const uint32_t b = (key >> shift) & 255u;
        atomicAdd(&sh.hsum[b], (unsigned long long)(w * FX_ONE));
        atomicAdd(&sh.hcnt[b], 1u);
      }
    }
    __syncthreads();
    if (tid == 0) {
      unsigned long long above = sh.above;
      int chosen = -1, lowest = 0;
      for (int b = 255; b >= 0; --b) {
        if (sh.hcnt[b] == 0u) continue;
        lowest = b;
        if (above + sh.hsum[b] > thr) { chosen = b; break; }
        above += sh.hsum[b];
      }
      if (chosen < 0) { chosen = lowest; above -= sh.hsum[lowest]; }   // rounding: the whole order is walked
      sh.above = above;
      sh.prefix = prefix | ((uint32_t)chosen << shift);
      if (pass == 3) {
        const float wT = __uint_as_float(sh.prefix);
        const unsigned long long fxT = (unsigned long long)(wT * FX_ONE);
        long long n = (fxT == 0ull || thr < above) ? (long long)sh.hcnt[chosen] : (long long)((thr - above) / fxT) + 1;
        if (n > (long long)sh.hcnt[chosen]) n = sh.hcnt[chosen];
        if (n < 1) n = 1;
        sh.need_eq = (int)n;
      }
    }
    mask |= 255u << shift;
    __syncthreads();
  }
}

// How many tokens of weight bits T lie in front of each thread's contiguous segment of the
// vocabulary (so that "the n-th such token by index" can be told segment by segment).
__device__ int topp_rank_of_segment(const float* __restrict__ l, int lo, int hi, float inv_temp, float mx, uint32_t T,
                                    ToppShared& sh) {
  const int tid = threadIdx.x;
  int eq = 0;
  for (int i = lo; i < hi; ++i)
    if (__float_as_uint(expf(cand_finite(l[i]) * inv_temp - mx)) == T) ++eq;
  __syncthreads();
  sh.seg_eq[tid] = eq;
  __syncthreads();
  if (tid == 0) {
    int c = 0;
    for (int t = 0; t < CAND_THREADS; ++t) { const int e = sh.seg_eq[t]; sh.seg_eq[t] = c; c += e; }
  }
  __syncthreads();
  return sh.seg_eq[tid];
}

__global__ void __launch_bounds__(CAND_THREADS)
sample_topp_kernel(const float* __restrict__ logits, int vocab, const int* __restrict__ rows,
                   const float* __restrict__ temperature, const float* __restrict__ uniform,
                   const float* __restrict__ min_p, const float* __restrict__ top_p, int* __restrict__ out) {
  __shared__ ToppShared sh;
  const int row = rows[blockIdx.x];
  const float* l = logits + (size_t)row * vocab;
  const int tid = threadIdx.x;
  const float inv_temp = 1.0f / temperature[row];

  float mx = -INFINITY;
  for (int i = tid; i < vocab; i += CAND_THREADS) mx = fmaxf(mx, cand_finite(l[i]) * inv_temp);
  mx = rl_warp_max(mx);
  if ((tid & 31) == 0) sh.red[tid >> 5] = mx;
  if (tid == 0) { sh.total = 0ull; sh.kept = 0ull; }
  __syncthreads();
  if (tid == 0) {
    float t = sh.red[0];
    for (int w = 1; w < CAND_THREADS / 32; ++w) t = fmaxf(t, sh.red[w]);
    sh.max = t;
  }
  __syncthreads();
  mx = sh.max;
  if (!(mx > -INFINITY)) { if (tid == 0) out[row] = 0; return; }
  // the highest weight is exp(0) = 1, so the reference's cut `w < min_p * w_max` is `w < min_p`
  const float cut = min_p[row];

  // total weight, exactly (integer sums do not depend on the order)
  unsigned long long mine = 0ull;
  for (int i = tid; i < vocab; i += CAND_THREADS)
    mine += (unsigned long long)(expf(cand_finite(l[i]) * inv_temp - mx) * FX_ONE);
  atomicAdd(&sh.total, mine);
  __syncthreads();

  // 1. the nucleus: the head of the order whose sum first exceeds top_p * total
  topp_walk(l, vocab, inv_temp, mx, (unsigned long long)((double)top_p[blockIdx.x] * (double)sh.total), sh);
  const uint32_t T = sh.prefix;
  const int need_eq = sh.need_eq;
  const int seg = (vocab + CAND_THREADS - 1) / CAND_THREADS;
  const int lo = min(tid * seg, vocab), hi = min(lo + seg, vocab);
  {
    // its weight, exactly, without what min-p drops (tokens below the cut are its tail)
    int rank = topp_rank_of_segment(l, lo, hi, inv_temp, mx, T, sh);
    unsigned long long sum = 0ull;
    for (int i = lo; i < hi; ++i) {
      const float w = expf(cand_finite(l[i]) * inv_temp - mx);
      const uint32_t key = __float_as_uint(w);
      bool kept = key > T;
      if (key == T) { kept = rank < need_eq; ++rank; }
      if (kept && w >= cut) sum += (unsigned long long)(w * FX_ONE);
    }
    if (sum) atomicAdd(&sh.kept, sum);
  }
  __syncthreads();
  const unsigned long long kept = sh.kept;
  if (kept == 0ull) { if (tid == 0) out[row] = 0; return; }

  // 2. the draw: the reference walks the kept tokens by descending weight until the running sum
  // exceeds u * kept (src/sampling.rs:186-209) - the same walk as the nucleus's, to another sum.
  // What it crosses at lies inside the kept head, because u * kept < kept.
  unsigned long long r = (unsigned long long)((double)uniform[row] * (double)kept);
  if (r >= kept) r = kept - 1;
  topp_walk(l, vocab, inv_temp, mx, r, sh);
  const uint32_t T2 = sh.prefix;
  const int nth = sh.need_eq;
  const int rank0 = topp_rank_of_segment(l, lo, hi, inv_temp, mx, T2, sh);
  int rank = rank0;
  for (int i = lo; i < hi; ++i) {
    if (__float_as_uint(expf(cand_finite(l[i]) * inv_temp - mx)) == T2) {
      ++rank;
      if (rank == nth) { out[row] = i; break; }
    }
  }
}

// rows: [R] indices of the logits rows to sample; temperature, uniform, min_p, out are
// indexed by logits row; top_k, top_p by position in ``rows``.  A row with top_k > 0
// takes the top-k path (top_k <= 1024), else the top-p path.
extern "C" int rl_sample_candidates(const float* logits, int vocab, const int* rows_topk, const int* top_k,
                                    const float* top_p_k, int num_topk, const int* rows_topp,
                                    const float* top_p_p, int num_topp, const float* temperature,
                                    const float* uniform, const float* min_p, int* out, cudaStream_t stream) {
  RL_REQUIRE(vocab > 0 && num_topk >= 0 && num_topp >= 0, "rl_sample_candidates: bad sizes");
  if (num_topk > 0) {
    sample_topk_kernel<<<num_topk, CAND_THREADS, 0, stream>>>(logits, vocab, rows_topk, temperature, uniform,
                                                              min_p, top_k, top_p_k, out);
    RL_LAUNCH_CHECK("rl_sample_candidates (top-k)");
  }
  if (num_topp > 0) {
    sample_topp_kernel<<<num_topp, CAND_THREADS, 0, stream>>>(logits, vocab, rows_topp, temperature, uniform,
                                                              min_p, top_p_p, out);
    RL_LAUNCH_CHECK("rl_sample_candidates (top-p)");
  }
  return RL_OK;
}

extern "C" int rl_sample_max_top_k() { return CAND_MAX_K; }
