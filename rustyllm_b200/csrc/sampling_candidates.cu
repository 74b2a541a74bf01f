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
//     nucleus is found by selection on the weights' bit patterns with exact (fixed-point)
//     sums: the smallest set of highest weights whose sum exceeds top_p * sum(all), ties at
//     the boundary to the lower index; min-p then drops w < min_p.  The draw walks the kept
//     tokens by descending weight like the reference's, by the same selection run to the sum
//     u * kept.  Sums are exact integers (2^-40 of the top weight) where the reference adds
//     float32 in sorted order, so a uniform within float rounding of a boundary may map to
//     the neighbour.
//
// The selection.  Tokens are ordered by a 32-bit key (the logit's bits made order-preserving,
// or the weight's bits), descending, ties by ascending index.  A histogram of the keys' top 12
// bits (counts; for top-p also exact sums) tells which class of keys the boundary falls in
// (the k-th token, or the token at which the running sum crosses a threshold); all classes
// above it belong whole.  The boundary class is small as a rule (some hundred tokens of
// 128,256): its tokens are gathered, sorted in shared memory and the boundary is found among
// them.  A class of more than 1,024 tokens is refined by the next 12 bits, then the last 8;
// tokens that agree in all 32 bits are told apart by index.  One pass over the row a histogram.
#include <math.h>

#include "common.cuh"

#define CAND_THREADS 1024
#define CAND_MAX_K 1024
#define CAND_CAP 1024                        // tokens of a boundary class that are gathered and sorted
#define CAND_LIST (CAND_MAX_K + CAND_CAP)
#define CAND_BINS 4096

typedef unsigned long long cand_u64;

__device__ __forceinline__ float cand_finite(float v) { return isfinite(v) ? v : -INFINITY; }
// order-preserving map from float to unsigned
__device__ __forceinline__ uint32_t ord_key(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float ord_value(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k);
}
// the class of a key at a prefix of pbits bits (1 <= pbits <= 32)
__device__ __forceinline__ uint32_t cand_class(uint32_t key, int pbits) { return pbits >= 32 ? key : key >> (32 - pbits); }

// Every pass over a row goes this way: warp w takes a contiguous stretch of the row (a multiple
// of 32 tokens, so that a warp instruction reads 128 consecutive bytes), eight loads a thread
// in flight before the first is used - the row lies in L2 after its first pass, and a pass is
// bound by how many loads are on their way, not by their number.  f(i, l[i]) is called for the
// stretch's tokens.
#define CAND_UNROLL 8
__device__ __forceinline__ int cand_stretch(int vocab) { return ((vocab + 31) / 32 + 31) / 32 * 32; }
// (the tokens [first, last) of the row; first a multiple of 128)
template <typename F>
__device__ __forceinline__ void cand_scan_range(const float* __restrict__ l, int vocab, int first, int last, F&& f) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int per = cand_stretch(last - first), lo = min(first + warp * per, last), hi = min(lo + per, last);
  if ((vocab & 3) == 0 && (((uintptr_t)l) & 15) == 0) {
    // rows that 16-byte loads can fetch: four tokens a lane and load (per is a multiple of 32, so
    // lo is one of 4; order within a stretch: not ascending, which these passes do not need)
    for (int base = lo; base < hi; base += 128 * CAND_UNROLL) {
      float4 v[CAND_UNROLL];
#pragma unroll
      for (int u = 0; u < CAND_UNROLL; ++u) {
        const int i = base + 128 * u + 4 * lane;
        v[u] = i < hi ? *reinterpret_cast<const float4*>(l + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < CAND_UNROLL; ++u) {
        const int i = base + 128 * u + 4 * lane;
        if (i < hi) { f(i, v[u].x); f(i + 1, v[u].y); f(i + 2, v[u].z); f(i + 3, v[u].w); }   // hi is a multiple of 4 too
      }
    }
    return;
  }
  for (int base = lo; base < hi; base += 32 * CAND_UNROLL) {
    float v[CAND_UNROLL];
#pragma unroll
    for (int u = 0; u < CAND_UNROLL; ++u) {
      const int i = base + 32 * u + lane;
      v[u] = i < hi ? l[i] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < CAND_UNROLL; ++u) {
      const int i = base + 32 * u + lane;
      if (i < hi) f(i, v[u]);
    }
  }
}
template <typename F>
__device__ __forceinline__ void cand_scan(const float* __restrict__ l, int vocab, F&& f) { cand_scan_range(l, vocab, 0, vocab, f); }
// The same walk for passes that tell tokens apart by index: g(i, l[i], live) is called by all 32
// lanes together for every 32 consecutive tokens (live: i lies in the row), in ascending order.
template <typename G>
__device__ __forceinline__ void cand_scan_ordered(const float* __restrict__ l, int vocab, G&& g) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int per = cand_stretch(vocab), lo = min(warp * per, vocab), hi = min(lo + per, vocab);
  for (int base = lo; base < hi; base += 32 * CAND_UNROLL) {
    float v[CAND_UNROLL];
#pragma unroll
    for (int u = 0; u < CAND_UNROLL; ++u) {
      const int i = base + 32 * u + lane;
      v[u] = i < hi ? l[i] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < CAND_UNROLL; ++u) {
      const int i = base + 32 * u + lane;
      if (base + 32 * u < hi) g(i, v[u], i < hi);
    }
  }
}
// Exclusive prefix over the warps of a per-warp count (in warp order = index order of the
// stretches); `scratch`: 32 ints of shared memory.  All threads call it.
__device__ __forceinline__ int cand_warp_prefix(int warp_count, int* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = warp_count;
  __syncthreads();
  int before = 0;
  for (int w = 0; w < warp; ++w) before += scratch[w];
  __syncthreads();
  return before;
}

// What a boundary search leaves behind (shared memory).
struct CandBoundary {
  int bin;                 // the bin the boundary falls in
  uint32_t above_cnt;      // tokens in the bins above it
  cand_u64 above_sum;      // their exact sum (sums mode)
  uint32_t bin_cnt;        // tokens in the bin
  int found;
  uint32_t wcnt[32];       // scratch of the block scan
  cand_u64 wsum[32];
};

// Among `nbins` bins (4096 or 256), from the highest down: the bin in which the running count
// reaches `need` (sum == nullptr), or in which the running sum first exceeds `thr`.  In sums
// mode, if the whole sum does not exceed thr (rounding), the lowest bin that holds a token.
// All threads call it; ends with a barrier.
__device__ void cand_find_boundary(const uint32_t* cnt, const cand_u64* sum, int nbins, uint32_t need, cand_u64 thr,
                                   CandBoundary& r) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int per = nbins >= CAND_THREADS ? nbins / CAND_THREADS : 1;
  const bool active = tid * per < nbins;
  uint32_t c[4] = {0u, 0u, 0u, 0u};
  cand_u64 s[4] = {0ull, 0ull, 0ull, 0ull};
  uint32_t lc = 0u;
  cand_u64 ls = 0ull;
  if (active) {
    for (int q = 0; q < per; ++q) {
      const int b = nbins - 1 - (tid * per + q);
      c[q] = cnt[b]; lc += c[q];
      if (sum != nullptr) { s[q] = sum[b]; ls += s[q]; }
    }
  }
  // exclusive scan over the threads (= over the bins from the highest down)
  uint32_t ic = lc;
  cand_u64 is = ls;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t vc = __shfl_up_sync(0xffffffffu, ic, o);
    const cand_u64 vs = __shfl_up_sync(0xffffffffu, is, o);
    if (lane >= o) { ic += vc; is += vs; }
  }
  if (tid == 0) r.found = 0;
  if (lane == 31) { r.wcnt[warp] = ic; r.wsum[warp] = is; }
  __syncthreads();
  uint32_t bc = 0u;
  cand_u64 bs = 0ull;
  for (int w = 0; w < warp; ++w) { bc += r.wcnt[w]; bs += r.wsum[w]; }
  uint32_t ac = bc + ic - lc;           // tokens above this thread's first bin
  cand_u64 as = bs + is - ls;
  if (active) {
    for (int q = 0; q < per; ++q) {
      const bool hit = sum == nullptr ? (ac < need && need <= ac + c[q]) : (c[q] > 0u && as <= thr && thr < as + s[q]);
      if (hit) { r.bin = nbins - 1 - (tid * per + q); r.above_cnt = ac; r.above_sum = as; r.bin_cnt = c[q]; r.found = 1; }
      ac += c[q]; as += s[q];
    }
  }
  __syncthreads();
  if (sum != nullptr && !r.found && tid == 0) {
    uint32_t tc = 0u;
    cand_u64 ts = 0ull;
    for (int w = 0; w < CAND_THREADS / 32; ++w) { tc += r.wcnt[w]; ts += r.wsum[w]; }
    int b = 0;
    while (b < nbins - 1 && cnt[b] == 0u) ++b;
    r.bin = b; r.bin_cnt = cnt[b]; r.above_cnt = tc - cnt[b]; r.above_sum = ts - sum[b]; r.found = 1;
  }
  __syncthreads();
}

// one more token in bin `bin`.  With 4,096 bins the fullest holds about one token in a hundred of a
// row of logits, so plain shared-memory atomics meet seldom (with 256 bins a third of the row
// fell into one bin and its additions ran one after another: 125 us a row; finding the lanes that
// meet in a bin first, __match_any_sync, cost more than it saved: 240,000 clocks a pass).
__device__ __forceinline__ void cand_count(uint32_t* cnt, uint32_t bin) { atomicAdd(&cnt[bin], 1u); }

// Bitonic sort of list[0, n2) (n2 a power of two <= CAND_LIST): key descending, index ascending.
__device__ void cand_sort(uint32_t* lkey, int* lidx, int n2) {
  for (int k = 2; k <= n2; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int t = threadIdx.x; t < n2; t += CAND_THREADS) {
        const int partner = t ^ j;
        if (partner > t) {
          const uint32_t ka = lkey[t], kb = lkey[partner];
          const int ia = lidx[t], ib = lidx[partner];
          const bool a_first = ka > kb || (ka == kb && ia < ib);   // a belongs before b
          const bool ascending_block = (t & k) == 0;
          if (a_first != ascending_block) { lkey[t] = kb; lkey[partner] = ka; lidx[t] = ib; lidx[partner] = ia; }
        }
      }
      __syncthreads();
    }
  }
}
__device__ __forceinline__ int cand_pow2(int n) { int p = 32; while (p < n) p <<= 1; return p; }

// ------------------------------------------------------------------ top-k
struct TopkShared {
  uint32_t cnt[CAND_BINS];
  uint32_t lkey[CAND_LIST];
  int lidx[CAND_LIST];
  int seg_eq[CAND_THREADS];
  CandBoundary bd;
  uint32_t prefix;
  int pbits, count;
  uint32_t need;
};

// A row of a large vocabulary is the work of up to eight CTAs (one cluster; as many as leave every
// CTA of the launch an SM of its own): each takes its share of the row in the passes (a pass is
// bound by instruction issue: some 25 instructions a token), the first CTA adds the histograms
// through distributed shared memory, finds the boundary and tells the others; all of them append
// their tokens to the first CTA's list, which sorts and draws.  8 rows of 128,256 logits, top-k 40:
// 40 us with one CTA a row, 19 us with eight; 16 rows: 31 us with eight, 24 us with four; 64 rows:
// 42 us with one, 32 us with two, 68 us with eight (two waves).
__device__ __forceinline__ uint32_t cc_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cc_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address of `p` (in this CTA's shared memory) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t cc_map(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"((uint32_t)__cvta_generic_to_shared(p)), "r"(rank));
  return r;
}
__device__ __forceinline__ uint32_t cc_ld(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void cc_st(uint32_t addr, uint32_t v) { asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t cc_add(uint32_t addr, uint32_t v) {
  uint32_t old;
  asm volatile("atom.shared::cluster.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(addr), "r"(v) : "memory");
  return old;
}

template <int CL>      // CTAs a row: 1, or 2, 4 or 8 as one cluster
__global__ void __launch_bounds__(CAND_THREADS)
sample_topk_kernel(const float* __restrict__ logits, int vocab, const int* __restrict__ rows,
                   const float* __restrict__ temperature, const float* __restrict__ uniform,
                   const float* __restrict__ min_p, const int* __restrict__ top_k,
                   const float* __restrict__ top_p, int* __restrict__ out) {
  extern __shared__ __align__(16) uint8_t cand_smem[];
  TopkShared& sh = *reinterpret_cast<TopkShared*>(cand_smem);
  const int which = blockIdx.x / CL;
  const uint32_t crank = CL > 1 ? cc_rank() : 0u;
  const int row = rows[which];
  const float* l = logits + (size_t)row * vocab;
  const int K = min(min(top_k[which], CAND_MAX_K), vocab);
  const int tid = threadIdx.x;
  // this CTA's part of the row in the passes (whole multiples of 128 tokens)
  const int part = CL > 1 ? ((vocab + CL - 1) / CL + 127) / 128 * 128 : vocab;
  const int p_lo = min((int)crank * part, vocab), p_hi = min(p_lo + part, vocab);
  if (tid == 0) sh.count = 0;             // (the first CTA's is the list's; set before the first cluster barrier)

  // 1. the class of keys the K-th largest lies in
  uint32_t prefix = 0u, need = (uint32_t)K, class_cnt = 0u;
  int pbits = 0;
  for (int level = 0; level < 3; ++level) {
    const int nb = level < 2 ? 12 : 8, nbins = 1 << nb, shift = 32 - pbits - nb;
    for (int i = tid; i < nbins; i += CAND_THREADS) sh.cnt[i] = 0u;
    __syncthreads();
    cand_scan_range(l, vocab, p_lo, p_hi, [&](int, float v) {
      const uint32_t key = ord_key(cand_finite(v));
      if (pbits == 0 || cand_class(key, pbits) == prefix) cand_count(sh.cnt, (key >> shift) & (uint32_t)(nbins - 1));
    });
    __syncthreads();
    if (CL > 1) {
      cc_sync();                          // every CTA's histogram is complete
      if (crank == 0) {
        for (int i = tid; i < nbins; i += CAND_THREADS) {
          uint32_t v[CL];
#pragma unroll
          for (int r = 1; r < CL; ++r) v[r] = cc_ld(cc_map(&sh.cnt[i], (uint32_t)r));
          uint32_t c = sh.cnt[i];
#pragma unroll
          for (int r = 1; r < CL; ++r) c += v[r];
          sh.cnt[i] = c;
        }
        __syncthreads();
      }
    }
    if (crank == 0) cand_find_boundary(sh.cnt, nullptr, nbins, need, 0ull, sh.bd);
    uint32_t b_bin, b_above, b_cnt;
    if (CL > 1) {
      cc_sync();                          // the boundary is known; the others' histograms have been read
      b_bin = cc_ld(cc_map(&sh.bd.bin, 0u)); b_above = cc_ld(cc_map(&sh.bd.above_cnt, 0u)); b_cnt = cc_ld(cc_map(&sh.bd.bin_cnt, 0u));
    } else {
      b_bin = (uint32_t)sh.bd.bin; b_above = sh.bd.above_cnt; b_cnt = sh.bd.bin_cnt;
    }
    need -= b_above;
    prefix = (prefix << nb) | b_bin;
    pbits += nb;
    class_cnt = b_cnt;
    if (CL > 1) cc_sync(); else __syncthreads();     // everyone has read the boundary before the next level writes it
    if (class_cnt <= CAND_CAP || pbits == 32) break;
  }
  // need >= 1 tokens of the class belong to the set, all tokens of higher classes do (K - need of them)

  // 2. gather into the (first CTA's) list: higher classes whole; the boundary class whole if it is
  // small (the sort puts its best first), else - all its keys are equal - its `need` lowest indices
  const bool whole = class_cnt <= CAND_CAP;
  const int n_above = K - (int)need;
  const uint32_t a_count = CL > 1 ? cc_map(&sh.count, 0u) : 0u, a_key = CL > 1 ? cc_map(&sh.lkey[0], 0u) : 0u,
                 a_idx = CL > 1 ? cc_map(&sh.lidx[0], 0u) : 0u;
  cand_scan_range(l, vocab, p_lo, p_hi, [&](int i, float v) {
    const uint32_t key = ord_key(cand_finite(v));
    const uint32_t cls = cand_class(key, pbits);
    if (cls > prefix || (whole && cls == prefix)) {
      if (CL > 1) {
        const uint32_t slot = cc_add(a_count, 1u);
        cc_st(a_key + 4u * slot, key); cc_st(a_idx + 4u * slot, (uint32_t)i);
      } else {
        const int slot = atomicAdd(&sh.count, 1);
        sh.lkey[slot] = key; sh.lidx[slot] = i;
      }
    }
  });
  if (CL > 1) {
    cc_sync();                            // the list is complete; the other CTAs are done
    if (crank != 0) return;
  }
  const int list_n = n_above + (whole ? (int)class_cnt : (int)need);
  if (!whole) {
    // all keys of the class are equal: its `need` lowest indices (the whole row, by this CTA)
    int eq = 0;
    cand_scan(l, vocab, [&](int, float v) { if (ord_key(cand_finite(v)) == prefix) ++eq; });
    int rank = cand_warp_prefix((int)__reduce_add_sync(0xffffffffu, (unsigned)eq), sh.seg_eq);
    cand_scan_ordered(l, vocab, [&](int i, float v, bool live) {
      const bool is = live && ord_key(cand_finite(v)) == prefix;
      const unsigned m = __ballot_sync(0xffffffffu, is);
      const int mine = rank + __popc(m & ((1u << (tid & 31)) - 1u));
      if (is && mine < (int)need) { sh.lkey[n_above + mine] = prefix; sh.lidx[n_above + mine] = i; }
      rank += __popc(m);
    });
  }
  const int n2 = cand_pow2(list_n);
  __syncthreads();
  for (int i = list_n + tid; i < n2; i += CAND_THREADS) { sh.lkey[i] = 0u; sh.lidx[i] = 0x7fffffff; }
  __syncthreads();

  // 3. sort: the first K entries are the candidates in the reference's order
  cand_sort(sh.lkey, sh.lidx, n2);

  // 4. the reference's sequential procedure over the sorted candidates: the weights by all
  // threads, the sums - float, in the candidates' order, as the reference adds them - by one
  const float v0 = ord_value(sh.lkey[0]);
  float* w = reinterpret_cast<float*>(sh.lkey);            // weights overwrite the keys in place
  __syncthreads();
  if (v0 > -INFINITY) {
    const float inv_temp = 1.0f / temperature[row];
    for (int j = tid; j < K; j += CAND_THREADS) w[j] = expf((ord_value(sh.lkey[j]) - v0) * inv_temp);
  }
  __syncthreads();
  if (tid == 0) {
    const int* cidx = sh.lidx;
    if (!(v0 > -INFINITY)) { out[row] = 0; return; }       // nothing finite (src/sampling.rs:242-244)
    float sum = 0.f;
    for (int j = 0; j < K; ++j) sum += w[j];
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
    const float tp = top_p[which];
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
  uint32_t limb[4][CAND_BINS];    // a histogram's sums while it is being made: four limbs of 11 bits (see topp_add)
  uint32_t cnt[CAND_BINS];        // histogram of a deeper level
  cand_u64 sum[CAND_BINS];
  uint32_t cnt1[CAND_BINS];       // the first level's, made once and used by both walks
  cand_u64 sum1[CAND_BINS];
  uint32_t lkey[CAND_CAP];
  int lidx[CAND_CAP];
  int seg_eq[CAND_THREADS];
  float red[CAND_THREADS / 32];
  CandBoundary bd;
  cand_u64 total, above, kept;
  uint32_t prefix;
  int need_eq, count;
  int hit_idx;                    // the token a walk ended at, if its class was gathered (else -1)
  float max;
};

__device__ __forceinline__ cand_u64 cand_fx(float w) { return (cand_u64)(w * FX_ONE); }

// Exact sums of a histogram's bins without 64-bit shared-memory atomics (which took 140 of this
// kernel's 200 us): a weight's fixed-point value (at most 2^40) is added limb by limb, 11 bits
// each, into four 32-bit arrays - a limb's sum over a vocabulary of up to two million tokens
// stays below 2^32 - and the bins' 64-bit sums are put together afterwards.  Zero limbs are skipped.
__device__ __forceinline__ void topp_add(uint32_t (*limb)[CAND_BINS], uint32_t bin, cand_u64 fx) {
  const uint32_t l0 = (uint32_t)fx & 2047u, l1 = (uint32_t)(fx >> 11) & 2047u, l2 = (uint32_t)(fx >> 22) & 2047u, l3 = (uint32_t)(fx >> 33);
  if (l0) atomicAdd(&limb[0][bin], l0);
  if (l1) atomicAdd(&limb[1][bin], l1);
  if (l2) atomicAdd(&limb[2][bin], l2);
  if (l3) atomicAdd(&limb[3][bin], l3);
}
__device__ __forceinline__ void topp_clear(uint32_t (*limb)[CAND_BINS], uint32_t* cnt, int nbins) {
  for (int i = threadIdx.x; i < nbins; i += CAND_THREADS) { cnt[i] = 0u; limb[0][i] = limb[1][i] = limb[2][i] = limb[3][i] = 0u; }
}
__device__ __forceinline__ void topp_sums(uint32_t (*limb)[CAND_BINS], cand_u64* sum, int nbins) {
  for (int i = threadIdx.x; i < nbins; i += CAND_THREADS)
    sum[i] = (cand_u64)limb[0][i] + ((cand_u64)limb[1][i] << 11) + ((cand_u64)limb[2][i] << 22) + ((cand_u64)limb[3][i] << 33);
}

// The first level's histogram of the row's weights: counts and exact sums by the top 12 bits.
__device__ void topp_level1(const float* __restrict__ l, int vocab, float inv_temp, float mx, ToppShared& sh) {
  topp_clear(sh.limb, sh.cnt1, CAND_BINS);
  __syncthreads();
  cand_scan(l, vocab, [&](int, float v) {
    const float w = expf(cand_finite(v) * inv_temp - mx);
    const uint32_t bin = __float_as_uint(w) >> 20;     // w >= 0: bit order is value order
    cand_count(sh.cnt1, bin);
    topp_add(sh.limb, bin, cand_fx(w));
  });
  __syncthreads();
  topp_sums(sh.limb, sh.sum1, CAND_BINS);
  __syncthreads();
}

// Walks the vocabulary's weights from the highest down (ties: lower index first) until their
// running sum exceeds thr, without sorting the vocabulary (see the head of the file).  Leaves in
// sh.prefix the weight (as bits) of the token at which the sum crosses thr, in sh.need_eq which
// of the tokens of that weight it is (1 = the first by index), in sh.above the sum of all
// greater weights.  If the whole sum does not exceed thr, it is the last token of the order.
// All threads call it; needs topp_level1 before.
__device__ void topp_walk(const float* __restrict__ l, int vocab, float inv_temp, float mx, cand_u64 thr, ToppShared& sh) {
  const int tid = threadIdx.x;
  cand_find_boundary(sh.cnt1, sh.sum1, CAND_BINS, 0u, thr, sh.bd);
  uint32_t prefix = (uint32_t)sh.bd.bin, class_cnt = sh.bd.bin_cnt;
  int pbits = 12;
  cand_u64 above = sh.bd.above_sum;
  __syncthreads();
  while (class_cnt > CAND_CAP && pbits < 32) {
    const int nb = pbits < 24 ? 12 : 8, nbins = 1 << nb, shift = 32 - pbits - nb;
    topp_clear(sh.limb, sh.cnt, nbins);
    __syncthreads();
    cand_scan(l, vocab, [&](int, float v) {
      const float w = expf(cand_finite(v) * inv_temp - mx);
      const uint32_t key = __float_as_uint(w);
      if (cand_class(key, pbits) == prefix) {
        const uint32_t bin = (key >> shift) & (uint32_t)(nbins - 1);
        cand_count(sh.cnt, bin);
        topp_add(sh.limb, bin, cand_fx(w));
      }
    });
    __syncthreads();
    topp_sums(sh.limb, sh.sum, nbins);
    __syncthreads();
    // what is left of the threshold inside this class; beyond its whole sum: the class's last token
    cand_find_boundary(sh.cnt, sh.sum, nbins, 0u, thr >= above ? thr - above : 0ull, sh.bd);
    above += sh.bd.above_sum;
    prefix = (prefix << nb) | (uint32_t)sh.bd.bin;
    pbits += nb;
    class_cnt = sh.bd.bin_cnt;
    __syncthreads();
  }
  if (class_cnt > CAND_CAP) {
    // more than 1,024 tokens of one and the same weight: the crossing is a matter of counting
    if (tid == 0) {
      const cand_u64 fxT = cand_fx(__uint_as_float(prefix));
      long long n = (fxT == 0ull || thr < above) ? (long long)class_cnt : (long long)((thr - above) / fxT) + 1;
      if (n > (long long)class_cnt) n = class_cnt;
      if (n < 1) n = 1;
      sh.prefix = prefix; sh.need_eq = (int)n; sh.above = above; sh.hit_idx = -1;
    }
    __syncthreads();
    return;
  }
  // the class's tokens, sorted; one thread walks them
  if (tid == 0) sh.count = 0;
  __syncthreads();
  cand_scan(l, vocab, [&](int i, float v) {
    const uint32_t key = __float_as_uint(expf(cand_finite(v) * inv_temp - mx));
    if (cand_class(key, pbits) == prefix) {
      const int slot = atomicAdd(&sh.count, 1);
      sh.lkey[slot] = key; sh.lidx[slot] = i;
    }
  });
  const int n2 = cand_pow2((int)class_cnt);
  __syncthreads();
  for (int i = (int)class_cnt + tid; i < n2; i += CAND_THREADS) { sh.lkey[i] = 0u; sh.lidx[i] = 0x7fffffff; }
  __syncthreads();
  cand_sort(sh.lkey, sh.lidx, n2);
  if (tid == 0) {
    cand_u64 run = above, gt = above;     // gt: the sum of everything greater than the current key
    uint32_t cur = sh.lkey[0];
    int eq = 0, at = (int)class_cnt - 1;    // never crossed: the last token of the class, which is the last of the order then
    for (int j = 0; j < (int)class_cnt; ++j) {
      const uint32_t key = sh.lkey[j];
      if (key != cur) { cur = key; eq = 0; gt = run; }
      ++eq;
      run += cand_fx(__uint_as_float(key));
      if (run > thr) { at = j; break; }
    }
    sh.prefix = cur; sh.need_eq = eq; sh.above = gt; sh.hit_idx = sh.lidx[at];
  }
  __syncthreads();
}

// How many tokens of weight bits T lie in front of this warp's stretch of the row (so that "the
// n-th such token by index" can be told stretch by stretch).  All threads call it.
__device__ int topp_rank_before(const float* __restrict__ l, int vocab, float inv_temp, float mx, uint32_t T, ToppShared& sh) {
  int eq = 0;
  cand_scan(l, vocab, [&](int, float v) {
    if (__float_as_uint(expf(cand_finite(v) * inv_temp - mx)) == T) ++eq;
  });
  return cand_warp_prefix((int)__reduce_add_sync(0xffffffffu, (unsigned)eq), sh.seg_eq);
}

__global__ void __launch_bounds__(CAND_THREADS)
sample_topp_kernel(const float* __restrict__ logits, int vocab, const int* __restrict__ rows,
                   const float* __restrict__ temperature, const float* __restrict__ uniform,
                   const float* __restrict__ min_p, const float* __restrict__ top_p, int* __restrict__ out) {
  extern __shared__ __align__(16) uint8_t cand_smem[];
  ToppShared& sh = *reinterpret_cast<ToppShared*>(cand_smem);
  const int row = rows[blockIdx.x];
  const float* l = logits + (size_t)row * vocab;
  const int tid = threadIdx.x;
  const float inv_temp = 1.0f / temperature[row];

  float mx = -INFINITY;
  cand_scan(l, vocab, [&](int, float v) { mx = fmaxf(mx, cand_finite(v) * inv_temp); });
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

  // the first level's histogram; the total weight is the sum of its bins, exactly (integer sums
  // do not depend on the order)
  topp_level1(l, vocab, inv_temp, mx, sh);
  {
    cand_u64 mine = 0ull;
    for (int i = tid; i < CAND_BINS; i += CAND_THREADS) mine += sh.sum1[i];
    if (mine) atomicAdd(&sh.total, mine);
  }
  __syncthreads();

  // 1. the nucleus: the head of the order whose sum first exceeds top_p * total
  topp_walk(l, vocab, inv_temp, mx, (cand_u64)((double)top_p[blockIdx.x] * (double)sh.total), sh);
  const uint32_t T = sh.prefix;
  const int need_eq = sh.need_eq;
  const unsigned below = (1u << (tid & 31)) - 1u;       // the lanes in front of this one
  if (cut <= __uint_as_float(T)) {
    // min-p drops nothing of it: everything above T and need_eq tokens of T, exactly
    if (tid == 0) sh.kept = sh.above + (cand_u64)need_eq * cand_fx(__uint_as_float(T));
  } else {
    // its weight without what min-p drops (tokens below the cut are its tail)
    int rank = topp_rank_before(l, vocab, inv_temp, mx, T, sh);
    cand_u64 sum = 0ull;
    cand_scan_ordered(l, vocab, [&](int, float v, bool live) {
      const float w = expf(cand_finite(v) * inv_temp - mx);
      const uint32_t key = __float_as_uint(w);
      const bool is = live && key == T;
      const unsigned m = __ballot_sync(0xffffffffu, is);
      const bool kept = live && (key > T || (is && rank + __popc(m & below) < need_eq));
      rank += __popc(m);
      if (kept && w >= cut) sum += cand_fx(w);
    });
    if (sum) atomicAdd(&sh.kept, sum);
  }
  __syncthreads();
  const cand_u64 kept = sh.kept;
  if (kept == 0ull) { if (tid == 0) out[row] = 0; return; }

  // 2. the draw: the reference walks the kept tokens by descending weight until the running sum
  // exceeds u * kept (src/sampling.rs:186-209) - the same walk as the nucleus's, to another sum.
  // What it crosses at lies inside the kept head, because u * kept < kept.
  cand_u64 r = (cand_u64)((double)uniform[row] * (double)kept);
  if (r >= kept) r = kept - 1;
  topp_walk(l, vocab, inv_temp, mx, r, sh);
  const uint32_t T2 = sh.prefix;
  const int nth = sh.need_eq;
  if (sh.hit_idx >= 0) {                  // the walk ended at a token of a gathered class: that one
    if (tid == 0) out[row] = sh.hit_idx;
    return;
  }
  int rank = topp_rank_before(l, vocab, inv_temp, mx, T2, sh);
  cand_scan_ordered(l, vocab, [&](int i, float v, bool live) {
    const bool is = live && __float_as_uint(expf(cand_finite(v) * inv_temp - mx)) == T2;
    const unsigned m = __ballot_sync(0xffffffffu, is);
    if (is && rank + __popc(m & below) + 1 == nth) out[row] = i;
    rank += __popc(m);
  });
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
    static bool configured_k = false;
    if (!configured_k) {
      cudaError_t e = cudaFuncSetAttribute(sample_topk_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(TopkShared));
      if (e == cudaSuccess) e = cudaFuncSetAttribute(sample_topk_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(TopkShared));
      if (e == cudaSuccess) e = cudaFuncSetAttribute(sample_topk_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(TopkShared));
      if (e == cudaSuccess) e = cudaFuncSetAttribute(sample_topk_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(TopkShared));
      RL_REQUIRE(e == cudaSuccess, "rl_sample_candidates: cannot reserve %d bytes of shared memory: %s", (int)sizeof(TopkShared), cudaGetErrorString(e));
      configured_k = true;
    }
    // CTAs a row: the most that leave each CTA of the launch an SM of its own (clusters of eight
    // only while they fill no more than half of the SMs: sixteen of them no longer find room at once)
    const int sms = rl_num_sms();
    const int cl = vocab < 16384 ? 1 : num_topk * 16 <= sms ? 8 : num_topk * 4 <= sms ? 4 : num_topk * 2 <= sms ? 2 : 1;
    if (cl > 1) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(cl * num_topk);
      cfg.blockDim = dim3(CAND_THREADS);
      cfg.dynamicSmemBytes = sizeof(TopkShared);
      cfg.stream = stream;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = cl; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      cudaError_t e = cl == 8 ? cudaLaunchKernelEx(&cfg, sample_topk_kernel<8>, logits, vocab, rows_topk, temperature, uniform, min_p, top_k, top_p_k, out)
                    : cl == 4 ? cudaLaunchKernelEx(&cfg, sample_topk_kernel<4>, logits, vocab, rows_topk, temperature, uniform, min_p, top_k, top_p_k, out)
                              : cudaLaunchKernelEx(&cfg, sample_topk_kernel<2>, logits, vocab, rows_topk, temperature, uniform, min_p, top_k, top_p_k, out);
      RL_REQUIRE(e == cudaSuccess, "rl_sample_candidates (top-k): launch failed: %s", cudaGetErrorString(e));
    } else {
      sample_topk_kernel<1><<<num_topk, CAND_THREADS, sizeof(TopkShared), stream>>>(logits, vocab, rows_topk, temperature, uniform,
                                                                                    min_p, top_k, top_p_k, out);
    }
    RL_LAUNCH_CHECK("rl_sample_candidates (top-k)");
  }
  if (num_topp > 0) {
    static bool configured_p = false;
    if (!configured_p) {
      cudaError_t e = cudaFuncSetAttribute(sample_topp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(ToppShared));
      RL_REQUIRE(e == cudaSuccess, "rl_sample_candidates: cannot reserve %d bytes of shared memory: %s", (int)sizeof(ToppShared), cudaGetErrorString(e));
      configured_p = true;
    }
    sample_topp_kernel<<<num_topp, CAND_THREADS, sizeof(ToppShared), stream>>>(logits, vocab, rows_topp, temperature, uniform,
                                                                               min_p, top_p_p, out);
    RL_LAUNCH_CHECK("rl_sample_candidates (top-p)");
  }
  return RL_OK;
}

extern "C" int rl_sample_max_top_k() { return CAND_MAX_K; }
