// Prefill attention on the 5th-generation tensor cores (tcgen05), head sizes 64 and 128.
//
// Same math and the same packed, paged inputs as attention_prefill.cu (which stays the
// kernel for head size 64 and is the restatement this one is tested against): causal
// grouped-query attention of the step's query tokens over their sequence's cached keys
// and values, streaming softmax in float (SimonWaldherr/RustyLLM src/model.rs:7239-7294, 5807-5869).
//
// One CTA = 128 consecutive query tokens of one sequence and one query head.
//   S = Q K^T   tcgen05.mma 128 x 128 x 128, Q and the key tile in shared memory (TMA,
//               128-byte swizzle, K-major like the matrix products), S in tensor memory
//               (two buffers: the next tile's scores are computed while this tile's
//               are being exponentiated)
//   softmax     eight warps, two threads a query row (= one lane of tensor memory; two
//               warps may read the same lanes), 64 keys each: no shuffles, the two exchange
//               their maxima through shared memory once a tile; running maximum kept lazily - the accumulator is only rescaled
//               when the maximum has grown by more than 2^8, so most tiles skip the
//               read-modify-write of O in tensor memory; P is written as bf16 over the
//               first 64 columns of the S buffer it came from (tcgen05.st): it never
//               touches shared memory
//   O += P V    tcgen05.mma with P in tensor memory as A and the value tile as an
//               MN-major B operand (values are stored [position][head_dim]); O stays in
//               tensor memory over all key tiles.  The products of one thread run in the
//               order they were issued, so the S of tile i + 2, which overwrites P of
//               tile i, needs no barrier of its own
// A key tile is two cache pages (128 positions).  Warp 0 feeds TMA, warp 1 issues MMAs,
// warps 2-9 do the softmax and the final normalisation.  Every mbarrier wait is bounded; a
// softmax warp whose wait ran out stops working but keeps arriving at the softmax warps'
// own barrier until the loop ends, so that nobody waits there for ever.
//
// Rows of a page beyond the sequence's length are never selected (their probabilities
// are exactly 0), but they are multiplied: the cache pools must not hold NaN or Inf
// there (the cache zero-fills its pools when it allocates them; stale finite values of
// earlier sequences contribute exactly nothing).
#include <cuda.h>
#include <math.h>

#include "common.cuh"

namespace {

constexpr int TQ = 128;          // query rows per CTA
constexpr int TK = 128;          // keys per tile = two pages
constexpr int FA_THREADS = 320;       // warp 0: TMA, warp 1: MMA, warps 2-9: softmax
constexpr uint32_t FA_WAIT_LIMIT = 1u << 22;
constexpr int KV_STAGES = 2;
constexpr int HALF_BYTES = 128 * 64 * 2;               // [128 rows x 64 bf16], 16 KB
// sizes that depend on the head size HD (64 or 128): a head is HD / 64 halves of 64 dimensions
template <int HD> struct FaSizes {
  static constexpr int HALVES = HD / 64;
  static constexpr int Q_BYTES = HALVES * HALF_BYTES;          // 16 or 32 KB
  static constexpr int KV_STAGE_BYTES = 2 * HALVES * HALF_BYTES;  // K halves, then V halves: 32 or 64 KB
  // + alignment slack, barriers, and the softmax threads' exchange: row maxima (two tiles in turn) and row sums
  static constexpr int SMEM = Q_BYTES + KV_STAGES * KV_STAGE_BYTES + 1024 + 256 + 3 * 2 * TQ * 4;
};
constexpr float LAZY_LOG2 = 8.0f;                      // rescale O only when the maximum grew by more than 2^8

__device__ __forceinline__ uint32_t fa_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void fa_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fa_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void fa_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t fa_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok;
}
__device__ __forceinline__ bool fa_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < FA_WAIT_LIMIT; ++i) {
    if (fa_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  return false;
}
__device__ __forceinline__ void fa_tma_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void fa_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fa_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fa_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// the same with the A operand in tensor memory (rows = lanes, two bf16 a column)
__device__ __forceinline__ void fa_mma_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void fa_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void fa_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void fa_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void fa_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ float fa_exp2(float x) {       // one MUFU; 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// two floats an instruction (packed fp32 of sm_100) and a maximum of three
__device__ __forceinline__ float2 fa_ffma2(float2 a, float2 b, float2 c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d)
      : "l"(*reinterpret_cast<uint64_t*>(&a)), "l"(*reinterpret_cast<uint64_t*>(&b)), "l"(*reinterpret_cast<uint64_t*>(&c)));
  return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 fa_fadd2(float2 a, float2 b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(*reinterpret_cast<uint64_t*>(&a)), "l"(*reinterpret_cast<uint64_t*>(&b)));
  return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float fa_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// the 256 softmax threads among themselves (barrier 1; barrier 0 is __syncthreads)
__device__ __forceinline__ void fa_softmax_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ void fa_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fa_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// K-major operand: rows of 128 bytes, 128-byte swizzle, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t fa_desc_kmajor(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
// MN-major operand (the value tile as B: N = head dimension contiguous, K = positions):
// 64 N-elements (128 bytes) contiguous and swizzled, the next 64 N-elements `lbo` bytes
// further (leading byte offset), groups of 8 K-rows 1024 bytes apart (stride byte offset).
__device__ __forceinline__ uint64_t fa_desc_mnmajor(uint32_t addr, uint32_t lbo) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// kind::f16, float accumulator, bf16 A and B, A K-major, B K-major (b_mn = 0) or MN-major (1)
__host__ __device__ constexpr uint32_t fa_idesc(int m, int n, int b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

template <int HD>
__global__ void __launch_bounds__(FA_THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const int* __restrict__ page_table, int max_pages,
                            const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slots,
                            const int* __restrict__ kv_lens, int num_seqs, __nv_bfloat16* __restrict__ out, int ldo,
                            int H, int G, float scale_log2e, int window, int* __restrict__ err) {
  extern __shared__ uint8_t fa_smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)fa_smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* q_tile = smem;                                   // [2 halves][128 x 64]
  constexpr int HALVES = FaSizes<HD>::HALVES, Q_BYTES = FaSizes<HD>::Q_BYTES, KV_STAGE_BYTES = FaSizes<HD>::KV_STAGE_BYTES;
  uint8_t* kv_ring = smem + Q_BYTES;                        // [stage][K halves, V halves]
  uint64_t* bars = (uint64_t*)(kv_ring + KV_STAGES * KV_STAGE_BYTES);
  uint64_t* q_full = bars;                 // 1
  uint64_t* k_full = bars + 1;             // [KV_STAGES] each: keys and values of a stage are
  uint64_t* k_empty = k_full + KV_STAGES;  //   loaded and given back separately (the keys of a
  uint64_t* v_full = k_empty + KV_STAGES;  //   tile are done with one product earlier than its
  uint64_t* v_empty = v_full + KV_STAGES;  //   values, and wanted one product earlier)
  uint64_t* s_full = v_empty + KV_STAGES;  // [2]
  uint64_t* p_full = s_full + 2;           // 1
  uint64_t* p_empty = p_full + 1;          // 1
  uint64_t* o_full = p_empty + 1;          // 1
  uint32_t* tmem_slot = (uint32_t*)(o_full + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  int* s_seq = (int*)(tmem_slot + 2);
  int* s_tile = (int*)(tmem_slot + 3);
  float* x_max = (float*)((uint8_t*)bars + 256);            // [tile parity][key half][row]
  float* x_sum = x_max + 2 * 2 * TQ;                         // [key half][row]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  rl_pdl_trigger();
  if (threadIdx.x == 0) {
    fa_mbar_init(fa_smem_u32(q_full), 1);
    for (int i = 0; i < KV_STAGES; ++i) {
      fa_mbar_init(fa_smem_u32(&k_full[i]), 1); fa_mbar_init(fa_smem_u32(&k_empty[i]), 1);
      fa_mbar_init(fa_smem_u32(&v_full[i]), 1); fa_mbar_init(fa_smem_u32(&v_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) fa_mbar_init(fa_smem_u32(&s_full[i]), 1);
    fa_mbar_init(fa_smem_u32(p_full), 8);
    fa_mbar_init(fa_smem_u32(p_empty), 1);
    fa_mbar_init(fa_smem_u32(o_full), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(fa_smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  rl_pdl_wait();       // everything below reads what earlier kernels of the step wrote
  // ---- which sequence and which of its 128-row query tiles (heaviest first) ----
  if (threadIdx.x == 32) {
    int t = (int)(gridDim.x - 1 - blockIdx.x), b = 0;
    for (; b < num_seqs; ++b) {
      const int tiles = (cu_seqlens[b + 1] - cu_seqlens[b] + TQ - 1) / TQ;
      if (t < tiles) break;
      t -= tiles;
    }
    *s_seq = b; *s_tile = t;
  }
  fa_fence_before();
  __syncthreads();
  fa_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s0 = tmem_base, tmem_o = tmem_base + 256;      // S buffers at columns 0 and 128, O at 256
  const int b = *s_seq;
  const bool have_work = b < num_seqs;      // the grid is sized exactly; defensive
  const int h = blockIdx.y, gkv = h / (H / G);
  int row0 = 0, q_len = 0, kv_len = 0, qt0 = 0, rows_here = 0, kt_begin = 0, kt_end = 0, start_pos = 0;
  const int* pages = page_table;
  if (have_work) {
    row0 = cu_seqlens[b]; q_len = cu_seqlens[b + 1] - row0; kv_len = kv_lens[b];
    start_pos = kv_len - q_len;
    qt0 = *s_tile * TQ;
    rows_here = min(TQ, q_len - qt0);
    pages = page_table + (size_t)seq_slots[b] * max_pages;
    const int last_pos = start_pos + qt0 + rows_here - 1;
    const int first_key = window > 0 ? max(0, start_pos + qt0 + 1 - window) : 0;
    kt_begin = first_key / TK; kt_end = last_pos / TK + 1;
  }
  const int num_kt = kt_end - kt_begin;

  if (warp == 0) {
    if (lane == 0 && have_work) {
      // ---------------- TMA producer ----------------
      fa_expect_tx(fa_smem_u32(q_full), Q_BYTES);
#pragma unroll
      for (int half = 0; half < HALVES; ++half)
        fa_tma_2d(fa_smem_u32(q_tile + half * HALF_BYTES), &map_q, fa_smem_u32(q_full), h * HD + 64 * half, row0 + qt0);
      // keys of tile i + 1 are asked for before the values of tile i: the keys' stage is free as
      // soon as S of two tiles back is done, the values' only when that tile's P V is
      auto load = [&](int i, bool values) -> bool {
        const int kt = kt_begin + i, st = i % KV_STAGES;
        const uint32_t phase = (i / KV_STAGES) & 1;
        uint64_t* empty = values ? v_empty : k_empty;
        if (i >= KV_STAGES && !fa_wait(fa_smem_u32(&empty[st]), phase ^ 1, abort_flag)) {
          if (!*abort_flag) { *abort_flag = 1; atomicExch(err, 11); }
          return false;
        }
        const int p0 = pages[2 * kt];
        const int p1 = (2 * kt + 1) * RL_PAGE < kv_len ? pages[2 * kt + 1] : p0;   // beyond the sequence: any valid page (all masked)
        const int r0 = (p0 * G + gkv) * RL_PAGE, r1 = (p1 * G + gkv) * RL_PAGE;
        const uint32_t fb = fa_smem_u32(values ? &v_full[st] : &k_full[st]);
        uint8_t* base = kv_ring + (size_t)st * KV_STAGE_BYTES + (values ? HALVES * HALF_BYTES : 0);
        const CUtensorMap* map = values ? &map_v : &map_k;
        fa_expect_tx(fb, HALVES * HALF_BYTES);
#pragma unroll
        for (int half = 0; half < HALVES; ++half) {     // 64 head dimensions a half; 64 positions a page
          fa_tma_2d(fa_smem_u32(base + half * HALF_BYTES), map, fb, 64 * half, r0);
          fa_tma_2d(fa_smem_u32(base + half * HALF_BYTES + 64 * 128), map, fb, 64 * half, r1);
        }
        return true;
      };
      bool ok = num_kt == 0 || load(0, false);
      for (int i = 0; i < num_kt && ok; ++i) {
        if (i + 1 < num_kt) ok = load(i + 1, false);
        if (ok) ok = load(i, true);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && have_work) {
      // ---------------- MMA issuer ----------------
      constexpr uint32_t idesc_s = fa_idesc(TQ, TK, 0);     // S = Q K^T : both K-major
      constexpr uint32_t idesc_o = fa_idesc(TQ, HD, 1);     // O += P V  : V is MN-major
      bool ok = fa_wait(fa_smem_u32(q_full), 0, abort_flag);
      if (!ok && !*abort_flag) { *abort_flag = 1; atomicExch(err, 12); }
      auto issue_s = [&](int i) -> bool {                   // scores of tile i into S buffer i % 2
        const int st = i % KV_STAGES, sb = i & 1;
        if (!fa_wait(fa_smem_u32(&k_full[st]), (i / KV_STAGES) & 1, abort_flag)) return false;
        // S buffer sb still holds P of tile i - 2; that tile's P V was issued before this and
        // products run in the order of their issue
        fa_fence_after();
        uint8_t* base = kv_ring + (size_t)st * KV_STAGE_BYTES;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint64_t da = fa_desc_kmajor(fa_smem_u32(q_tile + (k / 4) * HALF_BYTES)) + 2 * (k % 4);
          const uint64_t db = fa_desc_kmajor(fa_smem_u32(base + (k / 4) * HALF_BYTES)) + 2 * (k % 4);
          fa_mma(tmem_s0 + (uint32_t)(sb * TK), da, db, idesc_s, k > 0 ? 1u : 0u);
        }
        fa_commit(fa_smem_u32(&s_full[sb]));
        fa_commit(fa_smem_u32(&k_empty[st]));               // the keys' half of the stage is free once S is done
        return true;
      };
      if (ok && num_kt > 0) ok = issue_s(0);
      for (int i = 0; i < num_kt && ok; ++i) {
        if (i + 1 < num_kt) ok = issue_s(i + 1);            // next tile's scores while this tile's softmax runs
        if (!ok) break;
        if (!fa_wait(fa_smem_u32(&v_full[i % KV_STAGES]), (i / KV_STAGES) & 1, abort_flag)) { ok = false; break; }
        if (!fa_wait(fa_smem_u32(p_full), i & 1, abort_flag)) { ok = false; break; }
        fa_fence_after();
        uint8_t* vbase = kv_ring + (size_t)(i % KV_STAGES) * KV_STAGE_BYTES + HALVES * HALF_BYTES;
#pragma unroll
        for (int k = 0; k < TK / 16; ++k) {                 // 16 positions a step
          // P of this tile: 16 keys = 8 columns of packed bf16 pairs a step, in its S buffer
          const uint64_t db = fa_desc_mnmajor(fa_smem_u32(vbase + k * 16 * 128), HALF_BYTES);
          fa_mma_a_tmem(tmem_o, tmem_s0 + (uint32_t)((i & 1) * TK + 8 * k), db, idesc_o, (i > 0 || k > 0) ? 1u : 0u);
        }
        fa_commit(fa_smem_u32(p_empty));                    // P and O are free again once these have completed
        fa_commit(fa_smem_u32(&v_empty[i % KV_STAGES]));
      }
      if (ok) fa_commit(fa_smem_u32(o_full));
      else if (!*abort_flag) { *abort_flag = 1; atomicExch(err, 13); }
    }
  } else if (have_work) {
    // ---------------- softmax warps: two threads a query row, 64 keys each ----------------
    constexpr int HK = TK / 2;                              // keys a thread
    constexpr int OC = HD / 2;                              // output columns a thread
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;                      // row of the tile = lane of tensor memory
    const int pos = start_pos + qt0 + r;                    // position of this row's query
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    float m_used = -INFINITY, l_run = 0.f;                  // maximum the probabilities are scaled by; running sum (own keys)
    bool ok = true;                                         // warp-uniform
    for (int i = 0; i < num_kt; ++i) {
      const int sb = i & 1, key0 = (kt_begin + i) * TK + half * HK;
      if (ok) ok = __all_sync(0xffffffffu, fa_wait(fa_smem_u32(&s_full[sb]), (i >> 1) & 1, abort_flag));
      uint32_t sv[HK];
      float mx_own = -INFINITY;
      if (ok) {
        fa_fence_after();
        const uint32_t s_addr = tmem_s0 + lane_addr + (uint32_t)(sb * TK + half * HK);
        // the thread's 64 scores into registers with one wait; everything below is straight-line
        // code over them, so the scheduler has independent work to cover every latency
#pragma unroll
        for (int c = 0; c < HK / 32; ++c) fa_ld32(s_addr + c * 32, sv + c * 32);
        fa_wait_ld();
        const bool need_mask = (kt_begin + i) * TK + TK - 1 > start_pos + qt0 || window > 0;
        if (need_mask) {
#pragma unroll
          for (int j = 0; j < HK; ++j) {
            const int key = key0 + j;
            const bool vis = key <= pos && (window <= 0 || key > pos - window);
            if (!vis) sv[j] = 0xff800000u;        // -inf
          }
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < HK; j += 2) mx4[(j >> 1) & 3] = fa_max3(mx4[(j >> 1) & 3], __uint_as_float(sv[j]), __uint_as_float(sv[j + 1]));
        mx_own = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      }
      // the row's maximum: the two threads of a row exchange theirs (buffers take turns, so one
      // barrier a tile is enough)
      x_max[(sb * 2 + half) * TQ + r] = mx_own;
      fa_softmax_sync();
      if (!ok) continue;
      const float mx = fmaxf(mx_own, x_max[(sb * 2 + (half ^ 1)) * TQ + r]) * scale_log2e;
      // lazy maximum: move it (and rescale O and the sum) only when it grew by more than 2^8
      float corr = 1.0f;
      if (mx > m_used + LAZY_LOG2 || (m_used == -INFINITY && mx > -INFINITY)) {
        corr = fa_exp2(m_used - mx);                          // 0 on the first visible tile
        m_used = mx;
      }
      const bool any_rescale = __any_sync(0xffffffffu, corr != 1.0f);
      // probabilities: exp2(score * scale - maximum), two scores an FMA; summed in float, rounded
      // to bf16 for the product with V and packed in place (sv[0..31] then hold the thread's 64)
      const float m_sub = m_used == -INFINITY ? 0.f : m_used;
      const float2 sc2 = make_float2(scale_log2e, scale_log2e), nm2 = make_float2(-m_sub, -m_sub);
      float2 sum2[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
#pragma unroll
      for (int j = 0; j < HK; j += 2) {
        const float2 t = fa_ffma2(make_float2(__uint_as_float(sv[j]), __uint_as_float(sv[j + 1])), sc2, nm2);
        const float2 p2 = make_float2(fa_exp2(t.x), fa_exp2(t.y));
        sum2[(j >> 1) & 3] = fa_fadd2(sum2[(j >> 1) & 3], p2);
        __nv_bfloat162 pb = __floats2bfloat162_rn(p2.x, p2.y);
        sv[j >> 1] = *reinterpret_cast<uint32_t*>(&pb);
      }
      const float2 s01 = fa_fadd2(sum2[0], sum2[1]), s23 = fa_fadd2(sum2[2], sum2[3]);
      const float sum = (s01.x + s01.y) + (s23.x + s23.y);
      // O is only touched once the previous tile's P V has completed: waited for only if this
      // warp has a row to rescale (the barrier cannot have run ahead: the next P V needs our arrival)
      if (any_rescale && i > 0) {
        ok = __all_sync(0xffffffffu, fa_wait(fa_smem_u32(p_empty), (i - 1) & 1, abort_flag));
        if (!ok) continue;
        fa_fence_after();
        l_run *= corr;
#pragma unroll 1
        for (int c = 0; c < OC / 32; ++c) {               // this thread's half of the row of O
          uint32_t v[32];
          const uint32_t o_addr = tmem_o + lane_addr + (uint32_t)(half * OC + c * 32);
          fa_ld32(o_addr, v);
          fa_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * corr);
          fa_st16(o_addr, *reinterpret_cast<uint32_t(*)[16]>(v));
          fa_st16(o_addr + 16, *reinterpret_cast<uint32_t(*)[16]>(v + 16));
        }
      }
      // P over the S buffer: this thread's 64 keys are columns 32 half .. 32 half + 31 (both threads of
      // the row had their scores in registers before the barrier above)
      {
        const uint32_t p_addr = tmem_s0 + lane_addr + (uint32_t)(sb * TK + half * (HK / 2));
        fa_st16(p_addr, *reinterpret_cast<uint32_t(*)[16]>(sv));
        fa_st16(p_addr + 16, *reinterpret_cast<uint32_t(*)[16]>(sv + 16));
        fa_wait_st();
      }
      l_run += sum;
      // P is ready for the tensor cores
      fa_fence_before();
      __syncwarp();
      if (lane == 0) fa_arrive(fa_smem_u32(p_full));
    }
    // ---- O / l -> out ----
    if (ok) ok = __all_sync(0xffffffffu, fa_wait(fa_smem_u32(o_full), 0, abort_flag));
    if (!ok && !*abort_flag) { *abort_flag = 1; atomicExch(err, 14); }
    x_sum[half * TQ + r] = l_run;
    fa_softmax_sync();
    fa_fence_after();
    if (ok) {
      const float l_row = half == 0 ? l_run + x_sum[TQ + r] : x_sum[r] + l_run;    // keys 0-63 first, either way
      const float inv = l_row > 0.f ? 1.0f / l_row : 0.f;
      __nv_bfloat16* orow = out + (size_t)(row0 + qt0 + r) * ldo + (size_t)h * HD + half * OC;
#pragma unroll 1
      for (int c = 0; c < OC / 16; ++c) {
        uint32_t v[16];
        fa_ld16(tmem_o + lane_addr + (uint32_t)(half * OC + c * 16), v);
        fa_wait_ld();
        if (r < rows_here) {
          uint32_t pk[8];
#pragma unroll
          for (int j = 0; j < 16; j += 2) {
            __nv_bfloat162 o2 = __floats2bfloat162_rn(__uint_as_float(v[j]) * inv, __uint_as_float(v[j + 1]) * inv);
            pk[j >> 1] = *reinterpret_cast<uint32_t*>(&o2);
          }
          *reinterpret_cast<uint4*>(orow + c * 16) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          *reinterpret_cast<uint4*>(orow + c * 16 + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        }
      }
    }
  }
  fa_fence_before();
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn fa_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = (EncodeTiledFn)p;
  return fn;
}

// bf16 matrix [rows, cols], row stride ld elements, boxes of box_rows x 64 columns, 128-byte swizzle
int fa_make_map(CUtensorMap* map, const void* base, long long rows, int cols, long long ld, int box_rows) {
  EncodeTiledFn enc = fa_encode_fn();
  RL_REQUIRE(enc != nullptr, "rl_attention_prefill_tc: the driver does not provide cuTensorMapEncodeTiled");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  RL_REQUIRE(r == CUDA_SUCCESS, "rl_attention_prefill_tc: cuTensorMapEncodeTiled failed with %d", (int)r);
  return RL_OK;
}

}  // namespace

// 1 if the tcgen05 prefill kernel takes this shape: head size 64 or 128.
extern "C" int rl_attention_prefill_tc_supported(int num_heads, int num_kv_heads, int head_dim) {
  if (num_kv_heads <= 0 || num_heads % num_kv_heads != 0) return 0;
  return head_dim == 64 || head_dim == 128;
}

// Same contract as rl_attention_prefill, with num_tiles = sum over sequences of
// ceil(tokens / 128), num_pages = pages in the cache pools, and err = device int that is set
// non-zero if a bounded wait in the kernel ran out.  The pools must hold finite values
// everywhere (see the note at the top of this file).
extern "C" int rl_attention_prefill_tc(const void* q, int ldq, const void* k_pool, const void* v_pool, int num_pages,
                                       const int* page_table, int max_pages, const int* cu_seqlens,
                                       const int* seq_slots, const int* kv_lens, int num_seqs, int num_tiles,
                                       int num_tokens, void* out, int ldo, int num_heads, int num_kv_heads, int head_dim,
                                       float scale, int window, int* err, cudaStream_t stream) {
  RL_REQUIRE(rl_attention_prefill_tc_supported(num_heads, num_kv_heads, head_dim),
             "rl_attention_prefill_tc: unsupported shape (heads %d, KV heads %d, head_dim %d): needs head_dim 64 or 128",
             num_heads, num_kv_heads, head_dim);
  RL_REQUIRE(num_seqs >= 0 && num_tiles >= 0 && num_tokens >= 0 && num_pages > 0 && num_heads <= 65535, "rl_attention_prefill_tc: bad sizes");
  RL_REQUIRE(ldq >= num_heads * head_dim && ldq % 8 == 0 && ldo >= num_heads * head_dim && ldo % 8 == 0,
             "rl_attention_prefill_tc: row strides must be multiples of 8 elements and hold all heads");
  RL_REQUIRE(((uintptr_t)q & 15) == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)k_pool & 15) == 0 && ((uintptr_t)v_pool & 15) == 0,
             "rl_attention_prefill_tc: pointers must be 16-byte aligned");
  RL_REQUIRE(window >= 0 && err != nullptr, "rl_attention_prefill_tc: negative window or null error word");
  if (num_seqs == 0 || num_tiles == 0) return RL_OK;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, FaSizes<128>::SMEM);
    RL_REQUIRE(e == cudaSuccess, "rl_attention_prefill_tc: cannot reserve %d bytes of shared memory: %s", FaSizes<128>::SMEM, cudaGetErrorString(e));
    e = cudaFuncSetAttribute(attention_prefill_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, FaSizes<64>::SMEM);
    RL_REQUIRE(e == cudaSuccess, "rl_attention_prefill_tc: cannot reserve %d bytes of shared memory: %s", FaSizes<64>::SMEM, cudaGetErrorString(e));
    configured = true;
  }
  CUtensorMap mq, mk, mv;
  int rc = fa_make_map(&mq, q, num_tokens, num_heads * head_dim, ldq, TQ);
  if (rc != RL_OK) return rc;
  const long long pool_rows = (long long)num_pages * num_kv_heads * RL_PAGE;
  rc = fa_make_map(&mk, k_pool, pool_rows, head_dim, head_dim, RL_PAGE);
  if (rc != RL_OK) return rc;
  rc = fa_make_map(&mv, v_pool, pool_rows, head_dim, head_dim, RL_PAGE);
  if (rc != RL_OK) return rc;
  cudaError_t e = head_dim == 128
      ? rl_launch_pdl(attention_prefill_tc_kernel<128>, dim3(num_tiles, num_heads), dim3(FA_THREADS), (size_t)FaSizes<128>::SMEM, stream,
                      mq, mk, mv, page_table, max_pages, cu_seqlens, seq_slots, kv_lens, num_seqs,
                      (__nv_bfloat16*)out, ldo, num_heads, num_kv_heads, scale * 1.4426950408889634f, window, err)
      : rl_launch_pdl(attention_prefill_tc_kernel<64>, dim3(num_tiles, num_heads), dim3(FA_THREADS), (size_t)FaSizes<64>::SMEM, stream,
                      mq, mk, mv, page_table, max_pages, cu_seqlens, seq_slots, kv_lens, num_seqs,
                      (__nv_bfloat16*)out, ldo, num_heads, num_kv_heads, scale * 1.4426950408889634f, window, err);
  if (e != cudaSuccess) {
    rl_set_error("rl_attention_prefill_tc: launch failed: %s", cudaGetErrorString(e));
    return RL_ERR_CUDA;
  }
  return RL_OK;
}
