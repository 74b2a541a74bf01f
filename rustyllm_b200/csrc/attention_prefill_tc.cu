// Prefill attention on the 5th-generation tensor cores (tcgen05), head sizes 64 and 128.
//
// Same math and the same packed, paged inputs as attention_prefill.cu (the mma.sync kernel,
// which this one is tested against): causal
// grouped-query attention of the step's query tokens over their sequence's cached keys
// and values, streaming softmax in float (SimonWaldherr/RustyLLM src/model.rs:7239-7294, 5807-5869).
//
// One CTA = 128 consecutive query tokens of one sequence and one query head.
//   S = Q K^T   tcgen05.mma 128 x 128 x 128, Q and the key tile in shared memory (TMA,
//               128-byte swizzle, K-major like the matrix products), S in tensor memory
//               (two buffers; a buffer is free for the scores of the tile after next as soon
//               as its softmax threads have the scores in registers, so those are computed
//               while this tile is being exponentiated)
//   softmax     eight warps in two groups of four that take the key tiles in turn (even tiles,
//               odd tiles), one thread a query row (= one lane of tensor memory) and tile, the
//               row's 128 scores in registers.  The two warps that share a scheduler work on
//               different tiles and are out of step: one's exponentials (the special-function
//               unit, 16 a clock and SM, is what bounds the kernel) run under the other's loads,
//               maxima and conversions.  The row's running maximum goes from a tile's thread to
//               the next tile's through shared memory (one mbarrier a warp pair and tile parity)
//               as soon as it is known, before the exponentials; it is kept lazily - the
//               accumulator is only rescaled when the maximum has grown by more than 2^8, so most
//               tiles skip the read-modify-write of O in tensor memory; each group sums its own
//               tiles' probabilities and the two sums meet at the end; P is written as bf16 into
//               a buffer of its own in tensor memory (64 columns a tile parity, tcgen05.st): it
//               never touches shared memory
//   O += P V    tcgen05.mma with P in tensor memory as A and the value tile as an
//               MN-major B operand (values are stored [position][head_dim]); O stays in
//               tensor memory over all key tiles
// Tensor memory: S 0-255, O 256-.., P behind O (512 columns at head size 128).
// A key tile is two cache pages (128 positions).  Warp 0 feeds TMA, warps 1 and 2 issue the two
// products (a thread each: issuing blocks while the tensor pipe is full, and one thread's waits
// and commits for one product would stand in the way of the other), warps 4-11 do the softmax and the final normalisation (with the registers that the
// first four warps give up: setmaxnreg).  Every wait inside the loop is an mbarrier
// wait and bounded; a softmax warp whose wait ran out leaves the loop and goes to the one named
// barrier behind it, which every softmax warp reaches.
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
constexpr int FA_THREADS = 384;       // warp 0: TMA, warp 1: S = Q K^T, warp 2: O += P V, warp 3: idle, warps 4-11: softmax
constexpr int FA_PV_WARP = 2;
// registers a thread: the first warpgroup hands most of its share to the two softmax warpgroups
constexpr int FA_REGS_FEED = 56, FA_REGS_SOFTMAX = 224;
constexpr uint32_t FA_WAIT_LIMIT = 1u << 22;
constexpr int HALF_BYTES = 128 * 64 * 2;               // [128 rows x 64 bf16], 16 KB
// sizes that depend on the head size HD (64 or 128): a head is HD / 64 halves of 64 dimensions
template <int HD> struct FaSizes {
  static constexpr int HALVES = HD / 64;
  static constexpr int Q_BYTES = HALVES * HALF_BYTES;          // 16 or 32 KB
  static constexpr int TILE_BYTES = HALVES * HALF_BYTES;       // a key tile or a value tile: 16 or 32 KB
  // keys are asked for a tile further ahead than values: the scores of a tile are computed as soon as the
  // buffer is free, a whole tile before its P V
  static constexpr int K_STAGES = HD == 64 ? 4 : 3;
  static constexpr int V_STAGES = HD == 64 ? 3 : 2;
  // + alignment slack, barriers, and the softmax threads' exchange: running maxima (two tiles in turn), and the
  // groups' last maxima and sums
  static constexpr int SMEM = Q_BYTES + (K_STAGES + V_STAGES) * TILE_BYTES + 1024 + 512 + 3 * 2 * TQ * 4;
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
                            int H, int G, float scale_log2e, int window, int* __restrict__ err,
                            const int* __restrict__ tile_order) {
  extern __shared__ uint8_t fa_smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)fa_smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* q_tile = smem;                                   // [2 halves][128 x 64]
  constexpr int HALVES = FaSizes<HD>::HALVES, Q_BYTES = FaSizes<HD>::Q_BYTES, TILE_BYTES = FaSizes<HD>::TILE_BYTES;
  constexpr int K_STAGES = FaSizes<HD>::K_STAGES, V_STAGES = FaSizes<HD>::V_STAGES;
  uint8_t* k_ring = smem + Q_BYTES;                         // [stage][halves]
  uint8_t* v_ring = k_ring + K_STAGES * TILE_BYTES;         // [stage][halves]
  uint64_t* bars = (uint64_t*)(v_ring + V_STAGES * TILE_BYTES);
  uint64_t* q_full = bars;                 // 1
  uint64_t* k_full = bars + 1;             // keys and values have rings of their own
  uint64_t* k_empty = k_full + K_STAGES;
  uint64_t* v_full = k_empty + K_STAGES;
  uint64_t* v_empty = v_full + V_STAGES;
  uint64_t* s_full = v_empty + V_STAGES;   // [2]
  uint64_t* s_free = s_full + 2;           // [2]: the scores of a tile are in its threads' registers
  uint64_t* p_full = s_free + 2;           // [2]: one a softmax group
  uint64_t* pv_done = p_full + 2;          // [2]: the P V of a tile (by parity) has completed
  uint64_t* o_full = pv_done + 2;          // 1
  uint64_t* m_ready = o_full + 1;          // [tile parity][quarter]: the running maximum after a tile
  uint32_t* tmem_slot = (uint32_t*)(m_ready + 8);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  int* s_seq = (int*)(tmem_slot + 2);
  int* s_tile = (int*)(tmem_slot + 3);
  float* m_shared = (float*)((uint8_t*)bars + 512);         // [tile parity][row]: running maximum after that tile
  float* x_m = m_shared + 2 * TQ;                            // [group][row]: the maximum the group's sum is scaled by
  float* x_sum = x_m + 2 * TQ;                               // [group][row]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  rl_pdl_trigger();
  if (threadIdx.x == 0) {
    fa_mbar_init(fa_smem_u32(q_full), 1);
    for (int i = 0; i < K_STAGES; ++i) { fa_mbar_init(fa_smem_u32(&k_full[i]), 1); fa_mbar_init(fa_smem_u32(&k_empty[i]), 1); }
    for (int i = 0; i < V_STAGES; ++i) { fa_mbar_init(fa_smem_u32(&v_full[i]), 1); fa_mbar_init(fa_smem_u32(&v_empty[i]), 1); }
    for (int i = 0; i < 2; ++i) fa_mbar_init(fa_smem_u32(&s_full[i]), 1);
    for (int i = 0; i < 2; ++i) {
      fa_mbar_init(fa_smem_u32(&s_free[i]), 4); fa_mbar_init(fa_smem_u32(&p_full[i]), 4);
      fa_mbar_init(fa_smem_u32(&pv_done[i]), 1);
    }
    for (int i = 0; i < 8; ++i) fa_mbar_init(fa_smem_u32(&m_ready[i]), 1);
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
  // ---- which sequence and which of its 128-row query tiles.  The grid is (heads, tiles) and
  // blocks start in the order of the grid: with the caller's table the tiles come by falling
  // number of keys, all heads of the heaviest tile first, so the last blocks to start are the
  // lightest; without it, the tiles of the step in reverse (right for one sequence) ----
  if (threadIdx.x == 32) {
    if (tile_order != nullptr) {
      *s_seq = tile_order[2 * blockIdx.y]; *s_tile = tile_order[2 * blockIdx.y + 1];
    } else {
      int t = (int)(gridDim.y - 1 - blockIdx.y), b = 0;
      for (; b < num_seqs; ++b) {
        const int tiles = (cu_seqlens[b + 1] - cu_seqlens[b] + TQ - 1) / TQ;
        if (t < tiles) break;
        t -= tiles;
      }
      *s_seq = b; *s_tile = t;
    }
  }
  fa_fence_before();
  __syncthreads();
  fa_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // S buffers at columns 0 and 128, O at 256, the two P buffers (64 columns each) behind O
  const uint32_t tmem_s0 = tmem_base, tmem_o = tmem_base + 256, tmem_p = tmem_base + 256 + HD;
  const int b = *s_seq;
  const bool have_work = b < num_seqs;      // the grid is sized exactly; defensive
  const int h = blockIdx.x, gkv = h / (H / G);
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

  if (warp < 4) {
    // ---- the feeding warps: a few registers are enough; the rest goes to the softmax warps ----
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(FA_REGS_FEED));
    if (warp == 0) {
      if (lane == 0 && have_work) {
        // ---------------- TMA producer ----------------
        fa_expect_tx(fa_smem_u32(q_full), Q_BYTES);
#pragma unroll
        for (int half = 0; half < HALVES; ++half)
          fa_tma_2d(fa_smem_u32(q_tile + half * HALF_BYTES), &map_q, fa_smem_u32(q_full), h * HD + 64 * half, row0 + qt0);
        // keys and values have rings of their own: the keys' stage is free once the S of its tile
        // is done, the values' once its P V is; whichever is free first is filled first
        auto load = [&](int i, bool values) {
          const int kt = kt_begin + i, st = i % (values ? V_STAGES : K_STAGES);
          const int p0 = pages[2 * kt];
          const int p1 = (2 * kt + 1) * RL_PAGE < kv_len ? pages[2 * kt + 1] : p0;   // beyond the sequence: any valid page (all masked)
          const int r0 = (p0 * G + gkv) * RL_PAGE, r1 = (p1 * G + gkv) * RL_PAGE;
          const uint32_t fb = fa_smem_u32(values ? &v_full[st] : &k_full[st]);
          uint8_t* base = (values ? v_ring : k_ring) + (size_t)st * TILE_BYTES;
          const CUtensorMap* map = values ? &map_v : &map_k;
          fa_expect_tx(fb, TILE_BYTES);
#pragma unroll
          for (int half = 0; half < HALVES; ++half) {     // 64 head dimensions a half; 64 positions a page
            fa_tma_2d(fa_smem_u32(base + half * HALF_BYTES), map, fb, 64 * half, r0);
            fa_tma_2d(fa_smem_u32(base + half * HALF_BYTES + 64 * 128), map, fb, 64 * half, r1);
          }
        };
        auto stage_free = [&](uint64_t* empty, int stages, int i) -> bool {      // without waiting
          return i < stages || fa_try_wait(fa_smem_u32(&empty[i % stages]), ((i / stages) & 1) ^ 1);
        };
        int nk = 0, nv = 0;
        uint32_t idle = 0;
        bool ok = true;
        while (ok && nv < num_kt) {
          bool moved = false;
          if (nk < num_kt && stage_free(k_empty, K_STAGES, nk)) { load(nk, false); ++nk; moved = true; }
          if (nv < nk && stage_free(v_empty, V_STAGES, nv)) { load(nv, true); ++nv; moved = true; }
          if (moved) idle = 0;
          else if (++idle > FA_WAIT_LIMIT || ((idle & 1023u) == 1023u && *abort_flag)) ok = false;
        }
        if (!ok && !*abort_flag) { *abort_flag = 1; atomicExch(err, 11); }
      }
    } else if (warp == 1) {
      if (lane == 0 && have_work) {
        // ---------------- issuer of S = Q K^T ----------------
        // The two products have a thread each, in different warps: issuing blocks while the tensor pipe
        // is full, so with one thread the waits, commits and loop of one product would stand in the
        // way of the other.  They need no order between them: every dependency is an mbarrier.
        constexpr uint32_t idesc_s = fa_idesc(TQ, TK, 0);     // both K-major
        bool ok = fa_wait(fa_smem_u32(q_full), 0, abort_flag);
        auto issue_s = [&](int i) -> bool {                   // scores of tile i into S buffer i % 2
          const int st = i % K_STAGES, sb = i & 1;
          if (!fa_wait(fa_smem_u32(&k_full[st]), (i / K_STAGES) & 1, abort_flag)) return false;
          fa_fence_after();
          uint8_t* base = k_ring + (size_t)st * TILE_BYTES;
#pragma unroll
          for (int k = 0; k < HD / 16; ++k) {
            const uint64_t da = fa_desc_kmajor(fa_smem_u32(q_tile + (k / 4) * HALF_BYTES)) + 2 * (k % 4);
            const uint64_t db = fa_desc_kmajor(fa_smem_u32(base + (k / 4) * HALF_BYTES)) + 2 * (k % 4);
            fa_mma(tmem_s0 + (uint32_t)(sb * TK), da, db, idesc_s, k > 0 ? 1u : 0u);
          }
          fa_commit(fa_smem_u32(&s_full[sb]));
          fa_commit(fa_smem_u32(&k_empty[st]));               // the keys' stage is free once S is done
          return true;
        };
        if (ok && num_kt > 0) ok = issue_s(0);
        if (ok && num_kt > 1) ok = issue_s(1);
        for (int i = 0; i + 2 < num_kt && ok; ++i) {
          // the scores of the tile after next, as soon as this tile's are in its threads' registers:
          // they are computed while this tile and the next are being exponentiated
          ok = fa_wait(fa_smem_u32(&s_free[i & 1]), (i >> 1) & 1, abort_flag);
          if (ok) ok = issue_s(i + 2);
        }
        if (!ok && !*abort_flag) { *abort_flag = 1; atomicExch(err, 12); }
      }
    } else if (warp == FA_PV_WARP) {
      if (lane == 0 && have_work) {
        // ---------------- issuer of O += P V ----------------
        constexpr uint32_t idesc_o = fa_idesc(TQ, HD, 1);     // P in tensor memory, V MN-major
        bool ok = true;
        for (int i = 0; i < num_kt && ok; ++i) {
          if (!fa_wait(fa_smem_u32(&v_full[i % V_STAGES]), (i / V_STAGES) & 1, abort_flag)) { ok = false; break; }
          if (!fa_wait(fa_smem_u32(&p_full[i & 1]), (i >> 1) & 1, abort_flag)) { ok = false; break; }
          fa_fence_after();
          uint8_t* vbase = v_ring + (size_t)(i % V_STAGES) * TILE_BYTES;
#pragma unroll
          for (int k = 0; k < TK / 16; ++k) {                 // 16 positions a step
            // P of this tile: 16 keys = 8 columns of packed bf16 pairs a step, in the P buffer of its parity
            const uint64_t db = fa_desc_mnmajor(fa_smem_u32(vbase + k * 16 * 128), HALF_BYTES);
            fa_mma_a_tmem(tmem_o, tmem_p + (uint32_t)((i & 1) * (TK / 2) + 8 * k), db, idesc_o, (i > 0 || k > 0) ? 1u : 0u);
          }
          fa_commit(fa_smem_u32(&pv_done[i & 1]));            // O, and this parity's P buffer, are free again once these have completed
          fa_commit(fa_smem_u32(&v_empty[i % V_STAGES]));
        }
        if (ok) fa_commit(fa_smem_u32(o_full));
        else if (!*abort_flag) { *abort_flag = 1; atomicExch(err, 13); }
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(FA_REGS_SOFTMAX));
    if (have_work) {
      // ---------------- softmax warps: group 0 takes the even key tiles, group 1 the odd ones ----------------
      constexpr int OC = HD / 2;                              // output columns a thread writes at the end
      const int quarter = warp & 3, grp = (warp - 4) >> 2;
      const int r = quarter * 32 + lane;                      // row of the tile = lane of tensor memory
      const int pos = start_pos + qt0 + r;                    // position of this row's query
      const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
      float m_mine = -INFINITY, l_run = 0.f;                  // maximum this group's sum is scaled by; the sum
      bool ok = true;                                         // warp-uniform
      const float2 sc2 = make_float2(scale_log2e, scale_log2e);
      for (int i = grp; i < num_kt && ok; i += 2) {
        const int sb = grp, key0 = (kt_begin + i) * TK;       // S buffer = tile parity = group
        ok = __all_sync(0xffffffffu, fa_wait(fa_smem_u32(&s_full[sb]), (i >> 1) & 1, abort_flag));
        if (!ok) break;
        fa_fence_after();
        const uint32_t s_addr = tmem_s0 + lane_addr + (uint32_t)(sb * TK);
        // the row's 128 scores into registers with one wait; the S buffer is then free for the tile
        // after next.  Everything below is straight-line code over the registers
        uint32_t sa[TK];
#pragma unroll
        for (int c = 0; c < TK / 32; ++c) fa_ld32(s_addr + 32 * c, sa + 32 * c);
        fa_wait_ld();
        fa_fence_before();
        __syncwarp();
        if (lane == 0) fa_arrive(fa_smem_u32(&s_free[sb]));
        // The tile on the diagonal (no window) has code of its own, by 32-key chunks; every other tile
        // runs straight-line code over all 128 scores, which the scheduler can reorder freely.
        const bool diag = window <= 0 && key0 + TK - 1 > start_pos + qt0;     // warp-uniform
        int live = TK / 32;                     // diagonal tile: chunks that some row of this warp sees
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        if (!diag) {
          if (window > 0) {
#pragma unroll
            for (int j = 0; j < TK; ++j) {
              const int key = key0 + j;
              if (!(key <= pos && key > pos - window)) sa[j] = 0xff800000u;          // -inf
            }
          }
#pragma unroll
          for (int j = 0; j < TK; j += 2) mx4[(j >> 1) & 3] = fa_max3(mx4[(j >> 1) & 3], __uint_as_float(sa[j]), __uint_as_float(sa[j + 1]));
        } else {
          // key j of the tile is visible to this row if j <= lim.  Rows grow with the lane, so the chunks
          // left of the warp's first row's limit need no mask, and those right of its last row's limit
          // are dropped whole: no maxima, no exponentials, P = 0
          const int lim = pos - key0;
          const int lim0 = __shfl_sync(0xffffffffu, lim, 0), lim31 = __shfl_sync(0xffffffffu, lim, 31);
          live = lim31 < 0 ? 0 : min(TK / 32, (lim31 >> 5) + 1);
#pragma unroll
          for (int c = 0; c < TK / 32; ++c) {
            if (c < live) {
              if (32 * c + 31 > lim0) {
#pragma unroll
                for (int j = 32 * c; j < 32 * c + 32; ++j) sa[j] = j > lim ? 0xff800000u : sa[j];
              }
#pragma unroll
              for (int j = 32 * c; j < 32 * c + 32; j += 2)
                mx4[(j >> 1) & 3] = fa_max3(mx4[(j >> 1) & 3], __uint_as_float(sa[j]), __uint_as_float(sa[j + 1]));
            }
          }
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2e;
        // the running maximum after the tile before (the other group's), and after this one: lazy, moved
        // (with O and the sums rescaled) only when it grew by more than 2^8
        float m_prev = -INFINITY;
        if (i > 0) {
          ok = __all_sync(0xffffffffu, fa_wait(fa_smem_u32(&m_ready[((i - 1) & 1) * 4 + quarter]), ((i - 1) >> 1) & 1, abort_flag));
          if (!ok) break;
          m_prev = m_shared[((i - 1) & 1) * TQ + r];
        }
        float m_now = m_prev;
        if (mx > m_prev + LAZY_LOG2 || (m_prev == -INFINITY && mx > -INFINITY)) m_now = mx;
        m_shared[(i & 1) * TQ + r] = m_now;
        __syncwarp();
        if (lane == 0) fa_arrive(fa_smem_u32(&m_ready[(i & 1) * 4 + quarter]));   // the next tile's threads may go on
        const float corr = m_now != m_prev ? fa_exp2(m_prev - m_now) : 1.0f;       // 0 on the first visible tile
        const bool any_rescale = __any_sync(0xffffffffu, corr != 1.0f);
        if (m_mine != m_now) { l_run *= fa_exp2(m_mine - m_now); m_mine = m_now; }
        // probabilities: exp2(score * scale - maximum), two scores an FMA; summed in float, rounded
        // to bf16 for the product with V and packed in place (sa[0..63] then hold the row's 128)
        const float m_sub = m_now == -INFINITY ? 0.f : m_now;
        const float2 nm2 = make_float2(-m_sub, -m_sub);
        float2 sum2[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
        auto soft2 = [&](int j) {               // scores j, j + 1 -> probabilities, packed into sa[j / 2]
          const float2 t = fa_ffma2(make_float2(__uint_as_float(sa[j]), __uint_as_float(sa[j + 1])), sc2, nm2);
          const float2 p2 = make_float2(fa_exp2(t.x), fa_exp2(t.y));
          sum2[(j >> 1) & 3] = fa_fadd2(sum2[(j >> 1) & 3], p2);
          __nv_bfloat162 pb = __floats2bfloat162_rn(p2.x, p2.y);
          sa[j >> 1] = *reinterpret_cast<uint32_t*>(&pb);
        };
        if (!diag) {
#pragma unroll
          for (int j = 0; j < TK; j += 2) {
            const float2 t = fa_ffma2(make_float2(__uint_as_float(sa[j]), __uint_as_float(sa[j + 1])), sc2, nm2);
            const float2 p2 = make_float2(fa_exp2(t.x), fa_exp2(t.y));
            sum2[(j >> 1) & 3] = fa_fadd2(sum2[(j >> 1) & 3], p2);
            __nv_bfloat162 pb = __floats2bfloat162_rn(p2.x, p2.y);
            sa[j >> 1] = *reinterpret_cast<uint32_t*>(&pb);
          }
        } else {
#pragma unroll
          for (int c = 0; c < TK / 32; ++c) {
            if (c < live) {
#pragma unroll
              for (int j = 32 * c; j < 32 * c + 32; j += 2) soft2(j);
            } else {
#pragma unroll
              for (int j = 16 * c; j < 16 * c + 16; ++j) sa[j] = 0u;
            }
          }
        }
        // the P buffer of this parity is free once the P V of the tile two back has completed; the barriers
        // take turns by tile parity, and this thread waited for the tile four back on the same one
        if (i >= 2) {
          ok = __all_sync(0xffffffffu, fa_wait(fa_smem_u32(&pv_done[i & 1]), ((i - 2) >> 1) & 1, abort_flag));
          if (!ok) break;
        }
        // O is only touched once the previous tile's P V has completed: waited for only if this warp has a
        // row to rescale (the tile three back is done, as the one two back is; the barrier cannot have run
        // ahead: the next P V needs our arrival)
        if (any_rescale && i > 0) {
          ok = __all_sync(0xffffffffu, fa_wait(fa_smem_u32(&pv_done[(i - 1) & 1]), ((i - 1) >> 1) & 1, abort_flag));
          if (!ok) break;
          fa_fence_after();
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {               // the whole row of O
            uint32_t v[32];
            const uint32_t o_addr = tmem_o + lane_addr + (uint32_t)(c * 32);
            fa_ld32(o_addr, v);
            fa_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * corr);
            fa_st16(o_addr, *reinterpret_cast<uint32_t(*)[16]>(v));
            fa_st16(o_addr + 16, *reinterpret_cast<uint32_t(*)[16]>(v + 16));
          }
        }
        fa_fence_after();
        // 16 keys are 8 columns of packed pairs
        const uint32_t p_addr = tmem_p + lane_addr + (uint32_t)(sb * (TK / 2));
#pragma unroll
        for (int c = 0; c < TK / 32; ++c) fa_st16(p_addr + 16 * c, *reinterpret_cast<uint32_t(*)[16]>(sa + 16 * c));
        fa_wait_st();
        const float2 s01 = fa_fadd2(sum2[0], sum2[1]), s23 = fa_fadd2(sum2[2], sum2[3]);
        l_run += (s01.x + s01.y) + (s23.x + s23.y);
        // P is ready for the tensor cores
        fa_fence_before();
        __syncwarp();
        if (lane == 0) fa_arrive(fa_smem_u32(&p_full[grp]));
      }
      // ---- O / l -> out ----
      if (ok) ok = __all_sync(0xffffffffu, fa_wait(fa_smem_u32(o_full), 0, abort_flag));
      if (!ok && !*abort_flag) { *abort_flag = 1; atomicExch(err, 14); }
      x_sum[grp * TQ + r] = l_run;
      x_m[grp * TQ + r] = m_mine;
      fa_softmax_sync();
      fa_fence_after();
      if (ok) {
        // O is scaled by the last tile's maximum, the larger of the two groups'; sums in group order
        const float m_other = x_m[(grp ^ 1) * TQ + r], l_other = x_sum[(grp ^ 1) * TQ + r];
        const float m_fin = fmaxf(m_mine, m_other);
        const float w_mine = m_mine == -INFINITY ? 0.f : fa_exp2(m_mine - m_fin);
        const float w_other = m_other == -INFINITY ? 0.f : fa_exp2(m_other - m_fin);
        const float l_row = grp == 0 ? l_run * w_mine + l_other * w_other : l_other * w_other + l_run * w_mine;
        const float inv = l_row > 0.f ? 1.0f / l_row : 0.f;
        __nv_bfloat16* orow = out + (size_t)(row0 + qt0 + r) * ldo + (size_t)h * HD + grp * OC;
#pragma unroll 1
        for (int c = 0; c < OC / 16; ++c) {
          uint32_t v[16];
          fa_ld16(tmem_o + lane_addr + (uint32_t)(grp * OC + c * 16), v);
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
// non-zero if a bounded wait in the kernel ran out.  tile_order (may be null): num_tiles pairs
// (sequence, tile of the sequence), every tile of the step once, in the order the blocks should
// start in (heaviest first).  The pools must hold finite values
// everywhere (see the note at the top of this file).
extern "C" int rl_attention_prefill_tc(const void* q, int ldq, const void* k_pool, const void* v_pool, int num_pages,
                                       const int* page_table, int max_pages, const int* cu_seqlens,
                                       const int* seq_slots, const int* kv_lens, int num_seqs, int num_tiles,
                                       int num_tokens, void* out, int ldo, int num_heads, int num_kv_heads, int head_dim,
                                       float scale, int window, int* err, const int* tile_order, cudaStream_t stream) {
  RL_REQUIRE(rl_attention_prefill_tc_supported(num_heads, num_kv_heads, head_dim),
             "rl_attention_prefill_tc: unsupported shape (heads %d, KV heads %d, head_dim %d): needs head_dim 64 or 128",
             num_heads, num_kv_heads, head_dim);
  RL_REQUIRE(num_seqs >= 0 && num_tiles >= 0 && num_tokens >= 0 && num_pages > 0 && num_tiles <= 65535, "rl_attention_prefill_tc: bad sizes");
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
      ? rl_launch_pdl(attention_prefill_tc_kernel<128>, dim3(num_heads, num_tiles), dim3(FA_THREADS), (size_t)FaSizes<128>::SMEM, stream,
                      mq, mk, mv, page_table, max_pages, cu_seqlens, seq_slots, kv_lens, num_seqs,
                      (__nv_bfloat16*)out, ldo, num_heads, num_kv_heads, scale * 1.4426950408889634f, window, err, tile_order)
      : rl_launch_pdl(attention_prefill_tc_kernel<64>, dim3(num_heads, num_tiles), dim3(FA_THREADS), (size_t)FaSizes<64>::SMEM, stream,
                      mq, mk, mv, page_table, max_pages, cu_seqlens, seq_slots, kv_lens, num_seqs,
                      (__nv_bfloat16*)out, ldo, num_heads, num_kv_heads, scale * 1.4426950408889634f, window, err, tile_order);
  if (e != cudaSuccess) {
    rl_set_error("rl_attention_prefill_tc: launch failed: %s", cudaGetErrorString(e));
    return RL_ERR_CUDA;
  }
  return RL_OK;
}
