// out[M, N] = A[M, K] * W[N, K]^T (+ bias) in bf16 on the 5th-generation tensor cores:
// tcgen05.mma with the accumulator in tensor memory, operands staged in shared
// memory by TMA (128-byte swizzle), a ring of stages between one producer thread and
// one MMA-issuing thread, and four epilogue warps that read the accumulator back
// with tcgen05.ld.
//
// The weight rows are the MMA's M dimension (128 per CTA) and the step's tokens its N
// dimension (16..256 per CTA): a decode step with a handful of tokens still fills
// the 128-row instruction with weight rows and streams each weight exactly once,
// and a prefill uses 128 x 256 tiles.  Both operands are K-major, as every weight
// of the model is stored ([out x in], SimonWaldherr/RustyLLM src/model.rs:185-186); no
// transposes anywhere.  Accumulation is float; the epilogue adds the optional bias
// and stores bf16, stores float, or adds into a float buffer (the residual sum).
//
// Split-K over a thread-block cluster: with few tokens a product has too few 128-row
// tiles to keep 148 SMs streaming, so the K range of a tile is cut into 2, 4 or 8 parts
// that run as the CTAs of one cluster.  Each CTA leaves its float partial tile in its
// own shared memory; after a cluster barrier every CTA reads "its" token columns from
// all parts through distributed shared memory, adds them in the order of the parts
// (0, 1, 2, ...: the result does not depend on timing) and runs the epilogue for those
// columns.  No global scratch, no atomics.
//
// RMSNorm folded into the products around it (both optional).  A product that adds into
// the residual can, in the same epilogue, write `residual * norm weight` in bf16 and, for
// every token and every 32 output columns (one epilogue warp of one tile), the sum of the
// squares of the new residual values, each in its own place (no atomics, no barrier).  The
// product that consumes that bf16 matrix multiplies its accumulator rows by
// rsqrt(sum of those sums / K + eps) before the bias: W (r x g) = r W (x g), r being
// one number a token.  Sums and r are float; the norm's own kernel, one more launch
// between two products, is not needed then.  For up to 64 tokens (where a launch costs as
// much as the norm itself); above, the norm keeps its kernel.
//
// Rotary encoding and the cache write folded into the QKV product (optional, head size 128,
// up to 64 tokens, K split over a cluster): a tile of 128 output columns is one head, and
// in the cluster epilogue one warp holds all of it for a token, so the pair (i, i + 64) is
// an exchange between two lanes.  Query heads are rotated and stored to the output; key
// heads are rotated and stored to their place in the paged cache, value heads stored
// there as they are (SimonWaldherr/RustyLLM src/model.rs:5562-5647, 7233-7236): the separate
// rotation kernel and its launch are not needed.  Angles are float(pos) * inv_freq in
// 32-bit with the accurate sincosf, applied to the float accumulator (one rounding to
// bf16 instead of two).
//
// Every wait on an mbarrier is bounded: when it runs out the kernel records a code
// in the error word, all roles leave their loops, tensor memory is freed and the
// kernel returns.
#include <stdio.h>

#include "tc_device.cuh"

// DEEP (few tokens only): two CTAs an SM with rings half as deep again, for products whose whole
// grid fits two CTAs an SM.  A CTA streams at (bytes it has in flight) / latency, so a grid that
// leaves SMs half empty is the faster the more each of its CTAs has in flight - and the more
// weights it has asked for before the kernel in front of it has finished.
template <int BT, bool DEEP = false>
struct TcConfig {
  static constexpr int STAGE_BYTES = (BLOCK_N_OUT + BT) * BLOCK_K * 2;
  // few tokens: the product streams weights, three stages a CTA and three or four CTAs an
  // SM keep more loads in flight than one deep ring; many tokens: one CTA, a deep ring
  static constexpr int RING_BYTES_MAX = BT <= 64 ? (DEEP ? 110592 : 73728) : 196608;
  static constexpr int STAGES = (RING_BYTES_MAX / STAGE_BYTES) < 8 ? (RING_BYTES_MAX / STAGE_BYTES) : 8;
  static constexpr int MIN_CTAS = BT <= 64 ? (DEEP ? 2 : 3) : 1;
  static constexpr int TMEM_COLS = BT < 32 ? 32 : BT;
  static constexpr int FUSE_FLOATS = 3 * BT;       // the tile's row scales; its tokens' positions and cache rows
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + FUSE_FLOATS * 4;
};

// The epilogue of one finished tile: the accumulator (128 weight rows x BT tokens, float,
// in tensor memory at `tmem_acc`) goes to the output in the asked form.  Called by the four
// epilogue warps; `quarter` = warp index % 4 = the 32 lanes of tensor memory the warp may read.
template <int BT>
__device__ __forceinline__ void tile_epilogue(uint32_t tmem_acc, int quarter, int lane, int n0, int m0, int cols, int M, int N,
                                              int ldo, const float* __restrict__ bias, void* __restrict__ out,
                                              int out_mode, const TcFuse& fuse, float* fuse_smem) {
  const int n = n0 + quarter * 32 + lane;          // output feature of this thread
  const float b = (bias != nullptr && n < N) ? bias[n] : 0.f;
  const float* rs = fuse_smem;                     // row scales (made by epilogue_row_scales)
  const bool make_norm = fuse.norm_weight != nullptr && out_mode == TC_OUT_ADD_F32;
  const float g = (make_norm && n < N) ? fuse.norm_weight[n] : 0.f;
  if (BT >= 128 && out_mode == TC_OUT_ADD_F32 && !make_norm && fuse.scale_partials == nullptr) {
    // Many tokens, adding into the residual: the epilogue moves 8 bytes a result and is bound
    // by how many of its loads are in flight.  The residual values of the next 32 tokens are
    // requested before this thread turns to the 32 it holds, stores behind loads.
    float* of = (float*)out;
    const bool live = n < N;
    float cur[32], nxt[32];
    auto fetch = [&](float (&dst)[32], int c0) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int m = m0 + c0 * 16 + j;
        dst[j] = (live && c0 * 16 + j < cols && m < M) ? __ldcg(of + (size_t)m * ldo + n) : 0.f;
      }
    };
    fetch(cur, 0);
#pragma unroll 1
    for (int c = 0; c < BT / 16; c += 2) {
      if (c * 16 >= cols) break;
      if ((c + 2) * 16 < cols) fetch(nxt, c + 2);
      uint32_t r[32];
      tmem_ld16(tmem_acc + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c * 16), *reinterpret_cast<uint32_t(*)[16]>(r));
      tmem_ld16(tmem_acc + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c * 16 + 16), *reinterpret_cast<uint32_t(*)[16]>(r + 16));
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int m = m0 + c * 16 + j;
        if (live && c * 16 + j < cols && m < M) of[(size_t)m * ldo + n] = cur[j] + __uint_as_float(r[j]) + b;
      }
#pragma unroll
      for (int j = 0; j < 32; ++j) cur[j] = nxt[j];
    }
    return;
  }
#pragma unroll 1
  for (int c = 0; c < BT / 16; ++c) {
    if (c * 16 >= cols) break;       // cols: the tile's tokens (a multiple of 16, or what is left of M)
    uint32_t r[16];
    tmem_ld16(tmem_acc + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c * 16), r);
    tmem_ld_wait();
    if (fuse.scale_partials != nullptr) {
#pragma unroll
      for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * rs[c * 16 + j]);
    }
    if (out_mode == TC_OUT_SWIGLU) {
      // weight rows are (gate_0, up_0, gate_1, up_1, ...): the even lane holds the gate, its
      // odd neighbour the up value of the same output column n / 2
      // ... the even lane finishes columns 0-7 of the chunk, the odd lane columns 8-15: each
      // sends the other the half it does not need (one shuffle a column pair).
      __nv_bfloat16* ob = (__nv_bfloat16*)out;
      const bool even = (lane & 1) == 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float lo = __uint_as_float(r[j]) + b, hi = __uint_as_float(r[j + 8]) + b;
        const float got = __shfl_xor_sync(0xffffffffu, even ? hi : lo, 1);
        const float gate = even ? lo : got, up = even ? got : hi;
        const int m = m0 + c * 16 + (even ? j : j + 8);
        if ((n | 1) < N && m < M) ob[(size_t)m * ldo + (n >> 1)] = __float2bfloat16_rn(silu_mul(gate, up));
      }
    } else if (out_mode == TC_OUT_ADD_F32) {
      // all sixteen loads of the residual first, then the stores: a load placed after
      // a store to the same array would wait for it, one memory latency a column
      float* of = (float*)out;
      const bool live = n < N;
      float nv[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int m = m0 + c * 16 + j;
        nv[j] = (live && m < M) ? __ldcg(of + (size_t)m * ldo + n) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int m = m0 + c * 16 + j;
        nv[j] = (live && m < M) ? nv[j] + __uint_as_float(r[j]) + b : 0.f;
        if (live && m < M) of[(size_t)m * ldo + n] = nv[j];
      }
      if (make_norm) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int m = m0 + c * 16 + j;
          if (live && m < M) fuse.norm_out[(size_t)m * fuse.ld_norm + n] = __float2bfloat16_rn(nv[j] * g);
          const float sq = tc_warp_sum(nv[j] * nv[j]);      // this warp's 32 columns of token m
          if (lane == 0 && m < M) fuse.norm_partials[(size_t)m * fuse.norm_count + 4 * (n0 / BLOCK_N_OUT) + quarter] = sq;
        }
      }
    } else if (n < N) {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int m = m0 + c * 16 + j;
        if (m < M) {
          const float v = __uint_as_float(r[j]) + b;
          const size_t o = (size_t)m * ldo + n;
          if (out_mode == TC_OUT_BF16) ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(v);
          else ((float*)out)[o] = v;
        }
      }
    }
  }
}

// BT: tokens per CTA (MMA N).  Grid: (parts * ceil(N_out / 128), ceil(M_tokens / BT)) in
// clusters of `parts` CTAs along x; the CTA's rank in its cluster is its part of K.
template <int BT, bool DEEP>
__global__ void __launch_bounds__(TC_THREADS, TcConfig<BT, DEEP>::MIN_CTAS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
               const float* __restrict__ bias, void* __restrict__ out, int out_mode, int M, int N, int K,
               int ldo, int* __restrict__ err, int kb_per_split, const TcFuse fuse) {
  using Cfg = TcConfig<BT, DEEP>;
  extern __shared__ uint8_t smem_raw[];
  // tiles need 1024-byte alignment for the 128-byte swizzle pattern
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* tiles = smem;
  uint64_t* bars = (uint64_t*)(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
  float* fuse_smem = (float*)(smem + Cfg::STAGES * Cfg::STAGE_BYTES + 256);
  uint64_t* full_bar = bars;                       // [STAGES]
  uint64_t* empty_bar = bars + Cfg::STAGES;        // [STAGES]
  uint64_t* accum_bar = bars + 2 * Cfg::STAGES;    // [1]
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * Cfg::STAGES + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_splits = (int)cluster_size(), split = (int)cluster_rank();
  const int n0 = (blockIdx.x / num_splits) * BLOCK_N_OUT;   // first weight row (output feature) of this CTA
  const int m0 = blockIdx.y * BT;                           // first token of this CTA
  const int total_kb = (K + BLOCK_K - 1) / BLOCK_K;
  const int kb0 = split * kb_per_split;                            // this CTA's part of the K range
  const int num_kb = min(kb_per_split, total_kb - kb0);            // > 0: the host sizes the parts so

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    mbar_init(smem_u32(accum_bar), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  rl_pdl_trigger();   // the next kernel on the stream may begin its own prologue
  if (warp == 0) {
    if (lane == 0) {
      // ---------------- producer: TMA loads into the ring ----------------
      // Weights are written by no kernel of a step: the first ring of weight tiles is
      // requested before the wait for the preceding kernels, the activations after it.
      const int pre = min(num_kb, Cfg::STAGES);
      for (int kb = 0; kb < pre; ++kb) {
        const uint32_t fb = smem_u32(&full_bar[kb]);
        mbar_expect_tx(fb, Cfg::STAGE_BYTES);
        tma_load_2d(smem_u32(tiles + (size_t)kb * Cfg::STAGE_BYTES), &map_w, fb, (kb0 + kb) * BLOCK_K, n0);
      }
      rl_pdl_wait();
      for (int kb = 0; kb < pre; ++kb)
        tma_load_2d(smem_u32(tiles + (size_t)kb * Cfg::STAGE_BYTES + BLOCK_N_OUT * BLOCK_K * 2), &map_a,
                    smem_u32(&full_bar[kb]), (kb0 + kb) * BLOCK_K, m0);
      for (int kb = pre; kb < num_kb; ++kb) {
        const int s = kb % Cfg::STAGES;
        const uint32_t phase = (kb / Cfg::STAGES) & 1;
        if (!mbar_wait(smem_u32(&empty_bar[s]), phase ^ 1, abort_flag)) {
          if (!*abort_flag) { *abort_flag = 1; atomicExch(err, 1); }
          break;
        }
        const uint32_t fb = smem_u32(&full_bar[s]);
        mbar_expect_tx(fb, Cfg::STAGE_BYTES);
        uint8_t* st = tiles + (size_t)s * Cfg::STAGE_BYTES;
        tma_load_2d(smem_u32(st), &map_w, fb, (kb0 + kb) * BLOCK_K, n0);
        tma_load_2d(smem_u32(st + BLOCK_N_OUT * BLOCK_K * 2), &map_a, fb, (kb0 + kb) * BLOCK_K, m0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer ----------------
      constexpr uint32_t idesc = make_idesc(BLOCK_N_OUT, BT);
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % Cfg::STAGES;
        const uint32_t phase = (kb / Cfg::STAGES) & 1;
        if (!mbar_wait(smem_u32(&full_bar[s]), phase, abort_flag)) {
          if (!*abort_flag) { *abort_flag = 1; atomicExch(err, 2); }
          ok = false;
          break;
        }
        tc_fence_after();
        uint8_t* st = tiles + (size_t)s * Cfg::STAGE_BYTES;
        const uint64_t da = make_smem_desc(smem_u32(st));
        const uint64_t db = make_smem_desc(smem_u32(st + BLOCK_N_OUT * BLOCK_K * 2));
#pragma unroll
        for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
          // advancing 16 elements = 32 bytes inside the swizzled row: +2 in units of 16 bytes
          umma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(&empty_bar[s]));   // the stage is free once these MMAs have read it
      }
      if (ok) umma_commit(smem_u32(accum_bar));  // the accumulator is complete
    }
  } else {
    // ---------------- epilogue: warps 2..5, each its quarter of the 128 lanes ----------------
    rl_pdl_wait();      // before this warp reads or writes global memory
    if constexpr (BT <= 64) {
      if (fuse.scale_partials != nullptr)    // while the products still run
        epilogue_row_scales<BT>(fuse, m0, M, K, warp & 3, lane, fuse_smem);
    }
    if (out_mode == TC_OUT_ROPE_KV) {
      // position of every token of the tile and the row of the cache pools it is stored in
      int* tok_pos = (int*)(fuse_smem + BT);
      int* tok_row = tok_pos + BT;
      for (int t = threadIdx.x - 64; t < BT; t += 128) {
        const int m = m0 + t;
        int pos = 0, row = 0;
        if (m < M) {
          pos = fuse.positions[m];
          if (fuse.k_pool != nullptr) {
            const int page = fuse.page_table[(size_t)fuse.slot_of_token[m] * fuse.max_pages + pos / RL_PAGE];
            row = page * fuse.num_kv_heads * RL_PAGE + pos % RL_PAGE;        // + kv head * RL_PAGE
          }
        }
        tok_pos[t] = pos; tok_row[t] = row;
      }
      epilogue_sync();
    }
    const bool ok = mbar_wait(smem_u32(accum_bar), 0, abort_flag);
    if (!ok && !*abort_flag) { *abort_flag = 1; atomicExch(err, 3); }
    tc_fence_after();
    const int quarter = warp & 3;                    // lanes this warp may read
    const int row = quarter * 32 + lane;             // accumulator row = weight row of the tile
    if (ok && num_splits == 1) {
      tile_epilogue<BT>(tmem_base, quarter, lane, n0, m0, min(BT, M - m0), M, N, ldo, bias, out, out_mode, fuse, fuse_smem);
    } else if (num_splits > 1 && ok) {
      // this part's partial tile -> own shared memory (the ring is free: every MMA has
      // completed), as [token column][weight row] floats
      float* red = reinterpret_cast<float*>(tiles);
      const int cols = min(BT, M - m0);
#pragma unroll 1
      for (int c = 0; c < BT / 16; ++c) {
        if (c * 16 >= cols) break;
        uint32_t r[16];
        tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c * 16), r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (c * 16 + j < cols) red[(c * 16 + j) * BLOCK_N_OUT + row] = __uint_as_float(r[j]);
      }
    }
  }
  if (num_splits > 1) {
    // ---- all parts of the tile have their partial in shared memory ----
    __syncwarp();
    cluster_sync_all();
    if (warp >= 2 && !*abort_flag) {
      // 32 lanes x 4 consecutive weight rows cover the 128 rows with 16-byte loads.  This CTA
      // owns the token columns j with j % parts == its rank; its four epilogue warps take
      // them in turn.  Parts are added in order 0, 1, 2, ...
      const int et = threadIdx.x - 64;
      const int r4 = (et & 31) * 4, cg = et >> 5;
      const int nn = n0 + r4;
      const int cols = min(BT, M - m0);
      const uint32_t red_local = smem_u32(tiles);
      const bool vec_ok = (nn + 3 < N) && ((ldo & 3) == 0) && (((uintptr_t)out & 15) == 0);
      float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
      if (bias != nullptr) {
        bv.x = nn < N ? bias[nn] : 0.f; bv.y = nn + 1 < N ? bias[nn + 1] : 0.f;
        bv.z = nn + 2 < N ? bias[nn + 2] : 0.f; bv.w = nn + 3 < N ? bias[nn + 3] : 0.f;
      }
      // Four columns a warp at a time, every load of the four (the parts' sums through the cluster's
      // shared memory, the residual's old values) issued before the first is used: with 128 or 256
      // token columns a tile this loop is bound by the latency of its loads, not their number.
      constexpr int U = BT > 128 ? 8 : BT > 64 ? 4 : 1;
      const bool add_vec = out_mode == TC_OUT_ADD_F32 && vec_ok;
      const int step = num_splits * 4;
      for (int j0 = split + num_splits * cg; j0 < cols; j0 += step * U) {
        float4 v[U], old[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int j = j0 + u * step;
          v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          old[u] = v[u];
          if (U > 1 && add_vec && j < cols) old[u] = __ldcg(reinterpret_cast<const float4*>((const float*)out + (size_t)(m0 + j) * ldo + nn));
        }
        for (int sp = 0; sp < num_splits; ++sp) {       // parts are added in the order 0, 1, 2, ...
          float4 t[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int j = j0 + u * step;
            t[u] = j < cols ? dsmem_ld4(dsmem_addr(red_local + (uint32_t)((j * BLOCK_N_OUT + r4) * 4), (uint32_t)sp))
                            : make_float4(0.f, 0.f, 0.f, 0.f);
          }
#pragma unroll
          for (int u = 0; u < U; ++u) { v[u].x += t[u].x; v[u].y += t[u].y; v[u].z += t[u].z; v[u].w += t[u].w; }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int j = j0 + u * step;
          if (j < cols)
            tc_finish_column<BT>(v[u], j, r4, et & 31, n0, m0, N, ldo, bv, out, out_mode, fuse, fuse_smem, vec_ok,
                                 U > 1 && add_vec, old[u]);
        }
      }
    }
    __syncwarp();
    cluster_sync_all();      // nobody leaves while another part still reads its shared memory
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

// ------------------------------------------------------------------ persistent variant (128 or 256 tokens a tile)
// One CTA an SM walks over the tiles (tile index = blockIdx.x, + gridDim.x, ...; token tiles of
// the same weight rows are neighbours, so CTAs that run together share weight tiles in L2).
// Tensor memory holds two accumulators: while the epilogue warps drain one, the MMA thread
// fills the other, and the TMA producer runs ahead through the ring across tile borders.
// The tiles behind the last full wave of CTAs are cut narrower along the tokens, so that
// there are about as many of them as CTAs: the last wave then takes bt / BT of a full
// wave's time instead of a whole one with most CTAs idle.  No partial sums, no fix-up:
// a narrow tile is a whole tile of its own.
struct TcTail {
  int first;         // index of the first narrow tile = number of tiles of full width
  int bt;            // tokens a narrow tile (a multiple of 16, <= BT)
  int n_first;       // weight-row tile the narrow tiles begin in
  int t0_first;      // first token that is not covered by full-width tiles there
  int count_first;   // narrow tiles in that weight-row tile
  int per_n;         // narrow tiles in every weight-row tile after it
};
struct TcTileAt { int n0, m0, bt; };
__device__ __forceinline__ TcTileAt tc_tile_at(int tile, int tiles_m, int BT, const TcTail& t) {
  if (tile < t.first) return {(tile / tiles_m) * BLOCK_N_OUT, (tile % tiles_m) * BT, BT};
  int idx = tile - t.first;
  if (idx < t.count_first) return {t.n_first * BLOCK_N_OUT, t.t0_first + idx * t.bt, t.bt};
  idx -= t.count_first;
  return {(t.n_first + 1 + idx / t.per_n) * BLOCK_N_OUT, (idx % t.per_n) * t.bt, t.bt};
}


template <int BT>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                          const __grid_constant__ CUtensorMap map_a_tail, const float* __restrict__ bias,
                          void* __restrict__ out, int out_mode, int M, int N, int K,
                          int ldo, int* __restrict__ err, int tiles_m, int num_tiles, const TcTail tail) {
  using Cfg = TcConfig<BT>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* tiles = smem;
  uint64_t* bars = (uint64_t*)(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
  uint64_t* full_bar = bars;                         // [STAGES]
  uint64_t* empty_bar = bars + Cfg::STAGES;          // [STAGES]
  uint64_t* acc_full = bars + 2 * Cfg::STAGES;       // [2]
  uint64_t* acc_empty = bars + 2 * Cfg::STAGES + 2;  // [2]
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * Cfg::STAGES + 4);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (K + BLOCK_K - 1) / BLOCK_K;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&acc_full[i]), 1);
      mbar_init(smem_u32(&acc_empty[i]), 4);       // one arrival per epilogue warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a_tail) : "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 2 * BT);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  rl_pdl_trigger();
  if (warp == 0) {
    if (lane == 0) {
      // ---------------- producer ----------------
      int it = 0;                                   // k-blocks issued so far, over all tiles
      bool waited = false, ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const TcTileAt at = tc_tile_at(tile, tiles_m, BT, tail);
        const int n0 = at.n0, m0 = at.m0;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % Cfg::STAGES;
          const uint32_t phase = (it / Cfg::STAGES) & 1;
          if (it >= Cfg::STAGES && !mbar_wait(smem_u32(&empty_bar[s]), phase ^ 1, abort_flag)) {
            if (!*abort_flag) { *abort_flag = 1; atomicExch(err, 1); }
            ok = false;
            break;
          }
          const uint32_t fb = smem_u32(&full_bar[s]);
          mbar_expect_tx(fb, (BLOCK_N_OUT + at.bt) * BLOCK_K * 2);
          uint8_t* st = tiles + (size_t)s * Cfg::STAGE_BYTES;
          tma_load_2d(smem_u32(st), &map_w, fb, kb * BLOCK_K, n0);
          // weights may be requested before the preceding kernels have finished, activations not
          if (!waited) { rl_pdl_wait(); waited = true; }
          uint8_t* sa = st + BLOCK_N_OUT * BLOCK_K * 2;
          tma_load_2d(smem_u32(sa), at.bt == BT ? &map_a : &map_a_tail, fb, kb * BLOCK_K, m0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer ----------------
      int it = 0, t = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++t) {
        const uint32_t idesc = make_idesc(BLOCK_N_OUT, tc_tile_at(tile, tiles_m, BT, tail).bt);
        const int buf = t & 1;
        const uint32_t acc_phase = (t >> 1) & 1;
        if (t >= 2 && !mbar_wait(smem_u32(&acc_empty[buf]), acc_phase ^ 1, abort_flag)) {   // epilogue done with this accumulator
          if (!*abort_flag) { *abort_flag = 1; atomicExch(err, 4); }
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * BT);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % Cfg::STAGES;
          const uint32_t phase = (it / Cfg::STAGES) & 1;
          if (!mbar_wait(smem_u32(&full_bar[s]), phase, abort_flag)) {
            if (!*abort_flag) { *abort_flag = 1; atomicExch(err, 2); }
            ok = false;
            break;
          }
          tc_fence_after();
          uint8_t* st = tiles + (size_t)s * Cfg::STAGE_BYTES;
          const uint64_t da = make_smem_desc(smem_u32(st));
          const uint64_t db = make_smem_desc(smem_u32(st + BLOCK_N_OUT * BLOCK_K * 2));
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; ++k)
            umma_bf16(tmem_acc, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(smem_u32(&empty_bar[s]));
        }
        if (ok) umma_commit(smem_u32(&acc_full[buf]));
      }
    }
  } else {
    // ---------------- epilogue warps ----------------
    rl_pdl_wait();
    const int quarter = warp & 3;
    int t = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++t) {
      const int buf = t & 1;
      const uint32_t acc_phase = (t >> 1) & 1;
      const TcTileAt at = tc_tile_at(tile, tiles_m, BT, tail);
      if (!mbar_wait(smem_u32(&acc_full[buf]), acc_phase, abort_flag)) {
        if (!*abort_flag) { *abort_flag = 1; atomicExch(err, 3); }
        break;
      }
      tc_fence_after();
      tile_epilogue<BT>(tmem_base + (uint32_t)(buf * BT), quarter, lane, at.n0, at.m0, min(at.bt, M - at.m0), M, N, ldo, bias, out,
                        out_mode, TcFuse{}, nullptr);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));    // this warp has read the accumulator
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 2 * BT);
}


template <int BT>
static int launch_tc_persistent(const CUtensorMap& mw, const CUtensorMap& ma, const void* A, int lda, const float* bias,
                                void* out, int out_mode, int M, int N, int K, int ldo, int* err, cudaStream_t stream) {
  using Cfg = TcConfig<BT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel<BT>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    RL_REQUIRE(e == cudaSuccess, "rl_gemm_tc: cannot reserve %d bytes of shared memory: %s", Cfg::SMEM_BYTES, cudaGetErrorString(e));
    configured = true;
  }
  const int num_sms = rl_num_sms();
  const int tiles_m = (M + BT - 1) / BT, tiles_n = (N + BLOCK_N_OUT - 1) / BLOCK_N_OUT;
  const int total = tiles_m * tiles_n;
  // the tiles behind the last full wave: the narrowest token tile (from 64 tokens: below, the
  // weight tile's trip through shared memory takes longer than the products) that leaves no
  // more of them than there are CTAs
  TcTail tail = {total, BT, 0, 0, 0, 1};
  int num_tiles = total;
  const int full = (total / num_sms) * num_sms;
  if (full < total) {
    const int n_first = full / tiles_m, t0_first = (full % tiles_m) * BT;
    for (int bt = 64; bt < BT; bt += 16) {
      const int count_first = (M - t0_first + bt - 1) / bt, per_n = (M + bt - 1) / bt;
      const int cnt = count_first + (tiles_n - n_first - 1) * per_n;
      if (cnt <= num_sms) {
        tail = {full, bt, n_first, t0_first, count_first, per_n};
        num_tiles = full + cnt;
        break;
      }
    }
  }
  CUtensorMap ma_tail = ma;      // the same activations in boxes as tall as a narrow tile
  if (tail.bt != BT) {
    const int rc = tc_make_map(&ma_tail, A, M, K, lda, tail.bt);
    if (rc != RL_OK) return rc;
  }
  const int grid = num_tiles < num_sms ? num_tiles : num_sms;
  cudaError_t e = rl_launch_pdl(gemm_tc_persistent_kernel<BT>, dim3(grid), dim3(TC_THREADS), (size_t)Cfg::SMEM_BYTES, stream,
                                mw, ma, ma_tail, bias, out, out_mode, M, N, K, ldo, err, tiles_m, num_tiles, tail);
  if (e != cudaSuccess) {
    rl_set_error("rl_gemm_tc: launch of the persistent kernel failed: %s", cudaGetErrorString(e));
    return RL_ERR_CUDA;
  }
  return RL_OK;
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
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

// A row-major bf16 matrix [rows, cols] with row stride ld (elements), tiled in boxes
// of box_rows x 64 columns, 128-byte swizzle, zero fill outside.
int tc_make_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  RL_REQUIRE(enc != nullptr, "rl_gemm_tc: the driver does not provide cuTensorMapEncodeTiled");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BLOCK_K, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  RL_REQUIRE(r == CUDA_SUCCESS, "rl_gemm_tc: cuTensorMapEncodeTiled failed with %d (rows=%d cols=%d ld=%d box_rows=%d)",
             (int)r, rows, cols, ld, box_rows);
  return RL_OK;
}

template <int BT, bool DEEP>
static int launch_tc_as(const CUtensorMap& mw, const CUtensorMap& ma, const float* bias, void* out, int out_mode,
                     int M, int N, int K, int ldo, int* err, int splits, int kb_per_split, const TcFuse& fuse,
                     cudaStream_t stream) {
  using Cfg = TcConfig<BT, DEEP>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BT, DEEP>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    RL_REQUIRE(e == cudaSuccess, "rl_gemm_tc: cannot reserve %d bytes of shared memory: %s", Cfg::SMEM_BYTES, cudaGetErrorString(e));
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(splits * ((N + BLOCK_N_OUT - 1) / BLOCK_N_OUT), (M + BT - 1) / BT, 1);
  cfg.blockDim = dim3(TC_THREADS);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (g_rl_pdl_enabled) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (splits > 1) {     // the parts of a tile are the CTAs of one cluster
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = splits;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BT, DEEP>, mw, ma, bias, out, out_mode, M, N, K, ldo, err, kb_per_split, fuse);
  if (e != cudaSuccess) {
    rl_set_error("rl_gemm_tc: launch failed (%d parts): %s", splits, cudaGetErrorString(e));
    return RL_ERR_CUDA;
  }
  return RL_OK;
}


static int g_deep_rings = 1;
// 1 (default): the deep-ring variant where it was measured to pay; 0: never (for measurements)
extern "C" void rl_set_deep_rings(int enabled) { g_deep_rings = enabled ? 1 : 0; }

// The deep-ring variant where the whole grid fits two CTAs an SM (up to 64 tokens) and the product
// is not split over K, or the step has more than 32 tokens.  Measured on whole decode steps of the
// 8B shape (ms a step, rings off / on for every such product / on by this rule): one sequence
// 3.03 / 2.96 / 2.95, 8 sequences 3.18 / 3.23 / 3.18, 64 sequences 5.49 / 5.34 / 5.34.  With few
// tokens the split products (QKV, O, down) lose more by leaving no room for the next kernel's
// CTAs, which load their first weights while this one still runs, than their own rings gain.
template <int BT>
static int launch_tc(const CUtensorMap& mw, const CUtensorMap& ma, const float* bias, void* out, int out_mode,
                     int M, int N, int K, int ldo, int* err, int splits, int kb_per_split, const TcFuse& fuse,
                     cudaStream_t stream) {
  if constexpr (BT <= 64) {
    const long long ctas = (long long)splits * ((N + BLOCK_N_OUT - 1) / BLOCK_N_OUT) * ((M + BT - 1) / BT);
    if (g_deep_rings && (splits == 1 || BT == 64) && ctas <= 2LL * rl_num_sms())
      return launch_tc_as<BT, true>(mw, ma, bias, out, out_mode, M, N, K, ldo, err, splits, kb_per_split, fuse, stream);
  }
  return launch_tc_as<BT, false>(mw, ma, bias, out, out_mode, M, N, K, ldo, err, splits, kb_per_split, fuse, stream);
}

// 1 if the tensor-core kernel takes these operands: TMA needs 16-byte aligned bases
// and row strides that are multiples of 16 bytes.
extern "C" int rl_gemm_tc_supported(const void* A, const void* W, int M, int N, int K, int lda) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 8 != 0 || lda % 8 != 0 || lda < K) return 0;
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return 0;
  return 1;
}

static int token_tile(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256; }

// How many parts (1, 2, 4 or 8: the cluster size) the K range is cut into for M tokens.
// Up to 64 tokens: the smallest that gives about two CTAs an SM, with at least four 64-wide
// K blocks a part; products with 148 tiles or more are not split.  Above 64 tokens (one CTA
// an SM): the largest that still fits one wave of 148 CTAs - one SM cannot pull more than
// about 100 GB/s, so a product with few tiles needs more CTAs to stream its weights (4,096 x
// 14,336 weights, 256 tokens: 74 us as 32 tiles, 37 us in four parts each; 512 tokens: 80 us
// unsplit, 58 us in two parts; 4,096 x 4,096, 512 tokens: 29 us and 26 us) - but two parts of
// 256-token tiles that fill no more than two thirds of the SMs gain nothing over the unsplit
// tiles unless K is long (6,144 x 4,096, 256 tokens: 25 us and 26 us; 128-token tiles, 128
// tokens: 23 us and 18 us).  From half a wave of tiles on the persistent kernel takes the
// product unsplit.  Cluster sizes that are no power of two were measured too and lose: clusters
// of three do not all fit the GPCs at once (48 tiles in three parts: 41 us).
// A function of the shapes only, so a captured step keeps its grid.
extern "C" int rl_gemm_tc_splits(int M, int N, int K) {
  const int bt = token_tile(M);
  const int tiles = ((N + BLOCK_N_OUT - 1) / BLOCK_N_OUT) * ((M + bt - 1) / bt);
  const int total_kb = (K + BLOCK_K - 1) / BLOCK_K;
  const int sms = rl_num_sms();
  int splits = 1;
  if (bt > 64) {
    while (splits < 8 && tiles * splits * 2 <= sms && total_kb / (splits * 2) >= 4) splits *= 2;
    if (splits == 2 && tiles * 3 <= sms && bt > 128 && total_kb < 96) splits = 1;
    return splits;
  }
  // up to 64 tokens (three CTAs an SM).  From a sweep over the products of the three shapes measured
  // here (us at 8 tokens, unsplit / 2 / 4 / 8 parts): 48 tiles 19.8 / 14.3 / 11.2 / 10.6; 96 tiles
  // 21.3 / 19.1 / 18.1 / 21.0; 128 tiles 13.4 / 15.1 / 15.7 / 19.9; 172 tiles 33.5 / 29.4 / 32.6 / 36.2;
  // 224 tiles 37.5 / 42.8 / 42.7 / 45.6.  So: nearly a CTA an SM already - unsplit; a little more than
  // one wave of SMs - two parts, which still run together as one wave of three CTAs an SM (whole
  // steps of the Llama-2-7B shape: one sequence 2.75 -> 2.68 ms, sixteen 3.60 -> 3.58 ms).
  if (tiles >= sms) return (tiles * 2 <= sms * 12 / 5 && total_kb >= 8) ? 2 : 1;
  if (tiles * 8 >= sms * 7) return 1;
  while (splits < 8 && tiles * splits < 256 && total_kb / (splits * 2) >= 4) splits *= 2;
  return splits;
}

// A: [M, K] bf16, row stride lda; W: [N, K] bf16 contiguous; out: [M, N] with row stride
// ldo, bf16 (out_mode 0) or float (1 store, 2 add); out_mode 3: W's rows are (gate_0, up_0,
// gate_1, ...) and out is bf16 [M, N/2] = silu(gate) * up.  err: device int, set non-zero if a
// bounded wait inside the kernel ran out.  force_splits: 0 = number of K parts chosen
// from the shapes; 1 to 8 = as given (for measurements; the rule itself picks powers of two).
// RMSNorm folded in, both optional (null = not):
//  scale_partials [M, scale_count] float: A is `x * norm weight`, not yet divided by the rms
//    of x; the sums of squares of x's rows come in scale_count pieces a row, and row m of
//    the product is multiplied by rsqrt(sum / K + scale_eps) before the bias.
//  norm_weight [N] float, norm_out [M, ld_norm] bf16, norm_partials [M, 4 * ceil(N / 128)]
//    float (out_mode 2 only): besides out += product, norm_out = bf16(out * norm_weight) and
//    the sums of squares of out's rows in 4 * ceil(N / 128) pieces a row, for the next product.
static int gemm_tc_run(const void* A, const void* W, const float* bias, void* out, int out_mode, int M, int N,
                       int K, int lda, int ldo, int* err, int force_splits, TcFuse fuse, cudaStream_t stream) {
  const float* scale_partials = fuse.scale_partials;
  const float* norm_weight = fuse.norm_weight;
  RL_REQUIRE(rl_gemm_tc_supported(A, W, M, N, K, lda), "rl_gemm_tc: operands not supported (M=%d N=%d K=%d lda=%d; K and lda "
             "must be multiples of 8 and the bases 16-byte aligned)", M, N, K, lda);
  RL_REQUIRE(out_mode >= 0 && out_mode <= 4, "rl_gemm_tc: unknown output mode %d", out_mode);
  RL_REQUIRE(out_mode != TC_OUT_SWIGLU || N % 2 == 0, "rl_gemm_tc: the SwiGLU epilogue needs an even number of weight rows, got %d", N);
  RL_REQUIRE(ldo >= (out_mode == TC_OUT_SWIGLU ? N / 2 : N) && err != nullptr, "rl_gemm_tc: bad output stride or null error word");
  RL_REQUIRE(force_splits >= 0 && force_splits <= 8, "rl_gemm_tc: the number of K parts must be 1 to 8 (0: chosen from the shapes), got %d", force_splits);
  RL_REQUIRE(scale_partials == nullptr || fuse.scale_count > 0, "rl_gemm_tc: row scales without their sums");
  RL_REQUIRE(norm_weight == nullptr || (out_mode == TC_OUT_ADD_F32 && fuse.norm_out != nullptr && fuse.norm_partials != nullptr && fuse.ld_norm >= N),
             "rl_gemm_tc: the norm for the next product needs the add-into-residual mode, its two outputs and ld_norm >= N");
  fuse.norm_count = 4 * ((N + BLOCK_N_OUT - 1) / BLOCK_N_OUT);
  const int bt = token_tile(M);
  RL_REQUIRE((scale_partials == nullptr && norm_weight == nullptr) || bt <= 64,
             "rl_gemm_tc: a norm rides in the epilogue only for up to 64 tokens, got %d", M);
  const int total_kb = (K + BLOCK_K - 1) / BLOCK_K;
  int splits = force_splits > 0 ? force_splits : rl_gemm_tc_splits(M, N, K);
  while (splits > 1 && (splits - 1) * ((total_kb + splits - 1) / splits) >= total_kb)                // no part is empty
    splits = (splits & (splits - 1)) == 0 ? splits / 2 : splits - 1;                                 // (a power of two stays one)
  RL_REQUIRE(out_mode != TC_OUT_ROPE_KV || (splits > 1 && bt <= 64),
             "rl_gemm_tc_qkv_rope: the rotation rides only in the cluster epilogue (up to 64 tokens, K in 2 or more parts); "
             "M=%d N=%d K=%d give %d part(s)", M, N, K, splits);
  const int kb_per = (total_kb + splits - 1) / splits;
  CUtensorMap mw, ma;
  int rc = tc_make_map(&mw, W, N, K, K, BLOCK_N_OUT);
  if (rc != RL_OK) return rc;
  rc = tc_make_map(&ma, A, M, K, lda, bt);
  if (rc != RL_OK) return rc;
  switch (bt) {
    case 16: return launch_tc<16>(mw, ma, bias, out, out_mode, M, N, K, ldo, err, splits, kb_per, fuse, stream);
    case 32: return launch_tc<32>(mw, ma, bias, out, out_mode, M, N, K, ldo, err, splits, kb_per, fuse, stream);
    case 64: return launch_tc<64>(mw, ma, bias, out, out_mode, M, N, K, ldo, err, splits, kb_per, fuse, stream);
    default: break;
  }
  if (splits > 1) {       // few tiles of many tokens: the parts of a tile as a cluster, as for few tokens
    if (bt == 128) return launch_tc<128>(mw, ma, bias, out, out_mode, M, N, K, ldo, err, splits, kb_per, fuse, stream);
    return launch_tc<256>(mw, ma, bias, out, out_mode, M, N, K, ldo, err, splits, kb_per, fuse, stream);
  }
  if (bt == 128) return launch_tc_persistent<128>(mw, ma, A, lda, bias, out, out_mode, M, N, K, ldo, err, stream);
  return launch_tc_persistent<256>(mw, ma, A, lda, bias, out, out_mode, M, N, K, ldo, err, stream);
}

extern "C" int rl_gemm_tc(const void* A, const void* W, const float* bias, void* out, int out_mode, int M, int N,
                          int K, int lda, int ldo, int* err, int force_splits, const float* scale_partials,
                          int scale_count, float scale_eps, const float* norm_weight, void* norm_out, int ld_norm,
                          float* norm_partials, cudaStream_t stream) {
  RL_REQUIRE(out_mode != TC_OUT_ROPE_KV, "rl_gemm_tc: the rotation epilogue has its own entry point, rl_gemm_tc_qkv_rope");
  TcFuse fuse = {};
  fuse.scale_partials = scale_partials; fuse.scale_count = scale_count; fuse.scale_eps = scale_eps;
  fuse.norm_weight = norm_weight; fuse.norm_out = (__nv_bfloat16*)norm_out; fuse.ld_norm = ld_norm;
  fuse.norm_partials = norm_partials;
  return gemm_tc_run(A, W, bias, out, out_mode, M, N, K, lda, ldo, err, force_splits, fuse, stream);
}

// 1 if rl_gemm_tc_qkv_rope takes the shape: head size 128 or 64, the whole head rotated, a step
// of up to 64 tokens whose product is split over K (a function of the shapes only).
extern "C" int rl_gemm_tc_qkv_rope_supported(int M, int num_heads, int num_kv_heads, int head_dim, int rotary_dim, int K) {
  if ((head_dim != 128 && head_dim != 64) || rotary_dim != head_dim || M <= 0 || M > 64 || K % 8 != 0) return 0;
  const int N = (num_heads + 2 * num_kv_heads) * head_dim;
  const int total_kb = (K + BLOCK_K - 1) / BLOCK_K;
  int splits = rl_gemm_tc_splits(M, N, K);
  while (splits > 1 && (splits - 1) * ((total_kb + splits - 1) / splits) >= total_kb) splits /= 2;
  return splits > 1;
}

// The QKV product of an attention layer with rotary encoding and cache write in its
// epilogue.  W: [(H + 2G) * head_dim, K] (query heads, key heads, value heads; head_dim 128 or
// 64); out: [M, ldo] bf16, of which the H query heads are written (rotated); keys (rotated) and
// values go to k_pool / v_pool [pages, G, RL_PAGE, head_dim] at each token's position (null
// pools: they are not stored at all).  positions, slot_of_token: [M]; inv_freq: [head_dim / 2]
// float.  scale_*: as in rl_gemm_tc.  Refused unless rl_gemm_tc_qkv_rope_supported(...).
extern "C" int rl_gemm_tc_qkv_rope(const void* A, const void* W, const float* bias, void* out, int M, int K, int lda, int ldo,
                                   int* err, const float* scale_partials, int scale_count, float scale_eps,
                                   const int* positions, const int* slot_of_token, const int* page_table, int max_pages,
                                   const float* inv_freq, int interleaved, int num_heads, int num_kv_heads, int head_dim,
                                   void* k_pool, void* v_pool, cudaStream_t stream) {
  RL_REQUIRE(num_heads > 0 && num_kv_heads > 0 && positions != nullptr && inv_freq != nullptr,
             "rl_gemm_tc_qkv_rope: bad head counts or null positions / frequencies");
  RL_REQUIRE(head_dim == 128 || head_dim == 64, "rl_gemm_tc_qkv_rope: head size %d; 128 and 64 are taken", head_dim);
  RL_REQUIRE((k_pool == nullptr) == (v_pool == nullptr), "rl_gemm_tc_qkv_rope: give both pools or neither");
  RL_REQUIRE(k_pool == nullptr || (slot_of_token != nullptr && page_table != nullptr && max_pages > 0),
             "rl_gemm_tc_qkv_rope: the cache write needs slots and the page table");
  RL_REQUIRE(((uintptr_t)out & 7) == 0 && ldo % 4 == 0 && ((uintptr_t)k_pool & 7) == 0 && ((uintptr_t)v_pool & 7) == 0,
             "rl_gemm_tc_qkv_rope: output and pools must be 8-byte aligned, ldo a multiple of 4");
  const int N = (num_heads + 2 * num_kv_heads) * head_dim;
  TcFuse fuse = {};
  fuse.head_dim = head_dim;
  fuse.scale_partials = scale_partials; fuse.scale_count = scale_count; fuse.scale_eps = scale_eps;
  fuse.positions = positions; fuse.slot_of_token = slot_of_token; fuse.page_table = page_table; fuse.max_pages = max_pages;
  fuse.inv_freq = inv_freq; fuse.interleaved = interleaved; fuse.num_heads = num_heads; fuse.num_kv_heads = num_kv_heads;
  fuse.k_pool = (__nv_bfloat16*)k_pool; fuse.v_pool = (__nv_bfloat16*)v_pool;
  return gemm_tc_run(A, W, bias, out, TC_OUT_ROPE_KV, M, N, K, lda, ldo, err, 0, fuse, stream);
}
