// Device-side pieces of the tensor-core matrix products (gemm_tc.cu):
// output modes, the optional norm / rotary work of an epilogue, PTX wrappers for mbarriers,
// TMA, tensor memory and tcgen05.mma, the shared-memory and instruction descriptors, and the
// finishing of one token column of a tile.
#pragma once
#include <cuda.h>

#include "common.cuh"

enum { TC_OUT_BF16 = 0, TC_OUT_F32 = 1, TC_OUT_ADD_F32 = 2, TC_OUT_SWIGLU = 3, TC_OUT_ROPE_KV = 4 };

// silu(g) * u for a result that is stored in bf16: the fast exponential and division are
// accurate to a few units in the last place of a float, far below bf16's rounding step
__device__ __forceinline__ float silu_mul(float g, float u) { return g * __fdividef(1.0f, 1.0f + __expf(-g)) * u; }

// The optional norm work of an epilogue.
struct TcFuse {
  // consumer: sums of squares of the input rows, [M, scale_count]; the accumulator row of
  // token m is multiplied by rsqrt(sum_i scale_partials[m][i] / K + scale_eps).  null: none
  const float* scale_partials;
  int scale_count;
  float scale_eps;
  // producer (add-into-residual only): norm_out[m][n] = bf16(new residual * norm_weight[n]),
  // norm_partials[m][4 * tile + w] = sum of (new residual)^2 over columns 32 w .. 32 w + 31
  // of the tile, norm_count = 4 * tiles numbers a token.  null: none
  const float* norm_weight;
  __nv_bfloat16* norm_out;
  int ld_norm;
  float* norm_partials;
  int norm_count;
  // rotary encoding + cache write (out_mode TC_OUT_ROPE_KV only)
  const int* positions;         // [M]
  const int* slot_of_token;     // [M]
  const int* page_table;        // [slots, max_pages]
  int max_pages;
  const float* inv_freq;        // [head_dim / 2]
  int interleaved;              // pairs (2i, 2i+1) instead of (i, i + head_dim / 2)
  int num_heads, num_kv_heads;
  int head_dim;                 // 128 (a tile of 128 output columns is one head) or 64 (two heads)
  __nv_bfloat16* k_pool;        // [pages, kv_heads, RL_PAGE, head_dim]; null: keys and values are not stored
  __nv_bfloat16* v_pool;
};

static constexpr int BLOCK_N_OUT = 128;   // weight rows per CTA (MMA M)
static constexpr int BLOCK_K = 64;        // bf16 elements per stage along K = one 128-byte swizzle row
static constexpr int UMMA_K = 16;
static constexpr int TC_THREADS = 192;    // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-5: epilogue
static constexpr uint32_t WAIT_LIMIT = 1u << 22;

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Bounded wait.  Returns false when the limit ran out or another role gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float tc_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- thread-block cluster ----
__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t cluster_size() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory location in the cluster's CTA `rank`
__device__ __forceinline__ uint32_t dsmem_addr(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ float4 dsmem_ld4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bf16)
// and swizzled with the 128-byte pattern: start address / 16 in bits 0-13, leading
// byte offset (unused for this layout, set to 16 bytes) in bits 16-29, stride between
// groups of 8 rows = 1024 bytes in bits 32-45, descriptor version 1 in bits 46-47,
// layout type 2 (128-byte swizzle) in bits 61-63.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor for kind::f16: float accumulator (bits 4-5 = 1), A and B bf16
// (bits 7-9 and 10-12 = 1), both K-major (bits 15, 16 = 0), N/8 in bits 17-22, M/16 in
// bits 24-28.
__host__ __device__ constexpr uint32_t make_idesc(int mma_m, int mma_n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(mma_n >> 3) << 17) | ((uint32_t)(mma_m >> 4) << 24);
}


// the 128 epilogue threads among themselves (barrier 1; barrier 0 is __syncthreads).  Used
// only where all four epilogue warps arrive whatever happens (before their first bounded wait).
__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Row scales of the tile's tokens from the producer's sums of squares, into rs[BT] in shared
// memory.  Epilogue warp q takes tokens q, q + 4, ...; a token's pieces are summed over the
// lanes (32 neighbouring numbers a load, all tokens' loads of a round issued together) and
// then over the warp: the same order everywhere.  Ends with the epilogue warps' barrier.
template <int BT>
__device__ __forceinline__ void epilogue_row_scales(const TcFuse& f, int m0, int M, int K, int q, int lane, float* rs) {
  static_assert(BT <= 64, "row scales are made in the kernel for up to 64 tokens");
  constexpr int PER = BT / 4;
  float acc[PER];
#pragma unroll
  for (int u = 0; u < PER; ++u) acc[u] = 0.f;
  for (int i = lane; i < f.scale_count; i += 32) {
    float v[PER];
#pragma unroll
    for (int u = 0; u < PER; ++u) {
      const int m = m0 + q + 4 * u;
      v[u] = m < M ? f.scale_partials[(size_t)m * f.scale_count + i] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < PER; ++u) acc[u] += v[u];
  }
#pragma unroll
  for (int u = 0; u < PER; ++u) {
    const float sum = tc_warp_sum(acc[u]);
    if (lane == 0) rs[q + 4 * u] = rsqrtf(sum / (float)K + f.scale_eps);
  }
  epilogue_sync();
}

// A row-major bf16 matrix [rows, cols] with row stride ld (elements), tiled in boxes of
// box_rows x 64 columns, 128-byte swizzle, zero fill outside (host; defined in gemm_tc.cu).
int tc_make_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows);

// One token column of a finished tile: v = the sums of output features nn .. nn + 3 (nn = n0 + r4,
// r4 = 4 * lane: a warp holds all 128 features of the tile) of token m0 + j.  Applies the row
// scale of a norm that this product finishes, the bias, and stores in the asked form: bf16,
// float, added into the float residual (with the start of the next norm), SwiGLU of
// interleaved gate / up rows, or rotary encoding with the write into the paged cache.
// fuse_smem: [0, BT) row scales, then the tokens' positions and cache rows (rotary mode).
// have_old, old_residual (add mode with vec_ok only): the four residual values, if already loaded.
template <int BT>
__device__ __forceinline__ void tc_finish_column(float4 v, int j, int r4, int lane32, int n0, int m0, int N, int ldo,
                                                 float4 bv, void* __restrict__ out, int out_mode, const TcFuse& fuse,
                                                 const float* fuse_smem, bool vec_ok, bool have_old = false,
                                                 float4 old_residual = make_float4(0.f, 0.f, 0.f, 0.f)) {
  const int nn = n0 + r4;
  const int et = lane32;          // lane within the warp
  do {
        if (fuse.scale_partials != nullptr) { const float rj = fuse_smem[j]; v.x *= rj; v.y *= rj; v.z *= rj; v.w *= rj; }
        v.x += bv.x; v.y += bv.y; v.z += bv.z; v.w += bv.w;
        if (out_mode == TC_OUT_ROPE_KV) {
          // the tile holds one head of 128 (or two of 64) of (query heads, key heads, value heads);
          // this lane holds dimensions d .. d + 3 of its head for token m0 + j
          const int hd = fuse.head_dim, half = hd >> 1;
          const int head = nn / hd, d = nn - head * hd;
          const int H = fuse.num_heads, G = fuse.num_kv_heads;
          const int* tok_pos = (const int*)(fuse_smem + BT);
          const int* tok_row = tok_pos + BT;
          float e[4] = {v.x, v.y, v.z, v.w};
          // (all lanes take part in the exchange below, also those of a head beyond the last)
          if (head < H + G || hd < BLOCK_N_OUT) {
            const bool rotate = head < H + G;
            const float pos = (float)tok_pos[j];
            if (fuse.interleaved) {             // pairs (d, d + 1) and (d + 2, d + 3), frequencies d / 2 and d / 2 + 1
              if (rotate) {
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                  float sn, cs;
                  sincosf(pos * fuse.inv_freq[d / 2 + u], &sn, &cs);
                  const float x0 = e[2 * u], x1 = e[2 * u + 1];
                  e[2 * u] = x0 * cs - x1 * sn;
                  e[2 * u + 1] = x0 * sn + x1 * cs;
                }
              }
            } else {                            // pairs (i, i + hd / 2): the partner sits hd / 8 lanes away
              const bool low = d < half;
              const int away = hd >> 3;
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const float other = __shfl_xor_sync(0xffffffffu, e[u], away);
                if (rotate) {
                  float sn, cs;
                  sincosf(pos * fuse.inv_freq[(d & (half - 1)) + u], &sn, &cs);
                  e[u] = low ? e[u] * cs - other * sn : other * sn + e[u] * cs;
                }
              }
            }
          }
          __nv_bfloat162 lo = __floats2bfloat162_rn(e[0], e[1]), hi = __floats2bfloat162_rn(e[2], e[3]);
          const uint2 pk = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
          if (head < H) {
            *reinterpret_cast<uint2*>((__nv_bfloat16*)out + (size_t)(m0 + j) * ldo + nn) = pk;
          } else if (fuse.k_pool != nullptr && head < H + 2 * G) {
            const bool is_v = head >= H + G;
            const int g = head - (is_v ? H + G : H);
            __nv_bfloat16* pool = is_v ? fuse.v_pool : fuse.k_pool;
            *reinterpret_cast<uint2*>(pool + ((size_t)tok_row[j] + (size_t)g * RL_PAGE) * hd + d) = pk;
          }
          break;
        }
        if (out_mode == TC_OUT_SWIGLU) {      // v = (gate, up, gate, up) of output columns nn/2 and nn/2 + 1
          __nv_bfloat16* ob = (__nv_bfloat16*)out + (size_t)(m0 + j) * ldo + (nn >> 1);
          if (nn + 1 < N) ob[0] = __float2bfloat16_rn(silu_mul(v.x, v.y));
          if (nn + 3 < N) ob[1] = __float2bfloat16_rn(silu_mul(v.z, v.w));
          break;
        }
        const size_t o = (size_t)(m0 + j) * ldo + nn;
        if (vec_ok) {
          if (out_mode == TC_OUT_BF16) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
            uint2 pk = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
            *reinterpret_cast<uint2*>((__nv_bfloat16*)out + o) = pk;
          } else if (out_mode == TC_OUT_F32) {
            *reinterpret_cast<float4*>((float*)out + o) = v;
          } else {
            // (the caller may have fetched the residual's values already, with other columns' loads)
            float4 old = have_old ? old_residual : *reinterpret_cast<const float4*>((float*)out + o);
            old.x += v.x; old.y += v.y; old.z += v.z; old.w += v.w;
            *reinterpret_cast<float4*>((float*)out + o) = old;
            v = old;
          }
        } else {
          float e[4] = {v.x, v.y, v.z, v.w};
          for (int u = 0; u < 4; ++u) {
            if (nn + u >= N) { e[u] = 0.f; continue; }
            if (out_mode == TC_OUT_BF16) ((__nv_bfloat16*)out)[o + u] = __float2bfloat16_rn(e[u]);
            else if (out_mode == TC_OUT_F32) ((float*)out)[o + u] = e[u];
            else { e[u] += ((float*)out)[o + u]; ((float*)out)[o + u] = e[u]; }
          }
          v = make_float4(e[0], e[1], e[2], e[3]);
        }
        if (fuse.norm_weight != nullptr && out_mode == TC_OUT_ADD_F32) {
          // v = the new residual of token m0 + j in columns nn .. nn + 3 (0 beyond N); this warp
          // holds all 128 columns of the tile for this token
          const float e[4] = {v.x, v.y, v.z, v.w};
          for (int u = 0; u < 4; ++u)
            if (nn + u < N)
              fuse.norm_out[(size_t)(m0 + j) * fuse.ld_norm + nn + u] = __float2bfloat16_rn(e[u] * fuse.norm_weight[nn + u]);
          const float sq = tc_warp_sum((v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w));
          // one number for the whole tile here; the places of the other three warps hold 0
          if (et < 4)
            fuse.norm_partials[(size_t)(m0 + j) * fuse.norm_count + 4 * (n0 / BLOCK_N_OUT) + et] = et == 0 ? sq : 0.f;
        }
  } while (false);
}
