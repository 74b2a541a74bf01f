// Prefill attention: the step's query tokens (whole prompts or chunks of them, several
// sequences of unequal length packed one after another) attend causally to their
// sequence's keys and values in the paged bf16 cache, on the tensor cores.
//
// Math (SimonWaldherr/RustyLLM src/model.rs:7239-7294 with 5807-5869): query head h uses KV head
// g = h / (H/G); score = (q . k_t) / sqrt(head_dim) for t <= the query's position
// (t >= position + 1 - window under a window); streaming softmax with running
// (max, sum, output) in float; out = sum p_t v_t.  The reference scans one query at a
// time (its batched prefill too, src/model.rs:9985-10036); here 64 queries of one head
// share each 64-key tile.
//
// One CTA = 64 consecutive query tokens of one sequence and one query head; 4 warps of
// 16 query rows.  A key tile is exactly one cache page (64 positions of one KV head,
// contiguous), copied to shared memory with cp.async (two buffers, 16-byte chunks
// XOR-swizzled by row so that ldmatrix is conflict-free).  S = Q K^T and O += P V run on
// mma.sync m16n8k16 (bf16 in, float accumulate); rows of a page beyond the sequence's
// length are zero-filled on the way in, so stale contents of a reused page are never seen.
#include <math.h>

#include "common.cuh"

#define PF_WARPS 4
#define PF_QTILE 64     // query rows per CTA
#define PF_KTILE 64     // keys per tile = RL_PAGE

__device__ __forceinline__ void pf_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void pf_ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void pf_ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// 16-byte asynchronous copy; src_bytes = 0 writes zeros instead of reading
__device__ __forceinline__ void pf_cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void pf_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void pf_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t pf_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int HD>
__global__ void __launch_bounds__(PF_WARPS * 32)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, int ldq, const __nv_bfloat16* __restrict__ k_pool,
                         const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ page_table, int max_pages,
                         const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slots,
                         const int* __restrict__ kv_lens, int num_seqs, __nv_bfloat16* __restrict__ out, int ldo,
                         int H, int G, float scale_log2e, int window) {
  constexpr int ROW_BYTES = HD * 2;
  constexpr int CHUNKS = HD / 8;                   // 16-byte chunks per row
  constexpr int TILE_BYTES = PF_KTILE * ROW_BYTES;
  constexpr int NT_S = PF_KTILE / 8;               // score n-tiles per key tile
  constexpr int NT_O = HD / 8;                     // output n-tiles
  extern __shared__ __align__(128) uint8_t pf_smem[];   // [2 buffers][K tile | V tile]
  __shared__ int s_seq, s_tile;

  rl_pdl_trigger();
  rl_pdl_wait();
  // ---- which sequence and which of its query tiles (heaviest tiles first) ----
  if (threadIdx.x == 0) {
    int t = (int)(gridDim.x - 1 - blockIdx.x), b = 0;
    for (; b < num_seqs; ++b) {
      const int tiles = (cu_seqlens[b + 1] - cu_seqlens[b] + PF_QTILE - 1) / PF_QTILE;
      if (t < tiles) break;
      t -= tiles;
    }
    s_seq = b; s_tile = t;
  }
  __syncthreads();
  const int b = s_seq;
  if (b >= num_seqs) return;                       // the grid is sized exactly; defensive only
  const int h = blockIdx.y, gkv = h / (H / G);
  const int row0 = cu_seqlens[b], q_len = cu_seqlens[b + 1] - row0, kv_len = kv_lens[b];
  const int start_pos = kv_len - q_len;            // position of the sequence's first query token
  const int qt0 = s_tile * PF_QTILE;               // first query (within the sequence's step) of this CTA
  const int rows_here = min(PF_QTILE, q_len - qt0);
  const int* pages = page_table + (size_t)seq_slots[b] * max_pages;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int r_lo = warp * 16 + g, r_hi = r_lo + 8;          // this lane's two query rows within the tile
  const int pos_lo = start_pos + qt0 + r_lo, pos_hi = pos_lo + 8;
  const int last_pos = start_pos + qt0 + rows_here - 1;     // last query position of the CTA
  int first_key = 0;
  if (window > 0) first_key = max(0, start_pos + qt0 + 1 - window);
  const int kt_begin = first_key / PF_KTILE, kt_end = last_pos / PF_KTILE + 1;

  // ---- Q fragments straight from global memory ----
  uint32_t qf[HD / 16][4];
  {
    const __nv_bfloat16* qlo = q + (size_t)(row0 + qt0 + r_lo) * ldq + (size_t)h * HD;
    const __nv_bfloat16* qhi = qlo + (size_t)8 * ldq;
    const bool vlo = r_lo < rows_here, vhi = r_hi < rows_here;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      qf[ks][0] = vlo ? *reinterpret_cast<const uint32_t*>(qlo + 16 * ks + 2 * t4) : 0u;
      qf[ks][1] = vhi ? *reinterpret_cast<const uint32_t*>(qhi + 16 * ks + 2 * t4) : 0u;
      qf[ks][2] = vlo ? *reinterpret_cast<const uint32_t*>(qlo + 16 * ks + 2 * t4 + 8) : 0u;
      qf[ks][3] = vhi ? *reinterpret_cast<const uint32_t*>(qhi + 16 * ks + 2 * t4 + 8) : 0u;
    }
  }

  float acc[NT_O][4];
#pragma unroll
  for (int j = 0; j < NT_O; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(pf_smem);
  const size_t page_stride = (size_t)G * RL_PAGE * HD;
  const size_t head_off = (size_t)gkv * RL_PAGE * HD;

  auto load_tile = [&](int kt, int buf) {
    const size_t base = (size_t)pages[kt] * page_stride + head_off;
    const uint32_t kdst = smem_base + buf * 2 * TILE_BYTES, vdst = kdst + TILE_BYTES;
    const int valid_rows = kv_len - kt * PF_KTILE;           // rows beyond hold anything: zero-fill
    for (int c = threadIdx.x; c < PF_KTILE * CHUNKS; c += PF_WARPS * 32) {
      const int r = c / CHUNKS, ch = c % CHUNKS;
      const uint32_t off = (uint32_t)r * ROW_BYTES + (uint32_t)((ch ^ (r & 7)) * 16);
      const int bytes = r < valid_rows ? 16 : 0;
      pf_cp_async16(kdst + off, k_pool + base + (size_t)r * HD + ch * 8, bytes);
      pf_cp_async16(vdst + off, v_pool + base + (size_t)r * HD + ch * 8, bytes);
    }
  };

  load_tile(kt_begin, 0);
  pf_commit();

  for (int kt = kt_begin; kt < kt_end; ++kt) {
    const int buf = (kt - kt_begin) & 1;
    pf_wait<0>();
    __syncthreads();                                  // tile kt has landed; everyone is done with the other buffer
    if (kt + 1 < kt_end) load_tile(kt + 1, buf ^ 1);
    pf_commit();

    const uint32_t ksm = smem_base + buf * 2 * TILE_BYTES, vsm = ksm + TILE_BYTES;
    const int key0 = kt * PF_KTILE;

    // ---- S[16 x 64] = Q K^T ----
    float s[NT_S][4];
#pragma unroll
    for (int nt = 0; nt < NT_S; ++nt) {
      s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
      const int key = 8 * nt + (lane & 7);
#pragma unroll
      for (int kp = 0; kp < HD / 32; ++kp) {          // two k-steps (32 dims) per ldmatrix.x4
        const int ch = 4 * kp + (lane >> 3);
        uint32_t b0, b1, b2, b3;
        pf_ldmatrix_x4(ksm + (uint32_t)key * ROW_BYTES + (uint32_t)((ch ^ (key & 7)) * 16), b0, b1, b2, b3);
        pf_mma(s[nt], qf[2 * kp][0], qf[2 * kp][1], qf[2 * kp][2], qf[2 * kp][3], b0, b1);
        pf_mma(s[nt], qf[2 * kp + 1][0], qf[2 * kp + 1][1], qf[2 * kp + 1][2], qf[2 * kp + 1][3], b2, b3);
      }
    }
    // ---- causal (and window) mask, scale into the exp2 domain ----
    const bool need_mask = key0 + PF_KTILE - 1 > start_pos + qt0 + warp * 16 || window > 0;
#pragma unroll
    for (int nt = 0; nt < NT_S; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = s[nt][e] * scale_log2e;
        if (need_mask) {
          const int key = key0 + 8 * nt + 2 * t4 + (e & 1);
          const int pos = (e < 2) ? pos_lo : pos_hi;
          const bool ok = key <= pos && (window <= 0 || key > pos - window);
          v = ok ? v : -INFINITY;
        }
        s[nt][e] = v;
      }
    // ---- streaming softmax for rows g (e = 0, 1) and g + 8 (e = 2, 3) ----
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float mx = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < NT_S; ++nt) mx = fmaxf(mx, fmaxf(s[nt][2 * half], s[nt][2 * half + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[half], mx);
      // a row with nothing visible yet (rows past the step's end, or a window that starts later)
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = exp2f(m_run[half] - m_use);
      float sum = 0.f;
#pragma unroll
      for (int nt = 0; nt < NT_S; ++nt) {
        const float p0 = exp2f(s[nt][2 * half] - m_use), p1 = exp2f(s[nt][2 * half + 1] - m_use);
        s[nt][2 * half] = p0; s[nt][2 * half + 1] = p1;
        sum += p0 + p1;
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l_run[half] = l_run[half] * corr + sum;
      m_run[half] = m_new;
#pragma unroll
      for (int j = 0; j < NT_O; ++j) { acc[j][2 * half] *= corr; acc[j][2 * half + 1] *= corr; }
    }
    // ---- O += P V ----
#pragma unroll
    for (int kk = 0; kk < PF_KTILE / 16; ++kk) {
      const uint32_t a0 = pf_pack(s[2 * kk][0], s[2 * kk][1]), a1 = pf_pack(s[2 * kk][2], s[2 * kk][3]);
      const uint32_t a2 = pf_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]), a3 = pf_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
      const int key = 16 * kk + 8 * ((lane >> 3) & 1) + (lane & 7);
#pragma unroll
      for (int np = 0; np < NT_O / 2; ++np) {         // two output n-tiles per ldmatrix.x4.trans
        const int ch = 2 * np + (lane >> 4);
        uint32_t b0, b1, b2, b3;
        pf_ldmatrix_x4_trans(vsm + (uint32_t)key * ROW_BYTES + (uint32_t)((ch ^ (key & 7)) * 16), b0, b1, b2, b3);
        pf_mma(acc[2 * np], a0, a1, a2, a3, b0, b1);
        pf_mma(acc[2 * np + 1], a0, a1, a2, a3, b2, b3);
      }
    }
  }
  pf_wait<0>();

  // ---- write the 16 x HD outputs of this warp ----
  const float inv_lo = l_run[0] > 0.f ? 1.0f / l_run[0] : 0.f, inv_hi = l_run[1] > 0.f ? 1.0f / l_run[1] : 0.f;
  __nv_bfloat16* olo = out + (size_t)(row0 + qt0 + r_lo) * ldo + (size_t)h * HD;
  __nv_bfloat16* ohi = olo + (size_t)8 * ldo;
#pragma unroll
  for (int j = 0; j < NT_O; ++j) {
    if (r_lo < rows_here) *reinterpret_cast<uint32_t*>(olo + 8 * j + 2 * t4) = pf_pack(acc[j][0] * inv_lo, acc[j][1] * inv_lo);
    if (r_hi < rows_here) *reinterpret_cast<uint32_t*>(ohi + 8 * j + 2 * t4) = pf_pack(acc[j][2] * inv_hi, acc[j][3] * inv_hi);
  }
}

template <int HD>
static int launch_prefill(const void* q, int ldq, const void* k_pool, const void* v_pool, const int* page_table,
                          int max_pages, const int* cu_seqlens, const int* seq_slots, const int* kv_lens, int num_seqs,
                          int num_tiles, void* out, int ldo, int H, int G, float scale, int window, cudaStream_t stream) {
  constexpr int SMEM = 2 * 2 * PF_KTILE * HD * 2;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    RL_REQUIRE(e == cudaSuccess, "rl_attention_prefill: cannot reserve %d bytes of shared memory: %s", SMEM, cudaGetErrorString(e));
    configured = true;
  }
  dim3 grid(num_tiles, H);
  rl_launch_pdl(attention_prefill_kernel<HD>, grid, dim3(PF_WARPS * 32), (size_t)SMEM, stream,
      (const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, page_table, max_pages,
      cu_seqlens, seq_slots, kv_lens, num_seqs, (__nv_bfloat16*)out, ldo, H, G, scale * 1.4426950408889634f, window);
  RL_LAUNCH_CHECK("rl_attention_prefill");
  return RL_OK;
}

// 1 if the prefill kernel takes this shape: head_dim 64 or 128.
extern "C" int rl_attention_prefill_supported(int num_heads, int num_kv_heads, int head_dim) {
  if (num_kv_heads <= 0 || num_heads % num_kv_heads != 0) return 0;
  return head_dim == 64 || head_dim == 128;
}

// q: [M, ldq] bf16, the step's tokens packed by sequence (cu_seqlens: [B+1] offsets);
// kv_lens[b] = length of sequence b after this step (its query tokens take the last
// positions); num_tiles = sum over sequences of ceil(tokens / 64).  out: [M, ldo] bf16.
extern "C" int rl_attention_prefill(const void* q, int ldq, const void* k_pool, const void* v_pool,
                                    const int* page_table, int max_pages, const int* cu_seqlens,
                                    const int* seq_slots, const int* kv_lens, int num_seqs, int num_tiles, void* out,
                                    int ldo, int num_heads, int num_kv_heads, int head_dim, float scale, int window,
                                    cudaStream_t stream) {
  RL_REQUIRE(rl_attention_prefill_supported(num_heads, num_kv_heads, head_dim),
             "rl_attention_prefill: unsupported shape (heads %d, KV heads %d, head_dim %d): needs head_dim 64 or 128",
             num_heads, num_kv_heads, head_dim);
  RL_REQUIRE(num_seqs >= 0 && num_tiles >= 0 && num_heads <= 65535, "rl_attention_prefill: bad sizes");
  RL_REQUIRE(ldq >= num_heads * head_dim && ldo >= num_heads * head_dim && ldq % 2 == 0 && ldo % 2 == 0,
             "rl_attention_prefill: row strides too small or odd");
  RL_REQUIRE(((uintptr_t)q & 3) == 0 && ((uintptr_t)out & 3) == 0 && ((uintptr_t)k_pool & 15) == 0 && ((uintptr_t)v_pool & 15) == 0,
             "rl_attention_prefill: misaligned pointers");
  RL_REQUIRE(window >= 0, "rl_attention_prefill: negative window");
  if (num_seqs == 0 || num_tiles == 0) return RL_OK;
  if (head_dim == 64)
    return launch_prefill<64>(q, ldq, k_pool, v_pool, page_table, max_pages, cu_seqlens, seq_slots, kv_lens, num_seqs,
                              num_tiles, out, ldo, num_heads, num_kv_heads, scale, window, stream);
  return launch_prefill<128>(q, ldq, k_pool, v_pool, page_table, max_pages, cu_seqlens, seq_slots, kv_lens, num_seqs,
                             num_tiles, out, ldo, num_heads, num_kv_heads, scale, window, stream);
}
