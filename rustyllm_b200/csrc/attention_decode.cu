// Decode attention: one new token per sequence attends to its cached keys and values
// (bf16, paged), split over the context so that a handful of sequences still fills the
// GPU, with the partial results combined in a fixed order.
//
// Math (SimonWaldherr/RustyLLM src/model.rs:5807-5869, grouped as in 6034-6198): for query head h
// of KV head g = h / (H/G): softmax over t of (q_h . K[t, g]) / sqrt(head_dim), times
// V[t, g], with running (max, sum, output) in float.  The (H/G) query heads that share
// a KV head are the rows of one 16-row tensor-core tile (mma.sync m16n8k16, bf16 in,
// float accumulate), so each key and value row is read once for all of them, as the
// reference's grouped scan does on the CPU and its Metal kernel
// ``resident_gqa4_attention`` (src/metal_backend.m:542-592) does for groups of four.
//
// The kernel is bound by the read of the cache, and the cache is read fastest in whole
// lines: a block of 16 keys (and of 16 values) of one KV head is contiguous in its page, and
// every cp.async instruction of a warp copies 512 consecutive bytes of it (with 64 bytes a
// row and instruction, as the MMA fragments would have it, the same bytes arrive at three
// quarters of the rate).  The copies land in a ring in shared memory that belongs to the
// warp (so a warp barrier is all the synchronisation there is), 16-byte pieces XOR-swizzled
// by their row so that ldmatrix reads the fragments without bank conflicts - keys as they
// lie, values transposed: two blocks of 16 keys are in flight per warp while a third is
// being multiplied.
//
// Grid: (chunks, KV heads); 4 warps per CTA take their chunk's 16-key blocks in turn.
// The batch's sequences x `splits` chunks are dealt to the sequences in proportion to
// their lengths by a one-warp plan kernel: it finds, from the lengths on the device, the
// smallest chunk size (in rounds of 64 keys) with which all sequences together need no
// more chunks than the grid has, so a long sequence beside short ones is cut into more
// pieces and the CTAs carry equal loads.  The plan depends on the lengths only, so one
// plan serves every layer of a step; the grid depends on the batch's size only (a
// captured step keeps it while the lengths change).  With one chunk per sequence there is
// no plan and the CTA writes the output; otherwise a sequence of one chunk is still written by
// its CTA, and the chunks of a longer one write their (max, sum, unnormalised output) to
// scratch and a second kernel combines them in chunk order.
// Without a plan every sequence gets `splits` chunks (one sequence needs no dealing).
// A third way needs no scratch and no second kernel: with 2, 4 or 8 equal chunks a sequence
// the chunks' CTAs form a thread-block cluster, leave their (max, sum, output) in their own
// shared memory, and every CTA combines its share of the output columns from all of them
// through distributed shared memory, in chunk order.
// (Working the plan out in every CTA, and letting the last CTA of a sequence do the
// combining - found by an atomic ticket - were both measured and are slower: dependent
// round trips to memory at the start and the end of a kernel that runs for 10 us.)
#include <math.h>

#include "common.cuh"

#define DEC_WARPS 4
#define DEC_BLOCK 16   // keys per MMA step

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

#define DEC_STAGES 3
__device__ __forceinline__ void dec_cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void dec_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void dec_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// four 8x8 bf16 matrices, row addresses from lanes 8i .. 8i+7; register i = matrix i, lane (g, t)
// holding row g, columns 2t, 2t+1 (`trans`: column g, rows 2t, 2t+1)
__device__ __forceinline__ void dec_ldmatrix4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void dec_ldmatrix4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ uint32_t ldg_pair(const __nv_bfloat16* p) {
  return __ldg(reinterpret_cast<const uint32_t*>(p));
}

// ---- thread-block cluster ----
__device__ __forceinline__ uint32_t dec_cluster_size() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t dec_cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void dec_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the float at `p` (an address in this CTA's shared memory) in CTA `rank` of the cluster
__device__ __forceinline__ float dec_peer_f32(const float* p, uint32_t rank) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  uint32_t ra;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ra) : "memory");
  return v;
}

// ---- dealing chunks to sequences (warp-wide: call with all 32 lanes) ----
// rounds of 64 keys (16 for each of the 4 warps) that sequence holds inside its window
__device__ __forceinline__ int dec_rounds(int len, int window) {
  const int start = (window > 0 && len - window > 0) ? len - window : 0;
  const int num_blk = (len + DEC_BLOCK - 1) / DEC_BLOCK - start / DEC_BLOCK;
  const int r = (num_blk + DEC_WARPS - 1) / DEC_WARPS;
  return r > 0 ? r : 1;
}
__device__ __forceinline__ int dec_chunks_needed(const int* __restrict__ kv_lens, int B, int window, int c, int lane) {
  int n = 0;
  for (int b = lane; b < B; b += 32) n += (dec_rounds(kv_lens[b], window) + c - 1) / c;
  return __reduce_add_sync(0xffffffffu, n);
}
// smallest chunk size (rounds) with which the B sequences need at most `nchunk` (>= B) chunks
__device__ __forceinline__ int dec_chunk_rounds(const int* __restrict__ kv_lens, int B, int window, int nchunk, int lane) {
  int tot = 0, mx = 1;
  for (int b = lane; b < B; b += 32) { const int u = dec_rounds(kv_lens[b], window); tot += u; mx = max(mx, u); }
  tot = __reduce_add_sync(0xffffffffu, tot);
  mx = __reduce_max_sync(0xffffffffu, mx);
  int lo = max(1, (tot + nchunk - 1) / nchunk), hi = mx;      // at hi every sequence is one chunk
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (dec_chunks_needed(kv_lens, B, window, mid, lane) <= nchunk) hi = mid; else lo = mid + 1;
  }
  return lo;
}
// The plan: entries[x] for chunk x of the grid = {sequence, chunk of the sequence |
// chunks of the sequence << 16, length, cache slot} (sequence -1: a spare chunk), then
// seqs[b] = {first chunk of sequence b, number of its chunks}.  One warp.
__global__ void attention_decode_plan_kernel(const int* __restrict__ seq_slots, const int* __restrict__ kv_lens, int B,
                                             int window, int nchunk, int4* __restrict__ entries, int2* __restrict__ seqs) {
  // No early release of the kernels behind this one: whatever is launched after it begins
  // only when the plan is complete, so those kernels may read the plan before they wait
  // for their own predecessor.
  rl_pdl_wait();
  const int lane = threadIdx.x;
  const int c = dec_chunk_rounds(kv_lens, B, window, nchunk, lane);
  int base = 0;
  for (int b0 = 0; b0 < B; b0 += 32) {
    const int b = b0 + lane;
    const int len = b < B ? kv_lens[b] : 0;
    const int n = b < B ? (dec_rounds(len, window) + c - 1) / c : 0;
    int incl = n;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += v; }
    if (b < B) {
      const int first = base + incl - n, slot = seq_slots[b];
      seqs[b] = make_int2(first, n);
      for (int j = 0; j < n; ++j) entries[first + j] = make_int4(b, j | (n << 16), len, slot);
    }
    base += __shfl_sync(0xffffffffu, incl, 31);
  }
  for (int x = base + lane; x < nchunk; x += 32) entries[x] = make_int4(-1, 0, 0, 0);
}

// A plan of whole sequences, the longest first (inside `window` if it is not 0; ties in the order of
// the batch): entries[x] = {sequence, 0 | 1 << 16, length, cache slot}, seqs[b] = {place of sequence b, 1}.
// Where a batch is more CTAs than the SMs hold at once, the CTAs that start last should be the
// shortest.  One CTA, a thread a sequence (at most 1,024), every thread counting who goes before it.
__global__ void __launch_bounds__(1024)
attention_decode_order_kernel(const int* __restrict__ seq_slots, const int* __restrict__ kv_lens, int B, int window,
                              int4* __restrict__ entries, int2* __restrict__ seqs) {
  __shared__ int s_len[1024];
  rl_pdl_wait();         // no early release of the kernels behind this one, as in the plan kernel
  const int b = threadIdx.x;
  int len = 0, inside = 0;
  if (b < B) { len = kv_lens[b]; inside = (window > 0 && len > window) ? window : len; }
  s_len[b] = inside;
  __syncthreads();
  if (b < B) {
    int place = 0;
    for (int j = 0; j < B; ++j) { const int other = s_len[j]; place += (other > inside || (other == inside && j < b)) ? 1 : 0; }
    entries[place] = make_int4(b, 1 << 16, len, seq_slots[b]);
    seqs[b] = make_int2(place, 1);
  }
}

// shared memory of one CTA: the ring [warp][stage][keys | values][16 rows][HD] of bf16 (16-byte
// pieces swizzled within their row), reused after the loop for the warps' (max, sum, output)
template <int HD>
struct DecSmem {
  static constexpr int ROW_BYTES = HD * 2;
  static constexpr int TILE_BYTES = DEC_BLOCK * ROW_BYTES;          // 16 keys (or values) of one KV head
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  static constexpr int RING_BYTES = DEC_WARPS * DEC_STAGES * STAGE_BYTES;
  static constexpr int MERGE_BYTES = (DEC_WARPS * 16 * (HD + 4) + 2 * DEC_WARPS * 16) * 4;
  static constexpr int RESULT_BYTES = (16 * HD + 2 * 16) * 4;      // the CTA's own (output, max, sum), read by its cluster
  static constexpr int BYTES = RING_BYTES > MERGE_BYTES + RESULT_BYTES ? RING_BYTES : MERGE_BYTES + RESULT_BYTES;
};

template <int HD>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, int ldq, const __nv_bfloat16* __restrict__ k_pool,
                        const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ page_table, int max_pages,
                        const int* __restrict__ seq_slots, const int* __restrict__ kv_lens,
                        const int4* __restrict__ plan, __nv_bfloat16* __restrict__ out, int ldo,
                        float* __restrict__ part_o, float* __restrict__ part_ml, int H, int G, float scale_log2e,
                        int window, int even_splits) {
  constexpr int NT = HD / 8;        // output n-tiles of 8 columns
  constexpr int KS = HD / 16;       // k-steps of the Q.K product
  extern __shared__ __align__(128) uint8_t dec_smem[];
  float (*s_acc)[16][HD + 4] = reinterpret_cast<float (*)[16][HD + 4]>(dec_smem);
  float (*s_m)[16] = reinterpret_cast<float (*)[16]>(dec_smem + DEC_WARPS * 16 * (HD + 4) * 4);
  float (*s_l)[16] = s_m + DEC_WARPS;

  rl_pdl_trigger();
  // Before waiting for the kernel in front (which writes this step's queries, keys and
  // values): the plan, the sequence's length and slot and its page numbers were complete
  // before that kernel began, so these dependent loads overlap with its tail.
  // Chunks along x and KV heads along y where the chunks of a sequence form a cluster (a cluster lies
  // along x); else KV heads along x, the faster index: CTAs start in the order of the chunks, all KV
  // heads of one before the next, which is what makes a plan's order (longest first) the order of work.
  const bool clustered = dec_cluster_size() > 1;          // the chunks of a sequence are the CTAs of a cluster
  const int gkv = clustered ? blockIdx.y : blockIdx.x;
  const int chunk_id = clustered ? blockIdx.x : blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int m = H / G;                                   // query heads per KV head (<= 16)
  // which sequence, and which share of its keys
  int b = chunk_id, split = 0, num_splits = 1, len, cache_slot;
  if (plan == nullptr) {                                 // no plan: every sequence in `even_splits` chunks
    b = chunk_id / even_splits; split = chunk_id % even_splits; num_splits = even_splits;
    len = kv_lens[b]; cache_slot = seq_slots[b];
  } else {
    const int4 e = __ldg(&plan[chunk_id]);
    if (e.x < 0) return;                                 // spare chunk
    b = e.x; split = e.y & 0xffff; num_splits = e.y >> 16; len = e.z; cache_slot = e.w;
  }
  // a sequence that is one chunk (always so without splits; with a plan, the short ones beside
  // long ones) is finished here: no scratch, nothing for the combining kernel to do
  const bool direct = num_splits == 1;
  const int start = (window > 0 && len - window > 0) ? len - window : 0;
  const int* pages = page_table + (size_t)cache_slot * max_pages;

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  // ---- this split's blocks of 16 keys, dealt to the warps in turn ----
  const int first_blk = start / DEC_BLOCK;
  const int num_blk = (len + DEC_BLOCK - 1) / DEC_BLOCK - first_blk;
  const int rounds = (num_blk + DEC_WARPS - 1) / DEC_WARPS;
  const int per_split = (rounds + num_splits - 1) / num_splits * DEC_WARPS;   // whole rounds: every warp gets a block of each
  const int blk_lo = first_blk + split * per_split;
  const int blk_hi = min(blk_lo + per_split, first_blk + num_blk);
  const size_t page_stride = (size_t)G * RL_PAGE * HD;
  const size_t head_off = (size_t)gkv * RL_PAGE * HD;

  // A tile is 16 rows of HD bf16; the 16-byte piece `ch` of row `row` lies at
  // row * ROW_BYTES + ((ch ^ (row & 7)) * 16).  A warp instruction copies 32 consecutive pieces.
  constexpr int ROWB = DecSmem<HD>::ROW_BYTES, TILEB = DecSmem<HD>::TILE_BYTES, STAGEB = DecSmem<HD>::STAGE_BYTES;
  constexpr int CH = HD / 8;                             // pieces a row
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(dec_smem) + (uint32_t)(warp * DEC_STAGES * STAGEB);
  auto issue = [&](int blk, int st, int page) {
    const int key0 = blk * DEC_BLOCK;
    const size_t base = (size_t)page * page_stride + head_off + (size_t)(key0 % RL_PAGE) * HD;
    const __nv_bfloat16* kb = k_pool + base + 8 * lane;
    const __nv_bfloat16* vb = v_pool + base + 8 * lane;
    const uint32_t kd = ring + (uint32_t)(st * STAGEB), vd = kd + TILEB;
#pragma unroll
    for (int i = 0; i < TILEB / 512; ++i) {
      const int piece = i * 32 + lane, row = piece / CH, ch = piece % CH;
      const uint32_t off = (uint32_t)(row * ROWB + ((ch ^ (row & 7)) << 4));
      dec_cp_async16(kd + off, kb + i * 256, 16);
      // rows beyond the sequence may hold anything: zeros instead (their weights are zero)
      dec_cp_async16(vd + off, vb + i * 256, key0 + row < len ? 16 : 0);
    }
  };
  // ldmatrix row addresses of this lane within a tile.  Keys (as they lie): matrix lane/8 is piece
  // 4c + lane/8 of keys 8nt + (lane & 7).  Values (transposed): matrix lane/8 is piece 2jp + lane/16
  // of keys (lane & 7) + 8 * ((lane / 8) & 1).
  const int swz = lane & 7;
  const uint32_t k_row = (uint32_t)(swz * ROWB), k_piece = (uint32_t)(lane >> 3);
  const uint32_t v_row = (uint32_t)((swz + 8 * ((lane >> 3) & 1)) * ROWB), v_piece = (uint32_t)(lane >> 4);

  {
    int first_pages[DEC_STAGES - 1];
#pragma unroll
    for (int st = 0; st < DEC_STAGES - 1; ++st) {
      const int pre = blk_lo + warp + st * DEC_WARPS;
      first_pages[st] = pre < blk_hi ? __ldg(&pages[pre * DEC_BLOCK / RL_PAGE]) : 0;
    }
    rl_pdl_wait();
#pragma unroll
    for (int st = 0; st < DEC_STAGES - 1; ++st) {
      const int pre = blk_lo + warp + st * DEC_WARPS;
      if (pre < blk_hi) issue(pre, st, first_pages[st]);
      dec_commit();
    }
  }
  // ---- Q fragments (after the first key/value copies are on their way): rows = the m heads
  // of this KV head ----
  uint32_t qf[KS][4];
  {
    const __nv_bfloat16* q0 = q + (size_t)b * ldq + (size_t)(gkv * m + g) * HD + 2 * t;
    const __nv_bfloat16* q1 = q0 + (size_t)8 * HD;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      qf[ks][0] = g < m ? ldg_pair(q0 + 16 * ks) : 0u;
      qf[ks][1] = g + 8 < m ? ldg_pair(q1 + 16 * ks) : 0u;
      qf[ks][2] = g < m ? ldg_pair(q0 + 16 * ks + 8) : 0u;
      qf[ks][3] = g + 8 < m ? ldg_pair(q1 + 16 * ks + 8) : 0u;
    }
  }

  int it = 0;
  for (int blk = blk_lo + warp; blk < blk_hi; blk += DEC_WARPS, ++it) {
    const int key0 = blk * DEC_BLOCK;
    const int st = it % DEC_STAGES;
    {
      const int ahead = blk + (DEC_STAGES - 1) * DEC_WARPS;
      if (ahead < blk_hi) issue(ahead, (it + DEC_STAGES - 1) % DEC_STAGES, __ldg(&pages[ahead * DEC_BLOCK / RL_PAGE]));
      dec_commit();
    }
    dec_wait<DEC_STAGES - 1>();     // this lane's pieces of block `blk` have landed,
    __syncwarp();                   // and so have the other lanes'
    const uint32_t kt = ring + (uint32_t)(st * STAGEB), vt = kt + TILEB;

    // scores S[16 heads x 16 keys] = Q . K^T
    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t kr[4];
        dec_ldmatrix4(kr, kt + (uint32_t)(8 * nt * ROWB) + k_row + (((4 * c + k_piece) ^ swz) << 4));
        mma_bf16_16816(s[nt], qf[2 * c][0], qf[2 * c][1], qf[2 * c][2], qf[2 * c][3], kr[0], kr[1]);
        mma_bf16_16816(s[nt], qf[2 * c + 1][0], qf[2 * c + 1][1], qf[2 * c + 1][2], qf[2 * c + 1][3], kr[2], kr[3]);
      }
    }
    // mask keys outside [start, len), scale into the exp2 domain
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + 8 * nt + 2 * t + (e & 1);
        s[nt][e] = (key < len && key >= start) ? s[nt][e] * scale_log2e : -INFINITY;
      }
    // streaming softmax for rows g (e = 0, 1) and g + 8 (e = 2, 3)
    uint32_t pa[4];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float mx = fmaxf(fmaxf(s[0][2 * half], s[0][2 * half + 1]), fmaxf(s[1][2 * half], s[1][2 * half + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[half], mx);           // finite: the block holds a valid key
      const float corr = exp2f(m_run[half] - m_new);        // exp2(-inf) = 0 on the first block
      const float p00 = exp2f(s[0][2 * half] - m_new), p01 = exp2f(s[0][2 * half + 1] - m_new);
      const float p10 = exp2f(s[1][2 * half] - m_new), p11 = exp2f(s[1][2 * half + 1] - m_new);
      float sum = (p00 + p01) + (p10 + p11);
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l_run[half] = l_run[half] * corr + sum;
      m_run[half] = m_new;
#pragma unroll
      for (int j = 0; j < NT; ++j) { acc[j][2 * half] *= corr; acc[j][2 * half + 1] *= corr; }
      pa[half] = pack_bf16(p00, p01);          // a0 / a1: keys 2t, 2t+1
      pa[2 + half] = pack_bf16(p10, p11);      // a2 / a3: keys 2t+8, 2t+9
    }
    // output += P . V ; n-tile j holds dimensions 8j .. 8j+7
#pragma unroll
    for (int jp = 0; jp < NT / 2; ++jp) {
      uint32_t vr[4];
      dec_ldmatrix4_trans(vr, vt + v_row + (((2 * jp + v_piece) ^ swz) << 4));
      mma_bf16_16816(acc[2 * jp], pa[0], pa[1], pa[2], pa[3], vr[0], vr[1]);
      mma_bf16_16816(acc[2 * jp + 1], pa[0], pa[1], pa[2], pa[3], vr[2], vr[3]);
    }
  }

  // ---- combine the four warps (the ring's memory is reused: every copy must have landed) ----
  dec_wait<0>();
  __syncthreads();
  if (t == 0) {
    s_m[warp][g] = m_run[0]; s_l[warp][g] = l_run[0];
    s_m[warp][g + 8] = m_run[1]; s_l[warp][g + 8] = l_run[1];
  }
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int d0 = 8 * j + 2 * t;
    if (g < m) *reinterpret_cast<float2*>(&s_acc[warp][g][d0]) = make_float2(acc[j][0], acc[j][1]);
    if (g + 8 < m) *reinterpret_cast<float2*>(&s_acc[warp][g + 8][d0]) = make_float2(acc[j][2], acc[j][3]);
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < m * HD; idx += DEC_WARPS * 32) {
    const int r = idx / HD, d = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, s_m[w][r]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float wgt = (s_m[w][r] > -INFINITY) ? exp2f(s_m[w][r] - M) : 0.f;
      L += s_l[w][r] * wgt;
      O += s_acc[w][r][d] * wgt;
    }
    const int h = gkv * m + r;
    if (direct) {
      out[(size_t)b * ldo + (size_t)h * HD + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
    } else if (clustered) {
      float* c_o = reinterpret_cast<float*>(dec_smem + DecSmem<HD>::MERGE_BYTES);
      c_o[r * HD + d] = O;
      if (d == 0) { c_o[16 * HD + r] = M; c_o[16 * HD + 16 + r] = L; }
    } else {
      const size_t p = (size_t)chunk_id * H + h;           // partial results lie in the order of the chunks
      part_o[p * HD + d] = O;
      if (d == 0) { part_ml[2 * p] = M; part_ml[2 * p + 1] = L; }
    }
  }
  if (clustered) {
    // every chunk of the sequence has its result in shared memory; this CTA finishes its share
    // of the m x HD outputs, adding the chunks in their order
    dec_cluster_sync();
    const float* c_o = reinterpret_cast<const float*>(dec_smem + DecSmem<HD>::MERGE_BYTES);
    const int per = (m * HD + num_splits - 1) / num_splits;
    const int lo = split * per, hi = min(lo + per, m * HD);
    for (int idx = lo + threadIdx.x; idx < hi; idx += DEC_WARPS * 32) {
      const int r = idx / HD, d = idx % HD;
      float M = -INFINITY;
      for (int c = 0; c < num_splits; ++c) M = fmaxf(M, dec_peer_f32(c_o + 16 * HD + r, c));
      float L = 0.f, O = 0.f;
      for (int c = 0; c < num_splits; ++c) {
        const float mc = dec_peer_f32(c_o + 16 * HD + r, c);
        const float wgt = (mc > -INFINITY) ? exp2f(mc - M) : 0.f;
        L += dec_peer_f32(c_o + 16 * HD + 16 + r, c) * wgt;
        O += dec_peer_f32(c_o + r * HD + d, c) * wgt;
      }
      out[(size_t)b * ldo + (size_t)(gkv * m + r) * HD + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
    }
    dec_cluster_sync();      // nobody leaves while its shared memory may still be read
  }
}

// Combines the chunks of one (sequence, head) in chunk order.
template <int HD>
__global__ void attention_decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                const int2* __restrict__ plan_seqs, int even_splits,
                                                __nv_bfloat16* __restrict__ out, int ldo, int H) {
  rl_pdl_trigger();
  const int h = blockIdx.x, b = blockIdx.y;
  int first = b * even_splits, count = even_splits;
  if (plan_seqs != nullptr) {
    const int2 fc = __ldg(&plan_seqs[b]);      // complete long before the kernel in front began
    first = fc.x; count = fc.y;
  }
  rl_pdl_wait();
  if (count == 1) return;        // written by its only chunk
  constexpr int FAST = 16;       // chunks whose loads are all requested before the first is used
  const int d = threadIdx.x;     // the block has HD threads or 64 (then two dimensions a thread)
  if (count <= FAST && (int)blockDim.x == HD) {
    // one trip to L2 instead of two in a row (the maxima, then the outputs): this kernel is all latency
    float2 ml[FAST];
    float o[FAST];
#pragma unroll
    for (int s = 0; s < FAST; ++s) {
      const size_t p = (size_t)(first + (s < count ? s : 0)) * H + h;
      ml[s] = s < count ? __ldcg(reinterpret_cast<const float2*>(part_ml + 2 * p)) : make_float2(-INFINITY, 0.f);
      o[s] = s < count ? __ldcg(part_o + p * HD + d) : 0.f;
    }
    float M = -INFINITY;
#pragma unroll
    for (int s = 0; s < FAST; ++s) M = fmaxf(M, ml[s].x);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int s = 0; s < FAST; ++s) {       // in chunk order, as below
      const float wgt = (ml[s].x > -INFINITY) ? exp2f(ml[s].x - M) : 0.f;
      L += ml[s].y * wgt;
      O += o[s] * wgt;
    }
    out[(size_t)b * ldo + (size_t)h * HD + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
    return;
  }
  float M = -INFINITY;
  for (int s = 0; s < count; ++s) M = fmaxf(M, part_ml[2 * ((size_t)(first + s) * H + h)]);
  for (int dd = threadIdx.x; dd < HD; dd += blockDim.x) {
    float L = 0.f, O = 0.f;
#pragma unroll 4
    for (int s = 0; s < count; ++s) {
      const size_t p = (size_t)(first + s) * H + h;
      const float ms = part_ml[2 * p];
      const float wgt = (ms > -INFINITY) ? exp2f(ms - M) : 0.f;
      L += part_ml[2 * p + 1] * wgt;
      O += part_o[p * HD + dd] * wgt;
    }
    out[(size_t)b * ldo + (size_t)h * HD + dd] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
  }
}

template <int HD>
static int launch_decode(const void* q, int ldq, const void* k_pool, const void* v_pool, const int* page_table,
                         int max_pages, const int* seq_slots, const int* kv_lens, void* out, int ldo,
                         float* part_o, float* part_ml, const int* plan, int B, int H, int G, float scale, int window,
                         int num_splits, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecSmem<HD>::BYTES);
    RL_REQUIRE(e == cudaSuccess, "rl_attention_decode: cannot reserve %d bytes of shared memory: %s", DecSmem<HD>::BYTES, cudaGetErrorString(e));
    configured = true;
  }
  const int nchunk = B * num_splits;
  const int4* entries = (const int4*)plan;                                   // null without a plan
  const int2* seqs = plan ? (const int2*)(plan + 4 * (size_t)nchunk) : nullptr;
  if (num_splits > 1 && part_o == nullptr) {
    dim3 grid(nchunk, G);
    // no scratch: the chunks of a sequence are the CTAs of a cluster and combine through shared memory
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(DEC_WARPS * 32);
    cfg.dynamicSmemBytes = DecSmem<HD>::BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (g_rl_pdl_enabled) {
      attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[na].val.programmaticStreamSerializationAllowed = 1;
      ++na;
    }
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = num_splits; attr[na].val.clusterDim.y = 1; attr[na].val.clusterDim.z = 1;
    ++na;
    cfg.attrs = attr;
    cfg.numAttrs = na;
    cudaError_t e = cudaLaunchKernelEx(&cfg, attention_decode_kernel<HD>,
        (const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, page_table, max_pages,
        seq_slots, kv_lens, (const int4*)nullptr, (__nv_bfloat16*)out, ldo, (float*)nullptr, (float*)nullptr, H, G,
        scale * 1.4426950408889634f, window, num_splits);
    RL_REQUIRE(e == cudaSuccess, "rl_attention_decode: cluster launch failed: %s", cudaGetErrorString(e));
    RL_LAUNCH_CHECK("rl_attention_decode");
    return RL_OK;
  }
  dim3 grid(G, nchunk);
  rl_launch_pdl(attention_decode_kernel<HD>, grid, dim3(DEC_WARPS * 32), (size_t)DecSmem<HD>::BYTES, stream,
      (const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, page_table, max_pages,
      seq_slots, kv_lens, entries, (__nv_bfloat16*)out, ldo, part_o, part_ml, H, G, scale * 1.4426950408889634f, window,
      num_splits);
  RL_LAUNCH_CHECK("rl_attention_decode");
  if (num_splits > 1) {
    rl_launch_pdl(attention_decode_combine_kernel<HD>, dim3(H, B), dim3(HD), 0, stream,
                  (const float*)part_o, (const float*)part_ml, seqs, num_splits, (__nv_bfloat16*)out, ldo, H);
    RL_LAUNCH_CHECK("rl_attention_decode (combine)");
  }
  return RL_OK;
}

// 1 if the decode kernel takes this shape: bf16, head_dim 64 or 128, at most 16 query
// heads per KV head.  Other shapes go to the any-shape kernel.
extern "C" int rl_attention_decode_supported(int num_heads, int num_kv_heads, int head_dim) {
  if (num_kv_heads <= 0 || num_heads % num_kv_heads != 0) return 0;
  if (num_heads / num_kv_heads > 16) return 0;
  return head_dim == 64 || head_dim == 128;
}

// Ints of a plan for the given sizes (0 with one split): 4 a chunk, 2 a sequence.
extern "C" long long rl_attention_decode_plan_ints(int num_seqs, int num_splits) {
  if (num_splits <= 1) return 0;
  return 4LL * num_seqs * num_splits + 2LL * num_seqs;
}

// Floats of scratch the call needs for the given sizes (0 with one split).
extern "C" long long rl_attention_decode_scratch_floats(int num_seqs, int num_heads, int head_dim, int num_splits) {
  if (num_splits <= 1) return 0;
  return (long long)num_seqs * num_heads * num_splits * (head_dim + 2);
}

// Deals num_seqs * num_splits chunks to the sequences by their lengths (inside `window`
// if it is not 0).  plan: rl_attention_decode_plan_ints(...) ints, 16-byte aligned.  The
// plan holds for every rl_attention_decode call with the same seq_slots, kv_lens, window
// and num_splits: all layers of a step whose caches have the same window.
extern "C" int rl_attention_decode_plan(const int* seq_slots, const int* kv_lens, int num_seqs, int window,
                                        int num_splits, int* plan, cudaStream_t stream) {
  RL_REQUIRE(num_seqs >= 0 && num_splits >= 1 && window >= 0, "rl_attention_decode_plan: bad sizes");
  if (num_seqs == 0 || num_splits == 1) return RL_OK;
  RL_REQUIRE((long long)num_seqs * num_splits <= 65535, "rl_attention_decode_plan: %d sequences x %d splits exceed 65535 "
             "chunks; use fewer splits", num_seqs, num_splits);
  RL_REQUIRE(plan != nullptr && ((uintptr_t)plan & 15) == 0, "rl_attention_decode_plan: plan is null or not 16-byte aligned");
  const int nchunk = num_seqs * num_splits;
  rl_launch_pdl(attention_decode_plan_kernel, dim3(1), dim3(32), 0, stream, seq_slots, kv_lens, num_seqs, window, nchunk,
                (int4*)plan, (int2*)(plan + 4 * (size_t)nchunk));
  RL_LAUNCH_CHECK("rl_attention_decode_plan");
  return RL_OK;
}

// How many CTAs of the decode kernel the GPU holds at once at this head size (CTAs an SM by shared
// memory and registers, times SMs), and how many bytes of keys and values one CTA keeps in flight:
// what the choice between equal chunks, whole sequences and dealt chunks goes by.
extern "C" int rl_attention_decode_places(int head_dim) {
  static int places[2] = {0, 0};
  RL_REQUIRE(head_dim == 64 || head_dim == 128, "rl_attention_decode_places: head_dim %d is not 64 or 128", head_dim);
  int& p = places[head_dim == 128];
  if (p == 0) {
    int per_sm = 0;
    cudaError_t e;
    if (head_dim == 64) {
      e = cudaFuncSetAttribute(attention_decode_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecSmem<64>::BYTES);
      if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_decode_kernel<64>, DEC_WARPS * 32, DecSmem<64>::BYTES);
    } else {
      e = cudaFuncSetAttribute(attention_decode_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecSmem<128>::BYTES);
      if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_decode_kernel<128>, DEC_WARPS * 32, DecSmem<128>::BYTES);
    }
    RL_REQUIRE(e == cudaSuccess && per_sm > 0, "rl_attention_decode_places: occupancy query failed: %s", cudaGetErrorString(e));
    p = per_sm * rl_num_sms();
  }
  return p;
}
extern "C" int rl_attention_decode_ring_bytes(int head_dim) { return head_dim == 64 ? DecSmem<64>::RING_BYTES : DecSmem<128>::RING_BYTES; }

// Ints of an order plan for num_seqs sequences.
extern "C" long long rl_attention_decode_order_ints(int num_seqs) { return 6LL * num_seqs; }

// The sequences whole, the longest first: a plan for rl_attention_decode with num_splits 1, for batches
// that are more CTAs than the SMs hold at once (their last CTAs should be the shortest).  At most
// 1,024 sequences.  plan: rl_attention_decode_order_ints(...) ints, 16-byte aligned; holds for every
// rl_attention_decode call with the same seq_slots, kv_lens and window.
extern "C" int rl_attention_decode_order(const int* seq_slots, const int* kv_lens, int num_seqs, int window, int* plan,
                                         cudaStream_t stream) {
  RL_REQUIRE(num_seqs >= 0 && num_seqs <= 1024 && window >= 0, "rl_attention_decode_order: takes 0 to 1024 sequences (got %d) "
             "and a window that is not negative", num_seqs);
  if (num_seqs == 0) return RL_OK;
  RL_REQUIRE(plan != nullptr && ((uintptr_t)plan & 15) == 0, "rl_attention_decode_order: plan is null or not 16-byte aligned");
  rl_launch_pdl(attention_decode_order_kernel, dim3(1), dim3((num_seqs + 31) / 32 * 32), 0, stream, seq_slots, kv_lens, num_seqs,
                window, (int4*)plan, (int2*)(plan + 4 * (size_t)num_seqs));
  RL_LAUNCH_CHECK("rl_attention_decode_order");
  return RL_OK;
}

// q: [B, ldq] bf16, one token per sequence; seq_slots, kv_lens: [B] (kv_lens counts the
// new token, whose key and value are already in the cache); out: [B, ldo] bf16.
// scratch: rl_attention_decode_scratch_floats(...) floats (may be null with one split).
// plan: what rl_attention_decode_plan made for these sequences, window and splits (with one
// split: what rl_attention_decode_order made), or null: then every sequence is cut into num_splits
// equal chunks whatever its length (right for one sequence, or for sequences of like lengths).  Null scratch with 2, 4 or 8
// splits and no plan: the chunks of a sequence run as a thread-block cluster and combine
// through distributed shared memory (no scratch, no second kernel).
extern "C" int rl_attention_decode(const void* q, int ldq, const void* k_pool, const void* v_pool,
                                   const int* page_table, int max_pages, const int* seq_slots, const int* kv_lens,
                                   void* out, int ldo, float* scratch, const int* plan, int num_seqs, int num_heads,
                                   int num_kv_heads, int head_dim, float scale, int window, int num_splits,
                                   cudaStream_t stream) {
  RL_REQUIRE(rl_attention_decode_supported(num_heads, num_kv_heads, head_dim),
             "rl_attention_decode: unsupported shape (heads %d, KV heads %d, head_dim %d): needs head_dim 64 or 128 "
             "and at most 16 heads per KV head", num_heads, num_kv_heads, head_dim);
  RL_REQUIRE(num_seqs >= 0 && num_splits >= 1, "rl_attention_decode: bad sizes");
  RL_REQUIRE(num_seqs <= 65535 && num_kv_heads <= 65535 && (long long)num_seqs * num_splits <= 65535,
             "rl_attention_decode: too many sequences, chunks (%d x %d splits) or KV heads for one grid", num_seqs, num_splits);
  RL_REQUIRE(ldq >= num_heads * head_dim && ldo >= num_heads * head_dim && ldq % 8 == 0,
             "rl_attention_decode: row strides too small or not a multiple of 8 elements");
  RL_REQUIRE(((uintptr_t)q & 15) == 0 && ((uintptr_t)k_pool & 15) == 0 && ((uintptr_t)v_pool & 15) == 0,
             "rl_attention_decode: q and the cache pools must be 16-byte aligned");
  RL_REQUIRE(num_splits == 1 || scratch != nullptr || (plan == nullptr && (num_splits == 2 || num_splits == 4 || num_splits == 8)),
             "rl_attention_decode: without scratch the chunks combine as a cluster, which takes 2, 4 or 8 splits and no plan (got %d)", num_splits);
  RL_REQUIRE(plan == nullptr || ((uintptr_t)plan & 15) == 0, "rl_attention_decode: plan is not 16-byte aligned");
  RL_REQUIRE(window >= 0, "rl_attention_decode: negative window");
  if (num_seqs == 0) return RL_OK;
  const size_t parts = (size_t)num_seqs * num_heads * num_splits;
  float* part_o = scratch;
  float* part_ml = scratch ? scratch + parts * head_dim : nullptr;
  if (head_dim == 64)
    return launch_decode<64>(q, ldq, k_pool, v_pool, page_table, max_pages, seq_slots, kv_lens, out, ldo, part_o,
                             part_ml, plan, num_seqs, num_heads, num_kv_heads, scale, window, num_splits, stream);
  return launch_decode<128>(q, ldq, k_pool, v_pool, page_table, max_pages, seq_slots, kv_lens, out, ldo, part_o,
                            part_ml, plan, num_seqs, num_heads, num_kv_heads, scale, window, num_splits, stream);
}

// ------------------------------------------------------------------ entry point that allocates nothing
// Declared in attention_decode_static.h.  Same kernels as rl_attention_decode; the
// scratch for the per-split partial results lives in the array below instead of in
// memory the caller allocates.  The array is part of the loaded library: every GPU
// that loads it holds these 4 MiB until the process exits.
#include <mutex>

#include "attention_decode_static.h"

static __device__ __align__(256) float g_decode_static_scratch[RL_DECODE_STATIC_SCRATCH_FLOATS];

// In host code the array's name stands for the symbol, not for device memory: its device
// address is asked for once per device (with that device current) and kept here.
static float* g_decode_static_ptr[RL_DECODE_STATIC_MAX_DEVICES] = {nullptr};
static std::mutex g_decode_static_mutex;

static int decode_static_scratch(float** ptr) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  RL_REQUIRE(e == cudaSuccess, "rl_attention_decode_static: cudaGetDevice failed: %s", cudaGetErrorString(e));
  RL_REQUIRE(dev >= 0 && dev < RL_DECODE_STATIC_MAX_DEVICES, "rl_attention_decode_static: device %d is beyond the %d "
             "devices this entry point keeps an address for", dev, RL_DECODE_STATIC_MAX_DEVICES);
  std::lock_guard<std::mutex> lock(g_decode_static_mutex);
  if (g_decode_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_decode_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      rl_set_error("rl_attention_decode_static: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
      return RL_ERR_CUDA;
    }
    g_decode_static_ptr[dev] = (float*)p;
  }
  *ptr = g_decode_static_ptr[dev];
  return RL_OK;
}

extern "C" int rl_attention_decode_static(const void* q, int ldq, const void* k_pool, const void* v_pool,
                                          const int* page_table, int max_pages, const int* seq_slots,
                                          const int* kv_lens, void* out, int ldo, int num_seqs, int num_heads,
                                          int num_kv_heads, int head_dim, float scale, int window, int num_splits,
                                          cudaStream_t stream) {
  RL_REQUIRE(num_seqs >= 0 && num_heads > 0 && head_dim > 0 && num_splits >= 1, "rl_attention_decode_static: bad sizes");
  const long long need = rl_attention_decode_scratch_floats(num_seqs, num_heads, head_dim, num_splits);
  RL_REQUIRE(need <= (long long)RL_DECODE_STATIC_SCRATCH_FLOATS,
             "rl_attention_decode_static: %d sequences x %d heads x %d splits x (head_dim %d + 2) = %lld floats of "
             "scratch exceed the built-in %lld; use fewer splits or rl_attention_decode with scratch of your own",
             num_seqs, num_heads, num_splits, head_dim, need, (long long)RL_DECODE_STATIC_SCRATCH_FLOATS);
  float* scratch = nullptr;
  const int rc = decode_static_scratch(&scratch);
  if (rc != RL_OK) return rc;
  return rl_attention_decode(q, ldq, k_pool, v_pool, page_table, max_pages, seq_slots, kv_lens, out, ldo, scratch, nullptr,
                             num_seqs, num_heads, num_kv_heads, head_dim, scale, window, num_splits, stream);
}
