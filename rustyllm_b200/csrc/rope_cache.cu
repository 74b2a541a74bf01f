// Rotary position encoding of the step's queries and keys, fused with the write of
// the rotated keys and the values into the paged cache.
//
// Formulas (SimonWaldherr/RustyLLM): angle = float(pos) * inv_freq[i], (sin, cos) of it in
// 32-bit, (x0, x1) <- (x0*cos - x1*sin, x0*sin + x1*cos) on every query and key
// head, values untouched (src/model.rs:5562-5647); then K[layer][pos] = k,
// V[layer][pos] = v (src/model.rs:7233-7236).  Pairing "half" rotates (i, i + r/2),
// "interleaved" rotates (2i, 2i+1), r being the rotary width (<= head size; the
// rest of a head passes through unrotated).  The same fusion is the reference's
// Metal kernel ``rope_store`` (src/metal_backend.m:446-489).
//
// Cache layout: pool[page][kv_head][RL_PAGE][head_dim]; the page of position p of
// the sequence in slot s is page_table[s * max_pages + p / RL_PAGE].
#include "common.cuh"

#define ROPE_HEADS_PER_CTA 8
#define ROPE_THREADS 128

// Grid: (tokens, ceil((H + 2G) / ROPE_HEADS_PER_CTA)).  A CTA takes one token and a run of
// "head slots" (query heads, then key heads, then value heads); a thread takes pairs of
// elements, each pair independent of every other, so all its loads are in flight at once.
template <typename T>
__global__ void __launch_bounds__(ROPE_THREADS)
rope_kv_write_kernel(T* __restrict__ qkv, int ld, const int* __restrict__ positions,
                     const int* __restrict__ slot_of_token, const int* __restrict__ page_table, int max_pages,
                     const float* __restrict__ inv_freq, int H, int G, int hd, int vd, int rot, int interleaved,
                     T* __restrict__ k_pool, T* __restrict__ v_pool, int write_cache) {
  rl_pdl_trigger();
  rl_pdl_wait();
  const int m = blockIdx.x;
  const int pos = positions[m];
  T* row = qkv + (size_t)m * ld;
  size_t dst = 0, dst_v = 0;
  if (write_cache) {
    const int slot = slot_of_token[m];
    const int page = page_table[(size_t)slot * max_pages + pos / RL_PAGE];
    dst = ((size_t)page * G) * RL_PAGE * hd + (size_t)(pos % RL_PAGE) * hd;  // + g * RL_PAGE * hd
    dst_v = ((size_t)page * G) * RL_PAGE * vd + (size_t)(pos % RL_PAGE) * vd;
  }
  const int half = rot / 2, pairs = max(hd, vd) / 2;
  const int slot0 = blockIdx.y * ROPE_HEADS_PER_CTA;
  const int nslots = min(ROPE_HEADS_PER_CTA, H + 2 * G - slot0);
  for (int idx = threadIdx.x; idx < nslots * pairs; idx += ROPE_THREADS) {
    const int hs = slot0 + idx / pairs;       // head slot: [0, H) q, [H, H+G) k, [H+G, H+2G) v
    const int i = idx % pairs;
    const bool is_v = hs >= H + G;
    if (i >= (is_v ? vd : hd) / 2) continue;   // value heads may be narrower or wider than key heads
    const bool rotate = !is_v && i < half;
    int i0, i1;
    if (rotate) { i0 = interleaved ? 2 * i : i; i1 = interleaved ? 2 * i + 1 : i + half; }
    else if (is_v) { i0 = 2 * i; i1 = 2 * i + 1; }
    else { i0 = rot + 2 * (i - half); i1 = i0 + 1; }          // unrotated tail of a q or k head
    T* x = is_v ? row + (size_t)(H + G) * hd + (size_t)(hs - H - G) * vd : row + (size_t)hs * hd;
    float y0 = rl_ld(x + i0), y1 = rl_ld(x + i1);
    if (rotate) {
      float s, c;
      sincosf((float)pos * inv_freq[i], &s, &c);
      const float x0 = y0, x1 = y1;
      y0 = x0 * c - x1 * s;
      y1 = x0 * s + x1 * c;
    }
    if (hs < H) {
      if (rotate) { rl_st(x + i0, y0); rl_st(x + i1, y1); }
    } else if (write_cache) {
      T* d = is_v ? v_pool + dst_v + (size_t)(hs - H - G) * RL_PAGE * vd : k_pool + dst + (size_t)(hs - H) * RL_PAGE * hd;
      if (rotate) { rl_st(d + i0, y0); rl_st(d + i1, y1); }
      else { d[i0] = x[i0]; d[i1] = x[i1]; }                  // bit copy
    } else if (rotate) {
      rl_st(x + i0, y0); rl_st(x + i1, y1);                   // no cache: keys rotate in place
    }
  }
}

// Fast path: bf16, half-split pairing over the whole head, head size a multiple of 16,
// 16-byte aligned rows.  A thread rotates eight pairs (two 16-byte loads, two 16-byte
// stores) or copies sixteen value elements.  The token's sines and cosines are the same
// for all its heads: the CTA computes them once into shared memory.
#define ROPE_FAST_HEADS_PER_CTA 16
__global__ void __launch_bounds__(ROPE_THREADS)
rope_kv_write_bf16_half_kernel(__nv_bfloat16* __restrict__ qkv, int ld, const int* __restrict__ positions,
                               const int* __restrict__ slot_of_token, const int* __restrict__ page_table, int max_pages,
                               const float* __restrict__ inv_freq, int H, int G, int hd,
                               __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool) {
  __shared__ float2 cs[128];                              // (cos, sin) of the token's hd / 2 <= 128 angles
  rl_pdl_trigger();
  rl_pdl_wait();
  const int m = blockIdx.x;
  const int pos = positions[m];
  __nv_bfloat16* row = qkv + (size_t)m * ld;
  const int slot = slot_of_token[m];
  const int page = page_table[(size_t)slot * max_pages + pos / RL_PAGE];
  const size_t dst = ((size_t)page * G) * RL_PAGE * hd + (size_t)(pos % RL_PAGE) * hd;
  const int half = hd / 2, per_head = half / 8;          // groups of eight pairs a head
  const int slot0 = blockIdx.y * ROPE_FAST_HEADS_PER_CTA;
  const int nslots = min(ROPE_FAST_HEADS_PER_CTA, H + 2 * G - slot0);
  for (int i = threadIdx.x; i < half; i += ROPE_THREADS) {
    float sn, c;
    sincosf((float)pos * inv_freq[i], &sn, &c);
    cs[i] = make_float2(c, sn);
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < nslots * per_head; idx += ROPE_THREADS) {
    const int hs = slot0 + idx / per_head;
    const int i = (idx % per_head) * 8;
    __nv_bfloat16* x = row + (size_t)hs * hd;
    const uint4 lo = *reinterpret_cast<const uint4*>(x + i);
    const uint4 hi = *reinterpret_cast<const uint4*>(x + i + half);
    if (hs >= H + G) {                                     // values: bit copy
      __nv_bfloat16* d = v_pool + dst + (size_t)(hs - H - G) * RL_PAGE * hd;
      *reinterpret_cast<uint4*>(d + i) = lo;
      *reinterpret_cast<uint4*>(d + i + half) = hi;
      continue;
    }
    const __nv_bfloat162* l2 = reinterpret_cast<const __nv_bfloat162*>(&lo);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&hi);
    uint4 olo, ohi;
    __nv_bfloat162* ol = reinterpret_cast<__nv_bfloat162*>(&olo);
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&ohi);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 a = __bfloat1622float2(l2[k]), b = __bfloat1622float2(h2[k]);
      const float c0 = cs[i + 2 * k].x, s0 = cs[i + 2 * k].y, c1 = cs[i + 2 * k + 1].x, s1 = cs[i + 2 * k + 1].y;
      ol[k] = __floats2bfloat162_rn(a.x * c0 - b.x * s0, a.y * c1 - b.y * s1);
      oh[k] = __floats2bfloat162_rn(a.x * s0 + b.x * c0, a.y * s1 + b.y * c1);
    }
    __nv_bfloat16* d = hs < H ? x : k_pool + dst + (size_t)(hs - H) * RL_PAGE * hd;
    *reinterpret_cast<uint4*>(d + i) = olo;
    *reinterpret_cast<uint4*>(d + i + half) = ohi;
  }
}

// qkv: [M, ld] holding per token H query heads and G key heads of head_dim, then G value
// heads of value_dim (even; it may differ from head_dim).  Queries are rotated in place;
// rotated keys go to k_pool [pages, G, RL_PAGE, head_dim] and the values to v_pool
// [pages, G, RL_PAGE, value_dim] (same dtype as qkv).  With k_pool == nullptr nothing is
// cached and the keys are rotated in place as well.
extern "C" int rl_rope_kv_write(void* qkv, int dtype, int ld, const int* positions,
                                const int* slot_of_token, const int* page_table, int max_pages,
                                const float* inv_freq, int num_tokens, int num_heads, int num_kv_heads,
                                int head_dim, int value_dim, int rotary_dim, int interleaved, void* k_pool,
                                void* v_pool, cudaStream_t stream) {
  RL_REQUIRE(num_tokens >= 0 && num_heads > 0 && num_kv_heads > 0, "rl_rope_kv_write: bad sizes");
  RL_REQUIRE(head_dim > 0 && head_dim <= 256, "rl_rope_kv_write: head_dim %d outside (0, 256]", head_dim);
  RL_REQUIRE(rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0,
             "rl_rope_kv_write: rotary_dim %d must be even and <= head_dim %d", rotary_dim, head_dim);
  RL_REQUIRE(value_dim > 0 && value_dim <= 256 && value_dim % 2 == 0, "rl_rope_kv_write: value_dim %d must be even and in (0, 256]", value_dim);
  RL_REQUIRE(ld >= (num_heads + num_kv_heads) * head_dim + num_kv_heads * value_dim, "rl_rope_kv_write: row stride %d too small", ld);
  RL_REQUIRE((k_pool == nullptr) == (v_pool == nullptr), "rl_rope_kv_write: give both cache pools or none");
  if (num_tokens == 0) return RL_OK;
  const int write_cache = k_pool != nullptr;
  RL_REQUIRE(head_dim % 2 == 0, "rl_rope_kv_write: head_dim %d must be even", head_dim);
  const dim3 grid(num_tokens, (num_heads + 2 * num_kv_heads + ROPE_HEADS_PER_CTA - 1) / ROPE_HEADS_PER_CTA);
  const int threads = ROPE_THREADS;
  if (dtype == RL_BF16 && write_cache && !interleaved && rotary_dim == head_dim && value_dim == head_dim && head_dim % 16 == 0 && ld % 8 == 0 &&
      ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)k_pool & 15) == 0 && ((uintptr_t)v_pool & 15) == 0)
    rl_launch_pdl(rope_kv_write_bf16_half_kernel,
                  dim3(num_tokens, (num_heads + 2 * num_kv_heads + ROPE_FAST_HEADS_PER_CTA - 1) / ROPE_FAST_HEADS_PER_CTA),
                  threads, 0, stream, (__nv_bfloat16*)qkv, ld, positions,
                  slot_of_token, page_table, max_pages, inv_freq, num_heads, num_kv_heads, head_dim,
                  (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool);
  else if (dtype == RL_F32)
    rl_launch_pdl(rope_kv_write_kernel<float>, grid, threads, 0, stream,
        (float*)qkv, ld, positions, slot_of_token, page_table, max_pages, inv_freq, num_heads,
        num_kv_heads, head_dim, value_dim, rotary_dim, interleaved, (float*)k_pool, (float*)v_pool, write_cache);
  else if (dtype == RL_BF16)
    rl_launch_pdl(rope_kv_write_kernel<__nv_bfloat16>, grid, threads, 0, stream,
        (__nv_bfloat16*)qkv, ld, positions, slot_of_token, page_table, max_pages, inv_freq, num_heads,
        num_kv_heads, head_dim, value_dim, rotary_dim, interleaved, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, write_cache);
  else
    RL_REQUIRE(false, "rl_rope_kv_write: unknown dtype %d", dtype);
  RL_LAUNCH_CHECK("rl_rope_kv_write");
  return RL_OK;
}
