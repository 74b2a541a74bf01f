// The launch chain of a decoder step in native code: embedding, every scheduled layer
// (pre-norm block of grouped-query attention and gated feed-forward), and the final norm with
// the head at the wanted rows - the same kernels, in the same order and with the same choices
// (norms folded into products up to 64 tokens, rotation in the QKV epilogue, the attention
// kernel for the step's shape) as the Python parts make them, without the interpreter between
// two launches.  SimonWaldherr/RustyLLM's runtime is native throughout (src/runtime.rs:3145-3428,
// src/model.rs:7177-7358); here the description of the model stays data (which parts, which
// constants), handed over once as plain structs, and this file is the executor for the parts
// it knows.  A model with any other part runs through the Python parts instead.
//
// An eager step of a few tokens is bound by how fast its ~7 launches a layer are issued; from
// Python that is about 16 us a launch, from here about 3.
#include <stdint.h>

#include "common.cuh"
#include "decoder_forward.h"

extern "C" {
int rl_embedding(const void* table, int table_dtype, const int* ids, float* out, int num_tokens, int dim, int vocab, int* err_flag, cudaStream_t stream);
int rl_rmsnorm(const float* x, const float* weight, void* out, int out_dtype, const int* rows, int num_rows, int dim, float eps, cudaStream_t stream);
int rl_gemm_tc_supported(const void* A, const void* W, int M, int N, int K, int lda);
int rl_gemm_tc(const void* A, const void* W, const float* bias, void* out, int out_mode, int M, int N, int K, int lda, int ldo, int* err,
               int force_splits, const float* scale_partials, int scale_count, float scale_eps, const float* norm_weight, void* norm_out,
               int ld_norm, float* norm_partials, cudaStream_t stream);
int rl_gemm_tc_qkv_rope_supported(int M, int num_heads, int num_kv_heads, int head_dim, int rotary_dim, int K);
int rl_gemm_tc_qkv_rope(const void* A, const void* W, const float* bias, void* out, int M, int K, int lda, int ldo, int* err,
                        const float* scale_partials, int scale_count, float scale_eps, const int* positions, const int* slot_of_token,
                        const int* page_table, int max_pages, const float* inv_freq, int interleaved, int num_heads, int num_kv_heads,
                        int head_dim, void* k_pool, void* v_pool, cudaStream_t stream);
int rl_rope_kv_write(void* qkv, int dtype, int ld, const int* positions, const int* slot_of_token, const int* page_table, int max_pages,
                     const float* inv_freq, int num_tokens, int num_heads, int num_kv_heads, int head_dim, int value_dim, int rotary_dim,
                     int interleaved, void* k_pool, void* v_pool, cudaStream_t stream);
int rl_attention_simt(const void* q, int ldq, const void* k_pool, const void* v_pool, int dtype, const int* page_table, int max_pages,
                      const int* slot_of_token, const int* positions, void* out, int ldo, int num_tokens, int num_heads, int num_kv_heads,
                      int head_dim, int value_dim, float scale, int window, cudaStream_t stream);
int rl_attention_decode_supported(int num_heads, int num_kv_heads, int head_dim);
long long rl_attention_decode_plan_ints(int num_seqs, int num_splits);
long long rl_attention_decode_scratch_floats(int num_seqs, int num_heads, int head_dim, int num_splits);
int rl_attention_decode_plan(const int* seq_slots, const int* kv_lens, int num_seqs, int window, int num_splits, int* plan, cudaStream_t stream);
int rl_attention_decode_places(int head_dim);
int rl_attention_decode_ring_bytes(int head_dim);
int rl_attention_decode_order(const int* seq_slots, const int* kv_lens, int num_seqs, int window, int* plan, cudaStream_t stream);
int rl_attention_decode(const void* q, int ldq, const void* k_pool, const void* v_pool, const int* page_table, int max_pages,
                        const int* seq_slots, const int* kv_lens, void* out, int ldo, float* scratch, const int* plan, int num_seqs,
                        int num_heads, int num_kv_heads, int head_dim, float scale, int window, int num_splits, cudaStream_t stream);
int rl_attention_prefill_supported(int num_heads, int num_kv_heads, int head_dim);
int rl_attention_prefill(const void* q, int ldq, const void* k_pool, const void* v_pool, const int* page_table, int max_pages,
                         const int* cu_seqlens, const int* seq_slots, const int* kv_lens, int num_seqs, int num_tiles, void* out, int ldo,
                         int num_heads, int num_kv_heads, int head_dim, float scale, int window, cudaStream_t stream);
int rl_attention_prefill_tc_supported(int num_heads, int num_kv_heads, int head_dim);
int rl_attention_prefill_tc(const void* q, int ldq, const void* k_pool, const void* v_pool, int num_pages, const int* page_table,
                            int max_pages, const int* cu_seqlens, const int* seq_slots, const int* kv_lens, int num_seqs, int num_tiles,
                            int num_tokens, void* out, int ldo, int num_heads, int num_kv_heads, int head_dim, float scale, int window,
                            int* err, const int* tile_order, cudaStream_t stream);
}

namespace {

thread_local int g_launches = 0;     // kernels launched by the last rl_decoder_forward / rl_decoder_logits of this thread

enum { OUT_SAME = 0, OUT_F32 = 1, OUT_ADD_F32 = 2, OUT_SWIGLU = 3 };
constexpr int FOLD_NORMS_UP_TO = 64;     // tokens: above, a norm's own kernel costs less than what folding adds to the products

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
inline int norm_pieces(int n) { return 4 * ((n + 127) / 128); }

// A norm that a product has started: x * weight in bf16 and the rows' sums of squares in pieces.
struct Normed {
  const void* weighted;     // [M, d] bf16
  const float* sumsq;       // [M, pieces]; null: `weighted` is the finished norm (its own kernel made it)
  int pieces;
  float eps;
};

// bump allocator over the step's workspace
struct Arena {
  uint8_t* base;
  size_t size, used;
  void* take(size_t bytes) {
    const size_t at = align_up(used, 256);
    if (at + bytes > size) return nullptr;
    used = at + bytes;
    return base + at;
  }
};

struct StepBuffers {
  // One buffer serves every norm of the step: a norm is read by exactly one product (QKV, or gate
  // and up), and the product that writes the next norm into it is launched behind that reader.
  void* normed;             // [M, d] bf16
  float* sumsq;             // [M, pieces(d)]
  void* qkv;                // [M, widest qkv row]
  void* attn;               // [M, widest H * vd]
  void* hidden;             // [M, widest intermediate]
  float* dec_scratch;
  int* dec_plan;
  int plan_window, plan_splits;     // what the plan in dec_plan was made for (-1: none yet)
};

int decode_splits(int num_seqs, int num_kv_heads) {
  const int most = num_seqs == 1 ? 16 : 8, least = num_seqs == 1 ? 1 : 2;
  int s = (3 * rl_num_sms() + 2 * num_seqs * num_kv_heads - 1) / (2 * num_seqs * num_kv_heads);
  if (s > most) s = most;
  if (s < least) s = least;
  return s;
}

// Whole sequences that are more CTAs than the GPU holds at once (and keep 30 MB in flight among
// them) start in the order of their lengths, the longest first (64 sequences of 128 to 2,047 tokens
// at head size 128: 43 us, 6.45 TB/s, against 54 us in the order of the batch); the order kernel
// takes up to 1,024 sequences.
bool decode_order_wanted(int num_seqs, int num_kv_heads, int head_dim) {
  const long long ctas = (long long)num_seqs * num_kv_heads;
  return ctas > rl_attention_decode_places(head_dim) && ctas * rl_attention_decode_ring_bytes(head_dim) >= 30000000LL && num_seqs <= 1024;
}

// How the decode attention cuts the sequences of a step: 8, 4 or 2 = so many equal chunks a sequence
// as one cluster; 1 = every sequence whole in one CTA a KV head; 0 = chunks dealt to the sequences by
// their lengths and combined by a second kernel.  Equal chunks cost a kernel less (about 2.5 us a
// layer) and lose where sequences are unequal.  length_spread: 0 the longest sequence within 16
// tokens of the mean of all, 1 within 768, 2 within 4,096 and no more than a twentieth of all
// tokens, 3 the rest.  One sequence alone takes eight chunks up to the long-context mark.  Whole
// sequences in order (decode_order_wanted) serve every batch up to spread 2.  Else, lengths that
// are equal or near (spread 0, 1): where two chunks a sequence no longer fit the GPU at once (a
// second wave of clusters costs more than it brings), every sequence whole if that keeps 15 MB in
// flight; else the largest power of two within their splits - for spread 1 only if nothing is
// lost to the rounding.  (kernels.decode_cluster_size is the same rule; measured on whole steps of
// 2 to 64 sequences at head size 128 and on the kernel alone at head size 64.)
int decode_cluster(int num_seqs, int num_kv_heads, int head_dim, int splits, int long_context, int length_spread) {
  if (num_seqs == 1) return (splits >= 8 && !long_context) ? 8 : 0;
  if (splits < 2) return 0;
  if (decode_order_wanted(num_seqs, num_kv_heads, head_dim)) return length_spread <= 2 ? 1 : 0;
  if (length_spread > 1) return 0;
  const int places = rl_attention_decode_places(head_dim);
  const long long ctas = (long long)num_seqs * num_kv_heads;
  if (ctas * 2 > places) return ctas * rl_attention_decode_ring_bytes(head_dim) >= 15000000LL ? 1 : 0;
  const int size = splits >= 8 ? 8 : splits >= 4 ? 4 : 2;
  if (length_spread == 1 && size != splits) return 0;
  return ctas * size <= places ? size : 0;
}

bool can_fold(const RlLinear& l, int M) {
  return M <= FOLD_NORMS_UP_TO && l.w != nullptr && l.k % 8 == 0 && ((uintptr_t)l.w & 15) == 0;
}

// out = a W^T (+ bias) on the tensor cores, with the norm work around it: `in` may be a started
// norm (finished here), `then` a norm to start (add-into-residual mode).  Returns RL_OK or a code.
int product(const RlLinear& l, const void* a, int lda, const Normed* in, void* out, int ldo, int mode, int M, int* err,
            const RlNormW* then, void* then_out, float* then_sumsq, cudaStream_t stream) {
  const float* sp = (in != nullptr && in->sumsq != nullptr) ? in->sumsq : nullptr;
  ++g_launches;
  return rl_gemm_tc(a, l.w, l.bias, out, mode, M, l.n, l.k, lda, ldo, err, 0, sp, sp ? in->pieces : 0, sp ? in->eps : 0.f,
                    then ? then->w : nullptr, then ? then_out : nullptr, l.n, then ? then_sumsq : nullptr, stream);
}

int attention(const RlLayerDesc& L, const RlRunDesc& R, const RlStepDesc& S, StepBuffers& B, int ldq, int* err, cudaStream_t stream) {
  const int H = L.num_heads, G = L.num_kv_heads, hd = L.head_dim, vd = L.value_dim;
  const bool same = vd == hd;
  if (same && S.is_decode && rl_attention_decode_supported(H, G, hd)) {
    const int splits = decode_splits(S.B, G);
    ++g_launches;
    const int cluster = decode_cluster(S.B, G, hd, splits, S.long_context, S.length_spread);
    if (cluster > 0) {     // equal chunks a sequence as one cluster, combined through shared memory, or whole sequences: one kernel
      const int* order = nullptr;
      if (cluster == 1 && decode_order_wanted(S.B, G, hd)) {
        if (B.plan_window != L.window || B.plan_splits != 1) {        // once a step for all layers of one window
          const int rc = rl_attention_decode_order(S.seq_slots, S.kv_lens, S.B, L.window, B.dec_plan, stream);
          if (rc != RL_OK) return rc;
          ++g_launches;
          B.plan_window = L.window; B.plan_splits = 1;
        }
        order = B.dec_plan;
      }
      return rl_attention_decode(B.qkv, ldq, R.k_pool, R.v_pool, R.page_table, R.max_pages, S.seq_slots, S.kv_lens, B.attn, H * hd,
                                 nullptr, order, S.B, H, G, hd, L.scale, L.window, cluster, stream);
    }
    const int* plan = nullptr;
    if (splits > 1 && S.B > 1) {
      if (B.plan_window != L.window || B.plan_splits != splits) {     // once a step for all layers of one window
        const int rc = rl_attention_decode_plan(S.seq_slots, S.kv_lens, S.B, L.window, splits, B.dec_plan, stream);
        if (rc != RL_OK) return rc;
        ++g_launches;
        B.plan_window = L.window; B.plan_splits = splits;
      }
      plan = B.dec_plan;
    }
    if (splits > 1) ++g_launches;       // the combining kernel
    return rl_attention_decode(B.qkv, ldq, R.k_pool, R.v_pool, R.page_table, R.max_pages, S.seq_slots, S.kv_lens, B.attn, H * hd,
                               splits > 1 ? B.dec_scratch : nullptr, plan, S.B, H, G, hd, L.scale, L.window, splits, stream);
  }
  ++g_launches;
  if (same && !S.is_decode && rl_attention_prefill_tc_supported(H, G, hd) && ldq % 8 == 0 && ((uintptr_t)B.qkv & 15) == 0)
    return rl_attention_prefill_tc(B.qkv, ldq, R.k_pool, R.v_pool, R.num_pages, R.page_table, R.max_pages, S.cu_seqlens, S.seq_slots,
                                   S.kv_lens, S.B, S.tiles_tc, S.M, B.attn, H * hd, H, G, hd, L.scale, L.window, err,
                                   S.B > 1 ? S.tile_order : nullptr, stream);
  if (same && !S.is_decode && rl_attention_prefill_supported(H, G, hd))
    return rl_attention_prefill(B.qkv, ldq, R.k_pool, R.v_pool, R.page_table, R.max_pages, S.cu_seqlens, S.seq_slots, S.kv_lens, S.B,
                                S.tiles_mma, B.attn, H * hd, H, G, hd, L.scale, L.window, stream);
  return rl_attention_simt(B.qkv, ldq, R.k_pool, R.v_pool, RL_BF16, R.page_table, R.max_pages, S.slot_of_token, S.positions, B.attn,
                           H * vd, S.M, H, G, hd, vd, L.scale, L.window, stream);
}

// One block: x += attention(norm1(x)); x += feed-forward(norm2(x)).  `pending`: the block's first
// norm has been started by the block in front (it lies in the norm buffer); `next`: the next
// block's first norm, to be started by the down product (null: none).
int block(const RlLayerDesc& L, const RlRunDesc& R, const RlStepDesc& S, StepBuffers& B, float* x, int d, bool pending,
          const RlNormW* next, int* err, cudaStream_t stream) {
  const int M = S.M, H = L.num_heads, G = L.num_kv_heads, hd = L.head_dim, vd = L.value_dim;
  const int ldq = (H + G) * hd + G * vd, pieces = norm_pieces(d);
  int rc;
  // ---- first norm: started by the block in front, or its own kernel ----
  Normed in1{B.normed, pending ? B.sumsq : nullptr, pieces, L.norm1.eps};
  if (!pending) {
    rc = rl_rmsnorm(x, L.norm1.w, B.normed, RL_BF16, nullptr, M, d, L.norm1.eps, stream);
    if (rc != RL_OK) return rc;
    ++g_launches;
  }
  // ---- query, key, value: rotation and cache write in the product's epilogue where it takes them ----
  void* kp = R.writes ? R.k_pool : nullptr;
  void* vp = R.writes ? R.v_pool : nullptr;
  if (vd == hd && rl_gemm_tc_qkv_rope_supported(M, H, G, hd, L.rotary_dim, L.qkv.k)) {
    const float* sp = in1.sumsq;
    rc = rl_gemm_tc_qkv_rope(in1.weighted, L.qkv.w, L.qkv.bias, B.qkv, M, L.qkv.k, d, ldq, err, sp, sp ? in1.pieces : 0, sp ? in1.eps : 0.f,
                             S.positions, S.slot_of_token, R.page_table, R.max_pages, L.inv_freq, L.interleaved_rope, H, G, hd, kp, vp, stream);
    if (rc != RL_OK) return rc;
    ++g_launches;
  } else {
    rc = product(L.qkv, in1.weighted, d, &in1, B.qkv, ldq, OUT_SAME, M, err, nullptr, nullptr, nullptr, stream);
    if (rc != RL_OK) return rc;
    rc = rl_rope_kv_write(B.qkv, RL_BF16, ldq, S.positions, S.slot_of_token, R.page_table, R.max_pages, L.inv_freq, M, H, G, hd, vd,
                          L.rotary_dim, L.interleaved_rope, kp, vp, stream);
    if (rc != RL_OK) return rc;
    ++g_launches;
  }
  rc = attention(L, R, S, B, ldq, err, stream);
  if (rc != RL_OK) return rc;
  // ---- output projection into the residual; it starts the second norm where the feed-forward can finish it ----
  const bool fold2 = can_fold(L.gate_up, M);
  rc = product(L.o, B.attn, H * vd, nullptr, x, d, OUT_ADD_F32, M, err, fold2 ? &L.norm2 : nullptr, B.normed, B.sumsq, stream);
  if (rc != RL_OK) return rc;
  Normed in2{B.normed, fold2 ? B.sumsq : nullptr, pieces, L.norm2.eps};
  if (!fold2) {
    rc = rl_rmsnorm(x, L.norm2.w, B.normed, RL_BF16, nullptr, M, d, L.norm2.eps, stream);
    if (rc != RL_OK) return rc;
    ++g_launches;
  }
  // ---- feed-forward: gate and up with the activation in the epilogue, then down into the residual ----
  rc = product(L.gate_up, in2.weighted, d, &in2, B.hidden, L.intermediate, OUT_SWIGLU, M, err, nullptr, nullptr, nullptr, stream);
  if (rc != RL_OK) return rc;
  return product(L.down, B.hidden, L.intermediate, nullptr, x, d, OUT_ADD_F32, M, err, next, B.normed, B.sumsq, stream);
}

}  // namespace

// Bytes of workspace rl_decoder_forward needs for a step of num_tokens tokens in num_seqs sequences.
extern "C" long long rl_decoder_workspace_bytes(const RlModelDesc* m, int num_tokens, int num_seqs) {
  size_t qkv = 0, attn = 0, hidden = 0;
  int max_heads = 1, max_hd = 1;
  for (int i = 0; i < m->num_layers; ++i) {
    const RlLayerDesc& L = m->layers[i];
    const size_t q = (size_t)(L.num_heads + L.num_kv_heads) * L.head_dim + (size_t)L.num_kv_heads * L.value_dim;
    if (q > qkv) qkv = q;
    if ((size_t)L.num_heads * L.value_dim > attn) attn = (size_t)L.num_heads * L.value_dim;
    if ((size_t)L.intermediate > hidden) hidden = L.intermediate;
    if (L.num_heads > max_heads) max_heads = L.num_heads;
    if (L.head_dim > max_hd) max_hd = L.head_dim;
  }
  const size_t M = num_tokens, d = m->hidden;
  size_t total = 0;
  auto add = [&](size_t bytes) { total = align_up(total, 256) + bytes; };
  add(M * d * 2);
  add(M * norm_pieces((int)d) * 4);
  add(M * qkv * 2); add(M * attn * 2); add(M * hidden * 2);
  add((size_t)rl_attention_decode_scratch_floats(num_seqs, max_heads, max_hd, 16) * 4);
  add((size_t)rl_attention_decode_plan_ints(num_seqs, 16) * 4);
  return (long long)align_up(total, 256);
}

// x: [M, hidden] float, written by the embedding here and updated by every scheduled layer.
// err: the device error word of the tensor-core kernels; bad_token: device int set if a token id
// lies outside the vocabulary.
extern "C" int rl_decoder_forward(const RlModelDesc* m, const RlStepDesc* s, float* x, void* workspace, long long workspace_bytes,
                                  int* err, int* bad_token, cudaStream_t stream) {
  RL_REQUIRE(m != nullptr && s != nullptr && x != nullptr && workspace != nullptr && err != nullptr, "rl_decoder_forward: null argument");
  RL_REQUIRE(s->M > 0 && s->B > 0, "rl_decoder_forward: a step needs tokens and sequences");
  RL_REQUIRE(workspace_bytes >= rl_decoder_workspace_bytes(m, s->M, s->B), "rl_decoder_forward: workspace of %lld bytes is too small", workspace_bytes);
  const int M = s->M, d = m->hidden;
  Arena arena{(uint8_t*)workspace, (size_t)workspace_bytes, 0};
  StepBuffers B = {};
  size_t qkv = 0, attn = 0, hidden = 0;
  int max_heads = 1, max_hd = 1;
  for (int i = 0; i < m->num_layers; ++i) {
    const RlLayerDesc& L = m->layers[i];
    const size_t q = (size_t)(L.num_heads + L.num_kv_heads) * L.head_dim + (size_t)L.num_kv_heads * L.value_dim;
    if (q > qkv) qkv = q;
    if ((size_t)L.num_heads * L.value_dim > attn) attn = (size_t)L.num_heads * L.value_dim;
    if ((size_t)L.intermediate > hidden) hidden = L.intermediate;
    if (L.num_heads > max_heads) max_heads = L.num_heads;
    if (L.head_dim > max_hd) max_hd = L.head_dim;
  }
  B.normed = arena.take((size_t)M * d * 2);
  B.sumsq = (float*)arena.take((size_t)M * norm_pieces(d) * 4);
  B.qkv = arena.take((size_t)M * qkv * 2); B.attn = arena.take((size_t)M * attn * 2); B.hidden = arena.take((size_t)M * hidden * 2);
  B.dec_scratch = (float*)arena.take((size_t)rl_attention_decode_scratch_floats(s->B, max_heads, max_hd, 16) * 4);
  B.dec_plan = (int*)arena.take((size_t)rl_attention_decode_plan_ints(s->B, 16) * 4);
  B.plan_window = -1; B.plan_splits = -1;
  RL_REQUIRE(B.dec_plan != nullptr, "rl_decoder_forward: workspace ran out");

  g_launches = 0;
  int rc = rl_embedding(m->embed, RL_BF16, s->tokens, x, M, d, m->vocab, bad_token, stream);
  if (rc != RL_OK) return rc;
  ++g_launches;
  // The norm a block begins with is started by the down product of the block in front where both
  // can (few tokens); otherwise the block runs the norm's own kernel.
  bool pending = false;
  for (int r = 0; r < m->num_runs; ++r) {
    const RlRunDesc& R = m->runs[r];
    const RlNormW* next = nullptr;
    if (r + 1 < m->num_runs) {
      const RlLayerDesc& N = m->layers[m->runs[r + 1].layer];
      if (can_fold(N.qkv, M)) next = &N.norm1;
    }
    rc = block(m->layers[R.layer], R, *s, B, x, d, pending, next, err, stream);
    if (rc != RL_OK) return rc;
    pending = next != nullptr;
  }
  return RL_OK;
}

// Kernels the last rl_decoder_forward or rl_decoder_logits of the calling thread launched.
extern "C" int rl_decoder_last_launches() { return g_launches; }

// Final norm and head at the wanted rows: logits [W, vocab] float.  xn: [W, hidden] bf16 scratch.
extern "C" int rl_decoder_logits(const RlModelDesc* m, const float* x, const int* want_rows, int num_rows, void* xn, float* logits,
                                 int* err, cudaStream_t stream) {
  RL_REQUIRE(m != nullptr && x != nullptr && want_rows != nullptr && xn != nullptr && logits != nullptr && num_rows > 0,
             "rl_decoder_logits: null argument or no rows");
  int rc = rl_rmsnorm(x, m->final_norm.w, xn, RL_BF16, want_rows, num_rows, m->hidden, m->final_norm.eps, stream);
  if (rc != RL_OK) return rc;
  g_launches = 2;
  return rl_gemm_tc(xn, m->head.w, m->head.bias, logits, OUT_F32, num_rows, m->head.n, m->head.k, m->hidden, m->head.n, err, 0,
                    nullptr, 0, 0.f, nullptr, nullptr, 0, nullptr, stream);
}
