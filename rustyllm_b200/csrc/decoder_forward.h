// Plain descriptions of a decoder whose parts this library's native executor knows
// (decoder_forward.cu), filled from Python through ctypes.  All pointers are device pointers
// that the caller keeps alive; all matrices are bfloat16, row-major [rows, columns].
#pragma once
#include <cuda_runtime.h>

struct RlLinear {
  const void* w;        // [n, k]
  const float* bias;    // [n] or null
  int n, k;
};

struct RlNormW {
  const float* w;       // [hidden]
  float eps;
};

struct RlLayerDesc {
  RlNormW norm1, norm2;
  RlLinear qkv;         // rows: query heads, key heads, value heads
  RlLinear o;
  RlLinear gate_up;     // rows: gate_0, up_0, gate_1, up_1, ...
  RlLinear down;
  int num_heads, num_kv_heads, head_dim, value_dim, rotary_dim, interleaved_rope, window;
  float scale;
  const float* inv_freq;
  int intermediate;
};

// One run of a layer in the schedule, with the cache entry it reads (and writes, if it owns it).
struct RlRunDesc {
  int layer;
  void* k_pool;         // [pages, kv_heads, page, head_dim]
  void* v_pool;         // [pages, kv_heads, page, value_dim]
  const int* page_table;
  int max_pages, num_pages, writes;
};

struct RlModelDesc {
  int hidden, vocab, num_layers, num_runs;
  const RlLayerDesc* layers;
  const RlRunDesc* runs;
  const void* embed;    // [vocab, hidden]
  RlNormW final_norm;
  RlLinear head;
};

// The integers of one step, on the device, and what the host knows of its shape.
struct RlStepDesc {
  int M, B, is_decode;
  const int* tokens;
  const int* positions;
  const int* slot_of_token;
  const int* cu_seqlens;
  const int* seq_slots;
  const int* kv_lens;
  int tiles_tc, tiles_mma;      // query tiles of 128 and of 64 tokens over the step's sequences
  const int* tile_order;        // for the tcgen05 prefill attention (may be null)
  int long_context;             // the longest sequence holds more tokens than one cluster of chunks serves well
  int length_spread;            // 0 the longest sequence within 16 tokens of the mean, 1 within 768, 2 within 4096 and at most a twentieth of all tokens, 3 the rest
};

#ifdef __cplusplus
extern "C" {
#endif
long long rl_decoder_workspace_bytes(const RlModelDesc* m, int num_tokens, int num_seqs);
int rl_decoder_forward(const RlModelDesc* m, const RlStepDesc* s, float* x, void* workspace, long long workspace_bytes,
                       int* err, int* bad_token, cudaStream_t stream);
int rl_decoder_last_launches(void);
int rl_decoder_logits(const RlModelDesc* m, const float* x, const int* want_rows, int num_rows, void* xn, float* logits,
                      int* err, cudaStream_t stream);
#ifdef __cplusplus
}
#endif
