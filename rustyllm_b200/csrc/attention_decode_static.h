// rl_attention_decode_static: decode attention for callers that cannot allocate.
//
// This entry point has no counterpart in SimonWaldherr/RustyLLM; it exists for users of
// this library.
//
// Who it is for.  rl_attention_decode splits long contexts over many thread blocks and
// needs a few hundred kilobytes of scratch for the per-split partial results, which the
// caller allocates.  Some callers cannot: a decode loop that must not call cudaMalloc or
// cudaFree because either may stall the whole device while it waits for running work; a
// host application that has handed every free byte of device memory to its own pools
// (this library's key/value cache is sized that way) so that a late allocation would
// fail; code that is handed only raw pointers and a stream and has no allocator to ask.
// For them the scratch is a fixed array inside the library.
//
// What it does.  Exactly what rl_attention_decode does without a plan (every sequence in
// num_splits equal chunks, a second kernel combines them), with the same arguments minus
// `scratch` and `plan`.  It calls no cudaMalloc, cudaFree or other allocating routine.
//
// Limits and rules.
//  * The built-in scratch holds RL_DECODE_STATIC_SCRATCH_FLOATS floats (4 MiB).  A call
//    needs num_seqs * num_heads * num_splits * (head_dim + 2) floats when num_splits > 1
//    and none with one split; a call that needs more is refused with an error that says
//    so (nothing is launched).  For example 64 sequences x 32 heads x 3 splits x 130.
//  * Every GPU that loads the library holds the array until the process exits.
//  * The first call on a device looks up the array's device address
//    (cudaGetSymbolAddress, with that device current) and keeps it; make that first
//    call before any stream capture begins.  Devices 0 .. RL_DECODE_STATIC_MAX_DEVICES-1.
//  * All calls share the one array and it keeps the last call's contents.  Nothing in it
//    has to start at zero: every element a call reads it has written before.  But two
//    calls that overlap on the GPU (different streams, no ordering between them) race
//    on it; order them, or give the second one rl_attention_decode with its own scratch.
#pragma once
#include <cuda_runtime.h>

#define RL_DECODE_STATIC_SCRATCH_FLOATS (1u << 20)
#define RL_DECODE_STATIC_MAX_DEVICES 64

#ifdef __cplusplus
extern "C" {
#endif
int rl_attention_decode_static(const void* q, int ldq, const void* k_pool, const void* v_pool,
                                          const int* page_table, int max_pages, const int* seq_slots,
                                          const int* kv_lens, void* out, int ldo, int num_seqs, int num_heads,
                                          int num_kv_heads, int head_dim, float scale, int window, int num_splits,
                                          cudaStream_t stream);
#ifdef __cplusplus
}
#endif
