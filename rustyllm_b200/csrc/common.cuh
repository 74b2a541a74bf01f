// Shared declarations of the kernel library: dtype tags, error reporting, small
// device helpers.  Every entry point is extern "C", takes raw device pointers and a
// stream, checks its sizes on the host and returns 0 or a negative code; the text
// of the last error is read with rl_last_error().
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

enum RlDtype { RL_F32 = 0, RL_BF16 = 1 };

enum RlStatus {
  RL_OK = 0,
  RL_ERR_ARG = -1,       // a size or option the kernel refuses
  RL_ERR_CUDA = -2,      // the CUDA runtime reported an error
  RL_ERR_TIMEOUT = -3,   // a bounded device-side wait ran out
};

// Tokens per page of the key/value cache.  Fixed for the library: attention
// kernels tile the keys by pages.
#define RL_PAGE 64

void rl_set_error(const char* fmt, ...);
int rl_num_sms();   // SMs of the current device (148 where no device can be asked)

#define RL_REQUIRE(cond, ...)            \
  do {                                   \
    if (!(cond)) {                       \
      rl_set_error(__VA_ARGS__);         \
      return RL_ERR_ARG;                 \
    }                                    \
  } while (0)

#define RL_LAUNCH_CHECK(what)                                            \
  do {                                                                   \
    cudaError_t e_ = cudaGetLastError();                                 \
    if (e_ != cudaSuccess) {                                             \
      rl_set_error("%s: %s", what, cudaGetErrorString(e_));              \
      return RL_ERR_CUDA;                                                \
    }                                                                    \
  } while (0)

// ---- loads and stores through float, for float and bf16 storage ----
__device__ __forceinline__ float rl_ld(const float* p) { return *p; }
__device__ __forceinline__ float rl_ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void rl_st(float* p, float v) { *p = v; }
__device__ __forceinline__ void rl_st(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float rl_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float rl_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- programmatic dependent launch ----
// Kernels of a step are launched so that a kernel may start while its predecessor on
// the stream still runs: its launch, block scheduling and prologue (and, in the matrix
// products, the first loads of weights, which no kernel of a step writes) overlap the
// predecessor's tail.  Every such kernel calls rl_pdl_trigger() first and rl_pdl_wait()
// before it reads anything a predecessor wrote or writes anything at all; the wait
// returns once all earlier kernels have completed and their writes are visible.  In a
// kernel launched the ordinary way both are no-ops.
__device__ __forceinline__ void rl_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void rl_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// 1 (default): launch with programmatic stream serialization; 0: ordinary launches
// (rl_set_pdl, for measurements and for bisecting a fault).
extern int g_rl_pdl_enabled;

template <typename... KArgs, typename... Args>
static inline cudaError_t rl_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                        cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_rl_pdl_enabled ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
