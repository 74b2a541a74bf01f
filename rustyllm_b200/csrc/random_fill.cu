// Random weights that are the same numbers wherever they are drawn: element i of a tensor is a
// function of (the tensor's seed, i) alone, made of integer arithmetic and one float multiply, so
// the device kernel here and the host code (weights/random_init.py) agree bit for bit.
//
// value = mean + std * z, z = (sum of twelve uniform 16-bit integers - 393,210) / 65,536: the
// classic twelve-uniform approximation of a standard normal (mean 0, variance 1 - 2^-32, steps of
// 2^-16, |z| <= 6).  The thirty-six bytes come from three rounds of the splitmix64 mixer over
// the counter seed + 3 i (+ 0, 1, 2).  The reference has random weights only in its tests (byte
// patterns, SimonWaldherr/RustyLLM src/model.rs:2451-2478); nothing here follows its generator.
#include "common.cuh"

__host__ __device__ __forceinline__ uint64_t rl_splitmix64(uint64_t x) {
  uint64_t z = x + 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

__host__ __device__ __forceinline__ int rl_twelve_uniforms(uint64_t seed, uint64_t i) {
  int sum = 0;
#pragma unroll
  for (int r = 0; r < 3; ++r) {
    const uint64_t h = rl_splitmix64(seed + 3ull * i + (uint64_t)r);
    sum += (int)(h & 0xffffu) + (int)((h >> 16) & 0xffffu) + (int)((h >> 32) & 0xffffu) + (int)(h >> 48);
  }
  return sum - 393210;      // 12 * 32767.5
}

template <typename T>
__global__ void random_fill_kernel(T* __restrict__ out, long long n, uint64_t seed, float mean, float step) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    rl_st(out + i, __fadd_rn(mean, __fmul_rn((float)rl_twelve_uniforms(seed, (uint64_t)i), step)));   // two roundings, never fused: as the host's
}

// out[i] = mean + std * z_i for i in [0, n), rounded once to the tensor's dtype (nearest even).
extern "C" int rl_random_fill(void* out, int dtype, long long n, unsigned long long seed, float mean, float std, cudaStream_t stream) {
  RL_REQUIRE(n >= 0 && out != nullptr, "rl_random_fill: null output or negative size");
  if (n == 0) return RL_OK;
  const float step = std * (1.0f / 65536.0f);
  const int threads = 256;
  const long long want = (n + threads - 1) / threads;
  const int blocks = (int)(want < (long long)rl_num_sms() * 32 ? want : (long long)rl_num_sms() * 32);
  if (dtype == RL_F32) random_fill_kernel<float><<<blocks, threads, 0, stream>>>((float*)out, n, seed, mean, step);
  else if (dtype == RL_BF16) random_fill_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((__nv_bfloat16*)out, n, seed, mean, step);
  else RL_REQUIRE(false, "rl_random_fill: unknown dtype %d", dtype);
  RL_LAUNCH_CHECK("rl_random_fill");
  return RL_OK;
}
