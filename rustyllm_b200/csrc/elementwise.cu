// Embedding gather, RMSNorm, SwiGLU and dtype conversion.
//
// Math in 32-bit throughout; storage of inputs/outputs is float or bf16 as the
// dtype tags say.  The residual stream these kernels read and write is always
// float.
//
// Formulas (SimonWaldherr/RustyLLM):
//   embedding : x = E[token, :]                         src/model.rs:7193
//   rms_norm  : y_i = x_i * 1/sqrt(sum(x^2)/n + eps) * w_i   src/model.rs:5429-5437
//   swiglu    : h_i = g_i / (1 + exp(-g_i)) * u_i       src/simd.rs:2403-2408
#include "common.cuh"

// ------------------------------------------------------------------ embedding
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ out, int d, int vocab, int* __restrict__ err) {
  rl_pdl_trigger();
  rl_pdl_wait();
  const int m = blockIdx.x;
  int id = ids[m];
  if (id < 0 || id >= vocab) {  // refuse instead of reading outside the table
    if (threadIdx.x == 0) atomicExch(err, 1);
    id = 0;
  }
  const T* row = table + (size_t)id * d;
  float* o = out + (size_t)m * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = rl_ld(row + i);
}

// err: optional device int, set to 1 when a token id lies outside [0, vocab).
extern "C" int rl_embedding(const void* table, int table_dtype, const int* ids, float* out,
                            int num_tokens, int hidden, int vocab, int* err, cudaStream_t stream) {
  RL_REQUIRE(num_tokens >= 0 && hidden > 0 && vocab > 0, "rl_embedding: bad sizes M=%d d=%d V=%d",
             num_tokens, hidden, vocab);
  RL_REQUIRE(err != nullptr, "rl_embedding: the error flag pointer is null");
  if (num_tokens == 0) return RL_OK;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (table_dtype == RL_F32)
    rl_launch_pdl(embedding_kernel<float>, num_tokens, threads, 0, stream, (const float*)table, ids, out, hidden, vocab, err);
  else if (table_dtype == RL_BF16)
    rl_launch_pdl(embedding_kernel<__nv_bfloat16>, num_tokens, threads, 0, stream, (const __nv_bfloat16*)table, ids, out, hidden, vocab, err);
  else
    RL_REQUIRE(false, "rl_embedding: unknown table dtype %d", table_dtype);
  RL_LAUNCH_CHECK("rl_embedding");
  return RL_OK;
}

// ------------------------------------------------------------------ RMSNorm
// One block per output row.  The sum of squares is taken in a fixed order that
// depends only on the row length and the block size, never on the batch.
template <typename TO, int THREADS>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                               TO* __restrict__ out, const int* __restrict__ rows, int d, float eps) {
  rl_pdl_trigger();
  rl_pdl_wait();
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * d;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += THREADS) {
    const float v = xr[i];
    ss = fmaf(v, v, ss);
  }
  __shared__ float part[THREADS / 32];
  __shared__ float total;
  ss = rl_warp_sum(ss);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < THREADS / 32; ++i) t += part[i];
    total = 1.0f / sqrtf(t / (float)d + eps);
  }
  __syncthreads();
  const float s = total;
  TO* o = out + (size_t)r * d;
  for (int i = threadIdx.x; i < d; i += THREADS) rl_st(o + i, xr[i] * s * w[i]);
}

// Rows of up to THREADS * 4 * MAXV floats, a multiple of 4 long, 16-byte aligned: the row
// stays in registers between the sum and the scaling, 16-byte loads, 8- or 16-byte stores.
template <typename TO, int THREADS, int MAXV>
__global__ void __launch_bounds__(THREADS)
rmsnorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ out,
                   const int* __restrict__ rows, int d, float eps) {
  rl_pdl_trigger();
  rl_pdl_wait();
  const int r = blockIdx.x;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * d);
  const int nv = d / 4;
  float4 v[MAXV];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int i = threadIdx.x + k * THREADS;
    v[k] = i < nv ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    ss = fmaf(v[k].x, v[k].x, ss); ss = fmaf(v[k].y, v[k].y, ss);
    ss = fmaf(v[k].z, v[k].z, ss); ss = fmaf(v[k].w, v[k].w, ss);
  }
  __shared__ float part[THREADS / 32];
  __shared__ float total;
  ss = rl_warp_sum(ss);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < THREADS / 32; ++i) t += part[i];
    total = 1.0f / sqrtf(t / (float)d + eps);
  }
  __syncthreads();
  const float s = total;
  const float4* w4 = reinterpret_cast<const float4*>(w);
  TO* o = out + (size_t)r * d;
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int i = threadIdx.x + k * THREADS;
    if (i < nv) {
      const float4 g = w4[i];
      const float a = v[k].x * s * g.x, b = v[k].y * s * g.y, c = v[k].z * s * g.z, e = v[k].w * s * g.w;
      if constexpr (sizeof(TO) == 2) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, e);
        *reinterpret_cast<uint2*>(o + 4 * i) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
      } else {
        *reinterpret_cast<float4*>(o + 4 * i) = make_float4(a, b, c, e);
      }
    }
  }
}

// out[r, :] = rms_norm(x[rows ? rows[r] : r, :]) * w, for r in [0, num_rows).
extern "C" int rl_rmsnorm(const float* x, const float* weight, void* out, int out_dtype,
                          const int* rows, int num_rows, int hidden, float eps, cudaStream_t stream) {
  RL_REQUIRE(num_rows >= 0 && hidden > 0, "rl_rmsnorm: bad sizes rows=%d d=%d", num_rows, hidden);
  RL_REQUIRE(eps > 0.f, "rl_rmsnorm: eps must be > 0, got %g", (double)eps);
  if (num_rows == 0) return RL_OK;
  const bool vec = hidden % 4 == 0 && hidden <= 256 * 4 * 8 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)weight & 15) == 0 &&
                   ((uintptr_t)out & 15) == 0;
  if (vec && out_dtype == RL_BF16 && hidden <= 256 * 4 * 4)
    rl_launch_pdl(rmsnorm_vec_kernel<__nv_bfloat16, 256, 4>, num_rows, 256, 0, stream, x, weight, (__nv_bfloat16*)out, rows, hidden, eps);
  else if (vec && out_dtype == RL_BF16)
    rl_launch_pdl(rmsnorm_vec_kernel<__nv_bfloat16, 256, 8>, num_rows, 256, 0, stream, x, weight, (__nv_bfloat16*)out, rows, hidden, eps);
  else if (vec && out_dtype == RL_F32)
    rl_launch_pdl(rmsnorm_vec_kernel<float, 256, 8>, num_rows, 256, 0, stream, x, weight, (float*)out, rows, hidden, eps);
  else if (out_dtype == RL_F32)
    rl_launch_pdl(rmsnorm_kernel<float, 256>, num_rows, 256, 0, stream, x, weight, (float*)out, rows, hidden, eps);
  else if (out_dtype == RL_BF16)
    rl_launch_pdl(rmsnorm_kernel<__nv_bfloat16, 256>, num_rows, 256, 0, stream, x, weight, (__nv_bfloat16*)out, rows, hidden, eps);
  else
    RL_REQUIRE(false, "rl_rmsnorm: unknown output dtype %d", out_dtype);
  RL_LAUNCH_CHECK("rl_rmsnorm");
  return RL_OK;
}

// ------------------------------------------------------------------ SwiGLU
// gate_up: [M, 2*I] with the gate in columns [0, I) and up in [I, 2I); or, interleaved,
// gate_i in column 2i and up_i in column 2i + 1.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int M, int I, int interleaved) {
  rl_pdl_trigger();
  rl_pdl_wait();
  const size_t total = (size_t)M * I;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t m = idx / I;
    const int i = (int)(idx - m * I);
    const float g = rl_ld(gu + m * 2 * I + (interleaved ? 2 * i : i));
    const float u = rl_ld(gu + m * 2 * I + (interleaved ? 2 * i + 1 : I + i));
    rl_st(out + idx, g / (1.0f + expf(-g)) * u);
  }
}

// bf16, I a multiple of 8, 16-byte aligned rows: eight elements a thread
__global__ void swiglu_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int M, int I) {
  rl_pdl_trigger();
  rl_pdl_wait();
  const int per_row = I / 8;
  const size_t total = (size_t)M * per_row;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t m = idx / per_row;
    const int c = (int)(idx - m * per_row) * 8;
    const uint4 g4 = *reinterpret_cast<const uint4*>(gu + m * 2 * I + c);
    const uint4 u4 = *reinterpret_cast<const uint4*>(gu + m * 2 * I + I + c);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
      o2[k] = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(out + m * I + c) = o4;
  }
}

// bf16, interleaved (gate_i, up_i) pairs: four pairs in, four results out a thread
__global__ void swiglu_bf16_interleaved_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, size_t quads) {
  rl_pdl_trigger();
  rl_pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < quads; idx += (size_t)gridDim.x * blockDim.x) {
    const uint4 v = *reinterpret_cast<const uint4*>(gu + idx * 8);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
    float r[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 gu2 = __bfloat1622float2(p[k]);
      r[k] = gu2.x / (1.0f + expf(-gu2.x)) * gu2.y;
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(r[0], r[1]), hi = __floats2bfloat162_rn(r[2], r[3]);
    *reinterpret_cast<uint2*>(out + idx * 4) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
  }
}

extern "C" int rl_swiglu(const void* gate_up, void* out, int dtype, int num_tokens,
                         int intermediate, int interleaved, cudaStream_t stream) {
  RL_REQUIRE(num_tokens >= 0 && intermediate > 0, "rl_swiglu: bad sizes M=%d I=%d", num_tokens, intermediate);
  if (num_tokens == 0) return RL_OK;
  const size_t total = (size_t)num_tokens * intermediate;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < rl_num_sms() * 16 ? (total + threads - 1) / threads : rl_num_sms() * 16);
  if (dtype == RL_BF16 && interleaved && intermediate % 4 == 0 && ((uintptr_t)gate_up & 15) == 0 && ((uintptr_t)out & 7) == 0) {
    const size_t quads = total / 4;      // rows are contiguous: [M, 2I] in, [M, I] out
    const int qblocks = (int)((quads + threads - 1) / threads < rl_num_sms() * 16 ? (quads + threads - 1) / threads : rl_num_sms() * 16);
    rl_launch_pdl(swiglu_bf16_interleaved_kernel, qblocks, threads, 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, quads);
  } else if (dtype == RL_BF16 && !interleaved && intermediate % 8 == 0 && ((uintptr_t)gate_up & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    const size_t vec = total / 8;
    const int vblocks = (int)((vec + threads - 1) / threads < rl_num_sms() * 16 ? (vec + threads - 1) / threads : rl_num_sms() * 16);
    rl_launch_pdl(swiglu_bf16x8_kernel, vblocks, threads, 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, num_tokens, intermediate);
  } else if (dtype == RL_F32)
    rl_launch_pdl(swiglu_kernel<float>, blocks, threads, 0, stream, (const float*)gate_up, (float*)out, num_tokens, intermediate, interleaved);
  else if (dtype == RL_BF16)
    rl_launch_pdl(swiglu_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, num_tokens, intermediate, interleaved);
  else
    RL_REQUIRE(false, "rl_swiglu: unknown dtype %d", dtype);
  RL_LAUNCH_CHECK("rl_swiglu");
  return RL_OK;
}

// ------------------------------------------------------------------ dtype conversion
template <typename TI, typename TO>
__global__ void convert_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    rl_st(out + i, rl_ld(in + i));
}

extern "C" int rl_convert(const void* in, int in_dtype, void* out, int out_dtype, long long n,
                          cudaStream_t stream) {
  RL_REQUIRE(n >= 0, "rl_convert: negative length");
  if (n == 0) return RL_OK;
  const int threads = 256;
  const long long want = (n + threads - 1) / threads;
  const int blocks = (int)(want < rl_num_sms() * 16 ? want : rl_num_sms() * 16);
  if (in_dtype == RL_F32 && out_dtype == RL_BF16)
    convert_kernel<<<blocks, threads, 0, stream>>>((const float*)in, (__nv_bfloat16*)out, (size_t)n);
  else if (in_dtype == RL_BF16 && out_dtype == RL_F32)
    convert_kernel<<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)in, (float*)out, (size_t)n);
  else
    RL_REQUIRE(false, "rl_convert: unsupported conversion %d -> %d", in_dtype, out_dtype);
  RL_LAUNCH_CHECK("rl_convert");
  return RL_OK;
}
