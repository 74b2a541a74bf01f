// out[M, N] = A[M, K] * W[N, K]^T (+ bias[N]) on the CUDA cores, for any M, N, K.
//
// This is the matrix product of the true 32-bit path (float inputs, FFMA, float
// accumulation, no tensor cores and no reduced-precision mode) and the fallback of
// the bf16 path for shapes the tensor-core kernel refuses (bf16 inputs widened to
// float, float accumulation).  Both operands are K-major, as every weight of the
// model is stored ([out x in], out = W x; SimonWaldherr/RustyLLM src/model.rs:185-186).
//
// Each output element is accumulated over k = 0..K-1 in order, whatever the tile
// it falls in: the result for one row does not depend on the other rows of the
// batch.
#include "common.cuh"

enum { RL_OUT_SAME = 0, RL_OUT_F32 = 1, RL_OUT_ADD_F32 = 2 };

template <typename T, int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_simt_kernel(const T* __restrict__ A, const T* __restrict__ W, const float* __restrict__ bias,
                 void* __restrict__ out, int out_mode, int M, int N, int K, int lda, int ldo) {
  constexpr int THREADS = (BM / TM) * (BN / TN);
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int idx = tid; idx < BM * BK; idx += THREADS) {
      const int r = idx / BK, k = idx % BK;
      const int gm = m0 + r, gk = k0 + k;
      As[k][r] = (gm < M && gk < K) ? rl_ld(A + (size_t)gm * lda + gk) : 0.f;
    }
    for (int idx = tid; idx < BN * BK; idx += THREADS) {
      const int r = idx / BK, k = idx % BK;
      const int gn = n0 + r, gk = k0 + k;
      Ws[k][r] = (gn < N && gk < K) ? rl_ld(W + (size_t)gn * K + gk) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Ws[k][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[gn];
      const size_t o = (size_t)gm * ldo + gn;
      if (out_mode == RL_OUT_SAME) rl_st((T*)out + o, v);
      else if (out_mode == RL_OUT_F32) ((float*)out)[o] = v;
      else ((float*)out)[o] += v;
    }
  }
}

// Few tokens (up to 64), float operands: the product is a single pass over W, so what counts is
// how many of its bytes are on their way at any time and how many warps an SM has to hide the
// latency of a chain of dependent FFMAs.  A CTA of four warps takes 32 weight rows; 16-byte
// asynchronous copies fill a ring of four stages of 64 k-values (8 KB of W a stage, the tokens'
// slice of A beside it; 39 to 100 KB a CTA, five to two CTAs an SM); thread (lane, warp) holds
// weight row `lane` and the tokens [warp * TM, (warp + 1) * TM) and reads its row four k-values
// a load (rows 68 floats apart: no bank conflicts), the tokens' values as broadcasts.  Each
// output element is still the chain fmaf(a[k], w[k], acc) over k = 0, 1, 2, ...: bit-equal to
// the tiled kernel below.
constexpr int STREAM_BN = 32, STREAM_BK = 64, STREAM_STAGES = 4, STREAM_WS = STREAM_BK + 4, STREAM_MAX_M = 64;
template <int TM> constexpr int stream_smem() { return STREAM_STAGES * (STREAM_BN * STREAM_WS + 4 * TM * STREAM_BK) * 4; }

__device__ __forceinline__ void stream_copy16(float* dst, const float* src, bool live) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int bytes = live ? 16 : 0;         // 0: the sixteen bytes are filled with zeros, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

template <int TM>
__global__ void __launch_bounds__(128)
gemm_simt_stream_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                        void* __restrict__ out, int out_mode, int M, int N, int K, int lda, int ldo) {
  extern __shared__ __align__(16) float stream_ring[];
  float* Wt = stream_ring;                                                 // [STAGES][BN][WS]
  float* At = stream_ring + STREAM_STAGES * STREAM_BN * STREAM_WS;          // [STAGES][4 TM][BK]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n0 = blockIdx.x * STREAM_BN;
  const int num_kb = (K + STREAM_BK - 1) / STREAM_BK;
  auto fill = [&](int kb) {
    const int s = kb % STREAM_STAGES, k0 = kb * STREAM_BK;
    float* wt = Wt + s * STREAM_BN * STREAM_WS;
    float* at = At + s * (4 * TM) * STREAM_BK;
#pragma unroll
    for (int i = 0; i < (STREAM_BN * STREAM_BK / 4) / 128; ++i) {
      const int idx = tid + i * 128, r = idx / (STREAM_BK / 4), c = idx % (STREAM_BK / 4);
      const bool live = n0 + r < N && k0 + 4 * c < K;
      stream_copy16(wt + r * STREAM_WS + 4 * c, live ? W + (size_t)(n0 + r) * K + k0 + 4 * c : W, live);
    }
    for (int idx = tid; idx < 4 * TM * (STREAM_BK / 4); idx += 128) {
      const int r = idx / (STREAM_BK / 4), c = idx % (STREAM_BK / 4);
      const bool live = r < M && k0 + 4 * c < K;
      stream_copy16(at + r * STREAM_BK + 4 * c, live ? A + (size_t)r * lda + k0 + 4 * c : A, live);
    }
  };
  for (int kb = 0; kb < STREAM_STAGES - 1; ++kb) {
    if (kb < num_kb) fill(kb);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  float acc[TM];
#pragma unroll
  for (int i = 0; i < TM; ++i) acc[i] = 0.f;
  for (int kb = 0; kb < num_kb; ++kb) {
    asm volatile("cp.async.wait_group %0;" ::"n"(STREAM_STAGES - 2) : "memory");
    __syncthreads();                       // stage kb has arrived for every thread; stage kb - 1 has been read by all
    if (kb + STREAM_STAGES - 1 < num_kb) fill(kb + STREAM_STAGES - 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const int s = kb % STREAM_STAGES;
    const float* wt = Wt + s * STREAM_BN * STREAM_WS + lane * STREAM_WS;
    const float* at = At + s * (4 * TM) * STREAM_BK + warp * TM * STREAM_BK;
#pragma unroll 4
    for (int k = 0; k < STREAM_BK; k += 4) {
      const float4 w = *reinterpret_cast<const float4*>(wt + k);
#pragma unroll
      for (int i = 0; i < TM; ++i) {
        const float4 a = *reinterpret_cast<const float4*>(at + i * STREAM_BK + k);
        acc[i] = fmaf(a.x, w.x, acc[i]);
        acc[i] = fmaf(a.y, w.y, acc[i]);
        acc[i] = fmaf(a.z, w.z, acc[i]);
        acc[i] = fmaf(a.w, w.w, acc[i]);
      }
    }
  }
  const int gn = n0 + lane;
  if (gn >= N) return;
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = warp * TM + i;
    if (gm >= M) continue;
    float v = acc[i];
    if (bias) v += bias[gn];
    const size_t o = (size_t)gm * ldo + gn;
    if (out_mode == RL_OUT_ADD_F32) ((float*)out)[o] += v;
    else ((float*)out)[o] = v;             // float operands: "same" and "float" are one
  }
}

template <int TM>
static int launch_gemm_simt_stream(const float* A, const float* W, const float* bias, void* out, int out_mode, int M, int N,
                                   int K, int lda, int ldo, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_simt_stream_kernel<TM>, cudaFuncAttributeMaxDynamicSharedMemorySize, stream_smem<TM>());
    RL_REQUIRE(e == cudaSuccess, "rl_gemm_simt: cannot reserve %d bytes of shared memory: %s", stream_smem<TM>(), cudaGetErrorString(e));
    configured = true;
  }
  gemm_simt_stream_kernel<TM><<<(N + STREAM_BN - 1) / STREAM_BN, 128, stream_smem<TM>(), stream>>>(A, W, bias, out, out_mode, M, N, K, lda, ldo);
  RL_LAUNCH_CHECK("rl_gemm_simt");
  return RL_OK;
}

// Many tokens, float operands with rows that 16-byte loads can fetch: the classic register tile.
// 256 threads own 8 x 8 outputs each of a 128 x 128 tile (two groups of four rows and of four
// columns, 64 apart, so that shared memory is read 16 bytes a time without conflicts); a
// thread fetches one 16-byte piece of A and one of W for the next 8 k-values into registers
// while the current ones are multiplied, and stores them transposed ([k][row]) into the other
// of two buffers.  Every output element is still the chain fmaf(a[k], w[k], acc), k = 0, 1, 2, ...
__global__ void __launch_bounds__(256)
gemm_simt_big_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                     void* __restrict__ out, int out_mode, int M, int N, int K, int lda, int ldo) {
  constexpr int BM = 128, BN = 128, BK = 8, LD = BM + 4;
  __shared__ __align__(16) float As[2][BK][LD];
  __shared__ __align__(16) float Ws[2][BK][LD];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int lr = tid >> 1, lk = (tid & 1) * 4;             // this thread's piece of a tile: row lr, k-values lk .. lk + 3
  const bool a_row = m0 + lr < M, w_row = n0 + lr < N;
  const float* ap = A + (size_t)(a_row ? m0 + lr : 0) * lda + lk;
  const float* wp = W + (size_t)(w_row ? n0 + lr : 0) * K + lk;
  auto fetch = [&](int k0, float4& a, float4& w) {
    const bool live = k0 + lk < K;                          // K is a multiple of 4: a piece is whole or beyond the end
    a = (a_row && live) ? *reinterpret_cast<const float4*>(ap + k0) : make_float4(0.f, 0.f, 0.f, 0.f);
    w = (w_row && live) ? *reinterpret_cast<const float4*>(wp + k0) : make_float4(0.f, 0.f, 0.f, 0.f);
  };
  auto stash = [&](int buf, const float4& a, const float4& w) {
    As[buf][lk + 0][lr] = a.x; As[buf][lk + 1][lr] = a.y; As[buf][lk + 2][lr] = a.z; As[buf][lk + 3][lr] = a.w;
    Ws[buf][lk + 0][lr] = w.x; Ws[buf][lk + 1][lr] = w.y; Ws[buf][lk + 2][lr] = w.z; Ws[buf][lk + 3][lr] = w.w;
  };
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  float4 na, nw;
  fetch(0, na, nw);
  stash(0, na, nw);
  __syncthreads();
  const int num_kb = (K + BK - 1) / BK;
  for (int kb = 0; kb < num_kb; ++kb) {
    const int buf = kb & 1;
    if (kb + 1 < num_kb) fetch((kb + 1) * BK, na, nw);
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][k][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Ws[buf][k][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Ws[buf][k][64 + tx * 4]);
      const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (kb + 1 < num_kb) stash(buf ^ 1, na, nw);            // the other buffer was last read an iteration ago
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + i - 4);
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int gn = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + j - 4);
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[gn];
      const size_t o = (size_t)gm * ldo + gn;
      if (out_mode == RL_OUT_ADD_F32) ((float*)out)[o] += v;
      else ((float*)out)[o] = v;
    }
  }
}

template <typename T>
static int launch_gemm_simt(const T* A, const T* W, const float* bias, void* out, int out_mode, int M,
                            int N, int K, int lda, int ldo, cudaStream_t stream) {
  if constexpr (sizeof(T) == 4) {
    // few tokens, rows that 16-byte copies can fetch: the streaming kernel
    if (M <= STREAM_MAX_M && K % 4 == 0 && lda % 4 == 0 && (((uintptr_t)A | (uintptr_t)W) & 15) == 0) {
      if (M <= 4) return launch_gemm_simt_stream<1>(A, W, bias, out, out_mode, M, N, K, lda, ldo, stream);
      if (M <= 8) return launch_gemm_simt_stream<2>(A, W, bias, out, out_mode, M, N, K, lda, ldo, stream);
      if (M <= 16) return launch_gemm_simt_stream<4>(A, W, bias, out, out_mode, M, N, K, lda, ldo, stream);
      if (M <= 32) return launch_gemm_simt_stream<8>(A, W, bias, out, out_mode, M, N, K, lda, ldo, stream);
      return launch_gemm_simt_stream<16>(A, W, bias, out, out_mode, M, N, K, lda, ldo, stream);
    }
    if (M > STREAM_MAX_M && K % 4 == 0 && lda % 4 == 0 && (((uintptr_t)A | (uintptr_t)W) & 15) == 0) {
      dim3 grid((N + 127) / 128, (M + 127) / 128);
      gemm_simt_big_kernel<<<grid, 256, 0, stream>>>(A, W, bias, out, out_mode, M, N, K, lda, ldo);
      RL_LAUNCH_CHECK("rl_gemm_simt");
      return RL_OK;
    }
  }
  if (M > 64) {
    dim3 grid((N + 127) / 128, (M + 127) / 128);
    gemm_simt_kernel<T, 128, 128, 8, 8, 8><<<grid, 256, 0, stream>>>(A, W, bias, out, out_mode, M, N, K, lda, ldo);
  } else if (M > 16) {
    dim3 grid((N + 63) / 64, (M + 63) / 64);
    gemm_simt_kernel<T, 64, 64, 16, 4, 4><<<grid, 256, 0, stream>>>(A, W, bias, out, out_mode, M, N, K, lda, ldo);
  } else {
    dim3 grid((N + 31) / 32, (M + 15) / 16);
    gemm_simt_kernel<T, 16, 32, 32, 2, 2><<<grid, 128, 0, stream>>>(A, W, bias, out, out_mode, M, N, K, lda, ldo);
  }
  RL_LAUNCH_CHECK("rl_gemm_simt");
  return RL_OK;
}

// dtype: storage of A and W (RL_F32 or RL_BF16).  out_mode: 0 store in that dtype,
// 1 store float, 2 add into a float buffer (the residual sum).  lda/ldo: row strides
// of A and out in elements.
extern "C" int rl_gemm_simt(const void* A, const void* W, const float* bias, void* out, int dtype,
                            int out_mode, int M, int N, int K, int lda, int ldo, cudaStream_t stream) {
  RL_REQUIRE(M >= 0 && N > 0 && K > 0, "rl_gemm_simt: bad sizes M=%d N=%d K=%d", M, N, K);
  RL_REQUIRE(lda >= K && ldo >= N, "rl_gemm_simt: row strides lda=%d (< K=%d?) ldo=%d (< N=%d?)", lda, K, ldo, N);
  RL_REQUIRE(out_mode >= 0 && out_mode <= 2, "rl_gemm_simt: unknown output mode %d", out_mode);
  if (M == 0) return RL_OK;
  if (dtype == RL_F32)
    return launch_gemm_simt<float>((const float*)A, (const float*)W, bias, out, out_mode, M, N, K, lda, ldo, stream);
  if (dtype == RL_BF16)
    return launch_gemm_simt<__nv_bfloat16>((const __nv_bfloat16*)A, (const __nv_bfloat16*)W, bias, out, out_mode, M, N, K, lda, ldo, stream);
  RL_REQUIRE(false, "rl_gemm_simt: unknown dtype %d", dtype);
}
