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

template <typename T>
static int launch_gemm_simt(const T* A, const T* W, const float* bias, void* out, int out_mode, int M,
                            int N, int K, int lda, int ldo, cudaStream_t stream) {
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
