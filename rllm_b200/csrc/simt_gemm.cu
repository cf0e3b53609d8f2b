// Plain matrix product on the CUDA cores, float accumulate, both storage types:
//   C[T, N] = A[T, K] * W[N, K]^T      (weights row-major [out, in], as stored)
// It is the product of the true 32-bit path (float storage, FMA only, no
// reduced-precision matrix mode) and the fallback of the bfloat16 path for
// sizes the tensor-core kernel refuses. Every output element is summed over k
// in ascending order by one thread, so a row's result does not depend on which
// other rows share the batch.
//
// Epilogues: store (activation type), store float (logits), accumulate into the
// float residual stream, and SwiGLU over a gate/up pair of weight tiles
// (W holds [2N, K]: gate rows first, up rows after; out[t, n] = silu(g) * u).
// Reference counterparts: src/gpu/cuda/shaders/matmul.cu:49-77, 216-248 and
// moe.cu:86-147 (fused gate-up).
#include "common.cuh"
using namespace rllm;

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;   // 256 threads, 4x4 outputs each

enum : int { EPI_STORE = 0, EPI_STORE_F32 = 1, EPI_ACCUM_F32 = 2, EPI_SWIGLU = 3 };

template <typename TI, int EPI>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TI* __restrict__ A, const TI* __restrict__ W, void* __restrict__ Cv,
                 const TI* __restrict__ bias, int T, int N, int K, int lda, int ldc) {
  pdl_launch();
  pdl_wait();
  constexpr bool DUAL = (EPI == EPI_SWIGLU);
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  __shared__ float Us[DUAL ? BK : 1][BN + 4];

  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

  float acc[TM][TN] = {};
  float acu[DUAL ? TM : 1][TN] = {};

  const int lrow = tid / 4, lk = (tid % 4) * 4;   // each thread stages 4 consecutive k of one row

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lk + j;
      const int am = m0 + lrow, wn = n0 + lrow;
      As[lk + j][lrow] = (am < T && k < K) ? to_f32(A[(size_t)am * lda + k]) : 0.f;
      Ws[lk + j][lrow] = (wn < N && k < K) ? to_f32(W[(size_t)wn * K + k]) : 0.f;
      if (DUAL) Us[lk + j][lrow] = (wn < N && k < K) ? to_f32(W[((size_t)N + wn) * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], w[TN], u[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
      if (DUAL) {
#pragma unroll
        for (int j = 0; j < TN; ++j) u[j] = Us[kk][tx * TN + j];
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
          if (DUAL) acu[i][j] = fmaf(a[i], u[j], acu[i][j]);
        }
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= T) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += to_f32(bias[n]);
      const size_t o = (size_t)m * ldc + n;
      if (EPI == EPI_STORE) ((TI*)Cv)[o] = from_f32<TI>(v);
      else if (EPI == EPI_STORE_F32) ((float*)Cv)[o] = v;
      else if (EPI == EPI_ACCUM_F32) ((float*)Cv)[o] += v;
      else { float g = v, uu = acu[DUAL ? i : 0][j]; ((TI*)Cv)[o] = from_f32<TI>(g / (1.f + expf(-g)) * uu); }
    }
  }
}

template <typename TI>
int launch(int epi, const void* A, const void* W, void* C, const void* bias, int T, int N, int K,
           int lda, int ldc, cudaStream_t s) {
  dim3 grid((N + BN - 1) / BN, (T + BM - 1) / BM), block(256);
  int rc = 0;
#define GO(E) rc = launch_ex(gemm_simt_kernel<TI, E>, dim3(grid), dim3(block), 0, s, 1, (const TI*)A, (const TI*)W, C, (const TI*)bias, T, N, K, lda, ldc)
  switch (epi) {
    case EPI_STORE: GO(EPI_STORE); break;
    case EPI_STORE_F32: GO(EPI_STORE_F32); break;
    case EPI_ACCUM_F32: GO(EPI_ACCUM_F32); break;
    case EPI_SWIGLU: GO(EPI_SWIGLU); break;
    default: return ERR_BAD_SIZE;
  }
#undef GO
  return rc;
}

}  // namespace

// A: [T, K] with row stride lda; W: [N, K] ([2N, K] for the SwiGLU epilogue);
// C: [T, N] with row stride ldc, of the type the epilogue names; bias [N] or null.
RLLM_API int rllm_gemm_simt(int dt, int epi, const void* A, const void* W, void* C, const void* bias,
                            int T, int N, int K, int lda, int ldc, void* stream) {
  if (T <= 0 || N <= 0) return 0;
  if (K <= 0) return ERR_BAD_SIZE;
  if ((T + BM - 1) / BM > 65535) return ERR_TOO_LARGE;
  cudaStream_t s = (cudaStream_t)stream;
  if (dt == DT_F32) return launch<float>(epi, A, W, C, bias, T, N, K, lda, ldc, s);
  if (dt == DT_BF16) return launch<bf16>(epi, A, W, C, bias, T, N, K, lda, ldc, s);
  return ERR_BAD_DTYPE;
}
