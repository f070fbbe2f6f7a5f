// C[M,N] = A[M,K] · W[N,K]^T (+ bias[N]) with an optional activation, or added
// into a 32-bit residual stream in place.  Plain FFMA on the CUDA cores: the
// 32-bit path of the model (no tensor-core mode, no reduced-precision products),
// and the fallback of the bfloat16 path for shapes the tensor-core kernel refuses.
// Every output element is one accumulator that takes k = 0..K-1 in ascending
// order, so a row's result does not depend on M or on its place in the batch.
// The reference's counterpart: sgl_matmul (src/ops.c:160-197) on the CPU and
// cublasSgemm / k_gemm_nt (src/cuda_backend.cu:2843-2867, 333-349) on the GPU.
// Weights are stored [N,K] (the reference transposes Conv1D weights the same
// way at upload, src/cuda_backend.cu:5232-5241).
#include "common.cuh"

SGLC_DEFINE_ERROR_STRING()

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W, const float* __restrict__ bias,
                 TO* __restrict__ out, float* __restrict__ residual, int M, int N, int K,
                 int lda, int ldo, int act) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; i++)
#pragma unroll
    for (int j = 0; j < TN; j++) acc[i][j] = 0.0f;

  // each thread stages 4 consecutive k of one row of A and of W
  int lrow = threadIdx.x / 4, lk = (threadIdx.x % 4) * 4;
  for (int k0 = 0; k0 < K; k0 += BK) {
    {
      int m = m0 + lrow;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        int k = k0 + lk + j;
        As[lk + j][lrow] = (m < M && k < K) ? to_f32(A[(size_t)m * lda + k]) : 0.0f;
      }
      int n = n0 + lrow;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        int k = k0 + lk + j;
        Ws[lk + j][lrow] = (n < N && k < K) ? to_f32(W[(size_t)n * K + k]) : 0.0f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; k++) {
      float a[TM], w[TN];
#pragma unroll
      for (int i = 0; i < TM; i++) a[i] = As[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; j++) w[j] = Ws[k][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; i++) {
    int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; j++) {
      int n = n0 + tx * TN + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      v = apply_act(v, act);
      if (residual) {
        size_t o = (size_t)m * ldo + n;
        residual[o] = residual[o] + v;
      } else {
        out[(size_t)m * ldo + n] = from_f32<TO>(v);
      }
    }
  }
}
}  // namespace

// A: [M,K] with row stride lda (elements); W: [N,K] contiguous; bias: float[N] or null.
// If `residual` is given (float [M,N], row stride ldo) the result is added into it and
// `out` is not written; else `out` ([M,N], row stride ldo, out_dtype) takes it.
SGLC_API int sglc_gemm_simt(const void* A, const void* W, const float* bias, void* out,
                            float* residual, int M, int N, int K, int lda, int ldo, int in_dtype,
                            int out_dtype, int act, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return SGLC_OK;
  if (K <= 0) return SGLC_ERR_ARGUMENT;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return SGLC_ERR_UNSUPPORTED;
  if (in_dtype == SGLC_F32 && (out_dtype == SGLC_F32 || residual)) {
    gemm_simt_kernel<float, float, float><<<grid, 256, 0, stream>>>(
        (const float*)A, (const float*)W, bias, (float*)out, residual, M, N, K, lda, ldo, act);
  } else if (in_dtype == SGLC_BF16 && (out_dtype == SGLC_F32 || residual)) {
    gemm_simt_kernel<__nv_bfloat16, __nv_bfloat16, float><<<grid, 256, 0, stream>>>(
        (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, bias, (float*)out, residual, M, N, K, lda,
        ldo, act);
  } else if (in_dtype == SGLC_BF16 && out_dtype == SGLC_BF16) {
    gemm_simt_kernel<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>(
        (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, bias, (__nv_bfloat16*)out, residual, M, N,
        K, lda, ldo, act);
  } else {
    return SGLC_ERR_ARGUMENT;
  }
  return sglc_launch_status();
}
