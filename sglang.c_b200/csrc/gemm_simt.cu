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
// Many rows and many features (a prompt portion of the 32-bit path): a block of 128 x 128 outputs,
// a thread 8 x 8 of them (two 4 x 4 corners 64 apart each way, so that a warp's shared-memory reads
// are two broadcasts and one contiguous run), which is four times the arithmetic per shared-memory
// read of the 64 x 64 kernel (NW = 1: 128 x 64 outputs, 8 x 4 a thread, for products whose 128 x 128
// blocks would leave most of the GPU idle).  The next k-tile is on its way from global memory into registers
// while this one is multiplied.  One accumulator per output, k ascending: the same bits again.
constexpr int LM = 128, LK = 16, LP = LM + 4;

template <int NW>
__global__ void __launch_bounds__(256, 2)          // two blocks an SM: at most 128 registers a thread
gemm_simt_large_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                       float* __restrict__ out, float* __restrict__ residual, int M, int N, int K, int lda,
                       int ldo, int act) {
  __shared__ __align__(16) float As[2][LK][LP];
  constexpr int LN = 64 * NW;
  __shared__ __align__(16) float Ws[2][LK][LN + 4];
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const int m0 = blockIdx.y * LM, n0 = blockIdx.x * LN;
  const int lrow = tid / 4, lk = (tid % 4) * 4;      // rows lrow and lrow + 64, four k from lk
  float4 ra[2], rw[NW];
  auto gload = [&](int k0) {
    const int k = k0 + lk;
#pragma unroll
    for (int r = 0; r < 2; r++) {
      const int m = m0 + lrow + 64 * r;
      ra[r] = (m < M && k < K) ? *reinterpret_cast<const float4*>(A + (size_t)m * lda + k)
                               : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
#pragma unroll
    for (int r = 0; r < NW; r++) {
      const int n = n0 + lrow + 64 * r;
      rw[r] = (n < N && k < K) ? *reinterpret_cast<const float4*>(W + (size_t)n * K + k)
                               : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
  };
  auto sstore = [&](int buf) {
#pragma unroll
    for (int r = 0; r < 2; r++) {
      const int c = lrow + 64 * r;
      As[buf][lk + 0][c] = ra[r].x; As[buf][lk + 1][c] = ra[r].y;
      As[buf][lk + 2][c] = ra[r].z; As[buf][lk + 3][c] = ra[r].w;
    }
#pragma unroll
    for (int r = 0; r < NW; r++) {
      const int c = lrow + 64 * r;
      Ws[buf][lk + 0][c] = rw[r].x; Ws[buf][lk + 1][c] = rw[r].y;
      Ws[buf][lk + 2][c] = rw[r].z; Ws[buf][lk + 3][c] = rw[r].w;
    }
  };
  float acc[8][4 * NW];
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int j = 0; j < 4 * NW; j++) acc[i][j] = 0.0f;
  gload(0);
  sstore(0);
  __syncthreads();
  for (int k0 = 0, buf = 0; k0 < K; k0 += LK, buf ^= 1) {
    const bool more = k0 + LK < K;
    if (more) gload(k0 + LK);
#pragma unroll
    for (int k = 0; k < LK; k++) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][k][64 + ty * 4]);
      const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      float w[4 * NW];
#pragma unroll
      for (int r = 0; r < NW; r++) {
        const float4 w4 = *reinterpret_cast<const float4*>(&Ws[buf][k][64 * r + tx * 4]);
        w[4 * r] = w4.x; w[4 * r + 1] = w4.y; w[4 * r + 2] = w4.z; w[4 * r + 3] = w4.w;
      }
#pragma unroll
      for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 4 * NW; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    if (more) sstore(buf ^ 1);                       // (its readers passed the barrier of the tile before)
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + i - 4);
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4 * NW; j++) {
      const int n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + j - 4);
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      v = apply_act(v, act);
      const size_t o = (size_t)m * ldo + n;
      if (residual) residual[o] = residual[o] + v;
      else out[o] = v;
    }
  }
}

// Up to 16 rows (a decode step of the 32-bit path): the product is a read of the weights once, so
// what counts is bytes in flight.  A block takes 16 output features; the tiles of A (16 x 32 k)
// and W (16 x 32 k) come through a ring of eight shared-memory stages by asynchronous 16-byte
// copies, seven k-tiles ahead of the arithmetic.  A thread owns 2 rows of 1 feature and adds
// k = 0..K-1 in ascending order with the same fused multiply-add as the kernel above, so an
// output element has the same bits whichever of the two kernels computed it.
constexpr int SM_ = 16, SN = 16, SK = 32, ST = 8, PITCH = SK + 4;

__device__ __forceinline__ void cp_async16_zfill(void* dst, const void* src, bool on) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int n = on ? 16 : 0;                         // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}

__global__ void __launch_bounds__(128)
gemm_simt_small_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                       float* __restrict__ out, float* __restrict__ residual, int M, int N, int K, int lda,
                       int ldo, int act) {
  __shared__ __align__(16) float As[ST][SM_][PITCH];
  __shared__ __align__(16) float Ws[ST][SN][PITCH];
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const int m0 = blockIdx.y * SM_, n0 = blockIdx.x * SN;
  const int lrow = tid / 8, lk = (tid % 8) * 4;      // this thread's 16-byte piece of a tile row
  const int n_tiles = (K + SK - 1) / SK;
  auto issue = [&](int tile) {
    if (tile < n_tiles) {
      const int st = tile % ST, k = tile * SK + lk;
      const bool kin = k < K;                        // (K is a multiple of 4: a piece lies inside or outside)
      const int m = m0 + lrow;
      cp_async16_zfill(&As[st][lrow][lk], A + (size_t)(m < M ? m : 0) * lda + (kin ? k : 0), kin && m < M);
      const int n = n0 + lrow;
      cp_async16_zfill(&Ws[st][lrow][lk], W + (size_t)(n < N ? n : 0) * K + (kin ? k : 0), kin && n < N);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  for (int t = 0; t < ST - 1; t++) issue(t);
  float acc[2] = {0.0f, 0.0f};
  for (int tile = 0; tile < n_tiles; tile++) {
    asm volatile("cp.async.wait_group %0;" ::"n"(ST - 2) : "memory");
    __syncthreads();                                 // tile `tile` has landed; the stage of tile-1 is free
    issue(tile + ST - 1);
    const int st = tile % ST;
#pragma unroll
    for (int k = 0; k < SK; k += 4) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[st][2 * ty][k]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[st][2 * ty + 1][k]);
      const float4 w0 = *reinterpret_cast<const float4*>(&Ws[st][tx][k]);
      acc[0] = fmaf(a0.x, w0.x, acc[0]); acc[1] = fmaf(a1.x, w0.x, acc[1]);
      acc[0] = fmaf(a0.y, w0.y, acc[0]); acc[1] = fmaf(a1.y, w0.y, acc[1]);
      acc[0] = fmaf(a0.z, w0.z, acc[0]); acc[1] = fmaf(a1.z, w0.z, acc[1]);
      acc[0] = fmaf(a0.w, w0.w, acc[0]); acc[1] = fmaf(a1.w, w0.w, acc[1]);
    }
  }
#pragma unroll
  for (int i = 0; i < 2; i++) {
    const int m = m0 + 2 * ty + i;
    const int n = n0 + tx;
    if (m >= M || n >= N) continue;
    float v = acc[i];
    if (bias) v += bias[n];
    v = apply_act(v, act);
    const size_t o = (size_t)m * ldo + n;
    if (residual) residual[o] = residual[o] + v;
    else out[o] = v;
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
  const bool f32 = in_dtype == SGLC_F32 && (out_dtype == SGLC_F32 || residual);
  const bool wide_loads = K % 4 == 0 && lda % 4 == 0 && (((uintptr_t)A | (uintptr_t)W) & 15) == 0;
  const int m_blocks = (M + LM - 1) / LM;
  if (f32 && wide_loads && M > BM && m_blocks <= 65535 && (long long)m_blocks * ((N + 127) / 128) >= 240) {
    gemm_simt_large_kernel<2><<<dim3((N + 127) / 128, m_blocks), 256, 0, stream>>>(
        (const float*)A, (const float*)W, bias, (float*)out, residual, M, N, K, lda, ldo, act);
  } else if (f32 && wide_loads && M > BM && m_blocks <= 65535 && (long long)m_blocks * ((N + 63) / 64) >= 120) {
    gemm_simt_large_kernel<1><<<dim3((N + 63) / 64, m_blocks), 256, 0, stream>>>(
        (const float*)A, (const float*)W, bias, (float*)out, residual, M, N, K, lda, ldo, act);
  } else if (f32 && wide_loads && M <= SM_) {
    gemm_simt_small_kernel<<<dim3((N + SN - 1) / SN, (M + SM_ - 1) / SM_), 128, 0, stream>>>(
        (const float*)A, (const float*)W, bias, (float*)out, residual, M, N, K, lda, ldo, act);
  } else if (in_dtype == SGLC_F32 && (out_dtype == SGLC_F32 || residual)) {
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
