// LayerNorm with gain and bias over rows of a 32-bit residual stream:
//   mean = sum(x)/E; var = sum((x-mean)^2)/E (biased); y = (x-mean)/sqrt(var+eps)*g + b
// (reference src/ops.c:199-218; GPU twin k_layernorm_b src/cuda_backend.cu:495-524).
// Statistics are two-pass in 32-bit; the output is float or bfloat16.  An
// optional row index gathers the rows to normalise (the wanted rows before the
// head), so nothing is computed for rows nobody reads.
#include "common.cuh"

SGLC_DEFINE_ERROR_STRING()

template <typename TO, int VEC>
__global__ void layernorm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                 const float* __restrict__ gamma, const float* __restrict__ beta,
                                 TO* __restrict__ out, int n_rows, int E, float eps) {
  extern __shared__ float srow[];   // E floats: the row, read from memory once
  __shared__ float red[33];
  int r = blockIdx.x;
  if (r >= n_rows) return;
  int src = rows ? rows[r] : r;
  const float* xr = x + (size_t)src * E;
  float s = 0.0f;
  if (VEC == 4) {
    const float4* x4 = reinterpret_cast<const float4*>(xr);
    for (int i = threadIdx.x; i < E / 4; i += blockDim.x) {
      float4 v = x4[i];
      reinterpret_cast<float4*>(srow)[i] = v;
      s += (v.x + v.y) + (v.z + v.w);
    }
  } else {
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
      float v = xr[i];
      srow[i] = v;
      s += v;
    }
  }
  float mean = block_sum(s, red) / (float)E;
  float q = 0.0f;
  for (int i = threadIdx.x; i < E; i += blockDim.x) {
    float d = srow[i] - mean;
    q += d * d;
  }
  float var = block_sum(q, red) / (float)E;
  float inv = 1.0f / sqrtf(var + eps);
  TO* o = out + (size_t)r * E;
  for (int i = threadIdx.x; i < E; i += blockDim.x) {
    float y = (srow[i] - mean) * inv * gamma[i] + beta[i];
    o[i] = from_f32<TO>(y);
  }
}

SGLC_API int sglc_layernorm(const float* x, const int* rows, const float* gamma, const float* beta,
                            void* out, int n_rows, int E, float eps, int out_dtype,
                            cudaStream_t stream) {
  if (n_rows <= 0) return SGLC_OK;
  size_t smem = (size_t)E * sizeof(float);
  if (smem > 200 * 1024) return SGLC_ERR_UNSUPPORTED;
  int threads = E >= 2048 ? 512 : (E >= 512 ? 256 : (E >= 128 ? 128 : 32));
  bool vec = (E % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
#define LAUNCH(TO, VEC)                                                                      \
  do {                                                                                       \
    if (smem > 48 * 1024)                                                                    \
      cudaFuncSetAttribute(layernorm_kernel<TO, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                           (int)smem);                                                       \
    layernorm_kernel<TO, VEC><<<n_rows, threads, smem, stream>>>(x, rows, gamma, beta, (TO*)out, \
                                                                 n_rows, E, eps);            \
  } while (0)
  if (out_dtype == SGLC_F32) {
    if (vec) LAUNCH(float, 4); else LAUNCH(float, 1);
  } else if (out_dtype == SGLC_BF16) {
    if (vec) LAUNCH(__nv_bfloat16, 4); else LAUNCH(__nv_bfloat16, 1);
  } else {
    return SGLC_ERR_ARGUMENT;
  }
#undef LAUNCH
  return sglc_launch_status();
}
