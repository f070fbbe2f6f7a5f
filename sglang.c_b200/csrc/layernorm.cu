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
  pdl_launch_dependents();
  pdl_wait();
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

// One float4 per thread: the row stays in registers, gain and bias are fetched while the
// row is in flight, and each reduction costs one barrier (every warp adds the per-warp
// partial sums itself, in the same order).
template <typename TO>
__global__ void layernorm_row4_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                      const float* __restrict__ gamma, const float* __restrict__ beta,
                                      TO* __restrict__ out, int n_rows, int E, float eps) {
  __shared__ float red1[32], red2[32];
  int r = blockIdx.x;
  if (r >= n_rows) return;
  pdl_launch_dependents();
  const int i = threadIdx.x, n4 = E / 4;
  const int lane = i & 31, w = i >> 5, nw = (blockDim.x + 31) >> 5;
  const bool has = i < n4;
  float4 g = make_float4(0, 0, 0, 0), b = g, v = g;
  if (has) {
    g = reinterpret_cast<const float4*>(gamma)[i];     // weights: not produced by an earlier kernel
    b = reinterpret_cast<const float4*>(beta)[i];
  }
  pdl_wait();
  int src = rows ? rows[r] : r;
  if (has) v = reinterpret_cast<const float4*>(x + (size_t)src * E)[i];
  float s = warp_sum((v.x + v.y) + (v.z + v.w));
  if (lane == 0) red1[w] = s;
  __syncthreads();
  float tot = 0.0f;
  for (int k = 0; k < nw; k++) tot += red1[k];
  const float mean = tot / (float)E;
  float dx = v.x - mean, dy = v.y - mean, dz = v.z - mean, dw = v.w - mean;
  float q = has ? (dx * dx + dy * dy) + (dz * dz + dw * dw) : 0.0f;
  q = warp_sum(q);
  if (lane == 0) red2[w] = q;
  __syncthreads();
  float qt = 0.0f;
  for (int k = 0; k < nw; k++) qt += red2[k];
  const float inv = 1.0f / sqrtf(qt / (float)E + eps);
  if (has) {
    float y0 = dx * inv * g.x + b.x, y1 = dy * inv * g.y + b.y, y2 = dz * inv * g.z + b.z,
          y3 = dw * inv * g.w + b.w;
    TO* o = out + (size_t)r * E + 4 * i;
    if constexpr (sizeof(TO) == 4) {
      *reinterpret_cast<float4*>(o) = make_float4(y0, y1, y2, y3);
    } else {
      __nv_bfloat162 h0 = __floats2bfloat162_rn(y0, y1), h1 = __floats2bfloat162_rn(y2, y3);
      uint2 pk = make_uint2(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1));
      *reinterpret_cast<uint2*>(o) = pk;
    }
  }
}

// Many rows (prompt portions of a thousand tokens and more), bfloat16 output: a warp per row, the row in registers (lane l
// holds the 16-byte pieces l, l+32, ...), no block-wide barrier.  Used for the bfloat16 path
// only: its order of additions differs from the kernels above, and in the 32-bit path a row's
// bits must not depend on how many rows share its step.
template <int NV>
__global__ void __launch_bounds__(256)
layernorm_warp_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                      const float* __restrict__ gamma, const float* __restrict__ beta,
                      __nv_bfloat16* __restrict__ out, int n_rows, int E, float eps) {
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int n4 = E / 4;
  // gain and bias are weights, not produced by the kernel ahead: up to 1,024 columns they are
  // fetched into registers before the dependency wait
  constexpr bool PRE = NV <= 8;
  float4 gp[PRE ? NV : 1], bp[PRE ? NV : 1];
  if (PRE) {
#pragma unroll
    for (int j = 0; j < (PRE ? NV : 1); j++) {
      const int i = lane + 32 * j;
      gp[j] = i < n4 ? reinterpret_cast<const float4*>(gamma)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      bp[j] = i < n4 ? reinterpret_cast<const float4*>(beta)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  pdl_wait();
  if (r >= n_rows) return;
  const int src = rows ? rows[r] : r;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)src * E);
  float4 v[NV];
  float s = 0.0f;
#pragma unroll
  for (int j = 0; j < NV; j++) {
    const int i = lane + 32 * j;
    v[j] = i < n4 ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
  }
  const float mean = warp_sum(s) / (float)E;
  float q = 0.0f;
#pragma unroll
  for (int j = 0; j < NV; j++) {
    if (lane + 32 * j < n4) {
      float dx = v[j].x - mean, dy = v[j].y - mean, dz = v[j].z - mean, dw = v[j].w - mean;
      q += (dx * dx + dy * dy) + (dz * dz + dw * dw);
    }
  }
  const float inv = 1.0f / sqrtf(warp_sum(q) / (float)E + eps);
  __nv_bfloat16* o = out + (size_t)r * E;
#pragma unroll
  for (int j = 0; j < NV; j++) {
    const int i = lane + 32 * j;
    if (i < n4) {
      const float4 g = PRE ? gp[PRE ? j : 0] : reinterpret_cast<const float4*>(gamma)[i];
      const float4 b = PRE ? bp[PRE ? j : 0] : reinterpret_cast<const float4*>(beta)[i];
      __nv_bfloat162 h0 = __floats2bfloat162_rn((v[j].x - mean) * inv * g.x + b.x, (v[j].y - mean) * inv * g.y + b.y);
      __nv_bfloat162 h1 = __floats2bfloat162_rn((v[j].z - mean) * inv * g.z + b.z, (v[j].w - mean) * inv * g.w + b.w);
      *reinterpret_cast<uint2*>(o + 4 * i) = make_uint2(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1));
    }
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
  int rc = SGLC_OK;
  bool al = vec && ((reinterpret_cast<uintptr_t>(gamma) & 15) == 0) &&
            ((reinterpret_cast<uintptr_t>(beta) & 15) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
  if (al && out_dtype == SGLC_BF16 && n_rows >= 1024 && E / 4 <= 32 * 16) {   // (8 rows a block: enough blocks for every SM)
    const int nv = (E / 4 + 31) / 32;
    const dim3 grid((n_rows + 7) / 8), block(256);
#define WARP_LAUNCH(NV)                                                                               \
  return sglc_launch(layernorm_warp_kernel<NV>, grid, block, 0, stream, 1, true, x, rows, gamma, beta, \
                     (__nv_bfloat16*)out, n_rows, E, eps)
    if (nv <= 2) WARP_LAUNCH(2);
    if (nv <= 4) WARP_LAUNCH(4);
    if (nv <= 6) WARP_LAUNCH(6);
    if (nv <= 8) WARP_LAUNCH(8);
    if (nv <= 13) WARP_LAUNCH(13);
    WARP_LAUNCH(16);
#undef WARP_LAUNCH
  }
  if (al && E / 4 <= 1024) {
    int th = ((E / 4 + 31) / 32) * 32;
    if (out_dtype == SGLC_F32)
      return sglc_launch(layernorm_row4_kernel<float>, dim3(n_rows), dim3(th), 0, stream, 1, true, x,
                         rows, gamma, beta, (float*)out, n_rows, E, eps);
    if (out_dtype == SGLC_BF16)
      return sglc_launch(layernorm_row4_kernel<__nv_bfloat16>, dim3(n_rows), dim3(th), 0, stream, 1,
                         true, x, rows, gamma, beta, (__nv_bfloat16*)out, n_rows, E, eps);
    return SGLC_ERR_ARGUMENT;
  }
#define LAUNCH(TO, VEC)                                                                      \
  do {                                                                                       \
    if (smem > 48 * 1024)                                                                    \
      cudaFuncSetAttribute(layernorm_kernel<TO, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                           (int)smem);                                                       \
    rc = sglc_launch(layernorm_kernel<TO, VEC>, dim3(n_rows), dim3(threads), smem, stream, 1,  \
                     true, x, rows, gamma, beta, (TO*)out, n_rows, E, eps);                  \
  } while (0)
  if (out_dtype == SGLC_F32) {
    if (vec) LAUNCH(float, 4); else LAUNCH(float, 1);
  } else if (out_dtype == SGLC_BF16) {
    if (vec) LAUNCH(__nv_bfloat16, 4); else LAUNCH(__nv_bfloat16, 1);
  } else {
    return SGLC_ERR_ARGUMENT;
  }
#undef LAUNCH
  return rc;
}
