// Shared helpers of the kernels in this folder.  Every .cu file here builds to
// one shared library with a C interface; the bindings in ops.py load them.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#define SGLC_API extern "C" __attribute__((visibility("default")))

// element types a launcher takes, as small integers across the C interface
enum { SGLC_F32 = 0, SGLC_BF16 = 1 };
// epilogue activations
enum { SGLC_ACT_NONE = 0, SGLC_ACT_GELU_TANH = 1, SGLC_ACT_GELU_ERF = 2 };

// codes a launcher returns besides cudaError_t values (those are > 0)
enum { SGLC_OK = 0, SGLC_ERR_UNSUPPORTED = -2, SGLC_ERR_ARGUMENT = -3 };

SGLC_API const char* sglc_error_string(int code);

// Programmatic dependent launch: a kernel launched with it may start while the kernel before
// it in the stream still runs.  It calls pdl_launch_dependents() early (its successor may be
// scheduled) and pdl_wait() before it reads or overwrites anything an earlier kernel touches
// (returns at once when the launch had no programmatic dependency).  sglc_set_pdl(0) turns
// the launch attribute off for this library.
static int g_sglc_pdl = 1;
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Launch with optional cluster depth (blocks of one grid.z column form a cluster) and the
// programmatic-dependency attribute.
template <typename... KArgs, typename... Args>
static inline int sglc_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, int cluster_z, bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (cluster_z > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = 1;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = cluster_z;
    n++;
  }
  if (pdl && g_sglc_pdl) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    n++;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}

// The bounds-check build (-DSGLC_BOUNDS_CHECK, see build.set_bounds_check): every index that a
// kernel takes from device memory (a page id out of a block table, a cache slot, a row number) is
// compared with its range before it is used; an index outside is not dereferenced: the access is
// skipped and the error word gets SGLC_FLAG_INDEX.  (The stand-in for a memory checker where none
// can be run; the ordinary build trusts what the host validated when it built the step.)
enum { SGLC_FLAG_WAIT = 1, SGLC_FLAG_INDEX = 4 };
#ifdef SGLC_BOUNDS_CHECK
__device__ __forceinline__ bool sglc_index_ok(long long i, long long n, int* err) {
  if (i >= 0 && i < n) return true;
  if (err) atomicOr(err, SGLC_FLAG_INDEX);
  return false;
}
#else
__device__ __forceinline__ bool sglc_index_ok(long long, long long, int*) { return true; }
#endif

#define SGLC_DEFINE_ERROR_STRING()                                            \
  SGLC_API void sglc_set_pdl(int on) { g_sglc_pdl = on; }                     \
  SGLC_API const char* sglc_error_string(int code) {                          \
    if (code == SGLC_ERR_UNSUPPORTED) return "size not supported by this kernel"; \
    if (code == SGLC_ERR_ARGUMENT) return "bad argument";                     \
    return cudaGetErrorString((cudaError_t)code);                             \
  }

static inline int sglc_launch_status() { return (int)cudaGetLastError(); }

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// tanh form: 0.5*u*(1+tanh(sqrt(2/pi)*(u+0.044715*u^3)))  (reference src/ops.c:233-241)
__device__ __forceinline__ float gelu_tanh_f32(float u) {
  const float k = 0.7978845608028654f;
  float inner = k * (u + 0.044715f * u * u * u);
  return 0.5f * u * (1.0f + tanhf(inner));
}
// exact form: 0.5*u*(1+erf(u/sqrt(2)))
__device__ __forceinline__ float gelu_erf_f32(float u) {
  return 0.5f * u * (1.0f + erff(u * 0.70710678118654752440f));
}
__device__ __forceinline__ float apply_act(float u, int act) {
  if (act == SGLC_ACT_GELU_TANH) return gelu_tanh_f32(u);
  if (act == SGLC_ACT_GELU_ERF) return gelu_erf_f32(u);
  return u;
}

// The tanh form of GELU as u * sigmoid(2k(u + 0.044715 u^3)), which is the same function
// (0.5 (1 + tanh x) = sigmoid 2x) without the cancellation of 1 + tanh for negative inputs, by
// one exponential and one division of the fast kind (2 ulp each): a few instructions where
// tanhf takes twenty, and the tensor-core products' epilogues are made of them.
__device__ __forceinline__ float gelu_tanh_sigmoid(float u) {
  const float z = 1.5957691216057308f * (u + 0.044715f * u * u * u);
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-z * 1.4426950408889634f));
  return __fdividef(u, 1.0f + e);
}
__device__ __forceinline__ float act_tc(float u, int act) {
  if (act == SGLC_ACT_GELU_TANH) return gelu_tanh_sigmoid(u);
  if (act == SGLC_ACT_GELU_ERF) return gelu_erf_f32(u);
  return u;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; every thread gets the result.  `red` holds at least 33 floats.
// The order of additions depends only on blockDim, so a row's result does not
// depend on what else is in the batch.
__device__ __forceinline__ float block_sum(float v, float* red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = lane < nw ? red[lane] : 0.0f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = lane < nw ? red[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
