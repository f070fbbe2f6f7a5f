// Token embedding gather with an optional additive position table:
//   x[t,:] = wte[tok[t],:] (+ wpe[pos[t],:])      (reference src/gpt2.c:211-216,
//   GPU twin k_embed_pos src/cuda_backend.cu:477-483).
// Tables are float or bfloat16; the sum is formed and stored in 32-bit.
#include "common.cuh"

SGLC_DEFINE_ERROR_STRING()

template <typename TW>
__global__ void embed_kernel(const int* __restrict__ tokens, const int* __restrict__ positions,
                             const TW* __restrict__ wte, const TW* __restrict__ wpe,
                             float* __restrict__ out, int T, int E, int V, int P,
                             int* __restrict__ err) {
  int t = blockIdx.x;
  if (t >= T) return;
  pdl_launch_dependents();
  pdl_wait();
  int tok = tokens[t];
  bool bad = tok < 0 || tok >= V;
  int pos = 0;
  if (wpe) {
    pos = positions[t];
    bad = bad || pos < 0 || pos >= P;
  }
  if (bad) {
    // the host checks ids before a step; a bad id here means corrupted step data
    if (threadIdx.x == 0 && err) atomicExch(err, 1);
    for (int e = threadIdx.x; e < E; e += blockDim.x) out[(size_t)t * E + e] = 0.0f;
    return;
  }
  const TW* a = wte + (size_t)tok * E;
  const TW* b = wpe ? wpe + (size_t)pos * E : nullptr;
  float* o = out + (size_t)t * E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    float v = to_f32(a[e]);
    if (b) v += to_f32(b[e]);
    o[e] = v;
  }
}

// err: one int on the device, set to 1 if a token or position is out of range (may be null).
SGLC_API int sglc_embed(const int* tokens, const int* positions, const void* wte, const void* wpe,
                        float* out, int T, int E, int V, int P, int table_dtype, int* err,
                        cudaStream_t stream) {
  if (T <= 0) return SGLC_OK;
  int threads = E >= 1024 ? 256 : (E >= 256 ? 128 : 64);
  if (table_dtype == SGLC_F32)
    return sglc_launch(embed_kernel<float>, dim3(T), dim3(threads), 0, stream, 1, true, tokens,
                       positions, (const float*)wte, (const float*)wpe, out, T, E, V, P, err);
  else if (table_dtype == SGLC_BF16)
    return sglc_launch(embed_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, 1, true,
                       tokens, positions, (const __nv_bfloat16*)wte, (const __nv_bfloat16*)wpe, out, T,
                       E, V, P, err);
  else
    return SGLC_ERR_ARGUMENT;
  return sglc_launch_status();
}

// x[t,:] += table[pos[t],:]  — a position table added after the gather, for
// models whose embedding and position parts are not fused.
template <typename TW>
__global__ void add_rows_kernel(float* __restrict__ x, const int* __restrict__ idx,
                                const TW* __restrict__ table, int T, int E, int P) {
  int t = blockIdx.x;
  int r = idx[t];
  if (r < 0 || r >= P) return;
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    x[(size_t)t * E + e] += to_f32(table[(size_t)r * E + e]);
}

SGLC_API int sglc_add_rows(float* x, const int* idx, const void* table, int T, int E, int P,
                           int table_dtype, cudaStream_t stream) {
  if (T <= 0) return SGLC_OK;
  if (table_dtype == SGLC_F32)
    add_rows_kernel<float><<<T, 128, 0, stream>>>(x, idx, (const float*)table, T, E, P);
  else if (table_dtype == SGLC_BF16)
    add_rows_kernel<__nv_bfloat16><<<T, 128, 0, stream>>>(x, idx, (const __nv_bfloat16*)table, T, E, P);
  else
    return SGLC_ERR_ARGUMENT;
  return sglc_launch_status();
}
