// Causal attention over the paged cache, one block per (token, head), for any
// mix of prompt portions and single decoded tokens.  All arithmetic is 32-bit:
//   s[p] = (q·K_p)*scale for the keys p the query may see (p <= its position,
//   and p > position - window if a window is set); m = max s; e = exp(s-m);
//   o = sum_p e[p]*V_p / sum_p e[p]
// (reference src/gpt2.c:238-270; GPU twin k_attn, src/cuda_backend.cu:1600-1651).
// The work of one (token, head) depends only on that token's position and its
// request's pages, never on the rest of the batch, so the result is the same
// however the tokens were cut into steps.  This is the kernel of the 32-bit
// path and the general fallback of the bfloat16 path.
#include "common.cuh"

SGLC_DEFINE_ERROR_STRING()

template <typename TQ, typename TC, typename TO>
__global__ void attention_simt_kernel(const TQ* __restrict__ q, int q_stride,
                                      const TC* __restrict__ cache,
                                      const int* __restrict__ block_table, int bt_stride,
                                      const int* __restrict__ token_req,
                                      const int* __restrict__ positions, TO* __restrict__ out,
                                      int o_stride, int T, int H, int Hkv, int D, int page_size,
                                      float scale, int window, int max_keys, int n_pages, int* err) {
  extern __shared__ float smem[];
  __shared__ float red[33];
  int t = blockIdx.x, h = blockIdx.y;
  if (t >= T) return;
  int G = blockDim.x / D;          // groups of D threads that split the keys in the value pass
  if (G < 1) G = 1;
  float* sq = smem;                // D
  float* part = sq + D;            // G*D partial outputs
  float* sc = part + G * D;        // scores, up to max_keys
  int r = token_req[t];
  int pos = positions[t];
  int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  int n = pos - lo + 1;
  if (n > max_keys) n = max_keys;  // cannot happen when the host sized max_keys right
  int hk = h / (H / Hkv);
  const int* bt = block_table + (size_t)r * bt_stride;
  size_t page_elems = (size_t)2 * Hkv * page_size * D;
  size_t head_off = (size_t)hk * page_size * D;
  size_t v_off = (size_t)Hkv * page_size * D;

  const TQ* qp = q + (size_t)t * q_stride + (size_t)h * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) sq[d] = to_f32(qp[d]);
  __syncthreads();

  float lmax = -INFINITY;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    int p = lo + i;
    int page = bt[p / page_size];
    float s = 0.0f;
    if (sglc_index_ok(page, n_pages, err)) {
      const TC* kp = cache + (size_t)page * page_elems + head_off + (size_t)(p % page_size) * D;
      for (int d = 0; d < D; d++) s = fmaf(sq[d], to_f32(kp[d]), s);
    }
    s *= scale;
    sc[i] = s;
    lmax = fmaxf(lmax, s);
  }
  float m = block_max(lmax, red);
  float lsum = 0.0f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float e = expf(sc[i] - m);
    sc[i] = e;
    lsum += e;
  }
  float total = block_sum(lsum, red);   // also orders the writes of sc before the reads below

  int g = threadIdx.x / D, d0 = threadIdx.x % D;
  if (blockDim.x < D) { g = 0; d0 = threadIdx.x; }
  if (g < G) {
    int dstep = blockDim.x < D ? blockDim.x : D;
    for (int d = d0; d < D; d += dstep) {
      float acc = 0.0f;
      for (int i = g; i < n; i += G) {
        int p = lo + i;
        int page = bt[p / page_size];
        if (!sglc_index_ok(page, n_pages, nullptr)) continue;      // (flagged in the score pass)
        const TC* vp = cache + (size_t)page * page_elems + v_off + head_off +
                       (size_t)(p % page_size) * D;
        acc = fmaf(sc[i], to_f32(vp[d]), acc);
      }
      part[g * D + d] = acc;
    }
  }
  __syncthreads();
  TO* op = out + (size_t)t * o_stride + (size_t)h * D;
  float inv = 1.0f / total;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.0f;
    for (int gg = 0; gg < G; gg++) acc += part[gg * D + d];
    op[d] = from_f32<TO>(acc * inv);
  }
}

// q: first query element of token 0 (rows q_stride apart, heads side by side); cache: one
// layer's pages; block_table: [n_requests][bt_stride] page ids; token_req[t]: row of the
// block table for token t; positions[t]: absolute position of token t (its own key is the
// last one it sees); out: [T][o_stride].  max_keys: the most keys any token of this launch
// sees (sizes shared memory).  q/out dtype = act_dtype, cache dtype = cache_dtype.  n_pages and
// err serve the bounds-check build (page ids are compared with n_pages; err gets the flag).
SGLC_API int sglc_attention_simt(const void* q, int q_stride, const void* cache,
                                 const int* block_table, int bt_stride, const int* token_req,
                                 const int* positions, void* out, int o_stride, int T, int H,
                                 int Hkv, int D, int page_size, float scale, int window,
                                 int max_keys, int act_dtype, int cache_dtype, int n_pages, int* err,
                                 cudaStream_t stream) {
  if (T <= 0) return SGLC_OK;
  if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || D <= 0 || page_size <= 0 || max_keys <= 0)
    return SGLC_ERR_ARGUMENT;
  if (H > 65535) return SGLC_ERR_UNSUPPORTED;
  int threads = 128;
  if (D > 128) threads = 256;
  if (D > 256) return SGLC_ERR_UNSUPPORTED;
  int G = threads / D < 1 ? 1 : threads / D;
  size_t smem = ((size_t)D + (size_t)G * D + (size_t)max_keys) * sizeof(float);
  if (smem > 220 * 1024) return SGLC_ERR_UNSUPPORTED;
  dim3 grid(T, H);
#define LAUNCH(TQ, TC, TO)                                                                   \
  do {                                                                                       \
    if (smem > 48 * 1024)                                                                    \
      cudaFuncSetAttribute(attention_simt_kernel<TQ, TC, TO>,                                \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
    attention_simt_kernel<TQ, TC, TO><<<grid, threads, smem, stream>>>(                      \
        (const TQ*)q, q_stride, (const TC*)cache, block_table, bt_stride, token_req, positions, \
        (TO*)out, o_stride, T, H, Hkv, D, page_size, scale, window, max_keys, n_pages, err); \
  } while (0)
  if (act_dtype == SGLC_F32 && cache_dtype == SGLC_F32)
    LAUNCH(float, float, float);
  else if (act_dtype == SGLC_BF16 && cache_dtype == SGLC_BF16)
    LAUNCH(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
  else
    return SGLC_ERR_ARGUMENT;
#undef LAUNCH
  return sglc_launch_status();
}
