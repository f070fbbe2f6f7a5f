// Attention for single decoded tokens over the paged bfloat16 cache, with the keys of one
// query split across blocks (each block: one (token, head, key range)).
//   s[p] = (q·K_p)*scale; per range: m = max s, e = exp(s-m), l = sum e, o = sum e*V_p;
//   ranges are merged as  M = max m_i,  o = sum_i o_i*exp(m_i-M) / sum_i l_i*exp(m_i-M)
// always in range order by the block that finishes last, so the result does not depend on
// timing.  All arithmetic is 32-bit.  Lengths, positions and block tables are read from
// device arrays, so the launch has a fixed shape and can be replayed from a CUDA graph.
// The reference's closest kernels: k_attn_batch (src/cuda_backend.cu:3172-3223, decode over
// a contiguous cache, scores in shared memory) and k_attn_q_split_partial/_merge
// (:2056-2185, split keys over a paged, quantised pool with a separate merge launch).
#include "common.cuh"

SGLC_DEFINE_ERROR_STRING()

namespace {
constexpr int THREADS = 128;
constexpr int WARPS = THREADS / 32;

__device__ __forceinline__ void bf16x8_to_f32(const uint4& u, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_peer_f32(const float* local, int cta_rank) {
  uint32_t laddr = (uint32_t)__cvta_generic_to_shared(local), raddr;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"(laddr), "r"(cta_rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(raddr) : "memory");
  return v;
}

__global__ void __launch_bounds__(THREADS)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride,
                        const __nv_bfloat16* __restrict__ cache,
                        const int* __restrict__ block_table, int bt_stride,
                        const int* __restrict__ token_req, const int* __restrict__ positions,
                        __nv_bfloat16* __restrict__ out, int o_stride, int T, int H, int Hkv, int D,
                        int page_size, float scale, int window, int n_splits, int chunk_cap,
                        int use_cluster, float* __restrict__ ws, int* __restrict__ counters) {
  extern __shared__ float smem[];
  __shared__ float red[33];
  __shared__ int s_last;
  const int t = blockIdx.x, h = blockIdx.y, sp = blockIdx.z;
  float* sq = smem;                     // D
  float* part = sq + D;                 // WARPS * 256 partial outputs
  float* sc = part + WARPS * 256;       // chunk_cap scores
  int* spage = reinterpret_cast<int*>(sc + chunk_cap);   // pages of this range
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r = token_req[t];
  const int pos = positions[t];
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int n = pos - lo + 1;
  int chunk = (n + n_splits - 1) / n_splits;
  if (chunk > chunk_cap) chunk = chunk_cap;          // cannot happen when the host sized chunk_cap
  const int k0 = lo + sp * chunk;
  int k1 = k0 + chunk;
  if (k1 > pos + 1) k1 = pos + 1;
  const int nk = k1 > k0 ? k1 - k0 : 0;
  const int hk = h / (H / Hkv);
  const int* bt = block_table + (size_t)r * bt_stride;
  const size_t page_elems = (size_t)2 * Hkv * page_size * D;
  const size_t head_off = (size_t)hk * page_size * D;
  const size_t v_off = (size_t)Hkv * page_size * D;

  // the range's page ids once, so that the loops below issue independent loads
  const int b0 = k0 / page_size;
  const int nb = nk > 0 ? (k1 - 1) / page_size - b0 + 1 : 0;
  for (int i = tid; i < nb; i += THREADS) spage[i] = bt[b0 + i];
  const __nv_bfloat16* qp = q + (size_t)t * q_stride + (size_t)h * D;
  for (int d = tid; d < D; d += THREADS) sq[d] = __bfloat162float(qp[d]) * scale;
  __syncthreads();

  // scores: one key per thread, its row read as 16-byte vectors, eight in flight
  float lmax = -INFINITY;
  for (int i = tid; i < nk; i += THREADS) {
    int p = k0 + i;
    int page = spage[p / page_size - b0];
    const uint4* kp = reinterpret_cast<const uint4*>(cache + (size_t)page * page_elems + head_off +
                                                     (size_t)(p % page_size) * D);
    float s0 = 0.0f, s1 = 0.0f;
    for (int g = 0; g < D / 8; g += 8) {
      uint4 u[8];
#pragma unroll
      for (int x = 0; x < 8; x++)
        if (g + x < D / 8) u[x] = __ldg(kp + g + x);
#pragma unroll
      for (int x = 0; x < 8; x++) {
        if (g + x < D / 8) {
          float f[8];
          bf16x8_to_f32(u[x], f);
          const float* qq = sq + (g + x) * 8;
          s0 = fmaf(qq[0], f[0], s0); s1 = fmaf(qq[1], f[1], s1);
          s0 = fmaf(qq[2], f[2], s0); s1 = fmaf(qq[3], f[3], s1);
          s0 = fmaf(qq[4], f[4], s0); s1 = fmaf(qq[5], f[5], s1);
          s0 = fmaf(qq[6], f[6], s0); s1 = fmaf(qq[7], f[7], s1);
        }
      }
    }
    float s = s0 + s1;
    sc[i] = s;
    lmax = fmaxf(lmax, s);
  }
  const float m = block_max(lmax, red);
  float lsum = 0.0f;
  for (int i = tid; i < nk; i += THREADS) {
    float e = expf(sc[i] - m);
    sc[i] = e;
    lsum += e;
  }
  const float l = block_sum(lsum, red);     // also orders the writes of sc before the reads below

  // values: LPR lanes share one key's row (16 bytes each), so a warp reads KG keys per load;
  // key index = (j * WARPS + warp) * KG + kg, four loads in flight per lane
  const int LPR = D / 8;
  const int KG = 32 / LPR;
  const int kg = lane / LPR, dl = lane % LPR;
  const bool active = kg < KG;
  float acc[8];
#pragma unroll
  for (int x = 0; x < 8; x++) acc[x] = 0.0f;
  const int stride = WARPS * KG;
  for (int i0 = warp * KG + kg; i0 < nk; i0 += 4 * stride) {
    uint4 u[4];
    float w[4];
#pragma unroll
    for (int x = 0; x < 4; x++) {
      int i = i0 + x * stride;
      w[x] = 0.0f;
      u[x] = make_uint4(0u, 0u, 0u, 0u);
      if (active && i < nk) {
        int p = k0 + i;
        int page = spage[p / page_size - b0];
        u[x] = __ldg(reinterpret_cast<const uint4*>(cache + (size_t)page * page_elems + v_off +
                                                    head_off + (size_t)(p % page_size) * D) + dl);
        w[x] = sc[i];
      }
    }
#pragma unroll
    for (int x = 0; x < 4; x++) {
      float f[8];
      bf16x8_to_f32(u[x], f);
#pragma unroll
      for (int y = 0; y < 8; y++) acc[y] = fmaf(w[x], f[y], acc[y]);
    }
  }
  // part[warp][kg][d]; summed below in a fixed order
  if (active) {
#pragma unroll
    for (int y = 0; y < 8; y++) part[(warp * KG + kg) * D + dl * 8 + y] = acc[y];
  }
  __syncthreads();
  const int n_part = WARPS * KG;

  __nv_bfloat16* op = out + (size_t)t * o_stride + (size_t)h * D;
  if (n_splits == 1) {
    float inv = 1.0f / l;
    for (int d = tid; d < D; d += THREADS) {
      float o = 0.0f;
      for (int w = 0; w < n_part; w++) o += part[w * D + d];
      op[d] = __float2bfloat16_rn(o * inv);
    }
    return;
  }
  const int rec = D + 2;
  if (use_cluster) {
    // the ranges of one (token, head) are the blocks of a cluster: each leaves (m, l, o) in
    // its own shared memory, and after a cluster barrier block 0 merges them in range order
    float* mine = part + WARPS * 256 - rec;      // the tail of the partial-output area is free
    float osum[2];
    int cnt = 0;
    for (int d = tid; d < D; d += THREADS) {
      float o = 0.0f;
      for (int w = 0; w < n_part; w++) o += part[w * D + d];
      osum[cnt++] = o;
    }
    __syncthreads();
    cnt = 0;
    for (int d = tid; d < D; d += THREADS) mine[2 + d] = osum[cnt++];
    if (tid == 0) {
      mine[0] = m;
      mine[1] = l;
    }
    __syncthreads();
    cluster_sync_all();
    if (sp == 0) {
      float M = -INFINITY;
      for (int s = 0; s < n_splits; s++) M = fmaxf(M, ld_peer_f32(mine, s));
      float L = 0.0f;
      for (int s = 0; s < n_splits; s++) {
        float ls = ld_peer_f32(mine + 1, s);
        L += ls > 0.0f ? ls * expf(ld_peer_f32(mine, s) - M) : 0.0f;
      }
      float inv = 1.0f / L;
      for (int d = tid; d < D; d += THREADS) {
        float o = 0.0f;
        for (int s = 0; s < n_splits; s++) {
          float ls = ld_peer_f32(mine + 1, s);
          if (ls > 0.0f) o += ld_peer_f32(mine + 2 + d, s) * expf(ld_peer_f32(mine, s) - M);
        }
        op[d] = __float2bfloat16_rn(o * inv);
      }
    }
    cluster_sync_all();      // no block exits while block 0 still reads its shared memory
    return;
  }
  // more ranges than a cluster holds: (m, l, o) of this range go to a workspace in global
  // memory, and the block that arrives last merges all ranges
  float* mine = ws + ((size_t)(t * H + h) * n_splits + sp) * rec;
  for (int d = tid; d < D; d += THREADS) {
    float o = 0.0f;
    for (int w = 0; w < n_part; w++) o += part[w * D + d];
    mine[2 + d] = o;
  }
  if (tid == 0) {
    mine[0] = m;
    mine[1] = l;
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    int old = atomicAdd(&counters[t * H + h], 1);
    s_last = (old == n_splits - 1);
    if (old == n_splits - 1) counters[t * H + h] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const float* all = ws + (size_t)(t * H + h) * n_splits * rec;
  // the ranges' (m, l) into shared memory, then every thread merges its output elements
  float* sm = sc;                   // reuse: 2 * n_splits floats
  for (int s = tid; s < 2 * n_splits; s += THREADS) sm[s] = __ldcg(all + (size_t)(s >> 1) * rec + (s & 1));
  __syncthreads();
  float M = -INFINITY;
  for (int s = 0; s < n_splits; s++) M = fmaxf(M, sm[2 * s]);
  float L = 0.0f;
  for (int s = 0; s < n_splits; s++) L += sm[2 * s + 1] > 0.0f ? sm[2 * s + 1] * expf(sm[2 * s] - M) : 0.0f;
  float inv = 1.0f / L;
  for (int d = tid; d < D; d += THREADS) {
    float o = 0.0f;
#pragma unroll 8
    for (int s = 0; s < n_splits; s++) {
      float v = __ldcg(all + (size_t)s * rec + 2 + d);
      o += sm[2 * s + 1] > 0.0f ? v * expf(sm[2 * s] - M) : 0.0f;
    }
    op[d] = __float2bfloat16_rn(o * inv);
  }
}
}  // namespace

// Scratch the launch needs: floats of workspace and counters (zero between launches).
// Up to 8 ranges are merged inside a thread-block cluster and need no scratch.
SGLC_API int sglc_attention_decode_scratch(int T, int H, int D, int n_splits, long long* ws_floats,
                                           int* n_counters) {
  *ws_floats = n_splits > 8 ? (long long)T * H * n_splits * (D + 2) : 0;
  *n_counters = n_splits > 8 ? T * H : 0;
  return SGLC_OK;
}

// How many key ranges the launcher would use for T tokens of H heads with up to max_keys keys.
SGLC_API int sglc_attention_decode_splits(int T, int H, int max_keys) {
  long long blocks = (long long)T * H;
  int want = (int)((2 * 148 + blocks - 1) / blocks);
  int most = (max_keys + 63) / 64;
  if (want > most) want = most;
  // up to 8 ranges merge inside a cluster; more only when there are very few (token, head) pairs
  if (want > 8 && blocks * 8 >= 64) want = 8;
  if (want > 32) want = 32;
  if (want < 1) want = 1;
  return want;
}

// q, out: bfloat16 rows ([T][q_stride], [T][o_stride]), heads side by side; cache: one layer's
// bfloat16 pages [n_pages][2][Hkv][page_size][D]; positions[t]: the token's own position (the
// last key it sees); max_keys: the most keys any token sees (sizes shared memory).
SGLC_API int sglc_attention_decode(const void* q, int q_stride, const void* cache,
                                   const int* block_table, int bt_stride, const int* token_req,
                                   const int* positions, void* out, int o_stride, int T, int H,
                                   int Hkv, int D, int page_size, float scale, int window,
                                   int max_keys, int n_splits, float* ws, int* counters,
                                   cudaStream_t stream) {
  if (T <= 0) return SGLC_OK;
  if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || page_size <= 0 || max_keys <= 0 || n_splits < 1)
    return SGLC_ERR_ARGUMENT;
  if (D % 8 != 0 || D > 256 || H > 65535 || n_splits > 65535) return SGLC_ERR_UNSUPPORTED;
  if (q_stride % 8 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)cache & 15)) return SGLC_ERR_UNSUPPORTED;
  if (n_splits > 8 && (!ws || !counters)) return SGLC_ERR_ARGUMENT;
  int eff = window > 0 && window < max_keys ? window : max_keys;
  int chunk_cap = (eff + n_splits - 1) / n_splits;
  if (chunk_cap < 2 * n_splits) chunk_cap = 2 * n_splits;   // the merge reuses the score array
  size_t n_page_ids = (size_t)chunk_cap / page_size + 2;
  size_t smem = ((size_t)D + (size_t)WARPS * 256 + (size_t)chunk_cap + n_page_ids) * sizeof(float);
  if (smem > 200 * 1024) return SGLC_ERR_UNSUPPORTED;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)smem);
  dim3 grid(T, H, n_splits);
  int use_cluster = (n_splits > 1 && n_splits <= 8) ? 1 : 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = use_cluster ? n_splits : 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(
      &cfg, attention_decode_kernel, (const __nv_bfloat16*)q, q_stride,
      (const __nv_bfloat16*)cache, block_table, bt_stride, token_req, positions,
      (__nv_bfloat16*)out, o_stride, T, H, Hkv, D, page_size, scale, window, n_splits, chunk_cap,
      use_cluster, ws, counters);
  if (e != cudaSuccess) return (int)e;
  return sglc_launch_status();
}

// ---------------------------------------------------------------------------------------
// The same kernel for callers that cannot allocate: the merge scratch is a fixed array in
// this library (see attention_decode_noalloc.h for who needs this and the rules of use).
#include "attention_decode_noalloc.h"

// [SGLC_NOALLOC_MAX_WS_FLOATS floats of (m, l, o) records][SGLC_NOALLOC_MAX_COUNTERS ints]
static __device__ __align__(256) unsigned char g_noalloc_scratch[SGLC_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
// In host code `g_noalloc_scratch` is only a stand-in for the symbol, not a device address;
// the address a kernel can use comes from cudaGetSymbolAddress, once per device.
void* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};

int noalloc_scratch(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return SGLC_NOALLOC_ERR_SETUP;
  if (!g_noalloc_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);     // with `dev` current
    if (e != cudaSuccess) return (int)e;
    if (!p) return SGLC_NOALLOC_ERR_SETUP;
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return SGLC_OK;
}
}  // namespace

SGLC_API const char* sglc_attention_decode_noalloc_error(int code) {
  if (code == SGLC_NOALLOC_ERR_TOO_LARGE)
    return "sizes exceed the built-in scratch of the no-allocation entry point "
           "(T*H*n_splits*(D+2) floats <= 1048576 and T*H <= 16384)";
  if (code == SGLC_NOALLOC_ERR_SETUP)
    return "the address of the built-in scratch could not be looked up on this device";
  return sglc_error_string(code);
}

SGLC_API int sglc_attention_decode_noalloc(const void* q, int q_stride, const void* cache,
                                           const int* block_table, int bt_stride,
                                           const int* token_req, const int* positions, void* out,
                                           int o_stride, int T, int H, int Hkv, int D,
                                           int page_size, float scale, int window, int max_keys,
                                           int n_splits, cudaStream_t stream) {
  if (T <= 0) return SGLC_OK;
  if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || page_size <= 0 || max_keys <= 0 || n_splits < 1 || D <= 0)
    return SGLC_ERR_ARGUMENT;
  if (D % 8 != 0 || D > 256 || H > 65535 || n_splits > 32) return SGLC_ERR_UNSUPPORTED;
  if (q_stride % 8 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)cache & 15)) return SGLC_ERR_UNSUPPORTED;
  long long pairs = (long long)T * H;
  long long floats = pairs * n_splits * (D + 2);
  if (pairs > SGLC_NOALLOC_MAX_COUNTERS || floats > SGLC_NOALLOC_MAX_WS_FLOATS)
    return SGLC_NOALLOC_ERR_TOO_LARGE;
  void* base = nullptr;
  int rc = noalloc_scratch(&base);
  if (rc != SGLC_OK) return rc;
  float* ws = reinterpret_cast<float*>(base);
  int* counters = reinterpret_cast<int*>(reinterpret_cast<unsigned char*>(base) +
                                         (size_t)SGLC_NOALLOC_MAX_WS_FLOATS * 4);
  // the counters must start at zero; an earlier call that was cut short may have left some set
  cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)pairs * sizeof(int), stream);
  if (e != cudaSuccess) return (int)e;
  int eff = window > 0 && window < max_keys ? window : max_keys;
  int chunk_cap = (eff + n_splits - 1) / n_splits;
  if (chunk_cap < 2 * n_splits) chunk_cap = 2 * n_splits;
  size_t n_page_ids = (size_t)chunk_cap / page_size + 2;
  size_t smem = ((size_t)D + (size_t)WARPS * 256 + (size_t)chunk_cap + n_page_ids) * sizeof(float);
  if (smem > 200 * 1024) return SGLC_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    e = cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(T, H, n_splits);
  // ranges always merge through the scratch here (never through a cluster), so the launch is plain
  attention_decode_kernel<<<grid, THREADS, smem, stream>>>(
      (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)cache, block_table, bt_stride,
      token_req, positions, (__nv_bfloat16*)out, o_stride, T, H, Hkv, D, page_size, scale, window,
      n_splits, chunk_cap, /*use_cluster=*/0, ws, counters);
  return sglc_launch_status();
}
