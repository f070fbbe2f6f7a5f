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


// the shared::cluster address of `local` as it lies in the block of rank `cta_rank`
__device__ __forceinline__ uint32_t map_to_peer(const void* local, int cta_rank) {
  uint32_t laddr = (uint32_t)__cvta_generic_to_shared(local), raddr;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"(laddr), "r"(cta_rank));
  return raddr;
}
__device__ __forceinline__ void st_peer_f32(uint32_t raddr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(raddr), "f"(v) : "memory");
}

// ---- cross-block signalling inside a cluster (bounded waits) ----
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_init_local(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(bar)), "r"(count));
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_peer(uint32_t remote_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
// false if the limit ran out
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t addr = (uint32_t)__cvta_generic_to_shared(bar);
  for (uint32_t i = 0; i < (1u << 22); ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}

// New keys and values (k_new, v_new: the step's own rows, [T][new_stride], kv heads side by
// side) are optional.  When given, the token's own key and value are taken from them instead
// of the cache, and the block whose range holds the token's position also writes them into
// the cache at slots[t] (page*page_size + offset): the separate cache-write launch is saved.
// token_req may be null: token t is then the t-th request (a step of single tokens).
__global__ void __launch_bounds__(THREADS)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride,
                        __nv_bfloat16* __restrict__ cache,
                        const int* __restrict__ block_table, int bt_stride,
                        const int* __restrict__ token_req, const int* __restrict__ positions,
                        __nv_bfloat16* __restrict__ out, int o_stride, int T, int H, int Hkv, int D,
                        int page_size, float scale, int window, int n_splits, int chunk_cap,
                        int use_cluster, float* __restrict__ ws, int* __restrict__ counters,
                        const __nv_bfloat16* __restrict__ k_new, const __nv_bfloat16* __restrict__ v_new,
                        int new_stride, const int* __restrict__ slots, int nb_max, int* __restrict__ err,
                        const int* __restrict__ token_list, int n_pages) {
  extern __shared__ float smem[];
  __shared__ float red[33];
  __shared__ int s_last;
  __shared__ int s_meta[2];
  __shared__ __align__(8) uint64_t merge_bar;
  // token_list (optional): the tokens this launch serves, when only some of the step's tokens
  // are single decoded tokens (the others are prompt portions served by another kernel)
  const int t = token_list ? token_list[blockIdx.x] : blockIdx.x;
  const int h = blockIdx.y, sp = blockIdx.z;
  float* sq = smem;                     // D
  float* part = sq + D;                 // WARPS * 256 partial outputs
  float* sc = part + WARPS * 256;       // chunk_cap scores
  int* spage = reinterpret_cast<int*>(sc + chunk_cap);   // the request's page ids, nb_max of them
  float* recs = reinterpret_cast<float*>(spage + nb_max);   // merge records (block 0 of a cluster)
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  pdl_launch_dependents();
  if (use_cluster) {
    // block 0's merge barrier exists before any block may signal it: arrive now, wait later
    if (sp == 0 && tid == 0) mbar_init_local(&merge_bar, (uint32_t)(n_splits - 1));
    __syncwarp();
    cluster_arrive();
  }
  // Before waiting for the kernel ahead in the stream: everything that kernel cannot have
  // written.  The step's own data (positions, block tables) was copied in before the step
  // began, and keys and values of EARLIER positions were cached by earlier steps.  Only the
  // query and the token's own key and value (position `pos`) come from the kernel ahead.
  if (token_req == nullptr) {
    const int* bt = block_table + (size_t)t * bt_stride;
    for (int i = tid; i < nb_max; i += THREADS) spage[i] = bt[i];
    if (tid == 0) { s_meta[0] = t; s_meta[1] = positions[t]; }
  } else {
    if (tid == 0) { s_meta[0] = token_req[t]; s_meta[1] = positions[t]; }
  }
  __syncthreads();
  const int r = s_meta[0];
  const int pos = s_meta[1];
  if (token_req != nullptr) {
    const int* bt = block_table + (size_t)r * bt_stride;
    int need = pos / page_size + 1;
    if (need > nb_max) need = nb_max;
    for (int i = tid; i < need; i += THREADS) spage[i] = bt[i];
    __syncthreads();
  }
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int n = pos - lo + 1;
  int chunk = (n + n_splits - 1) / n_splits;
  // The launcher sized the score array and the page list from max_keys; a position beyond it (a
  // caller's max_keys smaller than some positions[t] + 1) would index past both.  Such a token
  // gets zeros and the error word instead; every block of the token takes this way out alike.
  if (pos < 0 || pos / page_size >= nb_max || chunk > chunk_cap) {
    if (sp == 0) {
      __nv_bfloat16* bad = out + (size_t)t * o_stride + (size_t)h * D;
      for (int d = tid; d < D; d += THREADS) bad[d] = __float2bfloat16_rn(0.0f);
      if (tid == 0 && err) atomicExch(err, 1);
    }
    return;
  }
#ifdef SGLC_BOUNDS_CHECK
  // the page ids this token's keys lie in, against the pool's size (see common.cuh)
  for (int i = lo / page_size + tid; i <= pos / page_size; i += THREADS)
    if (!sglc_index_ok(spage[i], n_pages, err)) spage[i] = 0;
  __syncthreads();
#endif
  const int k0 = lo + sp * chunk;
  int k1 = k0 + chunk;
  if (k1 > pos + 1) k1 = pos + 1;
  const int nk = k1 > k0 ? k1 - k0 : 0;
  const int G = H / Hkv;
  const int hk = h / G;
  const size_t page_elems = (size_t)2 * Hkv * page_size * D;
  const size_t head_off = (size_t)hk * page_size * D;
  const size_t v_off = (size_t)Hkv * page_size * D;
  const bool fused = k_new != nullptr;
  const __nv_bfloat16* kn = fused ? k_new + (size_t)t * new_stride + (size_t)hk * D : nullptr;
  const __nv_bfloat16* vn = fused ? v_new + (size_t)t * new_stride + (size_t)hk * D : nullptr;

  // LPR lanes share one key's row (16 bytes each), so a warp reads KG whole rows per load and
  // consecutive keys of a page are one contiguous stretch.  Key index of (round j, this lane)
  // = (j * WARPS + warp) * KG + kg.  The first NPRE rounds of keys AND values are requested
  // before anything is computed, so that they travel together.
  const int LPR = D / 8;
  const int KG = 32 / LPR;
  const int kg = lane / LPR, dl = lane % LPR;
  const bool active = kg < KG;
  const int stride = WARPS * KG;
  const int i_first = warp * KG + kg;
  constexpr int NPRE = 8;
  uint4 kpre[NPRE], vpre[NPRE];
#pragma unroll
  for (int x = 0; x < NPRE; x++) {
    int i = i_first + x * stride;
    kpre[x] = make_uint4(0u, 0u, 0u, 0u);
    vpre[x] = kpre[x];
    if (active && i < nk && k0 + i != pos) {
      int p = k0 + i;
      const __nv_bfloat16* krow =
          cache + (size_t)spage[p / page_size] * page_elems + head_off + (size_t)(p % page_size) * D;
      kpre[x] = __ldg(reinterpret_cast<const uint4*>(krow) + dl);
      vpre[x] = __ldg(reinterpret_cast<const uint4*>(krow + v_off) + dl);
    }
  }
  pdl_wait();
  // now the kernel ahead is complete: the query, and the token's own key and value
  const __nv_bfloat16* qp = q + (size_t)t * q_stride + (size_t)h * D;
  for (int d = tid; d < D; d += THREADS) sq[d] = __bfloat162float(qp[d]) * scale;
#pragma unroll
  for (int x = 0; x < NPRE; x++) {
    int i = i_first + x * stride;
    if (active && i < nk && k0 + i == pos) {
      const __nv_bfloat16* krow = fused ? kn
          : cache + (size_t)spage[pos / page_size] * page_elems + head_off + (size_t)(pos % page_size) * D;
      const __nv_bfloat16* vrow = fused ? vn : krow + v_off;
      // plain loads: this data was written by the kernel ahead, not before the step
      kpre[x] = *(reinterpret_cast<const uint4*>(krow) + dl);
      vpre[x] = *(reinterpret_cast<const uint4*>(vrow) + dl);
    }
  }
  // the token's own key and value into the cache (one head of a group does it)
  if (fused && pos >= k0 && pos < k1 && h % G == 0) {
    int slot = slots[t];
    if (slot >= 0) {
      __nv_bfloat16* dst = cache + (size_t)(slot / page_size) * page_elems + head_off +
                           (size_t)(slot % page_size) * D;
      for (int c = tid; c < D / 8; c += THREADS) {
        reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(kn)[c];
        reinterpret_cast<uint4*>(dst + v_off)[c] = reinterpret_cast<const uint4*>(vn)[c];
      }
    }
  }
  __syncthreads();
  float qreg[8];
#pragma unroll
  for (int y = 0; y < 8; y++) qreg[y] = active ? sq[dl * 8 + y] : 0.0f;
  const bool pow2 = (LPR & (LPR - 1)) == 0;
  auto row_dot = [&](const uint4& u) {
    float f[8];
    bf16x8_to_f32(u, f);
    float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
    for (int y = 0; y < 8; y += 2) {
      s0 = fmaf(qreg[y], f[y], s0);
      s1 = fmaf(qreg[y + 1], f[y + 1], s1);
    }
    float s = s0 + s1;
    if (pow2) {
      for (int o = 1; o < LPR; o <<= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    } else {
      float tot = s;
      for (int o = 1; o < LPR; o++) {
        int src = kg * LPR + (dl + o) % LPR;
        tot += __shfl_sync(0xffffffffu, s, active ? src : lane);
      }
      s = tot;
    }
    return s;
  };
  float lmax = -INFINITY;
#pragma unroll
  for (int x = 0; x < NPRE; x++) {
    int i = i_first + x * stride;
    float s = row_dot(kpre[x]);
    if (active && i < nk) {
      if (dl == 0) sc[i] = s;
      lmax = fmaxf(lmax, s);
    }
  }
  // further rounds; the loop bound is the same for every lane of a warp (shuffles inside)
  for (int wb = warp * KG + NPRE * stride; wb < nk; wb += 4 * stride) {
    const int i0 = wb + kg;
    uint4 u[4];
#pragma unroll
    for (int x = 0; x < 4; x++) {
      int i = i0 + x * stride;
      u[x] = make_uint4(0u, 0u, 0u, 0u);
      if (active && i < nk) {
        int p = k0 + i;
        const __nv_bfloat16* krow = (fused && p == pos)
            ? kn
            : cache + (size_t)spage[p / page_size] * page_elems + head_off + (size_t)(p % page_size) * D;
        u[x] = p == pos ? *(reinterpret_cast<const uint4*>(krow) + dl)
                        : __ldg(reinterpret_cast<const uint4*>(krow) + dl);
      }
    }
#pragma unroll
    for (int x = 0; x < 4; x++) {
      int i = i0 + x * stride;
      float s = row_dot(u[x]);
      if (active && i < nk) {
        if (dl == 0) sc[i] = s;
        lmax = fmaxf(lmax, s);
      }
    }
  }
  const float m = block_max(lmax, red);
  float lsum = 0.0f;
  for (int i = tid; i < nk; i += THREADS) {
    float e = expf(sc[i] - m);
    sc[i] = e;
    lsum += e;
  }
  const float l = block_sum(lsum, red);     // also orders the writes of sc before the reads below

  float acc[8];
#pragma unroll
  for (int x = 0; x < 8; x++) acc[x] = 0.0f;
#pragma unroll
  for (int x = 0; x < NPRE; x++) {
    int i = i_first + x * stride;
    float w = (active && i < nk) ? sc[i] : 0.0f;
    float f[8];
    bf16x8_to_f32(vpre[x], f);
#pragma unroll
    for (int y = 0; y < 8; y++) acc[y] = fmaf(w, f[y], acc[y]);
  }
  for (int wb = warp * KG + NPRE * stride; wb < nk; wb += 4 * stride) {
    const int i0 = wb + kg;
    uint4 u[4];
    float w[4];
#pragma unroll
    for (int x = 0; x < 4; x++) {
      int i = i0 + x * stride;
      w[x] = 0.0f;
      u[x] = make_uint4(0u, 0u, 0u, 0u);
      if (active && i < nk) {
        int p = k0 + i;
        const __nv_bfloat16* vp = (fused && p == pos)
            ? vn
            : cache + (size_t)spage[p / page_size] * page_elems + v_off + head_off +
                  (size_t)(p % page_size) * D;
        u[x] = p == pos ? *(reinterpret_cast<const uint4*>(vp) + dl)
                        : __ldg(reinterpret_cast<const uint4*>(vp) + dl);
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
    // the ranges of one (token, head) are the blocks of a cluster.  Blocks 1.. send their
    // (m, l, o) to block 0's shared memory and signal its barrier; block 0 waits for all of
    // them (with a limit) and merges in range order.  Nothing remote is touched by a block
    // after its signal, and block 0 outlives every store into it (when its wait runs out,
    // through the cluster's hardware barrier: see there).
    __syncwarp();
    cluster_wait();                  // pairs with the arrive at the top: block 0's barrier exists
    float* dst_local = recs + (size_t)sp * rec;
    if (sp == 0) {
      for (int d = tid; d < D; d += THREADS) {
        float o = 0.0f;
        for (int w = 0; w < n_part; w++) o += part[w * D + d];
        dst_local[2 + d] = o;
      }
      if (tid == 0) { dst_local[0] = m; dst_local[1] = l; }
      __syncthreads();
      if (!mbar_wait_cluster(&merge_bar, 0)) {
        if (tid == 0 && err) atomicExch(err, 1);
        // a peer that has not signalled may still be storing into this block's shared memory:
        // the cluster's hardware barrier completes when every block of it has arrived or
        // exited, and the peers exit right after their stores, so this block leaves last
        cluster_arrive();
        cluster_wait();
        return;
      }
    } else {
      const uint32_t dst = map_to_peer(dst_local, 0);
      for (int d = tid; d < D; d += THREADS) {
        float o = 0.0f;
        for (int w = 0; w < n_part; w++) o += part[w * D + d];
        st_peer_f32(dst + (uint32_t)(2 + d) * 4u, o);
      }
      if (tid == 0) {
        st_peer_f32(dst, m);
        st_peer_f32(dst + 4u, l);
      }
      __syncthreads();
      if (tid == 0) mbar_arrive_peer(map_to_peer(&merge_bar, 0));
      return;
    }
    float M = -INFINITY;
    for (int s = 0; s < n_splits; s++) M = fmaxf(M, recs[s * rec]);
    float L = 0.0f;
    for (int s = 0; s < n_splits; s++) L += recs[s * rec + 1] > 0.0f ? recs[s * rec + 1] * expf(recs[s * rec] - M) : 0.0f;
    float inv = 1.0f / L;
    for (int d = tid; d < D; d += THREADS) {
      float o = 0.0f;
      for (int s = 0; s < n_splits; s++)
        if (recs[s * rec + 1] > 0.0f) o += recs[s * rec + 2 + d] * expf(recs[s * rec] - M);
      op[d] = __float2bfloat16_rn(o * inv);
    }
    return;
  }
  // more ranges than a cluster holds: (m, l, o) of this range go to a workspace in global
  // memory, and the block that arrives last merges all ranges
  float* mine = ws + ((size_t)(blockIdx.x * H + h) * n_splits + sp) * rec;
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
    int old = atomicAdd(&counters[blockIdx.x * H + h], 1);
    s_last = (old == n_splits - 1);
    if (old == n_splits - 1) counters[blockIdx.x * H + h] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const float* all = ws + (size_t)(blockIdx.x * H + h) * n_splits * rec;
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
  // a block should not walk more than about 128 keys: beyond what it requests up front, every
  // further round of keys costs a trip to memory (measured at 8 requests of 512 keys: 8 ranges
  // 409 us a step, 4 ranges 415)
  int by_len = (max_keys + 127) / 128;
  if (by_len > 8) by_len = 8;
  if (want < by_len) want = by_len;
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
// T: the number of tokens this launch serves (all of the step's, or those named by token_list).
// k_new, v_new (bfloat16 [T][new_stride]) and slots (int32 [T]) may be null; when given, the
// tokens' own keys and values are read from them and written into the cache by this launch.
SGLC_API int sglc_attention_decode(const void* q, int q_stride, void* cache,
                                   const int* block_table, int bt_stride, const int* token_req,
                                   const int* positions, void* out, int o_stride, int T, int H,
                                   int Hkv, int D, int page_size, float scale, int window,
                                   int max_keys, int n_splits, float* ws, int* counters,
                                   const void* k_new, const void* v_new, int new_stride,
                                   const int* slots, int* err, const int* token_list, int n_pages,
                                   cudaStream_t stream) {
  if (T <= 0) return SGLC_OK;
  if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || page_size <= 0 || max_keys <= 0 || n_splits < 1)
    return SGLC_ERR_ARGUMENT;
  if (D % 8 != 0 || D > 256 || H > 65535 || n_splits > 65535) return SGLC_ERR_UNSUPPORTED;
  if (q_stride % 8 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)cache & 15)) return SGLC_ERR_UNSUPPORTED;
  if (n_splits > 8 && (!ws || !counters)) return SGLC_ERR_ARGUMENT;
  if (k_new && (!v_new || !slots || new_stride % 8 != 0 || ((uintptr_t)k_new & 15) || ((uintptr_t)v_new & 15)))
    return SGLC_ERR_UNSUPPORTED;
  int eff = window > 0 && window < max_keys ? window : max_keys;
  int chunk_cap = (eff + n_splits - 1) / n_splits;
  if (chunk_cap < 2 * n_splits) chunk_cap = 2 * n_splits;   // the merge reuses the score array
  int nb_max = (max_keys + page_size - 1) / page_size;
  if (nb_max > bt_stride) nb_max = bt_stride;
  size_t smem = ((size_t)D + (size_t)WARPS * 256 + (size_t)chunk_cap + (size_t)nb_max +
                 (size_t)8 * (D + 2)) * sizeof(float);
  if (smem > 200 * 1024) return SGLC_ERR_UNSUPPORTED;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)smem);
  dim3 grid(T, H, n_splits);
  int use_cluster = (n_splits > 1 && n_splits <= 8) ? 1 : 0;
  return sglc_launch(attention_decode_kernel, grid, dim3(THREADS), smem, stream,
                     use_cluster ? n_splits : 1, true, (const __nv_bfloat16*)q, q_stride,
                     (__nv_bfloat16*)cache, block_table, bt_stride, token_req, positions,
                     (__nv_bfloat16*)out, o_stride, T, H, Hkv, D, page_size, scale, window, n_splits,
                     chunk_cap, use_cluster, ws, counters, (const __nv_bfloat16*)k_new,
                     (const __nv_bfloat16*)v_new, new_stride, slots, nb_max, err, token_list, n_pages);
}

// ---------------------------------------------------------------------------------------
// The same kernel for callers that cannot allocate: the merge scratch is a fixed array in
// this library (see attention_decode_noalloc.h for who needs this and the rules of use).
#include "attention_decode_noalloc.h"

// [SGLC_NOALLOC_MAX_WS_FLOATS floats of (m, l, o) records][SGLC_NOALLOC_MAX_COUNTERS ints]
// [one int: set by a launch that met a position beyond its max_keys][padding]
static __device__ __align__(256) unsigned char g_noalloc_scratch[SGLC_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
// In host code `g_noalloc_scratch` is only a stand-in for the symbol, not a device address;
// the address a kernel can use comes from cudaGetSymbolAddress, once per device.
// (Filled without a lock: two host threads that make a device's first call at once both look the
// address up and both store the same value.)
void* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};
constexpr size_t NOALLOC_STATUS_OFFSET = (size_t)SGLC_NOALLOC_MAX_WS_FLOATS * 4 + (size_t)SGLC_NOALLOC_MAX_COUNTERS * 4;

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
  if (code == SGLC_NOALLOC_ERR_POSITION)
    return "a token's position lies beyond max_keys - 1 (its output was set to zero): pass a max_keys "
           "that covers every positions[t] + 1";
  return sglc_error_string(code);
}

SGLC_API int sglc_attention_decode_noalloc_check(cudaStream_t stream) {
  void* base = nullptr;
  int rc = noalloc_scratch(&base);
  if (rc != SGLC_OK) return rc;
  int word = 0;
  int* status = reinterpret_cast<int*>(reinterpret_cast<unsigned char*>(base) + NOALLOC_STATUS_OFFSET);
  cudaError_t e = cudaMemcpyAsync(&word, status, sizeof(int), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return (int)e;
  if (word == 0) return SGLC_OK;
  e = cudaMemsetAsync(status, 0, sizeof(int), stream);
  if (e != cudaSuccess) return (int)e;
  return SGLC_NOALLOC_ERR_POSITION;
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
  int nb_max = (max_keys + page_size - 1) / page_size;
  if (nb_max > bt_stride) nb_max = bt_stride;
  size_t smem = ((size_t)D + (size_t)WARPS * 256 + (size_t)chunk_cap + (size_t)nb_max +
                 (size_t)8 * (D + 2)) * sizeof(float);
  if (smem > 200 * 1024) return SGLC_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    e = cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(T, H, n_splits);
  // ranges always merge through the scratch here (never through a cluster), so the launch is plain
  attention_decode_kernel<<<grid, THREADS, smem, stream>>>(
      (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)const_cast<void*>(cache), block_table,
      bt_stride, token_req, positions, (__nv_bfloat16*)out, o_stride, T, H, Hkv, D, page_size, scale,
      window, n_splits, chunk_cap, /*use_cluster=*/0, ws, counters,
      /*k_new=*/(const __nv_bfloat16*)nullptr, /*v_new=*/(const __nv_bfloat16*)nullptr, 0,
      /*slots=*/(const int*)nullptr, nb_max,
      /*err=*/reinterpret_cast<int*>(reinterpret_cast<unsigned char*>(base) + NOALLOC_STATUS_OFFSET),
      /*token_list=*/(const int*)nullptr, /*n_pages=*/0x7fffffff);
  return sglc_launch_status();
}
