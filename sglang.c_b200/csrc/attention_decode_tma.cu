// Attention for single decoded tokens, keys and values staged through shared memory by TMA.
// The same arithmetic and the same merge as attention_decode.cu (one block per (token, head,
// key range); ranges merged in range order inside a thread-block cluster), but the range's
// pages are brought in as one 5-D TMA box per page and K/V instead of per-thread loads held in
// registers.  A block then needs few registers and about 40 KB of shared memory, so five or
// more blocks fit on an SM: at large batches, where the register version is bound by how many
// blocks an SM holds, this one keeps several times more bytes in flight.
// Head sizes 64 and 128, bfloat16, up to 8 key ranges (other cases: attention_decode.cu).
// The reference's counterparts are named in attention_decode.cu.
#include <string.h>

#include <mutex>
#include <utility>
#include <vector>

#include "common.cuh"
#include "tc_common.cuh"

SGLC_DEFINE_ERROR_STRING()

namespace {
using namespace tc;
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
__device__ __forceinline__ void st_peer_f32(uint32_t raddr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(raddr), "f"(v) : "memory");
}

struct Args {
  const __nv_bfloat16* q;
  int q_stride;
  __nv_bfloat16* cache;
  const int* block_table;
  int bt_stride;
  const int* token_req;      // null: token t is the step's t-th request
  const int* positions;
  const int* token_list;     // null: the launch serves tokens 0..T-1
  __nv_bfloat16* out;
  int o_stride;
  int H, Hkv, page_size;
  float scale;
  int window;
  int n_splits, chunk_cap, rows_cap, nb_max;
  const __nv_bfloat16* k_new;   // optional: the step's own keys / values and their cache slots
  const __nv_bfloat16* v_new;
  int new_stride;
  const int* slots;
  int* err;
};

template <int D>
__global__ void __launch_bounds__(THREADS)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_kv, const Args a) {
  extern __shared__ __align__(128) uint8_t smem[];
  // [K rows_cap x D][V rows_cap x D][q D floats][part WARPS*256][scores rows_cap][pages nb_max][records 8*(D+2)]
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smem);
  __nv_bfloat16* sV = sK + (size_t)a.rows_cap * D;
  float* sq = reinterpret_cast<float*>(sV + (size_t)a.rows_cap * D);
  float* part = sq + D;
  float* sc = part + WARPS * 256;
  int* spage = reinterpret_cast<int*>(sc + a.rows_cap);
  float* recs = reinterpret_cast<float*>(spage + a.nb_max);
  __shared__ float red[33];
  __shared__ int s_meta[2];
  __shared__ int s_abort;
  __shared__ __align__(8) uint64_t load_bar;
  __shared__ __align__(8) uint64_t merge_bar;

  const int t = a.token_list ? a.token_list[blockIdx.x] : blockIdx.x;
  const int h = blockIdx.y, sp = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_splits = a.n_splits, ps = a.page_size;
  pdl_launch_dependents();
  if (tid == 0) {
    mbar_init(&load_bar, 1);
    if (n_splits > 1 && sp == 0) mbar_init(&merge_bar, (uint32_t)(n_splits - 1));
    s_abort = 0;
    mbar_fence_init();
  }
  if (n_splits > 1) {
    // block 0's merge barrier exists before any block may signal it: arrive now, wait later
    __syncwarp();
    cluster_arrive();
  }
  // Before waiting for the kernel ahead: the step's metadata and the pages of EARLIER
  // positions, which that kernel cannot have written.
  if (a.token_req == nullptr) {
    const int* bt = a.block_table + (size_t)t * a.bt_stride;
    for (int i = tid; i < a.nb_max; i += THREADS) spage[i] = bt[i];
    if (tid == 0) { s_meta[0] = t; s_meta[1] = a.positions[t]; }
  } else {
    if (tid == 0) { s_meta[0] = a.token_req[t]; s_meta[1] = a.positions[t]; }
  }
  __syncthreads();
  const int r = s_meta[0];
  const int pos = s_meta[1];
  if (a.token_req != nullptr) {
    const int* bt = a.block_table + (size_t)r * a.bt_stride;
    int need = pos / ps + 1;
    if (need > a.nb_max) need = a.nb_max;
    for (int i = tid; i < need; i += THREADS) spage[i] = bt[i];
    __syncthreads();
  }
  const int lo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
  const int n = pos - lo + 1;
  int chunk = (n + n_splits - 1) / n_splits;
  if (chunk > a.chunk_cap) chunk = a.chunk_cap;      // cannot happen when the host sized chunk_cap
  const int k0 = lo + sp * chunk;
  int k1 = k0 + chunk;
  if (k1 > pos + 1) k1 = pos + 1;
  const int nk = k1 > k0 ? k1 - k0 : 0;
  const int G = a.H / a.Hkv;
  const int hk = h / G;
  const int pg0 = k0 / ps;
  const int pg1 = nk > 0 ? (k1 - 1) / ps : pg0 - 1;   // inclusive
  const int row0 = k0 - pg0 * ps;                     // the range's first key within the staged pages
  if (tid == 0 && nk > 0) {
    const int npg = pg1 - pg0 + 1;
    mbar_expect_tx(&load_bar, (uint32_t)npg * 2u * (uint32_t)ps * (uint32_t)D * 2u);
    for (int pi = pg0; pi <= pg1; pi++) {
      const int page = spage[pi];
      tma_load_5d(sK + (size_t)(pi - pg0) * ps * D, &map_kv, &load_bar, 0, 0, hk, 0, page);
      tma_load_5d(sV + (size_t)(pi - pg0) * ps * D, &map_kv, &load_bar, 0, 0, hk, 1, page);
    }
  }
  pdl_wait();
  // now the kernel ahead is complete: the query, and the token's own key and value
  const __nv_bfloat16* qp = a.q + (size_t)t * a.q_stride + (size_t)h * D;
  for (int d = tid; d < D; d += THREADS) sq[d] = __bfloat162float(qp[d]) * a.scale;
  bool ok = true;
  if (nk > 0) {
    volatile int* af = &s_abort;
    ok = mbar_wait(&load_bar, 0, af);
  }
  const bool fused = a.k_new != nullptr;
  if (ok && pos >= k0 && pos < k1) {
    // the token's own row: from the step's rows (and into the cache), or re-read from the cache,
    // where the kernel ahead put it after the page was requested
    const size_t page_elems = (size_t)2 * a.Hkv * ps * D;
    const size_t head_off = (size_t)hk * ps * D, v_off = (size_t)a.Hkv * ps * D;
    const __nv_bfloat16* ksrc;
    const __nv_bfloat16* vsrc;
    if (fused) {
      ksrc = a.k_new + (size_t)t * a.new_stride + (size_t)hk * D;
      vsrc = a.v_new + (size_t)t * a.new_stride + (size_t)hk * D;
    } else {
      ksrc = a.cache + (size_t)spage[pos / ps] * page_elems + head_off + (size_t)(pos % ps) * D;
      vsrc = ksrc + v_off;
    }
    const int row = pos - pg0 * ps;
    __nv_bfloat16* kdst = nullptr;
    if (fused && h % G == 0) {
      int slot = a.slots[t];
      if (slot >= 0) kdst = a.cache + (size_t)(slot / ps) * page_elems + head_off + (size_t)(slot % ps) * D;
    }
    for (int c = tid; c < D / 8; c += THREADS) {
      uint4 kv = reinterpret_cast<const uint4*>(ksrc)[c];
      uint4 vv = reinterpret_cast<const uint4*>(vsrc)[c];
      reinterpret_cast<uint4*>(sK + (size_t)row * D)[c] = kv;
      reinterpret_cast<uint4*>(sV + (size_t)row * D)[c] = vv;
      if (kdst) {
        reinterpret_cast<uint4*>(kdst)[c] = kv;
        reinterpret_cast<uint4*>(kdst + v_off)[c] = vv;
      }
    }
  }
  __syncthreads();

  // LPR lanes share one key's row (16 bytes each): a warp reads KG whole rows at a time
  constexpr int LPR = D / 8;
  constexpr int KG = 32 / LPR;
  const int kg = lane / LPR, dl = lane % LPR;
  const int stride = WARPS * KG;
  float qreg[8];
#pragma unroll
  for (int y = 0; y < 8; y++) qreg[y] = sq[dl * 8 + y];
  float lmax = -INFINITY;
  if (ok) {
    for (int wb = warp * KG; wb < nk; wb += stride) {      // the bound is the same for the whole warp
      const int i = wb + kg;
      float s = 0.0f;
      if (i < nk) {
        uint4 u = *reinterpret_cast<const uint4*>(sK + (size_t)(row0 + i) * D + dl * 8);
        float f[8];
        bf16x8_to_f32(u, f);
        float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
        for (int y = 0; y < 8; y += 2) {
          s0 = fmaf(qreg[y], f[y], s0);
          s1 = fmaf(qreg[y + 1], f[y + 1], s1);
        }
        s = s0 + s1;
      }
#pragma unroll
      for (int o = 1; o < LPR; o <<= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (i < nk) {
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
  if (ok) {
    for (int i = warp * KG + kg; i < nk; i += stride) {
      uint4 u = *reinterpret_cast<const uint4*>(sV + (size_t)(row0 + i) * D + dl * 8);
      float w = sc[i];
      float f[8];
      bf16x8_to_f32(u, f);
#pragma unroll
      for (int y = 0; y < 8; y++) acc[y] = fmaf(w, f[y], acc[y]);
    }
  }
#pragma unroll
  for (int y = 0; y < 8; y++) part[(warp * KG + kg) * D + dl * 8 + y] = acc[y];
  __syncthreads();
  constexpr int n_part = WARPS * KG;

  __nv_bfloat16* op = a.out + (size_t)t * a.o_stride + (size_t)h * D;
  if (n_splits == 1) {
    if (!ok) {
      if (tid == 0 && a.err) atomicExch(a.err, 1);
      return;
    }
    float inv = 1.0f / l;
    for (int d = tid; d < D; d += THREADS) {
      float o = 0.0f;
#pragma unroll
      for (int w = 0; w < n_part; w++) o += part[w * D + d];
      op[d] = __float2bfloat16_rn(o * inv);
    }
    return;
  }
  // Blocks 1.. send their (m, l, o) to block 0's shared memory and signal its barrier; block 0
  // waits for all of them (with a limit) and merges in range order.  Nothing remote is touched by
  // a block after its signal, and block 0 outlives every store into it (when its wait runs out,
  // through the cluster's hardware barrier: see there).
  constexpr int rec = D + 2;
  __syncwarp();
  cluster_wait();                    // pairs with the arrive at the top: block 0's barrier exists
  float* mine = recs + (size_t)sp * rec;
  if (sp != 0) {
    const uint32_t dst = map_to_peer(mine, 0);
    for (int d = tid; d < D; d += THREADS) {
      float o = 0.0f;
#pragma unroll
      for (int w = 0; w < n_part; w++) o += part[w * D + d];
      st_peer_f32(dst + (uint32_t)(2 + d) * 4u, o);
    }
    if (tid == 0) {
      st_peer_f32(dst, ok ? m : -INFINITY);
      st_peer_f32(dst + 4u, ok ? l : 0.0f);
      if (!ok && a.err) atomicExch(a.err, 1);
    }
    __syncthreads();
    if (tid == 0) mbar_arrive_peer(map_to_peer(&merge_bar, 0));
    return;
  }
  for (int d = tid; d < D; d += THREADS) {
    float o = 0.0f;
#pragma unroll
    for (int w = 0; w < n_part; w++) o += part[w * D + d];
    mine[2 + d] = o;
  }
  if (tid == 0) {
    mine[0] = m;
    mine[1] = l;
  }
  __syncthreads();
  {
    volatile int* af = &s_abort;
    if (!mbar_wait_cluster(&merge_bar, 0, af) || !ok) {
      if (tid == 0 && a.err) atomicExch(a.err, 1);
      // a peer that has not signalled may still be storing into this block's shared memory: the
      // cluster's hardware barrier completes when every block of it has arrived or exited, and
      // the peers exit right after their stores, so this block leaves after the last of them
      cluster_arrive();
      cluster_wait();
      return;
    }
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
}

// ---- host: the cache as a 5-D tensor, one box = one page's rows of one head (no swizzle) ----
struct KeyKV { const void* p; int D, ps, Hkv, n_pages, swizzled; };
std::mutex g_mutex;
std::vector<std::pair<KeyKV, CUtensorMap>> g_kvmaps;

// swizzled: boxes 64 elements (128 bytes) wide in the 128-byte swizzle (the streaming kernel's
// ldmatrix reads), else whole rows as they lie
bool get_kv_map(CUtensorMap* out, const void* cache, int D, int ps, int Hkv, int n_pages, bool swizzled = false) {
  std::lock_guard<std::mutex> lock(g_mutex);
  for (auto& e : g_kvmaps)
    if (e.first.p == cache && e.first.D == D && e.first.ps == ps && e.first.Hkv == Hkv &&
        e.first.n_pages == n_pages && e.first.swizzled == (int)swizzled) {
      *out = e.second;
      return true;
    }
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn || ((uintptr_t)cache & 15) || ps > 256 || D > 256) return false;
  cuuint64_t dims[5] = {(cuuint64_t)D, (cuuint64_t)ps, (cuuint64_t)Hkv, 2, (cuuint64_t)n_pages};
  cuuint64_t strides[4] = {(cuuint64_t)D * 2, (cuuint64_t)ps * D * 2, (cuuint64_t)Hkv * ps * D * 2,
                           (cuuint64_t)2 * Hkv * ps * D * 2};
  cuuint32_t box[5] = {(cuuint32_t)(swizzled ? 64 : D), (cuuint32_t)ps, 1, 1, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUtensorMap m;
  CUresult rc = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(cache), dims, strides, box,
                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzled ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return false;
  if (g_kvmaps.size() > 1024) g_kvmaps.clear();
  g_kvmaps.push_back({KeyKV{cache, D, ps, Hkv, n_pages, (int)swizzled}, m});
  *out = m;
  return true;
}

// ---- streaming variant for large batches -------------------------------------------------
// A fixed number of blocks per SM, each walking a list of (token, head) items.  One warp feeds
// a ring of shared-memory stages (64 keys and their values each) with the item's pages by TMA,
// in the 128-byte swizzle, and runs ahead of the four warps that consume them, across item
// boundaries, so a block never waits for a round trip between items: at large batches the
// one-shot kernels are bound by block lifetime times the number of blocks an SM holds, this
// one by bytes.  The four warps share every stage through the warp-level tensor-core
// instruction, the query being row 0 of a 16-row operand: each warp takes the scores of 16 of
// the stage's keys, the scores meet in shared memory (one block barrier a stage), every warp
// then does the same softmax step on all 64 and takes a quarter of the head's output columns.
// (The same sums on the CUDA cores cost eight times the instructions, and the kernel was bound
// by instruction issue.)  No merge at the end of an item: each warp holds the item's maximum
// and sum and its own columns.  The token's own key and value come from the step's rows (or
// the cache) by plain loads after the dependency wait, and are written into the cache here.
// 2^x by the special-function unit (arguments here are <= 0 up to rounding; -inf gives 0)
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// D[16x8] += A[16x16] B[16x8], bfloat16 operands, float accumulators; rows 8..15 of A are zero here
__device__ __forceinline__ void mma_row0(float* d, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

struct StreamArgs {
  Args b;
  int n_items;        // tokens served x heads
  int n_stages;
};
constexpr int S_WARPS = 4;                  // consumer warps; warp S_WARPS produces
constexpr int S_THREADS = (S_WARPS + 1) * 32;
constexpr int S_MAX_STAGES = 8;
constexpr int S_PMAX = 8;                   // page ids held per producer lane: 256 pages per item
constexpr int S_TILE = 64;                  // keys per stage

struct ItemGeom {
  int lo, first_page, k_base, n_rows, n_tiles, n_pages;
};
__device__ __forceinline__ ItemGeom item_geom(int pos, int window, int ps) {
  ItemGeom g;
  g.lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  g.first_page = g.lo / ps;
  g.k_base = g.first_page * ps;
  g.n_rows = pos - g.k_base;                       // cached rows ahead of the token's own
  g.n_tiles = (g.n_rows + S_TILE - 1) / S_TILE;
  g.n_pages = (g.n_rows + ps - 1) / ps;
  return g;
}

template <int D>
__global__ void __launch_bounds__(S_THREADS)
attention_decode_stream_kernel(const __grid_constant__ CUtensorMap map_kv, const StreamArgs sa) {
  const Args& a = sa.b;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // the 128-byte swizzle is a function of the address: stages start on 1024-byte boundaries
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int DH = D / 64;                // 128-byte column blocks of a row
  constexpr int NT = D / 8;                 // 8-wide output tiles of the head
  constexpr int NT_W = NT / S_WARPS;        // ... of one warp
  constexpr int KS = D / 16;                // 16-deep steps over the head dimension
  constexpr int LPR = D / 8;                // lanes that share the token's own row
  constexpr int HALF_BYTES = S_TILE * 128;               // one column block of a K or V tile
  constexpr int KV_BYTES = DH * HALF_BYTES;              // K (or V) of a stage
  constexpr int STAGE_BYTES = 2 * KV_BYTES;
  const int ps = a.page_size;
  const int tile_pages = S_TILE / ps;
  const int NS = sa.n_stages;
  __shared__ __align__(8) uint64_t full[S_MAX_STAGES];
  __shared__ __align__(8) uint64_t empty[S_MAX_STAGES];
  __shared__ float s_scores[2][S_TILE];     // a stage's scores, written by quarters, read by all
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int H = a.H, G = a.H / a.Hkv;
  pdl_launch_dependents();
  if (tid == 0) {
    for (int s = 0; s < NS; s++) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], S_WARPS);
    }
    s_abort = 0;
    mbar_fence_init();
  }
  __syncthreads();
  volatile int* af = &s_abort;
  auto token_of = [&](int item) { int ti = item / H; return a.token_list ? a.token_list[ti] : ti; };
  // A block's items: one of every run of gridDim.x, counted from the front in even runs and from
  // the back in odd ones.  A caller that lists long tokens first thus gives every block long and
  // short items alike.
  auto after = [&](int item) {
    const int k = item / (int)gridDim.x + 1;
    return k * (int)gridDim.x + ((k & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x);
  };

  if (warp == S_WARPS) {
    // ---- producer: metadata and pages of EARLIER positions only, which the kernel ahead
    // cannot have written, so nothing here waits for it ----
    auto pos_of = [&](int item) { return item < sa.n_items ? a.positions[token_of(item)] : 0; };
    auto load_ids = [&](int item, int pos, int* pid) {
      const int t = token_of(item);
      const int r = a.token_req ? a.token_req[t] : t;
      const ItemGeom g = item_geom(pos, a.window, ps);
      const int* bt = a.block_table + (size_t)r * a.bt_stride + g.first_page;
#pragma unroll
      for (int k = 0; k < S_PMAX; k++) {
        int i = k * 32 + lane;
        pid[k] = i < g.n_pages ? bt[i] : 0;
      }
    };
    int it = 0;
    int item = blockIdx.x;
    int pos_cur = pos_of(item), pos_nxt = pos_of(after(item));
    int pid_cur[S_PMAX], pid_nxt[S_PMAX];
    if (item < sa.n_items) load_ids(item, pos_cur, pid_cur);
    bool ok = true;
    while (item < sa.n_items && ok) {
      const int item_n = after(item);
      if (item_n < sa.n_items) load_ids(item_n, pos_nxt, pid_nxt);
      const int pos_n2 = pos_of(after(item_n));
      const ItemGeom g = item_geom(pos_cur, a.window, ps);
      const int hk = (item % H) / G;
      for (int j = 0; j < g.n_tiles && ok; j++, it++) {
        const int s = it % NS;
        if (it >= NS) {
          int w = 1;
          if (lane == 0) w = mbar_wait(&empty[s], ((it / NS) - 1) & 1, af) ? 1 : 0;
          ok = __shfl_sync(0xffffffffu, w, 0) != 0;
          if (!ok) break;
        }
        const int pg0 = j * tile_pages;
        const int npg = min(tile_pages, g.n_pages - pg0);
        uint8_t* sk = smem + (size_t)s * STAGE_BYTES;
        uint8_t* sv = sk + KV_BYTES;
        if (lane == 0) mbar_expect_tx(&full[s], (uint32_t)npg * 2u * (uint32_t)ps * (uint32_t)D * 2u);
        __syncwarp();
        // the lane that holds a page's id issues its copies: the pages of a stage go out side by side
        const int p = (lane - pg0) & 31;                 // this lane's page within the stage, if < npg
        if (p < npg) {
          const int idx = pg0 + p;
          int page = 0;
#pragma unroll
          for (int k = 0; k < S_PMAX; k++)
            if (k == (idx >> 5)) page = pid_cur[k];
#pragma unroll
          for (int hb = 0; hb < DH; hb++) {
            tma_load_5d(sk + hb * HALF_BYTES + p * ps * 128, &map_kv, &full[s], hb * 64, 0, hk, 0, page);
            tma_load_5d(sv + hb * HALF_BYTES + p * ps * 128, &map_kv, &full[s], hb * 64, 0, hk, 1, page);
          }
        }
      }
      item = item_n;
      pos_cur = pos_nxt;
      pos_nxt = pos_n2;
#pragma unroll
      for (int k = 0; k < S_PMAX; k++) pid_cur[k] = pid_nxt[k];
    }
    if (!ok && lane == 0) {
      // wait, with a limit, for the copies still in flight before the block may exit
      for (int i = max(0, it - NS); i < it; i++) mbar_wait(&full[i % NS], (i / NS) & 1, af);
    }
    return;
  }

  // ---- consumers ----
  const int gq = lane >> 2, tq = lane & 3;          // row group and column pair of the MMA fragments
  const int dl = lane % LPR;
  const float cexp = a.scale * 1.4426950408889634f; // scores in base-2 exponent units
  const size_t page_elems = (size_t)2 * a.Hkv * ps * D;
  const size_t v_off = (size_t)a.Hkv * ps * D;
  const bool fused = a.k_new != nullptr;
  // what an item needs from global memory is requested one item ahead: the position (step
  // metadata, readable at once), and the query as row 0 of the MMA's 16 x 16 operand (lanes
  // 0..3 hold it, the others zeros), which the kernel ahead writes
  int item = blockIdx.x;
  int t_nxt = item < sa.n_items ? token_of(item) : 0;
  int pos_nxt = item < sa.n_items ? a.positions[t_nxt] : 0;
  uint32_t qa_nxt[KS][2];
#pragma unroll
  for (int ks = 0; ks < KS; ks++) qa_nxt[ks][0] = qa_nxt[ks][1] = 0u;
  auto fetch_q = [&](int item_) {
    if (gq == 0) {
      const uint32_t* qp = reinterpret_cast<const uint32_t*>(a.q + (size_t)t_nxt * a.q_stride + (size_t)(item_ % H) * D);
#pragma unroll
      for (int ks = 0; ks < KS; ks++) {
        qa_nxt[ks][0] = qp[8 * ks + tq];
        qa_nxt[ks][1] = qp[8 * ks + 4 + tq];
      }
    }
  };
  pdl_wait();       // queries and the step's own keys and values come from the kernel ahead
  if (item < sa.n_items) fetch_q(item);
  int it = 0;
  for (; item < sa.n_items; item = after(item)) {
    const int t = t_nxt, pos = pos_nxt, h = item % H, hk = h / G;
    uint32_t qa[KS][2];
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
      qa[ks][0] = qa_nxt[ks][0];
      qa[ks][1] = qa_nxt[ks][1];
    }
    // the token's own key and value: every warp scores the key (lanes 0..LPR-1 hold 8 elements
    // of the query and of the key each) and takes the value's elements of its own columns
    const __nv_bfloat16* ksrc;
    const __nv_bfloat16* vsrc;
    int slot = -1;
    if (fused) {
      ksrc = a.k_new + (size_t)t * a.new_stride + (size_t)hk * D;
      vsrc = a.v_new + (size_t)t * a.new_stride + (size_t)hk * D;
      if (warp == 0) slot = a.slots[t];
    } else {
      const int r = a.token_req ? a.token_req[t] : t;
      const int page = a.block_table[(size_t)r * a.bt_stride + pos / ps];
      ksrc = a.cache + (size_t)page * page_elems + (size_t)hk * ps * D + (size_t)(pos % ps) * D;
      vsrc = ksrc + v_off;
    }
    uint4 kn = make_uint4(0u, 0u, 0u, 0u), qrow = kn, vn = kn;
    if (lane < LPR) {
      kn = reinterpret_cast<const uint4*>(ksrc)[dl];
      qrow = reinterpret_cast<const uint4*>(a.q + (size_t)t * a.q_stride + (size_t)h * D)[dl];
      if (warp == 0) vn = reinterpret_cast<const uint4*>(vsrc)[dl];
    }
    uint32_t v_own[NT_W];      // the value's elements 8 (NT_W warp + u) + 2 tq, +1 (lanes 0..3 use them)
#pragma unroll
    for (int u = 0; u < NT_W; u++)
      v_own[u] = reinterpret_cast<const uint32_t*>(vsrc)[4 * (NT_W * warp + u) + tq];
    if (after(item) < sa.n_items) {
      t_nxt = token_of(after(item));
      pos_nxt = a.positions[t_nxt];
      fetch_q(after(item));
    }
    const ItemGeom g = item_geom(pos, a.window, ps);
    float m_run = -INFINITY, l_run = 0.0f;      // l_run: this lane's share of the sum
    float o[NT_W][4];
#pragma unroll
    for (int u = 0; u < NT_W; u++) o[u][0] = o[u][1] = o[u][2] = o[u][3] = 0.0f;
    for (int j = 0; j < g.n_tiles; j++, it++) {
      const int s = it % NS;
      bool ok = !*af && mbar_wait(&full[s], (it / NS) & 1, af);
      ok = __all_sync(0xffffffffu, ok);
      const uint32_t sk = smem_u32(smem + (size_t)s * STAGE_BYTES);
      const uint32_t sv = sk + KV_BYTES;
      const int key0 = g.k_base + j * S_TILE;
      const bool whole = key0 >= g.lo && key0 + S_TILE <= pos;
      float* sc_buf = s_scores[it & 1];
      if (ok) {
        if (!whole && lane < 16) {
          // rows that hold no key of this item may hold anything: their values are zeroed (a
          // zero weight times a non-number would still spoil the sum), their scores masked below
          const int row = 16 * warp + lane, key = key0 + row;
          if (key < g.lo || key >= pos) {
#pragma unroll
            for (int hb = 0; hb < DH; hb++)
#pragma unroll
              for (int c = 0; c < 8; c++)
                asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(sv + hb * HALF_BYTES + row * 128 + c * 16), "r"(0u) : "memory");
          }
        }
        // scores of this warp's 16 keys (two tiles of 8) against row 0
        float sc[2][4];
#pragma unroll
        for (int u = 0; u < 2; u++) sc[u][0] = sc[u][1] = sc[u][2] = sc[u][3] = 0.0f;
        {
          const int mi = lane >> 3, row = lane & 7;
#pragma unroll
          for (int kp = 0; kp < KS; kp += 2) {
            const int c = 2 * kp + mi;                   // 16-byte column of the row
#pragma unroll
            for (int u = 0; u < 2; u++) {
              const int key = 16 * warp + 8 * u + row;
              uint32_t b0, b1, b2, b3;
              ldmatrix_x4(sk + (c >> 3) * HALF_BYTES + key * 128 + (((c & 7) ^ (key & 7)) << 4), b0, b1, b2, b3);
              mma_row0(sc[u], qa[kp][0], qa[kp][1], b0, b1);
              mma_row0(sc[u], qa[kp + 1][0], qa[kp + 1][1], b2, b3);
            }
          }
        }
        if (gq == 0) {
#pragma unroll
          for (int u = 0; u < 2; u++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
              const int i = 16 * warp + 8 * u + 2 * tq + e;
              const int key = key0 + i;
              sc_buf[i] = (whole || (key >= g.lo && key < pos)) ? sc[u][e] * cexp : -INFINITY;
            }
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(S_WARPS * 32) : "memory");     // scores and zeroed rows are there for all
      if (ok) {
        const float s0 = sc_buf[lane], s1 = sc_buf[lane + 32];
        const float m_new = fmaxf(m_run, warp_max(fmaxf(s0, s1)));
        if (m_new > -INFINITY) {
          const float corr = ex2(m_run - m_new);           // 0 at the first keys (m_run = -inf)
          const float p0 = ex2(s0 - m_new), p1 = ex2(s1 - m_new);
          m_run = m_new;
          l_run = l_run * corr + (p0 + p1);
#pragma unroll
          for (int u = 0; u < NT_W; u++) {
            o[u][0] *= corr;
            o[u][1] *= corr;
          }
          // the weights as row 0 of the MMA's 16 x 16 operand, 16 keys a step: this lane needs
          // keys 16 kk + 2 tq + {0, 1, 8, 9}; key i sits in lane i % 32 (p0 for i < 32, else p1)
          uint32_t pa[4][2];
#pragma unroll
          for (int kk = 0; kk < 4; kk++) {
            const float pv = kk < 2 ? p0 : p1;
            const int l0 = (16 * kk) % 32 + 2 * tq;
            const float w0 = __shfl_sync(0xffffffffu, pv, l0), w1 = __shfl_sync(0xffffffffu, pv, l0 + 1);
            const float w2 = __shfl_sync(0xffffffffu, pv, l0 + 8), w3 = __shfl_sync(0xffffffffu, pv, l0 + 9);
            pa[kk][0] = pack_bf16x2(w0, w1);
            pa[kk][1] = pack_bf16x2(w2, w3);
          }
          const int mi = lane >> 3, row = lane & 7;
#pragma unroll
          for (int kk = 0; kk < 4; kk++) {
            const int key = 16 * kk + (mi & 1) * 8 + row;
#pragma unroll
            for (int u = 0; u < NT_W; u += 2) {
              const int c = NT_W * warp + u + (mi >> 1);
              uint32_t b0, b1, b2, b3;
              ldmatrix_x4_trans(sv + (c >> 3) * HALF_BYTES + key * 128 + (((c & 7) ^ (key & 7)) << 4), b0, b1, b2, b3);
              mma_row0(o[u], pa[kk][0], pa[kk][1], b0, b1);
              mma_row0(o[u + 1], pa[kk][0], pa[kk][1], b2, b3);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);       // the stage may be refilled
    }
    // the token's own key and value, and the result
    {
      float fq[8], fk[8];
      bf16x8_to_f32(qrow, fq);
      bf16x8_to_f32(kn, fk);
      float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
      for (int y = 0; y < 8; y += 2) {
        s0 = fmaf(fq[y], fk[y], s0);
        s1 = fmaf(fq[y + 1], fk[y + 1], s1);
      }
      const float s_own = warp_sum(s0 + s1) * cexp;          // lanes beyond the row hold zeros
      const float m_fin = fmaxf(m_run, s_own);
      const float corr = ex2(m_run - m_fin), pw = ex2(s_own - m_fin);
      const float l_fin = warp_sum(l_run) * corr + pw;
      if (gq == 0 && !*af) {
        const float inv = 1.0f / l_fin;
        __nv_bfloat16* op = a.out + (size_t)t * a.o_stride + (size_t)h * D;
#pragma unroll
        for (int u = 0; u < NT_W; u++) {
          const __nv_bfloat162 vv = *reinterpret_cast<const __nv_bfloat162*>(&v_own[u]);
          const float2 vf = __bfloat1622float2(vv);
          const float y0 = (o[u][0] * corr + pw * vf.x) * inv, y1 = (o[u][1] * corr + pw * vf.y) * inv;
          *reinterpret_cast<uint32_t*>(op + 8 * (NT_W * warp + u) + 2 * tq) = pack_bf16x2(y0, y1);
        }
      }
      if (warp == 0 && lane < LPR && fused && slot >= 0 && h % G == 0) {
        __nv_bfloat16* kdst = a.cache + (size_t)(slot / ps) * page_elems + (size_t)hk * ps * D + (size_t)(slot % ps) * D;
        reinterpret_cast<uint4*>(kdst)[dl] = kn;
        reinterpret_cast<uint4*>(kdst + v_off)[dl] = vn;
      }
    }
  }
  if (tid == 0 && *af && a.err) atomicExch(a.err, 1);
}

template <int D>
int launch(const CUtensorMap& mkv, const Args& a, int T, cudaStream_t stream) {
  size_t smem = (size_t)2 * a.rows_cap * D * 2 +
                ((size_t)D + (size_t)WARPS * 256 + (size_t)a.rows_cap + (size_t)a.nb_max + (size_t)8 * (D + 2)) * 4;
  if (smem > 200 * 1024) return SGLC_ERR_UNSUPPORTED;
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_tma_kernel<D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cudaFuncSetAttribute(attention_decode_tma_kernel<D>, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    configured = smem;
  }
  dim3 grid(T, a.H, a.n_splits);
  return sglc_launch(attention_decode_tma_kernel<D>, grid, dim3(THREADS), smem, stream, a.n_splits, true, mkv, a);
}
}  // namespace

// Whether this kernel takes the case (else: the register-staged kernel of attention_decode.cu).
SGLC_API int sglc_attention_decode_tma_supports(int D, int page_size, int n_splits) {
  return (D == 64 || D == 128) && page_size >= 1 && page_size <= 256 && n_splits >= 1 && n_splits <= 8;
}

// Arguments as sglc_attention_decode (without the global-memory scratch); n_pages: pages of
// the cache tensor; token_list: optional list of the T tokens to serve.
SGLC_API int sglc_attention_decode_tma(const void* q, int q_stride, void* cache, const int* block_table,
                                       int bt_stride, const int* token_req, const int* positions,
                                       void* out, int o_stride, int T, int H, int Hkv, int D,
                                       int page_size, float scale, int window, int max_keys,
                                       int n_splits, const void* k_new, const void* v_new,
                                       int new_stride, const int* slots, int* err,
                                       const int* token_list, int n_pages, cudaStream_t stream) {
  if (T <= 0) return SGLC_OK;
  if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || page_size <= 0 || max_keys <= 0 || n_pages <= 0)
    return SGLC_ERR_ARGUMENT;
  if (!sglc_attention_decode_tma_supports(D, page_size, n_splits) || H > 65535) return SGLC_ERR_UNSUPPORTED;
  if (q_stride % 8 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)cache & 15)) return SGLC_ERR_UNSUPPORTED;
  if (k_new && (!v_new || !slots || new_stride % 8 != 0 || ((uintptr_t)k_new & 15) || ((uintptr_t)v_new & 15)))
    return SGLC_ERR_UNSUPPORTED;
  if ((page_size * D * 2) % 128 != 0) return SGLC_ERR_UNSUPPORTED;   // page blocks stay 128-byte aligned in shared memory
  CUtensorMap mkv;
  if (!get_kv_map(&mkv, cache, D, page_size, Hkv, n_pages)) return SGLC_ERR_UNSUPPORTED;
  Args a;
  a.q = (const __nv_bfloat16*)q; a.q_stride = q_stride;
  a.cache = (__nv_bfloat16*)cache;
  a.block_table = block_table; a.bt_stride = bt_stride;
  a.token_req = token_req; a.positions = positions; a.token_list = token_list;
  a.out = (__nv_bfloat16*)out; a.o_stride = o_stride;
  a.H = H; a.Hkv = Hkv; a.page_size = page_size;
  a.scale = scale; a.window = window;
  a.n_splits = n_splits;
  int eff = window > 0 && window < max_keys ? window : max_keys;
  a.chunk_cap = (eff + n_splits - 1) / n_splits;
  // whole pages are staged: the range may start and end inside a page
  a.rows_cap = ((a.chunk_cap + page_size - 1) / page_size + 1) * page_size;
  a.nb_max = (max_keys + page_size - 1) / page_size;
  if (a.nb_max > bt_stride) a.nb_max = bt_stride;
  a.k_new = (const __nv_bfloat16*)k_new; a.v_new = (const __nv_bfloat16*)v_new;
  a.new_stride = new_stride; a.slots = slots;
  a.err = err;
  if (D == 64) return launch<64>(mkv, a, T, stream);
  return launch<128>(mkv, a, T, stream);
}

// Whether the streaming kernel takes the case: head sizes 64 and 128, pages of 8, 16, 32 or 64
// positions (a stage holds 64 keys in whole pages, each page box on a 1024-byte boundary), and
// at most 256 pages per item.
SGLC_API int sglc_attention_decode_stream_supports(int D, int page_size, int max_keys, int window) {
  if (!(D == 64 || D == 128)) return 0;
  if (!(page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64)) return 0;
  int eff = window > 0 && window < max_keys ? window : max_keys;
  if ((eff + page_size - 1) / page_size + 1 > 32 * S_PMAX) return 0;
  return 1;
}

// Same arguments and result as sglc_attention_decode_tma (n_splits has no meaning here: a block
// walks whole (token, head) items).  Meant for many items; any number is served.
SGLC_API int sglc_attention_decode_stream(const void* q, int q_stride, void* cache, const int* block_table,
                                          int bt_stride, const int* token_req, const int* positions,
                                          void* out, int o_stride, int T, int H, int Hkv, int D,
                                          int page_size, float scale, int window, int max_keys,
                                          const void* k_new, const void* v_new, int new_stride,
                                          const int* slots, int* err, const int* token_list,
                                          int n_pages, cudaStream_t stream) {
  if (T <= 0) return SGLC_OK;
  if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || page_size <= 0 || max_keys <= 0 || n_pages <= 0)
    return SGLC_ERR_ARGUMENT;
  if (!sglc_attention_decode_stream_supports(D, page_size, max_keys, window)) return SGLC_ERR_UNSUPPORTED;
  if (q_stride % 8 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)cache & 15)) return SGLC_ERR_UNSUPPORTED;
  if (k_new && (!v_new || !slots || new_stride % 8 != 0 || ((uintptr_t)k_new & 15) || ((uintptr_t)v_new & 15)))
    return SGLC_ERR_UNSUPPORTED;
  if ((page_size * D * 2) % 128 != 0) return SGLC_ERR_UNSUPPORTED;
  if ((long long)T * H > 0x7fffffffLL) return SGLC_ERR_UNSUPPORTED;
  CUtensorMap mkv;
  if (!get_kv_map(&mkv, cache, D, page_size, Hkv, n_pages, true)) return SGLC_ERR_UNSUPPORTED;
  StreamArgs sa;
  memset(&sa, 0, sizeof(sa));
  Args& a = sa.b;
  a.q = (const __nv_bfloat16*)q; a.q_stride = q_stride;
  a.cache = (__nv_bfloat16*)cache;
  a.block_table = block_table; a.bt_stride = bt_stride;
  a.token_req = token_req; a.positions = positions; a.token_list = token_list;
  a.out = (__nv_bfloat16*)out; a.o_stride = o_stride;
  a.H = H; a.Hkv = Hkv; a.page_size = page_size;
  a.scale = scale; a.window = window;
  a.n_splits = 1;
  a.k_new = (const __nv_bfloat16*)k_new; a.v_new = (const __nv_bfloat16*)v_new;
  a.new_stride = new_stride; a.slots = slots;
  a.err = err;
  sa.n_items = T * H;
  const size_t stage_bytes = (size_t)2 * S_TILE * D * 2;   // 64 keys and 64 values
  // three blocks per SM (two at head size 128), and as many stages as then fit, three at least
  int n_stages = (int)(((size_t)72 * 1024 - 1024) / stage_bytes);
  if (n_stages > S_MAX_STAGES) n_stages = S_MAX_STAGES;
  if (n_stages < 3) n_stages = 3;
  sa.n_stages = n_stages;
  const size_t smem = (size_t)n_stages * stage_bytes + 1024;
  if (smem > 200 * 1024) return SGLC_ERR_UNSUPPORTED;
  static int n_sm = 0;
  if (n_sm == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0) n_sm = 148;
  }
  int per_sm = (int)((220 * 1024) / (smem + 2048));
  if (per_sm > 3) per_sm = 3;
  if (per_sm < 1) per_sm = 1;
  int grid = n_sm * per_sm;
  if (grid > sa.n_items) grid = sa.n_items;
  auto kern = D == 64 ? attention_decode_stream_kernel<64> : attention_decode_stream_kernel<128>;
  static size_t configured[2] = {0, 0};
  size_t& conf = configured[D == 64 ? 0 : 1];
  if (smem > 48 * 1024 && smem > conf) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    conf = smem;
  }
  return sglc_launch(kern, dim3(grid), dim3(S_THREADS), smem, stream, 1, true, mkv, sa);
}
