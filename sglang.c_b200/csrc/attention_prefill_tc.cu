// Causal attention of prompt portions over the paged bfloat16 cache on the tensor cores.
// One block per (request, head, tile of 128 queries).  For every tile of 128 keys that the
// queries may see:  S = Q·K^T (tcgen05.mma into tensor memory), then the eight softmax warps
// (16 query rows a warp, a row spread over a quad of threads as in the accumulator of the
// warp-level MMA) read S, apply the scale, the causal bound and the window, keep the running
// maximum and sum of an online softmax in 32-bit, write P = exp(S - max) as bfloat16 to shared
// memory, O_tile = P·V (second MMA, V taken as it lies in the cache: keys by rows), and the
// threads fold O_tile into their rows' output with the usual rescaling.  Keys and values come
// page by page through the block table (one TMA box per page, or 16-byte cp.async where the
// page size does not divide 128, into the 128-byte swizzle the MMA expects).  Lengths,
// positions and block tables are read on the device.
// The reference's prefill attention for this architecture is k_attn (scores of a whole row in
// shared memory, src/cuda_backend.cu:1600-1651); its tiled form for other architectures is
// k_attn_flash (:1838-1960, CUDA cores, warp-shuffle online softmax).
// Head sizes: 64 and 128 here (other sizes run on the plain kernel of attention_simt.cu).
#include <string.h>

#include <mutex>
#include <utility>
#include <vector>

#include "common.cuh"
#include "tc_common.cuh"

SGLC_DEFINE_ERROR_STRING()

namespace {
using namespace tc;

constexpr int BQ = 128;          // queries per block = MMA M = TMEM lanes
constexpr int BKV = 128;         // keys per tile = MMA N of S
constexpr int SOFTMAX_THREADS = 256;
constexpr int MMA_WARP = SOFTMAX_THREADS / 32;
constexpr int THREADS = SOFTMAX_THREADS + 128;     // warps 0-7 softmax, warp 8 MMA + TMEM, warps 9-11 loaders
constexpr int N_LOADERS = 96;
constexpr int KV_STAGES = 2;


struct Ctl {
  uint64_t q_full, s_full, p_ready, o_full;
  uint64_t land_free, land_full;       // the hand-over between the two blocks of a split tile
  uint64_t kv_full[KV_STAGES], kv_empty[KV_STAGES];
  uint32_t tmem_base;
  int abort_flag;
};

struct Args {
  const __nv_bfloat16* q;
  int q_stride;
  const __nv_bfloat16* cache;
  const int* block_table;
  int bt_stride;
  const int* q_start;     // [R+1] first token of each request in this step
  const int* kv_len;      // [R] length of each request after this step
  __nv_bfloat16* out;
  int o_stride;
  int H, Hkv, page_size;
  float scale_log2;       // scale * log2(e)
  int window;
  int use_tma;            // keys, values and queries arrive by TMA (page_size divides 128)
  int skip_single;        // requests that bring one token are served by the decode kernel
  int split_min;          // key tiles from which a query tile is shared by the cluster's two blocks
  int* err;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  int n = valid ? 16 : 0;     // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// 2^x by the special-function unit (inputs here are <= 0 up to rounding; -inf gives 0)
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// byte offset of 16-byte chunk `c` (0..7) of row `r` in a [rows][128 B] tile with the 128-byte swizzle
__device__ __forceinline__ uint32_t sw128(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }

template <int D>
__global__ void __launch_bounds__(THREADS, (D == 64 ? 2 : 1))
attention_prefill_kernel(const __grid_constant__ CUtensorMap map_q,
                         const __grid_constant__ CUtensorMap map_kv, const Args a) {
  constexpr int DB = D / 64;                       // 64-wide blocks of the head dimension
  constexpr int TILE_BYTES = BKV * 128 * DB;       // one K (or V, or Q) tile: [DB][128 rows][128 B]
  constexpr int P_BYTES = BQ * 128 * (BKV / 64);   // P: [2][128 rows][128 B]
  constexpr int TMEM_COLS = 256;                   // S: columns 0..127, O_tile: 128..128+D
  // All shared memory is dynamic and the kernel has no static shared memory, so the tiles
  // start at the block's first byte, which the 128-byte swizzle needs at a multiple of 1024.
  // Without alignment slack two blocks fit on one SM (head size 64).
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sP = sQ + TILE_BYTES;
  uint8_t* sK = sP + P_BYTES;                      // KV_STAGES tiles
  uint8_t* sV = sK + KV_STAGES * TILE_BYTES;       // KV_STAGES tiles
  Ctl& ctl = *reinterpret_cast<Ctl*>(sV + KV_STAGES * TILE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // The launch is a list of clusters of two blocks per (request, head), heaviest first (blocks
  // are handed out x first, then y, so every request's heaviest work starts first).  A query
  // tile with split_min or more key tiles takes a whole cluster: rank 0 walks the first half
  // of the key tiles and rank 1 the rest; each then fetches the other's running maximum and sum
  // and half of its output columns through distributed shared memory and finishes that half.  The lighter query tiles go two to a cluster,
  // the heaviest of them with the lightest (an idle partner would hold its place on the SM
  // until the cluster ends).  Without the split the launch lasts as long as its longest tile
  // (the last query tile of the longest request) while most SMs have long finished.
  const int r = blockIdx.x / a.H, h = blockIdx.x % a.H, rank = blockIdx.z, cl = blockIdx.y;
  pdl_launch_dependents();
  // What follows reads only the step's own arrays (request bounds, block tables), which no
  // kernel of the step writes: the block finds its work, sets up its barriers and tensor memory
  // and clears its stages while the kernel ahead still runs.  The loaders wait for that kernel
  // before they touch queries or cache pages; everything else in the block follows from what
  // they bring.
  const int t0 = a.q_start[r];
  const int q_len = a.q_start[r + 1] - t0;
  if (a.skip_single && q_len == 1) return;
  if (smem_u32(smem) & 1023u) {                    // never seen; the tiles would be mis-swizzled
    if (threadIdx.x == 0 && a.err) atomicExch(a.err, 1);
    return;
  }
  const int kv_len = a.kv_len[r];
  const int nq = (q_len + BQ - 1) / BQ;
  // key tiles of query tile t: from the tile of the first key its first row may see to the tile
  // of its last row's own position
  auto key_tiles = [&](int t, int& first_tile) {
    const int p0 = kv_len - q_len + t * BQ;
    const int lp = p0 + min(BQ, q_len - t * BQ) - 1;
    int fk = 0;
    if (a.window > 0 && p0 - a.window + 1 > 0) fk = p0 - a.window + 1;
    first_tile = fk / BKV;
    return lp / BKV - first_tile + 1;
  };
  int n_split = 0;
  for (int t = 0; t < nq; t++) {
    int ft;
    n_split += key_tiles(t, ft) >= a.split_min ? 1 : 0;
  }
  const bool split = cl < n_split;
  // this block's query tile: the cl-th split tile from the top, or among the others (from the
  // top) number cl - n_split for rank 0 and, from the bottom, the same number for rank 1
  int qt = -1;
  {
    const int n_rest = nq - n_split;
    const int want = split ? cl : (rank == 0 ? cl - n_split : n_rest - 1 - (cl - n_split));
    if (split || (cl - n_split < (n_rest + 1) / 2 && (rank == 0 || want > cl - n_split))) {
      int seen = 0;
      for (int t = nq - 1; t >= 0; t--) {
        int ft;
        const bool sp = key_tiles(t, ft) >= a.split_min;
        if (sp == split) {
          if (seen == want) {
            qt = t;
            break;
          }
          seen++;
        }
      }
    }
  }
  if (qt < 0) return;                              // nothing for this block (its partner knows)
  const int pos0 = kv_len - q_len + qt * BQ;       // position of the tile's first query
  const int rows = min(BQ, q_len - qt * BQ);
  const int last_pos = pos0 + rows - 1;
  int first_key = 0;
  if (a.window > 0 && pos0 - a.window + 1 > 0) first_key = pos0 - a.window + 1;
  int kt_first;
  const int n_all = key_tiles(qt, kt_first);
  // rank 1's half ends with the masked tile at the diagonal, which costs more than a plain one:
  // of an odd number rank 0 takes the larger half
  const int n_mine0 = split ? (n_all + 1) / 2 : n_all;
  const int kt0 = (!split || rank == 0) ? kt_first : kt_first + n_mine0;
  const int n_tiles = (!split || rank == 0) ? n_mine0 : n_all - n_mine0;
  const int hk = h / (a.H / a.Hkv);

  if (threadIdx.x == 0) {
    mbar_init(&ctl.q_full, a.use_tma ? 1 : N_LOADERS);
    mbar_init(&ctl.s_full, 1);
    mbar_init(&ctl.p_ready, SOFTMAX_THREADS);
    mbar_init(&ctl.o_full, 1);
    mbar_init(&ctl.land_free, SOFTMAX_THREADS);
    mbar_init(&ctl.land_full, SOFTMAX_THREADS);
    for (int s = 0; s < KV_STAGES; s++) {
      mbar_init(&ctl.kv_full[s], a.use_tma ? 1 : N_LOADERS);
      mbar_init(&ctl.kv_empty[s], 1);
    }
    ctl.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == MMA_WARP) {
    tmem_alloc(&ctl.tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl.tmem_base;
  volatile int* abort_flag = &ctl.abort_flag;
  if (split) {
    // both blocks' barriers exist before either signals the other's
    cluster_arrive();
    cluster_wait();
  }

  if (warp > MMA_WARP && a.use_tma) {
    // ---- loader by TMA: one box per (page, K or V, 64-wide block of the head) ----
    const int lt = threadIdx.x - (MMA_WARP + 1) * 32;
    // rows of a tile that no page fills (beyond the last key, before the window) must hold
    // finite numbers: zero both stages once; later tiles leave finite data behind
    for (int c = lt; c < (2 * KV_STAGES * TILE_BYTES) / 16; c += N_LOADERS)
      reinterpret_cast<uint4*>(sK)[c] = make_uint4(0u, 0u, 0u, 0u);
    fence_async_proxy();
    asm volatile("bar.sync 2, 96;" ::: "memory");
    if (lt == 0) {
      const int ps = a.page_size;
      const int* bt = a.block_table + (size_t)r * a.bt_stride;
      pdl_wait();
      mbar_expect_tx(&ctl.q_full, DB * BQ * 128);
      for (int blk = 0; blk < DB; blk++)
        tma_load_2d(sQ + blk * (BQ * 128), &map_q, &ctl.q_full, h * D + blk * 64, t0 + qt * BQ);
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; j++) {
        const int s = j % KV_STAGES;
        if (j >= KV_STAGES) ok = mbar_wait(&ctl.kv_empty[s], ((j / KV_STAGES) - 1) & 1, abort_flag);
        if (!ok) break;
        const int key0 = (kt0 + j) * BKV;
        int pg0 = key0 / ps;
        int pg1 = min(last_pos, key0 + BKV - 1) / ps;          // inclusive
        if (pg0 * ps + ps - 1 < first_key) pg0 = first_key / ps;   // pages wholly before the window
        const int npg = pg1 - pg0 + 1;
        mbar_expect_tx(&ctl.kv_full[s], (uint32_t)npg * 2u * DB * (uint32_t)ps * 128u);
        for (int pi = pg0; pi <= pg1; pi++) {
          const int page = bt[pi];
          const uint32_t row_off = (uint32_t)(pi * ps - key0) * 128u;
          for (int blk = 0; blk < DB; blk++) {
            tma_load_5d(sK + s * TILE_BYTES + blk * (BKV * 128) + row_off, &map_kv, &ctl.kv_full[s],
                        blk * 64, 0, hk, 0, page);
            tma_load_5d(sV + s * TILE_BYTES + blk * (BKV * 128) + row_off, &map_kv, &ctl.kv_full[s],
                        blk * 64, 0, hk, 1, page);
          }
        }
      }
    }
  } else if (warp > MMA_WARP) {
    // ---- loaders by cp.async: Q once, then K and V tiles through the block table ----
    const int lt = threadIdx.x - (MMA_WARP + 1) * 32;
    pdl_wait();
    {
      const __nv_bfloat16* qbase = a.q + (size_t)(t0 + qt * BQ) * a.q_stride + (size_t)h * D;
      const uint32_t dst = smem_u32(sQ);
      for (int c = lt; c < BQ * (D / 8); c += N_LOADERS) {
        int row = c / (D / 8), ch = c % (D / 8);
        bool valid = row < rows;
        const void* src = valid ? (const void*)(qbase + (size_t)row * a.q_stride + ch * 8) : (const void*)a.q;
        cp_async16(dst + (ch / 8) * (BQ * 128) + sw128(row, ch % 8), src, valid);
      }
      cp_async_commit();
    }
    const int* bt = a.block_table + (size_t)r * a.bt_stride;
    const size_t page_elems = (size_t)2 * a.Hkv * a.page_size * D;
    const size_t head_off = (size_t)hk * a.page_size * D;
    const size_t v_off = (size_t)a.Hkv * a.page_size * D;
    auto issue_tile = [&](int j) {
      const int s = j % KV_STAGES;
      const int key0 = (kt0 + j) * BKV;
      const uint32_t dk = smem_u32(sK + s * TILE_BYTES), dv = smem_u32(sV + s * TILE_BYTES);
      for (int c = lt; c < BKV * (D / 8); c += N_LOADERS) {
        int row = c / (D / 8), ch = c % (D / 8);
        int key = key0 + row;
        // keys before the window may lie in pages that were given back: never touched
        bool valid = key <= last_pos && key >= first_key;
        const __nv_bfloat16* src = a.cache;
        if (valid) {
          int page = bt[key / a.page_size];
          src = a.cache + (size_t)page * page_elems + head_off + (size_t)(key % a.page_size) * D + ch * 8;
        }
        uint32_t off = (ch / 8) * (BKV * 128) + sw128(row, ch % 8);
        cp_async16(dk + off, src, valid);
        cp_async16(dv + off, valid ? src + v_off : src, valid);
      }
      cp_async_commit();
    };
    // Both stages are free at the start, so tiles 0 and 1 are requested at once.  Afterwards a
    // tile is announced as soon as it has landed and BEFORE this thread waits for a stage to
    // come free: the MMA warp issues the scores of tile j+1 ahead of P.V of tile j, so the
    // stage of tile j is not given back until tile j+1 has been announced.
    static_assert(KV_STAGES == 2, "the loader's order of waits assumes two stages");
    bool ok = true;
    issue_tile(0);
    if (n_tiles > 1) {
      issue_tile(1);
      cp_async_wait<1>();             // all but the newest group: Q and tile 0 have landed
    } else {
      cp_async_wait<0>();
    }
    fence_async_proxy();
    mbar_arrive(&ctl.q_full);
    mbar_arrive(&ctl.kv_full[0]);
    for (int j = 0; j < n_tiles && ok; j++) {
      if (j + 1 < n_tiles) {
        cp_async_wait<0>();           // tile j+1, the only one on its way, has landed
        fence_async_proxy();
        mbar_arrive(&ctl.kv_full[(j + 1) % KV_STAGES]);
      }
      if (j + 2 < n_tiles) {
        ok = mbar_wait(&ctl.kv_empty[j % KV_STAGES], (j / KV_STAGES) & 1, abort_flag);   // P.V of tile j is done
        if (!ok) break;
        issue_tile(j + 2);
      }
    }
    cp_async_wait<0>();
  } else if (warp == MMA_WARP) {
    // ---- MMA issuer ----
    if (elect_one()) {
      constexpr uint32_t idesc_s = idesc_bf16_f32(BQ, BKV, 0, 0);       // Q, K both K-major
      constexpr uint32_t idesc_o = idesc_bf16_f32(BQ, D, 0, 1);         // P K-major, V MN-major
      const uint32_t tS = tmem_base, tO = tmem_base + 128;
      auto issue_s = [&](int s) {
        const uint32_t q0 = smem_u32(sQ), k0 = smem_u32(sK + s * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; k++) {
          uint32_t off = (k / 4) * (BQ * 128) + (k % 4) * 32;
          mma_bf16(tS, smem_desc_k_sw128(q0 + off), smem_desc_k_sw128(k0 + off), idesc_s, k > 0 ? 1u : 0u);
        }
        mma_commit(&ctl.s_full);
      };
      bool ok = mbar_wait(&ctl.q_full, 0, abort_flag) && mbar_wait(&ctl.kv_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        issue_s(0);
      }
      for (int j = 0; j < n_tiles && ok; j++) {
        const int s = j % KV_STAGES;
        ok = mbar_wait(&ctl.p_ready, j & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        // the next tile's scores go ahead of this tile's P.V: the softmax warps find them when
        // they come back from sending P, and this P.V runs under their first pass
        if (j + 1 < n_tiles) {
          ok = mbar_wait(&ctl.kv_full[(j + 1) % KV_STAGES], ((j + 1) / KV_STAGES) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          issue_s((j + 1) % KV_STAGES);
        }
        const uint32_t p0 = smem_u32(sP), v0 = smem_u32(sV + s * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < BKV / 16; k++) {
          uint64_t dp = smem_desc_k_sw128(p0 + (k / 4) * (BQ * 128) + (k % 4) * 32);
          // V: 16 keys = 16 rows of 128 bytes further; blocks of 64 head elements BKV*128 bytes apart
          uint64_t dv = smem_desc_mn_sw128(v0 + k * 2048, BKV * 128, 1024);
          mma_bf16(tO, dp, dv, idesc_o, k > 0 ? 1u : 0u);
        }
        mma_commit(&ctl.o_full);
        mma_commit(&ctl.kv_empty[s]);
      }
    }
  } else {
    // ---- softmax and output: eight warps; a warp has 16 query rows, a quad of threads a row ----
    // (the accumulators come out of tensor memory in the layout of the warp-level MMA's
    // accumulator: a thread holds two rows, g and g + 8, and of every 8 columns the pair 2q, 2q+1;
    // a row's maximum and sum are reduced over its quad by shuffles)
    const int q4 = lane & 3;
    const int lane0 = (warp & 3) * 32 + (warp >> 2) * 16;        // the warp's first lane of tensor memory
    const int row_r[2] = {lane0 + (lane >> 2), lane0 + (lane >> 2) + 8};
    const bool valid_r[2] = {row_r[0] < rows, row_r[1] < rows};
    const int pos_r[2] = {pos0 + row_r[0], pos0 + row_r[1]};
    int lo_r[2];
#pragma unroll
    for (int x = 0; x < 2; x++) lo_r[x] = (a.window > 0 && pos_r[x] - a.window + 1 > 0) ? pos_r[x] - a.window + 1 : 0;
    const uint32_t tS = tmem_base + ((uint32_t)lane0 << 16);
    const uint32_t tO = tS + 128;
    const int st = threadIdx.x;                                 // 0..SOFTMAX_THREADS-1
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};   // l: this thread's share of the row sums
    // output: for every 32 columns 16 registers in the order they are loaded in (index & 2: row g + 8)
    float o[D / 2];
#pragma unroll
    for (int d = 0; d < D / 2; d++) o[d] = 0.0f;
    float alpha[2] = {0.0f, 0.0f};     // of the last tile seen: what its maximum made of the sums before it
    // o = o * alpha + (the tile's P.V, from tensor memory)
    auto fold = [&](const float (&al)[2]) {
#pragma unroll
      for (int c = 0; c < D; c += 32) {
        uint32_t v[16];
        tmem_ld_16x256b_x4(tO + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; i++) o[c / 2 + i] = o[c / 2 + i] * al[(i >> 1) & 1] + __uint_as_float(v[i]);
      }
      tc_fence_before_sync();
    };
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; j++) {
      ok = mbar_wait(&ctl.s_full, j & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      const int key0 = (kt0 + j) * BKV;
      // a tile needs the mask only where it meets the diagonal, the window's edge or the end
      // of the rows; elsewhere every key is visible to every row of the tile
      const bool full_tile = (key0 + BKV - 1 <= pos0) && (rows == BQ) &&
                             (a.window <= 0 || key0 >= pos0 + BQ - a.window);
      // On such a tile row x sees the keys vis_first[x] .. vis_first[x] + vis_span[x], counted
      // from the tile's first key (a row that sees none: a first key beyond every tile).  With
      // rel = key - first, "visible" is one unsigned comparison: rel <= span.
      int rel0[2];                   // rel of this thread's first key of the tile (key 2 q4)
      uint32_t vis_span[2];
#pragma unroll
      for (int x = 0; x < 2; x++) {
        const int first = max(lo_r[x], key0), last = min(pos_r[x], key0 + BKV - 1);
        const bool any = valid_r[x] && last >= first;
        rel0[x] = any ? key0 + 2 * q4 - first : -(1 << 20);
        vis_span[x] = any ? (uint32_t)(last - first) : 0u;
      }
      // pass 1: the rows' maxima over the keys they may see
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll 1
      for (int c = 0; c < BKV; c += 32) {
        uint32_t v[16];
        tmem_ld_16x256b_x4(tS + c, v);
        tmem_ld_wait();
        if (full_tile) {
#pragma unroll
          for (int i = 0; i < 16; i++) mx[(i >> 1) & 1] = fmaxf(mx[(i >> 1) & 1], __uint_as_float(v[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 16; i++) {
            const int x = (i >> 1) & 1;
            const bool vis = (uint32_t)(rel0[x] + c + 8 * (i >> 2) + (i & 1)) <= vis_span[x];
            mx[x] = fmaxf(mx[x], vis ? __uint_as_float(v[i]) : -INFINITY);
          }
        }
      }
      if (j > 0) {
        // the tile before: its P.V ran under this pass; fold it in (its P may then be overwritten)
        ok = mbar_wait(&ctl.o_full, (j - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        fold(alpha);
      }
      float neg_m[2];
#pragma unroll
      for (int x = 0; x < 2; x++) {
        mx[x] = fmaxf(mx[x], __shfl_xor_sync(0xffffffffu, mx[x], 1));
        mx[x] = fmaxf(mx[x], __shfl_xor_sync(0xffffffffu, mx[x], 2));
        const float m_new = fmaxf(m[x], mx[x]);
        const float m_use = m_new == -INFINITY ? 0.0f : m_new;     // a row with no key yet
        alpha[x] = exp2f((m[x] - m_use) * a.scale_log2);           // m = -inf gives 0
        neg_m[x] = -m_use * a.scale_log2;
        m[x] = m_new;
      }
      // pass 2: p = exp(s - max) = 2^(s*c - max*c) as bfloat16 into shared memory, and the row sums
      float sum[2] = {0.0f, 0.0f};
#pragma unroll 1
      for (int c = 0; c < BKV; c += 32) {
        uint32_t v[16];
        tmem_ld_16x256b_x4(tS + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int b = 0; b < 4; b++) {
#pragma unroll
          for (int x = 0; x < 2; x++) {
            float p0 = ex2_approx(fmaf(__uint_as_float(v[4 * b + 2 * x]), a.scale_log2, neg_m[x]));
            float p1 = ex2_approx(fmaf(__uint_as_float(v[4 * b + 2 * x + 1]), a.scale_log2, neg_m[x]));
            if (!full_tile) {
              const uint32_t rel = (uint32_t)(rel0[x] + c + 8 * b);
              if (rel > vis_span[x]) p0 = 0.0f;
              if (rel + 1u > vis_span[x]) p1 = 0.0f;
            }
            sum[x] += p0 + p1;
            __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
            // keys c + 8b .. +7 are one 16-byte chunk of the row; this thread's pair is its q4-th word
            *reinterpret_cast<uint32_t*>(sP + (c / 64) * (BQ * 128) + sw128(row_r[x], (c % 64) / 8 + b) + 4 * q4) =
                *reinterpret_cast<uint32_t*>(&hh);
          }
        }
      }
#pragma unroll
      for (int x = 0; x < 2; x++) l[x] = l[x] * alpha[x] + sum[x];
      tc_fence_before_sync();       // the loads of S are done before the next S may be written
      fence_async_proxy();          // P is visible to the tensor core
      mbar_arrive(&ctl.p_ready);
    }
    if (ok && n_tiles > 0) {
      ok = mbar_wait(&ctl.o_full, (n_tiles - 1) & 1, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        fold(alpha);
      }
    }
    // A shared tile is finished by both blocks, each for half of the head's columns: a block
    // leaves its (maximum, sum) and the other half's output registers in its own K/V stages
    // (free once its last MMA is done, which its threads have waited for), tells its partner and
    // fetches the partner's through distributed shared memory.  The two blocks' threads hold the
    // same rows and columns in the same registers, so thread t's registers cross as 16-byte
    // pieces [piece][t]: piece 0 = (max, sum) of its two rows, then output registers by fours.
    constexpr int HP = D / 16;                       // pieces (8-column blocks) of half a head
    const int keep0 = (split && rank == 1) ? HP : 0; // first 8-column block this block finishes
    const int n_keep = split ? HP : D / 8;
    if (split) {
      float4* land = reinterpret_cast<float4*>(sK);
      const int give0 = HP - keep0;
      land[st] = make_float4(m[0], ok ? l[0] : 0.0f, m[1], ok ? l[1] : 0.0f);
#pragma unroll
      for (int c = 0; c < HP; c++) {
        // (constant register indices: both halves are written out, one is stored)
        const float4 lo4 = make_float4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
        const float4 hi4 = make_float4(o[4 * (HP + c)], o[4 * (HP + c) + 1], o[4 * (HP + c) + 2], o[4 * (HP + c) + 3]);
        land[(c + 1) * SOFTMAX_THREADS + st] = give0 == 0 ? lo4 : hi4;
      }
      mbar_arrive_peer(map_to_peer(&ctl.land_full, (uint32_t)(rank ^ 1)));
      const bool there = mbar_wait_cluster(&ctl.land_full, 0, abort_flag);
      if (there) {
        const uint32_t src = map_to_peer(land, (uint32_t)(rank ^ 1)) + (uint32_t)st * 16u;
        const uint4 ml = ld_peer_v4(src);
        uint4 v[HP];
#pragma unroll
        for (int c = 0; c < HP; c++) v[c] = ld_peer_v4(src + (uint32_t)(c + 1) * (SOFTMAX_THREADS * 16u));
        const float m2[2] = {__uint_as_float(ml.x), __uint_as_float(ml.z)};
        const float l2[2] = {__uint_as_float(ml.y), __uint_as_float(ml.w)};
        float a1[2], a2[2];
#pragma unroll
        for (int x = 0; x < 2; x++) {
          const float mm = fmaxf(m[x], m2[x]);
          const float m_use = mm == -INFINITY ? 0.0f : mm;
          a1[x] = exp2f((m[x] - m_use) * a.scale_log2);
          a2[x] = exp2f((m2[x] - m_use) * a.scale_log2);
          l[x] = l[x] * a1[x] + l2[x] * a2[x];
        }
#pragma unroll
        for (int c = 0; c < HP; c++) {
          // the kept half, again with constant register indices
#pragma unroll
          for (int half = 0; half < 2; half++) {
            if (half * HP != keep0) continue;
            const int b = 4 * (half * HP + c);
            o[b] = o[b] * a1[0] + __uint_as_float(v[c].x) * a2[0];
            o[b + 1] = o[b + 1] * a1[0] + __uint_as_float(v[c].y) * a2[0];
            o[b + 2] = o[b + 2] * a1[1] + __uint_as_float(v[c].z) * a2[1];
            o[b + 3] = o[b + 3] * a1[1] + __uint_as_float(v[c].w) * a2[1];
          }
        }
      } else {
        ok = false;
      }
      mbar_arrive_peer(map_to_peer(&ctl.land_free, (uint32_t)(rank ^ 1)));    // read (or given up)
    }
#pragma unroll
    for (int x = 0; x < 2; x++) {
      l[x] += __shfl_xor_sync(0xffffffffu, l[x], 1);
      l[x] += __shfl_xor_sync(0xffffffffu, l[x], 2);
    }
    if (ok) {
#pragma unroll
      for (int x = 0; x < 2; x++) {
        if (!valid_r[x]) continue;
        const float inv = 1.0f / l[x];
        __nv_bfloat16* op = a.out + (size_t)(t0 + qt * BQ + row_r[x]) * a.o_stride + (size_t)h * D + 2 * q4;
#pragma unroll
        for (int i = 0; i < D / 8; i++) {          // the row's i-th block of 8 columns
          if (i < keep0 || i >= keep0 + n_keep) continue;
          __nv_bfloat162 hh = __floats2bfloat162_rn(o[4 * i + 2 * x] * inv, o[4 * i + 2 * x + 1] * inv);
          *reinterpret_cast<__nv_bfloat162*>(op + 8 * i) = hh;
        }
      }
    }
    // the partner reads this block's shared memory: stay until it has
    if (split) mbar_wait_cluster(&ctl.land_free, 0, abort_flag);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && ctl.abort_flag && a.err) atomicExch(a.err, 1);
  if (warp == MMA_WARP) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- host: tensor maps, kept per (pointer, shape) ----
struct KeyQ { const void* p; uint64_t rows, cols, ld; };
struct KeyKV { const void* p; int D, ps, Hkv, n_pages; };
std::mutex g_mutex;
std::vector<std::pair<KeyQ, CUtensorMap>> g_qmaps;
std::vector<std::pair<KeyKV, CUtensorMap>> g_kvmaps;

bool get_q_map(CUtensorMap* out, const void* q, uint64_t rows, uint64_t cols, uint64_t ld) {
  std::lock_guard<std::mutex> lock(g_mutex);
  for (auto& e : g_qmaps)
    if (e.first.p == q && e.first.rows == rows && e.first.cols == cols && e.first.ld == ld) {
      *out = e.second;
      return true;
    }
  CUtensorMap m;
  if (!make_map_bf16_2d(&m, q, rows, cols, ld, BQ)) return false;
  if (g_qmaps.size() > 256) g_qmaps.clear();
  g_qmaps.push_back({KeyQ{q, rows, cols, ld}, m});
  *out = m;
  return true;
}

// One layer's pages [n_pages][2][Hkv][page_size][D] as a 5-D tensor, boxes of one page's rows of
// one head, 64 elements (128 bytes) wide, in the 128-byte swizzle.
bool get_kv_map(CUtensorMap* out, const void* cache, int D, int ps, int Hkv, int n_pages) {
  std::lock_guard<std::mutex> lock(g_mutex);
  for (auto& e : g_kvmaps)
    if (e.first.p == cache && e.first.D == D && e.first.ps == ps && e.first.Hkv == Hkv &&
        e.first.n_pages == n_pages) {
      *out = e.second;
      return true;
    }
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn || ((uintptr_t)cache & 15) || ps > 256) return false;
  cuuint64_t dims[5] = {(cuuint64_t)D, (cuuint64_t)ps, (cuuint64_t)Hkv, 2, (cuuint64_t)n_pages};
  cuuint64_t strides[4] = {(cuuint64_t)D * 2, (cuuint64_t)ps * D * 2, (cuuint64_t)Hkv * ps * D * 2,
                           (cuuint64_t)2 * Hkv * ps * D * 2};
  cuuint32_t box[5] = {64, (cuuint32_t)ps, 1, 1, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUtensorMap m;
  CUresult rc = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(cache), dims, strides, box,
                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return false;
  if (g_kvmaps.size() > 1024) g_kvmaps.clear();
  g_kvmaps.push_back({KeyKV{cache, D, ps, Hkv, n_pages}, m});
  *out = m;
  return true;
}

template <int D>
int launch(const CUtensorMap& mq, const CUtensorMap& mkv, const Args& a, int R, int max_q_len,
           cudaStream_t stream) {
  constexpr int DB = D / 64;
  size_t smem = (size_t)BQ * 128 * DB + (size_t)BQ * 128 * 2 + (size_t)2 * KV_STAGES * BKV * 128 * DB + 256;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cudaFuncSetAttribute(attention_prefill_kernel<D>, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    configured = true;
  }
  dim3 grid(a.H * R, (max_q_len + BQ - 1) / BQ, 2);      // two blocks (one cluster) per query tile
  return sglc_launch(attention_prefill_kernel<D>, grid, dim3(THREADS), smem, stream, 2, true, mq, mkv, a);
}
}  // namespace


// Tuning hook: key tiles from which a query tile is split over two blocks (default 5).
static int g_split_min = 5;
SGLC_API void sglc_attention_prefill_set_split_min(int n) { g_split_min = n < 2 ? 2 : n; }

// Head sizes this kernel takes.
SGLC_API int sglc_attention_prefill_tc_supports(int D) { return D == 64 || D == 128; }

// q, out: bfloat16 [T][stride], heads side by side, tokens of request r at q_start[r]..q_start[r+1];
// cache: one layer's pages [n_pages][2][Hkv][page_size][D]; kv_len[r]: the request's length after
// this step (its last query sits at kv_len-1); max_q_len: the longest portion (sizes the grid).
// T: rows of q; n_pages: pages of the cache tensor.
SGLC_API int sglc_attention_prefill_tc(const void* q, int q_stride, const void* cache,
                                       const int* block_table, int bt_stride, const int* q_start,
                                       const int* kv_len, void* out, int o_stride, int R,
                                       int max_q_len, int H, int Hkv, int D, int page_size,
                                       float scale, int window, int T, int n_pages, int skip_single,
                                       int* err, cudaStream_t stream) {
  if (R <= 0 || max_q_len <= 0) return SGLC_OK;
  if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || page_size <= 0) return SGLC_ERR_ARGUMENT;
  if (!(D == 64 || D == 128) || H > 65535 || R > 32767 || max_q_len > 65535 * BQ || !(scale > 0.0f)) return SGLC_ERR_UNSUPPORTED;
  if (q_stride % 8 != 0 || o_stride % 8 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)out & 15) ||
      ((uintptr_t)cache & 15))
    return SGLC_ERR_UNSUPPORTED;
  Args a;
  a.q = (const __nv_bfloat16*)q; a.q_stride = q_stride;
  a.cache = (const __nv_bfloat16*)cache;
  a.block_table = block_table; a.bt_stride = bt_stride;
  a.q_start = q_start; a.kv_len = kv_len;
  a.out = (__nv_bfloat16*)out; a.o_stride = o_stride;
  a.H = H; a.Hkv = Hkv; a.page_size = page_size;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.window = window;
  a.err = err;
  a.skip_single = skip_single;
  a.split_min = g_split_min;
  // TMA needs whole pages inside a 128-key tile and rows it can address
  CUtensorMap mq, mkv;
  memset(&mq, 0, sizeof(mq));
  memset(&mkv, 0, sizeof(mkv));
  a.use_tma = 0;
  if (BKV % page_size == 0 && T > 0 && n_pages > 0) {
    bool ok = get_q_map(&mq, q, (uint64_t)T, (uint64_t)H * D, (uint64_t)q_stride) &&
              get_kv_map(&mkv, cache, D, page_size, Hkv, n_pages);
    a.use_tma = ok ? 1 : 0;
  }
  if (D == 64) return launch<64>(mq, mkv, a, R, max_q_len, stream);
  return launch<128>(mq, mkv, a, R, max_q_len, stream);
}
