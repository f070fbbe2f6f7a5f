// bfloat16 GEMM on the 5th-generation tensor cores:
//   C[M,N] = A[M,K] · W[N,K]^T (+ bias[N]) with an optional GELU, stored as bfloat16 or float,
//   or added into the 32-bit residual stream in place.
// Operands arrive in shared memory by TMA (128-byte swizzle, K-major), one elected thread
// issues tcgen05.mma with float accumulators in tensor memory, and four warps read the
// accumulators back with tcgen05.ld for the fused epilogue.  The reference reaches the
// tensor cores only through cuBLAS (gemm_nt_cublas, src/cuda_backend.cu:2843-2903) and adds
// bias, GELU and the residual with separate kernels (k_fill_bias :2642, k_gelu :527,
// k_residual :2405); its small-M products are one-block-per-output GEMVs (:333-349,412-427).
//
// Three kernels, chosen by gemm_tc_run:
//   gemm_tc_stream_kernel   many tokens (prefill): 128 tokens x BN output features a tile, one
//                           resident block per SM walking its tiles with two accumulators
//   gemm_tc_pair_kernel     many tokens and enough columns: a cluster of two blocks on a tile of
//                           256 tokens x 256 features (cta_group::2), half the operand bytes per flop
//   gemm_tc_kernel          few tokens (decode): W on the MMA's 128-row side ("P"), the tokens as
//                           its N operand ("Q", padded to a tile of BN),
//                           with the K range split across the blocks of a thread-block
//                           cluster so that many SMs stream weights.  Each block leaves its
//                           float partial sums in its own shared memory; after a cluster
//                           barrier every block sums a slice of the tile's rows over all
//                           blocks through distributed shared memory, in split order (a
//                           fixed order: the result does not depend on timing), and runs the
//                           epilogue for that slice.
// Sizes: K a multiple of 8 and 16-byte aligned rows (TMA's rule); M, N anything (edges are
// zero-filled on load and masked on store).
#include <string.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tc_common.cuh"

SGLC_DEFINE_ERROR_STRING()

namespace {
using namespace tc;

constexpr int BM = 128;   // rows of P per tile = MMA M = TMEM lanes
constexpr int BK = 64;    // K per stage: 128 bytes of bfloat16, one swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;   // warp 0: TMA, warp 1: MMA + TMEM, warps 2-5: epilogue
constexpr int MAX_STAGES = 8;
constexpr int PAIR_THREADS = 64 + 256;   // the two-SM kernel: warp 0 TMA, warp 1 MMA, two groups of four epilogue warps
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

struct GemmArgs {
  int M, N, K;             // logical sizes
  int P_rows, Q_rows;      // rows of the two operands as mapped (P: 128-row operand)
  int swap;                // 0: P = A (tokens), Q = W (features); 1: P = W, Q = A
  int kb_total;            // K blocks of 64
  int kb_per_split;        // K blocks per split (grid.z splits)
  int splits;
  int stages;
  const float* bias;       // [N] or null
  void* out;               // [M][ldo], bfloat16 or float
  float* residual;         // float [M][ldo], updated in place (then `out` is unused)
  int ldo;
  int out_f32;             // out is float
  int tma_out;             // many-token tiles leave through shared memory and a TMA store / add
  int act;
  int* err;                // set to 1 if a bounded wait ran out
  int tiles_p, n_tiles;    // many-token kernel: row tiles, and all tiles (a block walks several)
};

// The many-token kernel's KV form: the output columns from q_cols on are keys and values of the
// step's tokens ([keys of `heads` heads of `dim`][values likewise]) and go straight into the paged
// cache [page][2][heads][page][dim] at slots[token] instead of into `out`.  (Its own structure and
// its own instantiation of the kernel: the other kernels of this file are compiled as they were
// without it; their register allocation, and with it their speed, moved when these fields were
// part of GemmArgs.)
struct KvArgs {
  void* cache;
  const int* slots;
  int q_cols, heads, dim, page, n_pages;
};

struct SharedCtl {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t accum;
  uint32_t tmem_base;
  int abort_flag;
};

template <int BN>
__device__ __forceinline__ void epilogue_store(const GemmArgs& a, int p_glob, int q0, const float* v,
                                               int nq) {
  // v[j]: value at (p_glob, q0 + j), already reduced over K; applies bias, activation, store.
  if (a.swap) {
    int n = p_glob;
    if (n >= a.N) return;
    float b = a.bias ? a.bias[n] : 0.0f;
#pragma unroll
    for (int j = 0; j < nq; j++) {
      int m = q0 + j;
      if (m >= a.M) break;
      float x = act_tc(v[j] + b, a.act);
      size_t o = (size_t)m * a.ldo + n;
      if (a.residual) a.residual[o] += x;
      else if (a.out_f32) ((float*)a.out)[o] = x;
      else ((__nv_bfloat16*)a.out)[o] = __float2bfloat16_rn(x);
    }
  } else {
    int m = p_glob;
    if (m >= a.M) return;
    size_t row = (size_t)m * a.ldo;
    bool vec_ok = (q0 + nq <= a.N);
    if (a.residual) {
      float* dst = a.residual + row + q0;
      if (vec_ok && ((uintptr_t)dst & 15) == 0 && nq % 4 == 0) {
#pragma unroll
        for (int j = 0; j < nq; j += 4) {
          float4 r = *reinterpret_cast<float4*>(dst + j);
          r.x += v[j] + (a.bias ? a.bias[q0 + j] : 0.0f);
          r.y += v[j + 1] + (a.bias ? a.bias[q0 + j + 1] : 0.0f);
          r.z += v[j + 2] + (a.bias ? a.bias[q0 + j + 2] : 0.0f);
          r.w += v[j + 3] + (a.bias ? a.bias[q0 + j + 3] : 0.0f);
          *reinterpret_cast<float4*>(dst + j) = r;
        }
      } else {
        for (int j = 0; j < nq && q0 + j < a.N; j++)
          dst[j] += v[j] + (a.bias ? a.bias[q0 + j] : 0.0f);
      }
    } else if (a.out_f32) {
      float* dst = (float*)a.out + row + q0;
      for (int j = 0; j < nq && q0 + j < a.N; j++)
        dst[j] = act_tc(v[j] + (a.bias ? a.bias[q0 + j] : 0.0f), a.act);
    } else {
      __nv_bfloat16* dst = (__nv_bfloat16*)a.out + row + q0;
      if (vec_ok && ((uintptr_t)dst & 15) == 0 && nq % 8 == 0) {
#pragma unroll
        for (int j = 0; j < nq; j += 8) {
          __align__(16) __nv_bfloat162 h[4];
#pragma unroll
          for (int t = 0; t < 4; t++) {
            float x0 = act_tc(v[j + 2 * t] + (a.bias ? a.bias[q0 + j + 2 * t] : 0.0f), a.act);
            float x1 =
                act_tc(v[j + 2 * t + 1] + (a.bias ? a.bias[q0 + j + 2 * t + 1] : 0.0f), a.act);
            h[t] = __floats2bfloat162_rn(x0, x1);
          }
          *reinterpret_cast<uint4*>(dst + j) = *reinterpret_cast<uint4*>(h);
        }
      } else {
        for (int j = 0; j < nq && q0 + j < a.N; j++)
          dst[j] = __float2bfloat16_rn(act_tc(v[j] + (a.bias ? a.bias[q0 + j] : 0.0f), a.act));
      }
    }
  }
}

template <int BN>
__global__ void __launch_bounds__(THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
               const __grid_constant__ CUtensorMap map_out, const GemmArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // stage buffers need 1024-byte alignment for the 128-byte swizzle
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int P_BYTES = BM * BK * 2;
  constexpr int Q_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = P_BYTES + Q_BYTES;
  constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
  __shared__ SharedCtl ctl;
  __shared__ float s_bias[BN];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pt = blockIdx.x, qt = blockIdx.y, split = blockIdx.z;
  const int kb0 = split * a.kb_per_split;
  const int kb1 = min(a.kb_total, kb0 + a.kb_per_split);
  const int n_kb = kb1 - kb0;
  const int stages = a.stages;

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; s++) {
      mbar_init(&ctl.full[s], 1);
      mbar_init(&ctl.empty[s], 1);
    }
    mbar_init(&ctl.accum, 1);
    ctl.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&map_p);
    tma_prefetch_desc(&map_q);
  }
  if (warp == 1) {
    tmem_alloc(&ctl.tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl.tmem_base;
  volatile int* abort_flag = &ctl.abort_flag;
  // split-K partial sums arrive here from the other blocks of the cluster at any time, so the
  // area is apart from the stage buffers (which this block's MMAs may still be reading)
  float* red_buf = reinterpret_cast<float*>(smem + (size_t)stages * STAGE_BYTES);

  if (warp == 0) {
    // ---- TMA producer ----
    if (elect_one()) {
      int issued = 0;
      // Weights never change during a step, so with weights on the P side their first tiles
      // are requested before waiting for the kernel that produces the activations.
      const int n_first = min(n_kb, stages);
      if (a.swap) {
        for (int i = 0; i < n_first; i++) {
          mbar_expect_tx(&ctl.full[i], STAGE_BYTES);
          tma_load_2d(smem + (size_t)i * STAGE_BYTES, &map_p, &ctl.full[i], (kb0 + i) * BK, pt * BM);
        }
        pdl_wait();
        for (int i = 0; i < n_first; i++)
          tma_load_2d(smem + (size_t)i * STAGE_BYTES + P_BYTES, &map_q, &ctl.full[i], (kb0 + i) * BK,
                      qt * BN);
        issued = n_first;
      } else {
        pdl_wait();
      }
      for (int i = issued; i < n_kb; i++) {
        int s = i % stages;
        if (i >= stages && !mbar_wait(&ctl.empty[s], ((i / stages) - 1) & 1, abort_flag)) break;
        uint8_t* sp = smem + (size_t)s * STAGE_BYTES;
        mbar_expect_tx(&ctl.full[s], STAGE_BYTES);
        tma_load_2d(sp, &map_p, &ctl.full[s], (kb0 + i) * BK, pt * BM);
        tma_load_2d(sp + P_BYTES, &map_q, &ctl.full[s], (kb0 + i) * BK, qt * BN);
        issued = i + 1;
      }
      if (*abort_flag) {
        // wait, with a limit, for the copies still in flight before the block may exit
        for (int i = max(0, issued - stages); i < issued; i++)
          mbar_wait(&ctl.full[i % stages], (i / stages) & 1, abort_flag);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (elect_one()) {
      constexpr uint32_t idesc = idesc_bf16_f32(BM, BN);
      bool ok = true;
      for (int i = 0; i < n_kb && ok; i++) {
        int s = i % stages;
        ok = mbar_wait(&ctl.full[s], (i / stages) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        uint32_t sp = smem_u32(smem + (size_t)s * STAGE_BYTES);
        uint64_t dp = smem_desc_k_sw128(sp);
        uint64_t dq = smem_desc_k_sw128(sp + P_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; k++) {
          // 16 bfloat16 = 32 bytes further along K inside the swizzled row: +2 in 16-byte units
          mma_bf16(tmem_base, dp + 2 * k, dq + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
        }
        mma_commit(&ctl.empty[s]);    // the stage is free once these MMAs have read it
      }
      if (ok) mma_commit(&ctl.accum);   // accumulator complete
    }
  } else {
    // ---- epilogue: warps 2..5 own TMEM lanes 32*(warp%4) .. +31 ----
    const int lane_base = (warp & 3) * 32;
    const int p_glob = pt * BM + lane_base + lane;
    // split-K: this block finishes rows [row0, row0 + n_rows) of the tile; thread e takes the
    // elements e, e + 128, ... of that slice (rows fastest).  Bias and residual of the first
    // four are fetched now, while the weights stream in.
    const int e = threadIdx.x - 64;
    const int rows_per = (BM + a.splits - 1) / a.splits;
    const int row0 = split * rows_per;
    const int n_rows = min(rows_per, BM - row0);
    constexpr int BNP = BN + 4;            // padded row of partial sums (bank spread, 16-byte aligned)
    const int total4 = (a.splits > 1 && n_rows > 0) ? n_rows * (BN / 4) : 0;   // (row, 4 columns) items
    float bs0[4], rs0[4];
    size_t off0[4];
    bool valid0[4];
    auto element = [&](int lr, int col, size_t& off, int& n) {
      int pg = pt * BM + row0 + lr, qg = qt * BN + col;
      int m = a.swap ? qg : pg;
      n = a.swap ? pg : qg;
      off = (size_t)m * a.ldo + n;
      return m < a.M && n < a.N;
    };
    if (a.splits > 1) {
      pdl_wait();              // the residual stream is written by the kernels ahead
      const bool has = e < total4;
      const int lr = has ? e % n_rows : 0, col = has ? (e / n_rows) * 4 : 0;
#pragma unroll
      for (int u = 0; u < 4; u++) {
        int n;
        valid0[u] = element(lr, col + u, off0[u], n) && has;
        bs0[u] = (valid0[u] && a.bias) ? a.bias[n] : 0.0f;
        rs0[u] = (valid0[u] && a.residual) ? a.residual[off0[u]] : 0.0f;
      }
    }
    bool ok = n_kb > 0 ? mbar_wait(&ctl.accum, 0, abort_flag) : true;
    tc_fence_after_sync();
    const uint32_t taddr = tmem_base + ((uint32_t)lane_base << 16);
    constexpr int CH = BN < 32 ? 16 : 32;
    if (ok && a.tma_out) {
      // Many tokens: the tile leaves through shared memory (the stage buffers, free now that
      // every MMA has read them) in the 128-byte swizzle and one thread hands it to the TMA
      // engine: a store for bfloat16 output, an add into the float residual stream otherwise.
      // The engine writes whole lines and drops what lies outside the matrix.
      if constexpr (BN >= 64) {
        if (e < BN) s_bias[e] = (a.bias && qt * BN + e < a.N) ? a.bias[qt * BN + e] : 0.0f;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int row = lane_base + lane;
        const bool to_f32 = a.residual != nullptr;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c, r);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] = act_tc(__uint_as_float(r[j]) + s_bias[c + j], a.act);
          if (to_f32) {
            // box = 32 floats (128 bytes) per row: this chunk is row `row` of box c/32
            uint8_t* box = smem + (size_t)(c / 32) * (BM * 128);
#pragma unroll
            for (int ch = 0; ch < 8; ch++)
              *reinterpret_cast<float4*>(box + row * 128 + ((ch ^ (row & 7)) << 4)) =
                  make_float4(v[4 * ch], v[4 * ch + 1], v[4 * ch + 2], v[4 * ch + 3]);
          } else {
            // box = 64 bfloat16 (128 bytes) per row: this chunk is half a row of box c/64
            uint8_t* box = smem + (size_t)(c / 64) * (BM * 128);
#pragma unroll
            for (int q4 = 0; q4 < 4; q4++) {
              int ch = (c % 64) / 8 + q4;
              __align__(16) __nv_bfloat162 hh[4];
#pragma unroll
              for (int x = 0; x < 4; x++) hh[x] = __floats2bfloat162_rn(v[8 * q4 + 2 * x], v[8 * q4 + 2 * x + 1]);
              *reinterpret_cast<uint4*>(box + row * 128 + ((ch ^ (row & 7)) << 4)) = *reinterpret_cast<uint4*>(hh);
            }
          }
        }
        fence_async_proxy();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) {
          if (to_f32) {
            for (int b = 0; b < BN / 32; b++)
              tma_reduce_add_2d(&map_out, smem + (size_t)b * (BM * 128), qt * BN + b * 32, pt * BM);
          } else {
            for (int b = 0; b < BN / 64; b++)
              tma_store_2d(&map_out, smem + (size_t)b * (BM * 128), qt * BN + b * 64, pt * BM);
          }
          tma_store_commit();
          tma_store_wait_read();
        }
      }
    } else if (ok && a.splits == 1) {
#pragma unroll 1
      for (int c = 0; c < BN; c += CH) {
        float v[CH];
        if (n_kb > 0) {
          if constexpr (CH == 32) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + c, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]);
          } else {
            uint32_t r[16];
            tmem_ld_32x16(taddr + c, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; j++) v[j] = __uint_as_float(r[j]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < CH; j++) v[j] = 0.0f;
        }
        epilogue_store<BN>(a, p_glob, qt * BN + c, v, CH);
      }
    } else if (ok) {
      // split-K: the tile's 128 rows are dealt out to the cluster's blocks; every block sends
      // each row of its partial sums to the shared memory of the block that owns the row,
      // as [split][column][row of the owner's slice] floats
      const int prow = lane_base + lane;
      const int owner = prow / rows_per, lr_mine = prow % rows_per;
      const float* slot0 = red_buf + ((size_t)split * rows_per + lr_mine) * BNP;
      const uint32_t remote = map_to_peer(slot0, (uint32_t)owner);
#pragma unroll 1
      for (int c = 0; c < BN; c += CH) {
        uint32_t r[CH];
        if (n_kb > 0) {
          if constexpr (CH == 32) tmem_ld_32x32(taddr + c, (uint32_t(&)[32])r);
          else tmem_ld_32x16(taddr + c, (uint32_t(&)[16])r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < CH; j++) r[j] = 0u;
        }
#pragma unroll
        for (int j = 0; j < CH; j += 4)
          st_peer_v4(remote + (uint32_t)(c + j) * 4u, r[j], r[j + 1], r[j + 2], r[j + 3]);
      }
    }
    if (a.splits > 1) {
      // one cluster barrier: every block's partial sums are where they are summed.  Nothing
      // remote is touched afterwards, so a block may exit as soon as it is done.
      __syncwarp();
      cluster_arrive();
      cluster_wait();
      ok = ok && !ctl.abort_flag;
      if (ok) {
        const float* buf = red_buf;
        // a thread sums four consecutive columns of one row at a time (16-byte reads of every
        // split's partial sums, added in split order); round 0's bias and residual were fetched above
        for (int base = e; base < total4; base += 128) {
          int lr = base % n_rows, col = (base / n_rows) * 4;
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int s2 = 0; s2 < a.splits; s2++) {
            float4 t4 = *reinterpret_cast<const float4*>(buf + ((size_t)s2 * rows_per + lr) * BNP + col);
            acc.x += t4.x; acc.y += t4.y; acc.z += t4.z; acc.w += t4.w;
          }
          float v[4] = {acc.x, acc.y, acc.z, acc.w};
          float bs[4], rs[4];
          size_t off[4];
          bool valid[4];
#pragma unroll
          for (int u = 0; u < 4; u++) {
            int n;
            valid[u] = element(lr, col + u, off[u], n);
            if (base == e) {
              bs[u] = bs0[u];
              rs[u] = rs0[u];
            } else {
              bs[u] = (valid[u] && a.bias) ? a.bias[n] : 0.0f;
              rs[u] = (valid[u] && a.residual) ? a.residual[off[u]] : 0.0f;
            }
          }
#pragma unroll
          for (int u = 0; u < 4; u++) {
            if (!valid[u]) continue;
            float x = act_tc(v[u] + bs[u], a.act);
            if (a.residual) a.residual[off[u]] = rs[u] + x;
            else if (a.out_f32) ((float*)a.out)[off[u]] = x;
            else ((__nv_bfloat16*)a.out)[off[u]] = __float2bfloat16_rn(x);
          }
        }
      }
    }
  }
  if (a.splits > 1 && warp < 2) {
    __syncwarp();
    cluster_arrive();        // the producer and MMA warps take part in the cluster barrier too
    cluster_wait();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && ctl.abort_flag && a.err) atomicExch(a.err, 1);
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- many tokens (prefill): one resident block per SM walks the tiles ----------------------
// At this model's widths a product is one to three 128 x 128 tiles per SM, and a tile's start
// (first operands 1 us after the block begins) and end (2 us of reading the accumulator, bias,
// activation and the way out through shared memory) weigh as much as its main loop.  Here a
// block stays and takes tile after tile: the operand ring never drains between tiles, and with
// two accumulators in tensor memory the four epilogue warps finish tile i while the MMA warp
// already works on tile i+1.  The tile leaves in boxes of 128 bytes a row through a ring of two
// 16 KB buffers (TMA store for bfloat16, TMA add into the float residual stream).
struct StreamCtl {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

template <int BN, bool KV>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_stream_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                      const __grid_constant__ CUtensorMap map_out, const GemmArgs a, const KvArgs kv) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int A_BYTES = BM * BK * 2;
  constexpr int W_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + W_BYTES;
  constexpr int BOX_BYTES = BM * 128;            // one outgoing box: 128 rows of 128 bytes
  __shared__ StreamCtl ctl;
  __shared__ float s_bias[2][BN];
  __shared__ int s_go[2];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = a.stages;
  uint8_t* epi = smem + (size_t)stages * STAGE_BYTES;       // two boxes

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; s++) {
      mbar_init(&ctl.full[s], 1);
      mbar_init(&ctl.empty[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(&ctl.acc_full[b], 1);
      mbar_init(&ctl.acc_empty[b], 4);           // one arrival per epilogue warp
    }
    ctl.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_w);
    if (a.tma_out) tma_prefetch_desc(&map_out);
  }
  if (warp == 1) {
    tmem_alloc(&ctl.tmem_base, 2 * BN);          // two accumulators side by side
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl.tmem_base;
  volatile int* abort_flag = &ctl.abort_flag;
  const int n_kb = a.kb_total;

  if (warp == 0) {
    // ---- TMA producer: one ring of stages across all of the block's tiles ----
    if (elect_one()) {
      // the weights do not come from the kernel ahead: the first tile's weight halves of the
      // ring's stages are asked for before the dependency wait, the token halves after it
      const int pre = n_kb < stages ? n_kb : stages;
      if (blockIdx.x < a.n_tiles) {
        const int qt = blockIdx.x / a.tiles_p;
        for (int i = 0; i < pre; i++) {
          mbar_expect_tx(&ctl.full[i], STAGE_BYTES);
          tma_load_2d(smem + (size_t)i * STAGE_BYTES + A_BYTES, &map_w, &ctl.full[i], i * BK, qt * BN);
        }
      }
      pdl_wait();
      int kc = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < a.n_tiles && ok; t += gridDim.x) {
        const int pt = t % a.tiles_p, qt = t / a.tiles_p;
        for (int i = 0; i < n_kb; i++, kc++) {
          const int s = kc % stages;
          if (kc >= stages && !mbar_wait(&ctl.empty[s], ((kc / stages) - 1) & 1, abort_flag)) {
            ok = false;
            break;
          }
          uint8_t* sp = smem + (size_t)s * STAGE_BYTES;
          if (kc < pre) {
            tma_load_2d(sp, &map_a, &ctl.full[s], i * BK, pt * BM);
            continue;
          }
          mbar_expect_tx(&ctl.full[s], STAGE_BYTES);
          tma_load_2d(sp, &map_a, &ctl.full[s], i * BK, pt * BM);
          tma_load_2d(sp + A_BYTES, &map_w, &ctl.full[s], i * BK, qt * BN);
        }
      }
      if (*abort_flag) {
        // wait, with a limit, for the copies still in flight before the block may exit
        for (int i = max(0, kc - stages); i < kc; i++)
          mbar_wait(&ctl.full[i % stages], (i / stages) & 1, abort_flag);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (elect_one()) {
      constexpr uint32_t idesc = idesc_bf16_f32(BM, BN);
      int kc = 0, n = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < a.n_tiles && ok; t += gridDim.x, n++) {
        const int buf = n & 1;
        if (n >= 2) {
          // the epilogue has read this accumulator's last tile out of tensor memory
          ok = mbar_wait(&ctl.acc_empty[buf], ((n >> 1) - 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
        }
        const uint32_t acc = tmem_base + (uint32_t)(buf * BN);
        for (int i = 0; i < n_kb; i++, kc++) {
          const int s = kc % stages;
          ok = mbar_wait(&ctl.full[s], (kc / stages) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t sp = smem_u32(smem + (size_t)s * STAGE_BYTES);
          const uint64_t da = smem_desc_k_sw128(sp);
          const uint64_t dw = smem_desc_k_sw128(sp + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; k++)
            mma_bf16(acc, da + 2 * k, dw + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
          mma_commit(&ctl.empty[s]);
        }
        if (ok) mma_commit(&ctl.acc_full[buf]);
      }
    }
  } else {
    // ---- epilogue: warps 2..5 own TMEM lanes 32*(warp%4) .. +31 ----
    const int e = threadIdx.x - 64;
    const int lane_base = (warp & 3) * 32;
    const int row = lane_base + lane;
    const bool to_f32 = a.residual != nullptr;
    const int box_cols = to_f32 ? 32 : 64;
    int n = 0, boxes = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < a.n_tiles; t += gridDim.x, n++) {
      const int pt = t % a.tiles_p, qt = t / a.tiles_p;
      const int buf = n & 1;
      float* bias_s = s_bias[buf];
      if (e < BN) bias_s[e] = (a.bias && qt * BN + e < a.N) ? a.bias[qt * BN + e] : 0.0f;
      if (ok) ok = mbar_wait(&ctl.acc_full[buf], (n >> 1) & 1, abort_flag);
      tc_fence_after_sync();
      // one thread decides for all whether the tile is finished or given up (a wait ran out
      // somewhere in the block): the barriers below need every thread on the same side
      if (threadIdx.x == 64) s_go[buf] = (ok && *abort_flag == 0) ? 1 : 0;
      asm volatile("bar.sync 1, 128;" ::: "memory");          // the bias row is there for all
      ok = s_go[buf] != 0;
      const uint32_t taddr = tmem_base + ((uint32_t)lane_base << 16) + (uint32_t)(buf * BN);
      if (ok && a.tma_out) {
        // where this row's keys and values go (one of the step's own arrays names the slot)
        size_t page = 0, off = 0;
        bool live = false;
        if (KV && qt * BN + BN > kv.q_cols) {
          const int tok = pt * BM + row;
          const int slot = tok < a.M ? kv.slots[tok] : -1;
          live = slot >= 0 && sglc_index_ok(slot / kv.page, kv.n_pages, a.err);
          if (live) {
            page = (size_t)(slot / kv.page);
            off = (size_t)(slot % kv.page);
          }
        }
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c, r);
          tmem_ld_wait();
          if (c + 32 >= BN) {
            // the accumulator has been read: the MMA warp may fill it again
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl.acc_empty[buf]);
          }
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] = act_tc(__uint_as_float(r[j]) + bias_s[c + j], a.act);
          if (KV && qt * BN + c >= kv.q_cols) {
            // 32 columns of keys or values (they lie within one head): 64 bytes of this token's
            // row in its page, straight from the registers
            if (!live || qt * BN + c >= a.N) continue;
            const int kv_width = kv.heads * kv.dim, cc = qt * BN + c - kv.q_cols;
            const int which = cc / kv_width, rem = cc - which * kv_width, head = rem / kv.dim, d = rem - head * kv.dim;
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(kv.cache) +
                                 (((page * 2 + which) * kv.heads + head) * kv.page + off) * kv.dim + d;
#pragma unroll
            for (int q4 = 0; q4 < 4; q4++) {
              __align__(16) __nv_bfloat162 hh[4];
#pragma unroll
              for (int x = 0; x < 4; x++) hh[x] = __floats2bfloat162_rn(v[8 * q4 + 2 * x], v[8 * q4 + 2 * x + 1]);
              *reinterpret_cast<uint4*>(dst + 8 * q4) = *reinterpret_cast<uint4*>(hh);
            }
            continue;
          }
          const bool first_of_box = (c % box_cols) == 0;
          uint8_t* box = epi + (size_t)(boxes & 1) * BOX_BYTES;
          if (first_of_box) {
            // the store that used this buffer two boxes ago has read it
            if (threadIdx.x == 64) tma_store_wait_read_but_one();
            asm volatile("bar.sync 1, 128;" ::: "memory");
          }
          if (to_f32) {
#pragma unroll
            for (int ch = 0; ch < 8; ch++)
              *reinterpret_cast<float4*>(box + row * 128 + ((ch ^ (row & 7)) << 4)) =
                  make_float4(v[4 * ch], v[4 * ch + 1], v[4 * ch + 2], v[4 * ch + 3]);
          } else {
#pragma unroll
            for (int q4 = 0; q4 < 4; q4++) {
              const int ch = (c % 64) / 8 + q4;
              __align__(16) __nv_bfloat162 hh[4];
#pragma unroll
              for (int x = 0; x < 4; x++) hh[x] = __floats2bfloat162_rn(v[8 * q4 + 2 * x], v[8 * q4 + 2 * x + 1]);
              *reinterpret_cast<uint4*>(box + row * 128 + ((ch ^ (row & 7)) << 4)) = *reinterpret_cast<uint4*>(hh);
            }
          }
          const bool last_of_box = ((c + 32) % box_cols) == 0;
          if (last_of_box) {
            fence_async_proxy();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (threadIdx.x == 64) {
              const int x0 = qt * BN + (c + 32 - box_cols);
              if (to_f32) tma_reduce_add_2d(&map_out, box, x0, pt * BM);
              else tma_store_2d(&map_out, box, x0, pt * BM);
              tma_store_commit();
            }
            boxes++;
          }
        }
      } else if (ok) {
        // output rows that a tensor map cannot address: plain stores
        const int p_glob = pt * BM + row;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c, r);
          tmem_ld_wait();
          if (c + 32 >= BN) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl.acc_empty[buf]);
          }
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]);
          epilogue_store<BN>(a, p_glob, qt * BN + c, v, 32);
        }
      }
    }
    if (threadIdx.x == 64) tma_store_wait_read();      // shared memory must outlive the last stores' reads
  }
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && ctl.abort_flag && a.err) atomicExch(a.err, 1);
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ---- many tokens, two SMs on one tile (cta_group::2) ------------------------------------------
// A block of the kernel above takes in 32 KB of operands per K block of its 128 x 128 tile, and an
// SM's way in from L2, not the tensor pipe, sets its pace.  Here a cluster of two blocks works on
// one tile of 256 rows by BN columns: each block loads its own 128 rows of A and its half of the
// BN rows of W, the even block issues MMAs that read both halves, and each block's 128 rows of
// the result land in its own tensor memory.  At BN = 256 a block brings in the same 32 KB per K
// block for twice the arithmetic; at BN = 128 24 KB for the same.  Barriers: the even block's
// full[s] counts the bytes of both blocks' loads; empty[s] and acc_full[b] of each block get an
// arrival from the even block's commits (the commit's multicast); the even block's acc_empty[b]
// gets one from each epilogue warp of both blocks.  Otherwise the kernel above: one ring across
// all of a pair's tiles, two accumulators, the same epilogues.
template <int BN, bool KV>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_out, const GemmArgs a, const KvArgs kv) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int A_BYTES = BM * BK * 2;
  constexpr int W_BYTES = (BN / 2) * BK * 2;     // this block's half of the tile's W rows
  constexpr int STAGE_BYTES = A_BYTES + W_BYTES;
  constexpr int BOX_BYTES = BM * 128;
  constexpr int TMEM_COLS = 2 * BN;              // 256 or 512
  static_assert(BN == 128 || BN == 256, "tensor memory is allocated in powers of two");
  // a block has 128 x BN results a tile to see off, twice the single-block kernel's: two groups
  // of four epilogue warps (a warp reads the 32 lanes of tensor memory that its number modulo 4
  // names), each with half of the columns, a box of its own and its own named barrier
  constexpr int GC = BN / 2;
  __shared__ StreamCtl ctl;
  __shared__ float s_bias[BN];
  __shared__ int s_go[2];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = blockIdx.x & 1;               // rank in the cluster (a cluster is two neighbours in x)
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int stages = a.stages;
  uint8_t* epi = smem + (size_t)stages * STAGE_BYTES;       // a box for each group of epilogue warps

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; s++) {
      mbar_init(&ctl.full[s], 1);
      mbar_init(&ctl.empty[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(&ctl.acc_full[b], 1);
      mbar_init(&ctl.acc_empty[b], 16);          // one arrival per epilogue warp of both blocks
    }
    ctl.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_w);
    if (a.tma_out) tma_prefetch_desc(&map_out);
  }
  if (warp == 1) {
    tmem_alloc_pair(&ctl.tmem_base, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  // both blocks' barriers exist before either signals the other's
  cluster_arrive();
  cluster_wait();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl.tmem_base;
  volatile int* abort_flag = &ctl.abort_flag;
  const int n_kb = a.kb_total;

  if (warp == 0) {
    // ---- TMA producer (both blocks): own rows of A, own half of W, bytes counted in the even block ----
    if (elect_one()) {
      const int pre = n_kb < stages ? n_kb : stages;
      if (pair < a.n_tiles) {
        const int qt = pair / a.tiles_p;
        for (int i = 0; i < pre; i++) {
          if (rank == 0) mbar_expect_tx(&ctl.full[i], 2 * STAGE_BYTES);
          tma_load_2d_pair(smem + (size_t)i * STAGE_BYTES + A_BYTES, &map_w, map_to_peer(&ctl.full[i], 0), i * BK,
                           qt * BN + rank * (BN / 2));
        }
      }
      pdl_wait();
      int kc = 0;
      bool ok = true;
      for (int t = pair; t < a.n_tiles && ok; t += n_pairs) {
        const int pt = 2 * (t % a.tiles_p) + rank, qt = t / a.tiles_p;
        for (int i = 0; i < n_kb; i++, kc++) {
          const int s = kc % stages;
          if (kc >= stages && !mbar_wait_cluster(&ctl.empty[s], ((kc / stages) - 1) & 1, abort_flag)) {
            ok = false;
            break;
          }
          uint8_t* sp = smem + (size_t)s * STAGE_BYTES;
          const uint32_t bar = map_to_peer(&ctl.full[s], 0);
          if (kc < pre) {
            tma_load_2d_pair(sp, &map_a, bar, i * BK, pt * BM);
            continue;
          }
          if (rank == 0) mbar_expect_tx(&ctl.full[s], 2 * STAGE_BYTES);
          tma_load_2d_pair(sp, &map_a, bar, i * BK, pt * BM);
          tma_load_2d_pair(sp + A_BYTES, &map_w, bar, i * BK, qt * BN + rank * (BN / 2));
        }
      }
      if (*abort_flag && rank == 0) {
        // wait, with a limit, for both blocks' copies still in flight (they are counted here)
        // before the pair may leave
        for (int i = max(0, kc - stages); i < kc; i++)
          mbar_wait_cluster(&ctl.full[i % stages], (i / stages) & 1, abort_flag);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: the even block, for both ----
    if (rank == 0 && elect_one()) {
      constexpr uint32_t idesc = idesc_bf16_f32(2 * BM, BN);
      int kc = 0, n = 0;
      bool ok = true;
      for (int t = pair; t < a.n_tiles && ok; t += n_pairs, n++) {
        const int buf = n & 1;
        if (n >= 2) {
          ok = mbar_wait_cluster(&ctl.acc_empty[buf], ((n >> 1) - 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
        }
        const uint32_t acc = tmem_base + (uint32_t)(buf * BN);
        for (int i = 0; i < n_kb; i++, kc++) {
          const int s = kc % stages;
          ok = mbar_wait_cluster(&ctl.full[s], (kc / stages) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t sp = smem_u32(smem + (size_t)s * STAGE_BYTES);
          const uint64_t da = smem_desc_k_sw128(sp);
          const uint64_t dw = smem_desc_k_sw128(sp + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; k++)
            mma_bf16_pair(acc, da + 2 * k, dw + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
          mma_commit_pair(&ctl.empty[s], 3);
        }
        if (ok) mma_commit_pair(&ctl.acc_full[buf], 3);
      }
    }
  } else {
    // ---- epilogue (both blocks): a warp owns TMEM lanes 32*(warp%4) .. +31 of its block's rows ----
    const int grp = (threadIdx.x - 64) >> 7, e = (threadIdx.x - 64) & 127;
    const bool leader = e == 0;
    const int bar_id = 1 + grp, c_lo = grp * GC;
    const int lane_base = (warp & 3) * 32;
    const int row = lane_base + lane;
    const bool to_f32 = a.residual != nullptr;
    const int box_cols = to_f32 ? 32 : 64;
    uint8_t* box = epi + (size_t)grp * BOX_BYTES;
    int n = 0;
    bool ok = true;
    for (int t = pair; t < a.n_tiles; t += n_pairs, n++) {
      const int pt = 2 * (t % a.tiles_p) + rank, qt = t / a.tiles_p;
      const int buf = n & 1;
      float* bias_s = s_bias;
      named_bar_sync(bar_id, 128);                              // the group is done with the last tile's bias
      if (e < GC) bias_s[c_lo + e] = (a.bias && qt * BN + c_lo + e < a.N) ? a.bias[qt * BN + c_lo + e] : 0.0f;
      if (ok) ok = mbar_wait_cluster(&ctl.acc_full[buf], (n >> 1) & 1, abort_flag);
      tc_fence_after_sync();
      if (leader) s_go[grp] = (ok && *abort_flag == 0) ? 1 : 0;
      named_bar_sync(bar_id, 128);                              // the bias row is there for the group
      ok = s_go[grp] != 0;
      const uint32_t taddr = tmem_base + ((uint32_t)lane_base << 16) + (uint32_t)(buf * BN);
      // the accumulator has been read: the even block's MMA warp may fill it again
      auto release = [&]() {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_peer(map_to_peer(&ctl.acc_empty[buf], 0));
      };
      if (ok && a.tma_out) {
        // where this row's keys and values go (one of the step's own arrays names the slot)
        size_t page = 0, off = 0;
        bool live = false;
        if (KV && qt * BN + BN > kv.q_cols) {
          const int tok = pt * BM + row;
          const int slot = tok < a.M ? kv.slots[tok] : -1;
          live = slot >= 0 && sglc_index_ok(slot / kv.page, kv.n_pages, a.err);
          if (live) {
            page = (size_t)(slot / kv.page);
            off = (size_t)(slot % kv.page);
          }
        }
#pragma unroll 1
        for (int c = c_lo; c < c_lo + GC; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c, r);
          tmem_ld_wait();
          if (c + 32 >= c_lo + GC) release();
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] = act_tc(__uint_as_float(r[j]) + bias_s[c + j], a.act);
          if (KV && qt * BN + c >= kv.q_cols) {
            // 32 columns of keys or values (within one head): 64 bytes of this token's row in its page
            if (!live || qt * BN + c >= a.N) continue;
            const int kv_width = kv.heads * kv.dim, cc = qt * BN + c - kv.q_cols;
            const int which = cc / kv_width, rem = cc - which * kv_width, head = rem / kv.dim, d = rem - head * kv.dim;
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(kv.cache) +
                                 (((page * 2 + which) * kv.heads + head) * kv.page + off) * kv.dim + d;
#pragma unroll
            for (int q4 = 0; q4 < 4; q4++) {
              __align__(16) __nv_bfloat162 hh[4];
#pragma unroll
              for (int x = 0; x < 4; x++) hh[x] = __floats2bfloat162_rn(v[8 * q4 + 2 * x], v[8 * q4 + 2 * x + 1]);
              *reinterpret_cast<uint4*>(dst + 8 * q4) = *reinterpret_cast<uint4*>(hh);
            }
            continue;
          }
          const bool first_of_box = (c % box_cols) == 0;
          if (first_of_box) {
            // the store that used the group's box before has read it (the values of this chunk
            // were computed meanwhile)
            if (leader) tma_store_wait_read();
            named_bar_sync(bar_id, 128);
          }
          if (to_f32) {
#pragma unroll
            for (int ch = 0; ch < 8; ch++)
              *reinterpret_cast<float4*>(box + row * 128 + ((ch ^ (row & 7)) << 4)) =
                  make_float4(v[4 * ch], v[4 * ch + 1], v[4 * ch + 2], v[4 * ch + 3]);
          } else {
#pragma unroll
            for (int q4 = 0; q4 < 4; q4++) {
              const int ch = (c % 64) / 8 + q4;
              __align__(16) __nv_bfloat162 hh[4];
#pragma unroll
              for (int x = 0; x < 4; x++) hh[x] = __floats2bfloat162_rn(v[8 * q4 + 2 * x], v[8 * q4 + 2 * x + 1]);
              *reinterpret_cast<uint4*>(box + row * 128 + ((ch ^ (row & 7)) << 4)) = *reinterpret_cast<uint4*>(hh);
            }
          }
          const bool last_of_box = ((c + 32) % box_cols) == 0;
          if (last_of_box) {
            fence_async_proxy();
            named_bar_sync(bar_id, 128);
            if (leader) {
              const int x0 = qt * BN + (c + 32 - box_cols);
              if (to_f32) tma_reduce_add_2d(&map_out, box, x0, pt * BM);
              else tma_store_2d(&map_out, box, x0, pt * BM);
              tma_store_commit();
            }
          }
        }
      } else if (ok) {
        release();                                   // (the host sends no such product here)
      }
    }
    if (leader) tma_store_wait_read();                 // shared memory must outlive the last stores' reads
  }
  // Neither block leaves, or frees tensor memory, while the other may still signal its barriers,
  // have its shared memory read by an MMA, or read its own accumulators.
  tc_fence_before_sync();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (threadIdx.x == 0 && ctl.abort_flag && a.err) atomicExch(a.err, 1);
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ---- host side ----------------------------------------------------------------
struct MapKey {
  const void* base;
  uint64_t rows, cols, ld;
  uint32_t box_rows;      // bit 16 set: a float map (output); else bfloat16
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = (size_t)k.base;
    h = h * 1315423911u + k.rows;
    h = h * 1315423911u + k.cols;
    h = h * 1315423911u + k.ld;
    h = h * 1315423911u + k.box_rows;
    return h;
  }
};
std::mutex g_map_mutex;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

bool get_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
             uint32_t box_rows) {
  MapKey key{base, rows, cols, ld, box_rows};
  std::lock_guard<std::mutex> lock(g_map_mutex);
  auto it = g_maps.find(key);
  if (it != g_maps.end()) {
    *out = it->second;
    return true;
  }
  CUtensorMap m;
  bool made = (box_rows & 0x10000u) ? make_map_f32_2d(&m, base, rows, cols, ld, box_rows & 0xFFFFu)
                                    : make_map_bf16_2d(&m, base, rows, cols, ld, box_rows);
  if (!made) return false;
  if (g_maps.size() > 4096) g_maps.clear();
  g_maps.emplace(key, m);
  *out = m;
  return true;
}

template <int BN>
int launch(const CUtensorMap& mp, const CUtensorMap& mq, const CUtensorMap& mo, const GemmArgs& a,
           dim3 grid, cudaStream_t stream) {
  size_t smem = (size_t)a.stages * (BM * BK * 2 + BN * BK * 2);
  if (a.splits > 1) smem += (size_t)((BM + a.splits - 1) / a.splits) * a.splits * (BN + 4) * 4;   // partial sums
  smem += 1024;
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    // ask for the largest shared-memory split of the SM, so that two blocks fit side by side
    // (one block's epilogue then overlaps the other's main loop)
    cudaFuncSetAttribute(gemm_tc_kernel<BN>, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    configured = smem;
  }
  if (a.tma_out) {
    // the outgoing tile is staged in the stage buffers: 16 KB per 128-byte-wide box
    size_t need = (size_t)(a.residual ? BN / 32 : BN / 64) * BM * 128 + 1024;
    if (smem < need) smem = need;
  }
  return sglc_launch(gemm_tc_kernel<BN>, grid, dim3(THREADS), smem, stream, a.splits, true, mp, mq, mo, a);
}
template <int BN, bool KV>
int launch_stream(const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mo, GemmArgs a, const KvArgs& kv,
                  cudaStream_t stream) {
  static int n_sm = 0;
  if (n_sm == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0) n_sm = 148;
  }
  const size_t stage_bytes = (size_t)BM * BK * 2 + (size_t)BN * BK * 2;
  int stages = (int)(((size_t)226 * 1024 - 2 * BM * 128 - 2048) / stage_bytes);
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  // (the first call settles how many stages the device grants beside the kernel's static part)
  static int granted = 0;
  if (granted == 0) {
    for (; stages >= 2; stages--) {
      const size_t want = (size_t)stages * stage_bytes + (size_t)2 * BM * 128 + 1024;
      if (cudaFuncSetAttribute(gemm_tc_stream_kernel<BN, KV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)want) ==
          cudaSuccess)
        break;
      cudaGetLastError();
    }
    if (stages < 2) return SGLC_ERR_UNSUPPORTED;
    granted = stages;
  }
  stages = granted;
  a.stages = stages;
  const size_t smem = (size_t)stages * stage_bytes + (size_t)2 * BM * 128 + 1024;
  int grid = a.n_tiles < n_sm ? a.n_tiles : n_sm;
  return sglc_launch(gemm_tc_stream_kernel<BN, KV>, dim3(grid), dim3(THREADS), smem, stream, 1, true, ma, mw, mo, a, kv);
}
// The two-SM kernel: clusters of two blocks, as many as the device holds at once (148 SMs: 74;
// what the first launch learns from the occupancy query replaces the guess).
int g_pairs_at_once = 74;
template <int BN, bool KV>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mo, GemmArgs a, const KvArgs& kv,
                cudaStream_t stream) {
  const size_t stage_bytes = (size_t)BM * BK * 2 + (size_t)(BN / 2) * BK * 2;
  static int granted = 0, max_pairs = 0;
  if (granted == 0) {
    int stages = (int)(((size_t)226 * 1024 - 2 * BM * 128 - 2048) / stage_bytes);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    for (; stages >= 2; stages--) {
      const size_t want = (size_t)stages * stage_bytes + (size_t)2 * BM * 128 + 1024;
      if (cudaFuncSetAttribute(gemm_tc_pair_kernel<BN, KV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)want) ==
          cudaSuccess)
        break;
      cudaGetLastError();
    }
    if (stages < 2) return SGLC_ERR_UNSUPPORTED;
    // how many clusters of two the device runs side by side (an SM without a free neighbour in
    // its group stays empty): the tile walk assumes that all launched pairs are resident
    cudaLaunchConfig_t probe = {};
    probe.gridDim = dim3(2 * 148);
    probe.blockDim = dim3(PAIR_THREADS);
    probe.dynamicSmemBytes = (size_t)stages * stage_bytes + (size_t)2 * BM * 128 + 1024;
    cudaLaunchAttribute pa[1];
    pa[0].id = cudaLaunchAttributeClusterDimension;
    pa[0].val.clusterDim.x = 2; pa[0].val.clusterDim.y = 1; pa[0].val.clusterDim.z = 1;
    probe.attrs = pa;
    probe.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_kernel<BN, KV>, &probe) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      return SGLC_ERR_UNSUPPORTED;
    }
    max_pairs = n;
    g_pairs_at_once = n;
    granted = stages;
  }
  a.stages = granted;
  const int pairs = a.n_tiles < max_pairs ? a.n_tiles : max_pairs;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(PAIR_THREADS);
  cfg.dynamicSmemBytes = (size_t)granted * stage_bytes + (size_t)2 * BM * 128 + 1024;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  attr[n].id = cudaLaunchAttributeClusterDimension;
  attr[n].val.clusterDim.x = 2; attr[n].val.clusterDim.y = 1; attr[n].val.clusterDim.z = 1;
  n++;
  if (g_sglc_pdl) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    n++;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<BN, KV>, ma, mw, mo, a, kv);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}
int pairs_at_once() { return g_pairs_at_once; }
}  // namespace

// Orientation, tile width and K split for a problem size.
// From 65 tokens on, a product over a short K goes to the many-token kernel although its one row
// of tiles is half empty: the few-token orientation would split K over a cluster and pass
// 128 x 128 partial sums, 64 KB a block, through distributed shared memory (measured at 96 and
// 128 tokens: a decode step 15-17 % shorter; at 64 tokens and fewer the split wins or ties).
constexpr int DIRECT_MIN_M = 65, DIRECT_MAX_KB = 32;
static void plan(int M, int N, int K, int* swap, int* bn, int* splits, int* kb_per_split,
                 int* tiles_p, int* tiles_q) {
  int kb_total = (K + BK - 1) / BK;
  if (M <= 128 && !(M >= DIRECT_MIN_M && kb_total <= DIRECT_MAX_KB)) {
    *swap = 1;
    *tiles_p = (N + BM - 1) / BM;
    // enough blocks to put most SMs on the weights, but few enough partial sums that the
    // last block's reduction stays short
    int want = (2 * 148) / (*tiles_p);
    if (want > 8) want = 8;
    if (want < 1) want = 1;
    if (want > kb_total) want = kb_total;
    int per = (kb_total + want - 1) / want;
    *kb_per_split = per;
    *splits = (kb_total + per - 1) / per;
    // The tokens' side of the tile: what a block passes through distributed shared memory for
    // the split-K sum grows with it (a 128 x 64 tile of partial sums is 32 KB a block: 3 us of
    // each product), so more than 16 tokens are dealt to several tiles of 16 or 32 (the weights of
    // the later ones come from L2) as long as all blocks of the product still find room on the
    // SMs at once (two a SM); tiles of 64 are not used at all.  Measured on decode steps of 24
    // to 128 requests: 5 to 13 % shorter at GPT-2 small's widths, about even at medium and XL
    // widths, where the blocks are many already and the rule mostly keeps the wide tiles.
    auto blocks = [&](int b) { return (long long)(*tiles_p) * ((M + b - 1) / b) * (*splits); };
    if (M <= 16) *bn = 16;
    else if (M <= 48) *bn = blocks(16) <= 2 * 148 ? 16 : 32;
    else if (M <= 64) *bn = 32;
    else *bn = blocks(32) <= 2 * 148 ? 32 : 128;
    *tiles_q = (M + *bn - 1) / *bn;
  } else {
    *swap = 0;
    int tiles128 = ((M + BM - 1) / BM) * ((N + 127) / 128);
    // a block of the many-token kernel walks its tiles one after the other: wide tiles (fewer
    // bytes from L2 per flop) as soon as they occupy half of the SMs
    *bn = (tiles128 >= 74 || N <= 64) ? 128 : 64;
    *tiles_p = (M + BM - 1) / BM;
    *tiles_q = (N + *bn - 1) / *bn;
    *splits = 1;
    *kb_per_split = kb_total;
  }
}

// One 128 x 128 tile a block, or 256 x 256 a pair of blocks?  The pair takes in half the bytes
// per flop, but its hand-shakes cost and one round of its tiles leaves fewer SMs busy.
// Measured in replayed graphs at 2,048 tokens (one block -> pair): 6400 columns over K 1600
// 54.6 -> 34.7 us, 1600 columns over K 6400 64.4 -> 39.0 us, 2304 columns over K 768 12.5 ->
// 11.0 us, 3072 columns with GELU over K 768 18.2 -> 17.6 us, but 768 columns over K 768
// 8.1 -> 11.6 us and over K 3072 19.3 -> 22.0 us.  These fit: rounds of tiles x K blocks x
// 0.31 us + 5 us alone, x 0.38 us + 6.4 us in a pair (2 us more with an activation either
// way); the pair is taken where that says a twentieth less (prefill of 2,048 tokens on one
// GPU: GPT-2 small widths 1.060 -> 1.054 ms, medium 2.91 -> 2.72 ms, XL 11.65 -> 8.50 ms).
// (tp x tq: the product's 128 x 128 tiles.)
static bool pair_pays(int M, int N, int K, int act, int tp, int tq) {
  if (M < 2 * BM) return false;
  const int kb_total = (K + BK - 1) / BK;
  const int rows2 = (M + 2 * BM - 1) / (2 * BM), t256 = rows2 * ((N + 255) / 256);
  const int rounds_alone = (tp * tq + 147) / 148, rounds_pair = (t256 + pairs_at_once() - 1) / pairs_at_once();
  const long long alone = (long long)rounds_alone * kb_total * 31 + 500 + (act != SGLC_ACT_NONE ? 200 : 0);
  const long long paired = (long long)rounds_pair * kb_total * 38 + 640 + (act != SGLC_ACT_NONE ? 200 : 0);
  return paired * 100 < alone * 95;
}

// A: bfloat16 [M,K], rows lda elements apart; W: bfloat16 [N,K] contiguous; bias float [N] or
// null; out [M,N] rows ldo apart (bfloat16, or float if out_f32), or residual (float, in place).
// err: device int, set to 1 if a wait ran out.
static int gemm_tc_run(const void* A, const void* W, const float* bias, void* out, float* residual, int M, int N,
                       int K, int lda, int ldo, int out_f32, int act, int* err, const KvArgs* kv,
                       cudaStream_t stream) {
  if (M <= 0 || N <= 0) return SGLC_OK;
  if (K <= 0) return SGLC_ERR_ARGUMENT;
  if (K % 8 != 0 || lda % 8 != 0 || ((uintptr_t)A & 15) || ((uintptr_t)W & 15))
    return SGLC_ERR_UNSUPPORTED;
  int swap, bn, splits, per, tp, tq;
  plan(M, N, K, &swap, &bn, &splits, &per, &tp, &tq);
  GemmArgs a;
  a.M = M; a.N = N; a.K = K;
  a.swap = swap;
  a.kb_total = (K + BK - 1) / BK;
  a.kb_per_split = per;
  a.splits = splits;
  a.bias = bias; a.out = out; a.residual = residual; a.ldo = ldo; a.out_f32 = out_f32; a.act = act;
  a.err = err;
  CUtensorMap mp, mq;
  bool ok;
  if (swap) {
    a.P_rows = N; a.Q_rows = M;
    ok = get_map(&mp, W, N, K, K, BM) && get_map(&mq, A, M, K, lda, bn);
  } else {
    a.P_rows = M; a.Q_rows = N;
    ok = get_map(&mp, A, M, K, lda, BM) && get_map(&mq, W, N, K, K, bn);
  }
  if (!ok) return SGLC_ERR_UNSUPPORTED;
  // many-token tiles leave by TMA when the output rows can be addressed by a tensor map
  CUtensorMap mo;
  memset(&mo, 0, sizeof(mo));
  a.tma_out = 0;
  if (!swap && bn >= 64) {
    if (residual) a.tma_out = get_map(&mo, residual, M, N, ldo, BM | 0x10000u) ? 1 : 0;
    else if (!out_f32) a.tma_out = get_map(&mo, out, M, N, ldo, BM) ? 1 : 0;
  }
  if (kv) {
    // only the many-token kernels scatter: 32-column chunks within a head, the queries' last
    // 64-column box ending where the keys begin
    if (swap || !a.tma_out || kv->dim % 32 != 0 || kv->q_cols % 64 != 0 || N != kv->q_cols + 2 * kv->heads * kv->dim ||
        kv->page <= 0 || ((uintptr_t)kv->cache & 15))
      return SGLC_ERR_UNSUPPORTED;
  }
  if (!swap && bn == 128 && a.tma_out && pair_pays(M, N, K, act, tp, tq)) {
    const int rows2 = (M + 2 * BM - 1) / (2 * BM), t256 = rows2 * ((N + 255) / 256);
    if (get_map(&mq, W, N, K, K, 128)) {
      a.tiles_p = rows2;
      a.n_tiles = t256;
      const KvArgs none = {};
      const int code = kv ? launch_pair<256, true>(mp, mq, mo, a, *kv, stream)
                          : launch_pair<256, false>(mp, mq, mo, a, none, stream);
      if (code != SGLC_ERR_UNSUPPORTED) return code;
    }
  }
  if (!swap) {
    a.tiles_p = tp;
    a.n_tiles = tp * tq;
    const KvArgs none = {};
    if (kv) return bn == 128 ? launch_stream<128, true>(mp, mq, mo, a, *kv, stream) : launch_stream<64, true>(mp, mq, mo, a, *kv, stream);
    return bn == 128 ? launch_stream<128, false>(mp, mq, mo, a, none, stream) : launch_stream<64, false>(mp, mq, mo, a, none, stream);
  }
  int stage_bytes = BM * BK * 2 + bn * BK * 2;
  int budget = swap ? 96 * 1024 : (bn == 128 ? 100 * 1024 : 100 * 1024);
  int stages = budget / stage_bytes;
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  if (stages > per) stages = per;
  // Many tiles and no split (the head over the vocabulary, a few tokens): with a deep ring two
  // blocks share an SM and the tiles take two waves, the second on a part of the SMs; each block
  // is bound by its start-up and the latency of its K blocks, not by bandwidth, so a shallower
  // ring that lets all tiles be resident at once ends sooner.
  if (swap && splits == 1 && tp * tq > 2 * 148) {
    const int per_sm = (tp * tq + 147) / 148;
    const int fit = (int)((224 * 1024 / per_sm - 4096) / stage_bytes);
    if (fit >= 2 && fit < stages) stages = fit;
  }
  if (stages < 1) stages = 1;
  a.stages = stages;
  dim3 grid(tp, tq, splits);
  switch (bn) {
    case 16: return launch<16>(mp, mq, mo, a, grid, stream);
    case 32: return launch<32>(mp, mq, mo, a, grid, stream);
    case 64: return launch<64>(mp, mq, mo, a, grid, stream);
    case 128: return launch<128>(mp, mq, mo, a, grid, stream);
  }
  return SGLC_ERR_ARGUMENT;
}

SGLC_API int sglc_gemm_tc(const void* A, const void* W, const float* bias, void* out,
                          float* residual, int M, int N, int K, int lda, int ldo, int out_f32,
                          int act, int* err, cudaStream_t stream) {
  return gemm_tc_run(A, W, bias, out, residual, M, N, K, lda, ldo, out_f32, act, err, nullptr, stream);
}

// The fused query/key/value projection of a step with prompt portions: out[:, :q_cols] takes the
// queries as sglc_gemm_tc would write them; the columns from q_cols on (keys of `heads` heads of
// `dim`, then values likewise) go straight into the paged cache
// [n_pages][2][heads][page_size][dim] (bfloat16) at slots[token] = page * page_size + offset, and
// not into `out`.  SGLC_ERR_UNSUPPORTED (nothing launched) when the product would not take the
// many-token kernel or the sizes do not fall on its tiles: the caller then projects and writes
// the cache separately.
SGLC_API int sglc_gemm_tc_kv(const void* A, const void* W, const float* bias, void* out, int M, int N, int K, int lda,
                             int ldo, int act, void* cache, const int* slots, int q_cols, int heads, int dim,
                             int page_size, int n_pages, int* err, cudaStream_t stream) {
  if (!cache || !slots || heads <= 0 || dim <= 0) return SGLC_ERR_ARGUMENT;
  const KvArgs kv{cache, slots, q_cols, heads, dim, page_size, n_pages};
  return gemm_tc_run(A, W, bias, out, nullptr, M, N, K, lda, ldo, 0, act, err, &kv, stream);
}

// Which kernel sglc_gemm_tc takes for a product whose output a tensor map can address (rows 16-byte
// aligned; any product of few tokens): 0 the few-token kernel, 1 the many-token kernel with one
// block a tile, 2 the many-token kernel on pairs of SMs.  (Tests ask, so that the sizes they
// choose for a kernel do reach it.)
SGLC_API int sglc_gemm_tc_form(int M, int N, int K, int act) {
  int swap, bn, splits, per, tp, tq;
  plan(M, N, K, &swap, &bn, &splits, &per, &tp, &tq);
  if (swap) return 0;
  return (bn == 128 && pair_pays(M, N, K, act, tp, tq)) ? 2 : 1;
}
