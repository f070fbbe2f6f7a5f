// The host side of a step in C++: walks a model made of the built-in parts (token table with a
// learned position table, LayerNorm, causal attention over the paged cache, GELU MLP, pre-norm
// blocks, final norm and linear head) and launches the step's kernels, one after the other, on
// the caller's stream.  It chooses the kernel for each product and each attention exactly as the
// Python parts do (engine/runtime.py, csrc/ops.py); the kernels and their launchers are the same
// (bound by address at start-up, they live in their own libraries).  What it saves is the host's
// cost per launch: a step that is not a replayed graph (a prompt portion beside decoded tokens,
// a shape seen for the first time) makes about a hundred launches, at some 15 us each from
// Python and 2-3 us from here.
//
// The reference drives its kernels from C as well, one launch per operation
// (gpt2_forward_seg, src/cuda_backend.cu:5752-5826); its API shape is the scheduler's
// (include/sgl/scheduler.h:33-67), which stays in Python here.
//
// A model with any other part (a toy mixer, a routed feed-forward, a turning position encoding)
// has no description in these terms and keeps the Python forward pass.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "common.cuh"

#include "step_walker.h"

extern "C" {

// ---- the launchers of the other libraries, bound at start-up --------------------------------------
typedef int (*fn_embed)(const int*, const int*, const void*, const void*, float*, int, int, int, int, int, int*,
                        cudaStream_t);
typedef int (*fn_layernorm)(const float*, const int*, const float*, const float*, void*, int, int, float, int,
                            cudaStream_t);
typedef int (*fn_gemm_simt)(const void*, const void*, const float*, void*, float*, int, int, int, int, int, int, int,
                            int, cudaStream_t);
typedef int (*fn_gemm_tc)(const void*, const void*, const float*, void*, float*, int, int, int, int, int, int, int,
                          int*, cudaStream_t);
typedef int (*fn_gemm_tc_kv)(const void*, const void*, const float*, void*, int, int, int, int, int, int, void*,
                             const int*, int, int, int, int, int, int*, cudaStream_t);
typedef int (*fn_gemm_few_supports)(int, int, int, int);
typedef int (*fn_gemm_few)(const void*, const void*, const float*, void*, float*, int, int, int, int, int, int, int,
                           cudaStream_t);
typedef int (*fn_kv_write)(const void*, const void*, int, void*, const int*, int, int, int, int, int, int, int,
                           cudaStream_t);
typedef int (*fn_attention_simt)(const void*, int, const void*, const int*, int, const int*, const int*, void*, int,
                                 int, int, int, int, int, float, int, int, int, int, int, int*, int, cudaStream_t);
typedef int (*fn_attention_prefill_tc)(const void*, int, const void*, const int*, int, const int*, const int*, void*,
                                       int, int, int, int, int, int, int, float, int, int, int, int, int*,
                                       cudaStream_t);
typedef int (*fn_decode_splits)(int, int, int);
typedef int (*fn_decode_scratch)(int, int, int, int, long long*, int*);
typedef int (*fn_attention_decode)(const void*, int, void*, const int*, int, const int*, const int*, void*, int, int,
                                   int, int, int, int, float, int, int, int, float*, int*, const void*, const void*,
                                   int, const int*, int*, const int*, int, cudaStream_t);
typedef int (*fn_attention_decode_tma)(const void*, int, void*, const int*, int, const int*, const int*, void*, int,
                                       int, int, int, int, int, float, int, int, int, const void*, const void*, int,
                                       const int*, int*, const int*, int, cudaStream_t);
typedef int (*fn_stream_supports)(int, int, int, int);
typedef int (*fn_attention_decode_stream)(const void*, int, void*, const int*, int, const int*, const int*, void*,
                                          int, int, int, int, int, int, float, int, int, const void*, const void*,
                                          int, const int*, int*, const int*, int, cudaStream_t);
}  // extern "C"

namespace {

struct Bound {
  fn_embed embed;
  fn_layernorm layernorm;
  fn_gemm_simt gemm_simt;
  fn_gemm_tc gemm_tc;
  fn_gemm_tc_kv gemm_tc_kv;
  fn_gemm_few_supports gemm_few_supports;
  fn_gemm_few gemm_few;
  fn_kv_write kv_write;
  fn_attention_simt attention_simt;
  fn_attention_prefill_tc attention_prefill_tc;
  fn_decode_splits decode_splits;
  fn_decode_scratch decode_scratch;
  fn_attention_decode attention_decode;
  fn_attention_decode_tma attention_decode_tma;
  fn_stream_supports stream_supports;
  fn_attention_decode_stream attention_decode_stream;
} g = {};

const char* const NAMES[] = {"sglc_embed", "sglc_layernorm", "sglc_gemm_simt", "sglc_gemm_tc", "sglc_gemm_tc_kv",
                             "sglc_gemm_few_supports", "sglc_gemm_few", "sglc_kv_write", "sglc_attention_simt",
                             "sglc_attention_prefill_tc", "sglc_attention_decode_splits",
                             "sglc_attention_decode_scratch", "sglc_attention_decode", "sglc_attention_decode_tma",
                             "sglc_attention_decode_stream_supports", "sglc_attention_decode_stream"};
constexpr int N_BOUND = sizeof(NAMES) / sizeof(NAMES[0]);
static_assert(sizeof(Bound) == N_BOUND * sizeof(void*), "one pointer per name");

struct Walk {
  const WalkModel& m;
  WalkStep& s;
  long long off = 0;
  int rc = 0;

  Walk(const WalkModel& m_, WalkStep& s_) : m(m_), s(s_) {}
  int elem() const { return m.bf16 ? 2 : 4; }
  int dt() const { return m.bf16 ? SGLC_BF16 : SGLC_F32; }

  // the step's bump allocator: 256-byte aligned pieces of one buffer, given back by mark/release
  unsigned char* alloc(long long rows, long long width, int size) {
    const long long start = (off + 255) & ~255LL;
    const long long bytes = rows * width * size;
    if (start + bytes > s.workspace_bytes) {
      fail(SGLC_ERR_ARGUMENT, "step workspace too small");
      return nullptr;
    }
    off = start + bytes;
    if (off > s.workspace_peak) s.workspace_peak = off;
    return s.workspace + start;
  }
  void fail(int code, const char* what) {
    if (rc == 0) {
      rc = code;
      strncpy(s.where, what, sizeof(s.where) - 1);
    }
  }
  bool check(int code, const char* what) {
    s.launches++;
    if (code != 0) fail(code, what);
    return rc == 0;
  }

  // out = act(a·wᵀ + b) or residual += a·wᵀ + b, by the kernel the runtime would choose
  void gemm(const void* a, int M, int lda, const WalkLinear& l, void* out, int ldo, bool out_f32, float* residual,
            int act) {
    if (rc) return;
    const bool tc_ok = m.bf16 && l.K % 8 == 0 && lda % 8 == 0 && ((uintptr_t)a & 15) == 0 && ((uintptr_t)l.w & 15) == 0;
    if (tc_ok) {
      if (s.few_ok && M <= s.few_max_tokens && (long long)l.N * l.K <= s.few_max_weight &&
          g.gemm_few_supports(M, l.N, l.K, lda)) {
        check(g.gemm_few(a, l.w, l.bias, out, residual, M, l.N, l.K, lda, ldo, out_f32 ? 1 : 0, act, s.stream),
              "gemm_few");
        return;
      }
      check(g.gemm_tc(a, l.w, l.bias, out, residual, M, l.N, l.K, lda, ldo, out_f32 ? 1 : 0, act, s.tc_err, s.stream),
            "gemm_tc");
      return;
    }
    const int dst_dt = (residual || out_f32) ? SGLC_F32 : dt();
    check(g.gemm_simt(a, l.w, l.bias, out, residual, M, l.N, l.K, lda, ldo, dt(), dst_dt, act, s.stream), "gemm_simt");
  }

  void norm(const float* x, const int* rows, const WalkNorm& n, void* out, int n_rows) {
    if (rc) return;
    check(g.layernorm(x, rows, n.gamma, n.beta, out, n_rows, n.size, n.eps, dt(), s.stream), "layernorm");
  }

  // single decoded tokens over the cache (csrc/ops.py: attention_decode), keys split across blocks
  void attention_decode(const unsigned char* q, int q_stride, const WalkCall& c, const WalkLayer& L, const int* bt,
                        const int* token_req, unsigned char* out, int o_stride, const unsigned char* k_new,
                        const unsigned char* v_new, int new_stride, const int* slots, const int* token_list,
                        int n_tokens) {
    const int H = L.n_heads, Hkv = L.n_kv_heads, D = L.head_dim, ps = m.page_size;
    int T = n_tokens;
    bool order_only = false;
    if (token_list && (token_req == nullptr || k_new != nullptr)) order_only = true;
    int splits = g.decode_splits(T, H, s.max_keys);
    long long need_ws = 0;
    int need_c = 0;
    g.decode_scratch(T, H, D, splits, &need_ws, &need_c);
    if (need_ws > s.tc_ws_floats || need_c > s.tc_n_counters) splits = 1;
    if (s.use_tma_decode && T * H >= s.stream_min_items && g.stream_supports(D, ps, s.max_keys, L.window) &&
        (ps * D * 2) % 128 == 0) {
      check(g.attention_decode_stream(q, q_stride, c.cache, bt, s.bt_stride, token_req, s.positions, out, o_stride, T,
                                      H, Hkv, D, ps, L.scale, L.window, s.max_keys, k_new, v_new, new_stride, slots,
                                      s.tc_err, token_list, c.n_pages, s.stream),
            "attention_decode_stream");
      return;
    }
    if (order_only) token_list = nullptr;
    if ((D == 64 || D == 128) && splits <= 8 && (ps * D * 2) % 128 == 0 && ps <= 256 && s.use_tma_decode &&
        T * H * splits <= 1536) {
      const int code = g.attention_decode_tma(q, q_stride, c.cache, bt, s.bt_stride, token_req, s.positions, out,
                                              o_stride, T, H, Hkv, D, ps, L.scale, L.window, s.max_keys, splits, k_new,
                                              v_new, new_stride, slots, s.tc_err, token_list, c.n_pages, s.stream);
      if (code != SGLC_ERR_UNSUPPORTED) {      // (that code: the range does not fit its shared memory)
        check(code, "attention_decode_tma");
        return;
      }
    }
    check(g.attention_decode(q, q_stride, c.cache, bt, s.bt_stride, token_req, s.positions, out, o_stride, T, H, Hkv,
                             D, ps, L.scale, L.window, s.max_keys, splits, s.tc_ws, s.tc_counters, k_new, v_new,
                             new_stride, slots, s.tc_err, token_list, c.n_pages, s.stream),
          "attention_decode");
  }

  // keys and values into the cache, then causal attention over it (engine/runtime.py: attend)
  // the query/key/value projection; true if its epilogue has written keys and values into the
  // cache (engine/runtime.py: project_qkv)
  bool project_qkv(const void* h, int T, const WalkLayer& L, const WalkCall& c, void* qkv, int wq) {
    if (rc) return false;
    const bool tc_ok = m.bf16 && L.qkv.K % 8 == 0 && m.hidden % 8 == 0 && ((uintptr_t)h & 15) == 0 &&
                       ((uintptr_t)L.qkv.w & 15) == 0;
    if (tc_ok && c.write && s.max_q_len > 1 && L.qkv.N == (L.n_heads + 2 * L.n_kv_heads) * L.head_dim) {
      const int code = g.gemm_tc_kv(h, L.qkv.w, L.qkv.bias, qkv, T, L.qkv.N, L.qkv.K, m.hidden, wq, SGLC_ACT_NONE, c.cache,
                                    s.slots[c.group], L.n_heads * L.head_dim, L.n_kv_heads, L.head_dim, m.page_size,
                                    c.n_pages, s.tc_err, s.stream);
      if (code != SGLC_ERR_UNSUPPORTED) {
        check(code, "gemm_tc_kv");
        return rc == 0;
      }
    }
    gemm(h, T, m.hidden, L.qkv, qkv, wq, false, nullptr, SGLC_ACT_NONE);
    return false;
  }

  void attend(const unsigned char* q, const unsigned char* k, const unsigned char* v, int stride, const WalkCall& c,
              const WalkLayer& L, unsigned char* o, int o_stride, bool kv_written) {
    if (rc) return;
    const int H = L.n_heads, Hkv = L.n_kv_heads, D = L.head_dim, ps = m.page_size;
    const int* bt = s.block_tables[c.group];
    const int* slots = s.slots[c.group];
    const bool bf16_ok = m.bf16 && D % 8 == 0 && stride % 8 == 0 && ((uintptr_t)q & 15) == 0;
    if (bf16_ok && s.max_q_len == 1) {
      const bool fuse = c.write && ((uintptr_t)k & 15) == 0 && ((uintptr_t)v & 15) == 0;
      if (c.write && !fuse)
        if (!check(g.kv_write(k, v, stride, c.cache, slots, s.T, Hkv, D, ps, c.n_pages, dt(), dt(), s.stream), "kv_write"))
          return;
      attention_decode(q, stride, c, L, bt, nullptr, o, o_stride, fuse ? k : nullptr, fuse ? v : nullptr,
                       fuse ? stride : 0, fuse ? slots : nullptr, s.decode_ordered ? s.decode_tokens : nullptr, s.T);
      return;
    }
    if (c.write && !kv_written)
      if (!check(g.kv_write(k, v, stride, c.cache, slots, s.T, Hkv, D, ps, c.n_pages, dt(), dt(), s.stream), "kv_write"))
        return;
    if (bf16_ok && (D == 64 || D == 128) && L.scale > 0 && o_stride % 8 == 0 && ((uintptr_t)o & 15) == 0) {
      const bool split = s.n_decode > 0;
      if (!check(g.attention_prefill_tc(q, stride, c.cache, bt, s.bt_stride, s.q_start, s.kv_len, o, o_stride, s.R,
                                        s.max_q_len, H, Hkv, D, ps, L.scale, L.window, s.T, c.n_pages, split ? 1 : 0,
                                        s.tc_err, s.stream),
                 "attention_prefill_tc"))
        return;
      if (split)
        attention_decode(q, stride, c, L, bt, s.token_req, o, o_stride, nullptr, nullptr, 0, nullptr, s.decode_tokens,
                         s.n_decode);
      return;
    }
    check(g.attention_simt(q, stride, c.cache, bt, s.bt_stride, s.token_req, s.positions, o, o_stride, s.T, H, Hkv, D,
                           ps, L.scale, L.window, s.max_keys, dt(), dt(), c.n_pages, s.tc_err, s.max_q_len, s.stream),
          "attention_simt");
  }

  void layer(const WalkLayer& L, const WalkCall& c, float* x) {
    const int T = s.T, E = m.hidden, es = elem();
    const long long mark = off;
    unsigned char* h = alloc(T, E, es);
    if (!h) return;
    norm(x, nullptr, L.norm1, h, T);
    const long long inner = off;
    {
      const int H = L.n_heads, Hkv = L.n_kv_heads, D = L.head_dim;
      const int wq = (H + 2 * Hkv) * D;
      unsigned char* qkv = alloc(T, wq, es);
      if (!qkv) return;
      const bool kv_written = project_qkv(h, T, L, c, qkv, wq);
      unsigned char* o = alloc(T, (long long)H * D, es);
      if (!o) return;
      attend(qkv, qkv + (size_t)H * D * es, qkv + (size_t)(H + Hkv) * D * es, wq, c, L, o, H * D, kv_written);
      gemm(o, T, H * D, L.out, nullptr, E, false, x, SGLC_ACT_NONE);
    }
    off = inner;                                     // the mixer's buffers make room for the feed-forward's
    norm(x, nullptr, L.norm2, h, T);
    unsigned char* u = alloc(T, L.inner_size, es);
    if (!u) return;
    gemm(h, T, E, L.up, u, L.inner_size, false, nullptr, L.act);
    gemm(u, T, L.inner_size, L.down, nullptr, E, false, x, SGLC_ACT_NONE);
    off = mark;
  }

  int run() {
    const int T = s.T, E = m.hidden;
    float* x = reinterpret_cast<float*>(alloc(T, E, 4));
    if (!x) return rc;
    check(g.embed(s.tokens, s.positions, m.table, m.pos_table, x, T, E, m.vocab, m.pos_table ? m.n_positions : 0, dt(),
                  s.err_flag, s.stream),
          "embed");
    for (int i = 0; i < m.n_calls && rc == 0; ++i) layer(m.layers[m.order[i].layer], m.order[i], x);
    if (rc == 0 && s.n_want > 0) {
      unsigned char* hf = alloc(s.n_want, E, elem());
      if (!hf) return rc;
      norm(x, s.want_rows, m.final_norm, hf, s.n_want);
      gemm(hf, s.n_want, E, m.head, s.logits, m.head.N, true, nullptr, SGLC_ACT_NONE);
    }
    return rc;
  }
};

}  // namespace

SGLC_DEFINE_ERROR_STRING()

// The names of the launchers to bind, in the order sglc_walker_bind expects their addresses.
SGLC_API int sglc_walker_names(const char* const** names) {
  *names = NAMES;
  return N_BOUND;
}
SGLC_API int sglc_walker_bind(void* const* fns, int n) {
  if (n != N_BOUND) return SGLC_ERR_ARGUMENT;
  for (int i = 0; i < n; ++i)
    if (!fns[i]) return SGLC_ERR_ARGUMENT;
  memcpy(&g, fns, sizeof(g));
  return SGLC_OK;
}
SGLC_API int sglc_walker_struct_sizes(int* sizes) {
  sizes[0] = (int)sizeof(WalkLinear); sizes[1] = (int)sizeof(WalkNorm); sizes[2] = (int)sizeof(WalkLayer);
  sizes[3] = (int)sizeof(WalkCall); sizes[4] = (int)sizeof(WalkModel); sizes[5] = (int)sizeof(WalkStep);
  return 6;
}

// One forward pass of the step: every token through every call of the running order, logits of
// the wanted rows into step->logits.  Returns 0 or the failing launcher's code (step->where
// names the operation).
SGLC_API int sglc_walker_forward(const WalkModel* model, WalkStep* step) {
  if (!g.embed) return SGLC_ERR_ARGUMENT;
  if (step->T <= 0) return SGLC_OK;
  step->launches = 0;
  step->workspace_peak = 0;
  step->where[0] = 0;
  Walk w(*model, *step);
  return w.run();
}
