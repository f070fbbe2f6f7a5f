// Sampling on the device, one block per logits row.
//   greedy: argmax, the lowest index among equal maxima (reference
//   sgl_sample_greedy, src/sampling.c:23-28; device k_argmax,
//   src/cuda_backend.cu:2584-2602).
//   temperature: w_i = exp((l_i - l_max)/T), then the cuts min_p -> top_k ->
//   top_p on the weights (src/sampling.c:124-181), then one draw by inverse CDF
//   with a uniform u in [0,1) that the host supplies (src/sampling.c:183-199).
// Differences from the reference, on purpose: it sorts candidates with qsort,
// whose order among equal probabilities is unspecified, and walks the CDF in
// that order; here nothing is sorted.  Cuts are thresholds on the weight found
// by bisection over its bit pattern (all weights equal to the threshold are
// kept), and the CDF is walked in index order.  The kept set and the
// distribution are the same; which token a given u maps to is not.
// Penalties (src/sampling.c:48-90) are applied to the row in place first, from
// (token, count) pairs of the request's history that the host prepares.
#include "common.cuh"

SGLC_DEFINE_ERROR_STRING()

namespace {
constexpr int THREADS = 1024;

__device__ __forceinline__ int block_sum_int(int v, int* red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    int t = lane < (THREADS >> 5) ? red[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

struct RowParams {
  float temperature, top_p, min_p, u;
  int top_k;
  float rep_penalty, freq_penalty, pres_penalty;
  int hist_begin, hist_end;   // range in the (token, count) pair arrays
};

__global__ void __launch_bounds__(THREADS)
sample_kernel(float* __restrict__ logits, int ld, int V, const RowParams* __restrict__ params,
              const int* __restrict__ hist_tok, const int* __restrict__ hist_cnt,
              int* __restrict__ out_tok, float* __restrict__ out_logprob) {
  __shared__ float redf[33];
  __shared__ int redi[33];
  __shared__ float chunk_sum[THREADS];
  __shared__ int s_pick;
  int row = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  float* l = logits + (size_t)row * ld;
  RowParams p = params[row];
  int tid = threadIdx.x;

  // penalties, in place (each history token appears once in the pair list)
  bool rep = p.rep_penalty > 0.0f && p.rep_penalty != 1.0f;
  if (rep || p.freq_penalty != 0.0f || p.pres_penalty != 0.0f) {
    for (int i = p.hist_begin + tid; i < p.hist_end; i += THREADS) {
      int t = hist_tok[i];
      if (t < 0 || t >= V) continue;
      float v = l[t];
      if (rep) v = v > 0.0f ? v / p.rep_penalty : v * p.rep_penalty;
      v -= p.freq_penalty * (float)hist_cnt[i];
      v -= p.pres_penalty;
      l[t] = v;
    }
    __syncthreads();
  }

  // max and its lowest index
  float m = -INFINITY;
  int mi = V;
  for (int i = tid; i < V; i += THREADS) {
    float v = l[i];
    if (v > m) { m = v; mi = i; }
  }
  float gm = block_max(m, redf);
  int cand = (m == gm) ? mi : V;
  // lowest index among the threads that hold the maximum
  {
    int v = cand;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if ((tid & 31) == 0) redi[tid >> 5] = v;
    __syncthreads();
    if (tid < 32) {
      int t = redi[tid];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) t = min(t, __shfl_xor_sync(0xffffffffu, t, o));
      if (tid == 0) redi[32] = t;
    }
    __syncthreads();
  }
  int arg = redi[32];
  if (arg >= V) arg = 0;   // a row of NaN: fall back to token 0, as first-max-wins would

  int pick = arg;
  if (p.temperature > 0.0f) {
    float invT = 1.0f / p.temperature;
    // total weight
    float s = 0.0f;
    for (int i = tid; i < V; i += THREADS) s += expf((l[i] - gm) * invT);
    float S = block_sum(s, redf);
    // threshold on the weight; w_max = 1
    float thr = 0.0f;
    if (p.min_p > 0.0f && p.min_p < 1.0f) thr = p.min_p;
    if (p.top_k > 0 && p.top_k < V) {
      // largest t with count(w >= max(t,thr)) >= k, by bits
      unsigned t = 0;
      for (int bit = 30; bit >= 0; bit--) {
        unsigned c = t | (1u << bit);
        float cf = __uint_as_float(c);
        if (!(cf <= 1.0f)) continue;   // weights lie in [0,1]; also skips NaN patterns
        float lim = fmaxf(cf, thr);
        int n = 0;
        for (int i = tid; i < V; i += THREADS) n += expf((l[i] - gm) * invT) >= lim;
        if (block_sum_int(n, redi) >= p.top_k) t = c;
      }
      thr = fmaxf(thr, __uint_as_float(t));
    }
    if (p.top_p > 0.0f && p.top_p < 1.0f) {
      float target = p.top_p * S;
      unsigned t = 0;
      for (int bit = 30; bit >= 0; bit--) {
        unsigned c = t | (1u << bit);
        float cf = __uint_as_float(c);
        if (!(cf <= 1.0f)) continue;   // weights lie in [0,1]; also skips NaN patterns
        float lim = fmaxf(cf, thr);
        float a = 0.0f;
        for (int i = tid; i < V; i += THREADS) {
          float w = expf((l[i] - gm) * invT);
          a += w >= lim ? w : 0.0f;
        }
        if (block_sum(a, redf) >= target) t = c;
      }
      thr = fmaxf(thr, __uint_as_float(t));
    }
    // inverse CDF in index order over the kept weights; thread t owns a contiguous chunk
    int per = (V + THREADS - 1) / THREADS;
    int c0 = tid * per, c1 = min(V, c0 + per);
    float cs = 0.0f;
    for (int i = c0; i < c1; i++) {
      float w = expf((l[i] - gm) * invT);
      cs += w >= thr ? w : 0.0f;
    }
    chunk_sum[tid] = cs;
    if (tid == 0) s_pick = -1;
    __syncthreads();
    if (tid == 0) {
      float run = 0.0f;
      for (int t = 0; t < THREADS; t++) {
        float v = chunk_sum[t];
        chunk_sum[t] = run;    // exclusive prefix
        run += v;
      }
      redf[32] = run;
    }
    __syncthreads();
    float R = redf[32];
    float target = p.u * R;
    float before = chunk_sum[tid];
    if (cs > 0.0f && target >= before && target < before + cs) {
      float run = before;
      int last_kept = -1;
      int found = -1;
      for (int i = c0; i < c1; i++) {
        float w = expf((l[i] - gm) * invT);
        if (w >= thr) {
          last_kept = i;
          run += w;
          if (target < run) { found = i; break; }
        }
      }
      if (found < 0) found = last_kept;   // rounding at the chunk's end
      s_pick = found;
    }
    __syncthreads();
    pick = s_pick;
    if (pick < 0) {
      // rounding put the target at or beyond the total: the last kept index
      int lk = -1;
      for (int i = c0; i < c1; i++)
        if (expf((l[i] - gm) * invT) >= thr) lk = i;
      __syncthreads();
      if (lk >= 0) atomicMax(&s_pick, lk);
      __syncthreads();
      pick = s_pick >= 0 ? s_pick : arg;
    }
  }
  if (out_logprob) {
    // log-softmax of the (penalised) logits at the pick (src/sampling.c:38-45,206-209)
    float s = 0.0f;
    for (int i = tid; i < V; i += THREADS) s += expf(l[i] - gm);
    float Z = block_sum(s, redf);
    if (tid == 0) out_logprob[row] = (l[pick] - gm) - logf(Z);
  }
  if (tid == 0) out_tok[row] = pick;
}
}  // namespace

// logits: [n_rows][ld] float (rows are changed in place by penalties).
// params: n_rows records of 10 32-bit words: temperature, top_p, min_p, u (floats), top_k
// (int), repetition, frequency, presence penalties (floats), hist_begin, hist_end (ints).
SGLC_API int sglc_sample(float* logits, int ld, int V, int n_rows, const void* params,
                         const int* hist_tok, const int* hist_cnt, int* out_tok,
                         float* out_logprob, cudaStream_t stream) {
  if (n_rows <= 0) return SGLC_OK;
  if (V <= 0) return SGLC_ERR_ARGUMENT;
  static_assert(sizeof(RowParams) == 40, "RowParams is 10 words");
  return sglc_launch(sample_kernel, dim3(n_rows), dim3(THREADS), 0, stream, 1, true, logits, ld, V,
                     (const RowParams*)params, hist_tok, hist_cnt, out_tok, out_logprob);
}
