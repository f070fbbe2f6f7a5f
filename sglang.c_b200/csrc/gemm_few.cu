// Products of a few tokens (1 to 8: single decoded tokens of one or two requests are its use)
// with a small weight matrix: out = act(A·Wᵀ + bias), or residual += A·Wᵀ + bias.
//
// With so few tokens every weight is used once, so nothing is staged in shared memory and no
// block waits for another: a block owns 8 output features over the whole of K, its warps share
// K in groups of 32, and each lane brings 16 bytes of a weight row and 16 bytes of a token row
// straight from global memory into the registers that the warp-level tensor-core instruction
// (m16n8k16: tokens as its 16 rows, features as its 8 columns) takes them from.  The sum over k
// does not care about the order of k as long as both operands agree on it, so a lane's eight
// consecutive k stand for the instruction's k = 2t, 2t+1, 2t+8, 2t+9 of two steps and no
// shuffle or transposing load is needed.  The weights do not depend on the kernel ahead: they
// are requested before the programmatic-dependency wait, the tokens after it.  The warps' partial
// sums meet in shared memory and are added in warp order.
//
// Blocks that hold their operands in registers are heavy, and a chain of kernels that start
// while the one ahead still runs lives on many light blocks fitting on an SM together: measured,
// this kernel shortens a decode step of one or two requests at GPT-2 small's widths by 8-12 %
// and lengthens it at wider layers and from four requests on, so the runtime gives it products
// of up to two tokens with weights of up to three million elements and nothing else.
//
// The reference also takes its products of 1 to 8 rows away from the library GEMM, to kernels
// of one block per output row that pass over the weight row once for all token rows
// (src/cuda_backend.cu:333-349, 412-427, 2816-2830); the weights are [out, in] as there.
#include "common.cuh"

namespace {

constexpr int MAX_WARPS = 16;
constexpr int FB = 8;            // output features of a block
constexpr int UN = 8;            // 32-wide groups of k a warp holds in registers at a time

struct FewArgs {
  const __nv_bfloat16* A;        // [M][lda]
  const __nv_bfloat16* W;        // [N][K]
  const float* bias;             // [N] or null
  void* out;                     // [M][ldo] bfloat16 or float
  float* residual;               // float [M][ldo], updated in place (then `out` is unused)
  int M, N, K, lda, ldo, out_f32, act;
};

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 16 bytes if `on`, else zeros.  Volatile, so that the loads of a batch stay ahead of the batch's
// first MMA (and the weights' ahead of the dependency wait) whatever the compiler would prefer.
__device__ __forceinline__ uint4 load16_weights(const uint4* p, bool on) {
  uint4 v;
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %5, 0;\n\tmov.b32 %0, 0;\n\tmov.b32 %1, 0;\n\tmov.b32 %2, 0;\n\t"
      "mov.b32 %3, 0;\n\t@q ld.global.nc.L1::no_allocate.v4.b32 {%0, %1, %2, %3}, [%4];\n\t}"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(p), "r"((int)on));
  return v;
}
__device__ __forceinline__ uint4 load16_tokens(const uint4* p, bool on) {
  uint4 v;
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %5, 0;\n\tmov.b32 %0, 0;\n\tmov.b32 %1, 0;\n\tmov.b32 %2, 0;\n\t"
      "mov.b32 %3, 0;\n\t@q ld.global.cg.v4.b32 {%0, %1, %2, %3}, [%4];\n\t}"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(p), "r"((int)on)
      : "memory");
  return v;
}

__global__ void __launch_bounds__(MAX_WARPS * 32) gemm_few_kernel(const FewArgs a) {
  __shared__ float red[MAX_WARPS][32][2];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int g = lane >> 2, tq = lane & 3;
  const int f0 = blockIdx.x * FB;
  const int n_chunks = a.K >> 3;                     // 16-byte pieces of a row
  const int n_groups = (n_chunks + 3) >> 2;
  const int mine = warp < n_groups ? (n_groups - warp + nw - 1) / nw : 0;     // groups warp, warp + nw, ...
  // this lane's row of the weights (feature f0 + g: the instruction's column g) and of the tokens
  const bool w_ok = f0 + g < a.N, x_ok = g < a.M;
  const uint4* wrow = reinterpret_cast<const uint4*>(a.W + (size_t)(w_ok ? f0 + g : 0) * a.K);
  const uint4* xrow = reinterpret_cast<const uint4*>(a.A + (size_t)(x_ok ? g : 0) * a.lda);
  pdl_launch_dependents();
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};           // (rows 8..15 of the instruction stay zero)
  for (int base = 0; base == 0 || base < mine; base += UN) {
    uint4 wv[UN], xv[UN];
#pragma unroll
    for (int i = 0; i < UN; i++) {
      const int c = (warp + nw * (base + i)) * 4 + tq;
      wv[i] = load16_weights(wrow + c, w_ok && base + i < mine && c < n_chunks);
    }
    if (base == 0) pdl_wait();                       // the tokens come from the kernel ahead
#pragma unroll
    for (int i = 0; i < UN; i++) {
      const int c = (warp + nw * (base + i)) * 4 + tq;
      xv[i] = load16_tokens(xrow + c, x_ok && base + i < mine && c < n_chunks);
    }
#pragma unroll
    for (int i = 0; i < UN; i++) {
      if (base + i < mine) {                         // (uniform in the warp)
        mma_16816(acc, xv[i].x, 0u, xv[i].y, 0u, wv[i].x, wv[i].y);
        mma_16816(acc, xv[i].z, 0u, xv[i].w, 0u, wv[i].z, wv[i].w);
      }
    }
  }
  // c0, c1: token g, features 2 tq, 2 tq + 1 of the block
  *reinterpret_cast<float2*>(red[warp][lane]) = make_float2(acc[0], acc[1]);
  __syncthreads();
  if (warp != 0) return;
  float2 s = *reinterpret_cast<const float2*>(red[0][lane]);
  for (int w = 1; w < nw; w++) {
    const float2 v = *reinterpret_cast<const float2*>(red[w][lane]);
    s.x += v.x;
    s.y += v.y;
  }
  const float vals[2] = {s.x, s.y};
#pragma unroll
  for (int e = 0; e < 2; e++) {
    const int m = g, f = f0 + 2 * tq + e;
    if (m >= a.M || f >= a.N) continue;
    const float v = vals[e] + (a.bias ? a.bias[f] : 0.0f);
    const size_t at = (size_t)m * a.ldo + f;
    if (a.residual) a.residual[at] += v;
    else if (a.out_f32) reinterpret_cast<float*>(a.out)[at] = act_tc(v, a.act);
    else reinterpret_cast<__nv_bfloat16*>(a.out)[at] = __float2bfloat16_rn(act_tc(v, a.act));
  }
}

}  // namespace

SGLC_DEFINE_ERROR_STRING()

// Whether sglc_gemm_few takes the product (it has no other limits than these).
SGLC_API int sglc_gemm_few_supports(int M, int N, int K, int lda) {
  return M >= 1 && M <= 8 && N >= 1 && K >= 8 && K % 8 == 0 && lda % 8 == 0;
}

// A: bfloat16 [M,K], rows lda elements apart, 16-byte aligned; W: bfloat16 [N,K] contiguous,
// 16-byte aligned; bias float [N] or null; out [M,N] rows ldo apart (bfloat16, or float if
// out_f32), or residual (float, in place).
SGLC_API int sglc_gemm_few(const void* A, const void* W, const float* bias, void* out, float* residual,
                           int M, int N, int K, int lda, int ldo, int out_f32, int act, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return SGLC_OK;
  if (!sglc_gemm_few_supports(M, N, K, lda) || ((uintptr_t)A & 15) || ((uintptr_t)W & 15))
    return SGLC_ERR_UNSUPPORTED;
  FewArgs a;
  a.A = (const __nv_bfloat16*)A; a.W = (const __nv_bfloat16*)W; a.bias = bias; a.out = out; a.residual = residual;
  a.M = M; a.N = N; a.K = K; a.lda = lda; a.ldo = ldo; a.out_f32 = out_f32; a.act = act;
  const int n_groups = (K / 8 + 3) / 4;
  int warps = (n_groups + 3) / 4;                    // about four groups a warp (measured against 3 and 6)
  warps = warps < 4 ? 4 : (warps > MAX_WARPS ? MAX_WARPS : warps);
  return sglc_launch(gemm_few_kernel, dim3((N + FB - 1) / FB), dim3(warps * 32), 0, stream, 1, true, a);
}
