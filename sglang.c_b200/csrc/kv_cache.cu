// Writing new keys and values into the paged cache.
// One layer's cache is [n_pages][2][n_kv_heads][page_size][head_dim]: a page holds
// page_size positions of every head, keys then values, so that one (page, head)
// tile of keys is one contiguous box.  The reference keeps [page][E] rows with
// one position per page (src/gpt2.c:133-134,227-235) and copies K and V columns
// of the fused qkv buffer with two 2-D copies per layer on the GPU
// (src/cuda_backend.cu:5780-5790); here one kernel scatters both through a
// per-token slot index (slot = page*page_size + offset; negative = skip).
#include "common.cuh"

SGLC_DEFINE_ERROR_STRING()

template <typename TS, typename TC>
__global__ void kv_write_kernel(const TS* __restrict__ k_src, const TS* __restrict__ v_src,
                                int src_stride, TC* __restrict__ cache,
                                const int* __restrict__ slots, int T, int Hkv, int D,
                                int page_size, int n_pages) {
  int t = blockIdx.x;
  if (t >= T) return;
  pdl_launch_dependents();
  pdl_wait();
  int slot = slots[t];
  if (slot < 0) return;
  int page = slot / page_size, off = slot % page_size;
  if (page >= n_pages) return;
  size_t page_elems = (size_t)2 * Hkv * page_size * D;
  TC* kp = cache + (size_t)page * page_elems;
  TC* vp = kp + (size_t)Hkv * page_size * D;
  const TS* ks = k_src + (size_t)t * src_stride;
  const TS* vs = v_src + (size_t)t * src_stride;
  int HD = Hkv * D;
  if (sizeof(TS) == sizeof(TC) && (D * sizeof(TC)) % 16 == 0 && (((uintptr_t)ks | (uintptr_t)vs) & 15) == 0 &&
      ((size_t)src_stride * sizeof(TS)) % 16 == 0) {
    // same type on both sides and 16-byte aligned rows: whole 16-byte pieces
    constexpr int PER = 16 / sizeof(TC);
    for (int i = threadIdx.x; i < HD / PER; i += blockDim.x) {
      int h = (i * PER) / D, d = (i * PER) % D;
      size_t o = ((size_t)h * page_size + off) * D + d;
      *reinterpret_cast<uint4*>(kp + o) = *reinterpret_cast<const uint4*>(ks + (size_t)i * PER);
      *reinterpret_cast<uint4*>(vp + o) = *reinterpret_cast<const uint4*>(vs + (size_t)i * PER);
    }
    return;
  }
  for (int i = threadIdx.x; i < HD; i += blockDim.x) {
    int h = i / D, d = i % D;
    size_t o = ((size_t)h * page_size + off) * D + d;
    kp[o] = from_f32<TC>(to_f32(ks[i]));
    vp[o] = from_f32<TC>(to_f32(vs[i]));
  }
}

// k_src / v_src: first key / value element of token 0 (rows src_stride elements apart,
// heads side by side).  src_dtype and cache_dtype must be equal (F32 or BF16).
SGLC_API int sglc_kv_write(const void* k_src, const void* v_src, int src_stride, void* cache,
                           const int* slots, int T, int Hkv, int D, int page_size, int n_pages,
                           int src_dtype, int cache_dtype, cudaStream_t stream) {
  if (T <= 0) return SGLC_OK;
  int threads = Hkv * D >= 2048 ? 256 : (Hkv * D >= 512 ? 128 : 64);
  if (src_dtype == SGLC_F32 && cache_dtype == SGLC_F32)
    return sglc_launch(kv_write_kernel<float, float>, dim3(T), dim3(threads), 0, stream, 1, true,
                       (const float*)k_src, (const float*)v_src, src_stride, (float*)cache, slots, T,
                       Hkv, D, page_size, n_pages);
  else if (src_dtype == SGLC_BF16 && cache_dtype == SGLC_BF16)
    return sglc_launch(kv_write_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(T), dim3(threads), 0,
                       stream, 1, true, (const __nv_bfloat16*)k_src, (const __nv_bfloat16*)v_src,
                       src_stride, (__nv_bfloat16*)cache, slots, T, Hkv, D, page_size, n_pages);
  else
    return SGLC_ERR_ARGUMENT;
  return sglc_launch_status();
}
