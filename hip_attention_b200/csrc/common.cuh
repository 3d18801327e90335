// Shared device / host helpers for libhipattn_sm100.so.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hipattn.h"

namespace hipattn {

// ---------------------------------------------------------------------------------------------
// host-side error reporting
// ---------------------------------------------------------------------------------------------
void set_error(const char* fmt, ...);

#define HIPATTN_REQUIRE(cond, code, ...) \
  do {                                   \
    if (!(cond)) {                       \
      ::hipattn::set_error(__VA_ARGS__); \
      return (code);                     \
    }                                    \
  } while (0)

#define HIPATTN_CUDA_OK(expr)                                                          \
  do {                                                                                 \
    cudaError_t e_ = (expr);                                                           \
    if (e_ != cudaSuccess) {                                                           \
      ::hipattn::set_error("%s failed: %s", #expr, cudaGetErrorString(e_));            \
      return HIPATTN_ERR_CUDA;                                                         \
    }                                                                                  \
  } while (0)

// kernels launched by this library in this process (every launch site goes through check_launch)
void count_launch();

inline int check_launch(const char* what) {
  count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("launch of %s failed: %s", what, cudaGetErrorString(e));
    return HIPATTN_ERR_CUDA;
  }
  return HIPATTN_OK;
}

int validate_tokens(const hipattn_tokens_t& t, int elem_bytes, int D, const char* name);

// ---------------------------------------------------------------------------------------------
// element types
// ---------------------------------------------------------------------------------------------
template <int DT>
struct Elem;
template <>
struct Elem<HIPATTN_F32> {
  using type = float;
  static constexpr int bytes = 4;
  __device__ static __forceinline__ float to_f32(float x) { return x; }
  __device__ static __forceinline__ float round(float x) { return x; }
  __device__ static __forceinline__ float from_f32(float x) { return x; }
};
template <>
struct Elem<HIPATTN_F16> {
  using type = __half;
  static constexpr int bytes = 2;
  __device__ static __forceinline__ float to_f32(__half x) { return __half2float(x); }
  __device__ static __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
  __device__ static __forceinline__ __half from_f32(float x) { return __float2half_rn(x); }
};
template <>
struct Elem<HIPATTN_BF16> {
  using type = __nv_bfloat16;
  static constexpr int bytes = 2;
  __device__ static __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
  __device__ static __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
  __device__ static __forceinline__ __nv_bfloat16 from_f32(float x) { return __float2bfloat16_rn(x); }
};

// ---------------------------------------------------------------------------------------------
// order-preserving score encoding: a < b  <=>  enc(a) < enc(b) as signed 32-bit integers, so the
// head max is an integer max (atomicMax on the device, MAX all-reduce on int32 across GPUs)
// ---------------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ int32_t encode_score_bits(uint32_t bits) {
  return (int32_t)((bits & 0x80000000u) ? (bits ^ 0x7fffffffu) : bits);
}
__host__ __device__ __forceinline__ uint32_t decode_score_bits(int32_t code) {
  const uint32_t c = (uint32_t)code;
  return (c & 0x80000000u) ? (c ^ 0x7fffffffu) : c;
}
__device__ __forceinline__ int32_t encode_score(float s) { return encode_score_bits(__float_as_uint(s)); }
__device__ __forceinline__ float decode_score(int32_t c) { return __uint_as_float(decode_score_bits(c)); }
// ascending sort key: best score first, lower position first among equal scores
__device__ __forceinline__ unsigned long long score_sort_key(int32_t code, unsigned position) {
  return ((unsigned long long)(~((uint32_t)code ^ 0x80000000u)) << 32) | position;
}

// ---------------------------------------------------------------------------------------------
// token addressing: dense K[b, t, h, :] or paged cache[block_table[b, t / P], t % P, h, :]
// ---------------------------------------------------------------------------------------------
// Returns the element offset of row (b, t, hkv) from the base pointer returned in *base.
// Out-of-range page ids are clamped to page 0 and flagged; positions at or beyond cache_seq_lens[b]
// read page 0 (as the reference does: the table lookup is masked with other=0).
__device__ __forceinline__ const char* token_row(const hipattn_tokens_t& tk, int b, int64_t t, int hkv, int elem_bytes,
                                                 uint32_t* status) {
  if (tk.fp8_e5m2) elem_bytes = 1;
  if (tk.cache == nullptr) {
    int64_t off = (int64_t)b * tk.stride_b + t * tk.stride_t + (int64_t)hkv * tk.stride_h;
    return (const char*)tk.dense + off * elem_bytes;
  }
  int64_t seq = tk.seq_lens_is_i64 ? ((const int64_t*)tk.cache_seq_lens)[b] : (int64_t)((const int32_t*)tk.cache_seq_lens)[b];
  int64_t page = 0;
  // page index and offset in 32-bit arithmetic (positions are below 2^31), by a shift when the page size is a power of
  // two: a 64-bit division costs about a hundred instructions, and this sits in the decode kernels' row loops
  const int ti = (int)t, ps = tk.page_size;
  int pi, poff;
  if ((ps & (ps - 1)) == 0) {
    pi = ti >> (31 - __clz(ps));
    poff = ti & (ps - 1);
  } else {
    pi = ti / ps;
    poff = ti - pi * ps;
  }
  if (t >= 0 && t < seq && pi < tk.table_width) {
    int64_t o = (int64_t)b * tk.table_stride_b + pi;
    page = tk.table_is_i64 ? ((const int64_t*)tk.block_table)[o] : (int64_t)((const int32_t*)tk.block_table)[o];
    if (page < 0 || page >= tk.n_pages) {
      if (status) atomicOr(status, HIPATTN_STATUS_PAGE_RANGE);
      page = 0;
    }
  }
  int64_t off = page * tk.stride_page + (int64_t)poff * tk.stride_off + (int64_t)hkv * tk.stride_ch;
  return (const char*)tk.cache + off * elem_bytes;
}

// Access statistics: 1 at the position (dense) or page (paged: the block-table entry, page 0 beyond the sequence) of
// token t in counter [B, HKV, n] (uvm_gpu_cache.py:846-909 stores the same 1 on every load).
__device__ __forceinline__ void mark_access(int32_t* counter, int64_t stride_b, int64_t stride_h, int n, const hipattn_tokens_t& tk,
                                            int b, int hkv, int64_t t) {
  int64_t i = t;
  if (tk.cache != nullptr) {
    const int64_t seq = tk.seq_lens_is_i64 ? ((const int64_t*)tk.cache_seq_lens)[b] : (int64_t)((const int32_t*)tk.cache_seq_lens)[b];
    const int64_t pi = (int)t / tk.page_size;
    i = 0;
    if (t >= 0 && t < seq && pi < tk.table_width) {
      const int64_t o = (int64_t)b * tk.table_stride_b + pi;
      i = tk.table_is_i64 ? ((const int64_t*)tk.block_table)[o] : (int64_t)((const int32_t*)tk.block_table)[o];
    }
  }
  if (i >= 0 && i < n) counter[(int64_t)b * stride_b + (int64_t)hkv * stride_h + i] = 1;
}

// two floats rounded to the 16-bit element type and packed, low half first
template <int DT>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if (DT == HIPATTN_BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Eight e5m2 values (8 bytes) as eight elements of the 16-bit type DT.  An e5m2 value is the upper byte of the
// half-precision number with the same value, and every such number is also exact in bfloat16, so the conversion
// loses nothing (the reference converts the same way on load, uvm_gpu_cache.py:1043-1046).
template <int DT>
__device__ __forceinline__ uint4 widen_fp8_e5m2(uint2 w) {
  const uint32_t h[4] = {__byte_perm(w.x, 0, 0x1404), __byte_perm(w.x, 0, 0x3424), __byte_perm(w.y, 0, 0x1404), __byte_perm(w.y, 0, 0x3424)};
  if (DT == HIPATTN_F16) return make_uint4(h[0], h[1], h[2], h[3]);
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h[i]));
    __nv_bfloat162 b2 = __floats2bfloat162_rn(f.x, f.y);
    o[i] = *reinterpret_cast<uint32_t*>(&b2);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
// The same copy to a shared-memory address, or sixteen zero bytes when `live` is false: a copy of zero source bytes
// fills its destination with zeros and reads nothing, so a loop of copies needs no branch around masked rows.
__device__ __forceinline__ void cp_async16_zfill(uint32_t smem_addr, const void* gmem, bool live) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr), "l"(gmem), "r"(live ? 16 : 0));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__host__ __device__ __forceinline__ int cdiv(int a, int b) { return (a + b - 1) / b; }

}  // namespace hipattn
