// Element widening and the rotary position embedding applied inside the kernels, shared by the scan and the
// attention kernels.
#pragma once
#include "common.cuh"

namespace hipattn {

template <int DT>
__device__ __forceinline__ void widen_piece(const uint4& w, float* out);
template <>
__device__ __forceinline__ void widen_piece<HIPATTN_F32>(const uint4& w, float* out) {
  out[0] = __uint_as_float(w.x); out[1] = __uint_as_float(w.y); out[2] = __uint_as_float(w.z); out[3] = __uint_as_float(w.w);
}
template <>
__device__ __forceinline__ void widen_piece<HIPATTN_BF16>(const uint4& w, float* out) {
  const uint32_t v[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(v[i] << 16);
    out[2 * i + 1] = __uint_as_float(v[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void widen_piece<HIPATTN_F16>(const uint4& w, float* out) {
  const uint32_t v[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v[i]));
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}

// ---- rotary position embedding applied inside the kernels (un-rotated q / k plus cos / sin tables) ----
// x * cos + rotate_half(x) * sin in the element type: both products and the sum are rounded to the element type,
// as the reference computes them (attention_extend.py:392-407, 690-703).  `x` holds one 16-byte piece of a row as
// floats, `xr` the piece half a row away (rotate_half pairs element d with d +- D / 2; the sign is negative for the
// first half of the row), `tc` / `ts` the cos / sin pieces of the target position.
template <int DT, int VEC>
__device__ __forceinline__ void rope_rotate_piece(float* x, const float* xr, const float* tc, const float* ts, bool first_half) {
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    const float a = Elem<DT>::round(__fmul_rn(x[e], tc[e]));
    const float r = Elem<DT>::round(__fmul_rn(first_half ? -xr[e] : xr[e], ts[e]));
    x[e] = Elem<DT>::round(__fadd_rn(a, r));
  }
}
// The same rotation on packed pairs of 16-bit elements: lo / hi are the 16-byte pieces of the first / second half of a
// row, c / s the cos / sin pieces.  A product of two 16-bit floats is exact in fp32, and a sum of two rounds to the same
// 16-bit value with or without an fp32 step in between, so the packed instructions give the bits of rope_rotate_piece.
template <int DT> struct Pair16;
template <> struct Pair16<HIPATTN_F16> { using type = __half2; };
template <> struct Pair16<HIPATTN_BF16> { using type = __nv_bfloat162; };
template <int DT>
__device__ __forceinline__ void rope_rotate_packed(uint4& lo, uint4& hi, const uint4& c, const uint4& s) {
  using P = typename Pair16<DT>::type;
  uint32_t l[4] = {lo.x, lo.y, lo.z, lo.w}, h[4] = {hi.x, hi.y, hi.z, hi.w};
  const uint32_t cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const P lv = *reinterpret_cast<const P*>(&l[i]), hv = *reinterpret_cast<const P*>(&h[i]);
    const P cv = *reinterpret_cast<const P*>(&cc[i]), sv = *reinterpret_cast<const P*>(&ss[i]);
    const P ol = __hadd2_rn(__hmul2_rn(lv, cv), __hmul2_rn(__hneg2(hv), sv));
    const P oh = __hadd2_rn(__hmul2_rn(hv, cv), __hmul2_rn(lv, sv));
    l[i] = *reinterpret_cast<const uint32_t*>(&ol);
    h[i] = *reinterpret_cast<const uint32_t*>(&oh);
  }
  lo = make_uint4(l[0], l[1], l[2], l[3]);
  hi = make_uint4(h[0], h[1], h[2], h[3]);
}
// raw 16-byte piece `piece` of table row `pos` (16-bit tables)
__device__ __forceinline__ uint4 rope_table_raw(const void* table, int64_t stride, int rows, int pos, int piece) {
  const int r = pos < 0 ? 0 : (pos >= rows ? rows - 1 : pos);
  return __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(table) + (int64_t)r * stride + piece * 8));
}
// 16-byte piece `piece` (of the first half of the row: the tables repeat) of table row `pos`, widened to floats
template <int DT>
__device__ __forceinline__ void rope_table_piece(const void* table, int64_t stride, int rows, int pos, int piece, float* out) {
  using T = typename Elem<DT>::type;
  constexpr int VEC = 16 / Elem<DT>::bytes;
  const int r = pos < 0 ? 0 : (pos >= rows ? rows - 1 : pos);
  widen_piece<DT>(__ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(table) + (int64_t)r * stride + piece * VEC)), out);
}

}  // namespace hipattn
