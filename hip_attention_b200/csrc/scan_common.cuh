// Pieces shared by the two scan kernels: pooled queries and the per-call work split.
#pragma once
#include "common.cuh"
#include "rope.cuh"

namespace hipattn {

// One 16-byte piece of a pooled, scaled query row (attention_extend.py:607-734, 924-931): the mean of
// stride_q consecutive query rows starting at row t, accumulated in fp32 in row order, divided by the
// number of rows present, rounded to the element type, multiplied by the query scale, rounded again.
template <int DT>
__device__ __forceinline__ void pooled_query_piece(const hipattn_scan_params_t& p, int b, int h, int t, int piece, float* out) {
  using T = typename Elem<DT>::type;
  constexpr int VEC = 16 / Elem<DT>::bytes;
  float sum[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) sum[e] = 0.f;
  float cnt = 0.f;
  const T* base = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_stride_b + (int64_t)h * p.q_stride_h + piece * VEC;
  // in-kernel RoPE: every row of the group is rotated to the position derived from the group's FIRST row
  // (attention_extend.py:630-647) before it is added up
  float tc[VEC], ts[VEC];
  const int pieces = p.D / VEC, half = pieces / 2;
  if (p.rope_mode != HIPATTN_ROPE_NONE) {
    long long pv = p.pos[(int64_t)b * p.pos_stride_b + (int64_t)t * p.pos_stride_t];
    const long long cap = (long long)p.n_chunks + p.scan_window;
    const int new_t = p.rope_mode == HIPATTN_ROPE_RELATIVE ? 1 + p.scan_window : (int)(pv < cap ? (pv < 0 ? 0 : pv) : cap);
    rope_table_piece<DT>(p.rope_cos, p.rope_stride, p.rope_rows, new_t, piece % half, tc);
    rope_table_piece<DT>(p.rope_sin, p.rope_stride, p.rope_rows, new_t, piece % half, ts);
  }
#pragma unroll 4
  for (int o = 0; o < p.stride_q; ++o) {
    if (t + o < p.TQ) {
      float v[VEC];
      widen_piece<DT>(*reinterpret_cast<const uint4*>(base + (int64_t)(t + o) * p.q_stride_t), v);
      if (p.rope_mode != HIPATTN_ROPE_NONE) {
        float vr[VEC];
        const int shift = (piece < half ? half : -half) * VEC;
        widen_piece<DT>(*reinterpret_cast<const uint4*>(base + (int64_t)(t + o) * p.q_stride_t + shift), vr);
        rope_rotate_piece<DT, VEC>(v, vr, tc, ts, piece < half);
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) sum[e] = __fadd_rn(sum[e], v[e]);
      cnt += 1.f;
    }
  }
  const float den = __fadd_rn(cnt, 1e-12f);
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    const float m = Elem<DT>::round(__fdiv_rn(sum[e], den));
    out[e] = Elem<DT>::round(__fmul_rn(m, p.q_scale));
  }
}

// The same piece from a copy of the query block's rows in shared memory (row i of the block at staged + i * row_bytes):
// identical arithmetic, but the rows were fetched with one batch of asynchronous copies instead of one dependent
// global load per row.  `r0` = first row of the group inside the block, `rows` = rows the block holds.
template <int DT>
__device__ __forceinline__ void pooled_query_piece_staged(const hipattn_scan_params_t& p, const unsigned char* staged, int row_bytes,
                                                          int r0, int rows, int piece, float* out, int b, int t0) {
  constexpr int VEC = 16 / Elem<DT>::bytes;
  float sum[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) sum[e] = 0.f;
  float cnt = 0.f;
  float tc[VEC], ts[VEC];
  const int pieces = p.D / VEC, half = pieces / 2;
  if (p.rope_mode != HIPATTN_ROPE_NONE) {   // as in pooled_query_piece: the position comes from the group's first row
    long long pv = p.pos[(int64_t)b * p.pos_stride_b + (int64_t)(t0 + r0) * p.pos_stride_t];
    const long long cap = (long long)p.n_chunks + p.scan_window;
    const int new_t = p.rope_mode == HIPATTN_ROPE_RELATIVE ? 1 + p.scan_window : (int)(pv < cap ? (pv < 0 ? 0 : pv) : cap);
    rope_table_piece<DT>(p.rope_cos, p.rope_stride, p.rope_rows, new_t, piece % half, tc);
    rope_table_piece<DT>(p.rope_sin, p.rope_stride, p.rope_rows, new_t, piece % half, ts);
  }
  for (int o = 0; o < p.stride_q; ++o) {
    if (r0 + o < rows) {
      float v[VEC];
      widen_piece<DT>(*reinterpret_cast<const uint4*>(staged + (size_t)(r0 + o) * row_bytes + piece * 16), v);
      if (p.rope_mode != HIPATTN_ROPE_NONE) {
        float vr[VEC];
        widen_piece<DT>(*reinterpret_cast<const uint4*>(staged + (size_t)(r0 + o) * row_bytes + (piece < half ? piece + half : piece - half) * 16), vr);
        rope_rotate_piece<DT, VEC>(v, vr, tc, ts, piece < half);
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) sum[e] = __fadd_rn(sum[e], v[e]);
      cnt += 1.f;
    }
  }
  const float den = __fadd_rn(cnt, 1e-12f);
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    const float m = Elem<DT>::round(__fdiv_rn(sum[e], den));
    out[e] = Elem<DT>::round(__fmul_rn(m, p.q_scale));
  }
}

// Smallest position among the strided rows of a query block (computed by one warp).
__device__ __forceinline__ int block_min_position(const hipattn_scan_params_t& p, int b, int t0, int Rv, int lane) {
  long long m = 0x7fffffffffffffffLL;
  for (int r = lane; r < Rv; r += 32) {
    const long long pv = p.pos[(int64_t)b * p.pos_stride_b + (int64_t)(t0 + r * p.stride_q) * p.pos_stride_t];
    m = pv < m ? pv : m;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const long long x = __shfl_xor_sync(0xffffffffu, m, o);
    m = x < m ? x : m;
  }
  return (int)(m > 0x7fffffffLL ? 0x7fffffffLL : m);
}

// ---- pieces of the tensor-core scan kernels ----

// Bound on |tensor-core dot - sequential fp32 dot| / (max|q'| * sum_d |k'_d|) used as the radius inside
// which a rounded score is not trusted (empirical; the check mode measures the observed fraction).
constexpr float kEps = 1.0f / (1 << 21);

// statistics words (mode 2)
enum { ST_KEYS = 0, ST_FALLBACK = 1, ST_WRONG = 2, ST_RATIO_BITS = 3 };

// element-wise product of two packed 16-bit pairs, rounded to nearest even (one rounding of the exact product)
template <int DT>
__device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
  if (DT == HIPATTN_BF16) {
    __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
template <int DT>
__device__ __forceinline__ float lo_f32(uint32_t w) {
  if (DT == HIPATTN_BF16) return __uint_as_float(w << 16);
  return __half2float(__ushort_as_half((unsigned short)(w & 0xffffu)));
}
template <int DT>
__device__ __forceinline__ float hi_f32(uint32_t w) {
  if (DT == HIPATTN_BF16) return __uint_as_float(w & 0xffff0000u);
  return __half2float(__ushort_as_half((unsigned short)(w >> 16)));
}
template <int DT>
__device__ __forceinline__ uint32_t pack_scalar2(float x) {
  if (DT == HIPATTN_BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(x, x);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(x, x);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Number of halving rounds of the lane's chunk: while (m >= 1) m /= 2 with m the largest chunk of the
// lane's group of block_chunk chunks (attention_extend.py:602-606, 736-737).  `wbase` is the first
// chunk of the warp; the warp's 32 chunks lie in one group when block_chunk is a multiple of 32.
__device__ __forceinline__ int chunk_rounds(const hipattn_scan_params_t& p, int64_t row, int n, int wbase, int lane,
                                            bool in_range, int left, int right) {
  int gmax;
  if ((p.block_chunk & 31) == 0) {
    const int gbase = (wbase / p.block_chunk) * p.block_chunk;
    gmax = 0;
    for (int i = lane; i < p.block_chunk; i += 32) {
      const int cc = gbase + i;
      if (cc < n) gmax = max(gmax, p.right[row * n + cc] - p.left[row * n + cc]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) gmax = max(gmax, __shfl_xor_sync(0xffffffffu, gmax, o));
  } else {  // block_chunk == 16: a group is one half-warp
    gmax = in_range ? (right - left) : 0;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) gmax = max(gmax, __shfl_xor_sync(0xffffffffu, gmax, o));
  }
  return gmax >= 1 ? 32 - __clz(gmax) : 0;
}

// CTAs per (batch, query block, head): enough to fill the GPU a few times over, never more than the
// number of chunk blocks.  With many query blocks (prefill) one CTA walks all chunk blocks and the
// pooled queries are computed once.
// `resident` (CTAs of the kernel the GPU holds at once; 0 = not given): with only a few waves of CTAs the last one
// runs on a part-empty GPU (2048 units on 888 slots: three waves' time for 2.3 waves' work), so the chunk blocks of a
// unit are split over 2 or 4 CTAs when that shortens the schedule by clearly more than the repeated prologue costs (measured:
// 1 % per extra CTA with 256-token chunks, 5 % with 8-token chunks, whose CTAs are short).
inline int scan_ctas_per_unit(int64_t units, int chunk_blocks, int resident = 0) {
  const int64_t want = (148 * 2 * 4 + units - 1) / units;
  int k = (int)(want < 1 ? 1 : (want > chunk_blocks ? chunk_blocks : want));
  if (resident > 0 && k == 1 && units < 8LL * resident) {
    auto cost = [&](int n) { return (double)((units * n + resident - 1) / resident) / n * (1.0 + 0.02 * (n - 1)); };
    double best = cost(1);
    for (int n = 2; n <= 4 && n <= chunk_blocks; n *= 2) {
      if (cost(n) < best * 0.97) {
        best = cost(n);
        k = n;
      }
    }
  }
  return k;
}

// the same for a staged key row that is first rotated to table position `new_t` (in-kernel RoPE,
// attention_extend.py:248-407): piece `pc` of the row at `row`, its partner half a row away, cos / sin of new_t
template <int DT, int D>
__device__ __forceinline__ void unpack_rope_scaled(const unsigned char* row, int pc, int new_t, const hipattn_scan_params_t& p,
                                                   float* out) {
  constexpr int VEC = 16 / Elem<DT>::bytes;
  constexpr int PIECES = D / VEC, HALF = PIECES / 2;
  if constexpr (DT != HIPATTN_F32) {
    // 16-bit types: rotation and key scale on packed pairs (the packed multiply and add round once to the element type,
    // which is what the scalar path does product by product: see rope_rotate_packed)
    using P = typename Pair16<DT>::type;
    const uint4 x = *reinterpret_cast<const uint4*>(row + pc * 16);
    const uint4 xr = *reinterpret_cast<const uint4*>(row + (pc < HALF ? pc + HALF : pc - HALF) * 16);
    const uint4 c = rope_table_raw(p.rope_cos, p.rope_stride, p.rope_rows, new_t, pc % HALF);
    const uint4 sn = rope_table_raw(p.rope_sin, p.rope_stride, p.rope_rows, new_t, pc % HALF);
    const uint32_t xv[4] = {x.x, x.y, x.z, x.w}, rv[4] = {xr.x, xr.y, xr.z, xr.w};
    const uint32_t cv[4] = {c.x, c.y, c.z, c.w}, sv[4] = {sn.x, sn.y, sn.z, sn.w};
    const uint32_t s2 = pack_scalar2<DT>(p.k_scale);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const P xp = *reinterpret_cast<const P*>(&xv[i]), rp = *reinterpret_cast<const P*>(&rv[i]);
      const P cp = *reinterpret_cast<const P*>(&cv[i]), sp = *reinterpret_cast<const P*>(&sv[i]);
      const P rot = __hadd2_rn(__hmul2_rn(xp, cp), __hmul2_rn(pc < HALF ? __hneg2(rp) : rp, sp));
      const uint32_t m = mul2<DT>(*reinterpret_cast<const uint32_t*>(&rot), s2);
      out[2 * i] = lo_f32<DT>(m);
      out[2 * i + 1] = hi_f32<DT>(m);
    }
  } else {
    float xr[VEC], tc[VEC], ts[VEC];
    widen_piece<DT>(*reinterpret_cast<const uint4*>(row + pc * 16), out);
    widen_piece<DT>(*reinterpret_cast<const uint4*>(row + (pc < HALF ? pc + HALF : pc - HALF) * 16), xr);
    rope_table_piece<DT>(p.rope_cos, p.rope_stride, p.rope_rows, new_t, pc % HALF, tc);
    rope_table_piece<DT>(p.rope_sin, p.rope_stride, p.rope_rows, new_t, pc % HALF, ts);
    rope_rotate_piece<DT, VEC>(out, xr, tc, ts, pc < HALF);
#pragma unroll
    for (int e = 0; e < VEC; ++e) out[e] = Elem<DT>::round(__fmul_rn(out[e], p.k_scale));
  }
}


}  // namespace hipattn
