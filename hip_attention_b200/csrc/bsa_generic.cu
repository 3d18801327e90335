// Block-sparse attention, general kernel (any element type, fp32 arithmetic on CUDA cores).
//
// Serves fp32 inputs, decode (one query row per head; the heads of a KV group are packed into one
// tile so every gathered key / value row is used by all of them) and shapes the tensor-core prefill
// kernel does not cover.  Decode may split the key list into ranges; each range writes a normalised
// partial output with its base-2 log-sum-exp.
//
// Tile: BM query rows x 32 keys.  K and V rows are gathered with 16-byte loads through the page
// table (or from the dense tensor), widened to fp32 and staged in shared memory; S = Q K^T and
// O += P V run as register-blocked FMA loops; softmax is online, in base 2.
#include "bsa_common.cuh"
#include "rope.cuh"

namespace hipattn {
namespace {

constexpr int kThreads = 256;
constexpr int TK = 32;
constexpr float kLog2e = 1.4426950408889634f;

template <int DT>
__device__ __forceinline__ void widen16(const uint4& w, float* out);
template <>
__device__ __forceinline__ void widen16<HIPATTN_F32>(const uint4& w, float* out) {
  out[0] = __uint_as_float(w.x); out[1] = __uint_as_float(w.y); out[2] = __uint_as_float(w.z); out[3] = __uint_as_float(w.w);
}
template <>
__device__ __forceinline__ void widen16<HIPATTN_BF16>(const uint4& w, float* out) {
  const uint32_t v[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(v[i] << 16);
    out[2 * i + 1] = __uint_as_float(v[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void widen16<HIPATTN_F16>(const uint4& w, float* out) {
  const uint32_t v[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v[i]));
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}

template <int DT, int D, int BM>
__global__ void __launch_bounds__(kThreads) bsa_generic_kernel(const hipattn_bsa_params_t p, int packed, int rows_per_head,
                                                               int n_sub) {
  using T = typename Elem<DT>::type;
  constexpr int RPT = BM == 64 ? 2 : 1;        // rows per thread
  constexpr int TPR = kThreads / (BM / RPT);   // threads per row: 8 or 16
  constexpr int TPT = TK / TPR;                // keys per thread: 4 or 2
  constexpr int DS = D + 4;                    // padded row stride in floats
  constexpr int NV = D / 4 / TPR;              // float4 output columns per thread
  constexpr int VEC = 16 / Elem<DT>::bytes;
  constexpr int PIECES = D / VEC;
  static_assert(NV >= 1, "head dimension too small for this tiling");

  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* Qs = reinterpret_cast<float*>(smem_raw);  // [BM][DS]
  float* Ks = Qs + BM * DS;                        // [TK][DS]
  float* Vs = Ks + TK * DS;                        // [TK][DS]
  float* Ps = Vs + TK * DS;                        // [BM][TK + 1]
  __shared__ int s_tpos[TK];
  __shared__ int s_twin[TK];
  __shared__ int s_rowpos[BM];
  __shared__ int s_pminmax[2];

  const int tid = threadIdx.x;
  const int Gq = p.H / p.HKV;
  const int NBLK = cdiv(p.TQ, p.block_size_q);
  int64_t bid = blockIdx.x;
  const int split = (int)(bid % p.n_splits); bid /= p.n_splits;
  const int sub = (int)(bid % n_sub); bid /= n_sub;
  const int d = (int)(bid % NBLK); bid /= NBLK;
  const int hslot = (int)(bid % (packed ? p.HKV : p.H)); bid /= (packed ? p.HKV : p.H);
  const int b = (int)bid;
  const int h0 = packed ? hslot * Gq : hslot;
  const int hkv = packed ? hslot : hslot / Gq;

  const int blk_t0 = d * p.block_size_q;
  const int blk_rows = min(p.block_size_q, p.TQ - blk_t0);
  // rows of this tile: packed -> (head g, query row i) pairs; otherwise BM consecutive rows of one head
  const int n_rows = packed ? Gq * rows_per_head : max(0, min(BM, blk_rows - sub * BM));

  // block-wide smallest / largest position (over all rows of the attention block)
  if (tid == 0) { s_pminmax[0] = 0x7fffffff; s_pminmax[1] = -1; }
  __syncthreads();
  {
    int lo = 0x7fffffff, hi = -1;
    for (int i = tid; i < blk_rows; i += kThreads) {
      const long long pv = p.pos[(int64_t)b * p.pos_stride_b + (int64_t)(blk_t0 + i) * p.pos_stride_t];
      const int v = (int)(pv > 0x7ffffff0LL ? 0x7ffffff0LL : (pv < 0 ? 0 : pv));
      lo = min(lo, v); hi = max(hi, v);
    }
    if (hi >= 0) { atomicMin(&s_pminmax[0], lo); atomicMax(&s_pminmax[1], hi); }
  }
  for (int r = tid; r < BM; r += kThreads) {
    int pv = -0x40000000;  // rows beyond the tile admit nothing
    if (r < n_rows) {
      const int i = packed ? r % rows_per_head : sub * BM + r;
      const long long x = p.pos[(int64_t)b * p.pos_stride_b + (int64_t)(blk_t0 + i) * p.pos_stride_t];
      pv = (int)(x > 0x7ffffff0LL ? 0x7ffffff0LL : (x < 0 ? 0 : x));
    }
    s_rowpos[r] = pv;
  }
  // Q tile -> fp32
  for (int i = tid; i < BM * PIECES; i += kThreads) {
    const int r = i / PIECES, pc = i % PIECES;
    float v[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) v[e] = 0.f;
    if (r < n_rows) {
      const int hh = packed ? h0 + r / rows_per_head : h0;
      const int ti = blk_t0 + (packed ? r % rows_per_head : sub * BM + r);
      const T* qp = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_stride_b + (int64_t)ti * p.q_stride_t +
                    (int64_t)hh * p.q_stride_h + pc * VEC;
      widen16<DT>(*reinterpret_cast<const uint4*>(qp), v);
      if (p.rope_cos) {   // in-kernel RoPE: the query row at its own position (attention_extend_bsa.py:797-856)
        constexpr int HALF = PIECES / 2;
        float vr[VEC], tc[VEC], ts[VEC];
        widen16<DT>(*reinterpret_cast<const uint4*>(qp + (pc < HALF ? HALF : -HALF) * VEC), vr);
        const long long x = p.pos[(int64_t)b * p.pos_stride_b + (int64_t)ti * p.pos_stride_t];
        const int qpos = (int)(x > 0x7ffffff0LL ? 0x7ffffff0LL : (x < 0 ? 0 : x));
        rope_table_piece<DT>(p.rope_cos, p.rope_stride, p.rope_rows, qpos, pc % HALF, tc);
        rope_table_piece<DT>(p.rope_sin, p.rope_stride, p.rope_rows, qpos, pc % HALF, ts);
        rope_rotate_piece<DT, VEC>(v, vr, tc, ts, pc < HALF);
      }
    }
#pragma unroll
    for (int e = 0; e < VEC; e += 4)
      *reinterpret_cast<float4*>(Qs + r * DS + pc * VEC + e) = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
  }
  __syncthreads();
  const int pmin = s_pminmax[0], pmax = s_pminmax[1];
  const KeyList kl = make_key_list(p, b, h0, d, pmin, pmax);
  const int per = cdiv(cdiv(kl.total, p.n_splits), TK) * TK;
  const int j_begin = split * per, j_end = min(kl.total, j_begin + per);

  const int ty = tid / TPR, tx = tid % TPR;
  float m_run[RPT], l_run[RPT];
  float4 acc[RPT][NV];
  int prow[RPT];
#pragma unroll
  for (int r = 0; r < RPT; ++r) {
    m_run[r] = -INFINITY;
    l_run[r] = 0.f;
    prow[r] = s_rowpos[ty * RPT + r];
#pragma unroll
    for (int v = 0; v < NV; ++v) acc[r][v] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const float cap = p.logit_softcap;

  for (int j0 = j_begin; j0 < j_end; j0 += TK) {
    __syncthreads();  // previous tile fully consumed
    if (tid < TK) {
      bool w;
      const int j = j0 + tid;
      const int t = j < j_end ? key_position(kl, j, &w) : -1;
      s_tpos[tid] = t;
      s_twin[tid] = (t >= 0 && w) ? 1 : 0;
    }
    __syncthreads();
    for (int i = tid; i < TK * PIECES; i += kThreads) {
      const int kk = i / PIECES, pc = i % PIECES;
      const int t = s_tpos[kk];
      float kv[VEC], vv[VEC];
#pragma unroll
      for (int e = 0; e < VEC; ++e) kv[e] = vv[e] = 0.f;
      if (t >= 0) {
        const char* kr = token_row(p.k, b, t, hkv, Elem<DT>::bytes, p.status);
        const char* vr = token_row(p.v, b, t, hkv, Elem<DT>::bytes, p.status);
        constexpr int KDT = DT == HIPATTN_F32 ? HIPATTN_F16 : DT;   // (an fp8 cache is only accepted with 16-bit queries)
        const bool k8 = DT != HIPATTN_F32 && p.k.fp8_e5m2, v8 = DT != HIPATTN_F32 && p.v.fp8_e5m2;
        widen16<DT>(k8 ? widen_fp8_e5m2<KDT>(*reinterpret_cast<const uint2*>(kr + pc * 8)) : *reinterpret_cast<const uint4*>(kr + pc * 16), kv);
        widen16<DT>(v8 ? widen_fp8_e5m2<KDT>(*reinterpret_cast<const uint2*>(vr + pc * 8)) : *reinterpret_cast<const uint4*>(vr + pc * 16), vv);
        if (p.rope_cos) {   // in-kernel RoPE: the key at the position its place in the list maps to
          constexpr int HALF = PIECES / 2;
          float xr[VEC], tc[VEC], ts[VEC];
          const int pr = pc < HALF ? pc + HALF : pc - HALF;
          widen16<DT>(k8 ? widen_fp8_e5m2<KDT>(*reinterpret_cast<const uint2*>(kr + pr * 8)) : *reinterpret_cast<const uint4*>(kr + pr * 16), xr);
          const int new_t = rope_key_position(kl, j0 + kk, t, p.window);
          rope_table_piece<DT>(p.rope_cos, p.rope_stride, p.rope_rows, new_t, pc % HALF, tc);
          rope_table_piece<DT>(p.rope_sin, p.rope_stride, p.rope_rows, new_t, pc % HALF, ts);
          rope_rotate_piece<DT, VEC>(kv, xr, tc, ts, pc < HALF);
        }
      }
#pragma unroll
      for (int e = 0; e < VEC; e += 4) {
        *reinterpret_cast<float4*>(Ks + kk * DS + pc * VEC + e) = make_float4(kv[e], kv[e + 1], kv[e + 2], kv[e + 3]);
        *reinterpret_cast<float4*>(Vs + kk * DS + pc * VEC + e) = make_float4(vv[e], vv[e + 1], vv[e + 2], vv[e + 3]);
      }
    }
    __syncthreads();

    // S = Q K^T for rows {ty * RPT + r}, keys {tx + TPR * c}
    float s[RPT][TPT];
#pragma unroll
    for (int r = 0; r < RPT; ++r)
#pragma unroll
      for (int c = 0; c < TPT; ++c) s[r][c] = 0.f;
#pragma unroll 4
    for (int e = 0; e < D; e += 4) {
      float4 qv[RPT], kv[TPT];
#pragma unroll
      for (int r = 0; r < RPT; ++r) qv[r] = *reinterpret_cast<const float4*>(Qs + (ty * RPT + r) * DS + e);
#pragma unroll
      for (int c = 0; c < TPT; ++c) kv[c] = *reinterpret_cast<const float4*>(Ks + (tx + TPR * c) * DS + e);
#pragma unroll
      for (int r = 0; r < RPT; ++r)
#pragma unroll
        for (int c = 0; c < TPT; ++c) {
          s[r][c] = fmaf(qv[r].x, kv[c].x, s[r][c]);
          s[r][c] = fmaf(qv[r].y, kv[c].y, s[r][c]);
          s[r][c] = fmaf(qv[r].z, kv[c].z, s[r][c]);
          s[r][c] = fmaf(qv[r].w, kv[c].w, s[r][c]);
        }
    }
    // mask, online softmax (base 2)
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < TPT; ++c) {
        const int kk = tx + TPR * c;
        float x = s[r][c];
        if (cap > 0.f) x = tanhf(x / cap) * cap;
        x *= kLog2e;
        if (!admits(prow[r], s_tpos[kk], s_twin[kk] != 0, p.window)) x = -INFINITY;
        s[r][c] = x;
        mx = fmaxf(mx, x);
      }
#pragma unroll
      for (int o = TPR >> 1; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_new = fmaxf(m_run[r], mx);
      float sum = 0.f;
      float alpha = 1.f;
      if (m_new > -INFINITY) {
        alpha = exp2f(m_run[r] - m_new);  // exp2(-inf) = 0 on the first admitted tile
#pragma unroll
        for (int c = 0; c < TPT; ++c) {
          const float pe = exp2f(s[r][c] - m_new);
          s[r][c] = pe;
          sum += pe;
        }
      } else {
#pragma unroll
        for (int c = 0; c < TPT; ++c) s[r][c] = 0.f;
      }
#pragma unroll
      for (int o = TPR >> 1; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      l_run[r] = l_run[r] * alpha + sum;
      m_run[r] = m_new;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        acc[r][v].x *= alpha; acc[r][v].y *= alpha; acc[r][v].z *= alpha; acc[r][v].w *= alpha;
      }
#pragma unroll
      for (int c = 0; c < TPT; ++c) Ps[(ty * RPT + r) * (TK + 1) + tx + TPR * c] = s[r][c];
    }
    __syncthreads();
    // O += P V for rows {ty * RPT + r}, columns {(tx + TPR * v) * 4 .. + 3}
#pragma unroll 4
    for (int kk = 0; kk < TK; ++kk) {
      float pr[RPT];
#pragma unroll
      for (int r = 0; r < RPT; ++r) pr[r] = Ps[(ty * RPT + r) * (TK + 1) + kk];
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const float4 vv = *reinterpret_cast<const float4*>(Vs + kk * DS + (tx + TPR * v) * 4);
#pragma unroll
        for (int r = 0; r < RPT; ++r) {
          acc[r][v].x = fmaf(pr[r], vv.x, acc[r][v].x);
          acc[r][v].y = fmaf(pr[r], vv.y, acc[r][v].y);
          acc[r][v].z = fmaf(pr[r], vv.z, acc[r][v].z);
          acc[r][v].w = fmaf(pr[r], vv.w, acc[r][v].w);
        }
      }
    }
  }

  // epilogue
#pragma unroll
  for (int r = 0; r < RPT; ++r) {
    const int row = ty * RPT + r;
    if (row >= n_rows) continue;
    const int hh = packed ? h0 + row / rows_per_head : h0;
    const int ti = blk_t0 + (packed ? row % rows_per_head : sub * BM + row);
    const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
    const float lse = l_run[r] > 0.f ? m_run[r] + log2f(l_run[r]) : -INFINITY;
    if (p.n_splits > 1) {
      const int64_t o = ((int64_t)b * p.H + hh) * p.n_splits + split;
      if (tx == 0) p.part_lse[o] = lse;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        float4 x = acc[r][v];
        x.x *= inv; x.y *= inv; x.z *= inv; x.w *= inv;
        *reinterpret_cast<float4*>(p.part_o + o * D + (tx + TPR * v) * 4) = x;
      }
    } else {
      if (p.lse_out && tx == 0) p.lse_out[((int64_t)b * p.TQ + ti) * p.H + hh] = lse;
      T* op = reinterpret_cast<T*>(p.out) + (int64_t)b * p.o_stride_b + (int64_t)ti * p.o_stride_t + (int64_t)hh * p.o_stride_h;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const int c0 = (tx + TPR * v) * 4;
        op[c0 + 0] = Elem<DT>::from_f32(acc[r][v].x * inv);
        op[c0 + 1] = Elem<DT>::from_f32(acc[r][v].y * inv);
        op[c0 + 2] = Elem<DT>::from_f32(acc[r][v].z * inv);
        op[c0 + 3] = Elem<DT>::from_f32(acc[r][v].w * inv);
      }
    }
  }
}

template <int DT, int D, int BM>
int launch(const hipattn_bsa_params_t& p, int packed, int rows_per_head, int n_sub, cudaStream_t stream) {
  constexpr int DS = D + 4;
  const size_t smem = sizeof(float) * ((size_t)BM * DS + 2 * TK * DS + (size_t)BM * (TK + 1));
  const int NBLK = cdiv(p.TQ, p.block_size_q);
  const int64_t grid = (int64_t)p.B * (packed ? p.HKV : p.H) * NBLK * n_sub * p.n_splits;
  HIPATTN_REQUIRE(grid > 0 && grid < 0x7fffffffLL, HIPATTN_ERR_INVALID, "attention grid of %lld blocks", (long long)grid);
  auto kern = bsa_generic_kernel<DT, D, BM>;
  HIPATTN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<(unsigned)grid, kThreads, smem, stream>>>(p, packed, rows_per_head, n_sub);
  return check_launch("bsa_generic_kernel");
}

template <int DT, int D>
int dispatch_tile(const hipattn_bsa_params_t& p, cudaStream_t stream) {
  const int Gq = p.H / p.HKV;
  const int rows_in_block = p.TQ < p.block_size_q ? p.TQ : p.block_size_q;
  // pack the heads of a KV group into one tile when the whole group fits and shares its key list
  if (p.heads_share_mask && p.TQ <= p.block_size_q && Gq * rows_in_block <= 16)
    return launch<DT, D, 16>(p, 1, rows_in_block, 1, stream);
  if (p.heads_share_mask && p.TQ <= p.block_size_q && Gq * rows_in_block <= 64)
    return launch<DT, D, 64>(p, 1, rows_in_block, 1, stream);
  HIPATTN_REQUIRE(p.n_splits == 1, HIPATTN_ERR_INVALID, "attention: key splits need one query row per head");
  if (rows_in_block <= 16) return launch<DT, D, 16>(p, 0, 0, 1, stream);
  return launch<DT, D, 64>(p, 0, 0, cdiv(p.block_size_q, 64), stream);
}

template <int DT>
int dispatch_dim(const hipattn_bsa_params_t& p, cudaStream_t stream) {
  switch (p.D) {
    case 64: return dispatch_tile<DT, 64>(p, stream);
    case 128: return dispatch_tile<DT, 128>(p, stream);
    case 256: return dispatch_tile<DT, 256>(p, stream);
    default:
      set_error("attention: head dimension %d is not built (64, 128, 256)", p.D);
      return HIPATTN_ERR_UNSUPPORTED;
  }
}

}  // namespace

int bsa_generic(const hipattn_bsa_params_t& p, cudaStream_t stream) {
  switch (p.dtype) {
    case HIPATTN_F32: return dispatch_dim<HIPATTN_F32>(p, stream);
    case HIPATTN_F16: return dispatch_dim<HIPATTN_F16>(p, stream);
    case HIPATTN_BF16: return dispatch_dim<HIPATTN_BF16>(p, stream);
    default: set_error("attention: unknown dtype %d", p.dtype); return HIPATTN_ERR_INVALID;
  }
}

}  // namespace hipattn
