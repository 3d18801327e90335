// Block-sparse attention, decode (one query row per sequence): bandwidth-bound split-KV kernel.
//
// One CTA owns (batch, KV head, key range).  The G query heads of the KV group share every K / V row
// that is fetched.  A warp walks its part of the key list 32 keys at a time:
//   lanes resolve 32 list entries to positions, admission and row addresses (page-table lookups);
//   K rows are read with 16-byte loads, LPR lanes per row (a 256-byte row = 16 lanes), several rows
//   in flight per lane; partial dot products are reduced inside the LPR-lane group;
//   the 32 x G logits are soft-maxed as one group (base 2, running maximum per head);
//   V rows are read the same way and accumulated with the probabilities.
// Warps are merged through shared memory; the CTA writes either the final rows (one range) or a
// normalised partial output with its base-2 log-sum-exp (several ranges, merged by merge_kernel).
#include "bsa_common.cuh"

namespace hipattn {
namespace {

constexpr int kWarps = 8;
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
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v[i]));
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}

__device__ __forceinline__ uint4 ldg_nc16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// LPR = lanes per K / V row (row bytes / 16), G = query heads per KV head
template <int DT, int LPR, int G>
__global__ void __launch_bounds__(kWarps * 32) bsa_decode_kernel(const hipattn_bsa_params_t p) {
  using T = typename Elem<DT>::type;
  constexpr int VEC = 16 / Elem<DT>::bytes;
  constexpr int D = LPR * VEC;
  constexpr int TPP = 32 / LPR;        // keys per pass
  constexpr int NPASS = 32 / TPP;      // passes per group of 32 keys
  constexpr int BATCH = NPASS < 8 ? NPASS : 8;

  __shared__ unsigned long long s_kptr[kWarps][32];
  __shared__ unsigned long long s_vptr[kWarps][32];
  extern __shared__ __align__(16) float s_merge[];  // [kWarps][G][D + 2]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPR, piece = lane % LPR;  // key within a pass, 16-byte piece of the row
  int64_t bid = blockIdx.x;
  const int split = (int)(bid % p.n_splits); bid /= p.n_splits;
  const int hkv = (int)(bid % p.HKV); bid /= p.HKV;
  const int b = (int)bid;
  const int h0 = hkv * G;

  const long long px = p.pos[(int64_t)b * p.pos_stride_b];
  const int pq = (int)(px > 0x7ffffff0LL ? 0x7ffffff0LL : (px < 0 ? 0 : px));
  const KeyList kl = make_key_list(p, b, h0, 0, pq, pq);
  const int per = cdiv(cdiv(kl.total, p.n_splits), 32) * 32;
  const int j_begin = split * per, j_end = min(kl.total, j_begin + per);

  // this lane's slice of the G query rows
  float q[G][VEC];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const T* qp = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_stride_b + (int64_t)(h0 + g) * p.q_stride_h + piece * VEC;
    widen16<DT>(*reinterpret_cast<const uint4*>(qp), q[g]);
  }
  float m_run[G], l_run[G], acc[G][VEC];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m_run[g] = -INFINITY;
    l_run[g] = 0.f;
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[g][e] = 0.f;
  }
  const float cap = p.logit_softcap;

  for (int j0 = j_begin + warp * 32; j0 < j_end; j0 += kWarps * 32) {
    // ---- resolve 32 list entries ----
    {
      const int j = j0 + lane;
      bool w = false;
      const int t = j < j_end ? key_position(kl, j, &w) : -1;
      unsigned long long ka = 0, va = 0;
      if (admits(pq, t, w, p.window)) {
        ka = (unsigned long long)token_row(p.k, b, t, hkv, Elem<DT>::bytes, p.status);
        va = (unsigned long long)token_row(p.v, b, t, hkv, Elem<DT>::bytes, p.status);
      }
      s_kptr[warp][lane] = ka;
      s_vptr[warp][lane] = va;
    }
    __syncwarp();
    // ---- logits: lane (r + sub * NPASS ... ) layout: key r * TPP + sub ends up in lane sub * NPASS + r ----
    float s[G];
#pragma unroll
    for (int g = 0; g < G; ++g) s[g] = -INFINITY;
#pragma unroll
    for (int r0 = 0; r0 < NPASS; r0 += BATCH) {
      uint4 kw[BATCH];
      bool ok[BATCH];
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        const unsigned long long a = s_kptr[warp][(r0 + i) * TPP + sub];
        ok[i] = a != 0ull;
        kw[i] = ok[i] ? ldg_nc16((const char*)a + piece * 16) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        float kv[VEC];
        widen16<DT>(kw[i], kv);
        float part[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
          float a = 0.f;
#pragma unroll
          for (int e = 0; e < VEC; ++e) a = fmaf(q[g][e], kv[e], a);
          part[g] = a;
        }
#pragma unroll
        for (int o = LPR >> 1; o > 0; o >>= 1) {
#pragma unroll
          for (int g = 0; g < G; ++g) part[g] += __shfl_xor_sync(0xffffffffu, part[g], o);
        }
        if (piece == ((r0 + i) % LPR) && ok[i]) {
          // NPASS == LPR * (NPASS / LPR); with TPP * LPR = 32 and NPASS = LPR the keeper is lane sub * LPR + pass
#pragma unroll
          for (int g = 0; g < G; ++g) {
            float x = part[g];
            if (cap > 0.f) x = tanhf(x / cap) * cap;
            s[g] = x * kLog2e;
          }
        }
      }
    }
    // ---- group softmax ----
    float pr[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float mx = s[g];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_new = fmaxf(m_run[g], mx);
      float alpha = 1.f;
      pr[g] = 0.f;
      if (m_new > -INFINITY) {
        alpha = exp2f(m_run[g] - m_new);
        pr[g] = exp2f(s[g] - m_new);
      }
      float sum = pr[g];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      l_run[g] = l_run[g] * alpha + sum;
      m_run[g] = m_new;
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[g][e] *= alpha;
    }
    // ---- O += P V ----
#pragma unroll
    for (int r0 = 0; r0 < NPASS; r0 += BATCH) {
      uint4 vw[BATCH];
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        const unsigned long long a = s_vptr[warp][(r0 + i) * TPP + sub];
        vw[i] = a != 0ull ? ldg_nc16((const char*)a + piece * 16) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        float vv[VEC];
        widen16<DT>(vw[i], vv);
        const int keeper = sub * LPR + ((r0 + i) % LPR);
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float pg = __shfl_sync(0xffffffffu, pr[g], keeper);
#pragma unroll
          for (int e = 0; e < VEC; ++e) acc[g][e] = fmaf(pg, vv[e], acc[g][e]);
        }
      }
    }
    __syncwarp();
  }

  // ---- combine the TPP key slots of a warp (same maxima), then the warps ----
#pragma unroll
  for (int o = LPR; o < 32; o <<= 1) {
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[g][e] += __shfl_xor_sync(0xffffffffu, acc[g][e], o);
  }
  constexpr int MS = D + 2;
  if (sub == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float* dst = s_merge + ((size_t)warp * G + g) * MS;
#pragma unroll
      for (int e = 0; e < VEC; ++e) dst[piece * VEC + e] = acc[g][e];
      if (piece == 0) { dst[D] = m_run[g]; dst[D + 1] = l_run[g]; }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += kWarps * 32) {
    const int g = i / D, e = i % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) M = fmaxf(M, s_merge[((size_t)w * G + g) * MS + D]);
    float num = 0.f, den = 0.f;
    if (M > -INFINITY) {
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const float* src = s_merge + ((size_t)w * G + g) * MS;
        const float f = exp2f(src[D] - M);
        num += f * src[e];
        den += f * src[D + 1];
      }
    }
    const float val = den > 0.f ? num / den : 0.f;
    const float lse = den > 0.f ? M + log2f(den) : -INFINITY;
    const int hh = h0 + g;
    if (p.n_splits > 1) {
      const int64_t o = ((int64_t)b * p.H + hh) * p.n_splits + split;
      p.part_o[o * D + e] = val;
      if (e == 0) p.part_lse[o] = lse;
    } else {
      reinterpret_cast<T*>(p.out)[(int64_t)b * p.o_stride_b + (int64_t)hh * p.o_stride_h + e] = Elem<DT>::from_f32(val);
      if (e == 0 && p.lse_out) p.lse_out[(int64_t)b * p.H + hh] = lse;
    }
  }
}

template <int DT, int LPR, int G>
int launch(const hipattn_bsa_params_t& p, cudaStream_t stream) {
  constexpr int D = LPR * (16 / Elem<DT>::bytes);
  const size_t smem = sizeof(float) * (size_t)kWarps * G * (D + 2);
  const int64_t grid = (int64_t)p.B * p.HKV * p.n_splits;
  HIPATTN_REQUIRE(grid > 0 && grid < 0x7fffffffLL, HIPATTN_ERR_INVALID, "decode grid of %lld blocks", (long long)grid);
  auto kern = bsa_decode_kernel<DT, LPR, G>;
  HIPATTN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<(unsigned)grid, kWarps * 32, smem, stream>>>(p);
  return check_launch("bsa_decode_kernel");
}

template <int DT, int LPR>
int dispatch_group(const hipattn_bsa_params_t& p, cudaStream_t stream, bool* handled) {
  *handled = true;
  switch (p.H / p.HKV) {
    case 1: return launch<DT, LPR, 1>(p, stream);
    case 2: return launch<DT, LPR, 2>(p, stream);
    case 4: return launch<DT, LPR, 4>(p, stream);
    case 8: return launch<DT, LPR, 8>(p, stream);
    default: *handled = false; return HIPATTN_OK;
  }
}

template <int DT>
int dispatch_row(const hipattn_bsa_params_t& p, cudaStream_t stream, bool* handled) {
  const int lpr = p.D * Elem<DT>::bytes / 16;
  switch (lpr) {
    case 8: return dispatch_group<DT, 8>(p, stream, handled);
    case 16: return dispatch_group<DT, 16>(p, stream, handled);
    case 32: return dispatch_group<DT, 32>(p, stream, handled);
    default: return HIPATTN_OK;
  }
}

}  // namespace

// Decode shapes: one query row, 1 / 2 / 4 / 8 query heads per KV head, K / V rows of 128, 256 or 512 bytes.
int bsa_decode(const hipattn_bsa_params_t& p, cudaStream_t stream, bool* handled) {
  *handled = false;
  if (p.TQ != 1) return HIPATTN_OK;
  switch (p.dtype) {
    case HIPATTN_F32: return dispatch_row<HIPATTN_F32>(p, stream, handled);
    case HIPATTN_F16: return dispatch_row<HIPATTN_F16>(p, stream, handled);
    case HIPATTN_BF16: return dispatch_row<HIPATTN_BF16>(p, stream, handled);
    default: return HIPATTN_OK;
  }
}

}  // namespace hipattn
