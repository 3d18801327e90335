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
#include "mma_common.cuh"

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
__global__ void __launch_bounds__(kWarps * 32, 1) bsa_decode_kernel(const hipattn_bsa_params_t p) {
  using T = typename Elem<DT>::type;
  constexpr int VEC = 16 / Elem<DT>::bytes;
  constexpr int D = LPR * VEC;
  constexpr int TPP = 32 / LPR;                      // keys per pass (one 16-byte load per lane)
  constexpr int PBMAX = G > 4 ? 8 : 16;              // bounds the rows a lane keeps in flight (registers)
  constexpr int PB = LPR < PBMAX ? LPR : PBMAX;      // passes per group
  constexpr int GK = PB * TPP;                       // keys per group (<= 32)

  __shared__ unsigned long long s_kptr[kWarps][2][32];
  __shared__ unsigned long long s_vptr[kWarps][2][32];
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
  const int per = cdiv(cdiv(kl.total, p.n_splits), GK) * GK;
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

  // resolve the list entries of one group to row addresses (0 = not admitted)
  auto resolve = [&](int j0, int buf) {
    unsigned long long ka = 0, va = 0;
    const int j = j0 + lane;
    if (lane < GK && j < j_end) {
      bool w = false;
      const int t = key_position(kl, j, &w);
      if (admits(pq, t, w, p.window)) {
        ka = (unsigned long long)token_row(p.k, b, t, hkv, Elem<DT>::bytes, p.status);
        va = (unsigned long long)token_row(p.v, b, t, hkv, Elem<DT>::bytes, p.status);
      }
    }
    s_kptr[warp][buf][lane] = ka;
    s_vptr[warp][buf][lane] = va;
  };
  auto load_rows = [&](const unsigned long long* ptrs, uint4* regs) {
#pragma unroll
    for (int i = 0; i < PB; ++i) {
      const unsigned long long a = ptrs[i * TPP + sub];
      regs[i] = a != 0ull ? ldg_nc16((const char*)a + piece * 16) : make_uint4(0, 0, 0, 0);
    }
  };

  // software pipeline over groups: K rows of group i + 1 and V rows of group i are in flight while
  // group i is soft-maxed; addresses are resolved one group ahead
  const int stride = kWarps * GK;
  int j0 = j_begin + warp * GK;
  uint4 kw[PB], vw[PB];
  int buf = 0;
  if (j0 < j_end) {
    resolve(j0, 0);
    __syncwarp();
    load_rows(s_kptr[warp][0], kw);
  }
  for (; j0 < j_end; j0 += stride, buf ^= 1) {
    const bool more = j0 + stride < j_end;
    if (more) resolve(j0 + stride, buf ^ 1);
    load_rows(s_vptr[warp][buf], vw);
    // ---- logits: the key of pass r, slot sub ends up in lane sub * LPR + r ----
    float s[G];
#pragma unroll
    for (int g = 0; g < G; ++g) s[g] = -INFINITY;
#pragma unroll
    for (int i = 0; i < PB; ++i) {
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
      if (piece == i && s_kptr[warp][buf][i * TPP + sub] != 0ull) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
          float x = part[g];
          if (cap > 0.f) x = tanhf(x / cap) * cap;
          s[g] = x * kLog2e;
        }
      }
    }
    __syncwarp();
    if (more) load_rows(s_kptr[warp][buf ^ 1], kw);
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
    for (int i = 0; i < PB; ++i) {
      float vv[VEC];
      widen16<DT>(vw[i], vv);
      const int keeper = sub * LPR + i;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float pg = __shfl_sync(0xffffffffu, pr[g], keeper);
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[g][e] = fmaf(pg, vv[e], acc[g][e]);
      }
    }
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

// ---------------------------------------------------------------------------------------------------
// 16-bit types: tensor-core variant.  The G heads of the KV group are the rows of a 16-row MMA tile;
// a tile of 64 keys is split over the 4 warps (16 keys each), every warp keeping its own running
// maximum, sum and output, merged at the end.  K / V rows are gathered with 16-byte cp.async into a
// three-stage ring of swizzled tiles, addresses resolved one tile further ahead by 64 threads.
// ---------------------------------------------------------------------------------------------------
constexpr int TKD = 64;      // keys per tile
constexpr int kStages = 3;

struct DecodeMeta {
  long long koff[TKD];  // byte offsets from the base pointers, -1 = key not admitted
  long long voff[TKD];
  int rpos[TKD];        // in-kernel RoPE: table position the key is rotated to (-1: no key)
};

template <int DT, int D>
__global__ void __launch_bounds__(128) bsa_decode_mma_kernel(const hipattn_bsa_params_t p) {
  using T = typename Elem<DT>::type;
  constexpr int PIECES = D / 8;
  constexpr int KSTEPS = D / 16;
  constexpr int NO = D / 8;
  constexpr int TILE_BYTES = TKD * D * 2;
  constexpr int MS = D + 2;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* sQ = smem;                                   // [16][D]
  unsigned char* sK = sQ + 16 * D * 2;                        // kStages x [TKD][D]
  unsigned char* sV = sK + kStages * TILE_BYTES;              // kStages x [TKD][D]
  DecodeMeta* meta = reinterpret_cast<DecodeMeta*>(sV + kStages * TILE_BYTES);  // kStages + 1 entries
  float* s_merge = reinterpret_cast<float*>(sK);              // reused after the last tile: [4][16][MS]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.H / p.HKV;
  int64_t bid = blockIdx.x;
  const int split = (int)(bid % p.n_splits); bid /= p.n_splits;
  const int hkv = (int)(bid % p.HKV); bid /= p.HKV;
  const int b = (int)bid;
  const int h0 = hkv * G;

  const long long px = p.pos[(int64_t)b * p.pos_stride_b];
  const int pq = (int)(px > 0x7ffffff0LL ? 0x7ffffff0LL : (px < 0 ? 0 : px));
  const KeyList kl = make_key_list(p, b, h0, 0, pq, pq);
  const int per = cdiv(cdiv(kl.total, p.n_splits), TKD) * TKD;
  const int j_begin = split * per, j_end = min(kl.total, j_begin + per);
  const int n_tiles = j_end > j_begin ? cdiv(j_end - j_begin, TKD) : 0;

  for (int i = tid; i < 16 * PIECES; i += 128) {
    const int r = i / PIECES, pc = i % PIECES;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < G) {
      const T* qp = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_stride_b + (int64_t)(h0 + r) * p.q_stride_h + pc * 8;
      v = *reinterpret_cast<const uint4*>(qp);
    }
    *reinterpret_cast<uint4*>(sQ + swz<D>(r, pc)) = v;
  }
  const char* kbase = (const char*)(p.k.cache ? p.k.cache : p.k.dense);
  const char* vbase = (const char*)(p.v.cache ? p.v.cache : p.v.dense);

  auto make_meta = [&](int tile) {
    if (tid < TKD) {
      DecodeMeta& m = meta[tile % (kStages + 1)];
      const int j = j_begin + tile * TKD + tid;
      long long ko = -1, vo = -1;
      int rp = -1;
      if (j < j_end) {
        bool w = false;
        const int t = key_position(kl, j, &w);
        if (admits(pq, t, w, p.window)) {
          ko = token_row(p.k, b, t, hkv, 2, p.status) - kbase;
          vo = token_row(p.v, b, t, hkv, 2, p.status) - vbase;
          if (p.rope_cos) rp = rope_key_position(kl, j, t, p.window);
        }
      }
      m.koff[tid] = ko;
      m.voff[tid] = vo;
      m.rpos[tid] = rp;
    }
  };
  auto gather = [&](int tile) {
    const DecodeMeta& m = meta[tile % (kStages + 1)];
    unsigned char* kb = sK + (tile % kStages) * TILE_BYTES;
    unsigned char* vb = sV + (tile % kStages) * TILE_BYTES;
    // the offsets of this thread's rows are read first and the copies follow without a branch between them: a row that
    // the query does not admit (offset -1) is a copy of zero source bytes, which fills its sixteen bytes with zeros
    constexpr int N = TKD * PIECES / 128;
    static_assert(TKD * PIECES % 128 == 0, "a tile is a whole number of copies per thread");
    long long ko[N], vo[N];
#pragma unroll
    for (int n = 0; n < N; ++n) {
      const int r = (tid + n * 128) / PIECES;
      ko[n] = m.koff[r];
      vo[n] = m.voff[r];
    }
    const uint32_t kb_s = (uint32_t)__cvta_generic_to_shared(kb), vb_s = (uint32_t)__cvta_generic_to_shared(vb);
#pragma unroll
    for (int n = 0; n < N; ++n) {
      const int i = tid + n * 128, r = i / PIECES, pc = i % PIECES;
      const bool live = ko[n] >= 0;
      cp_async16_zfill(kb_s + swz<D>(r, pc), kbase + (live ? ko[n] : 0) + pc * 16, live);
      cp_async16_zfill(vb_s + swz<D>(r, pc), vbase + (live ? vo[n] : 0) + pc * 16, live);
    }
  };

  if (n_tiles > 0) make_meta(0);
  if (n_tiles > 1) make_meta(1);
  __syncthreads();  // Q tile and the first addresses are visible
  if (p.rope_cos) {   // in-kernel RoPE: the query rows at the query's position (attention_decode_bsa.py:174-215)
    rope_rotate_tile<DT, D>(sQ, 0, 16, p, tid, 128, [&](int r) { return r < G ? pq : -1; });
    __syncthreads();
  }
  uint32_t qf[KSTEPS][4];
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks)
    ldsm_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], sQ + swz<D>(lane & 15, ks * 2 + (lane >> 4)));
  if (n_tiles > 0) gather(0);
  cp_async_commit();
  if (n_tiles > 1) gather(1);
  cp_async_commit();
  if (n_tiles > 2) make_meta(2);

  float o[NO][2];
#pragma unroll
  for (int i = 0; i < NO; ++i) o[i][0] = o[i][1] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  const float cap = p.logit_softcap;

  for (int it = 0; it < n_tiles; ++it) {
    cp_async_wait<1>();
    __syncthreads();  // tile `it` landed; addresses of tile it + 2 visible; ring slot of tile it - 1 is free
    if (it + 2 < n_tiles) gather(it + 2);
    cp_async_commit();
    if (it + 3 < n_tiles) make_meta(it + 3);

    const DecodeMeta& mt = meta[it % (kStages + 1)];
    if (p.rope_cos) {   // in-kernel RoPE: this warp rotates the 16 key rows it is about to multiply
      rope_rotate_tile<DT, D>(sK + (it % kStages) * TILE_BYTES, warp * 16, 16, p, lane, 32, [&](int r) { return mt.rpos[r]; });
      __syncwarp();
    }
    const unsigned char* kb = sK + (it % kStages) * TILE_BYTES;
    const unsigned char* vb = sV + (it % kStages) * TILE_BYTES;
    // ---- S = Q K^T for this warp's 16 keys ----
    float s[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      uint32_t b0, b1, b2, b3;
      const int krow = warp * 16 + (lane & 7) + ((lane >> 4) << 3);
      const int kpc = ks * 2 + ((lane >> 3) & 1);
      ldsm_x4(b0, b1, b2, b3, kb + swz<D>(krow, kpc));
      mma16816<DT>(s[0], qf[ks], b0, b1);
      mma16816<DT>(s[1], qf[ks], b2, b3);
    }
    // ---- admission + online softmax (rows lane / 4 < G; rows 8..15 are padding) ----
    float mx = -INFINITY;
    if (cap > 0.f) {   // soft-cap behind its own uniform branch: inside the loop the tanh is evaluated under a predicate
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) s[nt][e] = tanhf(s[nt][e] / cap) * cap;
      }
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float x = s[nt][e];
        x *= kLog2e;
        const int col = warp * 16 + nt * 8 + (lane & 3) * 2 + e;
        if (mt.koff[col] < 0) x = -INFINITY;
        s[nt][e] = x;
        mx = fmaxf(mx, x);
      }
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);
    const float base = m_new > -INFINITY ? m_new : 0.f;
    const float alpha = exp2f(m_run - base);
    float sum = 0.f;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      s[nt][0] = exp2f(s[nt][0] - base);
      s[nt][1] = exp2f(s[nt][1] - base);
      sum += s[nt][0] + s[nt][1];
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    l_run = l_run * alpha + sum;
    m_run = m_new;
#pragma unroll
    for (int i = 0; i < NO; ++i) { o[i][0] *= alpha; o[i][1] *= alpha; }
    // ---- O += P V over this warp's 16 keys ----
    uint32_t pa[4];
    pa[0] = pack2<DT>(s[0][0], s[0][1]);
    pa[1] = 0u;
    pa[2] = pack2<DT>(s[1][0], s[1][1]);
    pa[3] = 0u;
#pragma unroll
    for (int np = 0; np < NO / 2; ++np) {
      uint32_t b0, b1, b2, b3;
      const int vrow = warp * 16 + (lane & 15);
      const int vpc = np * 2 + (lane >> 4);
      ldsm_x4_t(b0, b1, b2, b3, vb + swz<D>(vrow, vpc));
      float c0[4] = {o[np * 2][0], o[np * 2][1], 0.f, 0.f};
      float c1[4] = {o[np * 2 + 1][0], o[np * 2 + 1][1], 0.f, 0.f};
      mma16816<DT>(c0, pa, b0, b1);
      mma16816<DT>(c1, pa, b2, b3);
      o[np * 2][0] = c0[0]; o[np * 2][1] = c0[1];
      o[np * 2 + 1][0] = c1[0]; o[np * 2 + 1][1] = c1[1];
    }
  }
  cp_async_wait<0>();
  __syncthreads();  // every warp is done with the ring before it is reused for the merge

  // ---- merge the four warps ----
  {
    const int r = lane >> 2;
    if (r < G) {
      float* dst = s_merge + ((size_t)warp * 16 + r) * MS;
#pragma unroll
      for (int nt = 0; nt < NO; ++nt) {
        dst[nt * 8 + (lane & 3) * 2] = o[nt][0];
        dst[nt * 8 + (lane & 3) * 2 + 1] = o[nt][1];
      }
      if ((lane & 3) == 0) { dst[D] = m_run; dst[D + 1] = l_run; }
    }
  }
  __syncthreads();
  for (int i = tid; i < G * D; i += 128) {
    const int g = i / D, e = i % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, s_merge[((size_t)w * 16 + g) * MS + D]);
    float num = 0.f, den = 0.f;
    if (M > -INFINITY) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float* src = s_merge + ((size_t)w * 16 + g) * MS;
        const float f = exp2f(src[D] - M);
        num += f * src[e];
        den += f * src[D + 1];
      }
    }
    const float val = den > 0.f ? num / den : 0.f;
    const float lse = den > 0.f ? M + log2f(den) : -INFINITY;
    const int hh = h0 + g;
    if (p.n_splits > 1) {
      const int64_t oo = ((int64_t)b * p.H + hh) * p.n_splits + split;
      p.part_o[oo * D + e] = val;
      if (e == 0) p.part_lse[oo] = lse;
    } else {
      reinterpret_cast<T*>(p.out)[(int64_t)b * p.o_stride_b + (int64_t)hh * p.o_stride_h + e] = Elem<DT>::from_f32(val);
      if (e == 0 && p.lse_out) p.lse_out[(int64_t)b * p.H + hh] = lse;
    }
  }
}

template <int DT, int D>
int launch_mma(const hipattn_bsa_params_t& p, cudaStream_t stream) {
  const size_t smem = 16 * D * 2 + 2 * (size_t)kStages * TKD * D * 2 + (kStages + 1) * sizeof(DecodeMeta);
  const int64_t grid = (int64_t)p.B * p.HKV * p.n_splits;
  HIPATTN_REQUIRE(grid > 0 && grid < 0x7fffffffLL, HIPATTN_ERR_INVALID, "decode grid of %lld blocks", (long long)grid);
  auto kern = bsa_decode_mma_kernel<DT, D>;
  HIPATTN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<(unsigned)grid, 128, smem, stream>>>(p);
  return check_launch("bsa_decode_mma_kernel");
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
  const int G = p.H / p.HKV;
  if (p.dtype != HIPATTN_F32 && G <= 8 && (p.D == 64 || p.D == 128)) {
    *handled = true;
    if (p.dtype == HIPATTN_BF16) return p.D == 128 ? launch_mma<HIPATTN_BF16, 128>(p, stream) : launch_mma<HIPATTN_BF16, 64>(p, stream);
    return p.D == 128 ? launch_mma<HIPATTN_F16, 128>(p, stream) : launch_mma<HIPATTN_F16, 64>(p, stream);
  }
  if (p.rope_cos) return HIPATTN_OK;   // in-kernel RoPE: only the tensor-core variant above rotates; the rest is the general kernel's
  switch (p.dtype) {
    case HIPATTN_F32: return dispatch_row<HIPATTN_F32>(p, stream, handled);
    case HIPATTN_F16: return dispatch_row<HIPATTN_F16>(p, stream, handled);
    case HIPATTN_BF16: return dispatch_row<HIPATTN_BF16>(p, stream, handled);
    default: return HIPATTN_OK;
  }
}

}  // namespace hipattn
