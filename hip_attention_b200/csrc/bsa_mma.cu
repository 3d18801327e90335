// Block-sparse attention, prefill, 16-bit element types: warp-level tensor-core kernel.
//
// One CTA owns M = 64 or 128 query rows: one attention block of 128 rows, or two heads of a KV group
// x 64 rows (all heads of a batch element share the selected blocks, so both heads consume every
// gathered K / V tile), or a single 64-row block.  The key list [sink | selected blocks | window] is
// walked in tiles of 64 keys.  K and V rows are gathered with 16-byte cp.async through the page table
// (or from the dense tensor) into XOR-swizzled shared memory, double buffered; row offsets of a tile
// are computed once by 64 threads.  S = Q K^T and O += P V use mma.sync m16n8k16 with fp32
// accumulators; Q fragments live in registers; softmax is online in base 2; tiles whose keys are
// admitted for every row skip the per-element admission test.
#include "bsa_common.cuh"
#include "mma_common.cuh"
#include "rope.cuh"

namespace hipattn {
namespace {

constexpr int TKM = 64;  // keys per tile
constexpr float kLog2e = 1.4426950408889634f;

struct TileMeta {
  int tpos[TKM];       // key position, -1 = not admitted for any row
  int twin[TKM];       // 1 = window rule, 0 = far rule
  long long koff[TKM]; // byte offset of the K row from the K base pointer
  long long voff[TKM];
  int far_ok[2];       // per half tile: every key valid, far rule, admitted by every row
  int win_ok[2];       // per half tile: every key valid, window rule, admitted by every row
  int rpos[TKM];       // in-kernel RoPE: table position the key is rotated to (-1: no key)
};

template <int DT, int D, int M>
__global__ void __launch_bounds__(M * 2) bsa_mma_kernel(const hipattn_bsa_params_t p, int BQ, int n_sub) {
  constexpr int NT = M * 2;            // threads: one warp per 16 rows
  constexpr int PIECES = D / 8;        // 16-byte pieces per row
  constexpr int KSTEPS = D / 16;       // k-steps of S = Q K^T
  constexpr int NO = D / 8;            // n-tiles of O
  constexpr int TILE_BYTES = TKM * D * 2;
  using T = typename Elem<DT>::type;

  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* sQ = smem;                          // [M][D], reused as output staging
  unsigned char* sK = sQ + M * D * 2;                // 2 x [TKM][D]
  unsigned char* sV = sK + 2 * TILE_BYTES;           // 2 x [TKM][D]
  TileMeta* meta = reinterpret_cast<TileMeta*>(sV + 2 * TILE_BYTES);  // 3 entries
  __shared__ int s_rowpos[M];
  __shared__ int s_mm[4];  // block pmin, pmax; tile rows' smallest / largest position

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int Gq = p.H / p.HKV;
  const int NH = M / BQ;                // heads per CTA (1 or 2)
  const int NBLK = cdiv(p.TQ, p.block_size_q);
  const int hslots = p.H / NH;
  int64_t bid = blockIdx.x;
  const int sub = (int)(bid % n_sub); bid /= n_sub;     // n_sub > 1 never happens with NH > 1
  const int d = (int)(bid % NBLK); bid /= NBLK;
  const int hs = (int)(bid % hslots); bid /= hslots;
  const int b = (int)bid;
  const int h0 = hs * NH;
  const int hkv = h0 / Gq;
  const int blk_t0 = d * p.block_size_q;
  const int blk_rows = min(p.block_size_q, p.TQ - blk_t0);
  const int row_t0 = blk_t0 + sub * BQ;   // first query row of this CTA (BQ rows per head)
  const int rows_here = max(0, min(BQ, blk_rows - sub * BQ));

  if (tid < 4) s_mm[tid] = (tid & 1) ? -1 : 0x7fffffff;
  __syncthreads();
  {
    int lo = 0x7fffffff, hi = -1;
    for (int i = tid; i < blk_rows; i += NT) {
      const long long x = p.pos[(int64_t)b * p.pos_stride_b + (int64_t)(blk_t0 + i) * p.pos_stride_t];
      const int v = (int)(x > 0x7ffffff0LL ? 0x7ffffff0LL : (x < 0 ? 0 : x));
      lo = min(lo, v); hi = max(hi, v);
    }
    if (hi >= 0) { atomicMin(&s_mm[0], lo); atomicMax(&s_mm[1], hi); }
  }
  for (int r = tid; r < M; r += NT) {
    const int i = r % BQ;
    int pv = -0x40000000;
    if (i < rows_here) {
      const long long x = p.pos[(int64_t)b * p.pos_stride_b + (int64_t)(row_t0 + i) * p.pos_stride_t];
      pv = (int)(x > 0x7ffffff0LL ? 0x7ffffff0LL : (x < 0 ? 0 : x));
      atomicMin(&s_mm[2], pv);
      atomicMax(&s_mm[3], pv);
    }
    s_rowpos[r] = pv;
  }
  // Q tile -> swizzled shared memory (zero rows beyond the sequence)
  for (int i = tid; i < M * PIECES; i += NT) {
    const int r = i / PIECES, pc = i % PIECES;
    uint4 v = make_uint4(0, 0, 0, 0);
    if ((r % BQ) < rows_here) {
      const T* qp = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_stride_b + (int64_t)(row_t0 + r % BQ) * p.q_stride_t +
                    (int64_t)(h0 + r / BQ) * p.q_stride_h + pc * 8;
      v = *reinterpret_cast<const uint4*>(qp);
    }
    *reinterpret_cast<uint4*>(sQ + swz<D>(r, pc)) = v;
  }
  __syncthreads();
  if (p.rope_cos) {   // in-kernel RoPE: every query row at its own position (attention_extend_bsa.py:797-856)
    rope_rotate_tile<DT, D>(sQ, 0, M, p, tid, NT, [&](int r) { return s_rowpos[r]; });
    __syncthreads();
  }
  const int pmin = s_mm[0], pmax = s_mm[1];
  const int rmin = s_mm[2], rmax = s_mm[3];
  const KeyList kl = make_key_list(p, b, h0, d, pmin, pmax);
  const int n_tiles = cdiv(kl.total, TKM);

  // Q fragments
  uint32_t qf[KSTEPS][4];
  {
    const int r = warp * 16 + (lane & 15);
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) ldsm_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], sQ + swz<D>(r, ks * 2 + (lane >> 4)));
  }

  auto make_meta = [&](int tile) {
    if (tid < TKM) {
      TileMeta& m = meta[tile % 3];
      bool w;
      const int j = tile * TKM + tid;
      const int t = key_position(kl, j, &w);
      m.tpos[tid] = t;
      m.twin[tid] = (t >= 0 && w) ? 1 : 0;
      long long ko = -1, vo = -1;
      if (t >= 0) {
        ko = token_row(p.k, b, t, hkv, 2, p.status) - (const char*)(p.k.cache ? p.k.cache : p.k.dense);
        vo = token_row(p.v, b, t, hkv, 2, p.status) - (const char*)(p.v.cache ? p.v.cache : p.v.dense);
      }
      m.koff[tid] = ko;
      m.voff[tid] = vo;
      m.rpos[tid] = (t >= 0 && p.rope_cos) ? rope_key_position(kl, j, t, p.window) : -1;
      const bool far_ok = t >= 0 && !w && t <= rmin - p.window;
      const bool win_ok = t >= 0 && w && t > rmax - p.window && t <= rmin;
      const int f = __all_sync(0xffffffffu, far_ok), g = __all_sync(0xffffffffu, win_ok);
      if ((tid & 31) == 0) {
        m.far_ok[tid >> 5] = f;
        m.win_ok[tid >> 5] = g;
      }
    }
  };
  auto gather = [&](int tile) {
    const TileMeta& m = meta[tile % 3];
    unsigned char* kb = sK + (tile & 1) * TILE_BYTES;
    unsigned char* vb = sV + (tile & 1) * TILE_BYTES;
    const char* kbase = (const char*)(p.k.cache ? p.k.cache : p.k.dense);
    const char* vbase = (const char*)(p.v.cache ? p.v.cache : p.v.dense);
    for (int i = tid; i < TKM * PIECES; i += NT) {
      const int r = i / PIECES, pc = i % PIECES;
      const long long ko = m.koff[r], vo = m.voff[r];
      if (ko >= 0) {
        cp_async16(kb + swz<D>(r, pc), kbase + ko + pc * 16);
        cp_async16(vb + swz<D>(r, pc), vbase + vo + pc * 16);
      } else {
        *reinterpret_cast<uint4*>(kb + swz<D>(r, pc)) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(vb + swz<D>(r, pc)) = make_uint4(0, 0, 0, 0);
      }
    }
  };

  float o[NO][4];
#pragma unroll
  for (int i = 0; i < NO; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int prow0 = s_rowpos[warp * 16 + (lane >> 2)], prow1 = s_rowpos[warp * 16 + (lane >> 2) + 8];
  const float cap = p.logit_softcap;

  if (n_tiles > 0) {
    make_meta(0);
    __syncthreads();
    gather(0);
    cp_async_commit();
    if (n_tiles > 1) make_meta(1);
    __syncthreads();
  }
  for (int it = 0; it < n_tiles; ++it) {
    if (it + 1 < n_tiles) gather(it + 1);
    cp_async_commit();
    if (it + 2 < n_tiles) make_meta(it + 2);
    cp_async_wait<1>();
    __syncthreads();

    const TileMeta& mt = meta[it % 3];
    if (p.rope_cos) {   // in-kernel RoPE: the tile's keys at the positions their places in the list map to
      rope_rotate_tile<DT, D>(sK + (it & 1) * TILE_BYTES, 0, TKM, p, tid, NT, [&](int r) { return mt.rpos[r]; });
      __syncthreads();
    }
    const unsigned char* kb = sK + (it & 1) * TILE_BYTES;
    const unsigned char* vb = sV + (it & 1) * TILE_BYTES;
    // ---- S = Q K^T (16 rows x 64 keys per warp) ----
    float s[TKM / 8][4];
#pragma unroll
    for (int i = 0; i < TKM / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
      for (int np = 0; np < TKM / 16; ++np) {
        uint32_t b0, b1, b2, b3;
        const int krow = np * 16 + (lane & 7) + ((lane >> 4) << 3);
        const int kpc = ks * 2 + ((lane >> 3) & 1);
        ldsm_x4(b0, b1, b2, b3, kb + swz<D>(krow, kpc));
        mma16816<DT>(s[np * 2], qf[ks], b0, b1);
        mma16816<DT>(s[np * 2 + 1], qf[ks], b2, b3);
      }
    }
    // ---- admission + online softmax ----
    const bool full = (mt.far_ok[0] && mt.far_ok[1]) || (mt.win_ok[0] && mt.win_ok[1]);
    float mx0 = -INFINITY, mx1 = -INFINITY;
    if (cap > 0.f) {   // soft-cap behind its own uniform branch: inside the loop the tanh is evaluated under a predicate
#pragma unroll
      for (int nt = 0; nt < TKM / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] = tanhf(s[nt][e] / cap) * cap;
      }
    }
#pragma unroll
    for (int nt = 0; nt < TKM / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float x = s[nt][e];
        x *= kLog2e;
        if (!full) {
          const int col = nt * 8 + (lane & 3) * 2 + (e & 1);
          if (!admits(e < 2 ? prow0 : prow1, mt.tpos[col], mt.twin[col] != 0, p.window)) x = -INFINITY;
        }
        s[nt][e] = x;
        if (e < 2) mx0 = fmaxf(mx0, x); else mx1 = fmaxf(mx1, x);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
    const float base0 = mn0 > -INFINITY ? mn0 : 0.f, base1 = mn1 > -INFINITY ? mn1 : 0.f;
    const float al0 = exp2f(m_run[0] - base0), al1 = exp2f(m_run[1] - base1);  // exp2(-inf) = 0
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < TKM / 8; ++nt) {
      s[nt][0] = exp2f(s[nt][0] - base0); s[nt][1] = exp2f(s[nt][1] - base0);
      s[nt][2] = exp2f(s[nt][2] - base1); s[nt][3] = exp2f(s[nt][3] - base1);
      sum0 += s[nt][0] + s[nt][1];
      sum1 += s[nt][2] + s[nt][3];
    }
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1); sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1); sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
    l_run[0] = l_run[0] * al0 + sum0;
    l_run[1] = l_run[1] * al1 + sum1;
    m_run[0] = mn0;
    m_run[1] = mn1;
#pragma unroll
    for (int i = 0; i < NO; ++i) { o[i][0] *= al0; o[i][1] *= al0; o[i][2] *= al1; o[i][3] *= al1; }
    // ---- O += P V ----
#pragma unroll
    for (int kk = 0; kk < TKM / 16; ++kk) {
      uint32_t pa[4];
      pa[0] = pack2<DT>(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = pack2<DT>(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = pack2<DT>(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = pack2<DT>(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int np = 0; np < NO / 2; ++np) {
        uint32_t b0, b1, b2, b3;
        const int vrow = kk * 16 + (lane & 15);
        const int vpc = np * 2 + (lane >> 4);
        ldsm_x4_t(b0, b1, b2, b3, vb + swz<D>(vrow, vpc));
        mma16816<DT>(o[np * 2], pa, b0, b1);
        mma16816<DT>(o[np * 2 + 1], pa, b2, b3);
      }
    }
    __syncthreads();  // tile buffers and meta[it % 3] may be overwritten from here on
  }
  cp_async_wait<0>();

  // ---- epilogue: normalise, stage through shared memory, 16-byte stores ----
  const float inv0 = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, inv1 = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
  {
    const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
#pragma unroll
    for (int nt = 0; nt < NO; ++nt) {
      const int byte = (lane & 3) * 4;  // two elements
      *reinterpret_cast<uint32_t*>(sQ + swz<D>(r0, nt) + byte) = pack2<DT>(o[nt][0] * inv0, o[nt][1] * inv0);
      *reinterpret_cast<uint32_t*>(sQ + swz<D>(r1, nt) + byte) = pack2<DT>(o[nt][2] * inv1, o[nt][3] * inv1);
    }
    if (p.lse_out && (lane & 3) == 0) {
      const int i0 = r0 % BQ, i1 = r1 % BQ;
      if (i0 < rows_here)
        p.lse_out[((int64_t)b * p.TQ + row_t0 + i0) * p.H + h0 + r0 / BQ] = l_run[0] > 0.f ? m_run[0] + log2f(l_run[0]) : -INFINITY;
      if (i1 < rows_here)
        p.lse_out[((int64_t)b * p.TQ + row_t0 + i1) * p.H + h0 + r1 / BQ] = l_run[1] > 0.f ? m_run[1] + log2f(l_run[1]) : -INFINITY;
    }
  }
  __syncthreads();
  for (int i = tid; i < M * PIECES; i += NT) {
    const int r = i / PIECES, pc = i % PIECES;
    if ((r % BQ) < rows_here) {
      T* op = reinterpret_cast<T*>(p.out) + (int64_t)b * p.o_stride_b + (int64_t)(row_t0 + r % BQ) * p.o_stride_t +
              (int64_t)(h0 + r / BQ) * p.o_stride_h + pc * 8;
      *reinterpret_cast<uint4*>(op) = *reinterpret_cast<const uint4*>(sQ + swz<D>(r, pc));
    }
  }
}

template <int DT, int D, int M>
int launch(const hipattn_bsa_params_t& p, int BQ, int n_sub, cudaStream_t stream) {
  const size_t smem = (size_t)M * D * 2 + 4 * (size_t)TKM * D * 2 + 3 * sizeof(TileMeta);
  const int NH = M / BQ;
  const int NBLK = cdiv(p.TQ, p.block_size_q);
  const int64_t grid = (int64_t)p.B * (p.H / NH) * NBLK * n_sub;
  HIPATTN_REQUIRE(grid > 0 && grid < 0x7fffffffLL, HIPATTN_ERR_INVALID, "attention grid of %lld blocks", (long long)grid);
  auto kern = bsa_mma_kernel<DT, D, M>;
  HIPATTN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<(unsigned)grid, M * 2, smem, stream>>>(p, BQ, n_sub);
  return check_launch("bsa_mma_kernel");
}

template <int DT, int D>
int dispatch(const hipattn_bsa_params_t& p, cudaStream_t stream, bool* handled) {
  const int Gq = p.H / p.HKV;
  const int bq = p.block_size_q;
  *handled = true;
  if (bq == 64 && p.heads_share_mask && (Gq % 2) == 0) return launch<DT, D, 128>(p, 64, 1, stream);  // two heads per CTA
  if (bq == 64) return launch<DT, D, 64>(p, 64, 1, stream);
  if (bq % 128 == 0) return launch<DT, D, 128>(p, 128, bq / 128, stream);
  *handled = false;
  return HIPATTN_OK;
}

}  // namespace

// Handles 16-bit prefill shapes (attention blocks of 64 or a multiple of 128 rows, head dim 64 or 128,
// out rows 16-byte aligned); everything else is left to the general kernel.
int bsa_mma(const hipattn_bsa_params_t& p, cudaStream_t stream, bool* handled) {
  *handled = false;
  if (p.n_splits != 1 || p.dtype == HIPATTN_F32 || p.TQ < 16) return HIPATTN_OK;
  if (p.D != 64 && p.D != 128) return HIPATTN_OK;
  if (((uintptr_t)p.out % 16) || (p.o_stride_b % 8) || (p.o_stride_t % 8) || (p.o_stride_h % 8)) return HIPATTN_OK;
  if (p.dtype == HIPATTN_BF16) return p.D == 128 ? dispatch<HIPATTN_BF16, 128>(p, stream, handled) : dispatch<HIPATTN_BF16, 64>(p, stream, handled);
  if (p.dtype == HIPATTN_F16) return p.D == 128 ? dispatch<HIPATTN_F16, 128>(p, stream, handled) : dispatch<HIPATTN_F16, 64>(p, stream, handled);
  return HIPATTN_OK;
}

}  // namespace hipattn
