// Scan stage of the mask estimator for 16-bit prefill, small chunks, symmetric form: every token of every
// active chunk is scored once for all query heads of a KV head, then the halving search is replayed on the
// stored scores (see scan_dense_tcgen05.cu for why that gives the reference's bounds and scores while
// gathering fewer key rows).  Here the work is organised like the round-by-round kernel
// (scan_stage_tcgen05.cu): CTAs of 128 threads, several resident per SM, every thread owns one key row of a
// tile of 128 rows (128 / chunk whole chunks) from gather to score, so that many warps run the same short
// code instead of a few warps running long roles.
//
// Per tile: 16-byte cp.async gathers of the chunk's consecutive tokens from the head-major scaled key copy
// into the swizzled K-major A operand -> D / 16 tcgen05.mma with N = heads x pooled rows -> each thread
// reads its own TMEM lane, one row maximum per head -> rounding check with the error radius
// kEps * max|q'| * sum|k'| and strict re-score of uncertain (key, head) pairs from the staged row ->
// scores to shared memory -> one thread per (chunk, head) walks the search tree -> head-max atomics.
// The chunk bounds of the next tile and the key sums of the current one are requested a phase ahead, so
// that no global-memory latency other than the gather itself sits inside a tile.
#include <cstdlib>
#include <cstring>

#include "scan_common.cuh"
#include "tcgen05_common.cuh"

namespace hipattn {
namespace {

template <int DT, int D, int NR, int HB>
__global__ void __launch_bounds__(128) scan_chunks_tcgen05_kernel(const hipattn_scan_params_t p, int c_log2, int n_split, int tiles_total,
                                                                  int check) {
  constexpr int ROWB = D * 2;
  constexpr int PIECES = ROWB / 16;
  constexpr int KB = D / 64;
  constexpr int N = HB * NR;
  constexpr int K_BLOCK_BYTES = 128 * 128;
  constexpr int Q_BLOCK_BYTES = N * 128;
  constexpr uint32_t TMEM_COLS = N < 32 ? 32 : N;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  unsigned char* sK = smem;                                  // [KB][128 keys][128 B], swizzled
  unsigned char* sQ = sK + KB * K_BLOCK_BYTES;               // [KB][N rows][128 B], swizzled
  float* sS = reinterpret_cast<float*>(sQ + KB * Q_BLOCK_BYTES);     // [HB][128] rounded scores of the tile
  float* kf32 = sS + HB * 128;                               // [4 warps][D]: key of a strict re-score
  int* s_gmax = reinterpret_cast<int*>(kf32 + 4 * D);        // [groups of block_chunk chunks]
  __shared__ __align__(8) unsigned long long s_mbar;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  __shared__ int s_pmin;
  __shared__ float s_qmax[HB];
  __shared__ int s_cl[32], s_cr[32];                         // bounds of the tile's chunks

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int Gq = p.H / p.HKV;
  const int BDST = cdiv(p.TQ, p.block_size_q);
  const int n_hb = Gq / HB;
  int64_t bid = blockIdx.x;
  const int split = (int)(bid % n_split); bid /= n_split;
  const int hb = (int)(bid % n_hb); bid /= n_hb;
  const int d = (int)(bid % BDST); bid /= BDST;
  const int hkv = (int)(bid % p.HKV); bid /= p.HKV;
  const int b = (int)bid;
  const int h0 = hkv * Gq + hb * HB;

  const int R = p.block_size_q / p.stride_q;
  const int t0 = d * p.block_size_q;
  int Rv = 0;
  if (t0 < p.TQ) Rv = min(R, (p.TQ - t0 + p.stride_q - 1) / p.stride_q);
  const int C = 1 << c_log2;
  const int cpt_log2 = 7 - c_log2;
  const int n = p.n_chunks;
  const int64_t row = (int64_t)b * BDST + d;
  const int32_t* gl = p.left + row * n;
  const int32_t* gr = p.right + row * n;
  const int tiles_per = cdiv(tiles_total, n_split);
  const int tile0 = split * tiles_per;
  const int my_tiles = Rv > 0 ? max(0, min(tiles_per, tiles_total - tile0)) : 0;
  const int bc_log2 = 31 - __clz(p.block_chunk);
  const int n_groups = (n + p.block_chunk - 1) >> bc_log2;
  const int key_base = (b * p.HKV + hkv) * p.T;
  const uint32_t mbar = smem_u32(&s_mbar);

  // ---- set-up ----
  if (tid == 0) {
    mbar_init(mbar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    s_abort = 0;
  }
  if (tid < HB) s_qmax[tid] = 0.f;
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  for (int i = tid; i < n_groups; i += 128) s_gmax[i] = 0;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;

  if (my_tiles > 0) {
    for (int i = tid; i < N * PIECES; i += 128) {
      const int r = i / PIECES, pc = i % PIECES;
      const int hh = r / NR, rr = r % NR;
      float v[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = 0.f;
      if (rr < Rv) pooled_query_piece<DT>(p, b, h0 + hh, t0 + rr * p.stride_q, pc, v);
      uint4 w;
      w.x = pack2<DT>(v[0], v[1]); w.y = pack2<DT>(v[2], v[3]); w.z = pack2<DT>(v[4], v[5]); w.w = pack2<DT>(v[6], v[7]);
      *reinterpret_cast<uint4*>(sQ + (pc >> 3) * Q_BLOCK_BYTES + sw128(r, pc & 7)) = w;
      float m = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) m = fmaxf(m, fabsf(v[e]));
      if (m > 0.f) atomicMax(reinterpret_cast<int*>(&s_qmax[hh]), __float_as_int(m));   // non-negative floats order as ints
    }
    {
      const int c_lo = ((tile0 << cpt_log2) >> bc_log2) << bc_log2;
      const int c_hi = min(n, ((((tile0 + my_tiles) << cpt_log2) + p.block_chunk - 1) >> bc_log2) << bc_log2);
      for (int c = c_lo + tid; c < c_hi; c += 128) {
        const int len = gr[c] - gl[c];
        if (len > C) atomicOr(p.status, HIPATTN_STATUS_CHUNK_SIZE);
        if (len > 0) atomicMax(&s_gmax[c >> bc_log2], len);
      }
    }
    if (warp == 0) {
      const int m = block_min_position(p, b, t0, Rv, lane);
      if (lane == 0) s_pmin = m;
    }
  }
  fence_async_smem();
  __syncthreads();

  const int pt = max(s_pmin - p.scan_window, 0);
  const char* kbase = reinterpret_cast<const char*>(p.k_scaled);
  const uint32_t sK_u32 = smem_u32(sK), sQ_u32 = smem_u32(sQ);
  const uint32_t idesc = make_idesc(DT == HIPATTN_BF16 ? 1 : 0, 128, N, 0);
  const uint32_t my_tmem = tmem + ((uint32_t)(warp * 32) << 16);
  float* wkf = kf32 + warp * D;
  float eps_q[HB];
#pragma unroll
  for (int hh = 0; hh < HB; ++hh) eps_q[hh] = kEps * s_qmax[hh];
  unsigned long long st_keys = 0, st_fb = 0, st_wrong = 0;
  float st_ratio = 0.f;
  uint32_t phase = 0;
  const int rot = my_tiles > 0 ? (int)(((unsigned)d * 2654435761u >> 8) % (unsigned)my_tiles) : 0;
  auto tile_of = [&](int i) -> int { const int j = i + rot; return tile0 + (j >= my_tiles ? j - my_tiles : j); };

  // strict dot products of the key staged in row `srow` against the pooled rows of head hh, by the whole
  // warp (one pooled row per lane); returns the largest one before rounding
  auto strict_score = [&](int srow, int hh) -> float {
    __syncwarp();
    for (int e2 = lane; e2 < D / 2; e2 += 32) {
      const int pc = e2 >> 2;
      const uint32_t w = *reinterpret_cast<const uint32_t*>(sK + (pc >> 3) * K_BLOCK_BYTES + sw128(srow, pc & 7) + (e2 & 3) * 4);
      wkf[2 * e2] = lo_f32<DT>(w);
      wkf[2 * e2 + 1] = hi_f32<DT>(w);
    }
    __syncwarp();
    float best = -INFINITY;
    for (int r0 = 0; r0 < Rv; r0 += 32) {
      const int r = r0 + lane;
      if (r < Rv) {
        const int qr = hh * NR + r;
        float acc = 0.f;
#pragma unroll 4
        for (int pc = 0; pc < PIECES; ++pc) {
          const uint4 qw = *reinterpret_cast<const uint4*>(sQ + (pc >> 3) * Q_BLOCK_BYTES + sw128(qr, pc & 7));
          const float4 k0 = *reinterpret_cast<const float4*>(wkf + pc * 8);
          const float4 k1 = *reinterpret_cast<const float4*>(wkf + pc * 8 + 4);
          acc = fmaf(lo_f32<DT>(qw.x), k0.x, acc);
          acc = fmaf(hi_f32<DT>(qw.x), k0.y, acc);
          acc = fmaf(lo_f32<DT>(qw.y), k0.z, acc);
          acc = fmaf(hi_f32<DT>(qw.y), k0.w, acc);
          acc = fmaf(lo_f32<DT>(qw.z), k1.x, acc);
          acc = fmaf(hi_f32<DT>(qw.z), k1.y, acc);
          acc = fmaf(lo_f32<DT>(qw.w), k1.z, acc);
          acc = fmaf(hi_f32<DT>(qw.w), k1.w, acc);
        }
        best = fmaxf(best, acc);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, o));
    return best;
  };

  // bounds of the chunk of this thread's row in tile i (requested one tile ahead)
  auto load_bounds = [&](int i, int& l, int& rt) {
    l = 0; rt = 0;
    if (i < my_tiles) {
      const int c = (tile_of(i) << cpt_log2) + (tid >> c_log2);
      if (c < n) { l = gl[c]; rt = gr[c]; }
    }
  };
  int l_next, r_next;
  load_bounds(0, l_next, r_next);

  for (int i = 0; i < my_tiles; ++i) {
    const int tile = tile_of(i);
    const int l = l_next, rt = r_next;
    load_bounds(i + 1, l_next, r_next);
    // key row (index into the head-major copy, or -1) of this thread's tile row, and its key sum
    int idx = -1;
    if (l < rt && l <= pt && l >= 0) {
      int tk = l + (tid & (C - 1));
      if (tk < rt) {
        if (tk >= p.T) {
          atomicOr(p.status, HIPATTN_STATUS_TOKEN_RANGE);
          tk = p.T - 1;
        }
        idx = key_base + tk;
      }
    }
    const float s_abs = idx >= 0 ? p.key_abs[idx] : 0.f;      // consumed after the gather and the MMAs
    tc_fence_before();
    if (__syncthreads_or(*(volatile int*)&s_abort)) break;   // previous tile's scores and operand tile are free
    if ((tid & (C - 1)) == 0) {
      s_cl[tid >> c_log2] = l;
      s_cr[tid >> c_log2] = rt;
    }
    // ---- gather this warp's 32 rows: 8 lanes per row, 128 contiguous bytes per row and instruction ----
#pragma unroll
    for (int r0 = 0; r0 < 32; r0 += 4) {
      const int j = r0 + (lane >> 3);
      const int src = __shfl_sync(0xffffffffu, idx, j);
      if (src >= 0) {
        const int srow = warp * 32 + j;
        const char* gp = kbase + (int64_t)src * ROWB + (lane & 7) * 16;
        unsigned char* sp = sK + sw128(srow, lane & 7);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) cp_async16(sp + kb * K_BLOCK_BYTES, gp + kb * 128);
      }
    }
    cp_async_commit();
    cp_async_wait<0>();
    fence_async_smem();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int k = 0; k < D / 16; ++k) {
        const uint64_t da = make_desc(sK_u32 + (k >> 2) * K_BLOCK_BYTES + (k & 3) * 32, 16, 1024);
        const uint64_t db = make_desc(sQ_u32 + (k >> 2) * Q_BLOCK_BYTES + (k & 3) * 32, 16, 1024);
        umma(tmem, da, db, idesc, k > 0 ? 1u : 0u);
      }
      umma_commit(mbar);
    }
    __syncwarp();
    bool ok = mbar_wait(mbar, phase, &s_abort, p.status);
    phase ^= 1u;
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    if (ok) {
      constexpr int BW = N < 64 ? N : 64;
#pragma unroll
      for (int c0 = 0; c0 < N; c0 += BW) {
        float v[BW];
        if (BW == 16) tmem_ld16(my_tmem + c0, v);
        else if (BW == 32) tmem_ld32(my_tmem + c0, v);
        else tmem_ld64(my_tmem + c0, v);
#pragma unroll
        for (int h2 = 0; h2 < BW / NR; ++h2) {
          const int hh = c0 / NR + h2;
          float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
          if (Rv >= NR) {
#pragma unroll
            for (int j = 0; j < NR; ++j) m4[j & 3] = fmaxf(m4[j & 3], v[h2 * NR + j]);
          } else {
#pragma unroll
            for (int j = 0; j < NR; ++j)
              if (j < Rv) m4[j & 3] = fmaxf(m4[j & 3], v[h2 * NR + j]);
          }
          const float x = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
          // rounding check of (key, head); uncertain pairs are re-scored strictly, one after the other
          const float e_ = eps_q[hh] * s_abs * 1.01f;
          float sc = Elem<DT>::round(x);
          const bool sure = Elem<DT>::round(x - e_) == Elem<DT>::round(x + e_);
          unsigned need = __ballot_sync(0xffffffffu, idx >= 0 && (!sure || check));
          while (need) {
            const int owner = __ffs(need) - 1;
            need &= need - 1;
            const float rawv = strict_score(warp * 32 + owner, hh);
            const float ex = Elem<DT>::round(rawv);
            if (lane == owner) {
              if (check) {
                if (sure && sc != ex) ++st_wrong;
                if (e_ > 0.f) st_ratio = fmaxf(st_ratio, fabsf(x - rawv) / e_);
              }
              if (!sure) ++st_fb;
              sc = ex;
            }
          }
          if (idx >= 0) ++st_keys;
          sS[hh * 128 + tid] = sc;
        }
      }
    }
    tc_fence_before();
    if (__syncthreads_or((!ok || *(volatile int*)&s_abort) ? 1 : 0)) break;
    // ---- the halving search of every (chunk, head) of the tile over the stored scores ----
    {
      const int walkers = HB << cpt_log2;       // at most 128: chunks of at least 4 tokens, at most 4 heads
      const int hh = tid % HB, cl = tid / HB;
      const int c = (tile << cpt_log2) + cl;
      const bool live = tid < walkers && c < n;
      float score = HIPATTN_SCORE_INIT;
      if (live) {
        int wl = s_cl[cl], wr = s_cr[cl];
        const int base = wl;
        const int gm = s_gmax[c >> bc_log2];
        const int rounds = gm >= 1 ? 32 - __clz(gm) : 0;
        const float* sc = sS + hh * 128 + (cl << c_log2);
        for (int it = 0; it < rounds; ++it) {
          if (!(wl < wr && wl <= pt && wl >= 0)) break;
          const int mid = (wl + wr) >> 1;
          const float sl = sc[min(((wl + mid) >> 1) - base, C - 1)];
          const float sr = sc[min(((mid + wr) >> 1) - base, C - 1)];
          const bool win = sl > sr;
          if (win) wr = mid; else wl = mid;
          score = fmaxf(score, win ? sl : sr);
        }
        const int64_t o = (row * p.H + h0 + hh) * n + c;
        if (p.left_out) p.left_out[o] = wl;
        if (p.right_out) p.right_out[o] = wr;
        if (p.score_out) p.score_out[o] = score;
      }
      float best = score;
#pragma unroll
      for (int o = 1; o < HB; o <<= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, o));
      if (live && hh == 0 && best > HIPATTN_SCORE_INIT) atomicMax(p.score_max + row * n + c, encode_score(best));
    }
  }

  if (p.stats) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      st_keys += __shfl_xor_sync(0xffffffffu, st_keys, o);
      st_fb += __shfl_xor_sync(0xffffffffu, st_fb, o);
      st_wrong += __shfl_xor_sync(0xffffffffu, st_wrong, o);
    }
    unsigned long long* st = reinterpret_cast<unsigned long long*>(p.stats);
    if (lane == 0) {
      atomicAdd(st + ST_KEYS, st_keys);
      atomicAdd(st + ST_FALLBACK, st_fb);
      atomicAdd(st + ST_WRONG, st_wrong);
    }
    atomicMax(reinterpret_cast<unsigned int*>(p.stats + ST_RATIO_BITS), __float_as_uint(st_ratio));
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

template <int DT, int D, int NR, int HB>
int launch(const hipattn_scan_params_t& p, int c_log2, cudaStream_t stream) {
  constexpr int N = HB * NR;
  const int KB = D / 64;
  const int BDST = cdiv(p.TQ, p.block_size_q);
  const int Gq = p.H / p.HKV;
  const int cpt = 128 >> c_log2;
  const int tiles_total = cdiv(p.n_chunks, cpt);
  const int n_groups = cdiv(p.n_chunks, p.block_chunk);
  const size_t smem = 1024 + (size_t)KB * (128 * 128 + N * 128) + HB * 128 * sizeof(float) + 4 * D * sizeof(float) +
                      (size_t)n_groups * sizeof(int);
  HIPATTN_REQUIRE(smem <= 226 * 1024, HIPATTN_ERR_UNSUPPORTED, "chunk scan stage needs %zu bytes of shared memory", smem);
  const int64_t units = (int64_t)p.B * p.HKV * BDST * (Gq / HB);
  int n_split = 1;   // few units (short prefill chunks): split the tiles of a unit over several CTAs
  if (units < 148 * 2) {
    const int64_t want = (148 * 2 + units - 1) / units;
    n_split = (int)(want < tiles_total ? want : tiles_total);
  }
  const int64_t grid = units * n_split;
  HIPATTN_REQUIRE(grid > 0 && grid < 0x7fffffffLL, HIPATTN_ERR_INVALID, "scan grid of %lld blocks", (long long)grid);
  auto kern = scan_chunks_tcgen05_kernel<DT, D, NR, HB>;
  HIPATTN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<(unsigned)grid, 128, smem, stream>>>(p, c_log2, n_split, tiles_total, p.mode == HIPATTN_SCAN_CHECK ? 1 : 0);
  return check_launch("scan_chunks_tcgen05_kernel");
}

template <int DT, int D, int NR>
int dispatch_heads(const hipattn_scan_params_t& p, int c_log2, int HB, cudaStream_t stream) {
  switch (HB) {
    case 4: return launch<DT, D, NR, 4>(p, c_log2, stream);
    case 2: return launch<DT, D, NR, 2>(p, c_log2, stream);
    default: return launch<DT, D, NR, 1>(p, c_log2, stream);
  }
}

template <int DT, int D>
int dispatch_rows(const hipattn_scan_params_t& p, int c_log2, int HB, cudaStream_t stream) {
  const int R = p.block_size_q / p.stride_q;
  if (R <= 16) return dispatch_heads<DT, D, 16>(p, c_log2, HB, stream);
  if (R <= 32) return dispatch_heads<DT, D, 32>(p, c_log2, HB, stream);
  return dispatch_heads<DT, D, 64>(p, c_log2, HB, stream);
}

}  // namespace

// Takes the shapes of the round-based tcgen05 scan when the stage's chunk size is a known power of two
// between 4 and `HIPATTN_SCAN_CHUNKS_MAX`, or for every such stage with HIPATTN_SCAN_KERNEL=chunks.
// Off by default (limit 0): on benchmark configuration 2 it equals the round-by-round kernel on the last stage
// (chunk 8: 4.42 against 4.37 ms, with a quarter of the key rows gathered) and loses on chunk 32 (6.9
// against 4.8 ms): a tile is one long dependent chain per CTA and only two CTAs fit beside the pooled
// queries of four heads.
int scan_chunks_tcgen05(const hipattn_scan_params_t& p, cudaStream_t stream, bool* handled) {
  *handled = false;
  const int R = p.block_size_q / p.stride_q;
  const int rows = min(R, cdiv(p.TQ, p.stride_q));
  if (p.mode == HIPATTN_SCAN_STRICT || p.dtype == HIPATTN_F32 || rows <= 1 || (R % 16) != 0 || R > 64 || (p.D != 64 && p.D != 128)) return HIPATTN_OK;
  if (p.key_abs == nullptr || p.k_scaled == nullptr) return HIPATTN_OK;
  if ((int64_t)p.B * p.T * p.HKV >= 0x7fffffffLL) return HIPATTN_OK;
  const int C = p.chunk_size;
  if (C < 4 || C > 128 || (C & (C - 1)) != 0) return HIPATTN_OK;
  const char* v = getenv("HIPATTN_SCAN_KERNEL");
  const bool forced = v && strcmp(v, "chunks") == 0;
  if (v && !forced && strcmp(v, "auto") != 0) return HIPATTN_OK;
  const char* mc = getenv("HIPATTN_SCAN_CHUNKS_MAX");
  const int max_chunk = mc ? atoi(mc) : 0;
  if (!forced && C > max_chunk) return HIPATTN_OK;
  int c_log2 = 0;
  while ((1 << c_log2) < C) ++c_log2;
  const int Gq = p.H / p.HKV;
  const int NRp = R <= 16 ? 16 : (R <= 32 ? 32 : 64);
  int HB = 4;
  while (HB > 1 && (Gq % HB != 0 || HB * NRp > 256)) HB >>= 1;
  if (!forced && C > HB * 2 * (c_log2 + 1)) return HIPATTN_OK;   // no fewer rows than the rounds would gather
  *handled = true;
  if (p.dtype == HIPATTN_BF16) return p.D == 128 ? dispatch_rows<HIPATTN_BF16, 128>(p, c_log2, HB, stream) : dispatch_rows<HIPATTN_BF16, 64>(p, c_log2, HB, stream);
  return p.D == 128 ? dispatch_rows<HIPATTN_F16, 128>(p, c_log2, HB, stream) : dispatch_rows<HIPATTN_F16, 64>(p, c_log2, HB, stream);
}

}  // namespace hipattn
