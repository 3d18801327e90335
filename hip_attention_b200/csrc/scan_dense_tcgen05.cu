// Scan stage of the mask estimator for 16-bit prefill, small chunks: every token of every active chunk
// is scored once for all query heads of a KV group, then the halving search is replayed on the scores.
//
// The reference search (attention_extend.py:413-1249) scores two candidate keys per chunk, head and
// round; the candidates of round r depend on the decisions of round r - 1, which serialises a chunk
// into log2(chunk) + 1 dependent gathers, and the heads of a KV group gather overlapping keys
// independently.  All candidates of a chunk lie inside the chunk.  When the chunk is small
// (chunk <= heads x 2 x rounds) it is cheaper to gather the chunk's tokens ONCE, score them against
// the pooled queries of all heads of the group in one tensor-core pass and let one thread per
// (chunk, head) walk the search tree over the stored scores: the same per-key scores in the same
// comparisons, so bounds and scores equal the reference's, with fewer bytes gathered (8 instead of
// 32 key rows per chunk for a last stage of chunk 8 and 4 heads per KV head) and no dependent rounds.
//
// Per-key scores keep the contract of the other scan kernels: max over pooled rows of
// round_to_dtype(sequential fp32 dot).  The tensor-core value is used when rounding is certain within
// the error radius kEps * max|q'| * sum_d |k'_d|; otherwise the (key, head) pair is re-scored strictly.
//
// One CTA = one (batch, query block, KV head, head batch); 352 threads in four roles that hand tiles of
// 128 key rows (128 / chunk chunks x chunk tokens) to one another through mbarriers:
//   warps 5-6   producers: fill the tile's record (key index, absolute sum and chunk bounds per row) and
//               gather the rows with 16-byte cp.async from the pre-scaled dense key copy into a ring of
//               swizzled K-major operand tiles
//   warp 4      issuer: per tile D / 16 tcgen05.mma (M = 128 keys, N = heads x pooled rows) into one of two
//               TMEM accumulators
//   warps 0-3   scores: thread = key = TMEM lane; tcgen05.ld, row maximum per head, rounding check; rounded
//               scores and the mask of uncertain (key, head) pairs go to the tile's record
//   warps 7-10  search: warp w takes every fourth tile: strict re-scores of the uncertain pairs, then the
//               tree walk of every (chunk, head) and the head-max atomics.  Four tiles are in this stage
//               at once, so the latency of a re-score is off the critical path.
// Every wait is bounded; a wait that runs out raises HIPATTN_STATUS_TIMEOUT and all roles leave through
// the common exit, which frees the TMEM columns.
#include <cstdlib>
#include <cstring>

#include <cuda.h>

#include "scan_common.cuh"
#include "tcgen05_common.cuh"

namespace hipattn {
namespace {

// Optional cycle accounting per role (representative lanes only), added to words 8.. of the statistics
// buffer; compiled in with -DHIPATTN_SCAN_PROFILE for experiments, never in the shipped library.
#ifdef HIPATTN_SCAN_PROFILE
#define PROF_DECL(n) long long prof_[n] = {}; long long prof_t_ = clock64()
#define PROF_LAP(k) do { const long long t_ = clock64(); prof_[k] += t_ - prof_t_; prof_t_ = t_; } while (0)
#define PROF_FLUSH(base, n, who) do { if ((who) && p.stats) for (int k_ = 0; k_ < (n); ++k_) \
    atomicAdd(reinterpret_cast<unsigned long long*>(p.stats) + (base) + k_, (unsigned long long)prof_[k_]); } while (0)
#else
#define PROF_DECL(n)
#define PROF_LAP(k)
#define PROF_FLUSH(base, n, who)
#endif

constexpr int kDenseThreads = 448;   // 2 x 4 score warps, 1 issuer, 1 producer, 4 search warps
constexpr int kSearchWarps = 4;
constexpr int kMaxStages = 6;
constexpr int kRows = 14;       // row tables in flight (producer -> search warps)
constexpr int kScr = 10;        // score tables in flight (score warps -> search warps)
constexpr int kSideRows = 4;    // key rows of uncertain scores kept per tile for the strict re-score
constexpr int kSidePairs = 12;  // (key, head) pairs per tile served from those rows; the rest re-read the key
constexpr int kBoundsAhead = 4; // tiles between the request for a tile's chunk bounds and their use

// What the later roles need to know about the rows of one tile (chunks of at least 4 tokens: <= 32 per tile).
struct TileRows {
  float kabs[128];         // row -> sum_d |k'_d|
  int left[32];            // chunk of the tile -> bounds
  int right[32];
};

// Scores of one tile on their way from the score warps to the search warps.
template <int HB, int ROWB>
struct TileScores {
  float score[HB][128];    // (head, row) -> rounded score (check mode: the unrounded tensor-core value)
  unsigned need[HB][4];    // (head, score warp) -> rows to re-score strictly from the key in global memory
  __align__(16) unsigned char kraw[kSideRows][ROWB];   // copies of the rows of uncertain keys
  int n_slots, n_pairs;    // rows used in kraw, pairs listed below
  unsigned short pair_key[kSidePairs];
  unsigned char pair_head[kSidePairs], pair_slot[kSidePairs];
};

template <int DT, int D, int NR, int HB>
__global__ void __launch_bounds__(kDenseThreads, 1) scan_dense_tcgen05_kernel(const hipattn_scan_params_t p, const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap kmap_run,
                                                                            int c_log2, int n_split, int tiles_total, int n_stages, int check) {
  constexpr int ROWB = D * 2;
  constexpr int PIECES = ROWB / 16;
  constexpr int KB = D / 64;
  constexpr int N = HB * NR;                       // MMA N: pooled rows of all heads of the batch
  constexpr int K_BLOCK_BYTES = 128 * 128;
  constexpr int K_TILE_BYTES = KB * K_BLOCK_BYTES;
  constexpr int Q_BLOCK_BYTES = N * 128;
  constexpr uint32_t TMEM_COLS = 2 * N < 32 ? 32 : 2 * N;   // 32, 64, 128, 256 or 512
  using Scr = TileScores<HB, ROWB>;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  unsigned char* sQ = smem;                                          // [KB][N rows][128 B]
  unsigned char* sK = sQ + KB * Q_BLOCK_BYTES;                       // [n_stages][KB][128 keys][128 B]
  Scr* scrs = reinterpret_cast<Scr*>(sK + (size_t)n_stages * K_TILE_BYTES);   // [kScr]
  TileRows* rows_ring = reinterpret_cast<TileRows*>(scrs + kScr);    // [kRows]
  unsigned char* kscratch = reinterpret_cast<unsigned char*>(rows_ring + kRows);   // [kSearchWarps][ROWB]
  int* s_gmax = reinterpret_cast<int*>(kscratch + kSearchWarps * ROWB);         // [groups of block_chunk chunks]
  __shared__ __align__(8) unsigned long long s_full[kMaxStages], s_empty[kMaxStages], s_acc_full[2], s_acc_empty[2];
  __shared__ __align__(8) unsigned long long s_rows_full[kRows], s_rows_empty[kRows], s_scr_full[kScr], s_scr_empty[kScr];
  __shared__ int s_bounds[(kBoundsAhead + 1) * 64];   // ring of prefetched chunk bounds [slot][left | right][chunk]
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  __shared__ int s_pmin;
  __shared__ float s_qmax[HB];

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
  const int cpt_log2 = 7 - c_log2;                 // chunks per tile = 128 / C
  const int CPT = 1 << cpt_log2;
  const int n = p.n_chunks;
  const int64_t row = (int64_t)b * BDST + d;
  const int32_t* gl = p.left + row * n;
  const int32_t* gr = p.right + row * n;
  const int tiles_per = cdiv(tiles_total, n_split);
  const int tile0 = split * tiles_per;
  const int my_tiles = Rv > 0 ? max(0, min(tiles_per, tiles_total - tile0)) : 0;
  const int bc_log2 = 31 - __clz(p.block_chunk);
  const int n_groups = (n + p.block_chunk - 1) >> bc_log2;
  const int key_base = (b * p.HKV + hkv) * p.T;    // first row of this KV head in the head-major key copy

  // ---- set-up ----
  if (tid == 0) {
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(smem_u32(&s_full[s]), 1);
      mbar_init(smem_u32(&s_empty[s]), 1);
    }
    for (int r = 0; r < kRows; ++r) {
      mbar_init(smem_u32(&s_rows_full[r]), 64);   // 32 plain arrivals (bounds) + 32 on completion of the copies
      mbar_init(smem_u32(&s_rows_empty[r]), 1);
    }
    for (int r = 0; r < kScr; ++r) {
      mbar_init(smem_u32(&s_scr_full[r]), 128);
      mbar_init(smem_u32(&s_scr_empty[r]), 1);
      scrs[r].n_slots = 0;
      scrs[r].n_pairs = 0;
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&s_acc_full[a]), 1);
      mbar_init(smem_u32(&s_acc_empty[a]), 128);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&kmap)) : "memory");
    s_abort = 0;
  }
  if (tid < HB) s_qmax[tid] = 0.f;
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  for (int i = tid; i < n_groups; i += kDenseThreads) s_gmax[i] = 0;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;

  if (my_tiles > 0) {
    // pooled queries of the HB heads: rows hh * NR + r of the B operand
    for (int i = tid; i < N * PIECES; i += kDenseThreads) {
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
    // largest chunk of every group of block_chunk chunks that this CTA's tiles touch (fixes the rounds)
    {
      const int c_lo = ((tile0 << cpt_log2) >> bc_log2) << bc_log2;
      const int c_hi = min(n, ((((tile0 + my_tiles) << cpt_log2) + p.block_chunk - 1) >> bc_log2) << bc_log2);
      for (int c = c_lo + tid; c < c_hi; c += kDenseThreads) {
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
  // CTAs of neighbouring query blocks walk nearly the same keys; each starts at a different tile
  const int rot = my_tiles > 0 ? (int)(((unsigned)d * 2654435761u >> 8) % (unsigned)my_tiles) : 0;
  auto tile_of = [&](int i) -> int { const int j = i + rot; return tile0 + (j >= my_tiles ? j - my_tiles : j); };
  // key of row r of a tile whose chunk bounds are given: index into the head-major copy, or -1
  auto key_of = [&](const TileRows& tr, int r) -> int {
    const int l = tr.left[r >> c_log2], rt = tr.right[r >> c_log2];
    if (!(l < rt && l <= pt && l >= 0)) return -1;
    const int tk = l + (r & (C - 1));
    return tk < rt && tk < p.T ? key_base + tk : -1;
  };

  if (my_tiles > 0 && warp == 9) {
    // ================================ producer ================================
    // Lane c owns chunk c of every tile: one TMA box of C rows x 64 elements per 128-byte K-block brings the
    // chunk's tokens (contiguous in the head-major copy) into the swizzled operand tile.  The key sums of the
    // tile's rows follow with 4-byte cp.async, four rows per lane.
    // Four neighbouring chunks that follow one another in the key copy (the pieces of one chunk of the
    // previous stage) travel as one box of 4 C rows through the second tensor map.
    const uint64_t kmap_ptr = reinterpret_cast<uint64_t>(&kmap), krun_ptr = reinterpret_cast<uint64_t>(&kmap_run);
    const int RUN = min(4, CPT);
    auto fetch_bounds = [&](int i) {
      if (i < my_tiles) {
        int* slot = s_bounds + (i % (kBoundsAhead + 1)) * 64;
        const int c = (tile_of(i) << cpt_log2) + lane;
        if (lane < CPT && c < n) {
          asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_u32(slot + lane)), "l"(gl + c));
          asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_u32(slot + 32 + lane)), "l"(gr + c));
        } else {
          slot[lane] = 0; slot[32 + lane] = 0;
        }
      }
      cp_async_commit();
    };
    for (int i = 0; i < kBoundsAhead; ++i) fetch_bounds(i);
    bool ok = true;
    PROF_DECL(4);
    for (int i = 0; i < my_tiles; ++i) {
      const int s = i % n_stages, rr = i % kRows;
      fetch_bounds(i + kBoundsAhead);
      cp_async_wait<kBoundsAhead>();           // the bounds of tile i have landed
      const int* slot = s_bounds + (i % (kBoundsAhead + 1)) * 64;
      const int l = slot[lane], rt = slot[32 + lane];
      if (i >= kRows) ok = mbar_wait(smem_u32(&s_rows_empty[rr]), ((i / kRows) - 1) & 1, &s_abort, p.status);
      PROF_LAP(0);
      if (ok && i >= n_stages) ok = mbar_wait(smem_u32(&s_empty[s]), ((i / n_stages) - 1) & 1, &s_abort, p.status);
      ok = __all_sync(0xffffffffu, ok);
      PROF_LAP(1);
      if (!ok) break;
      TileRows& tr = rows_ring[rr];
      const bool active = lane < CPT && l < rt && l <= pt && l >= 0;
      if (active && rt > p.T) atomicOr(p.status, HIPATTN_STATUS_TOKEN_RANGE);
      if (lane < CPT) {
        tr.left[lane] = l;
        tr.right[lane] = rt;
      }
      const unsigned act_mask = __ballot_sync(0xffffffffu, active);
      const uint32_t full = smem_u32(&s_full[s]);
      if (lane == 0) {
        const uint32_t bytes = (uint32_t)__popc(act_mask) * (uint32_t)(C * ROWB);
        asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}\n" ::"r"(full), "r"(bytes) : "memory");
      }
      __syncwarp();
      // is the aligned group of RUN chunks of this lane one contiguous run?
      bool run = RUN > 1;
      {
        const int first = lane & ~(RUN - 1);
        const int l_first = __shfl_sync(0xffffffffu, l, first);
        bool fits = active && l == l_first + ((lane - first) << c_log2);
        for (int o = 1; o < RUN; o <<= 1) {
          const int other = __shfl_xor_sync(0xffffffffu, fits ? 1 : 0, o);   // every lane takes part in the exchange
          fits = fits && other != 0;
        }
        run = run && fits;
      }
      if (active && (!run || (lane & (RUN - 1)) == 0)) {
        const uint32_t dst = smem_u32(sK + (size_t)s * K_TILE_BYTES) + (uint32_t)(lane << c_log2) * 128u;
        const uint64_t mp = run ? krun_ptr : kmap_ptr;
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
          asm volatile(
              "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
              ::"r"(dst + kb * K_BLOCK_BYTES), "l"(mp), "r"(kb * 64), "r"(key_base + l), "r"(full) : "memory");
      }
      // key sums of rows lane, lane + 32, lane + 64, lane + 96
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const int r = q4 * 32 + lane;
        const int cl = r >> c_log2;
        const int cl_l = __shfl_sync(0xffffffffu, l, cl), cl_r = __shfl_sync(0xffffffffu, rt, cl);
        const bool cl_act = (act_mask >> cl) & 1u;
        const int tk = cl_l + (r & (C - 1));
        if (cl_act && tk < cl_r && tk < p.T)
          asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_u32(&tr.kabs[r])), "l"(p.key_abs + key_base + tk));
      }
      asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(smem_u32(&s_rows_full[rr])) : "memory");
      mbar_arrive(smem_u32(&s_rows_full[rr]));
      PROF_LAP(2);
    }
    cp_async_wait<0>();
    PROF_FLUSH(8, 4, lane == 0);
  } else if (my_tiles > 0 && warp == 8) {
    // ================================ MMA issuer ================================
    const uint32_t idesc = make_idesc(DT == HIPATTN_BF16 ? 1 : 0, 128, N, 0);
    // descriptors of the D / 16 k-steps for stage 0; a stage adds its offset to the 14-bit address field
    uint64_t da0[D / 16], db0[D / 16];
#pragma unroll
    for (int k = 0; k < D / 16; ++k) {
      da0[k] = make_desc(smem_u32(sK) + (k >> 2) * K_BLOCK_BYTES + (k & 3) * 32, 16, 1024);
      db0[k] = make_desc(smem_u32(sQ) + (k >> 2) * Q_BLOCK_BYTES + (k & 3) * 32, 16, 1024);
    }
    PROF_DECL(3);
#ifdef HIPATTN_SCAN_PROFILE
    long long prof_tm_[2] = {0, 0};
#endif
    for (int i = 0; i < my_tiles; ++i) {
      const int s = i % n_stages, a = i & 1;
      bool ok = mbar_wait(smem_u32(&s_full[s]), (i / n_stages) & 1, &s_abort, p.status);
      PROF_LAP(0);
      if (ok && i >= 2) ok = mbar_wait(smem_u32(&s_acc_empty[a]), ((i >> 1) - 1) & 1, &s_abort, p.status);
      ok = __all_sync(0xffffffffu, ok);
      PROF_LAP(1);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) {
        const uint64_t soff = (uint64_t)((s * K_TILE_BYTES) >> 4);
#ifdef HIPATTN_SCAN_PROFILE
        const long long tm0 = clock64();
#endif
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma(tmem + a * N, da0[k] + soff, db0[k], idesc, k > 0 ? 1u : 0u);
#ifdef HIPATTN_SCAN_PROFILE
        const long long tm1 = clock64();
#endif
        umma_commit(smem_u32(&s_empty[s]));
        umma_commit(smem_u32(&s_acc_full[a]));
#ifdef HIPATTN_SCAN_PROFILE
        prof_tm_[0] += tm1 - tm0; prof_tm_[1] += clock64() - tm1;
#endif
      }
      __syncwarp();
      PROF_LAP(2);
    }
    PROF_FLUSH(12, 3, lane == 0);
#ifdef HIPATTN_SCAN_PROFILE
    if (lane == 0 && p.stats) {
      atomicAdd(reinterpret_cast<unsigned long long*>(p.stats) + 30, (unsigned long long)prof_tm_[0]);
      atomicAdd(reinterpret_cast<unsigned long long*>(p.stats) + 31, (unsigned long long)prof_tm_[1]);
    }
#endif
  } else if (my_tiles > 0 && warp < 8) {
    // ================================ scores: thread = key = TMEM lane ================================
    // Two groups of four warps; group g takes the tiles of accumulator g (every other tile), so each has
    // two tile times for the TMEM reads and the rounding checks of one tile.
    const int wg = warp >> 2, qw = warp & 3, row_id = qw * 32 + lane;
    const uint32_t my_tmem = tmem + ((uint32_t)(qw * 32) << 16);
    const char* kbase = reinterpret_cast<const char*>(p.k_scaled);
    unsigned long long st_keys = 0;
    float eps_q[HB];
#pragma unroll
    for (int hh = 0; hh < HB; ++hh) eps_q[hh] = kEps * s_qmax[hh];
    int deferred = -1;      // tile whose score table waits for this warp's side-row copies
    PROF_DECL(4);
    for (int i = wg; i < my_tiles; i += 2) {
      const int a = i & 1, rr = i % kRows, sr = i % kScr;
      const TileRows& tr = rows_ring[rr];
      Scr& scr = scrs[sr];
      if (deferred >= 0 && i - deferred >= 4) {
        cp_async_wait<0>();
        mbar_arrive(smem_u32(&s_scr_full[deferred % kScr]));
        deferred = -1;
      }
      bool ok = mbar_wait(smem_u32(&s_rows_full[rr]), (i / kRows) & 1, &s_abort, p.status);
      PROF_LAP(0);
      ok = ok && mbar_wait(smem_u32(&s_acc_full[a]), (i >> 1) & 1, &s_abort, p.status);
      ok = __all_sync(0xffffffffu, ok);
      PROF_LAP(1);
      if (!ok) break;
      tc_fence_after();
      // the accumulator is read in as few TMEM loads as registers allow (64 columns per load and wait)
      float x[HB];
      constexpr int BW = N < 64 ? N : 64;     // 128 would not fit the register budget of 448 threads
#pragma unroll
      for (int c0 = 0; c0 < N; c0 += BW) {
        float v[BW];
        const uint32_t ta = my_tmem + a * N + c0;
        if (BW == 16) tmem_ld16(ta, v);
        else if (BW == 32) tmem_ld32(ta, v);
        else if (BW == 64) tmem_ld64(ta, v);
        else tmem_ld128(ta, v);
#pragma unroll
        for (int h2 = 0; h2 < BW / NR; ++h2) {
          float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four short chains instead of one long one
#pragma unroll
          for (int j = 0; j < NR; ++j)
            if (j < Rv) m4[j & 3] = fmaxf(m4[j & 3], v[h2 * NR + j]);
          x[c0 / NR + h2] = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&s_acc_empty[a]));
      PROF_LAP(2);
      if (i >= kScr) {
        ok = mbar_wait(smem_u32(&s_scr_empty[sr]), ((i / kScr) - 1) & 1, &s_abort, p.status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      const int idx = key_of(tr, row_id);
      const float s_abs = idx >= 0 ? tr.kabs[row_id] : 0.f;
      if (idx >= 0) st_keys += HB;
      unsigned unsure[HB], any = 0;
#pragma unroll
      for (int hh = 0; hh < HB; ++hh) {
        const float e_ = eps_q[hh] * s_abs * 1.01f;
        const bool sure = Elem<DT>::round(x[hh] - e_) == Elem<DT>::round(x[hh] + e_);
        unsure[hh] = __ballot_sync(0xffffffffu, idx >= 0 && (!sure || check));
        any |= unsure[hh];
        scr.score[hh][row_id] = check ? x[hh] : Elem<DT>::round(x[hh]);
      }
      // Rows of uncertain keys are fetched once more (asynchronously) into the score table, so that the
      // search warps re-score them from shared memory; what does not fit, and everything in check mode,
      // is left to the slower path that reads the key when it is needed.
      bool copies = false;
      if (any && !check) {
        if (deferred >= 0) {          // one outstanding group per warp
          cp_async_wait<0>();
          mbar_arrive(smem_u32(&s_scr_full[deferred % kScr]));
          deferred = -1;
        }
        unsigned todo = any;
        while (todo) {
          const int kl = __ffs(todo) - 1;
          todo &= todo - 1;
          int slot = 0;
          if (lane == 0) slot = atomicAdd(&scr.n_slots, 1);
          slot = __shfl_sync(0xffffffffu, slot, 0);
          if (slot >= kSideRows) continue;
          const int key = qw * 32 + kl;
          const int kidx = __shfl_sync(0xffffffffu, idx, kl);
          if (lane * 8 < ROWB) {
            const uint32_t dst = smem_u32(&scr.kraw[slot][lane * 8]);
            asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(dst), "l"(kbase + (int64_t)kidx * ROWB + lane * 8));
          }
          copies = true;
#pragma unroll
          for (int hh = 0; hh < HB; ++hh) {
            if ((unsure[hh] >> kl) & 1u) {
              int pi = kSidePairs;
              if (lane == 0) pi = atomicAdd(&scr.n_pairs, 1);
              pi = __shfl_sync(0xffffffffu, pi, 0);
              if (pi < kSidePairs) {
                if (lane == 0) {
                  scr.pair_key[pi] = (unsigned short)key;
                  scr.pair_head[pi] = (unsigned char)hh;
                  scr.pair_slot[pi] = (unsigned char)slot;
                }
                unsure[hh] &= ~(1u << kl);
              }
            }
          }
        }
        cp_async_commit();
      }
      if (lane == 0) {
#pragma unroll
        for (int hh = 0; hh < HB; ++hh) scr.need[hh][qw] = unsure[hh];
      }
      __syncwarp();
      if (copies) deferred = i;
      else mbar_arrive(smem_u32(&s_scr_full[sr]));
      PROF_LAP(3);
    }
    if (deferred >= 0) {
      cp_async_wait<0>();
      mbar_arrive(smem_u32(&s_scr_full[deferred % kScr]));
    }
    PROF_FLUSH(16, 4, warp == 0 && lane == 0);
    if (p.stats) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) st_keys += __shfl_xor_sync(0xffffffffu, st_keys, o);
      if (lane == 0) atomicAdd(reinterpret_cast<unsigned long long*>(p.stats) + ST_KEYS, st_keys);
    }
  } else if (my_tiles > 0 && warp >= 10) {
    // ================================ strict re-scores and the search ================================
    const int sw = warp - 10;
    const char* kbase = reinterpret_cast<const char*>(p.k_scaled);
    unsigned char* my_scratch = kscratch + sw * ROWB;
    unsigned long long st_fb = 0, st_wrong = 0;
    float st_ratio = 0.f;
    // Strict scores of up to BP (key, head) pairs at once: a lane runs up to four independent sequential
    // fp32 chains, one per (pair, pooled-row pass); GS lanes share a pair.
    constexpr int GS = NR < 32 ? NR : 32;     // lanes per pair
    constexpr int G = 32 / GS;                // pairs side by side in the warp
    constexpr int RP = NR / GS;               // row passes per pair
    constexpr int PPG = 2 / RP;               // pairs per lane group and batch (two chains per lane)
    constexpr int BP = G * PPG;
    const int grp = lane / GS, gl_lane = lane % GS;

    PROF_DECL(10);
    for (int i = sw; i < my_tiles; i += kSearchWarps) {
      const int rr = i % kRows, sr = i % kScr, tile = tile_of(i);
      const TileRows& tr = rows_ring[rr];
      Scr& scr = scrs[sr];
      bool ok = mbar_wait(smem_u32(&s_rows_full[rr]), (i / kRows) & 1, &s_abort, p.status);
      ok = ok && mbar_wait(smem_u32(&s_scr_full[sr]), (i / kScr) & 1, &s_abort, p.status);
      ok = __all_sync(0xffffffffu, ok);
      PROF_LAP(0);
      if (!ok) break;
      // bookkeeping of one re-scored pair (executed by one lane of the pair's group)
      auto commit_pair = [&](int key, int hh, float rawv) {
        const float ex = Elem<DT>::round(rawv);
        if (check) {
          const float x = scr.score[hh][key];
          const float e_ = kEps * s_qmax[hh] * tr.kabs[key] * 1.01f;
          const bool sure = Elem<DT>::round(x - e_) == Elem<DT>::round(x + e_);
          if (sure && Elem<DT>::round(x) != ex) ++st_wrong;
          if (e_ > 0.f) st_ratio = fmaxf(st_ratio, fabsf(x - rawv) / e_);
          if (!sure) ++st_fb;
        } else {
          ++st_fb;
        }
        scr.score[hh][key] = ex;
      };
      // Pairs [e0, e0 + cnt) of the tile's list (rows in scr.kraw), or, with `one_row` set, the single pair
      // (one_key, one_head) whose key row is at one_row.  A lane runs two sequential fp32 chains side by
      // side, branch-free, with the operands of four 16-byte pieces in registers at a time: a lone warp hides
      // no latency, so the loop is laid out as straight-line code the scheduler can overlap.
      auto strict_batch = [&](int e0, int cnt, const unsigned char* one_row, int one_key, int one_head) {
#ifdef HIPATTN_SCAN_PROFILE
        const long long tb0 = clock64();
        prof_[5] += 1; prof_[9] += cnt;
#endif
        uint32_t kp[2], qp[2];     // shared-space addresses of the chains' key rows / pooled-query rows
        bool valid[2];
        float acc[2] = {0.f, 0.f};
        const uint32_t sQ_s = smem_u32(sQ);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int e = (c / RP) * G + grp;
          const int r = (c % RP) * GS + gl_lane;
          valid[c] = e < cnt && r < Rv;
          const int ee = e0 + (e < cnt ? e : 0);
          const int hd = one_row ? one_head : (int)scr.pair_head[ee];
          kp[c] = smem_u32(one_row ? one_row : scr.kraw[scr.pair_slot[ee]]);
          const int qrow = hd * NR + (r < NR ? r : 0);
          qp[c] = sQ_s + qrow * 128;
          valid[c] = valid[c];
        }
        const uint32_t qx0 = (uint32_t)((qp[0] >> 7) & 7u), qx1 = (uint32_t)((qp[1] >> 7) & 7u);   // swizzle phase of the rows
#ifdef HIPATTN_SCAN_PROFILE
        const long long tb1 = clock64();
#endif
#pragma unroll
        for (int pb = 0; pb < PIECES; pb += 4) {
          uint4 q0[4], q1[4], k0[4], k1[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int pc = pb + j;
            q0[j] = lds128(qp[0] + (pc >> 3) * Q_BLOCK_BYTES + ((((uint32_t)pc & 7u) ^ qx0) << 4));
            q1[j] = lds128(qp[1] + (pc >> 3) * Q_BLOCK_BYTES + ((((uint32_t)pc & 7u) ^ qx1) << 4));
            k0[j] = lds128(kp[0] + pc * 16);
            k1[j] = lds128(kp[1] + pc * 16);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float a0 = acc[0], a1 = acc[1];
            a0 = fmaf(lo_f32<DT>(q0[j].x), lo_f32<DT>(k0[j].x), a0);  a1 = fmaf(lo_f32<DT>(q1[j].x), lo_f32<DT>(k1[j].x), a1);
            a0 = fmaf(hi_f32<DT>(q0[j].x), hi_f32<DT>(k0[j].x), a0);  a1 = fmaf(hi_f32<DT>(q1[j].x), hi_f32<DT>(k1[j].x), a1);
            a0 = fmaf(lo_f32<DT>(q0[j].y), lo_f32<DT>(k0[j].y), a0);  a1 = fmaf(lo_f32<DT>(q1[j].y), lo_f32<DT>(k1[j].y), a1);
            a0 = fmaf(hi_f32<DT>(q0[j].y), hi_f32<DT>(k0[j].y), a0);  a1 = fmaf(hi_f32<DT>(q1[j].y), hi_f32<DT>(k1[j].y), a1);
            a0 = fmaf(lo_f32<DT>(q0[j].z), lo_f32<DT>(k0[j].z), a0);  a1 = fmaf(lo_f32<DT>(q1[j].z), lo_f32<DT>(k1[j].z), a1);
            a0 = fmaf(hi_f32<DT>(q0[j].z), hi_f32<DT>(k0[j].z), a0);  a1 = fmaf(hi_f32<DT>(q1[j].z), hi_f32<DT>(k1[j].z), a1);
            a0 = fmaf(lo_f32<DT>(q0[j].w), lo_f32<DT>(k0[j].w), a0);  a1 = fmaf(lo_f32<DT>(q1[j].w), lo_f32<DT>(k1[j].w), a1);
            a0 = fmaf(hi_f32<DT>(q0[j].w), hi_f32<DT>(k0[j].w), a0);  a1 = fmaf(hi_f32<DT>(q1[j].w), hi_f32<DT>(k1[j].w), a1);
            acc[0] = a0; acc[1] = a1;
          }
        }
#ifdef HIPATTN_SCAN_PROFILE
        const long long tb2 = clock64();
#endif
        float best[PPG];
#pragma unroll
        for (int q_ = 0; q_ < PPG; ++q_) best[q_] = -INFINITY;
#pragma unroll
        for (int c = 0; c < 2; ++c)
          if (valid[c]) best[c / RP] = fmaxf(best[c / RP], acc[c]);
#pragma unroll
        for (int q_ = 0; q_ < PPG; ++q_) {
#pragma unroll
          for (int o = GS / 2; o > 0; o >>= 1) best[q_] = fmaxf(best[q_], __shfl_xor_sync(0xffffffffu, best[q_], o));
        }
        if (gl_lane == 0) {
#pragma unroll
          for (int q_ = 0; q_ < PPG; ++q_) {
            const int e = q_ * G + grp;
            if (e < cnt) {
              if (one_row) commit_pair(one_key, one_head, best[q_]);
              else commit_pair(scr.pair_key[e0 + e], scr.pair_head[e0 + e], best[q_]);
            }
          }
        }
#ifdef HIPATTN_SCAN_PROFILE
        const long long tb3 = clock64();
        prof_[6] += tb1 - tb0; prof_[7] += tb2 - tb1; prof_[8] += tb3 - tb2;
#endif
      };
      // ---- uncertain pairs whose key rows were set aside ----
      const int np = min(scr.n_pairs, kSidePairs);
      for (int e0 = 0; e0 < np; e0 += BP) strict_batch(e0, min(BP, np - e0), nullptr, 0, 0);
      PROF_LAP(3);
      // ---- the rest: the key row is fetched from global memory ----
      const unsigned my_need = lane < HB * 4 ? (&scr.need[0][0])[lane] : 0u;
      if (__any_sync(0xffffffffu, my_need != 0u)) {
#pragma unroll 1
        for (int hq = 0; hq < HB * 4; ++hq) {
          unsigned need = __shfl_sync(0xffffffffu, my_need, hq);
          while (need) {
            const int key = (hq & 3) * 32 + __ffs(need) - 1;
            need &= need - 1;
            __syncwarp();
            if (lane * 8 < ROWB)
              *reinterpret_cast<uint2*>(my_scratch + lane * 8) =
                  *reinterpret_cast<const uint2*>(kbase + (int64_t)key_of(tr, key) * ROWB + lane * 8);
            __syncwarp();
            strict_batch(0, 1, my_scratch, key, hq >> 2);
          }
        }
      }
      __syncwarp();
      PROF_LAP(1);
      // ---- the halving search of every (chunk, head) of the tile over the stored scores ----
      const int walkers = HB << cpt_log2;
      for (int w0 = 0; w0 < walkers; w0 += 32) {
        const int w = w0 + lane;
        const int hh = w % HB, cl = w / HB;
        const int c = (tile << cpt_log2) + cl;
        const bool live = w < walkers && c < n;
        float score = HIPATTN_SCORE_INIT;
        if (live) {
          int l = tr.left[cl], rt = tr.right[cl];
          const int base = l;
          const int gm = s_gmax[c >> bc_log2];
          const int rounds = gm >= 1 ? 32 - __clz(gm) : 0;
          const float* sc = &scr.score[hh][cl << c_log2];
          for (int it = 0; it < rounds; ++it) {
            if (!(l < rt && l <= pt && l >= 0)) break;
            const int mid = (l + rt) >> 1;
            const float sl = sc[min(((l + mid) >> 1) - base, C - 1)];
            const float sr_ = sc[min(((mid + rt) >> 1) - base, C - 1)];
            const bool win = sl > sr_;
            if (win) rt = mid; else l = mid;
            score = fmaxf(score, win ? sl : sr_);
          }
          const int64_t o = (row * p.H + h0 + hh) * n + c;
          if (p.left_out) p.left_out[o] = l;
          if (p.right_out) p.right_out[o] = rt;
          if (p.score_out) p.score_out[o] = score;
        }
        // head maximum inside the batch (adjacent lanes), then one atomic per chunk
        float best = score;
#pragma unroll
        for (int o = 1; o < HB; o <<= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, o));
        if (live && hh == 0 && best > HIPATTN_SCORE_INIT) atomicMax(p.score_max + row * n + c, encode_score(best));
      }
      __syncwarp();
      if (lane == 0) {
        scr.n_slots = 0;
        scr.n_pairs = 0;
        mbar_arrive(smem_u32(&s_scr_empty[sr]));
        mbar_arrive(smem_u32(&s_rows_empty[rr]));
      }
      PROF_LAP(2);
    }
    PROF_FLUSH(20, 10, warp == 10 && lane == 0);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      st_fb += __shfl_xor_sync(0xffffffffu, st_fb, o);
      st_wrong += __shfl_xor_sync(0xffffffffu, st_wrong, o);
      st_ratio = fmaxf(st_ratio, __shfl_xor_sync(0xffffffffu, st_ratio, o));
    }
    if (p.stats && lane == 0) {
      unsigned long long* st = reinterpret_cast<unsigned long long*>(p.stats);
      atomicAdd(st + ST_FALLBACK, st_fb);
      atomicAdd(st + ST_WRONG, st_wrong);
      atomicMax(reinterpret_cast<unsigned int*>(p.stats + ST_RATIO_BITS), __float_as_uint(st_ratio));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against the driver library)
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// The head-major key copy as a 2-D tensor [B * HKV * T rows, D elements]; a box is one chunk (C rows) of one
// 128-byte K-block (64 elements), written with the 128-byte swizzle of the MMA operand layout.
int make_key_map(const hipattn_scan_params_t& p, int box_rows, CUtensorMap* map) {
  EncodeTiledFn enc = encode_tiled_fn();
  HIPATTN_REQUIRE(enc != nullptr, HIPATTN_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {(cuuint64_t)p.D, (cuuint64_t)p.B * p.HKV * p.T};
  const cuuint64_t strides[1] = {(cuuint64_t)p.D * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, p.dtype == HIPATTN_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                         const_cast<void*>(p.k_scaled), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  HIPATTN_REQUIRE(r == CUDA_SUCCESS, HIPATTN_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return HIPATTN_OK;
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
  // shared memory: 1 KB alignment slack, pooled queries, the two table rings, scratch rows, group maxima, then
  // as many key tiles as fit beside ~2 KB of static data
  const size_t fixed = 1024 + (size_t)KB * N * 128 + kScr * sizeof(TileScores<HB, D * 2>) + kRows * sizeof(TileRows) +
                       kSearchWarps * D * 2 + (size_t)n_groups * sizeof(int);
  const size_t tile_bytes = (size_t)KB * 128 * 128;
  int n_stages = (int)((224 * 1024 - fixed) / tile_bytes);
  n_stages = n_stages > kMaxStages ? kMaxStages : n_stages;
  HIPATTN_REQUIRE(n_stages >= 2, HIPATTN_ERR_UNSUPPORTED, "dense scan stage: %zu bytes of fixed shared memory leave no room for the key ring", fixed);
  const size_t smem = fixed + n_stages * tile_bytes;
  CUtensorMap kmap, kmap_run;
  int rc = make_key_map(p, 1 << c_log2, &kmap);
  if (rc) return rc;
  rc = make_key_map(p, (4 << c_log2) > 128 ? 128 : (4 << c_log2), &kmap_run);
  if (rc) return rc;
  const int64_t units = (int64_t)p.B * p.HKV * BDST * (Gq / HB);
  int n_split = 1;   // few units (short prefill chunks): split the tiles of a unit over several CTAs
  if (units < 148) {
    const int64_t want = (148 + units - 1) / units;
    n_split = (int)(want < tiles_total ? want : tiles_total);
  }
  const int64_t grid = units * n_split;
  HIPATTN_REQUIRE(grid > 0 && grid < 0x7fffffffLL, HIPATTN_ERR_INVALID, "scan grid of %lld blocks", (long long)grid);
  auto kern = scan_dense_tcgen05_kernel<DT, D, NR, HB>;
  HIPATTN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<(unsigned)grid, kDenseThreads, smem, stream>>>(p, kmap, kmap_run, c_log2, n_split, tiles_total, n_stages, p.mode == HIPATTN_SCAN_CHECK ? 1 : 0);
  return check_launch("scan_dense_tcgen05_kernel");
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

// Takes the shapes of the round-based tcgen05 scan when the stage's chunk size is known, a power of
// two of at most 128, and small enough that scoring the whole chunk gathers no more key rows than the
// rounds of the heads that share it.
int scan_dense_tcgen05(const hipattn_scan_params_t& p, cudaStream_t stream, bool* handled) {
  *handled = false;
  const int R = p.block_size_q / p.stride_q;
  const int rows = min(R, cdiv(p.TQ, p.stride_q));
  if (p.mode == HIPATTN_SCAN_STRICT || p.dtype == HIPATTN_F32 || rows <= 1 || (R % 16) != 0 || R > 64 || (p.D != 64 && p.D != 128)) return HIPATTN_OK;
  if (p.key_abs == nullptr || p.k_scaled == nullptr) return HIPATTN_OK;
  if ((int64_t)p.B * p.T * p.HKV >= 0x7fffffffLL) return HIPATTN_OK;
  const int C = p.chunk_size;
  if (C < 8 || C > 128 || (C & (C - 1)) != 0) return HIPATTN_OK;   // a chunk is a whole number of 8-row swizzle atoms
  if (((uintptr_t)p.k_scaled % 16) != 0) return HIPATTN_OK;
  const char* v = getenv("HIPATTN_SCAN_KERNEL");
  if (v && (strcmp(v, "mma") == 0 || strcmp(v, "rounds") == 0)) return HIPATTN_OK;
  int c_log2 = 0;
  while ((1 << c_log2) < C) ++c_log2;
  const int Gq = p.H / p.HKV;
  const int NRp = R <= 16 ? 16 : (R <= 32 ? 32 : 64);
  int HB = 4;
  while (HB > 1 && (Gq % HB != 0 || HB * NRp > 256)) HB >>= 1;
  // Whole-chunk scoring gathers fewer rows than the rounds when C <= HB * 2 * (log2 C + 1), but its single
  // producer / issuer warps are not yet faster than the many CTAs of the round-by-round kernel: opt-in only.
  const char* mc = getenv("HIPATTN_SCAN_DENSE_MAX_CHUNK");   // chunk sizes up to this use whole-chunk scoring (default: none)
  const int max_chunk = mc ? atoi(mc) : 0;
  if (!(v && strcmp(v, "dense") == 0) && C > max_chunk) return HIPATTN_OK;
  *handled = true;
  if (p.dtype == HIPATTN_BF16) return p.D == 128 ? dispatch_rows<HIPATTN_BF16, 128>(p, c_log2, HB, stream) : dispatch_rows<HIPATTN_BF16, 64>(p, c_log2, HB, stream);
  return p.D == 128 ? dispatch_rows<HIPATTN_F16, 128>(p, c_log2, HB, stream) : dispatch_rows<HIPATTN_F16, 64>(p, c_log2, HB, stream);
}

}  // namespace hipattn
