// Scan stage of the mask estimator for 16-bit prefill on the tcgen05 tensor cores.
//
// Same contract as the strict kernel (scan_stage.cu): the score of a candidate key is
// max over pooled rows of round_to_dtype(dot), the dot product being the sequential fp32 accumulation
// over the head dimension.  As in the mma.sync kernel (scan_stage_mma.cu) the dot products are first
// computed approximately on the tensor cores and a key whose rounded score could change within the
// error radius eps = kEps * max|q'| * sum_d |k'_d| is re-scored by the strict definition, so decisions
// and stored scores are those of the strict kernel.
//
// Layout of one round: a CTA of 128 threads owns 64 chunks; thread t owns ONE candidate key
// (chunk t / 2, side t % 2).  The 128 candidate rows are gathered with 16-byte cp.async straight into
// the 128-byte-swizzled K-major operand layout (A, M = 128); the pooled queries sit in shared memory
// as the B operand (N = 16 / 32 / 64 / 128 rows).  D = K Q^T lands in TMEM with lane = key and
// column = pooled row, so thread t reads its own lane with one tcgen05.ld and takes the row maximum
// in registers: no shuffles, no ldmatrix, and one MMA issue per 16 head-dim elements for the whole CTA.
//
// The keys are read from a per-call copy that is already multiplied by the key scale and rounded
// (hipattn_scan_prepare_keys), dense and head-major [B, HKV, T, D] whatever the layout of the cache, so the
// gather needs no page-table lookups and no arithmetic between global and shared memory.
//
// Every mbarrier wait is bounded; when one runs out the CTA raises HIPATTN_STATUS_TIMEOUT and leaves
// through the normal exit, which frees its TMEM columns.
#include <cstdlib>
#include <cstring>

#include "scan_common.cuh"
#include "tcgen05_common.cuh"

namespace hipattn {
namespace {

// the CTA's small shared variables (behind the operand tiles in dynamic shared memory)
// (kept at 56 bytes: with the 16-row operand tiles six CTAs share a multiprocessor's shared memory to the byte)
struct ScanShared {
  unsigned long long mbar;
  uint32_t tmem;
  int abort;
  int g[2][4];      // per-warp largest chunk of the current chunk block, double buffered; during set-up g[1][2] holds the
                    // block's smallest position and g[1][3] the largest |pooled query| (read before g[1] is first written,
                    // which happens behind the first chunk block's barrier)
  unsigned char fetched[4];   // [r % 3]: "some warp fetched rows in round r"
  int pad_;
};
constexpr uint32_t kScanSlack = 896;   // padding reserved in front of the tiles

// Resident CTAs per multiprocessor the register allocation aims at: six with 16 or 32 pooled rows (80 registers; shared
// memory holds six 37 KB CTAs; at 92 registers only five are resident and stages 0 and 1 of the 128k prefill take 8 %
// longer), four with 64, three with 128 (shared memory).
// STREAM = in-kernel RoPE, backend "streaming": the prepared copy holds the keys as they are (head-major, neither scaled
// nor rotated); every thread rotates the row it asked for to its chunk's index, scales it and sums its magnitude in the
// operand tile, between the landing of the copies and the round's barrier.
template <int DT, int D, int NR, bool STREAM>
__global__ void __launch_bounds__(128, NR <= 32 ? (STREAM ? 5 : 6) : (NR <= 64 ? 4 : 3)) scan_stage_tcgen05_kernel(const hipattn_scan_params_t p, int nblk, int nblk_total, int check) {
  constexpr int ROWB = D * 2;                 // bytes per key / query row
  constexpr int PIECES = ROWB / 16;
  constexpr int KB = D / 64;                  // 128-byte K-blocks per row
  constexpr int K_BLOCK_BYTES = 128 * 128;    // one K-block of the key tile: 128 rows x 128 B
  constexpr int Q_BLOCK_BYTES = NR * 128;
  constexpr uint32_t TMEM_COLS = NR < 32 ? 32 : NR;
  // All shared memory is dynamic and the small variables sit behind the operand tiles, so that nothing precedes the
  // tiles in the CTA's window: the tiles then need no padding to their 1024-byte alignment and six CTAs of the
  // 16-row variant fit an SM (kScanSlack covers a window that is only 128-byte aligned).
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw & 1023u)) & 1023u;
  unsigned char* smem = smem_raw + pad;
  unsigned char* sK = smem;                                  // [KB][128 keys][128 B], swizzled
  unsigned char* sQ = sK + KB * K_BLOCK_BYTES;               // [KB][NR rows][128 B], swizzled
  ScanShared& sh = *reinterpret_cast<ScanShared*>(sQ + KB * Q_BLOCK_BYTES);
  if (pad > kScanSlack) {   // never expected: the launch reserved less padding than this window needs
    if (threadIdx.x == 0) atomicOr(p.status, HIPATTN_STATUS_TIMEOUT);
    return;
  }

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int Gq = p.H / p.HKV;
  const int BDST = cdiv(p.TQ, p.block_size_q);
  int64_t bid = blockIdx.x;
  const int cblk = (int)(bid % nblk); bid /= nblk;
  const int g = (int)(bid % Gq); bid /= Gq;
  const int d = (int)(bid % BDST); bid /= BDST;
  const int hkv = (int)(bid % p.HKV); bid /= p.HKV;
  const int b = (int)bid;
  const int h = hkv * Gq + g;

  const int R = p.block_size_q / p.stride_q;
  const int t0 = d * p.block_size_q;
  int Rv = 0;
  if (t0 < p.TQ) Rv = min(R, (p.TQ - t0 + p.stride_q - 1) / p.stride_q);
  const uint32_t mbar = smem_u32(&sh.mbar);

  // ---- set-up: barrier, TMEM, pooled queries as the B operand ----
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(mbar));
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    sh.abort = 0;
    sh.g[1][3] = 0;
    sh.fetched[0] = sh.fetched[1] = sh.fetched[2] = 0;
  }
  // The block's query rows go to shared memory (the key tile is free until the first round) with one batch of
  // asynchronous copies, issued before the TMEM allocation so that the trip to DRAM overlaps it: the pooled queries are
  // then computed from shared memory instead of through one dependent global load per row.
  const int rows_here = max(0, min(p.block_size_q, p.TQ - t0));
  const bool staged = (size_t)p.block_size_q * ROWB <= (size_t)KB * K_BLOCK_BYTES;
  if (staged) {
    using T = typename Elem<DT>::type;
    const T* qb = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_stride_b + (int64_t)h * p.q_stride_h;
    for (int i = tid; i < rows_here * PIECES; i += 128) {
      const int r = i / PIECES, pc = i % PIECES;
      cp_async16(sK + (size_t)r * ROWB + pc * 16, qb + (int64_t)(t0 + r) * p.q_stride_t + pc * 8);
    }
    cp_async_commit();
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&sh.tmem)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    const int m = block_min_position(p, b, t0, Rv, lane);
    if (lane == 0) sh.g[1][2] = m;
  }
  cp_async_wait<0>();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh.tmem;

  float qmax_local = 0.f;
  for (int i = tid; i < NR * PIECES; i += 128) {
    const int r = i / PIECES, pc = i % PIECES;
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = 0.f;
    if (r < Rv) {
      if (staged) pooled_query_piece_staged<DT>(p, sK, ROWB, r * p.stride_q, rows_here, pc, v, b, t0);
      else pooled_query_piece<DT>(p, b, h, t0 + r * p.stride_q, pc, v);
    }
    uint4 w;
    w.x = pack2<DT>(v[0], v[1]); w.y = pack2<DT>(v[2], v[3]); w.z = pack2<DT>(v[4], v[5]); w.w = pack2<DT>(v[6], v[7]);
    *reinterpret_cast<uint4*>(sQ + (pc >> 3) * Q_BLOCK_BYTES + sw128(r, pc & 7)) = w;
#pragma unroll
    for (int e = 0; e < 8; ++e) qmax_local = fmaxf(qmax_local, fabsf(v[e]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) qmax_local = fmaxf(qmax_local, __shfl_xor_sync(0xffffffffu, qmax_local, o));
  if (lane == 0) atomicMax(&sh.g[1][3], __float_as_int(qmax_local));  // non-negative floats order as ints
  fence_async_smem();
  __syncthreads();

  const int pt = max(sh.g[1][2] - p.scan_window, 0);
  const float eps_q = kEps * __int_as_float(sh.g[1][3]);
  const int n = p.n_chunks;
  const int64_t row = (int64_t)b * BDST + d;
  const char* kbase = reinterpret_cast<const char*>(p.k_scaled);
  const uint32_t sK_u32 = smem_u32(sK), sQ_u32 = smem_u32(sQ);
  const uint32_t idesc = make_idesc(DT == HIPATTN_BF16 ? 1 : 0, 128, NR, 0);
  const uint64_t da0 = make_desc(sK_u32, 16, 1024), db0 = make_desc(sQ_u32, 16, 1024);
  const uint32_t my_tmem = tmem + ((uint32_t)(warp * 32) << 16);
  const int side = tid & 1;
  // in-kernel RoPE, backend "relative": the prepared keys come in two copies (rotated to position 0 / 1 for the left /
  // right candidate), and a key's score depends on the side it is proposed for, so no score is carried over
  const bool roped = p.rope_mode != HIPATTN_ROPE_NONE;
  const int side_rows = (roped && !STREAM) ? p.B * p.HKV * p.T : 0;
  unsigned long long st_keys = 0, st_fb = 0, st_wrong = 0;
  float st_ratio = 0.f;
  uint32_t phase = 0;

  // strict dot products of the key staged in row `srow`, by the whole warp (one pooled row per lane);
  // returns the largest one before rounding (rounding is monotonic, so it commutes with the maximum).
  // The key is read piece by piece from the operand tile (every lane the same address: a broadcast) and the loop is
  // unrolled over the whole row, so that the loads run ahead of the one chain of fused multiply-adds per lane.
  auto strict_score = [&](int srow) -> float {
    float best = -INFINITY;
    for (int r0 = 0; r0 < Rv; r0 += 32) {
      const int r = r0 + lane;
      const int rr = r < Rv ? r : 0;
      float acc = 0.f;
#pragma unroll
      for (int pc = 0; pc < PIECES; ++pc) {
        const uint4 qw = lds128(sQ_u32 + (pc >> 3) * Q_BLOCK_BYTES + sw128(rr, pc & 7));
        const uint4 kw = lds128(sK_u32 + (pc >> 3) * K_BLOCK_BYTES + sw128(srow, pc & 7));
        acc = fmaf(lo_f32<DT>(qw.x), lo_f32<DT>(kw.x), acc);
        acc = fmaf(hi_f32<DT>(qw.x), hi_f32<DT>(kw.x), acc);
        acc = fmaf(lo_f32<DT>(qw.y), lo_f32<DT>(kw.y), acc);
        acc = fmaf(hi_f32<DT>(qw.y), hi_f32<DT>(kw.y), acc);
        acc = fmaf(lo_f32<DT>(qw.z), lo_f32<DT>(kw.z), acc);
        acc = fmaf(hi_f32<DT>(qw.z), hi_f32<DT>(kw.z), acc);
        acc = fmaf(lo_f32<DT>(qw.w), lo_f32<DT>(kw.w), acc);
        acc = fmaf(hi_f32<DT>(qw.w), hi_f32<DT>(kw.w), acc);
      }
      if (r < Rv) best = fmaxf(best, acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, o));
    return best;
  };

  bool aborted = Rv == 0;
  int cbi = 0;
  int rr = 0;   // rounds executed by this CTA so far (the same number in every thread)
  // the bounds of a thread's chunk are requested one chunk block ahead, so that their latency is not part of the chain
  int next_left = 0, next_right = 0;
  if (cblk < nblk_total && cblk * 64 + (tid >> 1) < n) {
    next_left = __ldg(p.left + row * n + cblk * 64 + (tid >> 1));
    next_right = __ldg(p.right + row * n + cblk * 64 + (tid >> 1));
  }
  for (int cb = cblk; cb < nblk_total && !aborted; cb += nblk, ++cbi) {
    const int c = cb * 64 + (tid >> 1);
    const bool in_range = c < n;
    int left = next_left, right = next_right;
    next_left = next_right = 0;
    {
      const int cn = c + nblk * 64;
      if (cb + nblk < nblk_total && cn < n) {
        next_left = __ldg(p.left + row * n + cn);
        next_right = __ldg(p.right + row * n + cn);
      }
    }
    // halving rounds: fixed by the largest chunk of the reference group of block_chunk chunks that
    // holds this thread's chunk; a warp covers 16 chunks, the CTA 64
    {
      int m = in_range ? right - left : 0;
      if (p.block_chunk > 64) {
        const int gbase = (cb * 64 / p.block_chunk) * p.block_chunk;
        for (int i = tid; i < p.block_chunk; i += 128) {
          const int cc = gbase + i;
          if (cc < n) m = max(m, p.right[row * n + cc] - p.left[row * n + cc]);
        }
      }
      m = __reduce_max_sync(0xffffffffu, m);
      if (lane == 0) sh.g[cbi & 1][warp] = m;
    }
    __syncthreads();
    const int cta_max = max(max(sh.g[cbi & 1][0], sh.g[cbi & 1][1]), max(sh.g[cbi & 1][2], sh.g[cbi & 1][3]));
    const int gmax = p.block_chunk >= 64 ? cta_max
                     : (p.block_chunk == 32 ? max(sh.g[cbi & 1][warp], sh.g[cbi & 1][warp ^ 1]) : sh.g[cbi & 1][warp]);
    const int my_rounds = gmax >= 1 ? 32 - __clz(gmax) : 0;
    const int cta_rounds = cta_max >= 1 ? 32 - __clz(cta_max) : 0;
    float score = HIPATTN_SCORE_INIT;
    // The candidate that won the previous round and its score.  When the halved chunk proposes the same key again
    // (always in the last round, for one of the two candidates in the round before it) the score is known: the same
    // key against the same pooled queries, so the row is neither fetched nor multiplied again.
    int won_t = -1;
    float won_score = 0.f;

    for (int it = 0; it < cta_rounds; ++it) {
      // A warp goes straight from its decisions to the copies of its next 32 rows: those rows are its own (only this
      // warp re-reads them for a strict re-score) and the MMA that read the tile has completed for every warp.  The one
      // CTA-wide barrier of a round sits between the copies and the MMA; it also carries "is anybody still searching".
      const bool act = in_range && it < my_rounds && left < right && left <= pt && left >= 0;
      const int mid = (left + right) >> 1;
      int tk = side ? ((mid + right) >> 1) : ((left + mid) >> 1);
      const int tk_asked = tk;
      const bool known = act && (!roped || STREAM) && tk == won_t;   // (streaming: a chunk's keys keep their rotation from round to round)
      int idx = -1;
      if (act && !known) {
        if (tk < 0 || tk >= p.T) {
          atomicOr(p.status, HIPATTN_STATUS_TOKEN_RANGE);
          tk = min(max(tk, 0), p.T - 1);
        }
        idx = (b * p.HKV + hkv) * p.T + tk + side * side_rows;   // (second copy: keys rotated for the right candidate)
        if (p.access_counter) mark_access(p.access_counter, p.access_stride_b, p.access_stride_h, p.access_n, p.k, b, hkv, tk);
      }
      // the key's magnitude is needed only after the MMA: requested here, its latency hides behind the row copies
      float s_abs = (!STREAM && idx >= 0) ? __ldg(p.key_abs + idx) : 0.f;
      // ---- gather this warp's 32 rows: 8 lanes per row, 128 contiguous bytes per row and instruction ----
      if (__any_sync(0xffffffffu, idx >= 0)) {   // a warp whose scores are all known (or inactive) copies nothing
      if (lane == 0) *(volatile unsigned char*)&sh.fetched[rr % 3] = 1;
#pragma unroll
      for (int r0 = 0; r0 < 32; r0 += 4) {
        const int j = r0 + (lane >> 3);
        const int src = __shfl_sync(0xffffffffu, idx, j);
        // no branch between the copies: the row of an inactive candidate is a copy of zero source bytes (zero fill)
        const bool live = src >= 0;
        const char* gp = kbase + (int64_t)(live ? src : 0) * ROWB + (lane & 7) * 16;
        const uint32_t sp = sK_u32 + sw128(warp * 32 + j, lane & 7);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) cp_async16_zfill(sp + kb * K_BLOCK_BYTES, gp + kb * 128, live);
      }
      }
      cp_async_commit();
      cp_async_wait<0>();
      if (STREAM) {
        // the 16 pieces of a row were copied by eight lanes: all of the warp's copies are visible after this point
        __syncwarp();
        if (idx >= 0) {
          if constexpr (D == 128) {
            const int r = warp * 32 + lane;
            const uint32_t s2 = pack_scalar2<DT>(p.k_scale);
#pragma unroll 2
            for (int pp = 0; pp < 8; ++pp) {
              const uint32_t a_lo = sK_u32 + sw128(r, pp), a_hi = a_lo + K_BLOCK_BYTES;
              uint4 lo = lds128(a_lo), hi = lds128(a_hi);
              rope_rotate_packed<DT>(lo, hi, rope_table_raw(p.rope_cos, p.rope_stride, p.rope_rows, c, pp),
                                     rope_table_raw(p.rope_sin, p.rope_stride, p.rope_rows, c, pp));
              uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                w[i] = mul2<DT>(w[i], s2);
                s_abs += fabsf(lo_f32<DT>(w[i])) + fabsf(hi_f32<DT>(w[i]));
              }
              sts128(a_lo, make_uint4(w[0], w[1], w[2], w[3]));
              sts128(a_hi, make_uint4(w[4], w[5], w[6], w[7]));
            }
          }
        }
      }
      fence_async_smem();
      tc_fence_before();
      // the barrier's result is one bit (any predicate non-zero): "somebody is still searching, or gave up"
      if (!__syncthreads_or(act || *(volatile int*)&sh.abort)) break;
      if (*(volatile int*)&sh.abort) { aborted = true; break; }
      // somebody fetched a row: the tile is multiplied; else every live score is known from the round before
      const bool scored = *(volatile unsigned char*)&sh.fetched[rr % 3] != 0;
      if (tid == 0) *(volatile unsigned char*)&sh.fetched[(rr + 2) % 3] = 0;   // next written two barriers from now
      ++rr;
      if (scored && tid == 0) {
        tc_fence_after();
        // the descriptors of the K-steps differ from the first one's in the start-address field only (shared-memory
        // addresses stay below 2^18, so the 14-bit field does not carry): one add each instead of building them anew
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma(tmem, da0 + (uint64_t)(((k >> 2) * K_BLOCK_BYTES + (k & 3) * 32) >> 4),
               db0 + (uint64_t)(((k >> 2) * Q_BLOCK_BYTES + (k & 3) * 32) >> 4), idesc, k > 0 ? 1u : 0u);
        umma_commit(mbar);
      }
      __syncwarp();
      bool ok = true;
      if (scored) {
        ok = mbar_wait(mbar, phase, &sh.abort, p.status);
        phase ^= 1u;
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
      }
      float x = -INFINITY;
      if (ok && scored) {
        // four short maximum chains; the row mask is only paid for by a ragged last query block.  128 pooled rows
        // are read as two halves of 64 columns so that the live registers stay those of the 64-row variant.
        constexpr int NLD = NR > 64 ? 64 : NR;
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c0 = 0; c0 < NR; c0 += NLD) {
          float v[NLD];
          if (NLD == 16) tmem_ld16(my_tmem + c0, v);
          else if (NLD == 32) tmem_ld32(my_tmem + c0, v);
          else tmem_ld64(my_tmem + c0, v);
          if (Rv >= NR) {
#pragma unroll
            for (int j = 0; j < NLD; ++j) m4[j & 3] = fmaxf(m4[j & 3], v[j]);
          } else {
#pragma unroll
            for (int j = 0; j < NLD; ++j)
              if (c0 + j < Rv) m4[j & 3] = fmaxf(m4[j & 3], v[j]);
          }
        }
        x = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      }
      const float e_ = eps_q * s_abs * 1.01f;
      float sc = Elem<DT>::round(x);
      const bool sure = Elem<DT>::round(x - e_) == Elem<DT>::round(x + e_);
      if (known) sc = won_score;
      unsigned need = __ballot_sync(0xffffffffu, idx >= 0 && ok && (!sure || check));
      while (need) {
        const int owner = __ffs(need) - 1;
        need &= need - 1;
        const float rawv = strict_score(warp * 32 + owner);
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
      const float other = __shfl_xor_sync(0xffffffffu, sc, 1);   // the other candidate of the same chunk
      const int other_t = __shfl_xor_sync(0xffffffffu, tk_asked, 1);
      if (act) {
        if (idx >= 0) st_keys += 1;
        const float sl = side ? other : sc, sr = side ? sc : other;
        const bool win = sl > sr;
        if (win) right = mid; else left = mid;
        score = fmaxf(score, win ? sl : sr);
        won_t = (win != (side != 0)) ? tk_asked : other_t;    // left candidate when it won, else the right one
        won_score = win ? sl : sr;
      }
    }

    if (in_range && side == 0 && !aborted) {
      if (score > HIPATTN_SCORE_INIT) atomicMax(p.score_max + row * n + c, encode_score(score));
      const int64_t o = (row * p.H + h) * n + c;
      if (p.left_out) p.left_out[o] = left;
      if (p.right_out) p.right_out[o] = right;
      if (p.score_out) p.score_out[o] = score;
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

template <int DT, int D, int NR, bool STREAM>
int launch(const hipattn_scan_params_t& p, cudaStream_t stream) {
  const size_t smem = kScanSlack + (size_t)(D / 64) * (128 * 128 + NR * 128) + sizeof(ScanShared);
  const int BDST = cdiv(p.TQ, p.block_size_q);
  const int nblk_total = cdiv(p.n_chunks, 64);
  const int64_t units = (int64_t)p.B * p.H * BDST;
  const int nblk = scan_ctas_per_unit(units, nblk_total, 148 * (NR <= 32 ? (STREAM ? 5 : 6) : (NR <= 64 ? 4 : 3)));
  const int64_t grid = units * nblk;
  HIPATTN_REQUIRE(grid > 0 && grid < 0x7fffffffLL, HIPATTN_ERR_INVALID, "scan grid of %lld blocks", (long long)grid);
  auto kern = scan_stage_tcgen05_kernel<DT, D, NR, STREAM>;
  HIPATTN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<(unsigned)grid, 128, smem, stream>>>(p, nblk, nblk_total, p.mode == HIPATTN_SCAN_CHECK ? 1 : 0);
  return check_launch("scan_stage_tcgen05_kernel");
}

template <int DT, int D>
int dispatch_rows(const hipattn_scan_params_t& p, cudaStream_t stream) {
  const int R = p.block_size_q / p.stride_q;
  if constexpr (D == 128) {
    if (p.rope_mode == HIPATTN_ROPE_STREAMING) {
      if (R <= 16) return launch<DT, D, 16, true>(p, stream);
      if (R <= 32) return launch<DT, D, 32, true>(p, stream);
      if (R <= 64) return launch<DT, D, 64, true>(p, stream);
      return launch<DT, D, 128, true>(p, stream);
    }
  }
  if (R <= 16) return launch<DT, D, 16, false>(p, stream);
  if (R <= 32) return launch<DT, D, 32, false>(p, stream);
  if (R <= 64) return launch<DT, D, 64, false>(p, stream);
  return launch<DT, D, 128, false>(p, stream);
}

// Scaled copy of the keys and their absolute sums: 16 / 8 lanes per row of 256 / 128 bytes.
struct PrepareRope {      // rotate every key to one fixed table position before scaling (scan backend "relative")
  const void* cos;
  const void* sin;
  int64_t stride;
  int rows, position;
};

template <int DT>
__global__ void scan_prepare_keys_kernel(const hipattn_tokens_t k, int D, int B, int T, int HKV, float k_scale, float* key_abs,
                                         unsigned char* k_scaled, uint32_t* status, const PrepareRope rope) {
  const int pieces = D * 2 / 16;
  const int rows_per_block = blockDim.x / pieces;
  const int sub = threadIdx.x / pieces, piece = threadIdx.x % pieces;
  const int64_t total = (int64_t)B * T * HKV;
  const uint32_t kscale2 = pack_scalar2<DT>(k_scale);
  for (int64_t r = (int64_t)blockIdx.x * rows_per_block + sub; r < total; r += (int64_t)gridDim.x * rows_per_block) {
    const int hkv = (int)(r % HKV);
    const int64_t bt = r / HKV;
    const int t = (int)(bt % T), b = (int)(bt / T);
    const char* src = token_row(k, b, t, hkv, 2, status);
    const uint4 w = k.fp8_e5m2 ? widen_fp8_e5m2<DT>(*reinterpret_cast<const uint2*>(src + piece * 8))
                               : *reinterpret_cast<const uint4*>(src + piece * 16);
    const int64_t ro = ((int64_t)b * HKV + hkv) * T + t;     // head-major: the tokens of a KV head are contiguous
    // scales a piece, sums its magnitude over the row and stores both into copy `side`
    auto emit = [&](uint32_t* v, int side) {
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[i] = mul2<DT>(v[i], kscale2);
        const uint32_t m = v[i] & 0x7fff7fffu;
        s += lo_f32<DT>(m) + hi_f32<DT>(m);
      }
      const int64_t rs = ro + (int64_t)side * total;
      if (k_scaled) *reinterpret_cast<uint4*>(k_scaled + rs * (int64_t)(D * 2) + piece * 16) = make_uint4(v[0], v[1], v[2], v[3]);
      for (int o = pieces >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (piece == 0 && key_abs) key_abs[rs] = s;
    };
    if (rope.cos != nullptr) {
      const int half = pieces >> 1, pr = piece < half ? piece + half : piece - half;
      const uint4 wr = k.fp8_e5m2 ? widen_fp8_e5m2<DT>(*reinterpret_cast<const uint2*>(src + pr * 8))
                                  : *reinterpret_cast<const uint4*>(src + pr * 16);
      // rotation on packed 16-bit pairs: products and sum round once to the element type, as the scalar form does
      using P = typename Pair16<DT>::type;
      const uint32_t xv[4] = {w.x, w.y, w.z, w.w}, rv[4] = {wr.x, wr.y, wr.z, wr.w};
      // position -1: both copies of the "relative" backend (table positions 0 and 1) from one read of the row
      const int n_pos = rope.position < 0 ? 2 : 1;
      for (int sd = 0; sd < n_pos; ++sd) {
        const int pos = rope.position < 0 ? sd : rope.position;
        const uint4 tc = rope_table_raw(rope.cos, rope.stride, rope.rows, pos, piece % half);
        const uint4 ts = rope_table_raw(rope.sin, rope.stride, rope.rows, pos, piece % half);
        const uint32_t cv[4] = {tc.x, tc.y, tc.z, tc.w}, sv[4] = {ts.x, ts.y, ts.z, ts.w};
        uint32_t v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const P xp = *reinterpret_cast<const P*>(&xv[i]), rp = *reinterpret_cast<const P*>(&rv[i]);
          const P cp = *reinterpret_cast<const P*>(&cv[i]), sp = *reinterpret_cast<const P*>(&sv[i]);
          const P rot = __hadd2_rn(__hmul2_rn(xp, cp), __hmul2_rn(piece < half ? __hneg2(rp) : rp, sp));
          v[i] = *reinterpret_cast<const uint32_t*>(&rot);
        }
        emit(v, sd);
      }
    } else {
      uint32_t v[4] = {w.x, w.y, w.z, w.w};
      emit(v, 0);
    }
  }
}

}  // namespace

int scan_prepare_keys(const hipattn_tokens_t& k, int dtype, int D, int B, int T, int HKV, float k_scale, float* key_abs,
                      void* k_scaled, uint32_t* status, cudaStream_t stream, const void* rope_cos, const void* rope_sin,
                      int64_t rope_stride, int rope_rows, int rope_position) {
  const PrepareRope rope{rope_cos, rope_sin, rope_stride, rope_rows, rope_position};
  HIPATTN_REQUIRE(dtype == HIPATTN_BF16 || dtype == HIPATTN_F16, HIPATTN_ERR_UNSUPPORTED, "scan_prepare_keys: 16-bit element types only");
  HIPATTN_REQUIRE(D == 64 || D == 128, HIPATTN_ERR_UNSUPPORTED, "scan_prepare_keys: head dimension %d is not built (64, 128)", D);
  const int64_t total = (int64_t)B * T * HKV;
  const int rows_per_block = 256 / (D * 2 / 16);
  int64_t grid = (total + rows_per_block - 1) / rows_per_block;
  if (grid > 148 * 32) grid = 148 * 32;
  if (dtype == HIPATTN_BF16)
    scan_prepare_keys_kernel<HIPATTN_BF16><<<(unsigned)grid, 256, 0, stream>>>(k, D, B, T, HKV, k_scale, key_abs, (unsigned char*)k_scaled, status, rope);
  else
    scan_prepare_keys_kernel<HIPATTN_F16><<<(unsigned)grid, 256, 0, stream>>>(k, D, B, T, HKV, k_scale, key_abs, (unsigned char*)k_scaled, status, rope);
  return check_launch("scan_prepare_keys_kernel");
}

// Takes 16-bit prefill shapes (16 to 128 pooled rows in multiples of 16, head dim 64 or 128) when the
// caller supplies the prepared keys; anything else is left to the other scan kernels.
int scan_stage_tcgen05(const hipattn_scan_params_t& p, cudaStream_t stream, bool* handled) {
  *handled = false;
  const int R = p.block_size_q / p.stride_q;
  const int rows = min(R, cdiv(p.TQ, p.stride_q));
  if (p.mode == HIPATTN_SCAN_STRICT || p.dtype == HIPATTN_F32 || rows <= 1 || (R % 16) != 0 || R > 128 || (p.D != 64 && p.D != 128)) return HIPATTN_OK;
  if (p.key_abs == nullptr || p.k_scaled == nullptr) return HIPATTN_OK;
  if ((int64_t)p.B * p.T * p.HKV * (p.rope_mode != HIPATTN_ROPE_NONE ? 2 : 1) >= 0x7fffffffLL) return HIPATTN_OK;
  // in-kernel RoPE: "relative" with the two rotated copies, "streaming" (head dim 128) with the plain head-major copy
  // (hipattn_scan_prepare_keys with k_scale = 1, k_scaled_sides = 1): the kernel rotates and scales in the operand tile
  if (p.rope_mode == HIPATTN_ROPE_RELATIVE && p.k_scaled_sides != 2) return HIPATTN_OK;
  if (p.rope_mode == HIPATTN_ROPE_STREAMING && !(p.k_scaled_sides == 1 && p.D == 128)) return HIPATTN_OK;
  const char* v = getenv("HIPATTN_SCAN_KERNEL");
  if (v && strcmp(v, "mma") == 0) return HIPATTN_OK;
  *handled = true;
  if (p.dtype == HIPATTN_BF16) return p.D == 128 ? dispatch_rows<HIPATTN_BF16, 128>(p, stream) : dispatch_rows<HIPATTN_BF16, 64>(p, stream);
  return p.D == 128 ? dispatch_rows<HIPATTN_F16, 128>(p, stream) : dispatch_rows<HIPATTN_F16, 64>(p, stream);
}

}  // namespace hipattn
