// Scan stage of the mask estimator for 16-bit prefill: warp-autonomous rounds, key rows held in registers.
//
// Same contract as the strict kernel (scan_stage.cu) and the same exact-fallback scheme as the other
// tensor-core scans: the dot products of a round are computed approximately with mma.sync, a key whose
// rounded score could change within eps = kEps * max|q'| * sum_d |k'_d| is re-scored by the strict
// definition, so decisions and stored scores are those of the strict kernel.
//
// What is different is where a round's chain of dependent steps lives.  A round is
//   decide -> addresses -> gather 2 key rows per chunk -> dot products -> maximum -> decide ...
// and its length, times the bytes a multiprocessor can keep in flight, sets the speed of the whole scan
// (the gathers hit L2).  Here a WARP owns 16 chunks (32 candidate keys) and runs that chain alone:
//   * the 32 rows go from global memory (the prepared, scaled, head-major key copy) straight into
//     registers in the B-operand layout of mma.sync m16n8k16 -- no shared-memory staging, no CTA-wide
//     barrier, no single MMA-issuing thread; four lanes read one row with 32-byte loads (lane t takes
//     bytes 32 t .. 32 t + 31 of every 128-byte line), so that one load instruction covers whole
//     128-byte lines of eight rows;
//   * the head dimension is contracted in a permuted order that the pooled-query (A) fragments follow:
//     the 8 elements of a 16-byte piece feed k-indices {2t, 2t+1, 2t+8, 2t+9} of two consecutive steps,
//     so that a piece is exactly the two B registers of two steps and nothing is shuffled;
//   * with 16 pooled rows the A fragments of the whole head dimension stay in registers for the life of
//     the CTA; with more rows they are re-read from a fragment-ordered shared-memory copy;
//   * the column maxima are reduced across the eight row groups by recursive halving (7 shuffles for a
//     round's 32 keys), which leaves every key's score in the lane that owns the key.
// What overlaps a warp's chain is the other resident warps (16 per multiprocessor at 128 registers).
#include <cstdlib>
#include <cstring>

#include "mma_common.cuh"
#include "scan_common.cuh"

namespace hipattn {
namespace {

constexpr int kQPad = 16;   // row padding of the row-major pooled-query copy (strict re-scores)

// 32 bytes from global memory through the read-only path with one instruction (the address is 32-byte aligned)
__device__ __forceinline__ void ldg256(const void* p, uint4& a, uint4& b) {
  asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
               : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(p));
}
// the 16-byte piece of a row that lane t holds as its ii-th: pieces 2 t and 2 t + 1 of every 128-byte line
__device__ __forceinline__ int piece_of(int t, int ii) { return 2 * t + (ii & 1) + 8 * (ii >> 1); }

template <int DT, int D, int MT>
__global__ void __launch_bounds__(128, MT == 1 ? 4 : 3) scan_stage_regs_kernel(const hipattn_scan_params_t p, int nblk, int nblk_total, int check) {
  constexpr int ROWB = D * 2;
  constexpr int PIECES = ROWB / 16;      // 16-byte pieces per row: 16 (D 128) or 8 (D 64)
  constexpr int NI = PIECES / 4;         // pieces per lane and row
  constexpr int QSTRIDE = ROWB + kQPad;
  constexpr int NR = 16 * MT;
  constexpr bool QREG = MT == 1;
  extern __shared__ __align__(16) unsigned char smem[];
  unsigned char* qrow = smem;                                   // [NR][QSTRIDE] row-major pooled queries
  uint4* qfrag = reinterpret_cast<uint4*>(smem + NR * QSTRIDE); // [MT][NI][2][32] fragment-ordered copy (MT > 1)
  __shared__ int s_pmin;
  __shared__ float s_qmax;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int Gq = p.H / p.HKV;
  const int BDST = cdiv(p.TQ, p.block_size_q);
  int64_t bid = blockIdx.x;
  const int cblk = (int)(bid % nblk); bid /= nblk;
  const int hg = (int)(bid % Gq); bid /= Gq;
  const int d = (int)(bid % BDST); bid /= BDST;
  const int hkv = (int)(bid % p.HKV); bid /= p.HKV;
  const int b = (int)bid;
  const int h = hkv * Gq + hg;

  const int R = p.block_size_q / p.stride_q;
  const int t0 = d * p.block_size_q;
  int Rv = 0;
  if (t0 < p.TQ) Rv = min(R, (p.TQ - t0 + p.stride_q - 1) / p.stride_q);

  // ---- pooled queries (identical arithmetic to the strict kernel), once per CTA ----
  if (tid == 0) s_qmax = 0.f;
  __syncthreads();
  float qmax_local = 0.f;
  for (int i = tid; i < NR * PIECES; i += 128) {
    const int r = i / PIECES, pc = i % PIECES;
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = 0.f;
    if (r < Rv) pooled_query_piece<DT>(p, b, h, t0 + r * p.stride_q, pc, v);
    uint4 w;
    w.x = pack2<DT>(v[0], v[1]); w.y = pack2<DT>(v[2], v[3]); w.z = pack2<DT>(v[4], v[5]); w.w = pack2<DT>(v[6], v[7]);
    *reinterpret_cast<uint4*>(qrow + r * QSTRIDE + pc * 16) = w;
    if (!QREG) {
      // piece pc = piece_of(t, ii) of row r is read by lane (r % 8) * 4 + t as half (r % 16) / 8 of its ii-th piece of
      // row tile r / 16
      const int t_ = (pc & 7) >> 1, ii_ = (pc & 1) + 2 * (pc >> 3);
      qfrag[(((r >> 4) * NI + ii_) * 2 + ((r >> 3) & 1)) * 32 + (r & 7) * 4 + t_] = w;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) qmax_local = fmaxf(qmax_local, fabsf(v[e]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) qmax_local = fmaxf(qmax_local, __shfl_xor_sync(0xffffffffu, qmax_local, o));
  if (lane == 0) atomicMax(reinterpret_cast<int*>(&s_qmax), __float_as_int(qmax_local));  // non-negative floats order as ints
  if (warp == 0) {
    const int m = block_min_position(p, b, t0, Rv, lane);
    if (lane == 0) s_pmin = m;
  }
  __syncthreads();
  if (Rv == 0) return;
  const int pt = max(s_pmin - p.scan_window, 0);
  const float eps_q = kEps * s_qmax;
  const int n = p.n_chunks;
  const int64_t row = (int64_t)b * BDST + d;
  const char* kbase = reinterpret_cast<const char*>(p.k_scaled);

  // A fragments of the 16 pooled rows, all steps, in registers
  uint4 qa[QREG ? NI : 1][2];
  if (QREG) {
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      qa[i][0] = *reinterpret_cast<const uint4*>(qrow + g * QSTRIDE + piece_of(t, i) * 16);
      qa[i][1] = *reinterpret_cast<const uint4*>(qrow + (g + 8) * QSTRIDE + piece_of(t, i) * 16);
    }
  }
  // rows of a ragged last block that do not exist: their dot products are masked out of the maximum
  const bool full_rows = Rv >= NR;

  // ownership: lane (g, t) owns the key of chunk (g / 2) * 4 + t of the warp's 16 chunks, side g % 2
  const int side = g & 1;
  const int my_chunk = (g >> 1) * 4 + t;
  unsigned long long st_keys = 0, st_fb = 0, st_wrong = 0;
  float st_ratio = 0.f;

  // strict dot products of key row `kidx` of the prepared copy, by the whole warp (one pooled row per lane); returns
  // the largest one before rounding (rounding is monotonic, so it commutes with the maximum)
  auto strict_score = [&](int kidx) -> float {
    const uint4* kr = reinterpret_cast<const uint4*>(kbase + (int64_t)kidx * ROWB);
    float best = -INFINITY;
    for (int r0 = 0; r0 < Rv; r0 += 32) {
      const int r = r0 + lane;
      const unsigned char* qr = qrow + (r < Rv ? r : 0) * QSTRIDE;
      float acc = 0.f;
#pragma unroll
      for (int pc = 0; pc < PIECES; ++pc) {
        const uint4 qw = *reinterpret_cast<const uint4*>(qr + pc * 16);
        const uint4 kw = __ldg(kr + pc);
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

  for (int cb = cblk; cb < nblk_total; cb += nblk) {
    const int wbase = cb * 64 + warp * 16;
    if (wbase >= n) continue;
    const int c = wbase + my_chunk;
    const bool in_range = c < n;
    int left = 0, right = 0;
    if (in_range) {
      left = __ldg(p.left + row * n + c);
      right = __ldg(p.right + row * n + c);
    }
    // halving rounds: fixed by the largest chunk of the reference group of block_chunk chunks that holds the chunk
    int gmax = in_range ? right - left : 0;
    if (p.block_chunk > 16) {
      const int gbase = (wbase / p.block_chunk) * p.block_chunk;
      for (int i = lane; i < p.block_chunk; i += 32) {
        const int cc = gbase + i;
        if (cc < n) gmax = max(gmax, __ldg(p.right + row * n + cc) - __ldg(p.left + row * n + cc));
      }
    }
    gmax = __reduce_max_sync(0xffffffffu, gmax);
    const int rounds = gmax >= 1 ? 32 - __clz(gmax) : 0;
    float score = HIPATTN_SCORE_INIT;
    // The candidate that won the previous round and its score.  When the halved chunk proposes the same key again (both
    // candidates of the last round, one of the round before it) the score is known -- the same key against the same
    // pooled queries -- and the row is neither fetched nor multiplied again.
    int won_t = -1;
    float won_score = 0.f;

    for (int it = 0; it < rounds; ++it) {
      const bool act = in_range && left < right && left <= pt && left >= 0;
      if (!__any_sync(0xffffffffu, act)) break;
      const int mid = (left + right) >> 1;
      int tk = side ? ((mid + right) >> 1) : ((left + mid) >> 1);
      const int tk_asked = tk;
      const bool known = act && tk == won_t;
      int idx = -1;
      if (act && !known) {
        if (tk < 0 || tk >= p.T) {
          atomicOr(p.status, HIPATTN_STATUS_TOKEN_RANGE);
          tk = min(max(tk, 0), p.T - 1);
        }
        idx = (b * p.HKV + hkv) * p.T + tk;
      }
      if (!__any_sync(0xffffffffu, idx >= 0)) {
        // every live chunk knows both scores (both candidates are the previous winner): equal scores keep the right half
        if (act) left = mid;
        continue;
      }
      const float s_abs = idx >= 0 ? __ldg(p.key_abs + idx) : 0.f;

      // ---- gather: group gi holds keys (gi, n), n = 0..7; lane (g, t) loads row n = g, 32 bytes of every line ----
      uint4 kv[4][NI];
#pragma unroll
      for (int gi = 0; gi < 4; ++gi) {
        const int src = __shfl_sync(0xffffffffu, idx, gi * 8 + (g & 1) * 4 + (g >> 1));
        const char* gp = kbase + (int64_t)(src >= 0 ? src : 0) * ROWB + t * 32;
#pragma unroll
        for (int i = 0; i < NI; i += 2) {
          if (src >= 0) ldg256(gp + (i >> 1) * 128, kv[gi][i], kv[gi][i + 1]);
          else kv[gi][i] = kv[gi][i + 1] = make_uint4(0, 0, 0, 0);
        }
      }

      // ---- dot products and column maxima: cm[gi * 2 + j] = max over rows of column 2 t + j of group gi ----
      float cm[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) cm[i] = -INFINITY;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        float acc[4][4];
#pragma unroll
        for (int gi = 0; gi < 4; ++gi) acc[gi][0] = acc[gi][1] = acc[gi][2] = acc[gi][3] = 0.f;
#pragma unroll
        for (int i = 0; i < NI; ++i) {
          uint4 a0, a1;
          if (QREG) { a0 = qa[i][0]; a1 = qa[i][1]; }
          else { a0 = qfrag[((mt * NI + i) * 2 + 0) * 32 + lane]; a1 = qfrag[((mt * NI + i) * 2 + 1) * 32 + lane]; }
          const uint32_t fa[4] = {a0.x, a1.x, a0.y, a1.y};
          const uint32_t fb[4] = {a0.z, a1.z, a0.w, a1.w};
#pragma unroll
          for (int gi = 0; gi < 4; ++gi) {
            mma16816<DT>(acc[gi], fa, kv[gi][i].x, kv[gi][i].y);
            mma16816<DT>(acc[gi], fb, kv[gi][i].z, kv[gi][i].w);
          }
        }
        const bool lo_ok = full_rows || mt * 16 + g < Rv, hi_ok = full_rows || mt * 16 + g + 8 < Rv;
#pragma unroll
        for (int gi = 0; gi < 4; ++gi) {
          if (lo_ok) { cm[gi * 2] = fmaxf(cm[gi * 2], acc[gi][0]); cm[gi * 2 + 1] = fmaxf(cm[gi * 2 + 1], acc[gi][1]); }
          if (hi_ok) { cm[gi * 2] = fmaxf(cm[gi * 2], acc[gi][2]); cm[gi * 2 + 1] = fmaxf(cm[gi * 2 + 1], acc[gi][3]); }
        }
      }
      // recursive halving over the row groups g: lane g ends with value index g = (g / 2) * 2 + g % 2, its own key
      float x;
      {
        const bool b2 = (g & 4) != 0, b1 = (g & 2) != 0, b0 = (g & 1) != 0;
        float h4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float keep = b2 ? cm[4 + i] : cm[i], send = b2 ? cm[i] : cm[4 + i];
          h4[i] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, send, 16));
        }
        float h2[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const float keep = b1 ? h4[2 + i] : h4[i], send = b1 ? h4[i] : h4[2 + i];
          h2[i] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, send, 8));
        }
        const float keep = b0 ? h2[1] : h2[0], send = b0 ? h2[0] : h2[1];
        x = fmaxf(keep, __shfl_xor_sync(0xffffffffu, send, 4));
      }

      // ---- exact value where the rounding is certain, strict re-scoring elsewhere ----
      const float e_ = eps_q * s_abs * 1.01f;
      float sc = Elem<DT>::round(x);
      const bool sure = Elem<DT>::round(x - e_) == Elem<DT>::round(x + e_);
      if (known) sc = won_score;
      unsigned need = __ballot_sync(0xffffffffu, idx >= 0 && (!sure || check));
      while (need) {
        const int owner = __ffs(need) - 1;
        need &= need - 1;
        const float rawv = strict_score(__shfl_sync(0xffffffffu, idx, owner));
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
      const float other = __shfl_xor_sync(0xffffffffu, sc, 4);   // the other candidate of the same chunk
      const int other_t = __shfl_xor_sync(0xffffffffu, tk_asked, 4);
      if (act) {
        if (idx >= 0) st_keys += 1;
        const float sl = side ? other : sc, sr = side ? sc : other;
        const bool win = sl > sr;
        if (win) right = mid; else left = mid;
        score = fmaxf(score, win ? sl : sr);
        won_t = (win != (side != 0)) ? tk_asked : other_t;    // the left candidate when it won, else the right one
        won_score = win ? sl : sr;
      }
    }

    if (in_range && side == 0) {
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
}

template <int DT, int D, int MT>
int launch(const hipattn_scan_params_t& p, cudaStream_t stream) {
  constexpr int NR = 16 * MT;
  const size_t smem = (size_t)NR * (D * 2 + kQPad) + (MT > 1 ? (size_t)NR * D * 2 : 0);
  const int BDST = cdiv(p.TQ, p.block_size_q);
  const int nblk_total = cdiv(p.n_chunks, 64);
  const int64_t units = (int64_t)p.B * p.H * BDST;
  const int nblk = scan_ctas_per_unit(units, nblk_total);
  const int64_t grid = units * nblk;
  HIPATTN_REQUIRE(grid > 0 && grid < 0x7fffffffLL, HIPATTN_ERR_INVALID, "scan grid of %lld blocks", (long long)grid);
  auto kern = scan_stage_regs_kernel<DT, D, MT>;
  HIPATTN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<(unsigned)grid, 128, smem, stream>>>(p, nblk, nblk_total, p.mode == HIPATTN_SCAN_CHECK ? 1 : 0);
  return check_launch("scan_stage_regs_kernel");
}

template <int DT, int D>
int dispatch_rows(const hipattn_scan_params_t& p, cudaStream_t stream) {
  const int R = p.block_size_q / p.stride_q;
  if (R <= 16) return launch<DT, D, 1>(p, stream);
  if (R <= 32) return launch<DT, D, 2>(p, stream);
  return launch<DT, D, 4>(p, stream);
}

}  // namespace

// Takes 16-bit prefill shapes (16 to 64 pooled rows in multiples of 16, head dim 64 or 128) when the caller supplies
// the prepared keys.  HIPATTN_SCAN_KERNEL = auto | regs | tcgen05 | mma picks between this kernel, the tcgen05 rounds
// and the shared-memory mma.sync kernel; `auto` uses this kernel up to `auto_max_rows` pooled rows.
int scan_stage_regs(const hipattn_scan_params_t& p, cudaStream_t stream, bool* handled) {
  *handled = false;
  const int R = p.block_size_q / p.stride_q;
  const int rows = min(R, cdiv(p.TQ, p.stride_q));
  if (p.mode == HIPATTN_SCAN_STRICT || p.dtype == HIPATTN_F32 || rows <= 1 || (R % 16) != 0 || R > 64 || (p.D != 64 && p.D != 128)) return HIPATTN_OK;
  if (p.key_abs == nullptr || p.k_scaled == nullptr) return HIPATTN_OK;
  if ((int64_t)p.B * p.T * p.HKV >= 0x7fffffffLL) return HIPATTN_OK;
  const char* v = getenv("HIPATTN_SCAN_KERNEL");
  constexpr int auto_max_rows = 0;
  if (v && strcmp(v, "regs") == 0) {}
  else if ((v == nullptr || strcmp(v, "auto") == 0) && R <= auto_max_rows) {}
  else return HIPATTN_OK;
  *handled = true;
  if (p.dtype == HIPATTN_BF16) return p.D == 128 ? dispatch_rows<HIPATTN_BF16, 128>(p, stream) : dispatch_rows<HIPATTN_BF16, 64>(p, stream);
  return p.D == 128 ? dispatch_rows<HIPATTN_F16, 128>(p, stream) : dispatch_rows<HIPATTN_F16, 64>(p, stream);
}

}  // namespace hipattn
