// Scan stage of the mask estimator for 16-bit prefill: tensor-core scores with an exact fallback.
//
// Same contract as the strict kernel (scan_stage.cu): the score of a key is
// max over pooled rows of round_to_dtype(dot), with the dot product defined as the sequential fp32
// accumulation over the head dimension.  Here the dot products of a whole warp-round (64 candidate
// keys x all pooled rows) are first computed approximately with mma.sync; a second set of MMAs with
// an all-ones left operand gives S_k = sum_d |k'_d| per key, from which an error radius
// eps = kEps * max|q'| * S_k follows.  If rounding (x - eps) and (x + eps) to the element type gives
// the same value, that value is the exact score; otherwise the key is re-scored by the strict
// definition, cooperatively by the warp (one pooled row per lane).  Decisions and stored scores are
// therefore those of the strict kernel, at a fraction of its instruction count.  kEps is an
// empirical bound on |tensor-core dot - sequential fp32 dot| / (max|q'| * S_k); the check mode
// (mode 2) re-scores every key strictly and records, in a statistics buffer the tests read, the
// largest observed deviation as a fraction of eps and the number of shortcuts that would have been
// wrong.
//
// Mapping: a warp owns 32 chunks (lane = chunk, both candidate keys); the key of chunk l, side e is
// staged in row (l / 4) * 8 + (l % 4) * 2 + e, which is the MMA column whose accumulator lives in
// lane l itself (columns are held by lanes with the same lane % 4), so no exchange is needed after
// the row reduction.
#include "mma_common.cuh"
#include "scan_common.cuh"

namespace hipattn {
namespace {

constexpr int kPadBytes = 16;


template <int DT, int D, int MT>
__global__ void __launch_bounds__(128) scan_stage_mma_kernel(const hipattn_scan_params_t p, int nblk, int nblk_total, int NW, int check) {
  using T = typename Elem<DT>::type;
  constexpr int ROWB = D * 2;                 // bytes per key / query row
  constexpr int STRIDE = ROWB + kPadBytes;    // padded row stride: conflict-free ldmatrix and lane reads
  constexpr int PIECES = ROWB / 16;
  constexpr int KSTEPS = D / 16;
  extern __shared__ __align__(16) unsigned char smem[];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int Gq = p.H / p.HKV;
  const int BDST = cdiv(p.TQ, p.block_size_q);
  int64_t bid = blockIdx.x;
  const int cblk = (int)(bid % nblk); bid /= nblk;
  const int g = (int)(bid % Gq); bid /= Gq;
  const int d = (int)(bid % BDST); bid /= BDST;
  const int hkv = (int)(bid % p.HKV); bid /= p.HKV;
  const int b = (int)bid;
  const int h = hkv * Gq + g;

  const int R = p.block_size_q / p.stride_q;   // multiple of 16
  const int t0 = d * p.block_size_q;
  int Rv = 0;
  if (t0 < p.TQ) Rv = min(R, (p.TQ - t0 + p.stride_q - 1) / p.stride_q);
  const int n_mgroups = cdiv(R, 16 * MT);
  const int Rpad = n_mgroups * 16 * MT;

  unsigned char* q16 = smem;                                   // [Rpad][STRIDE] scaled pooled queries
  unsigned char* kstage = q16 + (size_t)Rpad * STRIDE;         // [NW][64][STRIDE]
  float* kf32 = reinterpret_cast<float*>(kstage + (size_t)NW * 64 * STRIDE);  // [NW][D] scaled key of a fallback
  __shared__ int s_pmin;
  __shared__ float s_qmax;

  // ---- pooled queries (identical arithmetic to the strict kernel), once per CTA ----
  if (threadIdx.x == 0) s_qmax = 0.f;
  __syncthreads();
  float qmax_local = 0.f;
  for (int i = threadIdx.x; i < Rpad * PIECES; i += blockDim.x) {
    const int r = i / PIECES, pc = i % PIECES;
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = 0.f;
    if (r < Rv) pooled_query_piece<DT>(p, b, h, t0 + r * p.stride_q, pc, v);
    T* dst = reinterpret_cast<T*>(q16 + (size_t)r * STRIDE + pc * 16);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      dst[e] = Elem<DT>::from_f32(v[e]);
      qmax_local = fmaxf(qmax_local, fabsf(v[e]));
    }
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
  const bool have_abs = p.key_abs != nullptr;
  const int n = p.n_chunks;
  const int64_t row = (int64_t)b * BDST + d;

  unsigned char* wstage = kstage + (size_t)warp * 64 * STRIDE;
  float* wkf = kf32 + warp * D;
  const uint32_t kscale2 = pack_scalar2<DT>(p.k_scale);
  const uint32_t ones2 = pack_scalar2<DT>(1.0f);
  const uint32_t ones_frag[4] = {ones2, ones2, ones2, ones2};
  unsigned long long st_keys = 0, st_fb = 0, st_wrong = 0;
  float st_ratio = 0.f;

  // strict dot products of the key staged in row `srow`, by the whole warp (one pooled row per lane);
  // returns the largest one before rounding (rounding is monotonic, so it commutes with the maximum)
  auto strict_score = [&](int srow) -> float {
    __syncwarp();
    const unsigned char* kr = wstage + (size_t)srow * STRIDE;
    for (int e2 = lane; e2 < D / 2; e2 += 32) {
      const uint32_t w = mul2<DT>(*reinterpret_cast<const uint32_t*>(kr + e2 * 4), kscale2);
      wkf[2 * e2] = lo_f32<DT>(w);
      wkf[2 * e2 + 1] = hi_f32<DT>(w);
    }
    __syncwarp();
    float best = -INFINITY;
    for (int r0 = 0; r0 < Rv; r0 += 32) {
      const int r = r0 + lane;
      if (r < Rv) {
        const unsigned char* qr = q16 + (size_t)r * STRIDE;
        float acc = 0.f;
#pragma unroll 4
        for (int pc = 0; pc < PIECES; ++pc) {
          const uint4 qw = *reinterpret_cast<const uint4*>(qr + pc * 16);
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

  // ---- chunk blocks of this CTA ----
  for (int cb = cblk; cb < nblk_total; cb += nblk) {
  const int wbase = (cb * NW + warp) * 32;
  const int c = wbase + lane;
  int left = 0, right = 0;
  const bool in_range = c < n;
  if (in_range) {
    left = p.left[row * n + c];
    right = p.right[row * n + c];
  }
  const int my_rounds = chunk_rounds(p, row, n, wbase, lane, in_range, left, right);
  int max_rounds = my_rounds;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) max_rounds = max(max_rounds, __shfl_xor_sync(0xffffffffu, max_rounds, o));
  float score = HIPATTN_SCORE_INIT;
  // the candidate that won the previous round and its score: proposed again, it is neither fetched nor scored again
  int won_t = -1;
  float won_score = 0.f;

  for (int it = 0; it < max_rounds; ++it) {
    const bool act = in_range && it < my_rounds && left < right && left <= pt && left >= 0;
    if (!__any_sync(0xffffffffu, act)) break;
    const int mid = (left + right) >> 1;
    int tl = (left + mid) >> 1, tr = (mid + right) >> 1;
    const int tl_asked = tl, tr_asked = tr;
    const bool known_l = act && tl == won_t, known_r = act && tr == won_t;
    const char* src_l = nullptr;
    const char* src_r = nullptr;
    if (act) {
      if (p.k.cache == nullptr && (tl < 0 || tr >= p.T)) {
        atomicOr(p.status, HIPATTN_STATUS_TOKEN_RANGE);
        tl = min(max(tl, 0), p.T - 1);
        tr = min(max(tr, 0), p.T - 1);
      }
      if (!known_l) src_l = token_row(p.k, b, tl, hkv, 2, p.status);
      if (!known_r) src_r = token_row(p.k, b, tr, hkv, 2, p.status);
      if (p.access_counter) {   // (a candidate whose score is known was marked when it was fetched)
        if (!known_l) mark_access(p.access_counter, p.access_stride_b, p.access_stride_h, p.access_n, p.k, b, hkv, tl);
        if (!known_r) mark_access(p.access_counter, p.access_stride_b, p.access_stride_h, p.access_n, p.k, b, hkv, tr);
      }
    }
    if (!__any_sync(0xffffffffu, src_l != nullptr || src_r != nullptr)) {
      // every live chunk knows both scores (both candidates are the previous winner): equal scores keep the right half
      if (act) left = mid;
      continue;
    }
    // ---- gather the 64 candidate rows ----
    __syncwarp();
    {
      constexpr int RPI = 32 / PIECES;  // rows per iteration (2 for D = 128, 4 for D = 64)
      const int sub = lane / PIECES, piece = lane % PIECES;
#pragma unroll
      for (int side = 0; side < 2; ++side) {            // the side is uniform per shuffle: every lane offers that pointer
        const unsigned long long mine = (unsigned long long)(side ? src_r : src_l);
        for (int o0 = 0; o0 < 32; o0 += RPI) {
          const int owner = o0 + sub;
          const int rr = (owner >> 2) * 8 + (owner & 3) * 2 + side;  // staged row of (owner, side)
          const unsigned long long a = __shfl_sync(0xffffffffu, mine, owner);
          if (a != 0ull) cp_async16(wstage + (size_t)rr * STRIDE + piece * 16, (const char*)a + piece * 16);
        }
      }
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncwarp();

    // ---- approximate scores on tensor cores ----
    float xl = -INFINITY, xr = -INFINITY, sl_abs = 0.f, sr_abs = 0.f;
    if (have_abs && act && !(known_l && known_r)) {  // precomputed key magnitudes (one per key row of the call)
      sl_abs = p.key_abs[((int64_t)b * p.HKV + hkv) * p.T + tl];
      sr_abs = p.key_abs[((int64_t)b * p.HKV + hkv) * p.T + tr];
    }
    for (int mg = 0; mg < n_mgroups; ++mg) {
      float acc[MT][8][4];
      float sab[8][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        sab[nt][0] = sab[nt][1] = sab[nt][2] = sab[nt][3] = 0.f;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) acc[mt][nt][0] = acc[mt][nt][1] = acc[mt][nt][2] = acc[mt][nt][3] = 0.f;
      }
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        uint32_t bf[8][2];
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          const int krow = np * 16 + (lane & 7) + ((lane >> 4) << 3);
          const int kpc = ks * 2 + ((lane >> 3) & 1);
          ldsm_x4(bf[np * 2][0], bf[np * 2][1], bf[np * 2 + 1][0], bf[np * 2 + 1][1], wstage + (size_t)krow * STRIDE + kpc * 16);
        }
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          bf[nt][0] = mul2<DT>(bf[nt][0], kscale2);
          bf[nt][1] = mul2<DT>(bf[nt][1], kscale2);
        }
        if (mg == 0 && !have_abs) {
#pragma unroll
          for (int nt = 0; nt < 8; ++nt) mma16816<DT>(sab[nt], ones_frag, bf[nt][0] & 0x7fff7fffu, bf[nt][1] & 0x7fff7fffu);
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          uint32_t af[4];
          const int qrow = (mg * MT + mt) * 16 + (lane & 15);
          ldsm_x4(af[0], af[1], af[2], af[3], q16 + (size_t)qrow * STRIDE + (ks * 2 + (lane >> 4)) * 16);
#pragma unroll
          for (int nt = 0; nt < 8; ++nt) mma16816<DT>(acc[mt][nt], af, bf[nt][0], bf[nt][1]);
        }
      }
      // column maxima over this group's valid rows
      float cm[8][2];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        cm[nt][0] = cm[nt][1] = -INFINITY;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const int r0 = (mg * MT + mt) * 16 + (lane >> 2);
          if (r0 < Rv) { cm[nt][0] = fmaxf(cm[nt][0], acc[mt][nt][0]); cm[nt][1] = fmaxf(cm[nt][1], acc[mt][nt][1]); }
          if (r0 + 8 < Rv) { cm[nt][0] = fmaxf(cm[nt][0], acc[mt][nt][2]); cm[nt][1] = fmaxf(cm[nt][1], acc[mt][nt][3]); }
        }
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int o = 4; o <= 16; o <<= 1) {
          cm[nt][0] = fmaxf(cm[nt][0], __shfl_xor_sync(0xffffffffu, cm[nt][0], o));
          cm[nt][1] = fmaxf(cm[nt][1], __shfl_xor_sync(0xffffffffu, cm[nt][1], o));
        }
      }
      // this lane's two keys sit in n-tile lane / 4, columns (lane % 4) * 2 + {0, 1}: its own accumulators
      const int mynt = lane >> 2;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        if (nt == mynt) {
          xl = fmaxf(xl, cm[nt][0]);
          xr = fmaxf(xr, cm[nt][1]);
          if (mg == 0 && !have_abs) { sl_abs = sab[nt][0]; sr_abs = sab[nt][1]; }
        }
      }
    }
    // ---- exact value where the rounding is certain, strict re-scoring elsewhere ----
    const float el = eps_q * sl_abs * 1.01f, er = eps_q * sr_abs * 1.01f;
    float sl = Elem<DT>::round(xl), sr = Elem<DT>::round(xr);
    bool sure_l = Elem<DT>::round(xl - el) == Elem<DT>::round(xl + el);
    bool sure_r = Elem<DT>::round(xr - er) == Elem<DT>::round(xr + er);
    if (known_l) sl = won_score;
    if (known_r) sr = won_score;
    unsigned need_l = __ballot_sync(0xffffffffu, act && !known_l && (!sure_l || check));
    unsigned need_r = __ballot_sync(0xffffffffu, act && !known_r && (!sure_r || check));
    while (need_l | need_r) {
      const bool is_l = need_l != 0;
      const int owner = __ffs(is_l ? need_l : need_r) - 1;
      if (is_l) need_l &= need_l - 1; else need_r &= need_r - 1;
      const int srow = (owner >> 2) * 8 + (owner & 3) * 2 + (is_l ? 0 : 1);
      const float raw = strict_score(srow);
      const float ex = Elem<DT>::round(raw);
      if (lane == owner) {
        const bool sure = is_l ? sure_l : sure_r;
        if (check) {
          if (sure && (is_l ? sl : sr) != ex) ++st_wrong;
          const float e_ = is_l ? el : er;
          if (e_ > 0.f) st_ratio = fmaxf(st_ratio, fabsf((is_l ? xl : xr) - raw) / e_);
        }
        if (!sure) ++st_fb;
        if (is_l) sl = ex; else sr = ex;
      }
    }
    if (act) {
      st_keys += (known_l ? 0 : 1) + (known_r ? 0 : 1);
      const bool win = sl > sr;
      if (win) right = mid; else left = mid;
      score = fmaxf(score, win ? sl : sr);
      won_t = win ? tl_asked : tr_asked;
      won_score = win ? sl : sr;
    }
  }

  if (in_range) {
    if (score > HIPATTN_SCORE_INIT) atomicMax(p.score_max + row * n + c, encode_score(score));
    const int64_t o = (row * p.H + h) * n + c;
    if (p.left_out) p.left_out[o] = left;
    if (p.right_out) p.right_out[o] = right;
    if (p.score_out) p.score_out[o] = score;
  }
  }  // chunk blocks
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
  constexpr int STRIDE = D * 2 + kPadBytes;
  const int R = p.block_size_q / p.stride_q;
  const int Rpad = cdiv(R, 16 * MT) * 16 * MT;
  const size_t q_bytes = (size_t)Rpad * STRIDE;
  int NW = 4;
  while (NW > 1 && q_bytes + (size_t)NW * (64 * STRIDE + D * 4) > 110 * 1024) NW >>= 1;
  const size_t smem = q_bytes + (size_t)NW * (64 * STRIDE + D * 4);
  HIPATTN_REQUIRE(smem <= 227 * 1024, HIPATTN_ERR_UNSUPPORTED, "scan stage needs %zu bytes of shared memory", smem);
  const int BDST = cdiv(p.TQ, p.block_size_q);
  const int nblk_total = cdiv(p.n_chunks, 32 * NW);
  const int64_t units = (int64_t)p.B * p.H * BDST;
  const int nblk = scan_ctas_per_unit(units, nblk_total);
  const int64_t grid = units * nblk;
  HIPATTN_REQUIRE(grid > 0 && grid < 0x7fffffffLL, HIPATTN_ERR_INVALID, "scan grid of %lld blocks", (long long)grid);
  auto kern = scan_stage_mma_kernel<DT, D, MT>;
  HIPATTN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<(unsigned)grid, 32 * NW, smem, stream>>>(p, nblk, nblk_total, NW, p.mode == 2 ? 1 : 0);
  return check_launch("scan_stage_mma_kernel");
}

template <int DT, int D>
int dispatch_rows(const hipattn_scan_params_t& p, cudaStream_t stream) {
  const int R = p.block_size_q / p.stride_q;
  if (R <= 16) return launch<DT, D, 1>(p, stream);
  if (R <= 32) return launch<DT, D, 2>(p, stream);
  return launch<DT, D, 4>(p, stream);
}

}  // namespace

// Takes 16-bit prefill shapes (more than one pooled row, a multiple of 16 of them, head dim 64 or
// 128); anything else stays on the strict kernel.
int scan_stage_mma(const hipattn_scan_params_t& p, cudaStream_t stream, bool* handled) {
  *handled = false;
  const int R = p.block_size_q / p.stride_q;
  const int rows = min(R, cdiv(p.TQ, p.stride_q));
  if (p.mode == 1 || p.dtype == HIPATTN_F32 || rows <= 1 || (R % 16) != 0 || (p.D != 64 && p.D != 128)) return HIPATTN_OK;
  if (p.k.fp8_e5m2) return HIPATTN_OK;   // an fp8 cache is read by the strict kernel (or through the prepared 16-bit copy)
  *handled = true;
  if (p.dtype == HIPATTN_BF16) return p.D == 128 ? dispatch_rows<HIPATTN_BF16, 128>(p, stream) : dispatch_rows<HIPATTN_BF16, 64>(p, stream);
  return p.D == 128 ? dispatch_rows<HIPATTN_F16, 128>(p, stream) : dispatch_rows<HIPATTN_F16, 64>(p, stream);
}

}  // namespace hipattn
