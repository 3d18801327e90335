// Scan stage of the hierarchical mask estimator (strict arithmetic).
//
// For every (batch, query block, head, chunk) the kernel narrows [left, right) by repeated halving:
// each round fetches two representative key rows (the midpoints of the two halves), scores them
// against the mean-pooled query rows of the block and keeps the better half.  The score of a key is
// max over pooled rows of round_to_dtype(dot(q', k')), where the dot product is accumulated in fp32
// sequentially over the head dimension in ascending order, so that a CPU restatement reproduces it
// bit for bit.  The best score of the surviving halves is reduced over heads with an atomic max on
// an order-preserving integer image.
//
// Mapping: one CTA = 32 * NW consecutive chunks of one (batch, query block, head); a lane owns one
// chunk and both of its candidate keys.  Key rows are gathered with 16-byte cp.async (16 lanes per
// 256-byte row, fully coalesced) into a per-warp staging area; pooled queries sit in shared memory as
// fp32 and are read as warp-wide broadcasts, so the inner loop is 8 FMAs per shared-memory load.
// CTAs are ordered so that all query blocks and heads of one KV head run together and its keys stay
// resident in L2.
#include "scan_common.cuh"

namespace hipattn {
namespace {

constexpr int kPad = 16;  // bytes of padding per staged key row: keeps 16-byte lane reads conflict free

template <int DT, int D>
struct RowGeom {
  static constexpr int kRowBytes = D * Elem<DT>::bytes;
  static constexpr int kRowStride = kRowBytes + kPad;
  static constexpr int kPieces = kRowBytes / 16;   // 16-byte pieces per row
  static constexpr int kVec = 16 / Elem<DT>::bytes;  // elements per piece
};

// unpack one 16-byte piece of key elements, apply the key scale and round to the element type
template <int DT>
__device__ __forceinline__ void unpack_scaled(const uint4& w, float k_scale, float* out);

template <>
__device__ __forceinline__ void unpack_scaled<HIPATTN_F32>(const uint4& w, float k_scale, float* out) {
  out[0] = __fmul_rn(__uint_as_float(w.x), k_scale);
  out[1] = __fmul_rn(__uint_as_float(w.y), k_scale);
  out[2] = __fmul_rn(__uint_as_float(w.z), k_scale);
  out[3] = __fmul_rn(__uint_as_float(w.w), k_scale);
}
// 16-bit types: one packed multiply per element pair.  The product of two 16-bit floats is exact in fp32,
// so rounding it once to the element type (what the packed multiply does) equals multiplying in fp32 and
// converting, at a third of the instructions.
template <>
__device__ __forceinline__ void unpack_scaled<HIPATTN_BF16>(const uint4& w, float k_scale, float* out) {
  const uint32_t v[4] = {w.x, w.y, w.z, w.w};
  const uint32_t s2 = pack_scalar2<HIPATTN_BF16>(k_scale);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t m = mul2<HIPATTN_BF16>(v[i], s2);
    out[2 * i] = lo_f32<HIPATTN_BF16>(m);
    out[2 * i + 1] = hi_f32<HIPATTN_BF16>(m);
  }
}
template <>
__device__ __forceinline__ void unpack_scaled<HIPATTN_F16>(const uint4& w, float k_scale, float* out) {
  const uint32_t v[4] = {w.x, w.y, w.z, w.w};
  const uint32_t s2 = pack_scalar2<HIPATTN_F16>(k_scale);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t m = mul2<HIPATTN_F16>(v[i], s2);
    out[2 * i] = lo_f32<HIPATTN_F16>(m);
    out[2 * i + 1] = hi_f32<HIPATTN_F16>(m);
  }
}

template <int DT>
__device__ __forceinline__ float mac(float q, float k, float acc) {
  if (DT == HIPATTN_F32) return __fadd_rn(acc, __fmul_rn(q, k));  // two roundings, reproducible on a CPU
  return fmaf(q, k, acc);                                         // 16-bit inputs: the product is exact
}

// RT = pooled query rows processed per pass over a staged key pair; EXT = the call uses in-kernel RoPE, an fp8 cache or
// the access counters (the plain instantiation carries none of their branches: in decode they cost 60 % of the time)
template <int DT, int D, int RT, bool EXT>
// (decode, one pooled row: the kernel is bound by random row reads from HBM and lives on resident warps, so the
// register allocation aims at seven CTAs per multiprocessor)
__global__ void __launch_bounds__(128, RT == 1 ? 7 : 1) scan_stage_kernel(const hipattn_scan_params_t p, int nblk, int nblk_total, int NW) {
  using G = RowGeom<DT, D>;
  using T = typename Elem<DT>::type;
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

  const int R = p.block_size_q / p.stride_q;
  const int t0 = d * p.block_size_q;
  int Rv = 0;  // valid strided rows form a prefix
  if (t0 < p.TQ) Rv = min(R, (p.TQ - t0 + p.stride_q - 1) / p.stride_q);
  const int Rpad = cdiv(max(Rv, 1), RT) * RT;

  float* qtile = reinterpret_cast<float*>(smem);                       // [Rpad][D]
  unsigned char* kstage = smem + (size_t)Rpad * D * sizeof(float);     // [NW][2][32][kRowStride]
  __shared__ int s_pmin;

  // ---- pooled queries (once per CTA) ----
  for (int i = threadIdx.x; i < Rpad * G::kPieces; i += blockDim.x) {
    const int r = i / G::kPieces, pc = i % G::kPieces;
    float v[G::kVec];
#pragma unroll
    for (int e = 0; e < G::kVec; ++e) v[e] = 0.f;
    if (r < Rv) pooled_query_piece<DT>(p, b, h, t0 + r * p.stride_q, pc, v);
#pragma unroll
    for (int e = 0; e < G::kVec; e += 4)
      *reinterpret_cast<float4*>(qtile + (size_t)r * D + pc * G::kVec + e) = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
  }
  if (warp == 0) {
    const int m = block_min_position(p, b, t0, Rv, lane);
    if (lane == 0) s_pmin = m;
  }
  __syncthreads();
  if (Rv == 0) return;
  const int pmin = s_pmin;
  const int pt = max(pmin - p.scan_window, 0);
  const int n = p.n_chunks;
  const int64_t row = (int64_t)b * BDST + d;
  unsigned char* wstage = kstage + (size_t)warp * 64 * G::kRowStride;
  const unsigned char* my_l = wstage + (size_t)lane * G::kRowStride;
  const unsigned char* my_r = wstage + (size_t)(32 + lane) * G::kRowStride;
  const int ntile = Rpad / RT;

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
  // The candidate that won the previous round and its score.  When the halved chunk proposes the same key again (both
  // candidates of the last round, one of the round before it) the score is known -- the same key against the same
  // pooled queries -- and the row is not fetched again.
  int won_t = -1;
  float won_score = 0.f;

  for (int it = 0; it < max_rounds; ++it) {
    const bool act = in_range && it < my_rounds && left < right && left <= pt && left >= 0;
    if (!__any_sync(0xffffffffu, act)) break;  // a chunk that is inactive now stays inactive
    const int mid = (left + right) >> 1;
    int tl = (left + mid) >> 1, tr = (mid + right) >> 1;
    const int tl_asked = tl, tr_asked = tr;
    // (with in-kernel RoPE a key's score depends on the side it is proposed for: nothing is reused)
    const bool reuse = !EXT || p.rope_mode == HIPATTN_ROPE_NONE;
    const bool known_l = act && reuse && tl == won_t, known_r = act && reuse && tr == won_t;
    const char* src_l = nullptr;
    const char* src_r = nullptr;
    if (act) {
      if (p.k.cache == nullptr && (tl < 0 || tr >= p.T)) {
        atomicOr(p.status, HIPATTN_STATUS_TOKEN_RANGE);
        tl = min(max(tl, 0), p.T - 1);
        tr = min(max(tr, 0), p.T - 1);
      }
      if (!known_l) src_l = token_row(p.k, b, tl, hkv, Elem<DT>::bytes, p.status);
      if (!known_r) src_r = token_row(p.k, b, tr, hkv, Elem<DT>::bytes, p.status);
      if (EXT && p.access_counter) {   // (a candidate whose score is known was marked when it was fetched)
        if (!known_l) mark_access(p.access_counter, p.access_stride_b, p.access_stride_h, p.access_n, p.k, b, hkv, tl);
        if (!known_r) mark_access(p.access_counter, p.access_stride_b, p.access_stride_h, p.access_n, p.k, b, hkv, tr);
      }
    }
    if (!__any_sync(0xffffffffu, src_l != nullptr || src_r != nullptr)) {
      // every live chunk of the warp knows both scores (both candidates are the previous winner): the round decides
      // without touching memory; equal scores keep the right half and the chunk's best score is unchanged
      if (act) left = mid;
      continue;
    }
    // cooperative gather: 64 rows, kPieces lanes per row
    __syncwarp();
    constexpr int kRowsPerIter = 32 / G::kPieces > 0 ? 32 / G::kPieces : 1;
    if (G::kPieces <= 32) {
      const int sub = lane / G::kPieces, piece = lane % G::kPieces;
      for (int r0 = 0; r0 < 64; r0 += kRowsPerIter) {
        const int rr = r0 + sub;             // staged row: side * 32 + owner lane
        const int owner = rr & 31, side = rr >> 5;
        const unsigned long long a = __shfl_sync(0xffffffffu, (unsigned long long)(side ? src_r : src_l), owner);
        if (a != 0ull && sub < kRowsPerIter) {
          if (EXT && DT != HIPATTN_F32 && p.k.fp8_e5m2)   // an fp8 cache: 8 bytes become one 16-byte piece of the element type
            *reinterpret_cast<uint4*>(wstage + (size_t)rr * G::kRowStride + piece * 16) =
                widen_fp8_e5m2<DT == HIPATTN_F32 ? HIPATTN_F16 : DT>(__ldg(reinterpret_cast<const uint2*>((const char*)a + piece * 8)));
          else
            cp_async16(wstage + (size_t)rr * G::kRowStride + piece * 16, (const char*)a + piece * 16);
        }
      }
    } else {  // rows longer than 512 bytes: every lane copies several pieces
      for (int rr = 0; rr < 64; ++rr) {
        const int owner = rr & 31, side = rr >> 5;
        const unsigned long long a = __shfl_sync(0xffffffffu, (unsigned long long)(side ? src_r : src_l), owner);
        if (a != 0ull)
          for (int piece = lane; piece < G::kPieces; piece += 32)
            cp_async16(wstage + (size_t)rr * G::kRowStride + piece * 16, (const char*)a + piece * 16);
      }
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncwarp();

    float sl = -INFINITY, sr = -INFINITY;
    if (act) {
      for (int tile = 0; tile < ntile && !(known_l && known_r); ++tile) {
        float accl[RT], accr[RT];
#pragma unroll
        for (int r = 0; r < RT; ++r) accl[r] = accr[r] = 0.f;
        const float* qt = qtile + (size_t)tile * RT * D;
#pragma unroll 2
        for (int pc = 0; pc < G::kPieces; ++pc) {
          float kl[G::kVec], kr[G::kVec];
          if (!EXT || p.rope_mode == HIPATTN_ROPE_NONE) {
            unpack_scaled<DT>(*reinterpret_cast<const uint4*>(my_l + pc * 16), p.k_scale, kl);
            unpack_scaled<DT>(*reinterpret_cast<const uint4*>(my_r + pc * 16), p.k_scale, kr);
          } else {   // keys at their chunk's index (streaming) or at 0 / 1 for the left / right candidate (relative)
            const bool rel = p.rope_mode == HIPATTN_ROPE_RELATIVE;
            unpack_rope_scaled<DT, D>(my_l, pc, rel ? 0 : c, p, kl);
            unpack_rope_scaled<DT, D>(my_r, pc, rel ? 1 : c, p, kr);
          }
#pragma unroll
          for (int r = 0; r < RT; ++r) {
#pragma unroll
            for (int e4 = 0; e4 < G::kVec; e4 += 4) {
              const float4 qv = *reinterpret_cast<const float4*>(qt + r * D + pc * G::kVec + e4);
              accl[r] = mac<DT>(qv.x, kl[e4 + 0], accl[r]);
              accr[r] = mac<DT>(qv.x, kr[e4 + 0], accr[r]);
              accl[r] = mac<DT>(qv.y, kl[e4 + 1], accl[r]);
              accr[r] = mac<DT>(qv.y, kr[e4 + 1], accr[r]);
              accl[r] = mac<DT>(qv.z, kl[e4 + 2], accl[r]);
              accr[r] = mac<DT>(qv.z, kr[e4 + 2], accr[r]);
              accl[r] = mac<DT>(qv.w, kl[e4 + 3], accl[r]);
              accr[r] = mac<DT>(qv.w, kr[e4 + 3], accr[r]);
            }
          }
        }
#pragma unroll
        for (int r = 0; r < RT; ++r) {
          if (tile * RT + r < Rv) {
            sl = fmaxf(sl, Elem<DT>::round(accl[r]));
            sr = fmaxf(sr, Elem<DT>::round(accr[r]));
          }
        }
      }
      if (known_l) sl = won_score;
      if (known_r) sr = won_score;
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
}

template <int DT, int D, int RT, bool EXT>
int launch(const hipattn_scan_params_t& p, cudaStream_t stream) {
  using G = RowGeom<DT, D>;
  const int R = p.block_size_q / p.stride_q;
  const int rows = min(R, cdiv(p.TQ, p.stride_q));   // pooled rows that can be valid (1 for decode)
  const int Rpad = cdiv(rows, RT) * RT;
  const size_t q_bytes = (size_t)Rpad * D * sizeof(float);
  int NW = 4;
  while (NW > 1 && q_bytes + (size_t)NW * 64 * G::kRowStride > 100 * 1024) NW >>= 1;
  const size_t smem = q_bytes + (size_t)NW * 64 * G::kRowStride;
  HIPATTN_REQUIRE(smem <= 227 * 1024, HIPATTN_ERR_UNSUPPORTED,
                  "scan stage needs %zu bytes of shared memory (query rows %d, head dim %d)", smem, R, D);
  const int BDST = cdiv(p.TQ, p.block_size_q);
  const int nblk_total = cdiv(p.n_chunks, 32 * NW);
  const int64_t units = (int64_t)p.B * p.H * BDST;
  const int nblk = scan_ctas_per_unit(units, nblk_total);
  const int64_t grid = units * nblk;
  HIPATTN_REQUIRE(grid > 0 && grid < 0x7fffffffLL, HIPATTN_ERR_INVALID, "scan grid of %lld blocks", (long long)grid);
  auto kern = scan_stage_kernel<DT, D, RT, EXT>;
  HIPATTN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<(unsigned)grid, 32 * NW, smem, stream>>>(p, nblk, nblk_total, NW);
  return check_launch("scan_stage_kernel");
}

template <int DT, int D>
int dispatch_rows(const hipattn_scan_params_t& p, cudaStream_t stream) {
  const int R = p.block_size_q / p.stride_q;
  // rows that can be valid: a single query row (decode) needs one accumulator pair only
  const int rows = min(R, cdiv(p.TQ, p.stride_q));
  const bool ext = p.rope_mode != HIPATTN_ROPE_NONE || p.k.fp8_e5m2 || p.access_counter != nullptr;
  if (rows <= 1) return ext ? launch<DT, D, 1, true>(p, stream) : launch<DT, D, 1, false>(p, stream);
  if (R <= 16) return ext ? launch<DT, D, 16, true>(p, stream) : launch<DT, D, 16, false>(p, stream);
  if (R <= 32) return ext ? launch<DT, D, 32, true>(p, stream) : launch<DT, D, 32, false>(p, stream);
  return ext ? launch<DT, D, 64, true>(p, stream) : launch<DT, D, 64, false>(p, stream);
}

template <int DT>
int dispatch_dim(const hipattn_scan_params_t& p, cudaStream_t stream) {
  switch (p.D) {
    case 64: return dispatch_rows<DT, 64>(p, stream);
    case 128: return dispatch_rows<DT, 128>(p, stream);
    case 256: return dispatch_rows<DT, 256>(p, stream);
    default:
      set_error("scan stage: head dimension %d is not built (64, 128, 256)", p.D);
      return HIPATTN_ERR_UNSUPPORTED;
  }
}

}  // namespace

int scan_stage_mma(const hipattn_scan_params_t& p, cudaStream_t stream, bool* handled);
int scan_stage_tcgen05(const hipattn_scan_params_t& p, cudaStream_t stream, bool* handled);
int scan_chunks_strict(const hipattn_scan_params_t& p, cudaStream_t stream, bool* handled);
int scan_prepare_keys(const hipattn_tokens_t& k, int dtype, int D, int B, int T, int HKV, float k_scale, float* key_abs,
                      void* k_scaled, uint32_t* status, cudaStream_t stream, const void* rope_cos = nullptr,
                      const void* rope_sin = nullptr, int64_t rope_stride = 0, int rope_rows = 0, int rope_position = 0);

}  // namespace hipattn

extern "C" int hipattn_scan_stage(const hipattn_scan_params_t* p, void* stream) {
  using namespace hipattn;
  HIPATTN_REQUIRE(p != nullptr, HIPATTN_ERR_INVALID, "scan params are null");
  HIPATTN_REQUIRE(p->q && p->pos && p->left && p->right && p->score_max && p->status, HIPATTN_ERR_INVALID,
                  "scan stage: q, pos, left, right, score_max and status are required");
  HIPATTN_REQUIRE(p->B > 0 && p->TQ > 0 && p->H > 0 && p->HKV > 0 && p->H % p->HKV == 0 && p->T > 0,
                  HIPATTN_ERR_INVALID, "scan stage: bad shape B=%d TQ=%d H=%d HKV=%d T=%d", p->B, p->TQ, p->H, p->HKV, p->T);
  HIPATTN_REQUIRE(p->block_size_q > 0 && p->stride_q > 0 && p->block_size_q % p->stride_q == 0, HIPATTN_ERR_INVALID,
                  "scan stage: block_size_q %d must be a positive multiple of stride_q %d", p->block_size_q, p->stride_q);
  HIPATTN_REQUIRE(p->block_size_q / p->stride_q <= 256, HIPATTN_ERR_UNSUPPORTED, "scan stage: more than 256 pooled rows");
  HIPATTN_REQUIRE(p->n_chunks >= 0, HIPATTN_ERR_INVALID, "scan stage: negative chunk count");
  HIPATTN_REQUIRE(p->block_chunk >= 16 && (p->block_chunk & (p->block_chunk - 1)) == 0, HIPATTN_ERR_INVALID,
                  "scan stage: block_chunk %d must be a power of two >= 16", p->block_chunk);
  if (p->n_chunks == 0) return HIPATTN_OK;
  const int eb = p->dtype == HIPATTN_F32 ? 4 : 2;
  int rc = validate_tokens(p->k, eb, p->D, "k");
  if (rc) return rc;
  const int64_t ra = 16 / eb;
  HIPATTN_REQUIRE(((uintptr_t)p->q % 16) == 0 && p->q_stride_b % ra == 0 && p->q_stride_t % ra == 0 && p->q_stride_h % ra == 0,
                  HIPATTN_ERR_INVALID, "scan stage: q rows must start on 16-byte boundaries");
  cudaStream_t s = (cudaStream_t)stream;
  HIPATTN_REQUIRE(p->mode >= HIPATTN_SCAN_AUTO && p->mode <= HIPATTN_SCAN_CHECK, HIPATTN_ERR_INVALID, "scan stage: unknown mode %d", p->mode);
  bool handled = false;
  if (p->rope_mode != HIPATTN_ROPE_NONE) {
    // in-kernel RoPE is built into the strict kernel and, for backend "relative" with two prepared key copies, into the
    // tcgen05 kernel
    HIPATTN_REQUIRE(p->rope_mode == HIPATTN_ROPE_RELATIVE || p->rope_mode == HIPATTN_ROPE_STREAMING, HIPATTN_ERR_INVALID,
                    "scan stage: unknown rope_mode %d", p->rope_mode);
    HIPATTN_REQUIRE(p->rope_cos && p->rope_sin && p->rope_rows > 0, HIPATTN_ERR_INVALID, "scan stage: rope_mode without cos / sin tables");
    HIPATTN_REQUIRE(((uintptr_t)p->rope_cos % 16) == 0 && ((uintptr_t)p->rope_sin % 16) == 0 && p->rope_stride % ra == 0 &&
                        p->rope_stride >= p->D / 2,
                    HIPATTN_ERR_INVALID, "scan stage: cos / sin rows must start on 16-byte boundaries and hold D / 2 columns");
    if (p->rope_mode == HIPATTN_ROPE_STREAMING) {   // decode: every token of a chunk is rotated to the chunk's index
      rc = scan_chunks_strict(*p, s, &handled);
      if (handled) return rc;
    }
    // the tensor-core scan takes "relative" with the two rotated copies and "streaming" with the plain copy
    if ((p->rope_mode == HIPATTN_ROPE_RELATIVE && p->k_scaled_sides == 2) ||
        (p->rope_mode == HIPATTN_ROPE_STREAMING && p->k_scaled_sides == 1)) {
      rc = scan_stage_tcgen05(*p, s, &handled);
      if (handled) return rc;
    }
  } else {
  rc = scan_chunks_strict(*p, s, &handled);
  if (handled) return rc;
  rc = scan_stage_tcgen05(*p, s, &handled);
  if (handled) return rc;
  rc = scan_stage_mma(*p, s, &handled);
  if (handled) return rc;
  }
  switch (p->dtype) {
    case HIPATTN_F32: return dispatch_dim<HIPATTN_F32>(*p, s);
    case HIPATTN_F16: return dispatch_dim<HIPATTN_F16>(*p, s);
    case HIPATTN_BF16: return dispatch_dim<HIPATTN_BF16>(*p, s);
    default: set_error("scan stage: unknown dtype %d", p->dtype); return HIPATTN_ERR_INVALID;
  }
}

extern "C" int hipattn_key_abs_sum(const hipattn_tokens_t* k, int32_t dtype, int32_t D, int32_t B, int32_t T, int32_t HKV,
                                   float k_scale, float* out, uint32_t* status, void* stream) {
  using namespace hipattn;
  HIPATTN_REQUIRE(k && out && status, HIPATTN_ERR_INVALID, "key_abs_sum: null pointer");
  HIPATTN_REQUIRE(B > 0 && T > 0 && HKV > 0, HIPATTN_ERR_INVALID, "key_abs_sum: bad shape");
  int rc = validate_tokens(*k, dtype == HIPATTN_F32 ? 4 : 2, D, "k");
  if (rc) return rc;
  return scan_prepare_keys(*k, dtype, D, B, T, HKV, k_scale, out, nullptr, status, (cudaStream_t)stream);
}

extern "C" int hipattn_scan_prepare_keys_rope(const hipattn_tokens_t* k, int32_t dtype, int32_t D, int32_t B, int32_t T, int32_t HKV,
                                              float k_scale, const void* rope_cos, const void* rope_sin, int64_t rope_stride,
                                              int32_t rope_rows, int32_t position, float* key_abs, void* k_scaled, uint32_t* status,
                                              void* stream) {
  using namespace hipattn;
  HIPATTN_REQUIRE(k && status && key_abs && k_scaled && rope_cos && rope_sin, HIPATTN_ERR_INVALID, "scan_prepare_keys_rope: null pointer");
  HIPATTN_REQUIRE(B > 0 && T > 0 && HKV > 0 && rope_rows > 0 && position >= -1 && position < rope_rows &&
                      (position >= 0 || rope_rows >= 2),
                  HIPATTN_ERR_INVALID, "scan_prepare_keys_rope: bad shape or position");
  HIPATTN_REQUIRE(((uintptr_t)k_scaled % 16) == 0 && ((uintptr_t)rope_cos % 16) == 0 && ((uintptr_t)rope_sin % 16) == 0 &&
                      rope_stride % 8 == 0 && rope_stride >= D / 2,
                  HIPATTN_ERR_INVALID, "scan_prepare_keys_rope: k_scaled and the cos / sin rows must be 16-byte aligned");
  int rc = validate_tokens(*k, 2, D, "k");
  if (rc) return rc;
  return scan_prepare_keys(*k, dtype, D, B, T, HKV, k_scale, key_abs, k_scaled, status, (cudaStream_t)stream, rope_cos, rope_sin,
                           rope_stride, rope_rows, position);
}

extern "C" int hipattn_scan_prepare_keys(const hipattn_tokens_t* k, int32_t dtype, int32_t D, int32_t B, int32_t T, int32_t HKV,
                                         float k_scale, float* key_abs, void* k_scaled, uint32_t* status, void* stream) {
  using namespace hipattn;
  HIPATTN_REQUIRE(k && status && (key_abs || k_scaled), HIPATTN_ERR_INVALID, "scan_prepare_keys: null pointer");
  HIPATTN_REQUIRE(B > 0 && T > 0 && HKV > 0, HIPATTN_ERR_INVALID, "scan_prepare_keys: bad shape");
  HIPATTN_REQUIRE(((uintptr_t)k_scaled % 16) == 0, HIPATTN_ERR_INVALID, "scan_prepare_keys: k_scaled must be 16-byte aligned");
  int rc = validate_tokens(*k, dtype == HIPATTN_F32 ? 4 : 2, D, "k");
  if (rc) return rc;
  return scan_prepare_keys(*k, dtype, D, B, T, HKV, k_scale, key_abs, k_scaled, status, (cudaStream_t)stream);
}
