// Scan stage of the mask estimator for decode (one pooled query row per head), small chunks, strict
// arithmetic: every token of every active chunk is fetched ONCE for all query heads of a KV head, scored
// against each head's query with the strict dot product, and the halving search of the reference
// (attention_extend.py:413-1249) is replayed on the stored scores.
//
// The search of a chunk only ever scores tokens of that chunk, two per round and head.  In decode the key
// rows come from HBM (the cache of a batch is far larger than L2), so rows fetched are time: for a last
// stage of chunk 8 and four heads per KV head the rounds fetch 4 x 2 x 4 = 32 rows per chunk, the whole
// chunk is 8; for chunk 32 it is 48 against 32.  Scores are the strict kernel's (sequential fp32 dot over
// the head dimension of round(k * k_scale), rounded to the element type), comparisons are the reference's,
// so bounds and scores are identical to scan_stage_kernel's.
//
// Mapping: a warp takes 32 consecutive rows = 32 / chunk whole chunks per pass; lane = token.  The rows
// are gathered with 16-byte cp.async (through the page table when the keys are paged) into a per-warp
// staging area, every lane scores its own row against the HB head queries held in shared memory as fp32,
// the rounded scores go to a per-warp table and the first HB lanes of every chunk walk the search tree.
// No block-wide barrier after the prologue; six CTAs of four warps per SM keep about 190 KB of rows in flight.
#include <cstdlib>
#include <cstring>

#include "scan_common.cuh"

namespace hipattn {
namespace {

constexpr int kPadS = 16;  // bytes of padding per staged key row: keeps 16-byte lane reads conflict free

template <int DT>
__device__ __forceinline__ void unpack_scaled_s(const uint4& w, float k_scale, float* out);
template <>
__device__ __forceinline__ void unpack_scaled_s<HIPATTN_F32>(const uint4& w, float k_scale, float* out) {
  out[0] = __fmul_rn(__uint_as_float(w.x), k_scale);
  out[1] = __fmul_rn(__uint_as_float(w.y), k_scale);
  out[2] = __fmul_rn(__uint_as_float(w.z), k_scale);
  out[3] = __fmul_rn(__uint_as_float(w.w), k_scale);
}
// 16-bit types: one packed multiply per element pair.  The product of two 16-bit floats is exact in fp32,
// so rounding it once to the element type (what the packed multiply does) equals multiplying in fp32 and
// converting, at a third of the instructions.
template <>
__device__ __forceinline__ void unpack_scaled_s<HIPATTN_BF16>(const uint4& w, float k_scale, float* out) {
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
__device__ __forceinline__ void unpack_scaled_s<HIPATTN_F16>(const uint4& w, float k_scale, float* out) {
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
__device__ __forceinline__ float mac_s(float q, float k, float acc) {
  if (DT == HIPATTN_F32) return __fadd_rn(acc, __fmul_rn(q, k));  // two roundings, reproducible on a CPU
  return fmaf(q, k, acc);                                         // 16-bit inputs: the product is exact
}

// ROPE_S = in-kernel RoPE, backend "streaming": every token of a chunk is rotated to the chunk's index before the key
// scale (a token's score then does not depend on the side it is proposed for, so one score per token serves the search)
template <int DT, int D, int HB, bool ROPE_S>
__global__ void __launch_bounds__(128) scan_chunks_strict_kernel(const hipattn_scan_params_t p, int c_log2, int n_split, int passes_total) {
  constexpr int EB = Elem<DT>::bytes;
  constexpr int ROWB = D * EB;
  constexpr int STRIDE = ROWB + kPadS;
  constexpr int PIECES = ROWB / 16;
  constexpr int VEC = 16 / EB;
  extern __shared__ __align__(16) unsigned char smem[];
  float* qtile = reinterpret_cast<float*>(smem);                         // [HB][D]
  unsigned char* kstage = smem + (size_t)HB * D * sizeof(float);         // [4 warps][32][STRIDE]
  __shared__ int s_pmin;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
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
  const int t0 = d * p.block_size_q;
  const bool has_row = t0 < p.TQ;

  // the single pooled query row of every head of the batch
  for (int i = threadIdx.x; i < HB * PIECES; i += 128) {
    const int hh = i / PIECES, pc = i % PIECES;
    float v[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) v[e] = 0.f;
    if (has_row) pooled_query_piece<DT>(p, b, h0 + hh, t0, pc, v);
#pragma unroll
    for (int e = 0; e < VEC; e += 4)
      *reinterpret_cast<float4*>(qtile + hh * D + pc * VEC + e) = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
  }
  if (warp == 0) {
    const int m = block_min_position(p, b, t0, has_row ? 1 : 0, lane);
    if (lane == 0) s_pmin = m;
  }
  __syncthreads();
  if (!has_row) return;
  const int pt = max(s_pmin - p.scan_window, 0);
  const int C = 1 << c_log2;
  const int cpp_log2 = 5 - c_log2;                  // chunks per pass = 32 / C
  const int n = p.n_chunks;
  const int64_t row = (int64_t)b * BDST + d;
  const int32_t* gl = p.left + row * n;
  const int32_t* gr = p.right + row * n;
  const int bc_log2 = 31 - __clz(p.block_chunk);
  unsigned char* wstage = kstage + (size_t)warp * 32 * STRIDE;
  const unsigned char* my_row = wstage + (size_t)lane * STRIDE;
  float* wtab = reinterpret_cast<float*>(wstage);   // [HB][32] rounded scores: reuses the staging area once every lane has scored its row
  const int grp_base = lane & ~(C - 1);             // first lane of this lane's chunk
  const int cl = lane >> c_log2;                    // chunk of the pass
  int cur_group = -1, cur_gmax = 0;

  // What a pass needs before its rows can be requested: this lane's chunk bounds and the address of its token's row
  // (two dependent global reads: the bounds, then the page table).  Resolved one pass ahead, while the rows of the
  // current pass are on their way, so that neither read is part of a pass's chain.
  struct PassInput {
    int l, rt;
    bool valid;
    const char* src;
  };
  auto resolve_pass = [&](int ps) {
    PassInput in{0, 0, false, nullptr};
    if (ps >= passes_total) return in;
    const int c = (ps << cpp_log2) + cl;
    if (c < n) { in.l = __ldg(gl + c); in.rt = __ldg(gr + c); }
    if (in.rt - in.l > C) atomicOr(p.status, HIPATTN_STATUS_CHUNK_SIZE);
    const bool chunk_act = c < n && in.l < in.rt && in.l <= pt && in.l >= 0;
    int tk = in.l + (lane & (C - 1));
    in.valid = chunk_act && tk < in.rt;
    if (in.valid) {
      if (p.k.cache == nullptr && tk >= p.T) {
        atomicOr(p.status, HIPATTN_STATUS_TOKEN_RANGE);
        tk = p.T - 1;
      }
      in.src = token_row(p.k, b, tk, hkv, EB, p.status);
    }
    return in;
  };

  // passes of this warp: the unit's passes are dealt to the n_split CTAs x 4 warps round-robin
  const int ps_step = n_split * 4;
  PassInput next_in = resolve_pass(split * 4 + warp);
  for (int ps = split * 4 + warp; ps < passes_total; ps += ps_step) {
    const int c = (ps << cpp_log2) + cl;
    const PassInput in = next_in;
    const int l = in.l, rt = in.rt;
    // halving rounds: from the largest chunk of the reference group of block_chunk chunks (all chunks of a
    // pass lie in one group: a pass holds at most 8 chunks, a group at least 16, both powers of two)
    const int group = (ps << cpp_log2) >> bc_log2;
    if (group != cur_group) {
      int m = 0;
      const int gbase = group << bc_log2;
      for (int i = lane; i < p.block_chunk; i += 32) {
        const int cc = gbase + i;
        if (cc < n) m = max(m, gr[cc] - gl[cc]);
      }
      cur_gmax = __reduce_max_sync(0xffffffffu, m);
      cur_group = group;
    }
    const int rounds = cur_gmax >= 1 ? 32 - __clz(cur_gmax) : 0;
    const bool valid = in.valid;
    const char* src = in.src;
    const bool any_valid = __any_sync(0xffffffffu, valid);
    if (!any_valid) next_in = resolve_pass(ps + ps_step);
    if (any_valid) {   // chunks that are not active still report their (unchanged) bounds below
    // cooperative gather of the pass's 32 rows
    __syncwarp();
    if (PIECES <= 32) {
      constexpr int RPI = 32 / PIECES > 0 ? 32 / PIECES : 1;     // rows per instruction
      const int sub = lane / PIECES, piece = lane % PIECES;
#pragma unroll 4
      for (int r0 = 0; r0 < 32; r0 += RPI) {
        const int rr = r0 + sub;
        const unsigned long long a = __shfl_sync(0xffffffffu, (unsigned long long)src, rr & 31);
        if (a != 0ull && sub < RPI) cp_async16(wstage + (size_t)rr * STRIDE + piece * 16, (const char*)a + piece * 16);
      }
    } else {
      for (int rr = 0; rr < 32; ++rr) {
        const unsigned long long a = __shfl_sync(0xffffffffu, (unsigned long long)src, rr);
        if (a != 0ull)
          for (int piece = lane; piece < PIECES; piece += 32) cp_async16(wstage + (size_t)rr * STRIDE + piece * 16, (const char*)a + piece * 16);
      }
    }
    cp_async_commit();
    next_in = resolve_pass(ps + ps_step);   // the next pass's bounds and row address travel with this pass's rows
    cp_async_wait<0>();
    __syncwarp();
    // strict scores of this lane's token for the HB heads
    float acc[HB];
#pragma unroll
    for (int hh = 0; hh < HB; ++hh) acc[hh] = 0.f;
    if (valid) {
#pragma unroll 2
      for (int pc = 0; pc < PIECES; ++pc) {
        float kv[VEC];
        if (ROPE_S) unpack_rope_scaled<DT, D>(my_row, pc, c, p, kv);
        else unpack_scaled_s<DT>(*reinterpret_cast<const uint4*>(my_row + pc * 16), p.k_scale, kv);
#pragma unroll
        for (int hh = 0; hh < HB; ++hh) {
#pragma unroll
          for (int e4 = 0; e4 < VEC; e4 += 4) {
            const float4 qv = *reinterpret_cast<const float4*>(qtile + hh * D + pc * VEC + e4);
            acc[hh] = mac_s<DT>(qv.x, kv[e4 + 0], acc[hh]);
            acc[hh] = mac_s<DT>(qv.y, kv[e4 + 1], acc[hh]);
            acc[hh] = mac_s<DT>(qv.z, kv[e4 + 2], acc[hh]);
            acc[hh] = mac_s<DT>(qv.w, kv[e4 + 3], acc[hh]);
          }
        }
      }
    }
    __syncwarp();     // every lane is done with its staged row: the area now holds the score table
    if (valid) {
#pragma unroll
      for (int hh = 0; hh < HB; ++hh) wtab[hh * 32 + lane] = Elem<DT>::round(acc[hh]);
    }
    __syncwarp();
    }
    __syncwarp();
    // the first HB lanes of every chunk replay the search of one head each
    const int hh = lane - grp_base;
    const bool walker = hh < HB && c < n;
    float score = HIPATTN_SCORE_INIT;
    if (walker) {
      int wl = l, wr = rt;
      const float* sc = wtab + hh * 32 + grp_base;
      for (int it = 0; it < rounds; ++it) {
        if (!(wl < wr && wl <= pt && wl >= 0)) break;
        const int mid = (wl + wr) >> 1;
        if (p.access_counter) {   // the rows the reference's round would have loaded
          mark_access(p.access_counter, p.access_stride_b, p.access_stride_h, p.access_n, p.k, b, hkv, (wl + mid) >> 1);
          mark_access(p.access_counter, p.access_stride_b, p.access_stride_h, p.access_n, p.k, b, hkv, (mid + wr) >> 1);
        }
        const float sl = sc[min(((wl + mid) >> 1) - l, C - 1)];
        const float sr = sc[min(((mid + wr) >> 1) - l, C - 1)];
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
    if (walker && hh == 0 && best > HIPATTN_SCORE_INIT) atomicMax(p.score_max + row * n + c, encode_score(best));
    __syncwarp();
  }
}

template <int DT, int D, int HB, bool ROPE_S>
int launch(const hipattn_scan_params_t& p, int c_log2, cudaStream_t stream) {
  constexpr int EB = Elem<DT>::bytes;
  const size_t smem = (size_t)HB * D * sizeof(float) + (size_t)4 * 32 * (D * EB + kPadS);
  HIPATTN_REQUIRE(smem <= 227 * 1024, HIPATTN_ERR_UNSUPPORTED, "chunk scan stage needs %zu bytes of shared memory", smem);
  const int BDST = cdiv(p.TQ, p.block_size_q);
  const int Gq = p.H / p.HKV;
  const int passes_total = cdiv(p.n_chunks, 32 >> c_log2);
  const int64_t units = (int64_t)p.B * p.HKV * BDST * (Gq / HB);
  // enough CTAs to fill the GPU about six deep, never more than there are passes for four warps each
  int64_t want = (148 * 6 * 2 + units - 1) / units;
  const int64_t most = cdiv(passes_total, 4);
  int n_split = (int)(want < 1 ? 1 : (want > most ? most : want));
  if (n_split < 1) n_split = 1;
  const int64_t grid = units * n_split;
  HIPATTN_REQUIRE(grid > 0 && grid < 0x7fffffffLL, HIPATTN_ERR_INVALID, "scan grid of %lld blocks", (long long)grid);
  auto kern = scan_chunks_strict_kernel<DT, D, HB, ROPE_S>;
  HIPATTN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<(unsigned)grid, 128, smem, stream>>>(p, c_log2, n_split, passes_total);
  return check_launch("scan_chunks_strict_kernel");
}

template <int DT, int D>
int dispatch_heads(const hipattn_scan_params_t& p, int c_log2, int HB, cudaStream_t stream) {
  if (p.rope_mode == HIPATTN_ROPE_STREAMING) {
    switch (HB) {
      case 4: return launch<DT, D, 4, true>(p, c_log2, stream);
      case 2: return launch<DT, D, 2, true>(p, c_log2, stream);
      default: return launch<DT, D, 1, true>(p, c_log2, stream);
    }
  }
  switch (HB) {
    case 4: return launch<DT, D, 4, false>(p, c_log2, stream);
    case 2: return launch<DT, D, 2, false>(p, c_log2, stream);
    default: return launch<DT, D, 1, false>(p, c_log2, stream);
  }
}

template <int DT>
int dispatch_dim(const hipattn_scan_params_t& p, int c_log2, int HB, cudaStream_t stream) {
  switch (p.D) {
    case 64: return dispatch_heads<DT, 64>(p, c_log2, HB, stream);
    case 128: return dispatch_heads<DT, 128>(p, c_log2, HB, stream);
    default: return dispatch_heads<DT, 256>(p, c_log2, HB, stream);
  }
}

}  // namespace

// Decode shapes (a single pooled query row) whose chunk size is a known power of two between 4 and 32 and no
// larger than the number of rows the rounds of the heads sharing the chunk would fetch.
// HIPATTN_DECODE_SCAN=rounds keeps the round-by-round kernel.
int scan_chunks_strict(const hipattn_scan_params_t& p, cudaStream_t stream, bool* handled) {
  *handled = false;
  const int R = p.block_size_q / p.stride_q;
  const int rows = min(R, cdiv(p.TQ, p.stride_q));
  if (rows > 1 || (p.D != 64 && p.D != 128 && p.D != 256)) return HIPATTN_OK;
  if (p.k.fp8_e5m2) return HIPATTN_OK;   // an fp8 cache goes through the round-by-round kernel
  // in-kernel RoPE: "streaming" rotates a chunk's tokens alike; "relative" scores a token by the side it is proposed for
  if (p.rope_mode != HIPATTN_ROPE_NONE && p.rope_mode != HIPATTN_ROPE_STREAMING) return HIPATTN_OK;
  const int C = p.chunk_size;
  if (C < 4 || C > 32 || (C & (C - 1)) != 0) return HIPATTN_OK;
  const char* v = getenv("HIPATTN_DECODE_SCAN");
  if (v && strcmp(v, "rounds") == 0) return HIPATTN_OK;
  int c_log2 = 0;
  while ((1 << c_log2) < C) ++c_log2;
  const int Gq = p.H / p.HKV;
  int HB = 4;
  while (HB > 1 && Gq % HB != 0) HB >>= 1;
  if (C > HB * 2 * (c_log2 + 1)) return HIPATTN_OK;
  *handled = true;
  switch (p.dtype) {
    case HIPATTN_F32: return dispatch_dim<HIPATTN_F32>(p, c_log2, HB, stream);
    case HIPATTN_F16: return dispatch_dim<HIPATTN_F16>(p, c_log2, HB, stream);
    default: return dispatch_dim<HIPATTN_BF16>(p, c_log2, HB, stream);
  }
}

}  // namespace hipattn
