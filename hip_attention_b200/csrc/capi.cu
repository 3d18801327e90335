// C ABI glue: error reporting, argument validation, kernel selection for attention, and the
// log-sum-exp merge of partial outputs.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace hipattn {

static thread_local char g_error[512] = "";
static std::atomic<unsigned long long> g_launches{0};

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int validate_tokens(const hipattn_tokens_t& t, int elem_bytes, int D, const char* name) {
  if (t.fp8_e5m2) {
    HIPATTN_REQUIRE(elem_bytes == 2, HIPATTN_ERR_UNSUPPORTED, "%s: an fp8 cache needs 16-bit queries", name);
    elem_bytes = 2;   // 8-byte pieces of 1-byte elements: the same "multiple of 8 elements" rule as 16-byte pieces of 2-byte ones
  }
  const int64_t row_align = 16 / elem_bytes;
  if (t.cache != nullptr) {
    HIPATTN_REQUIRE(t.block_table && t.cache_seq_lens, HIPATTN_ERR_INVALID, "%s: paged cache without block_table / cache_seq_lens", name);
    HIPATTN_REQUIRE(t.page_size > 0 && t.n_pages > 0 && t.table_width > 0, HIPATTN_ERR_INVALID,
                    "%s: page_size %d, n_pages %lld, table_width %d must be positive", name, t.page_size,
                    (long long)t.n_pages, t.table_width);
    HIPATTN_REQUIRE(((uintptr_t)t.cache % 16) == 0 && t.stride_page % row_align == 0 && t.stride_off % row_align == 0 &&
                        t.stride_ch % row_align == 0,
                    HIPATTN_ERR_INVALID, "%s: cache rows must start on 16-byte boundaries", name);
  } else {
    HIPATTN_REQUIRE(t.dense != nullptr, HIPATTN_ERR_INVALID, "%s: neither a dense tensor nor a page pool was given", name);
    HIPATTN_REQUIRE(((uintptr_t)t.dense % 16) == 0 && t.stride_b % row_align == 0 && t.stride_t % row_align == 0 &&
                        t.stride_h % row_align == 0,
                    HIPATTN_ERR_INVALID, "%s: rows must start on 16-byte boundaries", name);
  }
  HIPATTN_REQUIRE(D % row_align == 0, HIPATTN_ERR_INVALID, "%s: head dimension %d is not a multiple of 16 bytes", name, D);
  return HIPATTN_OK;
}

int bsa_generic(const hipattn_bsa_params_t& p, cudaStream_t stream);
int bsa_mma(const hipattn_bsa_params_t& p, cudaStream_t stream, bool* handled);
int bsa_decode(const hipattn_bsa_params_t& p, cudaStream_t stream, bool* handled);
int bsa_tcgen05(const hipattn_bsa_params_t& p, cudaStream_t stream, bool* handled);
int bounded_wait_probe(uint32_t* status, cudaStream_t stream);

namespace {

template <int DT>
__global__ void merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse, int n_parts, int D,
                             typename Elem<DT>::type* __restrict__ out, int64_t out_stride, float* __restrict__ lse_out) {
  const int64_t row = blockIdx.x;
  const float* lse = part_lse + row * n_parts;
  float m = -INFINITY;
  for (int s = 0; s < n_parts; ++s) m = fmaxf(m, lse[s]);
  float tot = 0.f;
  for (int s = 0; s < n_parts; ++s)
    if (lse[s] > -INFINITY) tot += exp2f(lse[s] - m);
  for (int e = threadIdx.x; e < D; e += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < n_parts; ++s)
      if (lse[s] > -INFINITY) acc += exp2f(lse[s] - m) * part_o[(row * n_parts + s) * D + e];
    out[row * out_stride + e] = Elem<DT>::from_f32(tot > 0.f ? acc / tot : 0.f);
  }
  if (lse_out && threadIdx.x == 0) lse_out[row] = tot > 0.f ? m + log2f(tot) : -INFINITY;
}

// Access statistics of the attention: one CTA per (batch, KV head, attention block) marks the tokens the reference's
// kernels load for that block (see hipattn_mark_attention_access in the header).
__global__ void mark_attention_access_kernel(const hipattn_bsa_params_t p, int32_t* counter, int64_t stride_b, int64_t stride_h,
                                             int n, int window_block_rows) {
  __shared__ int s_pmax;
  const int NBLK = cdiv(p.TQ, p.block_size_q);
  int64_t bid = blockIdx.x;
  const int d = (int)(bid % NBLK); bid /= NBLK;
  const int hkv = (int)(bid % p.HKV); bid /= p.HKV;
  const int b = (int)bid;
  const int t0 = d * p.block_size_q, rows = min(p.block_size_q, p.TQ - t0);
  if (threadIdx.x == 0) s_pmax = -1;
  __syncthreads();
  int hi = -1;
  for (int i = threadIdx.x; i < rows; i += blockDim.x) {
    const long long x = p.pos[(int64_t)b * p.pos_stride_b + (int64_t)(t0 + i) * p.pos_stride_t];
    hi = max(hi, (int)(x > 0x7ffffff0LL ? 0x7ffffff0LL : (x < 0 ? 0 : x)));
  }
  if (hi >= 0) atomicMax(&s_pmax, hi);
  __syncthreads();
  const int cur = s_pmax + 1;   // one past the block's last position
  if (cur <= 0) return;
  const int h = hkv * (p.H / p.HKV);
  const int64_t nrow = (int64_t)b * p.H + h;
  const int d_idx = (int)(((int64_t)d * p.block_size_q) / p.index_block_q);
  long long ks = p.ks[nrow * p.ks_stride_n + (int64_t)d_idx * p.ks_stride_d];
  ks = ks < 0 ? 0 : (ks > p.K ? p.K : ks);
  const int64_t* idx = p.indices + nrow * p.idx_stride_n + (int64_t)d_idx * p.idx_stride_d;
  for (int t = threadIdx.x; t < min(p.sink, cur); t += blockDim.x) mark_access(counter, stride_b, stride_h, n, p.k, b, hkv, t);
  for (int j = threadIdx.x; j < (int)ks * p.block_size_k; j += blockDim.x) {
    const long long t = idx[j / p.block_size_k] + j % p.block_size_k;
    if (t >= p.sink && t < cur && t < p.T) mark_access(counter, stride_b, stride_h, n, p.k, b, hkv, t);
  }
  if (p.window > 0)
    for (int t = max(0, cur - p.window - window_block_rows) + threadIdx.x; t < cur; t += blockDim.x)
      mark_access(counter, stride_b, stride_h, n, p.k, b, hkv, t);
}

}  // namespace
}  // namespace hipattn

using namespace hipattn;

extern "C" int hipattn_mark_attention_access(const hipattn_bsa_params_t* p, int32_t* counter, int64_t stride_b, int64_t stride_h,
                                             int32_t n, int32_t window_block_rows, void* stream) {
  HIPATTN_REQUIRE(p != nullptr && counter != nullptr, HIPATTN_ERR_INVALID, "mark_attention_access: null pointer");
  HIPATTN_REQUIRE(p->pos && p->indices && p->ks, HIPATTN_ERR_INVALID, "mark_attention_access: pos, indices and ks are required");
  HIPATTN_REQUIRE(p->B > 0 && p->TQ > 0 && p->H > 0 && p->HKV > 0 && p->H % p->HKV == 0 && p->T > 0 && n > 0, HIPATTN_ERR_INVALID,
                  "mark_attention_access: bad shape");
  HIPATTN_REQUIRE(p->block_size_q > 0 && p->index_block_q >= p->block_size_q && p->index_block_q % p->block_size_q == 0 &&
                      p->block_size_k > 0 && p->K >= 0 && window_block_rows >= 0,
                  HIPATTN_ERR_INVALID, "mark_attention_access: bad mask geometry");
  if (p->k.cache != nullptr)
    HIPATTN_REQUIRE(p->k.block_table && p->k.cache_seq_lens && p->k.page_size > 0, HIPATTN_ERR_INVALID,
                    "mark_attention_access: paged keys without block_table / cache_seq_lens");
  const int64_t grid = (int64_t)p->B * p->HKV * cdiv(p->TQ, p->block_size_q);
  HIPATTN_REQUIRE(grid < 0x7fffffffLL, HIPATTN_ERR_INVALID, "mark_attention_access: grid of %lld blocks", (long long)grid);
  mark_attention_access_kernel<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(*p, counter, stride_b, stride_h, n, window_block_rows);
  return check_launch("mark_attention_access_kernel");
}

extern "C" int hipattn_bsa_attention(const hipattn_bsa_params_t* p, void* stream) {
  HIPATTN_REQUIRE(p != nullptr, HIPATTN_ERR_INVALID, "attention params are null");
  HIPATTN_REQUIRE(p->q && p->pos && p->indices && p->ks && p->status, HIPATTN_ERR_INVALID,
                  "attention: q, pos, indices, ks and status are required");
  HIPATTN_REQUIRE(p->B > 0 && p->TQ > 0 && p->H > 0 && p->HKV > 0 && p->H % p->HKV == 0 && p->T > 0, HIPATTN_ERR_INVALID,
                  "attention: bad shape B=%d TQ=%d H=%d HKV=%d T=%d", p->B, p->TQ, p->H, p->HKV, p->T);
  HIPATTN_REQUIRE(p->block_size_q > 0 && p->index_block_q >= p->block_size_q && p->index_block_q % p->block_size_q == 0,
                  HIPATTN_ERR_INVALID, "attention: index_block_q %d must be a multiple of block_size_q %d", p->index_block_q,
                  p->block_size_q);
  HIPATTN_REQUIRE(p->block_size_k > 0 && p->K >= 0 && p->sink >= 0 && p->window >= 0, HIPATTN_ERR_INVALID,
                  "attention: bad mask geometry");
  HIPATTN_REQUIRE(p->n_splits >= 1 && p->n_splits <= 64, HIPATTN_ERR_INVALID, "attention: n_splits %d outside [1, 64]", p->n_splits);
  if (p->n_splits > 1) {
    HIPATTN_REQUIRE(p->TQ == 1 && p->part_o && p->part_lse, HIPATTN_ERR_INVALID,
                    "attention: key splits need TQ == 1 and the part_o / part_lse buffers");
  } else {
    HIPATTN_REQUIRE(p->out != nullptr, HIPATTN_ERR_INVALID, "attention: out is null");
  }
  const int eb = p->dtype == HIPATTN_F32 ? 4 : 2;
  const int64_t ra = 16 / eb;
  HIPATTN_REQUIRE(((uintptr_t)p->q % 16) == 0 && p->q_stride_b % ra == 0 && p->q_stride_t % ra == 0 && p->q_stride_h % ra == 0,
                  HIPATTN_ERR_INVALID, "attention: q rows must start on 16-byte boundaries");
  int rc = validate_tokens(p->k, eb, p->D, "k");
  if (rc) return rc;
  rc = validate_tokens(p->v, eb, p->D, "v");
  if (rc) return rc;
  if (p->k.fp8_e5m2 || p->v.fp8_e5m2) {
    // an fp8 KV cache is read by the general kernel (prefill and decode, key splits included), RoPE or not
    if (p->rope_cos || p->rope_sin)
      HIPATTN_REQUIRE(p->rope_cos && p->rope_sin && p->rope_rows > 0, HIPATTN_ERR_INVALID, "attention: cos and sin tables go together");
    return bsa_generic(*p, (cudaStream_t)stream);
  }
  if (p->rope_cos || p->rope_sin) {
    // in-kernel RoPE is built into the tcgen05 prefill kernel (head dim 128), the mma.sync decode and prefill kernels
    // (16-bit, head dim 64 / 128) and the general kernel (everything else)
    HIPATTN_REQUIRE(p->rope_cos && p->rope_sin && p->rope_rows > 0, HIPATTN_ERR_INVALID, "attention: cos and sin tables go together");
    HIPATTN_REQUIRE(((uintptr_t)p->rope_cos % 16) == 0 && ((uintptr_t)p->rope_sin % 16) == 0 && p->rope_stride % ra == 0 &&
                        p->rope_stride >= p->D / 2,
                    HIPATTN_ERR_INVALID, "attention: cos / sin rows must start on 16-byte boundaries and hold D / 2 columns");
    bool done = false;
    rc = bsa_decode(*p, (cudaStream_t)stream, &done);
    if (done) return rc;
    const char* pk_ = getenv("HIPATTN_PREFILL_KERNEL");
    if (!(pk_ && strcmp(pk_, "mma") == 0)) {
      rc = bsa_tcgen05(*p, (cudaStream_t)stream, &done);
      if (done) return rc;
    }
    rc = bsa_mma(*p, (cudaStream_t)stream, &done);
    if (done) return rc;
    return bsa_generic(*p, (cudaStream_t)stream);
  }
  bool handled = false;
  rc = bsa_decode(*p, (cudaStream_t)stream, &handled);
  if (handled) return rc;
  // HIPATTN_PREFILL_KERNEL = tcgen05 (default: warp-specialised tcgen05 kernel) | mma (mma.sync kernel, for comparisons)
  const char* pk = getenv("HIPATTN_PREFILL_KERNEL");
  if (!(pk && strcmp(pk, "mma") == 0)) {
    rc = bsa_tcgen05(*p, (cudaStream_t)stream, &handled);
    if (handled) return rc;
  }
  rc = bsa_mma(*p, (cudaStream_t)stream, &handled);
  if (handled) return rc;
  return bsa_generic(*p, (cudaStream_t)stream);
}

extern "C" int hipattn_merge_partials(const float* part_o, const float* part_lse, int64_t rows, int32_t n_parts, int32_t D,
                                      int32_t dtype, void* out, int64_t out_stride, float* lse_out, void* stream) {
  HIPATTN_REQUIRE(part_o && part_lse && out, HIPATTN_ERR_INVALID, "merge_partials: null pointer");
  HIPATTN_REQUIRE(rows > 0 && n_parts > 0 && D > 0, HIPATTN_ERR_INVALID, "merge_partials: bad sizes");
  const int threads = D >= 128 ? 128 : 64;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case HIPATTN_F32:
      merge_kernel<HIPATTN_F32><<<(unsigned)rows, threads, 0, s>>>(part_o, part_lse, n_parts, D, (float*)out, out_stride, lse_out);
      break;
    case HIPATTN_F16:
      merge_kernel<HIPATTN_F16><<<(unsigned)rows, threads, 0, s>>>(part_o, part_lse, n_parts, D, (__half*)out, out_stride, lse_out);
      break;
    case HIPATTN_BF16:
      merge_kernel<HIPATTN_BF16><<<(unsigned)rows, threads, 0, s>>>(part_o, part_lse, n_parts, D, (__nv_bfloat16*)out, out_stride, lse_out);
      break;
    default: set_error("merge_partials: unknown dtype %d", dtype); return HIPATTN_ERR_INVALID;
  }
  return check_launch("merge_kernel");
}

extern "C" int32_t hipattn_encode_score(float score) {
  uint32_t bits;
  memcpy(&bits, &score, 4);
  return encode_score_bits(bits);
}
extern "C" float hipattn_decode_score(int32_t code) {
  uint32_t bits = decode_score_bits(code);
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

extern "C" int hipattn_debug_bounded_wait(uint32_t* status, void* stream) {
  HIPATTN_REQUIRE(status != nullptr, HIPATTN_ERR_INVALID, "debug_bounded_wait: status is null");
  return bounded_wait_probe(status, (cudaStream_t)stream);
}

extern "C" uint64_t hipattn_launch_count(void) { return hipattn::g_launches.load(std::memory_order_relaxed); }
extern "C" const char* hipattn_error_string(void) { return g_error; }
extern "C" int hipattn_abi_version(void) { return 9; }
