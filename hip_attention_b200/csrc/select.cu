// Chunk-list bookkeeping between scan stages: initial list, top-k selection + split into the next
// stage's chunks, and the final conversion to sorted unique block indices.
//
// One CTA owns one (batch, query block) row and sorts it in shared memory with a bitonic network on
// composite 64-bit keys (inverted score image << 32 | position), which makes the order total:
// higher score first, lower chunk position first among equal scores.
#include "common.cuh"

namespace hipattn {
namespace {

constexpr int kSortThreads = 512;

__host__ __device__ inline int next_pow2(int x) {
  int p = 1;
  while (p < x) p <<= 1;
  return p;
}

template <typename K>
__device__ void bitonic_sort(K* a, int N) {
  for (int k = 2; k <= N; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = threadIdx.x; i < (N >> 1); i += blockDim.x) {
        const int l = ((i & ~(j - 1)) << 1) | (i & (j - 1));
        const int r = l | j;
        const bool up = (l & k) == 0;
        const K x = a[l], y = a[r];
        if ((x > y) == up) {
          a[l] = y;
          a[r] = x;
        }
      }
      __syncthreads();
    }
  }
}

__global__ void init_chunks_kernel(int32_t* left, int32_t* right, int32_t* score_max, int64_t total, int n, int sink,
                                   int chunk, int T, int scan_window) {
  const int32_t init = encode_score(HIPATTN_SCORE_INIT);
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % n);
    const int l = sink + c * chunk;
    left[i] = l;
    right[i] = min(l + chunk, T - scan_window);
    score_max[i] = init;
  }
}

// Load the row's scores as ascending sort keys: best score first, lower position first on ties.
__device__ void load_score_keys(unsigned long long* keys, const int32_t* score_max, int n, int n_pad) {
  for (int i = threadIdx.x; i < n_pad; i += blockDim.x)
    keys[i] = i < n ? score_sort_key(score_max[i], (unsigned)i) : ~0ull;
  __syncthreads();
}

__global__ void __launch_bounds__(kSortThreads) select_stage_kernel(const int32_t* __restrict__ score_max,
                                                                    const int32_t* __restrict__ left, int n, int n_pad,
                                                                    int k_keep, int k_pad, int sink, int c_prev,
                                                                    int c_next, int32_t* __restrict__ next_left,
                                                                    int32_t* __restrict__ next_right,
                                                                    int32_t* __restrict__ next_score_max) {
  extern __shared__ __align__(16) unsigned char smem[];
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(smem);
  const int64_t row = blockIdx.x;
  load_score_keys(keys, score_max + row * n, n, n_pad);
  bitonic_sort(keys, n_pad);

  // the k_keep best chunks, realigned to the previous chunk grid, ordered by their left bound
  // (entry j is read and rewritten by the same thread, so the update is done in place)
  for (int j = threadIdx.x; j < k_pad; j += blockDim.x) {
    unsigned long long v = ~0ull;
    if (j < k_keep) {
      const int idx = (int)(keys[j] & 0xffffffffu);
      const int l = left[row * n + idx];
      const int la = (l - sink) / c_prev * c_prev + sink;  // l >= sink
      v = ((unsigned long long)(unsigned)la << 32) | (unsigned)j;
    }
    keys[j] = v;
  }
  __syncthreads();
  bitonic_sort(keys, k_pad);

  const int s = c_prev / c_next;
  const int64_t out_n = (int64_t)k_keep * s;
  const int32_t init = encode_score(HIPATTN_SCORE_INIT);
  for (int64_t o = threadIdx.x; o < out_n; o += blockDim.x) {
    const int j = (int)(o / s), i = (int)(o - (int64_t)j * s);
    const int la = (int)(keys[j] >> 32);
    const int ra = la + c_prev;
    // attention_extend.py:2133-2165: chunk sizes and offsets go through fp32
    const float w = fmaxf(__fdiv_rn((float)(ra - la), (float)s), 0.f);
    next_left[row * out_n + o] = la + (int)floorf(__fmul_rn((float)i, w));
    next_right[row * out_n + o] = ra - (int)floorf(__fmul_rn((float)(s - 1 - i), w));
    next_score_max[row * out_n + o] = init;
  }
}

__global__ void __launch_bounds__(kSortThreads)
    finalize_kernel(const int32_t* __restrict__ score_max, const int32_t* __restrict__ left_heads, int64_t left_row_stride,
                    int64_t left_head_stride, const int64_t* __restrict__ pos, int64_t pos_stride_b, int64_t pos_stride_t,
                    int BDST, int H, int n, int n_pad, int K, int K_pad, int c_last, int block_size_q,
                    int64_t* __restrict__ indices, int64_t* __restrict__ ks, int32_t* __restrict__ ks_start_end) {
  extern __shared__ __align__(16) unsigned char smem[];
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(smem);
  uint32_t* cand = reinterpret_cast<uint32_t*>(smem + (size_t)n_pad * sizeof(unsigned long long));
  __shared__ int s_count;
  const int64_t row = blockIdx.x;
  const int b = (int)(row / BDST), d = (int)(row % BDST);
  load_score_keys(keys, score_max + row * n, n, n_pad);
  bitonic_sort(keys, n_pad);

  const long long limit = pos[(int64_t)b * pos_stride_b + (int64_t)d * block_size_q * pos_stride_t] + block_size_q;
  const int n_heads_distinct = left_head_stride == 0 ? 1 : H;
  for (int hh = 0; hh < n_heads_distinct; ++hh) {
    const int32_t* lh = left_heads + row * left_row_stride + (int64_t)hh * left_head_stride;
    for (int j = threadIdx.x; j < K_pad; j += blockDim.x) {
      uint32_t v = 0xffffffffu;
      if (j < K) {
        const int idx = (int)(keys[j] & 0xffffffffu);
        v = (uint32_t)(lh[idx] / c_last * c_last);
      }
      cand[j] = v;
    }
    if (threadIdx.x == 0) s_count = 0;
    __syncthreads();
    bitonic_sort(cand, K_pad);
    // duplicates (compared with the previous entry, wrapping around) become padding
    uint32_t mine[4];
    int cnt = 0;
    for (int j = threadIdx.x, q = 0; j < K_pad; j += blockDim.x, ++q) {
      uint32_t v = 0xffffffffu;
      if (j < K) {
        const uint32_t prev = cand[(j + K - 1) % K];
        v = cand[j];
        if (prev == v) v = 0xffffffffu;
      }
      mine[q & 3] = v;
      ++cnt;
    }
    __syncthreads();
    for (int j = threadIdx.x, q = 0; j < K_pad; j += blockDim.x, ++q) cand[j] = mine[q & 3];
    __syncthreads();
    bitonic_sort(cand, K_pad);
    int local = 0;
    for (int j = threadIdx.x; j < K; j += blockDim.x) {
      const uint32_t v = cand[j];
      const long long v64 = v == 0xffffffffu ? INT64_MAX : (long long)v;
      local += v64 < limit ? 1 : 0;
      if (n_heads_distinct == 1) {
        for (int h = 0; h < H; ++h) indices[(((int64_t)b * H + h) * BDST + d) * K + j] = v64;
      } else {
        indices[(((int64_t)b * H + hh) * BDST + d) * K + j] = v64;
      }
    }
    atomicAdd(&s_count, local);
    __syncthreads();
    if (threadIdx.x == 0) {
      const int c = s_count;
      for (int h = (n_heads_distinct == 1 ? 0 : hh); h < (n_heads_distinct == 1 ? H : hh + 1); ++h) {
        const int64_t o = ((int64_t)b * H + h) * BDST + d;
        ks[o] = c;
        ks_start_end[o * 2] = 0;
        ks_start_end[o * 2 + 1] = c;
      }
    }
    __syncthreads();
  }
}

__global__ void decode_scores_kernel(const int32_t* codes, float* scores, int64_t count) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x)
    scores[i] = decode_score(codes[i]);
}
__global__ void widen_kernel(const int32_t* src, int64_t* dst, int64_t count) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x)
    dst[i] = src[i];
}

inline unsigned grid_for(int64_t total, int threads) {
  int64_t g = (total + threads - 1) / threads;
  return (unsigned)(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
}

}  // namespace
}  // namespace hipattn

using namespace hipattn;

extern "C" int hipattn_init_chunks(int32_t* left, int32_t* right, int32_t* score_max, int64_t rows, int32_t n,
                                   int32_t sink, int32_t chunk, int32_t T, int32_t scan_window, void* stream) {
  HIPATTN_REQUIRE(rows >= 0 && n >= 0 && chunk > 0 && sink >= 0, HIPATTN_ERR_INVALID, "init_chunks: bad sizes");
  if (rows * n == 0) return HIPATTN_OK;
  HIPATTN_REQUIRE(left && right && score_max, HIPATTN_ERR_INVALID, "init_chunks: null output");
  init_chunks_kernel<<<grid_for(rows * n, 256), 256, 0, (cudaStream_t)stream>>>(left, right, score_max, rows * n, n, sink,
                                                                                chunk, T, scan_window);
  return check_launch("init_chunks_kernel");
}

extern "C" int hipattn_select_stage(const int32_t* score_max, const int32_t* left, int64_t rows, int32_t n, int32_t k_keep,
                                    int32_t sink, int32_t c_prev, int32_t c_next, int32_t* next_left,
                                    int32_t* next_right, int32_t* next_score_max, void* stream) {
  HIPATTN_REQUIRE(score_max && left && next_left && next_right && next_score_max, HIPATTN_ERR_INVALID,
                  "select_stage: null pointer");
  HIPATTN_REQUIRE(rows > 0 && n > 0 && k_keep > 0 && k_keep <= n, HIPATTN_ERR_INVALID,
                  "select_stage: need 0 < k_keep (%d) <= n (%d)", k_keep, n);
  HIPATTN_REQUIRE(n <= HIPATTN_MAX_CHUNKS, HIPATTN_ERR_UNSUPPORTED, "select_stage: %d chunks per row exceed %d", n,
                  HIPATTN_MAX_CHUNKS);
  HIPATTN_REQUIRE(c_next > 0 && c_prev % c_next == 0, HIPATTN_ERR_INVALID,
                  "select_stage: chunk size %d is not a multiple of %d", c_prev, c_next);
  const int n_pad = next_pow2(n < 2 ? 2 : n), k_pad = next_pow2(k_keep < 2 ? 2 : k_keep);
  const size_t smem = (size_t)n_pad * sizeof(unsigned long long);
  HIPATTN_CUDA_OK(cudaFuncSetAttribute(select_stage_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  select_stage_kernel<<<(unsigned)rows, kSortThreads, smem, (cudaStream_t)stream>>>(
      score_max, left, n, n_pad, k_keep, k_pad, sink, c_prev, c_next, next_left, next_right, next_score_max);
  return check_launch("select_stage_kernel");
}

extern "C" int hipattn_finalize_indices(const int32_t* score_max, const int32_t* left_heads, int64_t left_row_stride,
                                        int64_t left_head_stride, const int64_t* pos, int64_t pos_stride_b,
                                        int64_t pos_stride_t, int32_t B, int32_t BDST, int32_t H, int32_t n, int32_t K,
                                        int32_t c_last, int32_t block_size_q, int64_t* indices, int64_t* ks,
                                        int32_t* ks_start_end, void* stream) {
  HIPATTN_REQUIRE(score_max && left_heads && pos && indices && ks && ks_start_end, HIPATTN_ERR_INVALID,
                  "finalize_indices: null pointer");
  HIPATTN_REQUIRE(B > 0 && BDST > 0 && H > 0 && n > 0 && K > 0 && K <= n && c_last > 0, HIPATTN_ERR_INVALID,
                  "finalize_indices: need 0 < K (%d) <= n (%d)", K, n);
  HIPATTN_REQUIRE(n <= HIPATTN_MAX_CHUNKS, HIPATTN_ERR_UNSUPPORTED, "finalize_indices: %d chunks per row exceed %d", n,
                  HIPATTN_MAX_CHUNKS);
  const int n_pad = next_pow2(n < 2 ? 2 : n), K_pad = next_pow2(K < 2 ? 2 : K);
  HIPATTN_REQUIRE(K_pad <= 4 * kSortThreads, HIPATTN_ERR_UNSUPPORTED, "finalize_indices: K = %d exceeds %d", K,
                  4 * kSortThreads);
  const size_t smem = (size_t)n_pad * sizeof(unsigned long long) + (size_t)K_pad * sizeof(uint32_t);
  HIPATTN_CUDA_OK(cudaFuncSetAttribute(finalize_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  finalize_kernel<<<(unsigned)(B * BDST), kSortThreads, smem, (cudaStream_t)stream>>>(
      score_max, left_heads, left_row_stride, left_head_stride, pos, pos_stride_b, pos_stride_t, BDST, H, n, n_pad, K,
      K_pad, c_last, block_size_q, indices, ks, ks_start_end);
  return check_launch("finalize_kernel");
}

extern "C" int hipattn_decode_scores(const int32_t* codes, float* scores, int64_t count, void* stream) {
  if (count <= 0) return HIPATTN_OK;
  HIPATTN_REQUIRE(codes && scores, HIPATTN_ERR_INVALID, "decode_scores: null pointer");
  decode_scores_kernel<<<grid_for(count, 256), 256, 0, (cudaStream_t)stream>>>(codes, scores, count);
  return check_launch("decode_scores_kernel");
}

extern "C" int hipattn_widen_i32(const int32_t* src, int64_t* dst, int64_t count, void* stream) {
  if (count <= 0) return HIPATTN_OK;
  HIPATTN_REQUIRE(src && dst, HIPATTN_ERR_INVALID, "widen_i32: null pointer");
  widen_kernel<<<grid_for(count, 256), 256, 0, (cudaStream_t)stream>>>(src, dst, count);
  return check_launch("widen_kernel");
}
