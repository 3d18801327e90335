// Split-KV decode attention for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc at all once they are running: an inference
// server that hands its whole memory budget to a KV-cache pool at start-up, a plugin that is only
// given pointers by its framework and has no allocator of its own, or code running where an
// allocation would synchronise the device.  The split-KV decode path needs a small scratch area
// (per-split partial outputs and their log-sum-exp) between its two kernels, which the regular entry
// point expects the caller to provide.  This file gives those hosts one extra entry point whose
// scratch lives in a fixed array inside the library image instead.
//
// Cost and limits: the array below occupies HIPATTN_NOALLOC_SCRATCH_BYTES on every GPU that loads
// the library, for the life of the process, whether or not the entry point is ever called.  All
// calls on one device share it, and it keeps whatever the previous call left there.  Every element
// a call reads is first written by that same call, so nothing has to be cleared; but two calls that
// overlap on the GPU (different streams, or graphs replayed concurrently) would race on it -- issue
// them so that they run one after the other.
#include <mutex>

#include "bsa_common.cuh"

namespace {

constexpr size_t kScratchFloats = HIPATTN_NOALLOC_SCRATCH_BYTES / sizeof(float);
static __device__ __align__(256) float g_noalloc_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
float* g_scratch_dev_ptr[kMaxDevices] = {};  // device address of g_noalloc_scratch, per device

// In host code the name g_noalloc_scratch is only a handle; the address a kernel can use has to be
// asked for, once per device, with that device current.
int scratch_for_current_device(float** out) {
  using namespace hipattn;
  int dev = -1;
  HIPATTN_CUDA_OK(cudaGetDevice(&dev));
  HIPATTN_REQUIRE(dev >= 0 && dev < kMaxDevices, HIPATTN_ERR_UNSUPPORTED, "device index %d is beyond %d", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_scratch_dev_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    HIPATTN_CUDA_OK(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
    HIPATTN_REQUIRE(ptr != nullptr, HIPATTN_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    g_scratch_dev_ptr[dev] = static_cast<float*>(ptr);
  }
  *out = g_scratch_dev_ptr[dev];
  return HIPATTN_OK;
}

}  // namespace

extern "C" int hipattn_bsa_decode_noalloc(const hipattn_bsa_params_t* p, void* stream) {
  using namespace hipattn;
  HIPATTN_REQUIRE(p != nullptr, HIPATTN_ERR_INVALID, "decode_noalloc: params are null");
  HIPATTN_REQUIRE(p->TQ == 1, HIPATTN_ERR_INVALID, "decode_noalloc: one query row per sequence expected, got TQ = %d", p->TQ);
  HIPATTN_REQUIRE(p->out != nullptr, HIPATTN_ERR_INVALID, "decode_noalloc: out is null");
  HIPATTN_REQUIRE(p->n_splits >= 1 && p->n_splits <= 64, HIPATTN_ERR_INVALID, "decode_noalloc: n_splits %d outside [1, 64]", p->n_splits);
  HIPATTN_REQUIRE(p->B > 0 && p->H > 0 && p->D > 0, HIPATTN_ERR_INVALID, "decode_noalloc: bad shape");
  HIPATTN_REQUIRE(p->o_stride_h == p->D && p->o_stride_b == (int64_t)p->H * p->D, HIPATTN_ERR_INVALID,
                  "decode_noalloc: out must be a contiguous [B, 1, H, D] tensor");
  const size_t rows = (size_t)p->B * p->H;
  const size_t need = rows * p->n_splits * ((size_t)p->D + 1);
  HIPATTN_REQUIRE(need <= kScratchFloats, HIPATTN_ERR_UNSUPPORTED,
                  "decode_noalloc: B * H * n_splits * (D + 1) = %zu floats exceeds the built-in scratch of %zu floats "
                  "(%d bytes); use hipattn_bsa_attention with caller-provided buffers, or fewer splits",
                  need, kScratchFloats, (int)HIPATTN_NOALLOC_SCRATCH_BYTES);
  float* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;

  hipattn_bsa_params_t q = *p;
  if (p->n_splits == 1) {  // a single range needs no scratch at all
    q.part_o = nullptr;
    q.part_lse = nullptr;
    return hipattn_bsa_attention(&q, stream);
  }
  q.lse_out = nullptr;  // with splits the log-sum-exp comes out of the merge
  q.part_o = scratch;
  q.part_lse = scratch + rows * p->n_splits * (size_t)p->D;
  rc = hipattn_bsa_attention(&q, stream);
  if (rc) return rc;
  return hipattn_merge_partials(q.part_o, q.part_lse, (int64_t)rows, p->n_splits, p->D, p->dtype, p->out, p->D, p->lse_out,
                                stream);
}
