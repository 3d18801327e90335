// Warp-level tensor-core helpers (mma.sync m16n8k16, ldmatrix) shared by the attention and scan kernels.
#pragma once
#include "common.cuh"
#include "rope.cuh"

namespace hipattn {

template <int DT>
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  if (DT == HIPATTN_BF16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}
__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}

// byte address of 16-byte piece `piece` of row `row` in an XOR-swizzled [rows][D] tile of 2-byte elements
template <int D>
__device__ __forceinline__ int swz(int row, int piece) {
  return row * (D * 2) + ((piece ^ (row & 7)) << 4);
}


// In-kernel RoPE on a swizzled [rows][D] tile of 16-bit elements in shared memory: rows row0 .. row0 + rows - 1 are
// rotated to table position pos(r) (rows with a negative position are left alone).  The work is dealt to `nthreads`
// threads numbered `tid`; the caller synchronises them around the call.
template <int DT, int D, typename PosFn>
__device__ __forceinline__ void rope_rotate_tile(unsigned char* tile, int row0, int rows, const hipattn_bsa_params_t& p, int tid,
                                                 int nthreads, PosFn pos) {
  constexpr int HALF = D / 16;   // 16-byte pieces per half row
  for (int i = tid; i < rows * HALF; i += nthreads) {
    const int r = row0 + i / HALF, pc = i % HALF;
    const int t = pos(r);
    if (t < 0) continue;
    uint4* plo = reinterpret_cast<uint4*>(tile + swz<D>(r, pc));
    uint4* phi = reinterpret_cast<uint4*>(tile + swz<D>(r, pc + HALF));
    uint4 lo = *plo, hi = *phi;
    rope_rotate_packed<DT>(lo, hi, rope_table_raw(p.rope_cos, p.rope_stride, p.rope_rows, t, pc),
                           rope_table_raw(p.rope_sin, p.rope_stride, p.rope_rows, t, pc));
    *plo = lo;
    *phi = hi;
  }
}

}  // namespace hipattn
