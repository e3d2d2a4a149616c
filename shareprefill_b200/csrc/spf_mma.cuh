// Warp-level tensor-core and async-copy helpers shared by the generic kernels
// (mma.sync m16n8k16 bf16, ldmatrix, cp.async).  The tcgen05/TMEM attention kernel has its
// own helpers; these serve the small contractions (last-block profile, pooled block scores)
// and the generic block-sparse attention for block sizes / head dims the tcgen05 kernel
// does not cover.
#pragma once

#include "spf_common.cuh"

namespace spf {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte async copy global -> shared; `valid` false zero-fills the destination.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// D(16x8, fp32) += A(16x16, bf16 row-major) * B(16x8, bf16 col-major)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);  // .x = lo (low 16 bits), .y = hi
  return *reinterpret_cast<uint32_t*>(&v);
}

// A [ROWS][D] bf16 tile in shared memory, rows of D*2 bytes, 16-byte chunks XOR-swizzled by
// (row & 7) so that ldmatrix (8 rows x 16 bytes) and row-wise cp.async are conflict free.
template <int D>
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  constexpr int CHUNKS = D / 8;  // 16-byte chunks per row
  return static_cast<uint32_t>(row * (D * 2) + (((chunk ^ (row & 7)) & (CHUNKS - 1)) << 4));
}

// Cooperative load of `rows_valid` rows (of ROWS) of a strided global tile into a swizzled
// shared tile; rows beyond rows_valid are zero filled.  NT threads participate.
template <int ROWS, int D, int NT>
__device__ __forceinline__ void load_tile_async(uint32_t smem_base, const __nv_bfloat16* g,
                                                int64_t stride_row, int rows_valid, int tid) {
  constexpr int CHUNKS = D / 8;
  constexpr int TOTAL = ROWS * CHUNKS;
#pragma unroll
  for (int i = tid; i < TOTAL; i += NT) {
    const int row = i / CHUNKS, ch = i % CHUNKS;
    const bool ok = row < rows_valid;
    const __nv_bfloat16* src = g + (ok ? (int64_t(row) * stride_row + ch * 8) : 0);
    cp_async16(smem_base + tile_off<D>(row, ch), src, ok);
  }
}

}  // namespace spf
