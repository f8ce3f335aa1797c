// Tensor-core building blocks of the bfloat16 attention kernels: asynchronous 16-byte copies
// into shared memory, 8x8 matrix loads from it, and the m16n8k16 bf16 multiply-accumulate.
//
// Fragment layouts (lane = 4 * gid + tid4):
//   A 16x16 row-major : a0 (row gid,   k 2*tid4..+1)  a1 (row gid+8, k 2*tid4..+1)
//                       a2 (row gid,   k 2*tid4+8..)  a3 (row gid+8, k 2*tid4+8..)
//   B 16x8            : b0 (k 2*tid4..+1, n gid)      b1 (k 2*tid4+8..+9, n gid)
//   C 16x8 float      : c0,c1 (row gid, n 2*tid4..+1) c2,c3 (row gid+8, n 2*tid4..+1)
// Tiles of keys and values sit in shared memory as [row][D + 8] bf16: the 16 bytes of padding
// per row shift consecutive rows by four banks, so the eight row reads of an 8x8 matrix load
// never collide, for every D that is a multiple of 16.
#pragma once

#include "common.cuh"

namespace q3 {

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// 16 bytes global -> shared; src_bytes = 0 writes zeros and reads nothing.
__device__ __forceinline__ void cp_async_16(void* dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(dst)), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* row_ptr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr(row_ptr)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* row_ptr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr(row_ptr)));
}

// c += a (16x16 bf16) * b (16x8 bf16), float accumulation
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// log2 of a page size that is a power of two, else -1 (the kernels then divide).
static inline int page_shift_of(int page_size) {
  if (page_size <= 0 || (page_size & (page_size - 1))) return -1;
  int s = 0;
  while ((1 << s) < page_size) ++s;
  return s;
}

}  // namespace q3
