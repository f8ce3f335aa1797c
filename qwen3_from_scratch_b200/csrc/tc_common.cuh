// Building blocks shared by the tcgen05 kernels: mbarriers with bounded waits, TMA tile loads,
// shared-memory matrix descriptors, tcgen05.mma / commit / ld / st, and tensor-map encoding.
//
// Layout facts the kernels rely on.  A tile of bfloat16 with rows of 64 values (128 bytes) and the
// 128-byte swizzle puts value (r, c) at byte  r * 128 + (((c / 8) ^ (r % 8)) * 16) + (c % 8) * 2
// from a 1024-byte aligned base; this is what TMA writes for a {64, rows} box and what the tensor
// cores read through a descriptor, either "K-major" (the 64 values are the reduction dimension:
// stride between groups of eight rows = 1024 bytes) or "MN-major" (the 64 values are the M or N
// dimension and the rows are the reduction dimension: groups of eight rows 1024 bytes apart, the
// next 64 values of M/N at the leading byte offset).
#pragma once

#include <cuda.h>
#include <cudaTypedefs.h>

#include "common.cuh"

namespace q3 {

constexpr int TC_BK = 64;  // one 128-byte swizzle atom of bfloat16
constexpr uint32_t TC_WAIT_LIMIT = 1u << 24;

// How many polls a wait on an mbarrier makes before it gives up, and a hook for the tests of that path:
// the loader of a kernel leaves out its copy number `tc_drop_copy` (and the barrier's expectation of it),
// so that the barrier never completes and every role of the block has to give up, flag the status word,
// free what it holds and return.  Each file that includes this header has its own copy of the two words
// and exports a setter for them (q3_*_wait_test); the defaults are what serving uses.
static __constant__ uint32_t tc_wait_limit = TC_WAIT_LIMIT;
static __constant__ int tc_drop_copy = -1;

__device__ __forceinline__ uint32_t s_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(s_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// The same question without any waiting: answers at once (about 160 clocks against 220 for try_wait).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(s_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false if the phase did not complete in time or another role gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_test_wait(bar, parity)) return true;  // most waits of these kernels find their phase complete
  const uint32_t limit = tc_wait_limit;
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  return false;
}

// Brings a tensor map into the descriptor cache ahead of its first use by a copy.
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(s_addr(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(s_addr(bar)), "r"(x), "r"(y)
      : "memory");
}

// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes with the 128-byte
// swizzle (what TMA wrote): start address, stride between groups of eight rows = 1024 bytes.
__device__ __forceinline__ uint64_t umma_desc_sw128(const void* tile) {
  uint64_t d = 0;
  d |= (uint64_t)((s_addr(tile) & 0x3FFFF) >> 4);   // start address, bits [0, 14)
  d |= (uint64_t)1 << 16;                           // leading byte offset (unused with this swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;                 // stride byte offset, bits [32, 46)
  d |= (uint64_t)1 << 46;                           // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                           // layout: 128-byte swizzle
  return d;
}

// Instruction descriptor: bf16 x bf16 -> f32, M = 128, N = n; A K-major; B K-major or (b_mn) MN-major.
__host__ __device__ constexpr uint32_t umma_idesc(int n, int b_mn = 0) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(128 >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same with the A operand in tensor memory: row i of the 128 x 16 tile in lane i, its 16 values
// of k in 8 consecutive 32-bit columns from `tmem_a` (value 2 c in the low half of column c).
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s_addr(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld_32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ uint32_t pack2(uint32_t lo_bits, uint32_t hi_bits) {
  __nv_bfloat162 p = __floats2bfloat162_rn(__uint_as_float(lo_bits), __uint_as_float(hi_bits));
  return *reinterpret_cast<uint32_t*>(&p);
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }


__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s_addr(bar)) : "memory");
}
// Writes made with ordinary stores become visible to the tensor cores and TMA (the async proxy).
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// MN-major operand with the 128-byte swizzle: rows are the reduction dimension (groups of eight
// rows 1024 bytes apart), the next 64 values of the M/N dimension start `lbo_bytes` further.
__device__ __forceinline__ uint64_t umma_desc_sw128_mn(const void* tile, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((s_addr(tile) & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__device__ __forceinline__ void tmem_st_32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// 2^x by the special-function unit (what exp2f uses, without its rescue of results below 2^-126,
// which flush to zero here: as probabilities they are zero in bfloat16 anyway).
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// ---------------------------------------------------------------- a pair of CTAs (cta_group::2)
// Two CTAs of a cluster of two work on one tile: each brings its own half of both operands into its own
// shared memory, the thread that issues for the pair sits in the CTA of rank 0, and every stage's barrier
// that this thread waits on is the one in rank 0's shared memory.  Barriers and tiles lie at the same
// offsets in both CTAs.
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The address, in the cluster's shared window, of `local` (an address in this CTA) in the CTA of `rank`.
__device__ __forceinline__ uint32_t cluster_addr(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
// Every thread of both CTAs.  Only used where nothing can keep a thread from getting there (before the
// first copy, after the last wait has been left one way or the other).
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_address, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_address), "r"(v) : "memory");
}
// A wait on a barrier that threads of the other CTA arrive on.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  const uint32_t limit = tc_wait_limit;
  for (uint32_t i = 0; i < limit; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(s_addr(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  return false;
}
// A tile into this CTA's shared memory whose arrival is counted by a barrier given by its address in the
// cluster's window (the pair's barrier in rank 0).  No multicast: each CTA fetches what it needs itself.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t cluster_bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(s_addr(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y)
      : "memory");
}
// Instruction descriptor of the pair's instruction: M = 256 (128 rows in each CTA), N = n (n / 2 rows of B in each).
__host__ __device__ constexpr uint32_t umma_idesc_pair(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrival on the barrier at this offset in both CTAs of the pair once the pair's instructions issued so
// far have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(s_addr(bar)), "h"((uint16_t)3)
               : "memory");
}

__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------- host side: the wait limit of this file's kernels
// `limit` polls per wait (0: the default) and the ordinal of the loader's copy that is left out (-1: none).
// The words are set for the current device, before the next launch (a blocking copy).
static int set_wait_test(unsigned limit, int drop) {
  const uint32_t polls = limit ? limit : TC_WAIT_LIMIT;
  cudaError_t e = cudaMemcpyToSymbol(tc_wait_limit, &polls, sizeof(polls));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(tc_drop_copy, &drop, sizeof(drop));
  return (int)e;
}

// ---------------------------------------------------------------- host side: tensor maps
static PFN_cuTensorMapEncodeTiled tensor_map_encoder() {
  static PFN_cuTensorMapEncodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(p);
  }
  return fn;
}

// A [rows, cols] bfloat16 row-major matrix as boxes of 64 columns x box_rows rows, 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  PFN_cuTensorMapEncodeTiled enc = tensor_map_encoder();
  if (!enc) return Q3_ERR_DRIVER;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)TC_BK, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : Q3_ERR_DRIVER;
}

// Encoding a tensor map costs microseconds on the host; weights and the engine's reused activation
// buffers come back with the same (address, shape), so the few maps a model needs are kept.
struct MapKey {
  const void* ptr;
  uint64_t rows, cols;
  uint32_t box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows;
  }
};
static int cached_map(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  constexpr int SLOTS = 1024;
  static MapKey keys[SLOTS];
  static CUtensorMap maps[SLOTS];
  static bool used[SLOTS] = {false};
  const MapKey key{ptr, rows, cols, box_rows};
  uint64_t h = (uint64_t)(uintptr_t)ptr * 0x9E3779B97F4A7C15ull ^ (rows * 0xBF58476D1CE4E5B9ull) ^ (cols << 7) ^ box_rows;
  const int slot = (int)((h >> 32) % SLOTS);
  if (used[slot] && keys[slot] == key) {
    *map = maps[slot];
    return 0;
  }
  const int code = make_map(map, ptr, rows, cols, box_rows);
  if (code == 0) {
    keys[slot] = key;
    maps[slot] = *map;
    used[slot] = true;
  }
  return code;
}

}  // namespace q3
