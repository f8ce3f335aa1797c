// Shared device helpers for the sm_100a kernels of this engine.
//
// Every launcher in this directory is an `extern "C"` function that takes raw
// device pointers, sizes and a stream, launches on that stream and returns the
// CUDA error code of the launch (0 = ok) or one of the Q3_ERR_* codes below for
// a size it refuses.  Nothing here allocates.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <atomic>

// dtype tags of the C ABI
#define Q3_F32 0
#define Q3_BF16 1

// refusals (negative so they never collide with cudaError_t)
#define Q3_ERR_DTYPE -1      // unknown dtype tag
#define Q3_ERR_SIZE -2       // a size this kernel does not take (see the launcher's comment)
#define Q3_ERR_ALIGN -3      // pointer or row pitch not aligned as the kernel needs
#define Q3_ERR_SCRATCH -4    // the call needs more scratch memory than the fixed array holds
#define Q3_ERR_DRIVER -5     // the CUDA driver refused a tensor-map request (or lacks the entry point)

// bits of the device status word that kernels OR into `status` instead of
// faulting when table data is bad; the host reads it after the step.
#define Q3_STATUS_BAD_TOKEN 1   // token id outside the embedding table
#define Q3_STATUS_BAD_PAGE 2    // page id outside the pool where a live position needs one
#define Q3_STATUS_BAD_POSITION 4  // negative position or sequence index, or a position beyond the block table's row
#define Q3_STATUS_BAD_LOGITS 8    // a row of logits with no comparable value (all NaN)
#define Q3_STATUS_TIMEOUT 16      // a bounded wait on an mbarrier ran out; the block gave up cleanly

namespace q3 {

// Entry `idx` of a request's block-table row of `table_stride` entries.  An index at or beyond the end of
// the row (a length or position that the table was not made for) is never read: the status word gets
// BAD_POSITION and the answer is "no page" (-1), which every caller treats like a hole in the table.
__device__ __forceinline__ int table_page(const int* table, int idx, int table_stride, int* status) {
  if (idx < 0 || idx >= table_stride) {
    atomicOr(status, Q3_STATUS_BAD_POSITION);
    return -1;
  }
  return table[idx];
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a whole block (blockDim.x a multiple of 32, at most 1024).  The order of
// the additions depends only on blockDim.x, so a row's result does not depend on
// which other rows are in the launch.  `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  float t = (lane < nwarps) ? scratch[lane] : 0.f;
  return warp_sum(t);
}

static inline int launch_status() { return (int)cudaGetLastError(); }

// Streaming multiprocessors of the current device (asked once per device; grids, split counts and the
// choice between kernel variants are sized by it, never by a constant).
static inline int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
  if (cached[dev] <= 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
    cached[dev] = n;
  }
  return cached[dev];
}

// ---------------------------------------------------------------- programmatic dependent launch
// Every kernel of this library starts with pdl_wait() and then pdl_launch_dependents().  Launched
// with the programmatic-serialization attribute (launch() below), a kernel's blocks may become
// resident while the kernel before it in the stream is still running; they stop at pdl_wait()
// until that kernel has completed and its memory is visible.  Only data that no kernel writes
// (weights, the step's integer arrays) may be touched before the wait.  Because every kernel
// waits for its predecessor before it can finish, completion stays ordered along the whole chain;
// because it releases its own dependents only after its wait, at most one kernel ahead of the
// running one holds resources on the SMs.
// Launched the ordinary way both calls do nothing.  Q3B200_PDL=0 in the environment turns the
// attribute off.
//
// What a kernel may read ahead of its wait.  Kernel N+1 starts once every block of kernel N has let
// its dependents go, which each does only after its own wait, that is after kernel N-1 has completed.
// So whatever kernel N-1 or an earlier one wrote is complete and visible to kernel N+1 from its first
// instruction; only what kernel N itself writes needs the wait.  (A kernel launched the ordinary way,
// a library's for instance, starts after the one before it has completed and lets the next one start
// when it has completed itself, so the rule holds across it.)  The residual stream is such data for a
// norm kernel unless the launch directly before it wrote the stream; last_launch_was_plain() tells.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

static inline bool pdl_enabled() {
  static int enabled = -1;
  if (enabled < 0) {
    const char* e = getenv("Q3B200_PDL");
    enabled = (e && e[0] == '0') ? 0 : 1;
  }
  return enabled == 1;
}

// The stream of this library's most recent launch if that launch wrote nothing that a later kernel
// reads ahead of its wait (a residual stream, the step's table of angles), else (or before any
// launch) all ones.  One word, so that a reader never sees half of an update.
extern std::atomic<uintptr_t> g_plain_launch_stream;
constexpr uintptr_t NO_PLAIN_LAUNCH = ~(uintptr_t)0;

// True if the most recent launch of this library went to `stream` and wrote no such data.
static inline bool last_launch_was_plain(cudaStream_t stream) {
  return g_plain_launch_stream.load(std::memory_order_relaxed) == (uintptr_t)stream;
}
// To be called right after launching a kernel that writes such data.
static inline void note_stream_written() { g_plain_launch_stream.store(NO_PLAIN_LAUNCH, std::memory_order_relaxed); }

// A launch made while this is false is an ordinary one: the kernel starts when the one before it in the stream
// has completed (set around a launch by a launcher that wants that: the merge of the decode attention's splits,
// attn_decode.cu).
extern thread_local bool g_launch_early;

template <typename... KArgs, typename... Args>
static inline int launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                         Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl_enabled() && g_launch_early) ? 1 : 0;
  g_plain_launch_stream.store((uintptr_t)stream, std::memory_order_relaxed);
  return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace q3
