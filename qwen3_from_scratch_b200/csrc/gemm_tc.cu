// Matrix product on the fifth-generation tensor cores: C[M, N] = A[M, K] * W[N, K]^T, bfloat16 in,
// float32 accumulate in tensor memory (TMEM), for the projections of prompt portions.
//
// A persistent kernel, one block per SM, that walks over 128 x BN output tiles.  Three roles:
//   warp 0 (one thread)  brings operand tiles of 64 values of k into shared memory by TMA
//                        (cp.async.bulk.tensor, 128-byte swizzle, no multicast) under a ring of mbarriers;
//   warp 1 (one thread)  issues tcgen05.mma (cta_group::1, kind::f16) straight from shared memory through
//                        matrix descriptors, four instructions of k = 16 per stage; tcgen05.commit hands
//                        each stage back to the loader and each finished accumulator to the epilogue;
//   warps 2..5           read the accumulator with tcgen05.ld (each thread owns one row of the tile) and
//                        store bfloat16 or float32, optionally applying SwiGLU to a weight whose rows
//                        alternate gate/up in blocks of eight.
// There are two accumulators in TMEM, so the epilogue of one tile runs under the main loop of the next.
//
// Every wait on an mbarrier is bounded: a wait that runs out sets the TIMEOUT bit of the status
// word and a block-wide abort flag, every role leaves its loop, TMEM is released and the block
// returns; nothing spins forever.
//
// Role in the reference: nn.Linear / cuBLAS (models/self_attn.py:358-386, models/feedback.py:28-34).
#include "tc_common.cuh"

namespace q3 {

constexpr int TC_BM = 128;
constexpr int TC_THREADS = 192;

template <int BN>
struct TcShape {
  static constexpr int A_BYTES = TC_BM * TC_BK * 2;
  static constexpr int B_BYTES = BN * TC_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (192 * 1024) / STAGE_BYTES;  // 4 stages of 48 KB or 6 of 32 KB
  static constexpr int BAR_BYTES = 256;  // 2 * STAGES + 4 barriers and the TMEM address
  static constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + BAR_BYTES + 1024;  // + room to align to 1024
  static constexpr uint32_t TMEM_COLS = 2 * BN;  // two accumulators
};

// Stores 32 consecutive columns of one row.  EPI 0: as they are.  EPI 1: SwiGLU on column blocks
// (gate 8, up 8, ...), 16 outputs at half the column index.
template <int EPI, typename OutT>
__device__ __forceinline__ void tc_store_chunk(const uint32_t (&v)[32], OutT* __restrict__ C, int row, int col0, int N,
                                               int ldc) {
  if (EPI == 0) {
    OutT* dst = C + (size_t)row * ldc + col0;
    if (col0 + 32 <= N && ((uintptr_t)dst & 15) == 0) {
      // the thread's 32 values are contiguous in its row: 16-byte stores
      if (sizeof(OutT) == 2) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 pk;
          pk.x = pack2(v[8 * j + 0], v[8 * j + 1]);
          pk.y = pack2(v[8 * j + 2], v[8 * j + 3]);
          pk.z = pack2(v[8 * j + 4], v[8 * j + 5]);
          pk.w = pack2(v[8 * j + 6], v[8 * j + 7]);
          reinterpret_cast<uint4*>(dst)[j] = pk;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          reinterpret_cast<uint4*>(dst)[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < N) dst[j] = from_float<OutT>(__uint_as_float(v[j]));
    }
  } else {
    // columns 16 j .. 16 j + 7 gate, 16 j + 8 .. 16 j + 15 up -> 8 outputs at col0 / 2 + 8 j
    OutT* dst = C + (size_t)row * ldc + (col0 >> 1);
    float r[16];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float gate = __uint_as_float(v[16 * j + i]), up = __uint_as_float(v[16 * j + 8 + i]);
        // silu by the fast exponential and division: their error (about 2^-21) is far below the
        // bfloat16 rounding of the result, and the exact forms made this epilogue longer than the main loop
        r[8 * j + i] = up * __fdividef(gate, 1.0f + __expf(-gate));
      }
    if (col0 + 32 <= N && ((uintptr_t)dst & 15) == 0 && sizeof(OutT) == 2) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        uint4 pk;
        pk.x = pack2(__float_as_uint(r[8 * j + 0]), __float_as_uint(r[8 * j + 1]));
        pk.y = pack2(__float_as_uint(r[8 * j + 2]), __float_as_uint(r[8 * j + 3]));
        pk.z = pack2(__float_as_uint(r[8 * j + 4]), __float_as_uint(r[8 * j + 5]));
        pk.w = pack2(__float_as_uint(r[8 * j + 6]), __float_as_uint(r[8 * j + 7]));
        reinterpret_cast<uint4*>(dst)[j] = pk;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (col0 + 16 * j + 8 + i < N) dst[8 * j + i] = from_float<OutT>(r[8 * j + i]);
    }
  }
}

template <int BN, int EPI, typename OutT>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               OutT* __restrict__ C, int M, int N, int K, int ldc, int* status) {
  using S = TcShape<BN>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* tiles = base;
  uint64_t* full = reinterpret_cast<uint64_t*>(base + (size_t)S::STAGES * S::STAGE_BYTES);
  uint64_t* empty = full + S::STAGES;
  uint64_t* acc_full = empty + S::STAGES;  // [2]
  uint64_t* acc_empty = acc_full + 2;      // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_tiles = (K + TC_BK - 1) / TC_BK;
  const int m_tiles = (M + TC_BM - 1) / TC_BM, n_tiles = (N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);  // one arrival from each epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_wait();  // the activations come from the kernel before this one
  pdl_launch_dependents();
  // Tensor memory is taken only after the wait: a block that holds TMEM while it waits for the
  // kernel before it could keep that kernel's own blocks from ever getting theirs.
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_addr(tmem_holder)),
                 "r"(S::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (lane == 0) {
      // ---- loader
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % m_tiles) * TC_BM, n0 = (tile / m_tiles) * BN;
        for (int kt = 0; kt < k_tiles; ++kt, ++it) {
          const int s = it % S::STAGES;
          const uint32_t use = it / S::STAGES;
          if (use > 0 && !mbar_wait(&empty[s], (use & 1) ^ 1, &abort_flag)) {
            abort_flag = 1;
            atomicOr(status, Q3_STATUS_TIMEOUT);
            ok = false;
            break;
          }
          unsigned char* a_s = tiles + (size_t)s * S::STAGE_BYTES;
          mbar_expect_tx(&full[s], S::STAGE_BYTES);
          tma_load_2d(a_s, &map_a, &full[s], kt * TC_BK, m0);
          tma_load_2d(a_s + S::A_BYTES, &map_b, &full[s], kt * TC_BK, n0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- tensor-core issue
      constexpr uint32_t idesc = umma_idesc(BN);
      uint32_t it = 0, t = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++t) {
        const uint32_t buf = t & 1;
        if (t >= 2 && !mbar_wait(&acc_empty[buf], ((t >> 1) & 1) ^ 1, &abort_flag)) {
          ok = false;
          break;
        }
        tcgen05_fence_after();
        const uint32_t tmem_acc = tmem_base + buf * BN;
        for (int kt = 0; kt < k_tiles; ++kt, ++it) {
          const int s = it % S::STAGES;
          const uint32_t use = it / S::STAGES;
          if (!mbar_wait(&full[s], use & 1, &abort_flag)) {
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const unsigned char* a_s = tiles + (size_t)s * S::STAGE_BYTES;
          const uint64_t a_desc = umma_desc_sw128(a_s), b_desc = umma_desc_sw128(a_s + S::A_BYTES);
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k)  // 16 values of k = 32 bytes further along the swizzled row
            umma_f16(tmem_acc, a_desc + 2 * k, b_desc + 2 * k, idesc, (kt | k) != 0);
          umma_commit(&empty[s]);  // the stage is free once these instructions have read it
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
      if (!ok) {
        abort_flag = 1;
        atomicOr(status, Q3_STATUS_TIMEOUT);
      }
    }
  } else {
    // ---- epilogue: a warp may read the 32 TMEM lanes of its quarter (warp index modulo 4)
    const int quarter = warp & 3;
    uint32_t t = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++t) {
      const int m0 = (tile % m_tiles) * TC_BM, n0 = (tile / m_tiles) * BN;
      const uint32_t buf = t & 1;
      const bool ready = mbar_wait(&acc_full[buf], (t >> 1) & 1, &abort_flag);
      if (!__all_sync(0xffffffffu, ready)) {
        if (lane == 0) {
          abort_flag = 1;
          atomicOr(status, Q3_STATUS_TIMEOUT);
        }
        ok = false;
        break;
      }
      tcgen05_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t tmem_acc = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        if (n0 + c0 >= N) break;  // uniform over the warp
        uint32_t v[32];
        tmem_ld_32(tmem_acc + (uint32_t)c0, v);
        tmem_wait_ld();
        if (row < M) tc_store_chunk<EPI, OutT>(v, C, row, n0 + c0, N, ldc);
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(S::TMEM_COLS) : "memory");
  }
}

static int tc_sm_count() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      sms = 0;
    if (sms <= 0) sms = 148;
  }
  return sms;
}

template <int BN, int EPI, typename OutT>
static int gemm_tc_launch(const void* A, const void* W, void* C, int M, int N, int K, int ldc, int* status,
                          cudaStream_t stream) {
  using S = TcShape<BN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, EPI, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)S::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  CUtensorMap map_a, map_b;
  int code = cached_map(&map_a, A, (uint64_t)M, (uint64_t)K, TC_BM);
  if (code) return code;
  code = cached_map(&map_b, W, (uint64_t)N, (uint64_t)K, BN);
  if (code) return code;
  const long long tiles = (long long)((N + BN - 1) / BN) * ((M + TC_BM - 1) / TC_BM);
  if (tiles > 0x7fffffffLL) return Q3_ERR_SIZE;
  const int grid = (int)(tiles < tc_sm_count() ? tiles : tc_sm_count());
  q3::launch(gemm_tc_kernel<BN, EPI, OutT>, dim3(grid), dim3(TC_THREADS), S::SMEM_BYTES, stream, map_a, map_b,
             (OutT*)C, M, N, K, ldc, status);
  return launch_status();
}

// The tile width that needs fewer rounds of the SMs: rounds x width is the cost of the slowest block.
static int tc_pick_bn(int M, int N) {
  const long long sms = tc_sm_count();
  const long long m_tiles = (M + TC_BM - 1) / TC_BM;
  const long long t256 = m_tiles * ((N + 255) / 256), t128 = m_tiles * ((N + 127) / 128);
  const long long c256 = ((t256 + sms - 1) / sms) * 256, c128 = ((t128 + sms - 1) / sms) * 128;
  return c256 <= c128 ? 256 : 128;
}

template <int EPI, typename OutT>
static int gemm_tc_dispatch(const void* A, const void* W, void* C, int M, int N, int K, int ldc, int* status,
                            cudaStream_t stream) {
  if (tc_pick_bn(M, N) == 256) return gemm_tc_launch<256, EPI, OutT>(A, W, C, M, N, K, ldc, status, stream);
  return gemm_tc_launch<128, EPI, OutT>(A, W, C, M, N, K, ldc, status, stream);
}

}  // namespace q3

// C[M, N] (row pitch ldc) = A[M, K] * W[N, K]^T; A, W bfloat16 with 16-byte aligned bases and K a multiple
// of 8 (TMA wants row pitches in multiples of 16 bytes).  out_f32: float32 output, else bfloat16.
// swiglu: W's rows alternate gate/up in blocks of eight, N a multiple of 16, C is [M, N / 2] bfloat16.
extern "C" int q3_gemm_tc(const void* A, const void* W, void* C, int M, int N, int K, int ldc, int out_f32,
                          int swiglu, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || (swiglu && (N % 16 || out_f32))) return Q3_ERR_SIZE;
  if ((uintptr_t)A % 16 || (uintptr_t)W % 16) return Q3_ERR_ALIGN;
  using bf16 = __nv_bfloat16;
  if (swiglu) return q3::gemm_tc_dispatch<1, bf16>(A, W, C, M, N, K, ldc, status, stream);
  if (out_f32) return q3::gemm_tc_dispatch<0, float>(A, W, C, M, N, K, ldc, status, stream);
  return q3::gemm_tc_dispatch<0, bf16>(A, W, C, M, N, K, ldc, status, stream);
}
