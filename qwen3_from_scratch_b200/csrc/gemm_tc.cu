// Matrix product on the fifth-generation tensor cores: C[M, N] = A[M, K] * W[N, K]^T, bfloat16 in,
// float32 accumulate in tensor memory (TMEM), for the projections of prompt portions.
//
// A persistent kernel, one block per SM, that walks over 128 x BN output tiles.  Three roles:
//   warp 0 (one thread)  brings operand tiles of 64 values of k into shared memory by TMA
//                        (cp.async.bulk.tensor, 128-byte swizzle, no multicast) under a ring of mbarriers; the
//                        W tiles of the ring's first round go out before the wait on the kernel before;
//   warp 1 (one thread)  issues tcgen05.mma (cta_group::1, kind::f16) straight from shared memory through
//                        matrix descriptors, four instructions of k = 16 per stage; tcgen05.commit hands
//                        each stage back to the loader and each finished accumulator to the epilogue;
//   warps 2..5 (2..9 for the SwiGLU and QKV epilogues)  read the accumulator with tcgen05.ld (each thread owns one row of the tile) and
//                        store bfloat16 or float32, optionally applying SwiGLU to a weight whose rows
//                        alternate gate/up in blocks of eight.
// There are two accumulators in TMEM, so the epilogue of one tile runs under the main loop of the next.
//
// A third epilogue serves the merged QKV projection of an attention layer: the tile's columns are
// whole heads, and instead of storing them the epilogue rounds them to bfloat16 (what a stored
// projection would hold), applies the per-head RMSNorm and the rotation to q and k heads and writes q
// to its buffer and k, v straight into their cache pages - the work of qkv_post.cu, without the
// projection ever going to memory (reference: models/self_attn.py:319-336).
//
// Every wait on an mbarrier is bounded: a wait that runs out sets the TIMEOUT bit of the status
// word and a block-wide abort flag, every role leaves its loop, TMEM is released and the block
// returns; nothing spins forever.
//
// A second kernel further down does the same product by pairs of CTAs (clusters of two, 256 x 256 tiles,
// tcgen05.mma.cta_group::2) with the same three epilogues; it runs at the library's rate where the
// single-CTA tile is held back by what one SM can fetch and read from shared memory per clock.
//
// Role in the reference: nn.Linear / cuBLAS (models/self_attn.py:358-386, models/feedback.py:28-34).
#include "tc_common.cuh"

namespace q3 {

constexpr int TC_BM = 128;

// The QKV epilogue has eight warps, two for each quarter of the accumulator's rows; each turns one head
// (up to 128 wide) of its 32 rows around in shared memory at a time.
constexpr int TC_QKV_EPI_WARPS = 8;
constexpr int TC_QKV_ROW_PAD = 16;  // a row's 1 / rms and cache offset; also keeps rows off each other's banks
constexpr int TC_HEAD_STAGE_BYTES = TC_QKV_EPI_WARPS * 32 * (128 * 2 + TC_QKV_ROW_PAD);

template <int EPI>
struct TcThreads {
  // the SwiGLU epilogue too has two warps per quarter of the rows (they take every second piece of 32 columns): with
  // one warp per scheduler a tile's epilogue is a single chain of latencies, which the last tile of a block shows
  static constexpr int EPI_WARPS = EPI == 2 ? TC_QKV_EPI_WARPS : (EPI == 1 ? 8 : 4);
  static constexpr int THREADS = 64 + 32 * EPI_WARPS;
};

template <int BN, int EPI = 0>
struct TcShape {
  static constexpr int A_BYTES = TC_BM * TC_BK * 2;
  static constexpr int B_BYTES = BN * TC_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_BYTES = 256;  // 2 * STAGES + 4 barriers and the TMEM address
  static constexpr int EPI_BYTES = EPI == 2 ? TC_HEAD_STAGE_BYTES : 0;  // where the QKV epilogue turns heads around
  // 4 stages of 48 KB or 6 of 32 KB; beside the QKV epilogue's 68 KB, three of 48 KB or four of 32 KB
  static constexpr int STAGES = ((EPI == 2 ? 156 : 192) * 1024) / STAGE_BYTES;
  static constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + BAR_BYTES + EPI_BYTES;
  static constexpr uint32_t TMEM_COLS = 2 * BN;  // two accumulators
};

// What the QKV epilogue needs beside the product (see q3_qkv_post for the meaning of each).
struct QkvEpilogue {
  __nv_bfloat16* q_out;
  __nv_bfloat16* k_pages;
  __nv_bfloat16* v_pages;
  const float* q_weight;
  const float* k_weight;
  const float* cos_sin;  // [M, D] cosines then sines of each row's position, or null: no rotation
  const int* positions;
  const int* tok_seq;
  const int* block_table;
  int table_stride, page_size, num_pages, Hq, Hkv;
  float eps;
  int write_kv;
};

// One head of the warp's 32 rows, in two passes.
// Pass 1, a thread per row (as tcgen05.ld hands the accumulator out): the head's D values are rounded to
// bfloat16, as a stored projection would be, and put into the row's place in shared memory; the thread sums
// the squares of its rounded row on the way and leaves 1 / rms and the row's cache offset behind the row.
// Pass 2, D / 8 neighbouring lanes per row.  A lane owns four values of the head's first half and the four
// values of the second half that they are rotated with, so that norm and rotation need no other lane; it
// reads them, the row's 1 / rms and its own cosines and sines (the lanes of a row read 2 D contiguous bytes
// of each) and stores two 8-byte pieces to q_out or the cache page.  No shuffles and three shared-memory
// reads per row: under the main loop the tensor core and TMA take the shared-memory pipe nearly whole, and
// an epilogue that went through it twenty times per row (shuffles count) set the kernel's pace.
// Cosines and sines are asked for four rows at a time and one such batch ahead, the first before pass 1; pass 1
// asks for the next 32 columns of the row before it works on those it has, and sums the squares in four chains.
// KIND (0 q, 1 k, 2 v, -1: found from `head`) and FAST (32 rows, and for q and k both norm and rotation) fix at
// compile time what the general form asks at run time: with two epilogue warps per scheduler the passes are bound
// by their own instruction count and latencies, and the fixed form has about half the instructions.
// Rows are TC_QKV_ROW_PAD bytes apart beyond their 2 D, which keeps pass 1's 16-byte writes (a thread per
// row, the same column) off each other's banks.
// `kv_off`: element offset of this lane's row in a page array (without the head), or -1.
// `release`: the barrier that hands the accumulator back, arrived on once pass 1 has read it, as its address
// in the cluster's shared window (the block's own address where there is no cluster), or 0.
template <int D, int KIND, bool FAST>
__device__ __forceinline__ void qkv_head_rows(uint32_t tmem_head, unsigned char* mine, int row_base, int rows_here_,
                                              int head, const QkvEpilogue& e, int lane, long long kv_off,
                                              uint32_t release) {
  constexpr int LPH = D / 8, RPW = 32 / LPH, STRIDE = D * 2 + TC_QKV_ROW_PAD;
  constexpr int ITER = 32 / RPW, BATCH = ITER < 4 ? ITER : 4, NB = ITER / BATCH;
  const bool is_q = KIND >= 0 ? KIND == 0 : head < e.Hq, is_k = KIND >= 0 ? KIND == 1 : (!is_q && head < e.Hq + e.Hkv);
  const float* w = is_q ? e.q_weight : (is_k ? e.k_weight : nullptr);
  const bool has_w = FAST ? KIND < 2 : w != nullptr;
  const bool rotate = FAST ? KIND < 2 : ((is_q || is_k) && e.cos_sin != nullptr);
  const int rows_here = FAST ? 32 : rows_here_;
  const int sub = lane / LPH, l = lane % LPH;
  float4 cs[2][BATCH][2];  // [.][.][0]: cosines of the lane's four pairs, [1]: sines
  const float* cs_row = e.cos_sin + (size_t)(row_base + sub) * D + l * 4;
  auto fetch = [&](int b, float4 (&buf)[BATCH][2]) {
#pragma unroll
    for (int i = 0; i < BATCH; ++i) {
      const int r = (b * BATCH + i) * RPW + sub;
      if (FAST || r < rows_here) {
        const float* row = cs_row + (size_t)((b * BATCH + i) * RPW) * D;
        buf[i][0] = *reinterpret_cast<const float4*>(row);
        buf[i][1] = *reinterpret_cast<const float4*>(row + D / 2);
      }
    }
  };
  if (!FAST) {
#pragma unroll
    for (int i = 0; i < BATCH; ++i) {
      cs[0][i][0] = cs[1][i][0] = make_float4(1.f, 1.f, 1.f, 1.f);
      cs[0][i][1] = cs[1][i][1] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  if (rotate) fetch(0, cs[0]);  // uniform over the warp
  float4 w_lo = make_float4(1.f, 1.f, 1.f, 1.f), w_hi = w_lo;
  if (has_w) {
    w_lo = *reinterpret_cast<const float4*>(w + l * 4);
    w_hi = *reinterpret_cast<const float4*>(w + D / 2 + l * 4);
  }

  // pass 1: the next piece of the row is asked for before this one is worked on; four sums side by side
  float ss4[4] = {0.f, 0.f, 0.f, 0.f};
  uint32_t v[2][32];
  tmem_ld_32(tmem_head, v[0]);
#pragma unroll
  for (int c0 = 0; c0 < D; c0 += 32) {
    uint32_t(&cur)[32] = v[(c0 / 32) & 1];
    tmem_wait_ld();
    if (c0 + 32 < D) tmem_ld_32(tmem_head + (uint32_t)(c0 + 32), v[((c0 / 32) & 1) ^ 1]);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t pk[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        pk[i] = pack2(cur[8 * c + 2 * i], cur[8 * c + 2 * i + 1]);
        const float lo = __uint_as_float(pk[i] << 16), hi = __uint_as_float(pk[i] & 0xffff0000u);
        ss4[i] = fmaf(lo, lo, ss4[i]);
        ss4[i] = fmaf(hi, hi, ss4[i]);
      }
      *reinterpret_cast<uint4*>(mine + lane * STRIDE + (c0 / 8 + c) * 16) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
  }
  {
    const float ss = (ss4[0] + ss4[1]) + (ss4[2] + ss4[3]);
    const float rs = has_w ? 1.0f / sqrtf(ss / (float)D + e.eps) : 1.0f;
    *reinterpret_cast<uint4*>(mine + lane * STRIDE + D * 2) =
        make_uint4(__float_as_uint(rs), (uint32_t)(unsigned long long)kv_off, (uint32_t)((unsigned long long)kv_off >> 32), 0u);
  }
  if (release) {  // uniform over the warp
    tcgen05_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive_cluster(release);
  }
  __syncwarp();

  const int hk = is_k ? head - e.Hq : head - e.Hq - e.Hkv;
  const float wl[4] = {w_lo.x, w_lo.y, w_lo.z, w_lo.w}, wh[4] = {w_hi.x, w_hi.y, w_hi.z, w_hi.w};
  // where the lane's pieces of row `sub` go: q rows are Hq D apart; k and v rows are found by the row's own offset
  __nv_bfloat16* const q_dst = e.q_out + ((size_t)(row_base + sub) * e.Hq + head) * D + l * 4;
  const size_t q_pitch = (size_t)e.Hq * D;
  __nv_bfloat16* const kv_dst = (is_k ? e.k_pages : e.v_pages) + (size_t)hk * e.page_size * D + l * 4;
  const unsigned char* const my_rows = mine + sub * STRIDE;
  auto work = [&](int b, const float4 (&buf)[BATCH][2]) {
    // the batch's rows in three sweeps (all reads, all arithmetic, all stores), so that the rows' chains of
    // dependent instructions run beside each other instead of one after the other
    uint4 meta[BATCH];
    uint2 lo2[BATCH], hi2[BATCH];
#pragma unroll
    for (int i = 0; i < BATCH; ++i) {
      const unsigned char* srow = my_rows + ((b * BATCH + i) * RPW) * STRIDE;
      meta[i] = *reinterpret_cast<const uint4*>(srow + D * 2);
      lo2[i] = *reinterpret_cast<const uint2*>(srow + l * 8);
      hi2[i] = *reinterpret_cast<const uint2*>(srow + D + l * 8);
    }
    if (is_q || is_k) {  // uniform over the warp
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        const float4(&c)[2] = buf[i];
        float lo[4] = {__uint_as_float(lo2[i].x << 16), __uint_as_float(lo2[i].x & 0xffff0000u),
                       __uint_as_float(lo2[i].y << 16), __uint_as_float(lo2[i].y & 0xffff0000u)};
        float hi[4] = {__uint_as_float(hi2[i].x << 16), __uint_as_float(hi2[i].x & 0xffff0000u),
                       __uint_as_float(hi2[i].y << 16), __uint_as_float(hi2[i].y & 0xffff0000u)};
        if (has_w) {
          const float rs_r = __uint_as_float(meta[i].x);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            lo[k] = lo[k] * rs_r * wl[k];
            hi[k] = hi[k] * rs_r * wh[k];
          }
        }
        if (rotate) {
          const float cv[4] = {c[0].x, c[0].y, c[0].z, c[0].w}, sv[4] = {c[1].x, c[1].y, c[1].z, c[1].w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float a = lo[k], b2 = hi[k];
            lo[k] = fmaf(-b2, sv[k], a * cv[k]);
            hi[k] = fmaf(a, sv[k], b2 * cv[k]);
          }
        }
        lo2[i].x = pack2(__float_as_uint(lo[0]), __float_as_uint(lo[1]));
        lo2[i].y = pack2(__float_as_uint(lo[2]), __float_as_uint(lo[3]));
        hi2[i].x = pack2(__float_as_uint(hi[0]), __float_as_uint(hi[1]));
        hi2[i].y = pack2(__float_as_uint(hi[2]), __float_as_uint(hi[3]));
      }
    }
#pragma unroll
    for (int i = 0; i < BATCH; ++i) {
      const int r = (b * BATCH + i) * RPW + sub;
      const long long off = (long long)(((unsigned long long)meta[i].z << 32) | meta[i].y);
      __nv_bfloat16* dst = is_q ? q_dst + (size_t)((b * BATCH + i) * RPW) * q_pitch : kv_dst + off;
      if ((FAST || r < rows_here) && (is_q || off >= 0)) {
        *reinterpret_cast<uint2*>(dst) = lo2[i];
        *reinterpret_cast<uint2*>(dst + D / 2) = hi2[i];
      }
    }
  };
  static_assert(NB % 2 == 0, "batches are worked on in pairs");
#pragma unroll 1
  for (int b = 0; b < NB; b += 2) {
    if (rotate) fetch(b + 1, cs[1]);
    work(b, cs[0]);
    if (rotate && b + 2 < NB) fetch(b + 2, cs[0]);
    work(b + 1, cs[1]);
  }
  __syncwarp();
}

// The QKV epilogue of one accumulator of 128 rows x BN columns (whole heads of HD), by the block's EPI_WARPS
// epilogue warps: two warps per quarter of the rows, each taking every second head of the tile.  The cache
// position of the thread's own row is looked up once per tile.  The accumulator goes back to the issuing thread
// (one arrival per warp on `release`, an address in the cluster's shared window) as soon as the warp's last head
// has been read out of it, before that head's second pass.  `tmem_acc` is the accumulator at the warp's lanes,
// `m0` the first row of these 128.
template <int HD, int BN, int EPI_WARPS>
__device__ __forceinline__ void qkv_tile_epilogue(uint32_t tmem_acc, unsigned char* head_stage, int warp, int lane,
                                                  int m0, int n0, int M, int N, const QkvEpilogue& qkv,
                                                  uint32_t release, int* status) {
  constexpr int SLOTS = EPI_WARPS / 4;
  const int quarter = warp & 3, row = m0 + quarter * 32 + lane;
  const int ew = warp - 2, slot = ew >> 2;
  unsigned char* mine = head_stage + ew * 32 * (HD * 2 + TC_QKV_ROW_PAD);
  const int rows_here = max(0, min(32, M - (m0 + quarter * 32)));
  long long kv_off = -1;
  if (qkv.write_kv && lane < rows_here && n0 + BN > qkv.Hq * HD) {
    const int pos = qkv.positions[row], seq = qkv.tok_seq[row];
    if (pos < 0 || seq < 0) {
      atomicOr(status, Q3_STATUS_BAD_POSITION);
    } else {
      const int page = table_page(qkv.block_table + (size_t)seq * qkv.table_stride, pos / qkv.page_size,
                                  qkv.table_stride, status);
      if (page < 0 || page >= qkv.num_pages)
        atomicOr(status, Q3_STATUS_BAD_PAGE);
      else
        kv_off = ((long long)page * qkv.Hkv * qkv.page_size + (pos % qkv.page_size)) * HD;
    }
  }
  bool released = false;
#pragma unroll 1
  for (int h0 = slot * HD; h0 < BN && n0 + h0 < N; h0 += SLOTS * HD) {  // uniform over the warp
    const bool last = h0 + SLOTS * HD >= BN || n0 + h0 + SLOTS * HD >= N;
    // Whole groups of 32 rows of a head that is normed and rotated (or a v head) take a form of the code in which
    // the kind of head, the norm, the rotation and the row count are fixed when it is compiled; the rest (the last
    // rows of the matrix, a layer without head norms or without rotation) the form that asks as it goes.
    const int head = (n0 + h0) / HD;
    const bool head_q = head < qkv.Hq, head_k = !head_q && head < qkv.Hq + qkv.Hkv;
    const bool fixed = rows_here == 32 && (!(head_q || head_k) || (qkv.cos_sin != nullptr &&
                                                                  (head_q ? qkv.q_weight : qkv.k_weight) != nullptr));
#define Q3_QKV_HEAD(KIND, FAST)                                                                                      \
  qkv_head_rows<HD, KIND, FAST>(tmem_acc + (uint32_t)h0, mine, m0 + quarter * 32, rows_here, head, qkv, lane, kv_off, \
                                last ? release : 0u)
    if (!fixed) Q3_QKV_HEAD(-1, false);  // every branch here is uniform over the warp
    else if (head_q) Q3_QKV_HEAD(0, true);
    else if (head_k) Q3_QKV_HEAD(1, true);
    else Q3_QKV_HEAD(2, true);
#undef Q3_QKV_HEAD
    released = released || last;
  }
  if (!released) {  // a warp without a head in the matrix's last tile
    tcgen05_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive_cluster(release);
  }
}

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

// EPI 0: store.  EPI 1: SwiGLU.  EPI 2: the QKV epilogue with heads of HD values (C is not written).
template <int BN, int EPI, typename OutT, int HD = 128>
__global__ void __launch_bounds__(TcThreads<EPI>::THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               OutT* __restrict__ C, int M, int N, int K, int ldc, const __grid_constant__ QkvEpilogue qkv, int* status) {
  using S = TcShape<BN, EPI>;
  // used as it is declared, so that the compiler knows these are shared-memory addresses (a base rounded up
  // through an integer made every access of the QKV epilogue's staging rows a generic one)
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = smem_raw;
  unsigned char* tiles = base;
  uint64_t* full = reinterpret_cast<uint64_t*>(base + (size_t)S::STAGES * S::STAGE_BYTES);
  uint64_t* empty = full + S::STAGES;
  uint64_t* acc_full = empty + S::STAGES;  // [2]
  uint64_t* acc_empty = acc_full + 2;      // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  unsigned char* head_stage = base + (size_t)S::STAGES * S::STAGE_BYTES + S::BAR_BYTES;  // EPI 2 only
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_tiles = (K + TC_BK - 1) / TC_BK;
  const int m_tiles = (M + TC_BM - 1) / TC_BM, n_tiles = (N + BN - 1) / BN;
  // the swizzled tiles need a base on a 1024-byte boundary; never seen otherwise, but a wrong answer must not be silent
  const bool aligned = (s_addr(smem_raw) & 1023u) == 0;
  const int num_tiles = aligned ? m_tiles * n_tiles : 0;
  if (!aligned && threadIdx.x == 0) atomicOr(status, Q3_STATUS_TIMEOUT);

  if (warp == 0 && lane == 0) {
    tma_prefetch_map(&map_a);
    tma_prefetch_map(&map_b);
  }
  int ahead = 0;  // thread 0 (the loader): how many of its first (tile, k tile) pairs have their W tile under way
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], TcThreads<EPI>::EPI_WARPS);  // one arrival from each epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // The weights do not depend on the kernel before this one: the W tiles of the ring's first round are
    // asked for now, the activations' tiles after the wait (the loader below leaves these W tiles out).
    for (int tile = blockIdx.x; tile < num_tiles && ahead < S::STAGES; tile += gridDim.x) {
      const int n0 = (tile / m_tiles) * BN;
      for (int kt = 0; kt < k_tiles && ahead < S::STAGES; ++kt, ++ahead) {
        mbar_expect_tx(&full[ahead], S::STAGE_BYTES);
        tma_load_2d(tiles + (size_t)ahead * S::STAGE_BYTES + S::A_BYTES, &map_b, &full[ahead], kt * TC_BK, n0);
      }
    }
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
          unsigned char* a_s = tiles + (size_t)s * S::STAGE_BYTES;
          if ((int)it >= ahead) {
            if (use > 0 && !mbar_wait(&empty[s], (use & 1) ^ 1, &abort_flag)) {
              abort_flag = 1;
              atomicOr(status, Q3_STATUS_TIMEOUT);
              ok = false;
              break;
            }
            mbar_expect_tx(&full[s], S::STAGE_BYTES);
            tma_load_2d(a_s + S::A_BYTES, &map_b, &full[s], kt * TC_BK, n0);
          }
          if ((int)it == tc_drop_copy) continue;  // tests of the give-up path only (see tc_common.cuh)
          tma_load_2d(a_s, &map_a, &full[s], kt * TC_BK, m0);
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
      if (EPI == 2) {
        qkv_tile_epilogue<HD, BN, TcThreads<EPI>::EPI_WARPS>(tmem_acc, head_stage, warp, lane, m0, n0, M, N, qkv,
                                                             s_addr(&acc_empty[buf]), status);
      } else {
#pragma unroll 1
        for (int c0 = ((warp - 2) >> 2) * 32; c0 < BN; c0 += (TcThreads<EPI>::EPI_WARPS / 4) * 32) {
          if (n0 + c0 >= N) break;  // uniform over the warp
          uint32_t v[32];
          tmem_ld_32(tmem_acc + (uint32_t)c0, v);
          tmem_wait_ld();
          if (row < M) tc_store_chunk<EPI == 2 ? 0 : EPI, OutT>(v, C, row, n0 + c0, N, ldc);
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(S::TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------- the same product by pairs of CTAs
// Two CTAs of a cluster work on one 256 x 256 tile with the paired instruction (cta_group::2, M = 256): the
// CTA of rank r holds rows 128 r .. 128 r + 127 of the A tile and of the W tile in its own shared memory and
// rows 128 r .. of the accumulator (all 256 columns) in its own tensor memory.  An instruction of k = 16 then
// reads 8 KB of operands per SM where the single CTA's 128 x 256 tile reads 12 KB, which with TMA writing as
// much was more than shared memory gives per clock; a stage is 32 KB per CTA.
//   warp 0 (one thread, both CTAs)  waits on its own CTA's `empty`, brings its halves in; every copy of
//                                   the pair is counted by rank 0's `full` barrier (rank 0 expects the bytes of both);
//   warp 1 (one thread, rank 0)     waits on `full`, issues for the pair, and commits with one arrival on
//                                   `empty` / `acc_full` in both CTAs;
//   warps 2..5 or 2..9 (both CTAs)  read their own CTA's accumulator rows, store, and arrive on rank 0's
//                                   `acc_empty` (the arrivals of both CTAs' epilogue warps hand an accumulator back).
// Every wait is bounded as above; a role that gives up raises the abort flag of both CTAs.  Both CTAs meet at a
// cluster barrier before the first copy (a barrier must be initialised before the other CTA's copy counts on
// it) and before they free tensor memory and return (no arrival or operand read may find a CTA gone).
template <int EPI = 0>
struct TcPairShape {
  static constexpr int BN = 256;
  static constexpr int A_BYTES = TC_BM * TC_BK * 2;        // this CTA's 128 rows of A
  static constexpr int B_BYTES = (BN / 2) * TC_BK * 2;     // this CTA's 128 rows of W
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;    // 32 KB
  static constexpr int EPI_BYTES = EPI == 2 ? TC_HEAD_STAGE_BYTES : 0;
  static constexpr int STAGES = EPI == 2 ? 4 : 7;          // beside the QKV epilogue's 68 KB, four
  static constexpr int BAR_BYTES = 256;
  static constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + BAR_BYTES + EPI_BYTES;
  static constexpr uint32_t TMEM_COLS = 2 * BN;
  static constexpr int THREADS = TcThreads<EPI>::THREADS;
};

template <int EPI, typename OutT, int HD = 128>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TcPairShape<EPI>::THREADS)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    OutT* __restrict__ C, int M, int N, int K, int ldc, const __grid_constant__ QkvEpilogue qkv,
                    int* status) {
  using S = TcPairShape<EPI>;
  constexpr int BN = S::BN;
  // used as it is declared, so that the compiler knows these are shared-memory addresses (a base rounded up
  // through an integer made every access of the QKV epilogue's staging rows a generic one)
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = smem_raw;
  unsigned char* tiles = base;
  uint64_t* full = reinterpret_cast<uint64_t*>(base + (size_t)S::STAGES * S::STAGE_BYTES);  // used in rank 0
  uint64_t* empty = full + S::STAGES;
  uint64_t* acc_full = empty + S::STAGES;  // [2]
  uint64_t* acc_empty = acc_full + 2;      // [2], used in rank 0
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  unsigned char* head_stage = base + (size_t)S::STAGES * S::STAGE_BYTES + S::BAR_BYTES;  // EPI 2 only
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int k_tiles = (K + TC_BK - 1) / TC_BK;
  const int m_tiles = (M + 2 * TC_BM - 1) / (2 * TC_BM), n_tiles = (N + BN - 1) / BN;
  const bool aligned = (s_addr(smem_raw) & 1023u) == 0;  // as above; the same in both CTAs
  const int num_tiles = aligned ? m_tiles * n_tiles : 0;
  if (!aligned && threadIdx.x == 0) atomicOr(status, Q3_STATUS_TIMEOUT);
  auto give_up = [&]() {  // one thread
    abort_flag = 1;
    st_cluster_u32(cluster_addr(s_addr(&abort_flag), rank ^ 1u), 1u);
    atomicOr(status, Q3_STATUS_TIMEOUT);
  };

  if (warp == 0 && lane == 0) {
    tma_prefetch_map(&map_a);
    tma_prefetch_map(&map_b);
  }
  if (threadIdx.x == 0) {
    abort_flag = 0;
    *tmem_holder = 0;
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 2 * TcThreads<EPI>::EPI_WARPS);  // the epilogue warps of both CTAs
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  cluster_sync_all();
  int ahead = 0;  // thread 0 (the loader): how many of its first (tile, k tile) pairs have their W tile under way
  if (threadIdx.x == 0) {
    // as in the kernel above: the W tiles of the ring's first round go out before the wait
    for (int tile = pair; tile < num_tiles && ahead < S::STAGES; tile += pairs) {
      const int n0 = (tile / m_tiles) * BN + (int)rank * (BN / 2);
      for (int kt = 0; kt < k_tiles && ahead < S::STAGES; ++kt, ++ahead) {
        if (rank == 0) mbar_expect_tx(&full[ahead], 2 * S::STAGE_BYTES);
        tma_load_2d_pair(tiles + (size_t)ahead * S::STAGE_BYTES + S::A_BYTES, &map_b,
                         cluster_addr(s_addr(&full[ahead]), 0), kt * TC_BK, n0);
      }
    }
  }
  pdl_wait();  // the activations come from the kernel before this one
  pdl_launch_dependents();
  // Tensor memory is taken only after the wait (see above); the same warp of both CTAs asks, for the pair.
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_addr(tmem_holder)),
                 "r"(S::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
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
      for (int tile = pair; tile < num_tiles && ok; tile += pairs) {
        const int m0 = (tile % m_tiles) * 2 * TC_BM + (int)rank * TC_BM;
        const int n0 = (tile / m_tiles) * BN + (int)rank * (BN / 2);
        for (int kt = 0; kt < k_tiles; ++kt, ++it) {
          const int s = it % S::STAGES;
          const uint32_t use = it / S::STAGES;
          unsigned char* a_s = tiles + (size_t)s * S::STAGE_BYTES;
          const uint32_t pair_full = cluster_addr(s_addr(&full[s]), 0);
          if ((int)it >= ahead) {
            if (use > 0 && !mbar_wait(&empty[s], (use & 1) ^ 1, &abort_flag)) {
              give_up();
              ok = false;
              break;
            }
            if (rank == 0) mbar_expect_tx(&full[s], 2 * S::STAGE_BYTES);
            tma_load_2d_pair(a_s + S::A_BYTES, &map_b, pair_full, kt * TC_BK, n0);
          }
          if ((int)it == tc_drop_copy && rank == 0) continue;  // tests of the give-up path only (see tc_common.cuh)
          tma_load_2d_pair(a_s, &map_a, pair_full, kt * TC_BK, m0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // ---- tensor-core issue, for the pair
      constexpr uint32_t idesc = umma_idesc_pair(BN);
      uint32_t it = 0, t = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += pairs, ++t) {
        const uint32_t buf = t & 1;
        if (t >= 2 && !mbar_wait_cluster(&acc_empty[buf], ((t >> 1) & 1) ^ 1, &abort_flag)) {
          ok = false;
          break;
        }
        tcgen05_fence_after();
        const uint32_t tmem_acc = tmem_base + buf * BN;
        for (int kt = 0; kt < k_tiles; ++kt, ++it) {
          const int s = it % S::STAGES;
          const uint32_t use = it / S::STAGES;
          if (!mbar_wait_cluster(&full[s], use & 1, &abort_flag)) {
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const unsigned char* a_s = tiles + (size_t)s * S::STAGE_BYTES;
          const uint64_t a_desc = umma_desc_sw128(a_s), b_desc = umma_desc_sw128(a_s + S::A_BYTES);
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k)
            umma_f16_pair(tmem_acc, a_desc + 2 * k, b_desc + 2 * k, idesc, (kt | k) != 0);
          umma_commit_pair(&empty[s]);
        }
        if (ok) umma_commit_pair(&acc_full[buf]);
      }
      if (!ok) give_up();
    }
  } else {
    // ---- epilogue: this CTA's 128 rows of the tile
    const int quarter = warp & 3;
    uint32_t t = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += pairs, ++t) {
      const int m0 = (tile % m_tiles) * 2 * TC_BM + (int)rank * TC_BM, n0 = (tile / m_tiles) * BN;
      const uint32_t buf = t & 1;
      const bool ready = mbar_wait(&acc_full[buf], (t >> 1) & 1, &abort_flag);
      if (!__all_sync(0xffffffffu, ready)) {
        if (lane == 0) give_up();
        ok = false;
        break;
      }
      tcgen05_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t tmem_acc = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
      const uint32_t release = cluster_addr(s_addr(&acc_empty[buf]), 0);
      if (EPI == 2) {
        qkv_tile_epilogue<HD, BN, TcThreads<EPI>::EPI_WARPS>(tmem_acc, head_stage, warp, lane, m0, n0, M, N, qkv, release,
                                                             status);
      } else {
#pragma unroll 1
        for (int c0 = ((warp - 2) >> 2) * 32; c0 < BN; c0 += (TcThreads<EPI>::EPI_WARPS / 4) * 32) {
          if (n0 + c0 >= N) break;  // uniform over the warp
          uint32_t v[32];
          tmem_ld_32(tmem_acc + (uint32_t)c0, v);
          tmem_wait_ld();
          if (row < M) tc_store_chunk<EPI == 2 ? 0 : EPI, OutT>(v, C, row, n0 + c0, N, ldc);
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(release);
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(S::TMEM_COLS) : "memory");
  }
}

// How many pairs of CTAs the device runs at a time (a cluster's two CTAs need SMs of one group).
template <int EPI, typename OutT, int HD>
static int tc_pair_slots() {
  static int slots[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (slots[dev] == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * sm_count());
    cfg.blockDim = dim3(TcPairShape<EPI>::THREADS);
    cfg.dynamicSmemBytes = TcPairShape<EPI>::SMEM_BYTES;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_kernel<EPI, OutT, HD>, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count() / 2;
    }
    slots[dev] = n < sm_count() / 2 ? n : sm_count() / 2;
  }
  return slots[dev];
}

template <int EPI, typename OutT, int HD = 128>
static int gemm_tc_pair_launch(const void* A, const void* W, void* C, int M, int N, int K, int ldc, int* status,
                               cudaStream_t stream, const QkvEpilogue& qkv = QkvEpilogue{}) {
  using S = TcPairShape<EPI>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<EPI, OutT, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)S::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  CUtensorMap map_a, map_b;
  int code = cached_map(&map_a, A, (uint64_t)M, (uint64_t)K, TC_BM);
  if (code) return code;
  code = cached_map(&map_b, W, (uint64_t)N, (uint64_t)K, S::BN / 2);
  if (code) return code;
  const long long tiles = (long long)((N + S::BN - 1) / S::BN) * ((M + 2 * TC_BM - 1) / (2 * TC_BM));
  if (tiles > 0x3fffffffLL) return Q3_ERR_SIZE;
  const int slots = tc_pair_slots<EPI, OutT, HD>();
  if (slots <= 0) return Q3_ERR_DRIVER;
  const int pairs = (int)(tiles < slots ? tiles : slots);
  q3::launch(gemm_tc_pair_kernel<EPI, OutT, HD>, dim3(2 * pairs), dim3(S::THREADS), S::SMEM_BYTES, stream, map_a, map_b,
             (OutT*)C, M, N, K, ldc, qkv, status);
  return launch_status();
}

template <int BN, int EPI, typename OutT, int HD = 128>
static int gemm_tc_launch(const void* A, const void* W, void* C, int M, int N, int K, int ldc, int* status,
                          cudaStream_t stream, const QkvEpilogue& qkv = QkvEpilogue{}) {
  using S = TcShape<BN, EPI>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, EPI, OutT, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
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
  const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
  q3::launch(gemm_tc_kernel<BN, EPI, OutT, HD>, dim3(grid), dim3(TcThreads<EPI>::THREADS), S::SMEM_BYTES, stream, map_a, map_b,
             (OutT*)C, M, N, K, ldc, qkv, status);
  return launch_status();
}

// The tile width that needs fewer rounds of the SMs: rounds x width is the cost of the slowest block.
static int tc_pick_bn(int M, int N) {
  const long long sms = sm_count();
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

// The same product by pairs of CTAs on 256 x 256 tiles (the paired tensor-core instruction); arguments and
// limits as q3_gemm_tc.
extern "C" int q3_gemm_tc_pair(const void* A, const void* W, void* C, int M, int N, int K, int ldc, int out_f32,
                               int swiglu, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || (swiglu && (N % 16 || out_f32))) return Q3_ERR_SIZE;
  if ((uintptr_t)A % 16 || (uintptr_t)W % 16) return Q3_ERR_ALIGN;
  using bf16 = __nv_bfloat16;
  if (swiglu) return q3::gemm_tc_pair_launch<1, bf16>(A, W, C, M, N, K, ldc, status, stream);
  if (out_f32) return q3::gemm_tc_pair_launch<0, float>(A, W, C, M, N, K, ldc, status, stream);
  return q3::gemm_tc_pair_launch<0, bf16>(A, W, C, M, N, K, ldc, status, stream);
}

// For the tests of the give-up path: see set_wait_test in tc_common.cuh.
extern "C" int q3_gemm_tc_wait_test(unsigned limit, int drop) { return q3::set_wait_test(limit, drop); }

// The merged QKV projection of an attention layer with the work of q3_qkv_post in its epilogue:
// qkv = A[T, K] * W[(Hq + 2 Hkv) D, K]^T is rounded to bfloat16 and, head by head, normed, rotated and
// written to q_out / the cache pages; it is never stored itself.  Arguments as q3_qkv_post, with A and W
// as q3_gemm_tc.  Takes bfloat16, D = 64 or 128 and a whole rotation (cos_sin from q3_rope_table) or
// none; refuses the rest.  pair: by pairs of CTAs (the paired instruction) instead of single CTAs.
extern "C" int q3_gemm_tc_qkv(const void* A, const void* W, int T, int K, int Hq, int Hkv, int D, const float* q_weight,
                              const float* k_weight, float eps, const float* cos_sin, const int* positions,
                              const int* tok_seq, const int* block_table, int table_stride, int page_size,
                              void* k_pages, void* v_pages, int num_pages, void* q_out, int write_kv, int pair,
                              int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (K <= 0 || K % 8 || (D != 64 && D != 128) || Hq < 0 || Hkv < 0 || page_size <= 0 || table_stride <= 0)
    return Q3_ERR_SIZE;
  if ((uintptr_t)A % 16 || (uintptr_t)W % 16 || (uintptr_t)q_out % 16 || (uintptr_t)k_pages % 16 ||
      (uintptr_t)v_pages % 16 || (uintptr_t)q_weight % 16 || (uintptr_t)k_weight % 16 || (uintptr_t)cos_sin % 16)
    return Q3_ERR_ALIGN;
  q3::QkvEpilogue e;
  e.q_out = (__nv_bfloat16*)q_out;
  e.k_pages = (__nv_bfloat16*)k_pages;
  e.v_pages = (__nv_bfloat16*)v_pages;
  e.q_weight = q_weight;
  e.k_weight = k_weight;
  e.cos_sin = cos_sin;
  e.positions = positions;
  e.tok_seq = tok_seq;
  e.block_table = block_table;
  e.table_stride = table_stride;
  e.page_size = page_size;
  e.num_pages = num_pages;
  e.Hq = Hq;
  e.Hkv = Hkv;
  e.eps = eps;
  e.write_kv = write_kv;
  const int N = (Hq + 2 * Hkv) * D;
  using bf16 = __nv_bfloat16;
  if (pair) {  // pairs of CTAs on tiles of 256 rows x 256 columns
    if (D == 128) return q3::gemm_tc_pair_launch<2, bf16, 128>(A, W, nullptr, T, N, K, 0, status, stream, e);
    return q3::gemm_tc_pair_launch<2, bf16, 64>(A, W, nullptr, T, N, K, 0, status, stream, e);
  }
  // tiles of 256 columns (two heads of 128) or of 128 (one): whichever needs fewer rounds of the SMs
  if (D == 128) {
    if (q3::tc_pick_bn(T, N) == 256) return q3::gemm_tc_launch<256, 2, bf16, 128>(A, W, nullptr, T, N, K, 0, status, stream, e);
    return q3::gemm_tc_launch<128, 2, bf16, 128>(A, W, nullptr, T, N, K, 0, status, stream, e);
  }
  if (q3::tc_pick_bn(T, N) == 256) return q3::gemm_tc_launch<256, 2, bf16, 64>(A, W, nullptr, T, N, K, 0, status, stream, e);
  return q3::gemm_tc_launch<128, 2, bf16, 64>(A, W, nullptr, T, N, K, 0, status, stream, e);
}
