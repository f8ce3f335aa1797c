// Paged causal attention for prompt portions (any number of query tokens per sequence), bfloat16.
//
// Grid (query tile, kv head, sequence).  The rows of a query tile are (token, head-in-group)
// pairs of one kv head, 128 (or 64 for large heads) to a block: row R -> token R / g, head hk * g + R % g, so the g
// query heads that share a kv head also share every key/value tile that is fetched.  Keys
// and values come from the pages in tiles of 64 keys (cp.async, two stages); S = Q K^T and
// O += P V run on the tensor cores (m16n8k16, bfloat16 in, float32 accumulate), the running
// maximum, denominator and output stay in float32 registers.  Causality is on absolute
// positions: the query at position p = kv_len - q_len + i reads keys n <= p, and with a window
// only n > p - window.  Keys of this step are already in the pages when this kernel runs.
//
// Reference: kernels/triton/paged_attn.py:314-465 (the same folding of the group into the rows,
// used there for decode and for portions alike), :89-181 (online softmax, exp2).
#include "attn_mma.cuh"

namespace q3 {

constexpr int AP_BN = 64;  // keys per tile

// Up to D = 128 a block has eight warps (128 query rows) and is held to 128 registers a thread,
// so that two blocks, sixteen warps, share an SM: with fewer warps the long dependent chains of
// the softmax leave the tensor cores idle.  Larger heads use four warps (64 rows).
template <int KT>
struct PrefillShape {
  static constexpr int D = 16 * KT;
  static constexpr int PITCH = D + 8;
  static constexpr int TILE = AP_BN * PITCH;
  static constexpr int WARPS = KT <= 8 ? 8 : 4;
  static constexpr int BM = 16 * WARPS;  // query rows per block
  static constexpr int MIN_BLOCKS = KT <= 8 ? 2 : 1;
  static constexpr size_t SMEM_BYTES = sizeof(__nv_bfloat16) * (size_t)(BM * PITCH + 4 * TILE);
};

template <int KT>
__global__ void __launch_bounds__(PrefillShape<KT>::WARPS * 32, PrefillShape<KT>::MIN_BLOCKS)
attn_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                    const __nv_bfloat16* __restrict__ v_pages, __nv_bfloat16* __restrict__ out,
                    const int* __restrict__ q_start, const int* __restrict__ kv_len,
                    const int* __restrict__ block_table, int table_stride, int page_size, int num_pages,
                    int Hq, int Hkv, float scale_log2, int window, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  using S = PrefillShape<KT>;
  constexpr int D = S::D, PITCH = S::PITCH, TILE = S::TILE, CPR = D / 8;
  constexpr int AP_WARPS = S::WARPS, AP_BM = S::BM;
  constexpr bool Q_IN_REGS = false;  // the query fragments are re-read from shared memory: registers go to the output
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* kv_s = q_s + AP_BM * PITCH;  // [stage][K | V][64][PITCH]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tid4 = lane & 3;
  const int qt = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int g = Hq / Hkv;
  const int qs = q_start[b];
  const int q_len = q_start[b + 1] - qs;
  const int len = kv_len[b];
  const int total_rows = q_len * g;
  const int row0 = qt * AP_BM;
  if (row0 >= total_rows) return;
  const int past = len - q_len;  // position of this step's first token
  if (past < 0) {
    if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
    return;
  }
  const int* table = block_table + (size_t)b * table_stride;
  const int last_row = min(total_rows, row0 + AP_BM) - 1;
  const int pos_first = past + row0 / g, pos_last = past + last_row / g;
  const int lo_key = (window > 0 && pos_first - window + 1 > 0) ? pos_first - window + 1 : 0;
  const int tile_lo = lo_key / AP_BN, tile_hi = pos_last / AP_BN;

  // query tile to shared memory (rows past the end are zero)
  for (int e = threadIdx.x; e < AP_BM * CPR; e += AP_WARPS * 32) {
    const int rr = e / CPR, c = e % CPR;
    const int R = row0 + rr;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (R < total_rows)
      v = *reinterpret_cast<const uint4*>(q + ((size_t)(qs + R / g) * Hq + hk * g + R % g) * D + c * 8);
    *reinterpret_cast<uint4*>(q_s + rr * PITCH + c * 8) = v;
  }

  constexpr int LANES_PER_ROW = AP_WARPS * 32 / AP_BN;  // threads that share a key row: 2 or 4
  auto load_tile = [&](int tile, int stage) {
    const int row = threadIdx.x / LANES_PER_ROW, half = threadIdx.x % LANES_PER_ROW;
    const int n = tile * AP_BN + row;
    const __nv_bfloat16 *ks = k_pages, *vs = v_pages;
    int bytes = 0;
    if (n >= lo_key && n <= pos_last) {
      const int page = table_page(table, n / page_size, table_stride, status);
      if (page >= 0 && page < num_pages) {
        const size_t off = (((size_t)page * Hkv + hk) * page_size + (n % page_size)) * D;
        ks = k_pages + off;
        vs = v_pages + off;
        bytes = 16;
      } else {
        atomicOr(status, Q3_STATUS_BAD_PAGE);
      }
    }
    __nv_bfloat16* kd = kv_s + (size_t)(stage * 2) * TILE + row * PITCH;
    __nv_bfloat16* vd = kd + TILE;
#pragma unroll
    for (int c = half; c < CPR; c += LANES_PER_ROW) {
      const int src = bytes ? c * 8 : 0;
      cp_async_16(kd + c * 8, ks + src, bytes);
      cp_async_16(vd + c * 8, vs + src, bytes);
    }
  };

  load_tile(tile_lo, 0);
  cp_async_commit();
  __syncthreads();  // the query tile is in place

  const __nv_bfloat16* q_warp = q_s + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + (lane >> 4) * 8;
  uint32_t qa[Q_IN_REGS ? KT : 1][4];
  if (Q_IN_REGS) {
#pragma unroll
    for (int kt = 0; kt < KT; ++kt) ldmatrix_x4(qa[Q_IN_REGS ? kt : 0], q_warp + kt * 16);
  }

  // the two rows this thread owns in the score and output fragments
  int row_pos[2], row_lo[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int R = row0 + warp * 16 + gid + 8 * r;
    row_pos[r] = R < total_rows ? past + R / g : pos_last;  // rows past the end compute something finite, unused
    row_lo[r] = (window > 0 && row_pos[r] - window + 1 > 0) ? row_pos[r] - window + 1 : 0;
  }

  float o[2 * KT][4];
#pragma unroll
  for (int i = 0; i < 2 * KT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  for (int tile = tile_lo; tile <= tile_hi; ++tile) {
    const int stage = (tile - tile_lo) & 1;
    if (tile + 1 <= tile_hi) load_tile(tile + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const __nv_bfloat16* kt_s = kv_s + (size_t)(stage * 2) * TILE;
    const __nv_bfloat16* vt_s = kt_s + TILE;

    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int kt = 0; kt < KT; ++kt) {
      uint32_t qf[4];
      if (Q_IN_REGS) {
        qf[0] = qa[Q_IN_REGS ? kt : 0][0]; qf[1] = qa[Q_IN_REGS ? kt : 0][1];
        qf[2] = qa[Q_IN_REGS ? kt : 0][2]; qf[3] = qa[Q_IN_REGS ? kt : 0][3];
      } else {
        ldmatrix_x4(qf, q_warp + kt * 16);
      }
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t kb[4];
        ldmatrix_x4(kb, kt_s + (np * 16 + (lane & 7) + ((lane >> 4) << 3)) * PITCH + kt * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[2 * np], qf, kb[0], kb[1]);
        mma_bf16(s[2 * np + 1], qf, kb[2], kb[3]);
      }
    }
    const int base_n = tile * AP_BN;
    const bool edge = window > 0 || base_n + AP_BN - 1 > pos_first;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = base_n + nt * 8 + 2 * tid4 + (j & 1);
        float v = s[nt][j] * scale_log2;
        if (edge && (n > row_pos[j >> 1] || n < row_lo[j >> 1])) v = -INFINITY;
        s[nt][j] = v;
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float mx = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) mx = fmaxf(mx, fmaxf(s[nt][2 * r], s[nt][2 * r + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m[r], mx);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = exp2f(m[r] - m_use);
      m[r] = m_new;
      l[r] *= alpha;
#pragma unroll
      for (int i = 0; i < 2 * KT; ++i) {
        o[i][2 * r] *= alpha;
        o[i][2 * r + 1] *= alpha;
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const float p0 = exp2f(s[nt][2 * r] - m_use), p1 = exp2f(s[nt][2 * r + 1] - m_use);
        s[nt][2 * r] = p0;
        s[nt][2 * r + 1] = p1;
        l[r] += p0 + p1;
      }
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t pa[4];
      pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int dt = 0; dt < KT; ++dt) {
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, vt_s + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + dt * 16 + (lane >> 4) * 8);
        mma_bf16(o[2 * dt], pa, vb[0], vb[1]);
        mma_bf16(o[2 * dt + 1], pa, vb[2], vb[3]);
      }
    }
    __syncthreads();  // this stage may be overwritten by the load issued in the next iteration
  }
  cp_async_wait<0>();

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    const int R = row0 + warp * 16 + gid + 8 * r;
    if (R >= total_rows) continue;
    const float inv = l[r] > 0.f ? 1.0f / l[r] : 0.f;
    __nv_bfloat16* dst = out + ((size_t)(qs + R / g) * Hq + hk * g + R % g) * D + 2 * tid4;
#pragma unroll
    for (int nt = 0; nt < 2 * KT; ++nt)
      *reinterpret_cast<__nv_bfloat162*>(dst + nt * 8) =
          __floats2bfloat162_rn(o[nt][2 * r] * inv, o[nt][2 * r + 1] * inv);
  }
}

template <int KT>
static int attn_prefill_launch(const void* q, const void* k_pages, const void* v_pages, void* out,
                               const int* q_start, const int* kv_len, const int* block_table, int table_stride,
                               int page_size, int num_pages, int B, int max_q_len, int Hq, int Hkv, float scale,
                               int window, int* status, cudaStream_t stream) {
  using S = PrefillShape<KT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<KT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)S::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int g = Hq / Hkv;
  const long long tiles = ((long long)max_q_len * g + S::BM - 1) / S::BM;
  if (tiles > 0x7fffffffLL) return Q3_ERR_SIZE;
  dim3 grid((unsigned)tiles, Hkv, B);
  q3::launch(attn_prefill_kernel<KT>, dim3(grid), dim3(S::WARPS * 32), S::SMEM_BYTES, stream, 
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, (__nv_bfloat16*)out,
      q_start, kv_len, block_table, table_stride, page_size, num_pages, Hq, Hkv, scale * 1.4426950408889634f, window,
      status);
  return launch_status();
}

}  // namespace q3

// Attention for B sequences that bring q_start[b + 1] - q_start[b] query tokens each (max_q_len at most).
// q, out: bf16 [T, Hq, D]; pages: bf16 [num_pages, Hkv, page_size, D].
// Takes D in multiples of 16 up to 256; refuses the rest.
extern "C" int q3_attn_prefill(const void* q, const void* k_pages, const void* v_pages, void* out,
                               const int* q_start, const int* kv_len, const int* block_table, int table_stride,
                               int page_size, int num_pages, int B, int max_q_len, int Hq, int Hkv, int D,
                               float scale, int window, int* status, cudaStream_t stream) {
  if (B <= 0 || max_q_len <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv || D % 16 || D < 16 || D > 256 || page_size <= 0 || table_stride <= 0 || B > 65535 ||
      Hkv > 65535)
    return Q3_ERR_SIZE;
  if ((uintptr_t)q % 16 || (uintptr_t)k_pages % 16 || (uintptr_t)v_pages % 16 || (uintptr_t)out % 4)
    return Q3_ERR_ALIGN;
#define Q3_AP_CASE(KT)                                                                                        \
  case KT:                                                                                                    \
    return q3::attn_prefill_launch<KT>(q, k_pages, v_pages, out, q_start, kv_len, block_table, table_stride,  \
                                       page_size, num_pages, B, max_q_len, Hq, Hkv, scale, window, status, stream);
  switch (D / 16) {
    Q3_AP_CASE(1) Q3_AP_CASE(2) Q3_AP_CASE(3) Q3_AP_CASE(4) Q3_AP_CASE(5) Q3_AP_CASE(6) Q3_AP_CASE(7) Q3_AP_CASE(8)
    Q3_AP_CASE(9) Q3_AP_CASE(10) Q3_AP_CASE(11) Q3_AP_CASE(12) Q3_AP_CASE(13) Q3_AP_CASE(14) Q3_AP_CASE(15)
    Q3_AP_CASE(16)
  }
#undef Q3_AP_CASE
  return Q3_ERR_SIZE;
}
