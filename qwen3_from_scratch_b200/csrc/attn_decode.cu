// Paged attention for decoding (one query token per sequence), bfloat16, split over the keys.
//
// Grid (split, kv head, sequence).  The Hq / Hkv query heads that share a kv head are the rows
// of one 16-row tensor-core tile, so every key and value is fetched once per kv head.  A
// sequence's keys (from the window's first key to the query's own) are cut into `num_splits`
// ranges of 16-key tiles; inside a block each of the four warps walks every fourth tile of the
// range with its own cp.async pipeline (no block-wide barrier in the loop), keeps a running
// maximum, denominator and output in float32, and the warps are merged through shared memory at
// the end.  With more than one split the block writes (output, maximum, denominator) to scratch
// memory and `attn_combine_kernel` merges the splits.
//
// The number of splits is a launch parameter; which tiles a split covers is computed from
// kv_len on the device, so one captured launch serves every context length.
//
// Formulas as in attn_ref.cu (reference: kernels/triton/paged_attn.py:89-181 — scores scaled by
// D^-0.5 with log2(e) folded in, exp2, probabilities rounded to bfloat16 before P.V).
#include "attn_mma.cuh"

namespace q3 {

constexpr int AD_WARPS = 4;
constexpr int AD_KEYS = 16;  // keys per warp tile

template <int KT>
struct DecodeShape {
  static constexpr int D = 16 * KT;
  static constexpr int PITCH = D + 8;
  static constexpr int TILE = AD_KEYS * PITCH;  // elements of one 16-row tile
  static constexpr int STAGES = 2;  // with two stages three blocks (twelve warps) fit an SM at D = 128
  static constexpr size_t PIPE_BYTES = sizeof(__nv_bfloat16) * (size_t)AD_WARPS * STAGES * 2 * TILE;
  static constexpr size_t MERGE_BYTES = sizeof(float) * (size_t)AD_WARPS * 16 * (D + 2);
  static constexpr size_t SMEM_BYTES =
      sizeof(__nv_bfloat16) * TILE + (PIPE_BYTES > MERGE_BYTES ? PIPE_BYTES : MERGE_BYTES);
};

template <int KT>
__global__ void __launch_bounds__(AD_WARPS * 32)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                   const __nv_bfloat16* __restrict__ v_pages, __nv_bfloat16* __restrict__ out,
                   float* __restrict__ partial, const int* __restrict__ q_start,
                   const int* __restrict__ kv_len, const int* __restrict__ block_table, int table_stride,
                   int page_size, int page_shift, int num_pages, int Hq, int Hkv, float scale_log2,
                   int window, int num_splits, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  using S = DecodeShape<KT>;
  constexpr int D = S::D, PITCH = S::PITCH, TILE = S::TILE, STAGES = S::STAGES, CPR = D / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* pipe = q_s + TILE;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tid4 = lane & 3;
  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int g = Hq / Hkv;
  const int tq = q_start[b];
  const int pos = kv_len[b] - 1;
  const int* table = block_table + (size_t)b * table_stride;

  // the range of 16-key tiles of this split
  int t_lo = 0, t_hi = 0, lo = 0;
  if (pos >= 0) {
    lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int first = lo / AD_KEYS, last = pos / AD_KEYS;
    const int per = (last - first + num_splits) / num_splits;  // ceil((last - first + 1) / num_splits)
    t_lo = first + split * per;
    t_hi = min(t_lo + per, last + 1);
  } else if (threadIdx.x == 0) {
    atomicOr(status, Q3_STATUS_BAD_POSITION);
  }

  // the query rows: row r < g is head hk * g + r, the rest of the 16 rows are zero
  for (int e = threadIdx.x; e < 16 * CPR; e += AD_WARPS * 32) {
    const int row = e / CPR, c = e % CPR;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < g) v = *reinterpret_cast<const uint4*>(q + ((size_t)tq * Hq + hk * g + row) * D + c * 8);
    *reinterpret_cast<uint4*>(q_s + row * PITCH + c * 8) = v;
  }
  __syncthreads();
  uint32_t qa[KT][4];
#pragma unroll
  for (int kt = 0; kt < KT; ++kt)
    ldmatrix_x4(qa[kt], q_s + ((lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + kt * 16 + (lane >> 4) * 8);

  float o[2 * KT][4];
#pragma unroll
  for (int i = 0; i < 2 * KT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  const int my_first = t_lo + warp;
  const int my_count = my_first < t_hi ? (t_hi - my_first + AD_WARPS - 1) / AD_WARPS : 0;
  __nv_bfloat16* my_pipe = pipe + (size_t)warp * STAGES * 2 * TILE;

  // Page ids are looked up one tile ahead of the copy that needs them, so that the copy's
  // address never waits for the table load.
  const int row = lane >> 1, half = lane & 1;
  auto key_of = [&](int ordinal) { return (my_first + ordinal * AD_WARPS) * AD_KEYS + row; };
  auto page_of = [&](int ordinal) -> int {
    const int n = key_of(ordinal);
    if (ordinal >= my_count || n < lo || n > pos) return -1;
    const int page = table_page(table, page_shift >= 0 ? (n >> page_shift) : (n / page_size), table_stride, status);
    if (page < 0 || page >= num_pages) {
      atomicOr(status, Q3_STATUS_BAD_PAGE);
      return -1;
    }
    return page;
  };
  auto issue = [&](int ordinal, int stage, int page) {
    const int n = key_of(ordinal);
    const __nv_bfloat16 *ks = k_pages, *vs = v_pages;
    int bytes = 0;
    if (page >= 0) {
      const int slot = page_shift >= 0 ? (n & (page_size - 1)) : (n % page_size);
      const size_t off = (((size_t)page * Hkv + hk) * page_size + slot) * D;
      ks = k_pages + off;
      vs = v_pages + off;
      bytes = 16;
    }
    __nv_bfloat16* kd = my_pipe + (size_t)(stage * 2) * TILE + row * PITCH;
    __nv_bfloat16* vd = kd + TILE;
#pragma unroll
    for (int c = half; c < CPR; c += 2) {
      const int src = bytes ? c * 8 : 0;
      cp_async_16(kd + c * 8, ks + src, bytes);
      cp_async_16(vd + c * 8, vs + src, bytes);
    }
  };

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    issue(s, s, page_of(s));
    cp_async_commit();
  }
  int next_page = page_of(STAGES - 1);

  for (int i = 0; i < my_count; ++i) {
    cp_async_wait<STAGES - 2>();
    __syncwarp();
    issue(i + STAGES - 1, (i + STAGES - 1) % STAGES, next_page);
    cp_async_commit();
    next_page = page_of(i + STAGES);

    const int stage = i % STAGES;
    const __nv_bfloat16* kt_s = my_pipe + (size_t)(stage * 2) * TILE;
    const __nv_bfloat16* vt_s = kt_s + TILE;
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int kt = 0; kt < KT; ++kt) {
      uint32_t kb[4];
      ldmatrix_x4(kb, kt_s + ((lane & 7) + ((lane >> 4) << 3)) * PITCH + kt * 16 + ((lane >> 3) & 1) * 8);
      mma_bf16(s[0], qa[kt], kb[0], kb[1]);
      mma_bf16(s[1], qa[kt], kb[2], kb[3]);
    }
    const int base_n = (my_first + i * AD_WARPS) * AD_KEYS;
    if (base_n < lo || base_n + AD_KEYS - 1 > pos) {  // only the first and the last tile of a sequence
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int n = base_n + nt * 8 + 2 * tid4 + (j & 1);
          if (n < lo || n > pos) s[nt][j] = -INFINITY;
        }
    }
    // The scale is positive, so the maximum can be taken on the raw scores and the scale folded
    // into the exponent: p = 2^(s * scale - m).
    float mx[2];
    mx[0] = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
    mx[1] = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
    float alpha[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m[r], mx[r] * scale_log2);
      m_use[r] = m_new == -INFINITY ? 0.f : m_new;
      alpha[r] = exp2f(m[r] - m_use[r]);
      m[r] = m_new;
    }
    // Once the running maximum has settled the correction factor is exactly one for every row of
    // the warp, and the pass over the output registers is skipped.
    if (__any_sync(0xffffffffu, alpha[0] != 1.0f || alpha[1] != 1.0f)) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        l[r] *= alpha[r];
#pragma unroll
        for (int i2 = 0; i2 < 2 * KT; ++i2) {
          o[i2][2 * r] *= alpha[r];
          o[i2][2 * r + 1] *= alpha[r];
        }
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const float p0 = exp2f(fmaf(s[nt][2 * r], scale_log2, -m_use[r]));
        const float p1 = exp2f(fmaf(s[nt][2 * r + 1], scale_log2, -m_use[r]));
        s[nt][2 * r] = p0;
        s[nt][2 * r + 1] = p1;
        l[r] += p0 + p1;
      }
    uint32_t pa[4];
    pa[0] = pack_bf16(s[0][0], s[0][1]);
    pa[1] = pack_bf16(s[0][2], s[0][3]);
    pa[2] = pack_bf16(s[1][0], s[1][1]);
    pa[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
    for (int dt = 0; dt < KT; ++dt) {
      uint32_t vb[4];
      ldmatrix_x4_trans(vb, vt_s + ((lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + dt * 16 + (lane >> 4) * 8);
      mma_bf16(o[2 * dt], pa, vb[0], vb[1]);
      mma_bf16(o[2 * dt + 1], pa, vb[2], vb[3]);
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  __syncthreads();  // every warp has left the pipeline memory, which now holds the merge buffers

  float* merge = reinterpret_cast<float*>(pipe);  // [warp][16 rows][D + 2]: output, maximum, denominator
  {
    float* mine = merge + (size_t)warp * 16 * (D + 2);
#pragma unroll
    for (int nt = 0; nt < 2 * KT; ++nt) {
      const int d = nt * 8 + 2 * tid4;
      mine[gid * (D + 2) + d] = o[nt][0];
      mine[gid * (D + 2) + d + 1] = o[nt][1];
      mine[(gid + 8) * (D + 2) + d] = o[nt][2];
      mine[(gid + 8) * (D + 2) + d + 1] = o[nt][3];
    }
    if (tid4 == 0) {
      mine[gid * (D + 2) + D] = m[0];
      mine[gid * (D + 2) + D + 1] = l[0];
      mine[(gid + 8) * (D + 2) + D] = m[1];
      mine[(gid + 8) * (D + 2) + D + 1] = l[1];
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < g * D; e += AD_WARPS * 32) {
    const int r = e / D, d = e % D;
    float big = -INFINITY;
#pragma unroll
    for (int w = 0; w < AD_WARPS; ++w) big = fmaxf(big, merge[((size_t)w * 16 + r) * (D + 2) + D]);
    float acc = 0.f, den = 0.f;
    if (big != -INFINITY) {
#pragma unroll
      for (int w = 0; w < AD_WARPS; ++w) {
        const float* row = merge + ((size_t)w * 16 + r) * (D + 2);
        const float wgt = row[D] == -INFINITY ? 0.f : exp2f(row[D] - big);
        acc += row[d] * wgt;
        den += row[D + 1] * wgt;
      }
    }
    const int head = hk * g + r;
    if (num_splits == 1) {
      out[((size_t)tq * Hq + head) * D + d] = __float2bfloat16_rn(den > 0.f ? acc / den : 0.f);
    } else {
      float* p = partial + (((size_t)b * Hq + head) * num_splits + split) * (D + 2);
      p[d] = acc;
      if (d == 0) {
        p[D] = big;
        p[D + 1] = den;
      }
    }
  }
}

// Merges the splits of one (sequence, head): out = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M).
// The splits are dealt to the warps of the block, four at a time per warp with all their loads in flight
// together, and each lane owns pairs of output values.  A warp sums its splits relative to its own running
// maximum; the warps' sums are brought to the common maximum when they are added, so the kernel is one round
// trip to memory long for up to 4 x 8 splits.  D is even and at most 256.
constexpr int AC_WARPS = 8;
constexpr int AC_MAX_D = 256;
constexpr int AC_AT_ONCE = 4;

__global__ void __launch_bounds__(AC_WARPS * 32)
attn_combine_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out,
                    const int* __restrict__ q_start, int Hq, int D, int num_splits) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float acc_s[AC_WARPS][AC_MAX_D];
  __shared__ float den_s[AC_WARPS];
  __shared__ float max_s[AC_WARPS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.x, b = blockIdx.y;
  const float* base = partial + ((size_t)b * Hq + head) * num_splits * (D + 2);
  constexpr int PAIRS = AC_MAX_D / 64;
  // lane owns the value pairs d = 2 * lane + 64 * j; warp owns the splits warp, warp + AC_WARPS, ...
  float2 acc[PAIRS];
#pragma unroll
  for (int j = 0; j < PAIRS; ++j) acc[j] = make_float2(0.f, 0.f);
  float den = 0.f, mine = -INFINITY;  // relative to 2^mine
  for (int s0 = warp; s0 < num_splits; s0 += AC_WARPS * AC_AT_ONCE) {
    float2 ml[AC_AT_ONCE], v[AC_AT_ONCE][PAIRS];
#pragma unroll
    for (int u = 0; u < AC_AT_ONCE; ++u) {
      const int s = s0 + u * AC_WARPS;
      const float* row = base + (size_t)s * (D + 2);
      ml[u] = s < num_splits ? *reinterpret_cast<const float2*>(row + D) : make_float2(-INFINITY, 0.f);
#pragma unroll
      for (int j = 0; j < PAIRS; ++j) {
        const int d = 2 * lane + 64 * j;
        v[u][j] = (s < num_splits && d < D) ? *reinterpret_cast<const float2*>(row + d) : make_float2(0.f, 0.f);
      }
    }
    float top = mine;
#pragma unroll
    for (int u = 0; u < AC_AT_ONCE; ++u) top = fmaxf(top, ml[u].x);
    if (top == -INFINITY) continue;  // nothing but empty splits so far
    const float keep = mine == -INFINITY ? 0.f : exp2f(mine - top);
    den *= keep;
#pragma unroll
    for (int j = 0; j < PAIRS; ++j) {
      acc[j].x *= keep;
      acc[j].y *= keep;
    }
    mine = top;
#pragma unroll
    for (int u = 0; u < AC_AT_ONCE; ++u) {
      const float wgt = ml[u].x == -INFINITY ? 0.f : exp2f(ml[u].x - top);
      den += ml[u].y * wgt;
#pragma unroll
      for (int j = 0; j < PAIRS; ++j) {
        acc[j].x += v[u][j].x * wgt;
        acc[j].y += v[u][j].y * wgt;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < PAIRS; ++j) {
    const int d = 2 * lane + 64 * j;
    if (d < D) {
      acc_s[warp][d] = acc[j].x;
      acc_s[warp][d + 1] = acc[j].y;
    }
  }
  if (lane == 0) {
    den_s[warp] = den;
    max_s[warp] = mine;
  }
  __syncthreads();
  float big = max_s[0];
#pragma unroll
  for (int w = 1; w < AC_WARPS; ++w) big = fmaxf(big, max_s[w]);
  float scale_w[AC_WARPS], dn = 0.f;
#pragma unroll
  for (int w = 0; w < AC_WARPS; ++w) {
    scale_w[w] = max_s[w] == -INFINITY ? 0.f : exp2f(max_s[w] - big);
    dn += den_s[w] * scale_w[w];
  }
  const int tq = q_start[b];
  for (int d = threadIdx.x; d < D; d += AC_WARPS * 32) {
    float a = 0.f;
#pragma unroll
    for (int w = 0; w < AC_WARPS; ++w) a += acc_s[w][d] * scale_w[w];
    out[((size_t)tq * Hq + head) * D + d] = __float2bfloat16_rn(dn > 0.f ? a / dn : 0.f);
  }
}

template <int KT>
static int attn_decode_launch(const void* q, const void* k_pages, const void* v_pages, void* out, float* partial,
                              const int* q_start, const int* kv_len, const int* block_table, int table_stride,
                              int page_size, int num_pages, int B, int Hq, int Hkv, float scale, int window,
                              int num_splits, int* status, cudaStream_t stream) {
  using S = DecodeShape<KT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<KT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)S::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(num_splits, Hkv, B);
  q3::launch(attn_decode_kernel<KT>, dim3(grid), dim3(AD_WARPS * 32), S::SMEM_BYTES, stream, 
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, (__nv_bfloat16*)out,
      partial, q_start, kv_len, block_table, table_stride, page_size, page_shift_of(page_size), num_pages, Hq, Hkv,
      scale * 1.4426950408889634f, window, num_splits, status);
  int code = launch_status();
  if (code != 0 || num_splits == 1) return code;
  dim3 cgrid(Hq, B);
  g_launch_early = false;  // as in q3_attn_combine
  q3::launch(attn_combine_kernel, dim3(cgrid), dim3(AC_WARPS * 32), 0, stream, partial, (__nv_bfloat16*)out, q_start, Hq, S::D, num_splits);
  g_launch_early = true;
  return launch_status();
}

}  // namespace q3

// Streaming multiprocessors of the current device.
extern "C" int q3_sm_count() { return q3::sm_count(); }

// Blocks of the decode kernel for head size D that one SM holds at once, as the CUDA runtime reckons it from
// the compiled kernel's registers and shared memory (0: a head size the kernel does not take, or an error).
extern "C" int q3_attn_decode_blocks_per_sm(int D) {
  if (D % 16 || D < 16 || D > 256) return 0;
  int blocks = 0;
  cudaError_t e = cudaErrorInvalidValue;
#define Q3_AD_OCC(KT)                                                                                          \
  case KT: {                                                                                                   \
    using S = q3::DecodeShape<KT>;                                                                             \
    e = cudaFuncSetAttribute(q3::attn_decode_kernel<KT>, cudaFuncAttributeMaxDynamicSharedMemorySize,          \
                             (int)S::SMEM_BYTES);                                                              \
    if (e == cudaSuccess)                                                                                      \
      e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, q3::attn_decode_kernel<KT>, q3::AD_WARPS * 32, \
                                                        S::SMEM_BYTES);                                        \
    break;                                                                                                     \
  }
  switch (D / 16) {
    Q3_AD_OCC(1) Q3_AD_OCC(2) Q3_AD_OCC(3) Q3_AD_OCC(4) Q3_AD_OCC(5) Q3_AD_OCC(6) Q3_AD_OCC(7) Q3_AD_OCC(8)
    Q3_AD_OCC(9) Q3_AD_OCC(10) Q3_AD_OCC(11) Q3_AD_OCC(12) Q3_AD_OCC(13) Q3_AD_OCC(14) Q3_AD_OCC(15) Q3_AD_OCC(16)
  }
#undef Q3_AD_OCC
  return e == cudaSuccess ? blocks : 0;
}

// Decode attention for B sequences that each bring one query token.
// q, out: bf16 [T, Hq, D] (the token of sequence b is row q_start[b]); pages: bf16 [num_pages, Hkv, page_size, D];
// partial: float32 scratch of at least B * Hq * num_splits * (D + 2) elements (unused when num_splits == 1).
// Takes D in multiples of 16 up to 256 and up to 16 query heads per kv head; refuses the rest.
extern "C" int q3_attn_decode(const void* q, const void* k_pages, const void* v_pages, void* out, float* partial,
                              const int* q_start, const int* kv_len, const int* block_table, int table_stride,
                              int page_size, int num_pages, int B, int Hq, int Hkv, int D, float scale, int window,
                              int num_splits, int* status, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv || Hq / Hkv > 16 || D % 16 || D < 16 || D > 256 || page_size <= 0 || num_splits < 1 ||
      table_stride <= 0 || B > 65535 || Hkv > 65535)
    return Q3_ERR_SIZE;
  if ((uintptr_t)q % 16 || (uintptr_t)k_pages % 16 || (uintptr_t)v_pages % 16) return Q3_ERR_ALIGN;
#define Q3_AD_CASE(KT)                                                                                          \
  case KT:                                                                                                      \
    return q3::attn_decode_launch<KT>(q, k_pages, v_pages, out, partial, q_start, kv_len, block_table,          \
                                      table_stride, page_size, num_pages, B, Hq, Hkv, scale, window, num_splits, \
                                      status, stream);
  switch (D / 16) {
    Q3_AD_CASE(1) Q3_AD_CASE(2) Q3_AD_CASE(3) Q3_AD_CASE(4) Q3_AD_CASE(5) Q3_AD_CASE(6) Q3_AD_CASE(7) Q3_AD_CASE(8)
    Q3_AD_CASE(9) Q3_AD_CASE(10) Q3_AD_CASE(11) Q3_AD_CASE(12) Q3_AD_CASE(13) Q3_AD_CASE(14) Q3_AD_CASE(15)
    Q3_AD_CASE(16)
  }
#undef Q3_AD_CASE
  return Q3_ERR_SIZE;
}

// ---------------------------------------------------------------------------------------------
// Decode attention for callers that cannot allocate (declared in attn_decode_noalloc.h).
// The split-KV partials go to a fixed array that is part of the library image instead of a
// buffer the caller provides.
namespace q3 {

constexpr size_t NOALLOC_SCRATCH_FLOATS = (size_t)4 << 20;  // 4 Mi floats = 16 MiB, per GPU that loads the library
constexpr int NOALLOC_MAX_DEVICES = 64;

static __device__ __align__(256) float g_decode_scratch[NOALLOC_SCRATCH_FLOATS];

// In host code `g_decode_scratch` is only a handle for the symbol, not an address a kernel can use:
// the device address is asked from the runtime once per device and kept.
static float* g_decode_scratch_ptr[NOALLOC_MAX_DEVICES] = {nullptr};

static int noalloc_scratch(float** ptr) {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return (int)e;
  if (device < 0 || device >= NOALLOC_MAX_DEVICES) return Q3_ERR_SIZE;
  if (g_decode_scratch_ptr[device] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_decode_scratch);
    if (e != cudaSuccess) return (int)e;
    g_decode_scratch_ptr[device] = p;
  }
  *ptr = g_decode_scratch_ptr[device];
  return 0;
}

}  // namespace q3

extern "C" long long q3_attn_decode_noalloc_capacity(void) { return (long long)q3::NOALLOC_SCRATCH_FLOATS; }

extern "C" int q3_attn_decode_noalloc(const void* q, const void* k_pages, const void* v_pages, void* out,
                                      const int* q_start, const int* kv_len, const int* block_table,
                                      int table_stride, int page_size, int num_pages, int B, int Hq, int Hkv, int D,
                                      float scale, int window, int num_splits, int* status, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (num_splits < 1 || Hq <= 0 || D <= 0) return Q3_ERR_SIZE;
  float* scratch = nullptr;
  if (num_splits > 1) {
    const unsigned long long need = (unsigned long long)B * Hq * num_splits * (unsigned long long)(D + 2);
    if (need > q3::NOALLOC_SCRATCH_FLOATS) return Q3_ERR_SCRATCH;
    const int code = q3::noalloc_scratch(&scratch);
    if (code != 0) return code;
  }
  return q3_attn_decode(q, k_pages, v_pages, out, scratch, q_start, kv_len, block_table, table_stride, page_size,
                        num_pages, B, Hq, Hkv, D, scale, window, num_splits, status, stream);
}

// The merge of the splits alone, for other decode kernels that write the same partial records.
extern "C" int q3_attn_combine(const float* partial, void* out, const int* q_start, int B, int Hq, int D,
                               int num_splits, cudaStream_t stream) {
  if (B <= 0 || num_splits <= 1) return 0;
  if (D <= 0 || D > q3::AC_MAX_D || (D & 1)) return Q3_ERR_SIZE;
  dim3 cgrid(Hq, B);
  // The merge starts when the attention has completed, not early (the one ordinary launch of a decode step):
  // its blocks, resident and waiting while the attention still has blocks to place, took the places of those
  // blocks.  With 256 merge blocks beside a grid of two waves (the 8B sizes, batch 8 at a context of 16,384)
  // the attention ran twice as long and the step 28 % longer.
  q3::g_launch_early = false;
  q3::launch(q3::attn_combine_kernel, cgrid, dim3(q3::AC_WARPS * 32), 0, stream, partial, (__nv_bfloat16*)out, q_start, Hq, D,
             num_splits);
  q3::g_launch_early = true;
  return q3::launch_status();
}
