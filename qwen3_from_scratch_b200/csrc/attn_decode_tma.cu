// Paged decode attention with a TMA producer: the same split-KV scheme and tensor-core arithmetic
// as attn_decode.cu, but the key/value tiles are brought in by a dedicated loader warp through
// TMA (cp.async.bulk.tensor, 128-byte swizzle) into a ring of stages shared by the consumer warps
// (eight stages and four warps; six and three in the form for four blocks per SM).
// How many bytes are in flight no longer depends on how fast a consumer gets through its
// tile: the loader runs up to a ring of 16-key tiles (64 KB per block at D = 128) ahead, which is what
// a bandwidth-bound kernel wants, and the consumers issue no copy instructions at all.
//
// Takes D = 64 or 128 and page sizes that are multiples of 16 (a 16-key tile then lies in one
// page); everything else goes to attn_decode.cu.  Mbarrier waits are bounded (tc_common.cuh).
#include "attn_mma.cuh"
#include "tc_common.cuh"

extern "C" int q3_attn_combine(const float* partial, void* out, const int* q_start, int B, int Hq, int D,
                               int num_splits, cudaStream_t stream);

namespace q3 {

constexpr int DT_KEYS = 16;

// BLOCKS: blocks per SM the kernel is compiled for.  Two or three: four consumer warps and a ring of eight
// stages.  Four: three consumer warps and six stages, so that four blocks' registers (128 x 128 threads) and
// shared memory (53 KB) fit an SM.
template <int BLOCKS>
struct DecodeTmaBlock {
  static constexpr int CONSUMERS = BLOCKS >= 4 ? 3 : 4;
  static constexpr int THREADS = (CONSUMERS + 1) * 32;
  static constexpr int STAGES = BLOCKS >= 4 ? 6 : 8;
};

template <int D, int BLOCKS = 2>
struct DecodeTmaShape {
  using B = DecodeTmaBlock<BLOCKS>;
  static constexpr int ATOMS = D / 64;
  static constexpr int TILE_BYTES = DT_KEYS * D * 2;        // K (or V) of one tile: ATOMS atoms of 2048 bytes
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  static constexpr int RING_BYTES = B::STAGES * STAGE_BYTES;
  static constexpr int Q_PITCH = D + 8;
  static constexpr int Q_BYTES = 16 * Q_PITCH * 2;
  static constexpr int MERGE_BYTES = B::CONSUMERS * 16 * (D + 2) * 4;
  static constexpr int BAR_BYTES = 2 * B::STAGES * 8 + 16;
  static constexpr size_t SMEM_BYTES =
      (size_t)(RING_BYTES > MERGE_BYTES ? RING_BYTES : MERGE_BYTES) + Q_BYTES + BAR_BYTES;
};

// address of 16-byte chunk `chunk` of row `row` in a tile made of [16 x 64] atoms with the 128-byte swizzle
__device__ __forceinline__ const unsigned char* sw_chunk(const unsigned char* tile, int row, int chunk) {
  return tile + (chunk >> 3) * 2048 + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
}

// Eight values of a head (chunk c of its CPR chunks; the head's chunks are in CPR neighbouring lanes):
// x / sqrt(mean(x^2) + eps) * w if w is given, then y_i = x_i cos_i - x_(i + D/2) sin_i and
// y_(i + D/2) = x_(i + D/2) cos_i + x_i sin_i if the token's cosines and sines are given.  float32 throughout,
// one rounding to bfloat16 at the end, as in qkv_post.
template <int CPR>
__device__ __forceinline__ uint4 norm_rotate_chunk(uint4 raw, int c, const float* __restrict__ w,
                                                   const float* __restrict__ cos_sin, float eps) {
  constexpr int D = CPR * 8, HALF = CPR / 2;
  float x[8];
  const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    x[2 * k] = __uint_as_float(rw[k] << 16);
    x[2 * k + 1] = __uint_as_float(rw[k] & 0xffff0000u);
  }
  if (w != nullptr) {
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) ss += x[k] * x[k];
#pragma unroll
    for (int o = CPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rs = 1.0f / sqrtf(ss / (float)D + eps);
    const float4 w0 = *reinterpret_cast<const float4*>(w + c * 8), w1 = *reinterpret_cast<const float4*>(w + c * 8 + 4);
    const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int k = 0; k < 8; ++k) x[k] = x[k] * rs * wv[k];
  }
  if (cos_sin != nullptr) {
    const float* row = cos_sin + (c % HALF) * 8;
    const float4 c0 = *reinterpret_cast<const float4*>(row), c1 = *reinterpret_cast<const float4*>(row + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(row + D / 2), s1 = *reinterpret_cast<const float4*>(row + D / 2 + 4);
    const float cv[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    const float sign = c < HALF ? -1.0f : 1.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float partner = __shfl_xor_sync(0xffffffffu, x[k], HALF);
      x[k] = fmaf(partner, sign * sv[k], x[k] * cv[k]);
    }
  }
  return make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]), pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
}

// With `qkv` set the kernel does the work of qkv_post for its own token too (a step in which every row
// decodes): the query rows are normed and rotated from the raw projection as they are loaded, and the block
// whose range holds the sequence's last position norms and rotates the new key, copies the new value, writes
// both to their page and puts them into its own tile of shared memory, which the loader fetched without them.
// (Head norm: models/self_attn.py:388-401 of the reference; rotation of pairs (i, i + D / 2): models/rope.py.)
struct DecodeQkv {
  const __nv_bfloat16* qkv;  // [T, (Hq + 2 Hkv) * D] rows ordered q heads, k heads, v heads; null: q and the pages are ready
  const float* q_weight;     // [D] or null
  const float* k_weight;     // [D] or null
  const float* cos_sin;      // [T, D]: cosines then sines of the token's D / 2 angles, or null (no rotation)
  float eps;
  __nv_bfloat16* k_pages;    // the pools, for the new row
  __nv_bfloat16* v_pages;
  int write_kv;              // 0: another layer wrote this cache; only the query is made
  int angles_early;          // cos_sin is older than the launch before this one
};

// BLOCKS: blocks per SM the kernel is compiled for.  Three (128 registers) give a large grid half as many
// places again as two; two (168 registers) are the faster code where the grid fits their places anyway; four
// (smaller blocks, see DecodeTmaBlock) are for a grid of several waves, where more blocks per SM in different
// stages of their lives keep the SM's stream over the cache going
// (figures: profiles/attn_decode_tma__decode_b8_ctx4096.md).
template <int D, int BLOCKS>
__global__ void __launch_bounds__(DecodeTmaBlock<BLOCKS>::THREADS, BLOCKS)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                       float* __restrict__ partial, const int* __restrict__ q_start,
                       const int* __restrict__ kv_len, const int* __restrict__ block_table, int table_stride,
                       int page_size, int num_pages, int Hq, int Hkv, float scale_log2, int window,
                       int num_splits, int* status, const DecodeQkv fq) {
  using S = DecodeTmaShape<D, BLOCKS>;
  constexpr int KT = D / 16, CPR = D / 8, PITCH = S::Q_PITCH;
  constexpr int DT_CONSUMERS = DecodeTmaBlock<BLOCKS>::CONSUMERS, DT_STAGES = DecodeTmaBlock<BLOCKS>::STAGES;
  constexpr int DT_THREADS = DecodeTmaBlock<BLOCKS>::THREADS;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* ring = smem_raw;
  constexpr int RING_OR_MERGE = S::RING_BYTES > S::MERGE_BYTES ? S::RING_BYTES : S::MERGE_BYTES;
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw + RING_OR_MERGE);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw + RING_OR_MERGE + S::Q_BYTES);
  uint64_t* empty = full + DT_STAGES;
  int* abort_word = reinterpret_cast<int*>(empty + DT_STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tid4 = lane & 3;
  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int g = Hq / Hkv;
  const int tq = q_start[b];
  const int pos = kv_len[b] - 1;
  const int* table = block_table + (size_t)b * table_stride;

  int t_lo = 0, t_hi = 0, lo = 0;
  if (pos >= 0) {
    lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int first = lo / DT_KEYS, last = pos / DT_KEYS;
    const int per = (last - first + num_splits) / num_splits;
    t_lo = first + split * per;
    t_hi = min(t_lo + per, last + 1);
  } else if (threadIdx.x == 0) {
    atomicOr(status, Q3_STATUS_BAD_POSITION);
  }
  const int count = max(0, t_hi - t_lo);

  if (warp == DT_CONSUMERS && lane == 0) {
    tma_prefetch_map(&map_k);
    tma_prefetch_map(&map_v);
  }
  if (threadIdx.x == 0) {
    *abort_word = (s_addr(smem_raw) & 1023u) ? 1 : 0;
    if (*abort_word) atomicOr(status, Q3_STATUS_TIMEOUT);
    for (int s = 0; s < DT_STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();  // the barriers exist
  // Keys and values of earlier steps are in memory already, and the lengths and tables were copied
  // before the step's first kernel: the loader starts on them at once, while the kernel before this
  // one (which writes this step's key, value and query) may still be running.  Only the tile that
  // holds the sequence's last position, and the query, wait for that kernel.
  if (warp != DT_CONSUMERS) {
    if (fq.qkv != nullptr) {
      // the norm weights, which no kernel writes, and the token's cosines and sines, if the launch before this
      // one did not write them, are asked into L1 ahead of the wait (D floats each: D / 32 lines of 128 bytes)
      constexpr int LINES = D / 32;
      const int which = threadIdx.x / LINES, line = threadIdx.x % LINES;
      const float* base = which == 0 ? fq.q_weight : which == 1 ? fq.k_weight
                          : (which == 2 && fq.angles_early && fq.cos_sin) ? fq.cos_sin + (size_t)tq * D : nullptr;
      if (base != nullptr) asm volatile("prefetch.global.L1 [%0];" ::"l"(base + line * 32));
    }
    pdl_wait();
    pdl_launch_dependents();
    for (int e = threadIdx.x; e < 16 * CPR; e += DT_CONSUMERS * 32) {
      const int row = e / CPR, c = e % CPR;  // a row's CPR chunks of eight values sit in neighbouring lanes
      uint4 v = make_uint4(0, 0, 0, 0);
      if (fq.qkv == nullptr) {
        if (row < g) v = *reinterpret_cast<const uint4*>(q + ((size_t)tq * Hq + hk * g + row) * D + c * 8);
      } else {
        // the raw projection's head hk * g + row: head norm, then rotation (every lane takes part in the shuffles)
        if (row < g) v = *reinterpret_cast<const uint4*>(fq.qkv + ((size_t)tq * (Hq + 2 * Hkv) + hk * g + row) * D + c * 8);
        v = norm_rotate_chunk<CPR>(v, c, fq.q_weight, fq.cos_sin ? fq.cos_sin + (size_t)tq * D : nullptr, fq.eps);
      }
      *reinterpret_cast<uint4*>(q_s + row * PITCH + c * 8) = v;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(DT_CONSUMERS * 32) : "memory");
  }

  float o[2 * KT][4];
#pragma unroll
  for (int i = 0; i < 2 * KT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  if (warp == DT_CONSUMERS) {
    // ------------------------------------------------------------------ loader
    bool ok = true;
    // tiles [i_lo, i_hi) of this block's range; the wait for the kernel before lies between two such
    // runs, not inside the loop
    auto issue = [&](int i_lo, int i_hi) {
      for (int chunk0 = i_lo; chunk0 < i_hi; chunk0 += 32) {
        // thirty-two page ids at once, one per lane
        int my_y = -1;
        if (chunk0 + lane < i_hi) {
          const int n0 = (t_lo + chunk0 + lane) * DT_KEYS;
          int page = table_page(table, n0 / page_size, table_stride, status);
          if (page < 0 || page >= num_pages) {
            atomicOr(status, Q3_STATUS_BAD_PAGE);
            page = 0;
          }
          my_y = (page * Hkv + hk) * page_size + (n0 % page_size);
        }
        const int in_chunk = min(32, i_hi - chunk0);
        for (int u = 0; u < in_chunk; ++u) {
          const int i = chunk0 + u;
          const int s = i % DT_STAGES;
          const uint32_t use = (uint32_t)i / DT_STAGES;
          const int y = __shfl_sync(0xffffffffu, my_y, u);
          if (use > 0) ok = ok && mbar_wait(empty + s, (use - 1) & 1, abort_word);
          if (lane == 0 && ok && i != tc_drop_copy) {  // (the test of the give-up path drops one copy: see tc_common.cuh)
            unsigned char* stage = ring + (size_t)s * S::STAGE_BYTES;
            mbar_expect_tx(full + s, S::STAGE_BYTES);
#pragma unroll
            for (int a = 0; a < S::ATOMS; ++a) {
              tma_load_2d(stage + a * 2048, &map_k, full + s, a * 64, y);
              tma_load_2d(stage + S::TILE_BYTES + a * 2048, &map_v, full + s, a * 64, y);
            }
          }
        }
      }
    };
    // this step's key and value are written into tile pos / 16 by the kernel before: everything
    // before that tile can be fetched while that kernel still runs
    const int early_tiles = min(count, max(0, pos / DT_KEYS - t_lo));
    issue(0, early_tiles);
    pdl_wait();
    pdl_launch_dependents();  // after the wait, as everywhere: the next kernel never starts before the one before this ended
    issue(early_tiles, count);
    if (!ok && lane == 0) {
      *abort_word = 1;
      atomicOr(status, Q3_STATUS_TIMEOUT);
    }
  } else {
    // ------------------------------------------------------------------ consumers
    uint32_t qa[KT][4];
#pragma unroll
    for (int kt = 0; kt < KT; ++kt)
      ldmatrix_x4(qa[kt], q_s + ((lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + kt * 16 + (lane >> 4) * 8);
    bool ok = true;
    for (int i = warp; i < count; i += DT_CONSUMERS) {
      const int s = i % DT_STAGES;
      // (no short cut once a wait has run out: a copy that the loader did issue is still waited for, within
      // the limit, before its stage is read and handed back)
      ok = mbar_wait(full + s, ((uint32_t)i / DT_STAGES) & 1, abort_word) && ok;
      const unsigned char* k_t = ring + (size_t)s * S::STAGE_BYTES;
      unsigned char* v_t = ring + (size_t)s * S::STAGE_BYTES + S::TILE_BYTES;
      const int base_n = (t_lo + i) * DT_KEYS;
      const bool edge = base_n < lo || base_n + DT_KEYS - 1 > pos;
      if (fq.qkv != nullptr && fq.write_kv && t_lo + i == pos / DT_KEYS) {
        // this step's key and value: made here from the raw projection, written to their page for the steps
        // to come and into this tile, which was fetched without them.  A lane holds D / 32 neighbouring values.
        constexpr int VPL = D / 32;
        const int r = pos - base_n, first = VPL * lane;
        const __nv_bfloat16* k_raw = fq.qkv + ((size_t)tq * (Hq + 2 * Hkv) + Hq + hk) * D + first;
        const __nv_bfloat16* v_raw = k_raw + (size_t)Hkv * D;
        __nv_bfloat16 kn[VPL], vn[VPL];
        float x[VPL];
#pragma unroll
        for (int k = 0; k < VPL; ++k) {
          x[k] = __bfloat162float(k_raw[k]);
          vn[k] = v_raw[k];
        }
        if (fq.k_weight != nullptr) {
          float ss = 0.f;
#pragma unroll
          for (int k = 0; k < VPL; ++k) ss += x[k] * x[k];
          ss = warp_sum(ss);
          const float rs = 1.0f / sqrtf(ss / (float)D + fq.eps);
#pragma unroll
          for (int k = 0; k < VPL; ++k) x[k] = x[k] * rs * fq.k_weight[first + k];
        }
        if (fq.cos_sin != nullptr) {
          const float* cs = fq.cos_sin + (size_t)tq * D + (first % (D / 2));
          const float sign = lane < 16 ? -1.0f : 1.0f;
#pragma unroll
          for (int k = 0; k < VPL; ++k) {
            const float partner = __shfl_xor_sync(0xffffffffu, x[k], 16);
            x[k] = fmaf(partner, sign * cs[D / 2 + k], x[k] * cs[k]);
          }
        }
#pragma unroll
        for (int k = 0; k < VPL; ++k) kn[k] = __float2bfloat16_rn(x[k]);
        const int chunk = first >> 3;
        const size_t in_tile = (size_t)(chunk >> 3) * 2048 + r * 128 + (((chunk & 7) ^ (r & 7)) << 4) + (first & 7) * 2;
        const int page = table_page(table, pos / page_size, table_stride, status);
        const bool page_ok = page >= 0 && page < num_pages;
        if (!page_ok && lane == 0) atomicOr(status, Q3_STATUS_BAD_PAGE);
        const size_t in_pool = (((size_t)(page_ok ? page : 0) * Hkv + hk) * page_size + pos % page_size) * D + first;
        if (VPL == 4) {
          const uint2 kp = *reinterpret_cast<const uint2*>(kn), vp = *reinterpret_cast<const uint2*>(vn);
          *reinterpret_cast<uint2*>(const_cast<unsigned char*>(k_t) + in_tile) = kp;
          *reinterpret_cast<uint2*>(v_t + in_tile) = vp;
          if (page_ok) {
            *reinterpret_cast<uint2*>(fq.k_pages + in_pool) = kp;
            *reinterpret_cast<uint2*>(fq.v_pages + in_pool) = vp;
          }
        } else {
          const uint32_t kp = *reinterpret_cast<const uint32_t*>(kn), vp = *reinterpret_cast<const uint32_t*>(vn);
          *reinterpret_cast<uint32_t*>(const_cast<unsigned char*>(k_t) + in_tile) = kp;
          *reinterpret_cast<uint32_t*>(v_t + in_tile) = vp;
          if (page_ok) {
            *reinterpret_cast<uint32_t*>(fq.k_pages + in_pool) = kp;
            *reinterpret_cast<uint32_t*>(fq.v_pages + in_pool) = vp;
          }
        }
        fence_async_proxy();
        __syncwarp();
      }
      if (base_n + DT_KEYS - 1 > pos) {
        // the page's slots past the sequence hold whatever was there: zero those value rows
        const int first_bad = pos - base_n + 1;
        for (int e = lane; e < (DT_KEYS - first_bad) * CPR; e += 32) {
          const int row = first_bad + e / CPR, c = e % CPR;
          *reinterpret_cast<uint4*>(v_t + (c >> 3) * 2048 + row * 128 + ((c & 7) << 4)) = make_uint4(0, 0, 0, 0);
        }
        fence_async_proxy();  // these stores are ordered before the loader's next copy into this stage
        __syncwarp();
      }
      float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int kt = 0; kt < KT; ++kt) {
        uint32_t kb[4];
        ldmatrix_x4(kb, sw_chunk(k_t, (lane & 7) + ((lane >> 4) << 3), kt * 2 + ((lane >> 3) & 1)));
        mma_bf16(sc[0], qa[kt], kb[0], kb[1]);
        mma_bf16(sc[1], qa[kt], kb[2], kb[3]);
      }
      if (edge) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int n = base_n + nt * 8 + 2 * tid4 + (j & 1);
            if (n < lo || n > pos) sc[nt][j] = -INFINITY;
          }
      }
      float mx[2];
      mx[0] = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1]));
      mx[1] = fmaxf(fmaxf(sc[0][2], sc[0][3]), fmaxf(sc[1][2], sc[1][3]));
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
          const float p0 = exp2f(fmaf(sc[nt][2 * r], scale_log2, -m_use[r]));
          const float p1 = exp2f(fmaf(sc[nt][2 * r + 1], scale_log2, -m_use[r]));
          sc[nt][2 * r] = p0;
          sc[nt][2 * r + 1] = p1;
          l[r] += p0 + p1;
        }
      uint32_t pa[4];
      pa[0] = pack_bf16(sc[0][0], sc[0][1]);
      pa[1] = pack_bf16(sc[0][2], sc[0][3]);
      pa[2] = pack_bf16(sc[1][0], sc[1][1]);
      pa[3] = pack_bf16(sc[1][2], sc[1][3]);
#pragma unroll
      for (int dt = 0; dt < KT; ++dt) {
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, sw_chunk(v_t, (lane & 7) + ((lane >> 3) & 1) * 8, dt * 2 + (lane >> 4)));
        mma_bf16(o[2 * dt], pa, vb[0], vb[1]);
        mma_bf16(o[2 * dt + 1], pa, vb[2], vb[3]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty + s);  // the stage goes back to the loader
    }
    if (!ok && lane == 0) {
      *abort_word = 1;
      atomicOr(status, Q3_STATUS_TIMEOUT);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
  }
  __syncthreads();  // every tile has been consumed: the ring now holds the merge buffers

  float* merge = reinterpret_cast<float*>(ring);  // [consumer][16 rows][D + 2]
  if (warp < DT_CONSUMERS) {
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
  for (int e = threadIdx.x; e < g * D; e += DT_THREADS) {
    const int r = e / D, d = e % D;
    float big = -INFINITY;
#pragma unroll
    for (int w = 0; w < DT_CONSUMERS; ++w) big = fmaxf(big, merge[((size_t)w * 16 + r) * (D + 2) + D]);
    float acc = 0.f, den = 0.f;
    if (big != -INFINITY) {
#pragma unroll
      for (int w = 0; w < DT_CONSUMERS; ++w) {
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

template <int D>
static int attn_decode_tma_launch(const void* q, const void* k_pages, const void* v_pages, void* out, float* partial,
                                  const int* q_start, const int* kv_len, const int* block_table, int table_stride,
                                  int page_size, int num_pages, int B, int Hq, int Hkv, float scale, int window,
                                  int num_splits, int* status, cudaStream_t stream, DecodeQkv fq = DecodeQkv{}) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_tma_kernel<D, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)DecodeTmaShape<D, 2>::SMEM_BYTES);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_decode_tma_kernel<D, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)DecodeTmaShape<D, 3>::SMEM_BYTES);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_decode_tma_kernel<D, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)DecodeTmaShape<D, 4>::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  CUtensorMap map_k, map_v;
  const uint64_t rows = (uint64_t)num_pages * Hkv * page_size;
  int code = cached_map(&map_k, k_pages, rows, D, DT_KEYS);
  if (code) return code;
  code = cached_map(&map_v, v_pages, rows, D, DT_KEYS);
  if (code) return code;
  dim3 grid(num_splits, Hkv, B);
  const long long blocks = (long long)num_splits * Hkv * B;
  // two blocks per SM where the grid fits them, three where it fits those, four for a grid of several waves
  const int per_sm = blocks <= 2LL * sm_count() ? 2 : blocks <= 3LL * sm_count() ? 3 : 4;
#define Q3_DT_LAUNCH(BL)                                                                                              \
  q3::launch(attn_decode_tma_kernel<D, BL>, grid, dim3(DecodeTmaBlock<BL>::THREADS), DecodeTmaShape<D, BL>::SMEM_BYTES,  \
             stream, map_k, map_v, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, partial, q_start, kv_len, block_table, \
             table_stride, page_size, num_pages, Hq, Hkv, scale * 1.4426950408889634f, window, num_splits, status, fq)
  if (per_sm == 2) Q3_DT_LAUNCH(2);
  else if (per_sm == 3) Q3_DT_LAUNCH(3);
  else Q3_DT_LAUNCH(4);
#undef Q3_DT_LAUNCH
  code = launch_status();
  if (code != 0 || num_splits == 1) return code;
  return q3_attn_combine(partial, out, q_start, B, Hq, D, num_splits, stream);
}

}  // namespace q3

// For the tests of the give-up path: see set_wait_test in tc_common.cuh.
extern "C" int q3_attn_decode_tma_wait_test(unsigned limit, int drop) { return q3::set_wait_test(limit, drop); }

// Same arguments as q3_attn_decode.  Takes D = 64 or 128, page sizes that are multiples of 16 and up to
// 16 query heads per kv head; refuses the rest.
extern "C" int q3_attn_decode_tma(const void* q, const void* k_pages, const void* v_pages, void* out, float* partial,
                                  const int* q_start, const int* kv_len, const int* block_table, int table_stride,
                                  int page_size, int num_pages, int B, int Hq, int Hkv, int D, float scale,
                                  int window, int num_splits, int* status, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv || Hq / Hkv > 16 || (D != 64 && D != 128) || page_size <= 0 || page_size % 16 ||
      num_splits < 1 || table_stride <= 0 || B > 65535 || Hkv > 65535)
    return Q3_ERR_SIZE;
  if ((uintptr_t)q % 16 || (uintptr_t)k_pages % 16 || (uintptr_t)v_pages % 16) return Q3_ERR_ALIGN;
  if (D == 64)
    return q3::attn_decode_tma_launch<64>(q, k_pages, v_pages, out, partial, q_start, kv_len, block_table,
                                          table_stride, page_size, num_pages, B, Hq, Hkv, scale, window, num_splits,
                                          status, stream);
  return q3::attn_decode_tma_launch<128>(q, k_pages, v_pages, out, partial, q_start, kv_len, block_table,
                                         table_stride, page_size, num_pages, B, Hq, Hkv, scale, window, num_splits,
                                         status, stream);
}

// The same with the work of q3_qkv_post for a step in which every row brings one token (see DecodeQkv):
// qkv [T, (Hq + 2 Hkv) * D] bfloat16 is the raw projection (token of sequence b: row q_start[b]), q_weight and
// k_weight float32 [D] or null, cos_sin float32 [T, D] from q3_rope_table or null; the new key and value go to
// k_pages / v_pages unless write_kv is 0.  No q is read.
extern "C" int q3_attn_decode_tma_qkv(const void* qkv, const float* q_weight, const float* k_weight, float eps,
                                      const float* cos_sin, int write_kv, void* k_pages, void* v_pages, void* out,
                                      float* partial, const int* q_start, const int* kv_len, const int* block_table,
                                      int table_stride, int page_size, int num_pages, int B, int Hq, int Hkv, int D,
                                      float scale, int window, int num_splits, int* status, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv || Hq / Hkv > 16 || (D != 64 && D != 128) || page_size <= 0 || page_size % 16 ||
      num_splits < 1 || table_stride <= 0 || B > 65535 || Hkv > 65535 || !qkv)
    return Q3_ERR_SIZE;
  if ((uintptr_t)qkv % 16 || (uintptr_t)k_pages % 16 || (uintptr_t)v_pages % 16 || (uintptr_t)q_weight % 16 ||
      (uintptr_t)k_weight % 16 || (uintptr_t)cos_sin % 16)
    return Q3_ERR_ALIGN;
  q3::DecodeQkv fq{};
  fq.qkv = (const __nv_bfloat16*)qkv;
  fq.q_weight = q_weight;
  fq.k_weight = k_weight;
  fq.cos_sin = cos_sin;
  fq.eps = eps;
  fq.k_pages = (__nv_bfloat16*)k_pages;
  fq.v_pages = (__nv_bfloat16*)v_pages;
  fq.write_kv = write_kv;
  fq.angles_early = q3::last_launch_was_plain(stream) ? 1 : 0;
  if (D == 64)
    return q3::attn_decode_tma_launch<64>(nullptr, k_pages, v_pages, out, partial, q_start, kv_len, block_table,
                                          table_stride, page_size, num_pages, B, Hq, Hkv, scale, window, num_splits,
                                          status, stream, fq);
  return q3::attn_decode_tma_launch<128>(nullptr, k_pages, v_pages, out, partial, q_start, kv_len, block_table,
                                         table_stride, page_size, num_pages, B, Hq, Hkv, scale, window, num_splits,
                                         status, stream, fq);
}
