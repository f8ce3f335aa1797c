// After the merged QKV projection, in one pass over the packed [T, (Hq + 2 Hkv) D] rows:
//   * per-head RMSNorm of every q and k head vector (weights shared by the heads),
//   * rotary position encoding of q and k (rotate-half pairing),
//   * q goes to a dense [T, Hq, D] buffer, k and v go straight into their cache pages.
// All arithmetic is float32 (statistics, angle = pos * inv_freq, sin/cos, rotation);
// each value is rounded once, when it is stored.
//
// Reference formulas: models/self_attn.py:319-336 (order: norm, then rotation; v untouched),
// models/rotary.py:13-22 (y1 = x1 cos - x2 sin, y2 = x2 cos + x1 sin, halves of the head),
// models/rotary.py:36-45 (angle = position * theta^(-2j/D)),
// inference/kv_cache/paged_cache.py:85-118 (slot of a position in its page).
//
// Cache layout of one layer: K and V each [num_pages, Hkv, page_size, D]; a page's
// keys of one head are contiguous.
#include "common.cuh"

#ifndef Q3_QPV_MANY
#define Q3_QPV_MANY 2  // warps per block of the bfloat16 fast path when there are many tokens
#endif

namespace q3 {

constexpr int QP_WARPS = 4;
constexpr int QP_MAX_D = 512;

template <typename T>
__global__ void __launch_bounds__(QP_WARPS * 32)
qkv_post_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ k_pages,
                T* __restrict__ v_pages, const float* __restrict__ q_weight,
                const float* __restrict__ k_weight, const float* __restrict__ inv_freq,
                const int* __restrict__ positions, const int* __restrict__ tok_seq,
                const int* __restrict__ block_table, int table_stride, int page_size, int num_pages,
                int Hq, int Hkv, int D, int rotary_dim, float eps, int write_kv, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float vec[QP_WARPS][QP_MAX_D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int head = blockIdx.y * QP_WARPS + warp;
  const int n_heads = Hq + 2 * Hkv;
  if (head >= n_heads) return;
  const bool is_q = head < Hq;
  const bool is_k = !is_q && head < Hq + Hkv;
  if (!is_q && !write_kv) return;

  const int pos = positions[t];
  const T* src = qkv + ((size_t)t * n_heads + head) * D;
  float* x = vec[warp];
  float ss = 0.f;
  for (int e = lane; e < D; e += 32) {
    const float v = to_float(src[e]);
    x[e] = v;
    ss += v * v;
  }
  ss = warp_sum(ss);
  __syncwarp();

  const float* w = is_q ? q_weight : (is_k ? k_weight : nullptr);
  const bool rotate = (is_q || is_k) && inv_freq != nullptr;
  const float rs = w ? 1.0f / sqrtf(ss / (float)D + eps) : 1.0f;

  T* dst;
  if (is_q) {
    dst = q_out + ((size_t)t * Hq + head) * D;
  } else {
    const int seq = tok_seq[t];
    if (pos < 0 || seq < 0) {
      if (lane == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
      return;
    }
    const int page = table_page(block_table + (size_t)seq * table_stride, pos / page_size, table_stride, status);
    if (page < 0 || page >= num_pages) {
      if (lane == 0) atomicOr(status, Q3_STATUS_BAD_PAGE);
      return;
    }
    const int hk = is_k ? head - Hq : head - Hq - Hkv;
    T* base = is_k ? k_pages : v_pages;
    dst = base + (((size_t)page * Hkv + hk) * page_size + (pos % page_size)) * D;
  }

  const int half = rotary_dim >> 1;
  for (int e = lane; e < D; e += 32) {
    float v = x[e];
    if (w) v = v * rs * w[e];
    if (rotate && e < rotary_dim) {
      const int j = e < half ? e : e - half;
      const int pe = e < half ? e + half : e - half;
      float partner = x[pe];
      if (w) partner = partner * rs * w[pe];
      float s, c;
      sincosf((float)pos * inv_freq[j], &s, &c);
      v = e < half ? v * c - partner * s : v * c + partner * s;
    }
    dst[e] = from_float<T>(v);
  }
}

// Sines and cosines of a step's tokens: table[t, j] = cos(pos_t * inv_freq[j]), table[t, half + j] = sin(...).
// Computed once per step and read by every layer's qkv_post, instead of once per layer and token.
__global__ void rope_table_kernel(const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                  float* __restrict__ table, int T, int half) {
  pdl_wait();
  pdl_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * half) return;
  const int t = i / half, j = i % half;
  float sn, c;
  sincosf((float)positions[t] * inv_freq[j], &sn, &c);
  table[(size_t)t * 2 * half + j] = c;
  table[(size_t)t * 2 * half + half + j] = sn;
}

// The same as qkv_post_kernel for bfloat16 when D is 16, 32, 64, 128 or 256, the whole head is
// rotated and the step's table of sines and cosines is given.  A head is served by LPH = D / 8
// neighbouring lanes, each owning eight consecutive values (one 16-byte load and store), so a warp
// works on 32 / LPH heads at once; the rotation partner of a lane is LPH / 2 lanes away.  No shared
// memory and no block-wide barrier.
constexpr int QPV_UNROLL = 2;

// QPV_WARPS: warps per block: few for many tokens (small blocks come and go quickly and keep more loads
// in flight per SM), eight for a few tokens (all heads of a token at once).
template <int LPH, int QPV_WARPS>
__global__ void __launch_bounds__(QPV_WARPS * 32, 1024 / (QPV_WARPS * 32))
qkv_post_vec_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                    __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages,
                    const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                    const float* __restrict__ cos_sin, const int* __restrict__ positions,
                    const int* __restrict__ tok_seq, const int* __restrict__ block_table, int table_stride,
                    int page_size, int num_pages, int Hq, int Hkv, float eps, int write_kv, int heads_per_block,
                    int* status) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int D = 8 * LPH, HPW = 32 / LPH, HALF = LPH / 2;
  // A block serves one token and the heads [blockIdx.y * heads_per_block, + heads_per_block) (all
  // heads of the token when there are many tokens, a few when there are few tokens).
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int n_heads = Hq + 2 * Hkv;
  const int sub = lane / LPH, l = lane % LPH;
  const int head_end = min(n_heads, (int)(blockIdx.y + 1) * heads_per_block);
  constexpr int STEP = QPV_WARPS * HPW * QPV_UNROLL;  // heads a block takes in one pass
  // The values of a pass are asked for before anything else, so that their latency runs beside the
  // token's table lookups; the next pass is asked for before the current one is worked on.
  uint4 raw[QPV_UNROLL];
  auto fetch = [&](int head0) {
#pragma unroll
    for (int u = 0; u < QPV_UNROLL; ++u) {
      const int head = head0 + (u * QPV_WARPS + warp) * HPW + sub;
      raw[u] = make_uint4(0, 0, 0, 0);
      if (head < head_end && (head < Hq || write_kv))
        raw[u] = *reinterpret_cast<const uint4*>(qkv + ((size_t)t * n_heads + head) * D + l * 8);
    }
  };
  fetch(blockIdx.y * heads_per_block);

  long long kv_off = -1;  // element offset of the token's row in a page array (every thread finds the same)
  if (write_kv) {
    const int pos = positions[t], seq = tok_seq[t];
    if (pos < 0 || seq < 0) {
      if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
    } else {
      const int page = table_page(block_table + (size_t)seq * table_stride, pos / page_size, table_stride, status);
      if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_PAGE);
      } else {
        kv_off = ((long long)page * Hkv * page_size + (pos % page_size)) * D;
      }
    }
  }
  float cv[8], sv[8];
  if (cos_sin != nullptr) {
    const float* row = cos_sin + (size_t)t * D + (l % HALF) * 8;  // the lane's eight pairs
    const float4 c0 = *reinterpret_cast<const float4*>(row), c1 = *reinterpret_cast<const float4*>(row + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(row + D / 2), s1 = *reinterpret_cast<const float4*>(row + D / 2 + 4);
    cv[0] = c0.x; cv[1] = c0.y; cv[2] = c0.z; cv[3] = c0.w; cv[4] = c1.x; cv[5] = c1.y; cv[6] = c1.z; cv[7] = c1.w;
    sv[0] = s0.x; sv[1] = s0.y; sv[2] = s0.z; sv[3] = s0.w; sv[4] = s1.x; sv[5] = s1.y; sv[6] = s1.z; sv[7] = s1.w;
    // y = x cos - partner sin in the first half of the head, x cos + partner sin in the second: the sign goes
    // into the sine once, so that the rotation is one multiply and one fused multiply-add per value
    if (l < HALF) {
#pragma unroll
      for (int k = 0; k < 8; ++k) sv[k] = -sv[k];
    }
  }
  for (int head0 = blockIdx.y * heads_per_block; head0 < head_end; head0 += STEP) {
    uint4 cur[QPV_UNROLL];
#pragma unroll
    for (int u = 0; u < QPV_UNROLL; ++u) cur[u] = raw[u];
    if (head0 + STEP < head_end) fetch(head0 + STEP);
#pragma unroll
    for (int u = 0; u < QPV_UNROLL; ++u) {
      const int head = head0 + (u * QPV_WARPS + warp) * HPW + sub;
      if (head0 + (u * QPV_WARPS + warp) * HPW >= head_end) break;  // uniform over the warp
      const bool live = head < head_end && (head < Hq || kv_off >= 0);
      const bool is_q = head < Hq;
      const bool is_k = !is_q && head < Hq + Hkv;
      uint4 packed = cur[u];
      // values (v) heads are copied as they are; a warp that holds only such heads skips the arithmetic
      if (__any_sync(0xffffffffu, is_q || is_k)) {
        float x[8];
        const uint32_t rw[4] = {cur[u].x, cur[u].y, cur[u].z, cur[u].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          x[2 * k] = __uint_as_float(rw[k] << 16);
          x[2 * k + 1] = __uint_as_float(rw[k] & 0xffff0000u);
        }
        // every lane takes part in the shuffles; what a lane without a q or k head computes is dropped
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) ss += x[k] * x[k];
#pragma unroll
        for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float* w = is_q ? q_weight : (is_k ? k_weight : nullptr);
        if (w) {
          const float rs = 1.0f / sqrtf(ss / (float)D + eps);
          const float4 w0 = *reinterpret_cast<const float4*>(w + l * 8), w1 = *reinterpret_cast<const float4*>(w + l * 8 + 4);
          const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
          for (int k = 0; k < 8; ++k) x[k] = x[k] * rs * wv[k];
        }
        if (cos_sin != nullptr) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float partner = __shfl_xor_sync(0xffffffffu, x[k], HALF);
            x[k] = fmaf(partner, sv[k], x[k] * cv[k]);
          }
        }
        if (is_q || is_k) {
          uint32_t o[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            __nv_bfloat162 p2 = __floats2bfloat162_rn(x[2 * k], x[2 * k + 1]);
            o[k] = *reinterpret_cast<uint32_t*>(&p2);
          }
          packed = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
      if (!live) continue;
      __nv_bfloat16* dst;
      if (is_q) {
        dst = q_out + ((size_t)t * Hq + head) * D;
      } else {
        const int hk = is_k ? head - Hq : head - Hq - Hkv;
        dst = (is_k ? k_pages : v_pages) + kv_off + (size_t)hk * page_size * D;
      }
      *reinterpret_cast<uint4*>(dst + l * 8) = packed;
    }
  }
}

}  // namespace q3

// qkv: [T, (Hq + 2 Hkv) * D] in `dtype`, rows ordered q heads, k heads, v heads.
// q_out: [T, Hq, D].  k_pages / v_pages: [num_pages, Hkv, page_size, D].
// q_weight / k_weight: float32 [D] or null (no head norm).  inv_freq: float32 [rotary_dim / 2]
// or null (no rotation).  cos_sin: float32 [T, rotary_dim] from q3_rope_table for the same positions and
// inv_freq, or null (the angles are then computed here).  positions, tok_seq: int32 [T] (absolute position, row of the block table).
// write_kv == 0: only q is produced (a layer that reads a cache another layer wrote).
// Refuses D > 512 or odd rotary_dim or rotary_dim > D.
extern "C" int q3_qkv_post(const void* qkv, int dtype, int T, int Hq, int Hkv, int D,
                           const float* q_weight, const float* k_weight, float eps,
                           const float* inv_freq, const float* cos_sin, int rotary_dim, const int* positions,
                           const int* tok_seq, const int* block_table, int table_stride,
                           int page_size, void* k_pages, void* v_pages, int num_pages, void* q_out,
                           int write_kv, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D <= 0 || D > q3::QP_MAX_D || (rotary_dim & 1) || rotary_dim > D || rotary_dim < 0) return Q3_ERR_SIZE;
  if (page_size <= 0 || table_stride <= 0) return Q3_ERR_SIZE;
  const int n_heads = Hq + 2 * Hkv;
  dim3 grid(T, (n_heads + q3::QP_WARPS - 1) / q3::QP_WARPS);
  if (grid.y > 65535) return Q3_ERR_SIZE;
  const bool whole_rotation = inv_freq == nullptr || rotary_dim == D;
  // few tokens: one pass of a block's warps (eight warps x 256 / D heads), so that more blocks share the work
  const int warps = T >= 256 ? Q3_QPV_MANY : 8;
  const int heads_per_block = T >= 256 ? n_heads : warps * (D <= 256 ? 256 / D : 1);
  if (dtype == Q3_BF16 && whole_rotation && (inv_freq == nullptr || cos_sin != nullptr) && (uintptr_t)cos_sin % 16 == 0 &&
      (D == 16 || D == 32 || D == 64 || D == 128 || D == 256) &&
      (q_weight == nullptr || (uintptr_t)q_weight % 16 == 0) && (k_weight == nullptr || (uintptr_t)k_weight % 16 == 0) &&
      (uintptr_t)qkv % 16 == 0 && (uintptr_t)q_out % 16 == 0 && (uintptr_t)k_pages % 16 == 0 &&
      (uintptr_t)v_pages % 16 == 0) {
#define Q3_QP_VEC_W(LPH, W)                                                                                       \
  q3::launch(q3::qkv_post_vec_kernel<LPH, W>, dim3(T, (n_heads + heads_per_block - 1) / heads_per_block),        \
             dim3(W * 32), 0, stream,                                                                             \
      (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, q_weight, \
      k_weight, inv_freq ? cos_sin : nullptr, positions, tok_seq, block_table, table_stride, page_size, num_pages, \
      Hq, Hkv, eps, write_kv, heads_per_block, status)
#define Q3_QP_VEC(LPH)                   \
  do {                                   \
    if (warps == 8) Q3_QP_VEC_W(LPH, 8); \
    else Q3_QP_VEC_W(LPH, Q3_QPV_MANY);  \
  } while (0)
    if (D == 16) Q3_QP_VEC(2);
    else if (D == 32) Q3_QP_VEC(4);
    else if (D == 64) Q3_QP_VEC(8);
    else if (D == 128) Q3_QP_VEC(16);
    else Q3_QP_VEC(32);
#undef Q3_QP_VEC
#undef Q3_QP_VEC_W
    return q3::launch_status();
  }
  if (dtype == Q3_F32)
    q3::launch(q3::qkv_post_kernel<float>, dim3(grid), dim3(q3::QP_WARPS * 32), 0, stream, 
        (const float*)qkv, (float*)q_out, (float*)k_pages, (float*)v_pages, q_weight, k_weight, inv_freq,
        positions, tok_seq, block_table, table_stride, page_size, num_pages, Hq, Hkv, D, rotary_dim, eps,
        write_kv, status);
  else if (dtype == Q3_BF16)
    q3::launch(q3::qkv_post_kernel<__nv_bfloat16>, dim3(grid), dim3(q3::QP_WARPS * 32), 0, stream, 
        (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages,
        q_weight, k_weight, inv_freq, positions, tok_seq, block_table, table_stride, page_size, num_pages,
        Hq, Hkv, D, rotary_dim, eps, write_kv, status);
  else
    return Q3_ERR_DTYPE;
  return q3::launch_status();
}

// table[t, j] = cos(positions[t] * inv_freq[j]), table[t, half + j] = sin(...); table float32 [T, 2 * half].
extern "C" int q3_rope_table(const float* inv_freq, const int* positions, float* table, int T, int half,
                             cudaStream_t stream) {
  if (T <= 0 || half <= 0) return 0;
  const long long n = (long long)T * half;
  if (n > 0x7fffffffLL) return Q3_ERR_SIZE;
  q3::launch(q3::rope_table_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, inv_freq, positions, table,
             T, half);
  q3::note_stream_written();  // what it writes must not be read ahead of the wait by the launch after it
  return q3::launch_status();
}
