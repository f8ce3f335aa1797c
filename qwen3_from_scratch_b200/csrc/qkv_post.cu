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
    const int page = block_table[(size_t)seq * table_stride + pos / page_size];
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

// The same for bfloat16 when D is a multiple of 32 and the whole head is rotated: lane l owns
// the D / 32 consecutive values from l * D / 32, so lanes 0..15 hold the first half of the head
// and lane l + 16 holds the rotation partners of lane l; no shared memory, 2 * VPL-byte accesses.
constexpr int QPV_WARPS = 8;
constexpr int QPV_UNROLL = 4;

template <int VPL>
__global__ void __launch_bounds__(QPV_WARPS * 32)
qkv_post_vec_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                    __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages,
                    const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                    const float* __restrict__ inv_freq, const int* __restrict__ positions,
                    const int* __restrict__ tok_seq, const int* __restrict__ block_table, int table_stride,
                    int page_size, int num_pages, int Hq, int Hkv, float eps, int write_kv, int heads_per_block,
                    int* status) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int D = 32 * VPL;
  // A block serves one token and the heads [blockIdx.y * heads_per_block, + heads_per_block): the
  // sines and cosines of the token's D / 2 angles are computed once per block and shared by its
  // heads (all heads of the token when there are many tokens, eight when there are few).
  __shared__ float cs[D];  // cos of pair j at [j], sin at [D / 2 + j]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int n_heads = Hq + 2 * Hkv;
  const int pos = positions[t];
  if (inv_freq != nullptr) {
    for (int j = threadIdx.x; j < D / 2; j += QPV_WARPS * 32) {
      float sn, c;
      sincosf((float)pos * inv_freq[j], &sn, &c);
      cs[j] = c;
      cs[D / 2 + j] = sn;
    }
  }
  __syncthreads();
  const int head_end = min(n_heads, (int)(blockIdx.y + 1) * heads_per_block);
  // Up to QPV_UNROLL heads of a warp are loaded before the first is worked on, so that a warp has
  // several loads in flight: with one it could not keep the memory system busy on a long prompt.
  for (int head0 = blockIdx.y * heads_per_block + warp; head0 < head_end; head0 += QPV_WARPS * QPV_UNROLL) {
    float x[QPV_UNROLL][VPL];
    bool live[QPV_UNROLL];
#pragma unroll
    for (int u = 0; u < QPV_UNROLL; ++u) {
      const int head = head0 + u * QPV_WARPS;
      live[u] = head < head_end && (head < Hq || write_kv);
      if (!live[u]) continue;
      const __nv_bfloat16* src = qkv + ((size_t)t * n_heads + head) * D + lane * VPL;
      if (VPL == 8) {
        const uint4 v = *reinterpret_cast<const uint4*>(src);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          x[u][(2 * k) % VPL] = __uint_as_float(w[k] << 16);
          x[u][(2 * k + 1) % VPL] = __uint_as_float(w[k] & 0xffff0000u);
        }
      } else if (VPL == 4) {
        const uint2 v = *reinterpret_cast<const uint2*>(src);
        x[u][0] = __uint_as_float(v.x << 16); x[u][1 % VPL] = __uint_as_float(v.x & 0xffff0000u);
        x[u][2 % VPL] = __uint_as_float(v.y << 16); x[u][3 % VPL] = __uint_as_float(v.y & 0xffff0000u);
      } else if (VPL == 2) {
        const uint32_t v = *reinterpret_cast<const uint32_t*>(src);
        x[u][0] = __uint_as_float(v << 16); x[u][1 % VPL] = __uint_as_float(v & 0xffff0000u);
      } else {
        x[u][0] = __bfloat162float(src[0]);
      }
    }
#pragma unroll
    for (int u = 0; u < QPV_UNROLL; ++u) {
      if (!live[u]) continue;  // uniform over the warp
      const int head = head0 + u * QPV_WARPS;
      const bool is_q = head < Hq;
      const bool is_k = !is_q && head < Hq + Hkv;
      const float* w = is_q ? q_weight : (is_k ? k_weight : nullptr);
      if (w) {
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < VPL; ++k) ss += x[u][k] * x[u][k];
        ss = warp_sum(ss);
        const float rs = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
        for (int k = 0; k < VPL; ++k) x[u][k] = x[u][k] * rs * w[lane * VPL + k];
      }
      if ((is_q || is_k) && inv_freq != nullptr) {
        const bool first_half = lane < 16;
#pragma unroll
        for (int k = 0; k < VPL; ++k) {
          const float partner = __shfl_xor_sync(0xffffffffu, x[u][k], 16);
          const int j = (lane & 15) * VPL + k;  // index of the pair
          const float c = cs[j], sn = cs[D / 2 + j];
          x[u][k] = first_half ? x[u][k] * c - partner * sn : x[u][k] * c + partner * sn;
        }
      }
      __nv_bfloat16* dst;
      if (is_q) {
        dst = q_out + ((size_t)t * Hq + head) * D;
      } else {
        const int seq = tok_seq[t];
        if (pos < 0 || seq < 0) {
          if (lane == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
          continue;
        }
        const int page = block_table[(size_t)seq * table_stride + pos / page_size];
        if (page < 0 || page >= num_pages) {
          if (lane == 0) atomicOr(status, Q3_STATUS_BAD_PAGE);
          continue;
        }
        const int hk = is_k ? head - Hq : head - Hq - Hkv;
        dst = (is_k ? k_pages : v_pages) + (((size_t)page * Hkv + hk) * page_size + (pos % page_size)) * D;
      }
      dst += lane * VPL;
      if (VPL == 8) {
        uint32_t o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          __nv_bfloat162 p = __floats2bfloat162_rn(x[u][(2 * k) % VPL], x[u][(2 * k + 1) % VPL]);
          o[k] = *reinterpret_cast<uint32_t*>(&p);
        }
        *reinterpret_cast<uint4*>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
      } else if (VPL == 4) {
        __nv_bfloat162 a = __floats2bfloat162_rn(x[u][0], x[u][1 % VPL]), b = __floats2bfloat162_rn(x[u][2 % VPL], x[u][3 % VPL]);
        *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
      } else if (VPL == 2) {
        *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(x[u][0], x[u][1 % VPL]);
      } else {
        dst[0] = __float2bfloat16_rn(x[u][0]);
      }
    }
  }
}

}  // namespace q3

// qkv: [T, (Hq + 2 Hkv) * D] in `dtype`, rows ordered q heads, k heads, v heads.
// q_out: [T, Hq, D].  k_pages / v_pages: [num_pages, Hkv, page_size, D].
// q_weight / k_weight: float32 [D] or null (no head norm).  inv_freq: float32 [rotary_dim / 2]
// or null (no rotation).  positions, tok_seq: int32 [T] (absolute position, row of the block table).
// write_kv == 0: only q is produced (a layer that reads a cache another layer wrote).
// Refuses D > 512 or odd rotary_dim or rotary_dim > D.
extern "C" int q3_qkv_post(const void* qkv, int dtype, int T, int Hq, int Hkv, int D,
                           const float* q_weight, const float* k_weight, float eps,
                           const float* inv_freq, int rotary_dim, const int* positions,
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
  const int heads_per_block = T >= 256 ? n_heads : q3::QPV_WARPS;
  if (dtype == Q3_BF16 && whole_rotation && (D == 32 || D == 64 || D == 128 || D == 256) &&
      (uintptr_t)qkv % 16 == 0 && (uintptr_t)q_out % 16 == 0 && (uintptr_t)k_pages % 16 == 0 &&
      (uintptr_t)v_pages % 16 == 0) {
#define Q3_QP_VEC(VPL)                                                                                            \
  q3::launch(q3::qkv_post_vec_kernel<VPL>, dim3(T, (n_heads + heads_per_block - 1) / heads_per_block),           \
             dim3(q3::QPV_WARPS * 32), 0, stream,                                            \
      (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, q_weight, \
      k_weight, inv_freq, positions, tok_seq, block_table, table_stride, page_size, num_pages, Hq, Hkv, eps,       \
      write_kv, heads_per_block, status)
    if (D == 32) Q3_QP_VEC(1);
    else if (D == 64) Q3_QP_VEC(2);
    else if (D == 128) Q3_QP_VEC(4);
    else Q3_QP_VEC(8);
#undef Q3_QP_VEC
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
