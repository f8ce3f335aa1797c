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
  if (dtype == Q3_F32)
    q3::qkv_post_kernel<float><<<grid, q3::QP_WARPS * 32, 0, stream>>>(
        (const float*)qkv, (float*)q_out, (float*)k_pages, (float*)v_pages, q_weight, k_weight, inv_freq,
        positions, tok_seq, block_table, table_stride, page_size, num_pages, Hq, Hkv, D, rotary_dim, eps,
        write_kv, status);
  else if (dtype == Q3_BF16)
    q3::qkv_post_kernel<__nv_bfloat16><<<grid, q3::QP_WARPS * 32, 0, stream>>>(
        (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages,
        q_weight, k_weight, inv_freq, positions, tok_seq, block_table, table_stride, page_size, num_pages,
        Hq, Hkv, D, rotary_dim, eps, write_kv, status);
  else
    return Q3_ERR_DTYPE;
  return q3::launch_status();
}
