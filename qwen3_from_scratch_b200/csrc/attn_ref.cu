// Paged causal attention, the plain kernel: one warp per (query token, query head),
// keys visited one by one in ascending position with a running maximum and
// denominator (float32 throughout; probabilities are never rounded).  A query's
// result depends only on its own keys and their order, not on how the batch was
// cut, so the 32-bit path gives the same bits for whole prompts, portions and
// single decoded tokens.  It serves the float32 path, sizes the fast bfloat16
// kernels refuse, and the tests as the on-device oracle of those kernels.
//
// Reference formulas (models/attn.py:402-499, kernels/triton/paged_attn.py:89-181):
//   query at absolute position p = kv_len - q_len + i sees keys n <= p
//   (and n > p - window when a window is set); s_n = (q . k_n) * scale;
//   o = sum softmax(s)_n v_n; q head h reads kv head h / (Hq / Hkv).
#include "common.cuh"

namespace q3 {

constexpr int AR_WARPS = 4;

template <typename T, int NJ>
__global__ void __launch_bounds__(AR_WARPS * 32)
attn_ref_kernel(const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                T* __restrict__ out, const int* __restrict__ q_start, const int* __restrict__ kv_len,
                const int* __restrict__ tok_seq, const int* __restrict__ block_table, int table_stride,
                int page_size, int num_pages, int Hq, int Hkv, int D, float scale, int window,
                int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int head = blockIdx.y * AR_WARPS + warp;
  if (head >= Hq) return;
  const int b = tok_seq[t];
  const int q_len = q_start[b + 1] - q_start[b];
  const int pos = kv_len[b] - q_len + (t - q_start[b]);
  const int hk = head / (Hq / Hkv);
  T* o = out + ((size_t)t * Hq + head) * D;
  if (pos < 0) {
    if (lane == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
    for (int e = lane; e < D; e += 32) o[e] = from_float<T>(0.f);
    return;
  }
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

  float qv[NJ], acc[NJ];
  const T* qp = q + ((size_t)t * Hq + head) * D;
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const int e = lane + 32 * j;
    qv[j] = e < D ? to_float(qp[e]) : 0.f;
    acc[j] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const int* table = block_table + (size_t)b * table_stride;
  for (int n = lo; n <= pos; ++n) {
    const int page = table_page(table, n / page_size, table_stride, status);
    if (page < 0 || page >= num_pages) {
      if (lane == 0) atomicOr(status, Q3_STATUS_BAD_PAGE);
      continue;
    }
    const size_t row = (((size_t)page * Hkv + hk) * page_size + (n % page_size)) * D;
    const T* kp = k_pages + row;
    const T* vp = v_pages + row;
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const int e = lane + 32 * j;
      if (e < D) dot = fmaf(qv[j], to_float(kp[e]), dot);
    }
    dot = warp_sum(dot) * scale;
    const float m_new = fmaxf(m, dot);
    const float f = expf(m - m_new);
    const float p = expf(dot - m_new);
    l = l * f + p;
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const int e = lane + 32 * j;
      if (e < D) acc[j] = acc[j] * f + p * to_float(vp[e]);
    }
    m = m_new;
  }
  const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const int e = lane + 32 * j;
    if (e < D) o[e] = from_float<T>(acc[j] * inv);
  }
}

template <typename T>
static int attn_ref_launch(const void* q, const void* k_pages, const void* v_pages, void* out,
                           const int* q_start, const int* kv_len, const int* tok_seq,
                           const int* block_table, int table_stride, int page_size, int num_pages,
                           int T_total, int Hq, int Hkv, int D, float scale, int window, int* status,
                           cudaStream_t stream) {
  dim3 grid(T_total, (Hq + AR_WARPS - 1) / AR_WARPS);
  if (grid.y > 65535) return Q3_ERR_SIZE;
#define Q3_AR_CASE(NJ)                                                                               \
  q3::launch(attn_ref_kernel<T, NJ>, dim3(grid), dim3(AR_WARPS * 32), 0, stream,                                         \
      (const T*)q, (const T*)k_pages, (const T*)v_pages, (T*)out, q_start, kv_len, tok_seq,          \
      block_table, table_stride, page_size, num_pages, Hq, Hkv, D, scale, window, status)
  if (D <= 32) Q3_AR_CASE(1);
  else if (D <= 64) Q3_AR_CASE(2);
  else if (D <= 128) Q3_AR_CASE(4);
  else if (D <= 256) Q3_AR_CASE(8);
  else if (D <= 512) Q3_AR_CASE(16);
  else return Q3_ERR_SIZE;
#undef Q3_AR_CASE
  return launch_status();
}

}  // namespace q3

// q: [T, Hq, D]; out: [T, Hq, D]; k_pages / v_pages: [num_pages, Hkv, page_size, D]; all in `dtype`.
// q_start: int32 [B + 1] token offsets of the sequences; kv_len: int32 [B] keys per sequence after
// this step's write; tok_seq: int32 [T] sequence of each token; block_table: int32 [B, table_stride].
// window <= 0: all earlier keys.  Refuses D > 512 and Hq not a multiple of Hkv.
extern "C" int q3_attn_ref(const void* q, int dtype, const void* k_pages, const void* v_pages, void* out,
                           const int* q_start, const int* kv_len, const int* tok_seq,
                           const int* block_table, int table_stride, int page_size, int num_pages,
                           int T_total, int Hq, int Hkv, int D, float scale, int window, int* status,
                           cudaStream_t stream) {
  if (T_total <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv || D <= 0 || page_size <= 0 || table_stride <= 0) return Q3_ERR_SIZE;
  if (dtype == Q3_F32)
    return q3::attn_ref_launch<float>(q, k_pages, v_pages, out, q_start, kv_len, tok_seq, block_table,
                                      table_stride, page_size, num_pages, T_total, Hq, Hkv, D, scale,
                                      window, status, stream);
  if (dtype == Q3_BF16)
    return q3::attn_ref_launch<__nv_bfloat16>(q, k_pages, v_pages, out, q_start, kv_len, tok_seq,
                                              block_table, table_stride, page_size, num_pages, T_total,
                                              Hq, Hkv, D, scale, window, status, stream);
  return Q3_ERR_DTYPE;
}
