// Embedding lookup and RMSNorm with the residual sum folded in.
//
// The residual stream of the model is kept in float32 for every compute dtype:
// the embedding writes it, every block adds its mixer's and its feed-forward's
// output into it, and the norms read it.  The sum and the statistics are float32;
// only the normed activations that feed the next matrix product are rounded to
// the compute dtype.
//
// RMSNorm formula (reference: models/norm.py:18-22, csrc/rms_norm/rms_norm.cpp:13-31):
//   y = x / sqrt(mean(x^2) + eps) * w
#include "common.cuh"

namespace q3 {

std::atomic<uintptr_t> g_plain_launch_stream{NO_PLAIN_LAUNCH};
thread_local bool g_launch_early = true;

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ resid, int H, int V, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int id = ids[t];
  float* dst = resid + (size_t)t * H;
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_TOKEN);
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = 0.f;
    return;
  }
  const T* src = table + (size_t)id * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = to_float(src[i]);
}

// ---------------------------------------------------------------- add + RMSNorm
// One block per output row.  rows == nullptr: row r of the launch is row r of the
// stream, and the updated sum is written back.  rows != nullptr: output row r is
// stream row rows[r]; nothing is written back (used for the last norm, which only
// the wanted rows need).
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                   const float* __restrict__ w, T* __restrict__ out,
                                   const int* __restrict__ rows, int H, float eps) {
  pdl_wait();
  pdl_launch_dependents();
  extern __shared__ float row_buf[];
  __shared__ float scratch[32];
  const int src_row = rows ? rows[blockIdx.x] : blockIdx.x;
  float* r = resid + (size_t)src_row * H;
  const T* d = delta ? delta + (size_t)src_row * H : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = r[i];
    if (d) v += to_float(d[i]);
    row_buf[i] = v;
    ss += v * v;
    if (!rows && d) r[i] = v;
  }
  ss = block_sum(ss, scratch);
  const float rs = 1.0f / sqrtf(ss / (float)H + eps);
  T* o = out + (size_t)blockIdx.x * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_float<T>(row_buf[i] * rs * w[i]);
}

// 4-wide variant for H % 4 == 0 and 16-byte aligned rows.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 x = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(x.x << 16); v[1] = __uint_as_float(x.x & 0xffff0000u);
    v[2] = __uint_as_float(x.y << 16); v[3] = __uint_as_float(x.y & 0xffff0000u);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[4]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]);
    __nv_bfloat162 b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 x;
    x.x = *reinterpret_cast<uint32_t*>(&a);
    x.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = x;
  }
};

// `early` != 0: the stream was not written by the launch directly before this one, so its row may be
// read ahead of the wait; the norm weight, which no kernel writes, always is.
template <typename T>
__global__ void add_rmsnorm_vec4_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                        const float* __restrict__ w, T* __restrict__ out,
                                        const int* __restrict__ rows, int H, float eps, int early) {
  extern __shared__ float row_buf[];
  __shared__ float scratch[32];
  const int src_row = rows ? rows[blockIdx.x] : blockIdx.x;
  float* r = resid + (size_t)src_row * H;
  const T* d = delta ? delta + (size_t)src_row * H : nullptr;
  const int i0 = threadIdx.x * 4;
  float w0[4] = {0.f, 0.f, 0.f, 0.f}, v0[4] = {0.f, 0.f, 0.f, 0.f};
  if (i0 < H) {
    Vec4<float>::load(w + i0, w0);
    if (early) Vec4<float>::load(r + i0, v0);
  }
  pdl_wait();
  pdl_launch_dependents();
  float ss = 0.f;
  for (int i = i0; i < H; i += blockDim.x * 4) {
    float v[4];
    if (early && i == i0) {
#pragma unroll
      for (int k = 0; k < 4; ++k) v[k] = v0[k];
    } else {
      Vec4<float>::load(r + i, v);
    }
    if (d) {
      float dv[4];
      Vec4<T>::load(d + i, dv);
#pragma unroll
      for (int k = 0; k < 4; ++k) v[k] += dv[k];
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) { row_buf[i + k] = v[k]; ss += v[k] * v[k]; }
    if (!rows && d) Vec4<float>::store(r + i, v);
  }
  ss = block_sum(ss, scratch);
  const float rs = 1.0f / sqrtf(ss / (float)H + eps);
  T* o = out + (size_t)blockIdx.x * H;
  for (int i = i0; i < H; i += blockDim.x * 4) {
    float wv[4], v[4];
    if (i == i0) {
#pragma unroll
      for (int k = 0; k < 4; ++k) wv[k] = w0[k];
    } else {
      Vec4<float>::load(w + i, wv);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = row_buf[i + k] * rs * wv[k];
    Vec4<T>::store(o + i, v);
  }
}

// One warp per row, for many rows of a width that is a multiple of 128 (up to 2048): a lane keeps
// its H / 32 values in registers, all of a row's loads are in flight together, and the only
// reduction is a warp shuffle.  Used for bfloat16 prompt portions; the float32 path keeps one
// kernel (and so one order of summation) for every number of rows.
constexpr int NW_WARPS = 8;

template <typename T, int NCH>
__global__ void __launch_bounds__(NW_WARPS * 32)
add_rmsnorm_warp_kernel(float* __restrict__ resid, const T* __restrict__ delta, const float* __restrict__ w,
                        T* __restrict__ out, const int* __restrict__ rows, int n_rows, float eps, int early) {
  constexpr int H = NCH * 128;
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * NW_WARPS + (threadIdx.x >> 5);
  const bool live = row < n_rows;
  const int src_row = !live ? 0 : rows ? rows[row] : row;
  float* r = resid + (size_t)src_row * H;
  float v[NCH][4];
  if (early && live) {  // the stream's row, ahead of the wait (see add_rmsnorm_vec4_kernel)
#pragma unroll
    for (int i = 0; i < NCH; ++i) Vec4<float>::load(r + (i * 32 + lane) * 4, v[i]);
  }
  pdl_wait();
  pdl_launch_dependents();
  if (!live) return;
  const T* d = delta ? delta + (size_t)src_row * H : nullptr;
  if (!early) {
#pragma unroll
    for (int i = 0; i < NCH; ++i) Vec4<float>::load(r + (i * 32 + lane) * 4, v[i]);
  }
  if (d) {
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      float dv[4];
      Vec4<T>::load(d + (i * 32 + lane) * 4, dv);
#pragma unroll
      for (int k = 0; k < 4; ++k) v[i][k] += dv[k];
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NCH; ++i)
#pragma unroll
    for (int k = 0; k < 4; ++k) ss += v[i][k] * v[i][k];
  ss = warp_sum(ss);
  const float rs = 1.0f / sqrtf(ss / (float)H + eps);
  if (!rows && d) {
#pragma unroll
    for (int i = 0; i < NCH; ++i) Vec4<float>::store(r + (i * 32 + lane) * 4, v[i]);
  }
  T* o = out + (size_t)row * H;
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    float wv[4], y[4];
    Vec4<float>::load(w + (i * 32 + lane) * 4, wv);
#pragma unroll
    for (int k = 0; k < 4; ++k) y[k] = v[i][k] * rs * wv[k];
    Vec4<T>::store(o + (i * 32 + lane) * 4, y);
  }
}

template <typename T, int NCH>
static void add_rmsnorm_warp_launch(float* resid, const T* delta, const float* w, T* out, const int* rows, int n_rows,
                                    float eps, int early, cudaStream_t stream) {
  q3::launch(add_rmsnorm_warp_kernel<T, NCH>, dim3((n_rows + NW_WARPS - 1) / NW_WARPS), dim3(NW_WARPS * 32), 0, stream,
             resid, delta, w, out, rows, n_rows, eps, early);
}

// ---------------------------------------------------------------- plain RMSNorm on vectors
// y[r, :] = rmsnorm(x[r, :]) * w, x and y in the compute dtype, one warp per row.
// For short vectors (a head) and for tests of the norm part alone.
template <typename T>
__global__ void rmsnorm_rows_kernel(const T* __restrict__ x, const float* __restrict__ w,
                                    T* __restrict__ y, int rows, int dim, float eps) {
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const T* src = x + (size_t)row * dim;
  float ss = 0.f;
  for (int i = lane; i < dim; i += 32) { const float v = to_float(src[i]); ss += v * v; }
  ss = warp_sum(ss);
  const float rs = 1.0f / sqrtf(ss / (float)dim + eps);
  T* dst = y + (size_t)row * dim;
  for (int i = lane; i < dim; i += 32) dst[i] = from_float<T>(to_float(src[i]) * rs * w[i]);
}

template <typename T>
static int add_rmsnorm_launch(float* resid, const void* delta, const float* w, void* out,
                              const int* rows, int n_rows, int H, float eps, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 200 * 1024) return Q3_ERR_SIZE;  // width beyond 51200 is refused
  const bool vec = (H % 4 == 0) && ((uintptr_t)resid % 16 == 0) && ((uintptr_t)w % 16 == 0) &&
                   ((uintptr_t)out % 16 == 0) && (!delta || (uintptr_t)delta % 16 == 0);
  // the stream may be read ahead of the wait unless the launch before this one wrote it; this launch
  // writes it when it has a delta to add and no row list
  const int early = last_launch_was_plain(stream) ? 1 : 0;
  const bool writes = !rows && delta;
  if (vec && sizeof(T) == 2 && n_rows >= 64 && H % 128 == 0 && H <= 2048) {
    switch (H / 128) {
#define Q3_NW(N) case N: add_rmsnorm_warp_launch<T, N>(resid, (const T*)delta, w, (T*)out, rows, n_rows, eps, early, stream); break;
      Q3_NW(1) Q3_NW(2) Q3_NW(3) Q3_NW(4) Q3_NW(5) Q3_NW(6) Q3_NW(7) Q3_NW(8)
      Q3_NW(9) Q3_NW(10) Q3_NW(11) Q3_NW(12) Q3_NW(13) Q3_NW(14) Q3_NW(15) Q3_NW(16)
#undef Q3_NW
    }
    if (writes) note_stream_written();
    return launch_status();
  }
  int threads = vec ? (H / 4) : H;
  threads = ((threads + 31) / 32) * 32;
  if (threads > 512) threads = 512;
  if (threads < 32) threads = 32;
  if (vec) {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_vec4_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    q3::launch(add_rmsnorm_vec4_kernel<T>, dim3(n_rows), dim3(threads), smem, stream, resid, (const T*)delta, w, (T*)out,
               rows, H, eps, early);
  } else {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    q3::launch(add_rmsnorm_kernel<T>, dim3(n_rows), dim3(threads), smem, stream, resid, (const T*)delta, w, (T*)out, rows,
               H, eps);
  }
  if (writes) note_stream_written();
  return launch_status();
}

}  // namespace q3

// resid[t, :] = table[ids[t], :] as float32.  table: [V, H] in `dtype`.
extern "C" int q3_embed(const void* table, int dtype, const int* ids, float* resid, int T, int H,
                        int V, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  int threads = ((H + 31) / 32) * 32;
  if (threads > 256) threads = 256;
  if (dtype == Q3_F32)
    q3::launch(q3::embed_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)table, ids, resid, H, V, status);
  else if (dtype == Q3_BF16)
    q3::launch(q3::embed_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (const __nv_bfloat16*)table, ids, resid, H, V, status);
  else
    return Q3_ERR_DTYPE;
  q3::note_stream_written();
  return q3::launch_status();
}

// resid[r, :] += delta[r, :] (if delta != null); out[r, :] = rmsnorm(resid[r, :]) * w.
// resid float32 [n_rows, H]; delta and out in `dtype`; w float32 [H].
extern "C" int q3_add_rmsnorm(float* resid, const void* delta, const float* w, void* out, int dtype,
                              int n_rows, int H, float eps, cudaStream_t stream) {
  if (dtype == Q3_F32) return q3::add_rmsnorm_launch<float>(resid, delta, w, out, nullptr, n_rows, H, eps, stream);
  if (dtype == Q3_BF16) return q3::add_rmsnorm_launch<__nv_bfloat16>(resid, delta, w, out, nullptr, n_rows, H, eps, stream);
  return Q3_ERR_DTYPE;
}

// out[r, :] = rmsnorm(resid[rows[r], :] + delta[rows[r], :]) * w for r < n_out; resid is not changed.
extern "C" int q3_add_rmsnorm_rows(float* resid, const void* delta, const float* w, void* out, int dtype,
                                   const int* rows, int n_out, int H, float eps, cudaStream_t stream) {
  if (!rows) return Q3_ERR_SIZE;
  if (dtype == Q3_F32) return q3::add_rmsnorm_launch<float>(resid, delta, w, out, rows, n_out, H, eps, stream);
  if (dtype == Q3_BF16) return q3::add_rmsnorm_launch<__nv_bfloat16>(resid, delta, w, out, rows, n_out, H, eps, stream);
  return Q3_ERR_DTYPE;
}

// y[r, :] = rmsnorm(x[r, :]) * w; x, y: [rows, dim] in `dtype`, w float32 [dim].
extern "C" int q3_rmsnorm(const void* x, const float* w, void* y, int dtype, int rows, int dim, float eps,
                          cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int warps = 4;
  const int grid = (rows + warps - 1) / warps;
  if (dtype == Q3_F32)
    q3::launch(q3::rmsnorm_rows_kernel<float>, dim3(grid), dim3(warps * 32), 0, stream, (const float*)x, w, (float*)y, rows, dim, eps);
  else if (dtype == Q3_BF16)
    q3::launch(q3::rmsnorm_rows_kernel<__nv_bfloat16>, dim3(grid), dim3(warps * 32), 0, stream, (const __nv_bfloat16*)x, w, (__nv_bfloat16*)y, rows, dim, eps);
  else
    return Q3_ERR_DTYPE;
  return q3::launch_status();
}
