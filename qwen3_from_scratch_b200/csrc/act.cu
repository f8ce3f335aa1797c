// SwiGLU gate on the merged gate/up projection:
//   out[t, i] = up[t, i] * gate[t, i] * sigmoid(gate[t, i])
// with gate = columns [0, I) and up = columns [I, 2I) of the [T, 2I] input.
// (or, with `interleave8`, gate and up alternating in blocks of eight columns, the layout the
// fused skinny product wants of its weight).  The gate is evaluated in float32 and the product rounded once.
// Reference: models/feedback.py:28-34 (up * silu(gate)), kernels/triton/feedback.py:145-158.
#include "common.cuh"

namespace q3 {

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int I, size_t total,
                              int interleave8) {
  pdl_wait();
  pdl_launch_dependents();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / I;
  const int i = (int)(idx - t * I);
  const T* row = gate_up + t * 2 * (size_t)I;
  const int gate_col = interleave8 ? ((i >> 3) << 4) + (i & 7) : i;
  const int up_col = interleave8 ? gate_col + 8 : I + i;
  const float g = to_float(row[gate_col]);
  const float u = to_float(row[up_col]);
  out[idx] = from_float<T>(u * (g / (1.0f + expf(-g))));
}

// Eight outputs per thread with 16-byte accesses (bfloat16, I a multiple of 8).
__global__ void swiglu_bf16x8_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out,
                                     int I, size_t total8, int interleave8) {
  pdl_wait();
  pdl_launch_dependents();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total8) return;
  const int per_row = I >> 3;
  const size_t t = idx / per_row;
  const int j = (int)(idx - t * per_row);  // block of eight outputs
  const __nv_bfloat16* row = gate_up + t * 2 * (size_t)I;
  const uint4 gv = *reinterpret_cast<const uint4*>(row + (interleave8 ? 16 * j : 8 * j));
  const uint4 uv = *reinterpret_cast<const uint4*>(row + (interleave8 ? 16 * j + 8 : I + 8 * j));
  const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
  uint32_t ow[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float g0 = __uint_as_float(gw[k] << 16), g1 = __uint_as_float(gw[k] & 0xffff0000u);
    const float u0 = __uint_as_float(uw[k] << 16), u1 = __uint_as_float(uw[k] & 0xffff0000u);
    __nv_bfloat162 o = __floats2bfloat162_rn(u0 * (g0 / (1.0f + expf(-g0))), u1 * (g1 / (1.0f + expf(-g1))));
    ow[k] = *reinterpret_cast<uint32_t*>(&o);
  }
  *reinterpret_cast<uint4*>(out + t * (size_t)I + 8 * j) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
}

}  // namespace q3

// gate_up: [T, 2I]; out: [T, I]; both in `dtype`.  interleave8: columns 16j..16j+7 gate, 16j+8..16j+15 up.
extern "C" int q3_swiglu(const void* gate_up, void* out, int dtype, int T, int I, int interleave8,
                         cudaStream_t stream) {
  if (T <= 0 || I <= 0) return 0;
  if (interleave8 && I % 8) return Q3_ERR_SIZE;
  const size_t total = (size_t)T * I;
  const int threads = 256;
  const size_t blocks = (total + threads - 1) / threads;
  if (blocks > 0x7fffffffull) return Q3_ERR_SIZE;
  if (dtype == Q3_BF16 && I % 8 == 0 && (uintptr_t)gate_up % 16 == 0 && (uintptr_t)out % 16 == 0) {
    const size_t total8 = total / 8;
    q3::launch(q3::swiglu_bf16x8_kernel, dim3((unsigned)((total8 + threads - 1) / threads)), dim3(threads), 0, stream, 
        (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, I, total8, interleave8);
    return q3::launch_status();
  }
  if (dtype == Q3_F32)
    q3::launch(q3::swiglu_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, stream, (const float*)gate_up, (float*)out, I, total, interleave8);
  else if (dtype == Q3_BF16)
    q3::launch(q3::swiglu_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(threads), 0, stream, 
        (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, I, total, interleave8);
  else
    return Q3_ERR_DTYPE;
  return q3::launch_status();
}
