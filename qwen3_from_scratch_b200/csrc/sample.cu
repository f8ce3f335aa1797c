// Token sampling from float32 logits, one block per row, no host round trip.
//
//   temperature <= 0          : argmax, ties to the lowest id   (reference: inference/sampler.py:17-21)
//   temperature > 0           : a draw from softmax(logits / T) (reference: inference/sampler.py:24-33)
//   temperature > 0, top_k > 0: the same among the k largest logits (inference/sampler.py:36-56)
//
// The draw uses the Gumbel-max form: argmax_i(logits_i / T + g_i) with
// g_i = -log(-log(u_i)) has exactly the softmax(logits / T) distribution and needs
// no normalisation pass.  u_i comes from a counter-based generator keyed by
// (seed, request key, position, i), so what a request samples does not depend on the
// batch it is in, on preemption, or on how its prompt was cut.
//
// Generator (64-bit mix of Steele, Lea and Flood's SplitMix finaliser):
//   mix(z):  z += 0x9E3779B97F4A7C15; z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9;
//            z = (z ^ (z >> 27)) * 0x94D049BB133111EB; return z ^ (z >> 31)
//   row_key = mix(mix(seed) + mix(request_key) * 3 + position)
//   u_i     = ((mix(row_key + i) >> 41) + 0.5) * 2^-23          in (0, 1), exact in float32
#include "common.cuh"

namespace q3 {

__host__ __device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

__device__ __forceinline__ uint32_t ordered_bits(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct Best {
  float val;
  int idx;
};

__device__ __forceinline__ Best better(Best a, Best b) {
  if (b.val > a.val || (b.val == a.val && b.idx < a.idx)) return b;
  return a;
}

__device__ __forceinline__ Best block_best(Best v, Best* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other;
    other.val = __shfl_xor_sync(0xffffffffu, v.val, o);
    other.idx = __shfl_xor_sync(0xffffffffu, v.idx, o);
    v = better(v, other);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  Best t;
  t.val = -INFINITY;
  t.idx = 0x7fffffff;
  if (lane < nwarps) t = scratch[lane];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other;
    other.val = __shfl_xor_sync(0xffffffffu, t.val, o);
    other.idx = __shfl_xor_sync(0xffffffffu, t.idx, o);
    t = better(t, other);
  }
  return t;
}

__device__ __forceinline__ int block_count(int v, int* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  int t = lane < nwarps ? scratch[lane] : 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

__global__ void __launch_bounds__(1024)
sample_kernel(const float* __restrict__ logits, int V, size_t row_pitch,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const long long* __restrict__ request_key, const int* __restrict__ position,
              unsigned long long seed, int* __restrict__ out, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ Best best_scratch[32];
  __shared__ int count_scratch[32];
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * row_pitch;
  const float temp = temperature ? temperature[r] : 0.f;
  const int k = top_k ? top_k[r] : 0;

  // threshold of the k largest logits, as order-preserving bits (0 = everything passes)
  uint32_t threshold = 0;
  if (temp > 0.f && k > 0 && k < V) {
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = threshold | (1u << bit);
      int c = 0;
      for (int i = threadIdx.x; i < V; i += blockDim.x) c += ordered_bits(row[i]) >= cand;
      c = block_count(c, count_scratch);
      if (c >= k) threshold = cand;
    }
  }

  Best mine;
  mine.val = -INFINITY;
  mine.idx = 0x7fffffff;
  if (temp > 0.f) {
    const uint64_t row_key = mix64(mix64(seed) + mix64((uint64_t)request_key[r]) * 3ull + (uint64_t)(int64_t)position[r]);
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float x = row[i];
      if (ordered_bits(x) < threshold) continue;
      const float u = ((float)(mix64(row_key + (uint64_t)i) >> 41) + 0.5f) * 1.1920928955078125e-7f;
      const float g = -logf(-logf(u));
      Best c;
      c.val = x / temp + g;
      c.idx = i;
      mine = better(mine, c);
    }
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      Best c;
      c.val = row[i];
      c.idx = i;
      mine = better(mine, c);
    }
  }
  const Best b = block_best(mine, best_scratch);
  if (threadIdx.x == 0) {
    int idx = b.idx;
    if (idx < 0 || idx >= V) {
      atomicOr(status, Q3_STATUS_BAD_LOGITS);
      idx = 0;
    }
    out[r] = idx;
  }
}

}  // namespace q3

// logits: float32 [R, V] with row pitch `row_pitch` elements.  temperature: float32 [R] or null
// (all greedy); top_k: int32 [R] or null; request_key: int64 [R] and position: int32 [R] (needed
// only where temperature > 0).  out: int32 [R].
extern "C" int q3_sample(const float* logits, int R, int V, long long row_pitch, const float* temperature,
                         const int* top_k, const long long* request_key, const int* position,
                         unsigned long long seed, int* out, int* status, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0) return Q3_ERR_SIZE;
  if (temperature && (!request_key || !position)) return Q3_ERR_SIZE;
  q3::launch(q3::sample_kernel, dim3(R), dim3(1024), 0, stream, logits, V, (size_t)row_pitch, temperature, top_k, request_key,
                                            position, seed, out, status);
  return q3::launch_status();
}
