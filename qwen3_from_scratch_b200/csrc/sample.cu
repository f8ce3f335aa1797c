// Token sampling from float32 logits on the device, no host round trip.
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
// A row of a large vocabulary is too long for one block (152 k logits took 32 us for an argmax and
// 1 ms with top-k): a row is cut into chunks, one block each; the block that finishes last among a
// row's chunks (a ticket per row, nobody waits) reduces their results.  For top-k a first kernel
// builds a histogram of the logits' leading 11 bits (order-preserving) per row and finds the bin
// that holds the k-th largest; the second kernel collects the logits from that bin upwards (a few
// hundred as a rule), and the last block finds the exact k-th largest among them and draws.  A row
// with more such candidates than the list holds (logits that nearly all share their leading bits)
// is handled by its last block alone, slowly and exactly.
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

constexpr int SP_THREADS = 256;
constexpr int SP_MAX_CHUNKS = 64;
constexpr int SP_BINS = 2048;        // leading 11 bits of the order-preserving key
constexpr int SP_CAND = 4096;        // candidates kept per row for top-k

struct Cand {
  float val;
  int idx;
};

// Scratch of one row; everything but `partial` and `cand` is zero between launches.
struct SampleRow {
  int hist_ticket, draw_ticket, cand_count;
  uint32_t edge_key;  // order-preserving key of the lower edge of the bin that holds the k-th largest
  int pad[4];
  Best partial[SP_MAX_CHUNKS];
  int hist[SP_BINS];
  Cand cand[SP_CAND];
};

__device__ __forceinline__ bool wants_top_k(float temp, int k, int V) { return temp > 0.f && k > 0 && k < V; }

__device__ __forceinline__ float gumbel_score(float x, float temp, uint64_t row_key, int i) {
  const float u = ((float)(mix64(row_key + (uint64_t)i) >> 41) + 0.5f) * 1.1920928955078125e-7f;
  return x / temp - logf(-logf(u));
}

// First kernel of top-k: per row the bin (of the leading 11 key bits) in which the k-th largest logit lies.
__global__ void __launch_bounds__(SP_THREADS)
sample_hist_kernel(const float* __restrict__ logits, int V, size_t row_pitch, int chunk,
                   const float* __restrict__ temperature, const int* __restrict__ top_k, SampleRow* __restrict__ rows) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ int hist[SP_BINS];
  __shared__ int scan[SP_THREADS];
  __shared__ int is_last;
  const int r = blockIdx.y;
  const int k = top_k ? top_k[r] : 0;
  if (!wants_top_k(temperature ? temperature[r] : 0.f, k, V)) return;
  SampleRow& me = rows[r];
  const float* row = logits + (size_t)r * row_pitch;
  for (int i = threadIdx.x; i < SP_BINS; i += SP_THREADS) hist[i] = 0;
  __syncthreads();
  const int lo = blockIdx.x * chunk, hi = min(V, lo + chunk);
  for (int i = lo + threadIdx.x; i < hi; i += SP_THREADS) atomicAdd(&hist[ordered_bits(row[i]) >> 21], 1);
  __syncthreads();
  for (int i = threadIdx.x; i < SP_BINS; i += SP_THREADS)
    if (hist[i]) atomicAdd(&me.hist[i], hist[i]);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(&me.hist_ticket, 1) == (int)gridDim.x - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // thread t owns the bins [2047 - 8 t - 7, 2047 - 8 t], the highest first; where does the count from the top reach k?
  constexpr int PER = SP_BINS / SP_THREADS;
  int mine[PER], sum = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    mine[j] = __ldcg(&me.hist[SP_BINS - 1 - (threadIdx.x * PER + j)]);
    sum += mine[j];
  }
  scan[threadIdx.x] = sum;
  __syncthreads();
  int above = 0;  // logits in the bins of the threads before this one
  for (int t = 0; t < (int)threadIdx.x; ++t) above += scan[t];
  if (above < k && above + sum >= k) {
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      if (above < k && above + mine[j] >= k) me.edge_key = (uint32_t)(SP_BINS - 1 - (threadIdx.x * PER + j)) << 21;
      above += mine[j];
    }
  }
  for (int i = threadIdx.x; i < SP_BINS; i += SP_THREADS) me.hist[i] = 0;
  if (threadIdx.x == 0) me.hist_ticket = 0;
}

// One block per (chunk of the vocabulary, row); the last block of a row finishes it.
__global__ void __launch_bounds__(SP_THREADS)
sample_kernel(const float* __restrict__ logits, int V, size_t row_pitch, int chunk,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const long long* __restrict__ request_key, const int* __restrict__ position,
              unsigned long long seed, SampleRow* __restrict__ rows, int* __restrict__ out, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ Best best_scratch[32];
  __shared__ int count_scratch[32];
  __shared__ int is_last;
  __shared__ Cand cands[SP_CAND];
  const int r = blockIdx.y;
  SampleRow& me = rows[r];
  const float* row = logits + (size_t)r * row_pitch;
  const float temp = temperature ? temperature[r] : 0.f;
  const int k = top_k ? top_k[r] : 0;
  const bool select = wants_top_k(temp, k, V);
  const uint64_t row_key =
      temp > 0.f ? mix64(mix64(seed) + mix64((uint64_t)request_key[r]) * 3ull + (uint64_t)(int64_t)position[r]) : 0;
  const int lo = blockIdx.x * chunk, hi = min(V, lo + chunk);

  Best mine;
  mine.val = -INFINITY;
  mine.idx = 0x7fffffff;
  if (select) {
    const uint32_t edge = me.edge_key;  // written by the kernel before this one
    for (int i = lo + threadIdx.x; i < hi; i += SP_THREADS) {
      const float x = row[i];
      if (ordered_bits(x) < edge) continue;
      const int slot = atomicAdd(&me.cand_count, 1);
      if (slot < SP_CAND) {
        me.cand[slot].val = x;
        me.cand[slot].idx = i;
      }
    }
  } else {
    for (int i = lo + threadIdx.x; i < hi; i += SP_THREADS) {
      Best c;
      c.val = temp > 0.f ? gumbel_score(row[i], temp, row_key, i) : row[i];
      c.idx = i;
      mine = better(mine, c);
    }
    const Best b = block_best(mine, best_scratch);
    if (threadIdx.x == 0) me.partial[blockIdx.x] = b;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(&me.draw_ticket, 1) == (int)gridDim.x - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();

  mine.val = -INFINITY;
  mine.idx = 0x7fffffff;
  if (!select) {
    for (int c = threadIdx.x; c < (int)gridDim.x; c += SP_THREADS) {
      Best other;
      other.val = __ldcg(&me.partial[c].val);
      other.idx = __ldcg(&me.partial[c].idx);
      mine = better(mine, other);
    }
  } else {
    const int n = __ldcg(&me.cand_count);
    if (n <= SP_CAND) {
      for (int i = threadIdx.x; i < n; i += SP_THREADS) {
        cands[i].val = __ldcg(&me.cand[i].val);
        cands[i].idx = __ldcg(&me.cand[i].idx);
      }
      __syncthreads();
      // the k-th largest among the candidates is the k-th largest of the row
      uint32_t threshold = 0;
      for (int bit = 31; bit >= 0; --bit) {
        const uint32_t cand = threshold | (1u << bit);
        int c = 0;
        for (int i = threadIdx.x; i < n; i += SP_THREADS) c += ordered_bits(cands[i].val) >= cand;
        c = block_count(c, count_scratch);
        if (c >= k) threshold = cand;
      }
      for (int i = threadIdx.x; i < n; i += SP_THREADS) {
        if (ordered_bits(cands[i].val) < threshold) continue;
        Best c;
        c.val = gumbel_score(cands[i].val, temp, row_key, cands[i].idx);
        c.idx = cands[i].idx;
        mine = better(mine, c);
      }
    } else {
      // more candidates than the list holds: the whole row again, by this block alone
      uint32_t threshold = 0;
      for (int bit = 31; bit >= 0; --bit) {
        const uint32_t cand = threshold | (1u << bit);
        int c = 0;
        for (int i = threadIdx.x; i < V; i += SP_THREADS) c += ordered_bits(row[i]) >= cand;
        c = block_count(c, count_scratch);
        if (c >= k) threshold = cand;
      }
      for (int i = threadIdx.x; i < V; i += SP_THREADS) {
        const float x = row[i];
        if (ordered_bits(x) < threshold) continue;
        Best c;
        c.val = gumbel_score(x, temp, row_key, i);
        c.idx = i;
        mine = better(mine, c);
      }
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
    me.draw_ticket = 0;
    me.cand_count = 0;
    me.edge_key = 0;
  }
}

}  // namespace q3

// Bytes of scratch that q3_sample needs for R rows (zero-filled once; the kernels leave it as they found
// it).  More than 1024 rows are taken in slices that use the same scratch one after the other.
extern "C" long long q3_sample_scratch_bytes(int R) {
  const int rows = R < 0 ? 0 : (R > 1024 ? 1024 : R);
  return (long long)rows * (long long)sizeof(q3::SampleRow);
}

// logits: float32 [R, V] with row pitch `row_pitch` elements.  temperature: float32 [R] or null
// (all greedy); top_k: int32 [R] or null; request_key: int64 [R] and position: int32 [R] (needed
// only where temperature > 0).  any_top_k: some row has temperature > 0 and 0 < top_k < V (the
// histogram kernel is launched only then).  scratch: q3_sample_scratch_bytes(R) bytes.  out: int32 [R].
extern "C" int q3_sample(const float* logits, int R, int V, long long row_pitch, const float* temperature,
                         const int* top_k, const long long* request_key, const int* position,
                         unsigned long long seed, int any_top_k, void* scratch, long long scratch_bytes, int* out,
                         int* status, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0) return Q3_ERR_SIZE;
  if (temperature && (!request_key || !position)) return Q3_ERR_SIZE;
  if (!scratch || scratch_bytes < q3_sample_scratch_bytes(R) || (uintptr_t)scratch % 8) return Q3_ERR_SCRATCH;
  int chunks = (V + 4095) / 4096;
  if (chunks > q3::SP_MAX_CHUNKS) chunks = q3::SP_MAX_CHUNKS;
  const int chunk = (V + chunks - 1) / chunks;
  q3::SampleRow* rows = reinterpret_cast<q3::SampleRow*>(scratch);
  for (int r0 = 0; r0 < R; r0 += 1024) {
    const int n = R - r0 < 1024 ? R - r0 : 1024;
    const float* lg = logits + (size_t)r0 * (size_t)row_pitch;
    const float* tp = temperature ? temperature + r0 : nullptr;
    const int* tk = top_k ? top_k + r0 : nullptr;
    if (any_top_k && tk && tp) {
      q3::launch(q3::sample_hist_kernel, dim3(chunks, n), dim3(q3::SP_THREADS), 0, stream, lg, V, (size_t)row_pitch, chunk,
                 tp, tk, rows);
      const int code = q3::launch_status();
      if (code) return code;
    }
    q3::launch(q3::sample_kernel, dim3(chunks, n), dim3(q3::SP_THREADS), 0, stream, lg, V, (size_t)row_pitch, chunk, tp, tk,
               request_key ? request_key + r0 : nullptr, position ? position + r0 : nullptr, seed, rows, out + r0, status);
    const int code = q3::launch_status();
    if (code) return code;
  }
  return 0;
}
