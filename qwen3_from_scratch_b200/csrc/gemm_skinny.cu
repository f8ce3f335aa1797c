// Skinny matrix product for decoding: out[T, N] = X[T, K] * W[N, K]^T with T <= 16 tokens, bfloat16
// in, float32 accumulate.  The step is bound by reading W once, so the kernel is built around that
// stream: W is the 16-row operand of the tensor-core tile ("swap-AB": 16 output features x 8 tokens
// per m16n8k16), every lane fetches 16 contiguous bytes of two W rows per 32 values of k straight
// from global memory into the registers the multiply uses, and K is split over the warps of a block
// so that enough blocks exist to keep every SM's memory pipeline full.
//
// Inside a group of 32 values of k the lanes use a fixed permutation (lane t of a row takes
// k = 8t .. 8t + 7): a dot product does not care about the order of its terms as long as both
// operands use the same one, and this order makes every load a 16-byte one.
//
// Epilogues: plain store (bfloat16 or float32), or SwiGLU for a weight whose rows alternate in
// blocks of eight between gate and up (rows 16j .. 16j+7 = gate[8j ..], rows 16j+8 .. 16j+15 =
// up[8j ..]): out[t, 8j + i] = up * gate * sigmoid(gate), so the gate/up product never goes to memory.
//
// Two more forms take the norm kernels out of a decode step (the reference's block: norm, mixer, add, norm,
// feed-forward, add; models/transformer_block.py:38-46).  RMSNorm is x * rs * w with one scalar rs per row,
// and a scalar commutes with the product: W (h * rs * w) = rs * (W (h * w)).  So
//   * "into the stream" (EPI 2): the product is added to the float32 stream in place; each block of 16
//     features leaves the sum of squares of its 16 new values per row, in a fixed order (no atomics), and,
//     given the weight of the norm that comes next, the new values times that weight, rounded once to bfloat16;
//   * "normed in" (NORMED): X is that bfloat16 operand h * w; the epilogue multiplies the result by
//     rs = 1 / sqrt(sum(h^2) / K + eps), the sum coming from the partial sums.
//
// Reference for the role: the projections of the reference are nn.Linear (models/self_attn.py:358-386,
// models/feedback.py:28-34); its fused variant merges up and gate the same way (models/feedback.py:52-62).
#include "common.cuh"

namespace q3 {

constexpr int GS_WARPS = 8;
constexpr int GS_UNROLL = 4;  // groups of 32 k-values fetched before they are multiplied

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  // weights are read once: do not keep them in L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// NT: token tiles of 8 (1 or 2).  WK: warps that share a group of 16 features and split K.
// EPI: 0 store, 1 SwiGLU on alternating blocks of eight rows, 2 added into the float32 stream.
// (The kernel is asked to fit three blocks per SM where K is not split in the block, which is the long
// stream of the output head, and with two token tiles: there, left to itself, the compiler used fewer registers
// than three blocks allow and took the loads one after the other.  Two token tiles are short of registers at
// three blocks per SM, though: where the grid fits two blocks per SM (ROOMY) the kernel is asked for two.  A warp
// that fetches two or three batches ahead gets all the registers it wants.  Figures:
// profiles/gemm_skinny__decode_b8.md.)
// PRE: batches of GS_UNROLL groups whose weights are fetched before the wait on the kernel before.  A
// product with few output features (o_proj, down_proj: 64 groups of 16, one block each) gives a warp two or
// three batches; with all of them under way before the wait, what is left after it is one round trip for
// the activations instead of one more to memory per batch.
struct SkinnyFuse {
  const float* ss_in;   // NORMED: [ss_parts][16] partial sums of squares of the stream's rows
  int ss_parts;
  float eps;
  float* ss_out;        // EPI 2: [ceil(N / 16)][16] partial sums of squares of the rows after the add
  const float* next_w;  // EPI 2, optional: weight [N] of the norm that comes next, and
  __nv_bfloat16* scaled_out;  // [T, N]: the new rows times that weight, the operand of a NORMED product
  int early;            // EPI 2: the stream may be read ahead of the wait (the launch before did not write it)
};

constexpr int GS_SS_ROWS = 16;  // row pitch of the partial sums

// EPI 2: out is the float32 stream [T, N] and is added to.  NORMED (see the head of the file): X is the stream
// times a norm's weight (scaled_out of the product that last added into the stream), and the result is
// multiplied by the row's 1 / rms.
// ROOMY (two token tiles, one batch ahead): the grid fits two blocks per SM, so the thread may have their registers.
// TIGHT (one token tile, K split in the block, one batch ahead): the grid needs three blocks per SM to be resident
// at once (more than two per SM, at most three); left to two, its last blocks would run as a wave of their own
// that cannot fill the memory pipeline (products of 5,120 features: 320 blocks).
template <int NT, int WK, int EPI, typename OutT, int PRE = 1, bool NORMED = false, bool ROOMY = false, bool TIGHT = false>
__global__ void __launch_bounds__(GS_WARPS * 32,
                                  TIGHT ? 3
                                  : ((NT == 1 && WK > 1 && !(NORMED && PRE == 1)) || (NT == 2 && PRE > 1)) ? 1
                                  : (NT == 2 && ROOMY) ? 2 : 3)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ W,
                   OutT* __restrict__ out, int T, int N, int K, int ldo, const SkinnyFuse fuse) {
  constexpr int GROUPS = GS_WARPS / WK;  // feature groups per block
  __shared__ float red[GS_WARPS][16][8 * NT + 1];
  __shared__ float rs_s[8 * NT];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tid4 = lane & 3;
  const int group_in_block = warp / WK, ksplit = warp % WK;
  const int row0 = (blockIdx.x * GROUPS + group_in_block) * 16;
  const bool active = row0 < N;

  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

  // this warp's share of K, in groups of 32
  const int groups32 = (K + 31) / 32;  // K is a multiple of 8: a lane's 8 values are all inside K or all outside
  const int per = (groups32 + WK - 1) / WK;
  const int g_lo = ksplit * per, g_hi = active ? min(groups32, g_lo + per) : g_lo;
  const int r_lo = min(row0 + gid, N - 1), r_hi = min(row0 + gid + 8, N - 1);  // rows past N are clamped, not stored
  const __nv_bfloat16* w_lo = W + (size_t)r_lo * K + 8 * tid4;
  const __nv_bfloat16* w_hi = W + (size_t)r_hi * K + 8 * tid4;
  uint4 wl[PRE][GS_UNROLL], wh[PRE][GS_UNROLL];
  auto load_w = [&](int g0, uint4 (&lo)[GS_UNROLL], uint4 (&hi)[GS_UNROLL]) {
#pragma unroll
    for (int u = 0; u < GS_UNROLL; ++u) {
      const size_t k = (size_t)(g0 + u) * 32;
      const bool in = g0 + u < g_hi && k + 8 * tid4 < (size_t)K;
      lo[u] = in ? ldg_stream(w_lo + k) : make_uint4(0, 0, 0, 0);
      hi[u] = in ? ldg_stream(w_hi + k) : make_uint4(0, 0, 0, 0);
    }
  };
  // The weights do not depend on the kernel before this one: their first batches are already on their
  // way while that kernel finishes.  The activations are read only after the wait.
#pragma unroll
  for (int p = 0; p < PRE; ++p) load_w(g_lo + p * GS_UNROLL, wl[p], wh[p]);
  // EPI 2: the next norm's weight for this lane's feature (the same for all its elements)
  const float next_weight = (EPI == 2 && fuse.scaled_out != nullptr && active && row0 + (lane & 15) < N)
                                ? fuse.next_w[row0 + (lane & 15)] : 0.f;
  // EPI 2: the stream's values that this warp will add to (element e = lane + 32 j of its 16 x 8 NT results)
  float before[EPI == 2 ? 4 * NT : 1];
  if (EPI == 2 && fuse.early && ksplit == 0 && active) {
#pragma unroll
    for (int j = 0; j < 4 * NT; ++j) {
      const int e = lane + 32 * j, f = e & 15, tok = e >> 4;
      before[j] = (tok < T && row0 + f < N) ? reinterpret_cast<const float*>(out)[(size_t)tok * ldo + row0 + f] : 0.f;
    }
  }
  pdl_wait();
  pdl_launch_dependents();
  // NORMED: warp w sums the partial sums of squares of rows w and w + 8; the first ones per lane are asked
  // for here and added after the main loop, so that their latency runs beside the loop's
  constexpr int SS_EARLY = NT == 1 ? 8 : 2;  // per lane: 32 SS_EARLY partial sums per row (a stream 4,096 wide has 256)
  float ss_early[NT][SS_EARLY];
  if (NORMED) {
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      const int tok = i * 8 + warp;
#pragma unroll
      for (int j = 0; j < SS_EARLY; ++j) {
        const int p = lane + 32 * j;
        ss_early[i][j] = (tok < T && p < fuse.ss_parts) ? fuse.ss_in[(size_t)p * GS_SS_ROWS + tok] : 0.f;
      }
    }
  }
  const __nv_bfloat16* x_row[NT];
  bool x_ok[NT];
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    const int tok = i * 8 + gid;
    x_ok[i] = tok < T;
    x_row[i] = X + (size_t)(x_ok[i] ? tok : 0) * K + 8 * tid4;
  }
  auto multiply = [&](int g0, const uint4 (&lo)[GS_UNROLL], const uint4 (&hi)[GS_UNROLL]) {
    constexpr int XU = GS_UNROLL;  // groups whose activations are fetched together
#pragma unroll
    for (int u0 = 0; u0 < GS_UNROLL; u0 += XU) {
      uint4 xv[XU][NT];
#pragma unroll
      for (int u = 0; u < XU; ++u) {
        const size_t k = (size_t)(g0 + u0 + u) * 32;
        const bool in = g0 + u0 + u < g_hi && k + 8 * tid4 < (size_t)K;
#pragma unroll
          for (int i = 0; i < NT; ++i)
            xv[u][i] = (in && x_ok[i]) ? __ldg(reinterpret_cast<const uint4*>(x_row[i] + k)) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < XU; ++u)
#pragma unroll
        for (int i = 0; i < NT; ++i) {
          mma_16816(acc[i], lo[u0 + u].x, hi[u0 + u].x, lo[u0 + u].y, hi[u0 + u].y, xv[u][i].x, xv[u][i].y);
          mma_16816(acc[i], lo[u0 + u].z, hi[u0 + u].z, lo[u0 + u].w, hi[u0 + u].w, xv[u][i].z, xv[u][i].w);
        }
    }
  };
  int g0 = g_lo;
#pragma unroll
  for (int p = 0; p < PRE; ++p) {  // batches past the warp's share hold zeros and are skipped
    if (g0 < g_hi) multiply(g0, wl[p], wh[p]);
    g0 += GS_UNROLL;
  }
  for (; g0 < g_hi; g0 += GS_UNROLL) {
    load_w(g0, wl[0], wh[0]);
    multiply(g0, wl[0], wh[0]);
  }
  if (NORMED) {
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      const int tok = i * 8 + warp;
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < SS_EARLY; ++j) ss += ss_early[i][j];
      if (tok < T)
        for (int p = lane + 32 * SS_EARLY; p < fuse.ss_parts; p += 32) ss += fuse.ss_in[(size_t)p * GS_SS_ROWS + tok];
      ss = warp_sum(ss);
      if (lane == 0) rs_s[tok] = 1.0f / sqrtf(ss / (float)K + fuse.eps);
    }
  }
  // acc[i][0..1]: feature row0 + gid, tokens 8i + 2 tid4, +1;  acc[i][2..3]: feature row0 + gid + 8
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    red[warp][gid][i * 8 + 2 * tid4] = acc[i][0];
    red[warp][gid][i * 8 + 2 * tid4 + 1] = acc[i][1];
    red[warp][gid + 8][i * 8 + 2 * tid4] = acc[i][2];
    red[warp][gid + 8][i * 8 + 2 * tid4 + 1] = acc[i][3];
  }
  __syncthreads();
  if (ksplit != 0 || !active) return;
  if (EPI == 0) {
    // 16 features x T tokens; consecutive lanes take consecutive features of one token
    for (int e = lane; e < 16 * 8 * NT; e += 32) {
      const int f = e & 15, tok = e >> 4;
      if (tok >= T || row0 + f >= N) continue;
      float v = 0.f;
#pragma unroll
      for (int s = 0; s < WK; ++s) v += red[warp + s][f][tok];
      if (NORMED) v *= rs_s[tok];
      out[(size_t)tok * ldo + row0 + f] = from_float<OutT>(v);
    }
  } else if (EPI == 2) {
    // added into the stream; the 16 lanes that share a row leave the sum of squares of their new values
    float* stream = reinterpret_cast<float*>(out);
    if (!fuse.early) {  // all of them asked for before the first store, which the compiler could not prove apart from them
#pragma unroll
      for (int j = 0; j < 4 * NT; ++j) {
        const int e = lane + 32 * j, f = e & 15, tok = e >> 4;
        before[j] = (tok < T && row0 + f < N) ? stream[(size_t)tok * ldo + row0 + f] : 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < 4 * NT; ++j) {
      const int e = lane + 32 * j, f = e & 15, tok = e >> 4;
      const bool live = tok < T && row0 + f < N;
      float h = 0.f;
      if (live) {
        float v = 0.f;
#pragma unroll
        for (int s = 0; s < WK; ++s) v += red[warp + s][f][tok];
        h = before[j] + v;
        stream[(size_t)tok * ldo + row0 + f] = h;
        if (fuse.scaled_out != nullptr)
          fuse.scaled_out[(size_t)tok * ldo + row0 + f] = __float2bfloat16_rn(h * next_weight);
      }
      float sq = h * h;
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
      if (f == 0 && tok < T) fuse.ss_out[(size_t)(row0 >> 4) * GS_SS_ROWS + tok] = sq;
    }
  } else {
    // features 0..7 of the group are gate values, 8..15 the matching up values
    for (int e = lane; e < 8 * 8 * NT; e += 32) {
      const int f = e & 7, tok = e >> 3;
      if (tok >= T) continue;
      float gate = 0.f, up = 0.f;
#pragma unroll
      for (int s = 0; s < WK; ++s) {
        gate += red[warp + s][f][tok];
        up += red[warp + s][f + 8][tok];
      }
      if (NORMED) {
        gate *= rs_s[tok];
        up *= rs_s[tok];
      }
      out[(size_t)tok * ldo + (row0 >> 1) + f] = from_float<OutT>(up * (gate / (1.0f + expf(-gate))));
    }
  }
}

template <int NT, int EPI, typename OutT, bool NORMED = false>
static int gemm_skinny_launch(const void* X, const void* W, void* out, int T, int N, int K, int ldo,
                              cudaStream_t stream, SkinnyFuse fuse = SkinnyFuse{}) {
  if (EPI == 2) fuse.early = last_launch_was_plain(stream) ? 1 : 0;
  const int groups = (N + 15) / 16;
  const int sms = sm_count();
  // split K over more warps while that still leaves every warp at least 128 values of k and the
  // grid is short of about four blocks per SM
  int wk = 1;
  while (wk < GS_WARPS && (groups * wk * 2) / GS_WARPS < sms * 4 && K / (wk * 2) >= 128) wk *= 2;
  const int per_block = GS_WARPS / wk;
  const unsigned grid = (groups + per_block - 1) / per_block;
#define Q3_GS_GO(WK, PRE)                                                                                         \
  do {                                                                                                            \
    if (NT == 2 && PRE == 1 && grid <= 2u * (unsigned)sms)                                                                  \
      q3::launch(gemm_skinny_kernel<NT, WK, EPI, OutT, PRE, NORMED, NT == 2 && PRE == 1>, dim3(grid),             \
                 dim3(GS_WARPS * 32), 0, stream, (const __nv_bfloat16*)X, (const __nv_bfloat16*)W, (OutT*)out, T, N, K, \
                 ldo, fuse);                                                                                      \
    else if (NT == 1 && WK > 1 && PRE == 1 && grid > 2u * (unsigned)sms && grid <= 3u * (unsigned)sms)            \
      q3::launch(gemm_skinny_kernel<NT, WK, EPI, OutT, PRE, NORMED, false, (NT == 1 && (WK > 1) && PRE == 1)>,    \
                 dim3(grid), dim3(GS_WARPS * 32), 0, stream, (const __nv_bfloat16*)X, (const __nv_bfloat16*)W,    \
                 (OutT*)out, T, N, K, ldo, fuse);                                                                 \
    else                                                                                                          \
      q3::launch(gemm_skinny_kernel<NT, WK, EPI, OutT, PRE, NORMED, false>, dim3(grid), dim3(GS_WARPS * 32), 0,   \
                 stream, (const __nv_bfloat16*)X, (const __nv_bfloat16*)W, (OutT*)out, T, N, K, ldo, fuse);       \
  } while (0)
  // batches of a warp's share of K; up to three are fetched ahead of the wait, but only where the grid is one
  // block per SM or less (o_proj and down_proj of a narrow model: 64 blocks): the registers of three batches
  // leave room for one block per SM, and a larger grid would then run in waves whose later blocks fetch
  // nothing ahead
  const int batches = ((K + 31) / 32 + wk * GS_UNROLL - 1) / (wk * GS_UNROLL);
  const bool few_blocks = grid <= (unsigned)sms && (NT == 1 || EPI == 2);
  const int pre = few_blocks && wk == GS_WARPS ? (batches < 3 ? batches : 3) : 1;
  if (wk == 1) Q3_GS_GO(1, 1);
  else if (wk == 2) Q3_GS_GO(2, 1);
  else if (wk == 4) Q3_GS_GO(4, 1);
  else if (pre <= 1) Q3_GS_GO(8, 1);
  else if constexpr (NT == 1 || EPI == 2) {
    if (pre == 2) Q3_GS_GO(8, 2);
    else Q3_GS_GO(8, 3);
  }
#undef Q3_GS_GO
  if (EPI == 2) note_stream_written();
  return launch_status();
}

}  // namespace q3

// out[T, N] (row pitch ldo) = X[T, K] * W[N, K]^T for T <= 16; X, W bfloat16, K a multiple of 8.
// out_f32 != 0: float32 output, else bfloat16.  swiglu != 0: W's rows alternate gate/up in blocks of
// eight, N is a multiple of 16 and out is [T, N / 2].
extern "C" int q3_gemm_skinny(const void* X, const void* W, void* out, int T, int N, int K, int ldo, int out_f32,
                              int swiglu, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  if (T > 16 || K <= 0 || K % 8 || (swiglu && (N % 16 || out_f32))) return Q3_ERR_SIZE;
  if ((uintptr_t)X % 16 || (uintptr_t)W % 16) return Q3_ERR_ALIGN;
  using bf16 = __nv_bfloat16;
  if (swiglu) {
    if (T <= 8) return q3::gemm_skinny_launch<1, 1, bf16>(X, W, out, T, N, K, ldo, stream);
    return q3::gemm_skinny_launch<2, 1, bf16>(X, W, out, T, N, K, ldo, stream);
  }
  if (out_f32) {
    if (T <= 8) return q3::gemm_skinny_launch<1, 0, float>(X, W, out, T, N, K, ldo, stream);
    return q3::gemm_skinny_launch<2, 0, float>(X, W, out, T, N, K, ldo, stream);
  }
  if (T <= 8) return q3::gemm_skinny_launch<1, 0, bf16>(X, W, out, T, N, K, ldo, stream);
  return q3::gemm_skinny_launch<2, 0, bf16>(X, W, out, T, N, K, ldo, stream);
}

// The forms that take the norm kernels out of a decode step (see the head of the file), T <= 16.
// mode 2: x is bfloat16 [T, K]; out is the float32 stream [T, N] and becomes out + x W^T; ss_out
// ([ceil(N / 16)][16] floats) receives the partial sums of squares of the new rows; if next_w (float32 [N]) and
// scaled_out (bfloat16 [T, N]) are given, scaled_out = new rows * next_w, rounded once.
// mode 3: x is such a scaled operand [T, K] of a stream whose rows' sums of squares add up from ss_in
// ([ss_parts][16] floats): out[T, N] bfloat16 = rs * (x W^T) with rs = 1 / sqrt(sum / K + eps), which is
// rmsnorm(stream) W^T.  mode 4: the same with W's rows alternating gate/up in blocks of eight and
// out [T, N / 2] = up * silu(gate).
extern "C" int q3_gemm_skinny_fused(const void* x, const void* W, void* out, int T, int N, int K, int ldo, int mode,
                                    const float* ss_in, int ss_parts, float eps, float* ss_out, const float* next_w,
                                    void* scaled_out, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  if (T > 16 || K <= 0 || K % 8 || mode < 2 || mode > 4 || (mode == 4 && N % 16)) return Q3_ERR_SIZE;
  if ((uintptr_t)x % 16 || (uintptr_t)W % 16 || (uintptr_t)out % 16) return Q3_ERR_ALIGN;
  using bf16 = __nv_bfloat16;
  q3::SkinnyFuse fuse{};
  if (mode == 2) {
    if (!ss_out || ((next_w == nullptr) != (scaled_out == nullptr))) return Q3_ERR_SIZE;
    fuse.ss_out = ss_out;
    fuse.next_w = next_w;
    fuse.scaled_out = (bf16*)scaled_out;
    if (T <= 8) return q3::gemm_skinny_launch<1, 2, float>(x, W, out, T, N, K, ldo, stream, fuse);
    return q3::gemm_skinny_launch<2, 2, float>(x, W, out, T, N, K, ldo, stream, fuse);
  }
  if (!ss_in || ss_parts <= 0) return Q3_ERR_SIZE;
  fuse.ss_in = ss_in;
  fuse.ss_parts = ss_parts;
  fuse.eps = eps;
  if (mode == 4) {
    if (T <= 8) return q3::gemm_skinny_launch<1, 1, bf16, true>(x, W, out, T, N, K, ldo, stream, fuse);
    return q3::gemm_skinny_launch<2, 1, bf16, true>(x, W, out, T, N, K, ldo, stream, fuse);
  }
  if (T <= 8) return q3::gemm_skinny_launch<1, 0, bf16, true>(x, W, out, T, N, K, ldo, stream, fuse);
  return q3::gemm_skinny_launch<2, 0, bf16, true>(x, W, out, T, N, K, ldo, stream, fuse);
}
