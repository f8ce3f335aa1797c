// Paged causal attention for prompt portions on the fifth-generation tensor cores (tcgen05),
// bfloat16, head size 64 or 128, pages of 8 to 64 tokens, no window.
//
// A block owns 128 query rows of one kv head (rows are (token, head-in-group) pairs as in
// attn_prefill.cu) and walks the keys in tiles of 128:
//   two loader warps (one for K, one for V): TMA brings the tile's pages into shared memory (128-byte
//                   swizzle), one box per page and per 64 values of the head, each lane issuing the
//                   boxes of one page; the page ids come from the block table, two tiles ahead; the
//                   tensor maps cover a layer's whole K (or V) pool.
//   issue thread    S = Q K^T   (tcgen05.mma, both operands K-major, accumulator: 128 TMEM columns)
//                   O += P V    (P from tensor memory, where it overwrites its own S; V MN-major from
//                                shared memory; accumulator: D columns)
//   512 softmax threads, four per query row (each takes 32 of the tile's 128 keys; they agree on
//                   the row maximum through shared memory): read S from TMEM (a thread owns a
//                   quarter of a row, no shuffles), mask the diagonal tile, keep a running
//                   reference maximum and denominator in float32, write P as bfloat16 pairs into
//                   the first 64 columns of the tile's S, and rescale O in TMEM when the reference
//                   maximum has to move (it moves only when the row maximum exceeds it by more
//                   than 2^8, so the rescale is rare after the first tiles; only then do the
//                   threads wait for the previous tile's P V).
// K and V tiles are double-buffered and so is S (with its P) in TMEM, so the loads, the next tile's
// Q K^T and the previous tile's P V run while the softmax threads work.  The time of a prompt is set by its last query tile, which walks
// every key one tile after the other: the more threads share a row, the shorter that chain.  One block per SM
// (164 KB of shared memory, all 512 TMEM columns).  All mbarrier waits are bounded (see tc_common.cuh).
//
// Reference for the math: kernels/triton/paged_attn.py:89-181 (online softmax with exp2, P rounded
// to the value dtype before P V), models/attn.py:388-400 (scale, causal on absolute positions).
#include "tc_common.cuh"

namespace q3 {

constexpr int AT_BM = 128;   // query rows per block
constexpr int AT_BN = 128;   // keys per tile
constexpr int AT_PARTS = 4;                    // softmax threads per query row
constexpr int AT_PART = AT_BN / AT_PARTS;      // keys per softmax thread: 32, one tcgen05.ld
constexpr int AT_SOFTMAX = AT_PARTS * AT_BM;   // softmax threads: warps 0..15
constexpr int AT_ISSUE_WARP = AT_SOFTMAX / 32, AT_LOAD_WARP = AT_ISSUE_WARP + 1;
constexpr int AT_THREADS = AT_SOFTMAX + 96;    // + issue warp and two loader warps (K, V)

template <int D>
struct AttnTcShape {
  static constexpr int ATOMS = D / 64;                 // 64-wide swizzle atoms along the head
  static constexpr int Q_BYTES = AT_BM * D * 2;
  static constexpr int K_BYTES = AT_BN * D * 2;
  static constexpr int V_BYTES = AT_BN * D * 2;
  static constexpr int BAR_BYTES = 128;
  static constexpr int XCHG_BYTES = 2 * AT_PARTS * AT_BM * 4;  // [tile parity][part][row]
  // K and V tiles are double-buffered; no slack for alignment: the dynamic shared memory of a block
  // that has no static shared memory starts on a 1024-byte boundary (checked in the kernel)
  static constexpr size_t SMEM_BYTES = (size_t)Q_BYTES + 2 * K_BYTES + 2 * V_BYTES + BAR_BYTES + XCHG_BYTES;
  static constexpr int TMEM_COLS = 512;                // S: two buffers of 128 columns at 0 and 128, O: D columns at 256
};

// byte offset of value (row, col) in a [rows x 64] bfloat16 tile with the 128-byte swizzle
__device__ __forceinline__ uint32_t sw128_offset(int row, int col) {
  return (uint32_t)row * 128u + ((((uint32_t)col >> 3) ^ ((uint32_t)row & 7u)) << 4) + (((uint32_t)col & 7u) << 1);
}

template <int D>
__global__ void __launch_bounds__(AT_THREADS, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
               const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
               const int* __restrict__ q_start, const int* __restrict__ kv_len,
               const int* __restrict__ block_table, int table_stride, int page_size, int num_pages, int Hq,
               int Hkv, float scale_log2, int* status) {
  using S = AttnTcShape<D>;
  constexpr int ATOMS = S::ATOMS;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* q_s = smem_raw;
  unsigned char* k_s = q_s + S::Q_BYTES;       // two stages
  unsigned char* v_s = k_s + 2 * S::K_BYTES;   // two stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + 2 * S::V_BYTES);
  uint64_t* k_full = bars + 0;   // [2]
  uint64_t* k_empty = bars + 2;  // [2]
  uint64_t* v_full = bars + 4;   // [2]
  uint64_t* v_empty = bars + 6;  // [2]
  uint64_t* s_ready = bars + 8;  // [2]
  uint64_t* p_ready = bars + 10;
  uint64_t* pv_done = bars + 11;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 12);
  int* abort_word = reinterpret_cast<int*>(bars + 13);
  float* row_xchg = reinterpret_cast<float*>(v_s + 2 * S::V_BYTES + S::BAR_BYTES);  // [2][parts][128] row maxima, then sums
#define abort_flag (*abort_word)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hk = blockIdx.x, b = blockIdx.z;
  const int g = Hq / Hkv;
  const int qs = q_start[b];
  const int q_len = q_start[b + 1] - qs;
  const int len = kv_len[b];
  const int total_rows = q_len * g;
  // Blocks are handed to the SMs in the order x, then y: the kv heads are x, so that the heaviest
  // query tiles (late queries, many keys) of all heads start first and the light ones fill the gaps.
  const int qt = (int)gridDim.y - 1 - (int)blockIdx.y;
  const int row0 = qt * AT_BM;
  if (row0 >= total_rows) return;  // before any barrier or allocation: the whole block leaves
  const int past = len - q_len;
  if (past < 0) {  // more new tokens than the request holds; also before any barrier or allocation
    if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
    return;
  }
  const int last_row = min(total_rows, row0 + AT_BM) - 1;
  const int pos_first = past + row0 / g, pos_last = past + last_row / g;
  const int n_tiles = pos_last / AT_BN + 1;
  const int* table = block_table + (size_t)b * table_stride;

  if (warp == AT_LOAD_WARP && lane == 0) tma_prefetch_map(&map_k);
  if (warp == AT_LOAD_WARP + 1 && lane == 0) tma_prefetch_map(&map_v);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    if (s_addr(smem_raw) & 1023u) {  // the swizzled tiles need this; never seen, but a wrong answer must not be silent
      abort_flag = 1;
      atomicOr(status, Q3_STATUS_TIMEOUT);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(k_full + i, 1);
      mbar_init(k_empty + i, 1);
      mbar_init(v_full + i, 1);
      mbar_init(v_empty + i, 1);
      mbar_init(s_ready + i, 1);
    }
    mbar_init(p_ready, AT_SOFTMAX / 32);
    mbar_init(pv_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_wait();  // q and the pages come from the kernels before this one
  pdl_launch_dependents();
  __syncthreads();  // the barriers exist; from here the loader warps go their own way until the end
  // Tensor memory is taken only after the wait: a block that holds TMEM while it waits for the
  // kernel before it could keep that kernel's own blocks from ever getting theirs.
  if (warp == AT_ISSUE_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_addr(tmem_holder)),
                 "r"((uint32_t)S::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }

  // the query tile, written in the swizzled K-major layout by the softmax threads; neighbouring
  // threads take neighbouring 16-byte chunks of a row, so a warp reads whole rows at a time
  if (warp < AT_ISSUE_WARP) {
    constexpr int CH = D / 8;                              // 16-byte chunks per row
    constexpr int PER_THREAD = AT_BM * CH / AT_SOFTMAX;    // 4 at D = 128, 2 at D = 64
    uint4 v[PER_THREAD];
#pragma unroll
    for (int i = 0; i < PER_THREAD; ++i) {
      const int idx = threadIdx.x + i * AT_SOFTMAX;
      const int r = idx / CH, c = idx % CH;
      const int R = row0 + r;
      v[i] = R < total_rows
                 ? *reinterpret_cast<const uint4*>(q + ((size_t)(qs + R / g) * Hq + hk * g + R % g) * D + c * 8)
                 : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < PER_THREAD; ++i) {
      const int idx = threadIdx.x + i * AT_SOFTMAX;
      const int r = idx / CH, c = idx % CH;
      *reinterpret_cast<uint4*>(q_s + (c / 8) * (AT_BM * 128) + sw128_offset(r, (c % 8) * 8)) = v[i];
    }
    fence_async_proxy();
  }
  uint32_t tmem_s = 0, tmem_o = 0;
  if (warp < AT_LOAD_WARP) {
    // the query tile and the tensor memory address, among the softmax and issue warps only: the
    // loaders are already fetching the first tiles meanwhile
    tcgen05_fence_before();
    asm volatile("bar.sync 2, %0;" ::"n"(AT_SOFTMAX + 32) : "memory");
    tcgen05_fence_after();
    tmem_s = *tmem_holder;           // S of tile j lives at column (j & 1) * 128
    tmem_o = tmem_s + 2 * AT_BN;
  }

  if (warp >= AT_LOAD_WARP) {
    // ------------------------------------------------------------------ loaders: one warp for K, one for V
    // Lane p of a loader warp owns page p of a tile: it looks its page id up two tiles ahead (so the
    // lookup's latency never stops the loop) and issues that page's boxes, so the sixteen lookups and
    // the copies of a tile go out together instead of one after the other.  Two warps, because one
    // warp alone does not issue the boxes of K and V (64 per tile at 16 tokens a page) fast enough.
    const bool is_v = warp != AT_LOAD_WARP;
    const CUtensorMap* map = is_v ? &map_v : &map_k;
    unsigned char* dst_base = is_v ? v_s : k_s;
    uint64_t* full = is_v ? v_full : k_full;
    uint64_t* empty = is_v ? v_empty : k_empty;
    const int pages_per_tile = AT_BN / page_size;
    auto page_id = [&](int j) -> int {  // lane's page of tile j, or -1 if the tile has no such page
      if (lane >= pages_per_tile || j >= n_tiles || j * AT_BN + lane * page_size >= len) return -1;
      return table_page(table, (j * AT_BN) / page_size + lane, table_stride, status);
    };
    int page = page_id(0), page_next = page_id(1);
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int st = j & 1;
      const uint32_t use = (uint32_t)j >> 1;
      const int page_after = page_id(j + 2);
      const bool wanted = lane < pages_per_tile && j * AT_BN + lane * page_size < len;
      if (wanted && (page < 0 || page >= num_pages)) {
        if (!is_v) atomicOr(status, Q3_STATUS_BAD_PAGE);
        page = -1;
      }
      const int y = page < 0 ? -1 : (page * Hkv + hk) * page_size;  // first row in the [pages * heads * page_size, D] view
      const uint32_t have = __popc(__ballot_sync(0xffffffffu, y >= 0));
      const uint32_t bytes = have * page_size * D * 2;
      if (use > 0) ok = ok && mbar_wait(empty + st, (use - 1) & 1, &abort_flag);
      const bool kept = is_v || j != tc_drop_copy;  // false only in the tests of the give-up path (see tc_common.cuh)
      if (lane == 0 && ok && kept) mbar_expect_tx(full + st, bytes);
      __syncwarp();
      if (y >= 0 && ok && kept) {
#pragma unroll
        for (int a = 0; a < ATOMS; ++a)
          tma_load_2d(dst_base + st * S::K_BYTES + a * (AT_BN * 128) + lane * page_size * 128, map, full + st, a * 64, y);
      }
      page = page_next;
      page_next = page_after;
    }
    if (!ok && lane == 0) {
      abort_flag = 1;
      atomicOr(status, Q3_STATUS_TIMEOUT);
    }
  } else if (warp == AT_ISSUE_WARP) {
    // ------------------------------------------------------------------ tensor-core issue
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc(AT_BN, 0);  // 128 x 128, K and Q both K-major
      constexpr uint32_t idesc_o = umma_idesc(D, 1);      // 128 x D, V MN-major
      // S of tile j + 1 is issued before the wait for tile j's probabilities, so it runs on the
      // tensor cores while the softmax threads work on tile j.
      // Descriptors are built once; inside the loops only constants are added to their address
      // field (in units of 16 bytes), so that the issuing thread is not held up by address arithmetic.
      const uint64_t q_desc = umma_desc_sw128(q_s);
      const uint64_t k_desc0 = umma_desc_sw128(k_s), k_desc1 = umma_desc_sw128(k_s + S::K_BYTES);
      const uint64_t v_desc0 = umma_desc_sw128_mn(v_s, AT_BN * 128), v_desc1 = umma_desc_sw128_mn(v_s + S::V_BYTES, AT_BN * 128);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(k_full + st, ((uint32_t)j >> 1) & 1, &abort_flag)) return false;
        tcgen05_fence_after();
        const uint64_t kd = st ? k_desc1 : k_desc0;
        const uint32_t acc = tmem_s + st * AT_BN;
#pragma unroll
        for (int t = 0; t < D / 16; ++t) {
          constexpr int ATOM16 = (AT_BM * 128) >> 4;  // one 64-wide atom of 128 rows, in 16-byte units
          umma_f16(acc, q_desc + (uint64_t)((t / 4) * ATOM16 + 2 * (t % 4)), kd + (uint64_t)((t / 4) * ATOM16 + 2 * (t % 4)),
                   idesc_s, t != 0);
        }
        umma_commit(s_ready + st);
        umma_commit(k_empty + st);
        return true;
      };
      bool ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1;
        if (j + 1 < n_tiles && !issue_s(j + 1)) { ok = false; break; }
        if (!mbar_wait(p_ready, j & 1, &abort_flag)) { ok = false; break; }
        if (!mbar_wait(v_full + st, ((uint32_t)j >> 1) & 1, &abort_flag)) { ok = false; break; }
        tcgen05_fence_after();
        const uint64_t vd = st ? v_desc1 : v_desc0;
        const uint32_t p_cols = tmem_s + st * AT_BN;
#pragma unroll
        for (int t = 0; t < AT_BN / 16; ++t)  // 16 keys: 8 packed columns of P, 16 rows (2048 bytes) of V
          umma_f16_ts(tmem_o, p_cols + 8 * t, vd + (uint64_t)(t * (2048 >> 4)), idesc_o, (j | t) != 0);
        umma_commit(pv_done);
        umma_commit(v_empty + st);
      }
      if (!ok) {
        abort_flag = 1;
        atomicOr(status, Q3_STATUS_TIMEOUT);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax, four threads per row
    // warps 4 p .. 4 p + 3 take keys 32 p .. 32 p + 31 of every tile; warp w sees TMEM lanes
    // (w % 4) * 32 .., i.e. row (w % 4) * 32 + lane.
    const int part = warp >> 2;
    const int rr = (warp & 3) * 32 + lane;
    const int R = row0 + rr;
    const bool valid_row = R < total_rows;
    const int my_pos = valid_row ? past + R / g : pos_last;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const int soft_tid = threadIdx.x;  // 0 .. 511
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    // Every softmax thread runs every iteration and meets the others at the named barrier even
    // after a wait has run out (the barrier itself cannot time out); `ok` only switches the work off.
    for (int j = 0; j < n_tiles; ++j) {
      const int st = j & 1;
      float* xchg = row_xchg + (j & 1) * (AT_PARTS * AT_BM);
      ok = ok && mbar_wait(s_ready + st, ((uint32_t)j >> 1) & 1, &abort_flag);
      tcgen05_fence_after();
      uint32_t sv[32];
      tmem_ld_32(tmem_s + st * AT_BN + part * AT_PART + lane_base, sv);
      tmem_wait_ld();
      const int base_n = j * AT_BN + part * AT_PART;
      float mx = -INFINITY;
      if (j * AT_BN + AT_BN - 1 > pos_first) {  // the diagonal: keys beyond this row's position are hidden
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const float v = (base_n + c <= my_pos) ? __uint_as_float(sv[c]) : -INFINITY;
          sv[c] = __float_as_uint(v);
          mx = fmaxf(mx, v);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c) mx = fmaxf(mx, __uint_as_float(sv[c]));
      }
      // the threads of a row agree on its maximum
      xchg[part * AT_BM + rr] = mx;
      asm volatile("bar.sync 1, %0;" ::"n"(AT_SOFTMAX) : "memory");
#pragma unroll
      for (int o = 0; o < AT_PARTS; ++o) mx = fmaxf(mx, xchg[o * AT_BM + rr]);
      mx *= scale_log2;
      // the reference maximum moves only when it must: probabilities up to 2^8 are harmless
      float alpha = 1.f;
      if (mx > m_ref + 8.f) {
        alpha = m_ref == -INFINITY ? 0.f : exp2f(m_ref - mx);
        m_ref = mx;
      }
      const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        // O belongs to the tensor cores until the previous tile's P V has finished
        ok = ok && mbar_wait(pv_done, (j - 1) & 1, &abort_flag);
        tcgen05_fence_after();
        // the row's threads rescale 32 output columns each (with D = 64 the first two of them)
        if (part * 32 < D) {
          uint32_t ov[32];
          tmem_ld_32(tmem_o + lane_base + part * 32, ov);
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * alpha);
          tmem_st_32(tmem_o + lane_base + part * 32, ov);
          tmem_wait_st();
        }
      }
      l *= alpha;
      float sum = 0.f;
      // P over the tile's own S: key k of the row goes to the half of column k / 2.  Every thread of
      // the row has its S in registers since the barrier above, so the columns may be overwritten.
      uint32_t pk[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        const float p0 = ex2_approx(fmaf(__uint_as_float(sv[2 * e]), scale_log2, -m_use));
        const float p1 = ex2_approx(fmaf(__uint_as_float(sv[2 * e + 1]), scale_log2, -m_use));
        sum += p0 + p1;
        pk[e] = pack2(__float_as_uint(p0), __float_as_uint(p1));
      }
      tmem_st_16(tmem_s + st * AT_BN + part * (AT_PART / 2) + lane_base, pk);
      tmem_wait_st();
      l += sum;
      // keys past the end of the sequence in the last tile: their V rows were not loaded; zero them
      if (j * AT_BN + AT_BN > len) {
        ok = ok && mbar_wait(v_full + st, ((uint32_t)j >> 1) & 1, &abort_flag);
        const int first_bad = len - j * AT_BN;
        for (int e = soft_tid; e < (AT_BN - first_bad) * (D / 8); e += AT_SOFTMAX) {
          const int key = first_bad + e / (D / 8), c = e % (D / 8);
          *reinterpret_cast<uint4*>(v_s + st * S::V_BYTES + (c / 8) * (AT_BN * 128) + sw128_offset(key, (c % 8) * 8)) =
              make_uint4(0, 0, 0, 0);
        }
      }
      // every thread has finished its own writes (the zeroed V rows go through the async proxy); one
      // arrival per warp then tells the issuing thread
      fence_async_proxy();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
    }
    if (!ok && lane == 0) {
      abort_flag = 1;
      atomicOr(status, Q3_STATUS_TIMEOUT);
    }
    // the last P V, then O / l with l summed over the row's threads; each writes 32 of the columns
    const bool done = ok && mbar_wait(pv_done, (n_tiles - 1) & 1, &abort_flag);
    float* xchg = row_xchg + (n_tiles & 1) * (AT_PARTS * AT_BM);
    xchg[part * AT_BM + rr] = l;
    asm volatile("bar.sync 1, %0;" ::"n"(AT_SOFTMAX) : "memory");
    if (done) {
      tcgen05_fence_after();
      float total = 0.f;
#pragma unroll
      for (int o = 0; o < AT_PARTS; ++o) total += xchg[o * AT_BM + rr];
      const float inv = total > 0.f ? 1.0f / total : 0.f;
      // The output tile goes through shared memory (where the query tile was: every product that read
      // it has finished), so that it leaves in whole rows instead of one 64-byte piece per thread.
      // Chunk c of row r sits at chunk position c ^ (r % CH) of its row, which spreads a warp's rows
      // over the banks.
      constexpr int CH = D / 8;
      if (part * 32 < D) {
        uint32_t ov[32];
        tmem_ld_32(tmem_o + lane_base + part * 32, ov);
        tmem_wait_ld();
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          uint4 pk;
          pk.x = pack2(__float_as_uint(__uint_as_float(ov[8 * v4 + 0]) * inv), __float_as_uint(__uint_as_float(ov[8 * v4 + 1]) * inv));
          pk.y = pack2(__float_as_uint(__uint_as_float(ov[8 * v4 + 2]) * inv), __float_as_uint(__uint_as_float(ov[8 * v4 + 3]) * inv));
          pk.z = pack2(__float_as_uint(__uint_as_float(ov[8 * v4 + 4]) * inv), __float_as_uint(__uint_as_float(ov[8 * v4 + 5]) * inv));
          pk.w = pack2(__float_as_uint(__uint_as_float(ov[8 * v4 + 6]) * inv), __float_as_uint(__uint_as_float(ov[8 * v4 + 7]) * inv));
          const int c = part * 4 + v4;
          *reinterpret_cast<uint4*>(q_s + rr * (D * 2) + ((c ^ (rr % CH)) << 4)) = pk;
        }
      }
    } else if (lane == 0) {
      abort_flag = 1;
      atomicOr(status, Q3_STATUS_TIMEOUT);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(AT_SOFTMAX) : "memory");
    if (done) {
      constexpr int CH = D / 8;
      constexpr int PER_THREAD = AT_BM * CH / AT_SOFTMAX;
#pragma unroll
      for (int i = 0; i < PER_THREAD; ++i) {
        const int idx = threadIdx.x + i * AT_SOFTMAX;
        const int r = idx / CH, c = idx % CH;
        const int Rr = row0 + r;
        if (Rr < total_rows)
          *reinterpret_cast<uint4*>(out + ((size_t)(qs + Rr / g) * Hq + hk * g + Rr % g) * D + c * 8) =
              *reinterpret_cast<const uint4*>(q_s + r * (D * 2) + ((c ^ (r % CH)) << 4));
      }
    }
  }
  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  if (warp == AT_ISSUE_WARP) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_s), "r"((uint32_t)S::TMEM_COLS)
                 : "memory");
  }
#undef abort_flag
}

template <int D>
static int attn_tc_launch(const void* q, const void* k_pages, const void* v_pages, void* out, const int* q_start,
                          const int* kv_len, const int* block_table, int table_stride, int page_size, int num_pages,
                          int B, int max_q_len, int Hq, int Hkv, float scale, int* status, cudaStream_t stream) {
  using S = AttnTcShape<D>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  CUtensorMap map_k, map_v;
  const uint64_t rows = (uint64_t)num_pages * Hkv * page_size;
  int code = cached_map(&map_k, k_pages, rows, D, (uint32_t)page_size);
  if (code) return code;
  code = cached_map(&map_v, v_pages, rows, D, (uint32_t)page_size);
  if (code) return code;
  const int g = Hq / Hkv;
  const long long tiles = ((long long)max_q_len * g + AT_BM - 1) / AT_BM;
  if (tiles > 65535) return Q3_ERR_SIZE;
  dim3 grid(Hkv, (unsigned)tiles, B);
  q3::launch(attn_tc_kernel<D>, grid, dim3(AT_THREADS), S::SMEM_BYTES, stream, map_k, map_v, (const __nv_bfloat16*)q,
             (__nv_bfloat16*)out, q_start, kv_len, block_table, table_stride, page_size, num_pages, Hq, Hkv,
             scale * 1.4426950408889634f, status);
  return launch_status();
}

}  // namespace q3

// For the tests of the give-up path: see set_wait_test in tc_common.cuh.
extern "C" int q3_attn_tc_wait_test(unsigned limit, int drop) { return q3::set_wait_test(limit, drop); }

// Same arguments as q3_attn_prefill, without a window.  Takes D = 64 or 128 and page sizes 8, 16, 32, 64;
// refuses the rest (the caller then uses q3_attn_prefill).
extern "C" int q3_attn_tc(const void* q, const void* k_pages, const void* v_pages, void* out, const int* q_start,
                          const int* kv_len, const int* block_table, int table_stride, int page_size, int num_pages,
                          int B, int max_q_len, int Hq, int Hkv, int D, float scale, int* status,
                          cudaStream_t stream) {
  if (B <= 0 || max_q_len <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv || (D != 64 && D != 128) || table_stride <= 0 || B > 65535 || Hkv > 65535 ||
      (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64))
    return Q3_ERR_SIZE;
  if ((uintptr_t)q % 16 || (uintptr_t)k_pages % 16 || (uintptr_t)v_pages % 16 || (uintptr_t)out % 16)
    return Q3_ERR_ALIGN;
  if (D == 64)
    return q3::attn_tc_launch<64>(q, k_pages, v_pages, out, q_start, kv_len, block_table, table_stride, page_size,
                                  num_pages, B, max_q_len, Hq, Hkv, scale, status, stream);
  return q3::attn_tc_launch<128>(q, k_pages, v_pages, out, q_start, kv_len, block_table, table_stride, page_size,
                                 num_pages, B, max_q_len, Hq, Hkv, scale, status, stream);
}
