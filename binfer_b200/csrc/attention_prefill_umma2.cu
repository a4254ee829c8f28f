// Causal flash attention for prompt portions on the 5th-generation tensor cores, second
// arrangement: one CTA per SM that takes TWO query tiles (256 consecutive queries of one
// portion, one head) and walks the keys once for both.
//
// attention_prefill_umma.cu puts two independent CTAs of 128 queries on an SM.  Each fetches
// its own K and V tiles and, with shared memory for only two stages, the copies of tile n+1
// cannot start before tile n-1 is wholly consumed; the chain "P V done -> copies -> S ready"
// is what bounds it.  Here the two query tiles share one ring of K/V stages: the same shared
// memory gives four stages, every K/V tile is fetched once for 256 queries instead of twice,
// and sixteen softmax warps (four per scheduler) hide each other's latencies.
//
//   warp 16     TMA producer: both Q tiles once; per key tile one cp.async.bulk.tensor copy
//               per (page, 64 columns) of K and of V, or one per 64 columns where the tile's
//               pages follow one another in the pool; four key tiles in flight; the block
//               table is read for 32 / (pages per tile) tiles at a time;
//   warps 17,18 one thread each issues the tcgen05.mma of one query tile: per key tile
//               S = Q K^T (into one of two S buffers of its own in tensor memory, so the
//               product of tile n+1 runs under the softmax of tile n), then O += P V with P
//               as the operand FROM TENSOR MEMORY, once the probabilities lie there.  All 512
//               columns of tensor memory are in use: 4 x 64 for S / P, 2 x 128 for O;
//   warps 0-7   softmax of query tile A, warps 8-15 of query tile B.  A warp takes 16 query
//               rows and reads their 64 scores in the shape of a tensor-core fragment
//               (tcgen05.ld.16x256b): a row lies in the four threads of a quad, so its
//               maximum and sum are two shuffles away and the warps of a group never wait
//               for each other.  Exponent reference that follows the maximum only when it
//               has grown by more than 8; O in tensor memory, rescaled only then.  P (bf16,
//               two keys a column, tcgen05.st.16x128b) goes over the first 32 columns of the
//               scores the warp has just read.
//
// Query tile A is the lower half of the 256 rows and needs up to two key tiles fewer than B
// (causal); its group then goes to its epilogue while B finishes.  A block whose second tile
// has no rows runs with group B idle.  Head size 128 only; the caller takes the first
// arrangement for head size 64 and for portions of at most 128 queries.
//
// Every mbarrier wait is bounded.  A barrier whose waiter could fall two phases behind exists
// once per parity of the tile number, so that its one-bit phase cannot alias: "P V of tile n
// done" (waited for only when O must be rescaled), and "P of tile n written" (a softmax
// group needs no answer from the MMA warp before it signals the next tile's P, while that
// warp may still be waiting for the other group's).  On a timeout
// the CTA sets BF_ERR_WAIT, all roles leave their loops, TMEM is freed and the CTA returns
// without storing.  No copy uses multicast.
#include <cuda.h>
#include <float.h>
#include <stdint.h>

#include "common.cuh"
#include "tma_utils.cuh"
#include "umma_utils.cuh"

namespace {

constexpr int A2_BM = 128;       // queries per tile; two tiles per CTA
constexpr int A2_BN = 64;        // keys per tile
constexpr int A2_STAGES = 4;
constexpr int A2_THREADS = 608;  // sixteen softmax warps, the TMA warp, two MMA warps
constexpr int A2_TMA_WARP = 16;
constexpr int A2_MMA_WARP = 17;  // 17 issues for query tile A, 18 for tile B
constexpr int A2_D = 128;

// Barrier among the 256 softmax threads of a group that also ANDs a predicate.
__device__ __forceinline__ bool group_all(int id, bool ok) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "barrier.cta.red.and.pred p, %2, 256, q;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)ok), "r"(id)
      : "memory");
  return r != 0;
}

__global__ void __launch_bounds__(A2_THREADS, 1)
prefill_attention_umma2_kernel(const __grid_constant__ CUtensorMap map_q,
                               const __grid_constant__ CUtensorMap map_k,
                               const __grid_constant__ CUtensorMap map_v,
                               const __grid_constant__ CUtensorMap map_k_run,
                               const __grid_constant__ CUtensorMap map_v_run,
                               const int* __restrict__ items,
                               const int* __restrict__ block_tables, int table_stride,
                               __nv_bfloat16* __restrict__ out, int nh, int nkv, int page_size,
                               int num_pages, int window, float scale_log2, int splits,
                               float* __restrict__ part_o, float* __restrict__ part_ml,
                               int* __restrict__ err) {
  constexpr int D = A2_D;
  constexpr int HALVES = D / 64;
  constexpr int QHALF_BYTES = A2_BM * 128;               // 128 query rows of 128 bytes
  constexpr int KHALF_BYTES = A2_BN * 128;               // 64 key rows of 128 bytes
  constexpr int Q_BYTES = HALVES * QHALF_BYTES;          // one Q tile
  constexpr int KV_BYTES = HALVES * KHALF_BYTES;         // one K (or V) tile of 64 keys
  constexpr int OH = D / 2;                              // O columns per softmax thread
  extern __shared__ __align__(16) uint8_t smem_raw[];
  uint8_t* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* Qs = base;                                    // [2][Q_BYTES]
  uint8_t* Ks = Qs + 2 * Q_BYTES;                        // [STAGES][KV_BYTES]
  uint8_t* Vs = Ks + A2_STAGES * KV_BYTES;               // [STAGES][KV_BYTES]
  float* xm = reinterpret_cast<float*>(Vs + A2_STAGES * KV_BYTES);   // [sums, references][2 groups][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(xm + 4 * 128);
  uint64_t* q_full = bars;                     // [1]
  uint64_t* kv_full = bars + 1;                // [STAGES]
  uint64_t* kv_empty = kv_full + A2_STAGES;    // [STAGES]
  uint64_t* s_full = kv_empty + A2_STAGES;     // [group][2]: one per S buffer
  uint64_t* p_full = s_full + 4;               // [group][2], 8 arrivals (one a warp): P of the tiles of that parity
  uint64_t* o_done = p_full + 4;               // [group][2]: P V of the tiles of that parity
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 4);
  volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  // with splits > 1 the keys of a block are shared out over `splits` CTAs, each of which leaves
  // an unnormalised O with its exponent reference and sum for the merge kernel below
  const int split = splits > 1 ? (int)blockIdx.y % splits : 0;
  const int* it = items + 4 * (splits > 1 ? (int)blockIdx.y / splits : (int)blockIdx.y);
  const int seq = it[0], row0 = it[1], qlen = it[2], pos0 = it[3];
  // The last query blocks see the most keys.  Blocks are handed out with x running fastest and
  // z slowest: z counts the query blocks down, so that the longest blocks of every head and
  // portion start first and the short ones fill in behind them (with the query block in x a
  // long block could start late and end alone: 80 us for 2048 tokens from position 0).
  const int qb = (int)gridDim.z - 1 - (int)blockIdx.z, h = blockIdx.x;
  if (qb * 2 * A2_BM >= qlen) return;
  const bool active_b = qb * 2 * A2_BM + A2_BM < qlen;
  const int g = h / (nh / nkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int* table = block_tables + (size_t)seq * table_stride;
  const int pages = A2_BN / page_size;

  const int p_first = pos0 + qb * 2 * A2_BM;                            // first row of tile A
  const int p_last_a = min(pos0 + qlen - 1, p_first + A2_BM - 1);
  const int p_last = active_b ? min(pos0 + qlen - 1, p_first + 2 * A2_BM - 1) : p_last_a;
  const int j_lo = window > 0 ? max(0, p_first - window + 1) : 0;
  int kt_first = j_lo / A2_BN;
  int tiles_a = p_last_a / A2_BN - kt_first + 1;
  int tiles = p_last / A2_BN - kt_first + 1;
  if (splits > 1) {                                       // this CTA's share of the key tiles
    const int b = tiles * split / splits, e = tiles * (split + 1) / splits;
    kt_first += b;
    tiles_a = max(0, min(tiles_a, e) - b);
    tiles = e - b;
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < A2_STAGES; ++s) {
      mbar_init(kv_full + s, 1);
      mbar_init(kv_empty + s, active_b ? 2 : 1);         // one arrival per MMA thread
    }
    for (int s = 0; s < 4; ++s) {
      mbar_init(s_full + s, 1);
      mbar_init(o_done + s, 1);
      mbar_init(p_full + s, 8);
    }
    *abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  constexpr int TMEM_COLS = 512;
  if (warp == A2_MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // columns: S of tile A (2 x 64), S of tile B (2 x 64), O of A (128), O of B (128)

  if (warp == A2_TMA_WARP) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0 && tiles > 0) {                        // (a share of the keys may be empty)
      mbar_expect_tx(q_full, 2 * Q_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int hh = 0; hh < HALVES; ++hh)
          tma_load_2d(Qs + t * Q_BYTES + hh * QHALF_BYTES, &map_q, q_full, h * D + hh * 64,
                      row0 + qb * 2 * A2_BM + t * A2_BM);
    }
    // The warp looks up the pages of several tiles at a time, lane (i, pg) the page pg of the
    // i-th of them: one gather of the block table per 32 / pages tiles, and per tile little
    // more than the wait for its stage and the copies.  (With a lookup, a fence and a dozen
    // warp-wide steps per tile this warp, which shares its scheduler with four softmax
    // warps, took 3 800 cycles a tile and the products waited for it.)
    const int tb = 32 / pages;                           // tiles per lookup
    const int my_i = lane / pages, my_pg = lane - my_i * pages;
    const unsigned gmask = (pages == 32 ? 0xffffffffu : ((1u << pages) - 1u)) << (my_i * pages);
    bool ok = true;
    for (int nb = 0; nb < tiles && ok && !*abort; nb += tb) {
      const int n_mine = nb + my_i;
      const int jp = (kt_first + n_mine) * A2_BN + my_pg * page_size;
      const bool wanted = my_i < tb && n_mine < tiles && jp <= p_last && jp + page_size > j_lo;
      int page = 0;
      if (wanted) {
        page = table[jp / page_size];
        if (page < 0 || page >= num_pages) {
          atomicOr(err, BF_ERR_PAGE);
          page = 0;
        }
      }
      // a tile whose pages lie one after the other in the pool (the pool hands them out so)
      // comes as one box of all its pages per half, instead of one box per page
      const int page0 = __shfl_sync(0xffffffffu, page, my_i * pages);
      const unsigned in_run = __ballot_sync(0xffffffffu, wanted && page == page0 + my_pg);
      const unsigned live = __ballot_sync(0xffffffffu, wanted);
      const bool run = pages > 1 && (in_run & gmask) == gmask;
      const uint32_t tile_bytes = (uint32_t)__popc(live & gmask) * page_size * D * 4;
      for (int i = 0; i < tb && nb + i < tiles; ++i) {
        const int n = nb + i, st = n % A2_STAGES;
        if (lane == 0 && n >= A2_STAGES)
          ok = mbar_wait(kv_empty + st, (uint32_t)(n / A2_STAGES - 1) & 1u, abort);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        uint8_t* vb = Vs + st * KV_BYTES;
        // V rows of pages that are not fetched must read as zero (the first tile of a
        // window, the last tile of the portion)
        const int t_first = (kt_first + n) * A2_BN;
        if (t_first + page_size <= j_lo || t_first + A2_BN - page_size > p_last) {
          for (int pg = 0; pg < pages; ++pg) {
            const int jq = t_first + pg * page_size;
            if (jq <= p_last && jq + page_size > j_lo) continue;
            for (int c = lane; c < page_size * 8 * HALVES; c += 32) {
              const int hh = c / (page_size * 8), rem = c - hh * page_size * 8;
              *reinterpret_cast<uint4*>(vb + hh * KHALF_BYTES + pg * page_size * 128 + rem * 16) =
                  make_uint4(0u, 0u, 0u, 0u);
            }
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
        }
        if (my_i == i) {                                 // the lanes that looked this tile up
          if (my_pg == 0) mbar_expect_tx(kv_full + st, tile_bytes);
          __syncwarp(gmask);
          if (run) {
            for (int j = my_pg; j < 2 * HALVES; j += pages) {
              const int hh = j >> 1;
              if (j & 1)
                bf_tma_load_4d(vb + hh * KHALF_BYTES, &map_v_run, kv_full + st, hh * 64, 0, g,
                               page0);
              else
                bf_tma_load_4d(Ks + st * KV_BYTES + hh * KHALF_BYTES, &map_k_run, kv_full + st,
                               hh * 64, 0, g, page0);
            }
          } else if (wanted) {
            const int y = (page * nkv + g) * page_size;
#pragma unroll
            for (int hh = 0; hh < HALVES; ++hh) {
              tma_load_2d(Ks + st * KV_BYTES + hh * KHALF_BYTES + my_pg * page_size * 128, &map_k,
                          kv_full + st, hh * 64, y);
              tma_load_2d(vb + hh * KHALF_BYTES + my_pg * page_size * 128, &map_v, kv_full + st,
                          hh * 64, y);
            }
          }
        }
      }
    }
  } else if (warp >= A2_MMA_WARP) {
    // ----------------------------------------------------------------- MMA issuers
    // One thread per query tile: issuing a tcgen05.mma costs the issuing thread about a
    // hundred cycles whatever its size, and with one thread for both tiles that, not the
    // tensor pipe (a quarter busy), set the pace.  The two threads' products touch disjoint
    // tensor memory; they share the K and V tiles, which are released when both have arrived.
    const int grp = warp - A2_MMA_WARP;
    const int my_tiles = grp == 0 ? tiles_a : (active_b ? tiles : 0);
    if (lane == 0) {
      // S: a = Q (K-major), b = K tile (K-major), N = 64 keys
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) |
                               ((uint32_t)(A2_BN >> 3) << 17) | ((uint32_t)(A2_BM >> 4) << 24);
      // O: a = P (K-major), b = V as stored (MN-major), N = head size
      const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                               ((uint32_t)(D >> 3) << 17) | ((uint32_t)(A2_BM >> 4) << 24);
      const uint32_t q_addr = smem_u32(Qs + grp * Q_BYTES);
      auto issue_s = [&](int n) {                        // S of tile n into S buffer n & 1
        const uint32_t k_addr = smem_u32(Ks + (n % A2_STAGES) * KV_BYTES);
        const uint32_t d_addr = tmem_base + (uint32_t)(grp * 128 + (n & 1) * A2_BN);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t qo = (uint32_t)((k >> 2) * QHALF_BYTES + (k & 3) * 32);
          const uint32_t ko = (uint32_t)((k >> 2) * KHALF_BYTES + (k & 3) * 32);
          umma_bf16(d_addr, umma_desc_k_sw128(q_addr + qo), umma_desc_k_sw128(k_addr + ko),
                    idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(s_full + grp * 2 + (n & 1));
      };
      bool ok = my_tiles == 0 || (mbar_wait(q_full, 0, abort) && mbar_wait(kv_full, 0, abort));
      if (ok && my_tiles > 0) {
        tc_fence_after();
        issue_s(0);
      }
      for (int n = 0; n < my_tiles && ok; ++n) {
        const int st = n % A2_STAGES;
        if (n + 1 < my_tiles) {
          // the next tile's product runs under this tile's softmax; its S buffer is free
          // since the group signalled P of the tile before this one
          const int s1 = (n + 1) % A2_STAGES;
          if (!(ok = mbar_wait(kv_full + s1, (uint32_t)((n + 1) / A2_STAGES) & 1u, abort))) break;
          tc_fence_after();
          issue_s(n + 1);
        }
        if (!(ok = mbar_wait(p_full + grp * 2 + (n & 1), (uint32_t)(n >> 1) & 1u, abort))) break;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(Vs + st * KV_BYTES);
        const uint32_t d_addr = tmem_base + (uint32_t)(256 + grp * 128);
        // P lies over the first 32 columns of the tile's S buffer, two keys a column; the
        // next product into that buffer (S of tile n + 2) is issued by this thread after
        // this one, and products of one thread run in the order issued
        const uint32_t p_tm = tmem_base + (uint32_t)(grp * 128 + (n & 1) * A2_BN);
#pragma unroll
        for (int k = 0; k < A2_BN / 16; ++k)
          umma_bf16_a_tmem(d_addr, p_tm + (uint32_t)(k * 8),
                           umma_desc_mn_sw128(v_addr + (uint32_t)(k * 2048), KHALF_BYTES),
                           idesc_o, (n > 0 || k > 0) ? 1u : 0u);
        umma_commit(o_done + grp * 2 + (n & 1));
        umma_commit(kv_empty + st);          // this thread's share: K and V of the tile
      }
      // tile A ends up to two key tiles before B: its thread still owes its arrival for the
      // stages of those tiles, each once the tile has been fetched (so that the arrival
      // cannot land in an earlier use of the stage)
      if (grp == 0 && active_b)
        for (int n = tiles_a; n < tiles && ok; ++n) {
          if (!(ok = mbar_wait(kv_full + n % A2_STAGES, (uint32_t)(n / A2_STAGES) & 1u, abort))) break;
          mbar_arrive(kv_empty + n % A2_STAGES);
        }
    }
  } else {
    // --------------------------------------------------------------------- softmax
    const int grp = warp >> 3;                           // 0: query tile A, 1: tile B
    const int my_tiles = grp == 0 ? tiles_a : (active_b ? tiles : 0);
    if (my_tiles > 0) {
      // A warp takes 16 query rows (16 lanes of its quarter of tensor memory) and all 64 keys
      // of a tile, in the shape of a tensor-core fragment: a row's scores lie in the four
      // threads of a quad, 16 each, and a thread holds two rows (r and r + 8).  The row's
      // maximum and sum are two shuffles away: the group's warps never wait for each other.
      const int wq = warp & 3, hb = (warp >> 2) & 1;
      const int q4 = lane & 3;
      const uint32_t lane_addr = (uint32_t)(wq * 32 + hb * 16) << 16;
      const uint32_t my_s = tmem_base + lane_addr + (uint32_t)(grp * 128);
      const uint32_t my_of = tmem_base + lane_addr + (uint32_t)(256 + grp * 128);
      int prr[2], jlr[2];
      bool validr[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int rr = wq * 32 + hb * 16 + (lane >> 2) + 8 * e;      // query row of the tile
        const int ll = qb * 2 * A2_BM + grp * A2_BM + rr;             // index inside the portion
        validr[e] = ll < qlen;
        prr[e] = pos0 + ll;
        jlr[e] = window > 0 ? max(0, prr[e] - window + 1) : 0;
      }
      uint64_t* my_s_full = s_full + grp * 2;
      uint64_t* my_o_done = o_done + grp * 2;
      float m_ref[2] = {-INFINITY, -INFINITY}, lsum[2] = {0.f, 0.f};
      bool alive = true;
      int n = 0;
      for (; n < my_tiles; ++n) {
        if (*abort || !mbar_wait(my_s_full + (n & 1), (uint32_t)(n >> 1) & 1u, abort)) {
          alive = false;
          break;
        }
        tc_fence_after();
        uint32_t v[32];            // v[4c + 2e + i]: row e, key column 8c + 2 q4 + i
        tmem_ld_frag64(my_s + (uint32_t)((n & 1) * A2_BN), v);
        const int t_lo = (kt_first + n) * A2_BN + 2 * q4;  // key of this thread's first column
        int hi[2], lo[2];          // last and first visible key, counted from t_lo
        bool need_mask[2];
        float tmax[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          hi[e] = validr[e] ? prr[e] - t_lo : -1;
          lo[e] = jlr[e] - t_lo;
          need_mask[e] = !validr[e] || t_lo + 63 > prr[e] || t_lo - 6 < jlr[e];
          float t2[2] = {-INFINITY, -INFINITY};
          if (need_mask[e]) {
#pragma unroll
            for (int c = 0; c < 8; ++c)
#pragma unroll
              for (int i = 0; i < 2; ++i)
                if (8 * c + i >= lo[e] && 8 * c + i <= hi[e])
                  t2[i] = fmaxf(t2[i], __uint_as_float(v[4 * c + 2 * e + i]));
          } else {
#pragma unroll
            for (int c = 0; c < 8; ++c)
              t2[c & 1] = max3f(t2[c & 1], __uint_as_float(v[4 * c + 2 * e]),
                                __uint_as_float(v[4 * c + 2 * e + 1]));
          }
          float t = fmaxf(t2[0], t2[1]);
          t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, 1));
          t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, 2));
          tmax[e] = t * scale_log2;                        // the scale is positive
        }
        float factor[2] = {1.f, 1.f};
        bool rescale = false;
#pragma unroll
        for (int e = 0; e < 2; ++e)
          if (tmax[e] > m_ref[e] + 8.f) {                  // also the first finite maximum
            const bool had = m_ref[e] != -INFINITY;        // before it, O and the sum are zero
            factor[e] = had ? exp2f(m_ref[e] - tmax[e]) : 0.f;
            rescale |= had;
            m_ref[e] = tmax[e];
          }
        if (n > 0 && __any_sync(0xffffffffu, rescale)) {
          // P V of the tile before must be complete; the warp goes on as one
          if (__all_sync(0xffffffffu, mbar_wait(my_o_done + ((n - 1) & 1),
                                                (uint32_t)((n - 1) >> 1) & 1u, abort))) {
            tc_fence_after();
            const float f0 = factor[0] == 0.f ? 1.f : factor[0];   // 0: the row had nothing yet
            const float f1 = factor[1] == 0.f ? 1.f : factor[1];
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 64) {
              uint32_t w[32];
              tmem_ld_frag64(my_of + c0, w);
#pragma unroll
              for (int c = 0; c < 8; ++c) {
                w[4 * c] = __float_as_uint(__uint_as_float(w[4 * c]) * f0);
                w[4 * c + 1] = __float_as_uint(__uint_as_float(w[4 * c + 1]) * f0);
                w[4 * c + 2] = __float_as_uint(__uint_as_float(w[4 * c + 2]) * f1);
                w[4 * c + 3] = __float_as_uint(__uint_as_float(w[4 * c + 3]) * f1);
              }
              tmem_st_frag64(my_of + c0, w);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          }
        }
        uint32_t packed[16];       // packed[2c + e]: row e, keys 8c + 2 q4, + 1 = P column 4c + q4
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          lsum[e] *= factor[e];
          const float m_use = m_ref[e] == -INFINITY ? 0.f : m_ref[e];
          float ts0 = 0.f, ts1 = 0.f;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            float x0, x1;
            fma2f(x0, x1, __uint_as_float(v[4 * c + 2 * e]), __uint_as_float(v[4 * c + 2 * e + 1]),
                  scale_log2, -m_use);
            float e0 = ex2_approx(x0), e1 = ex2_approx(x1);
            if (need_mask[e]) {
              if (8 * c < lo[e] || 8 * c > hi[e]) e0 = 0.f;
              if (8 * c + 1 < lo[e] || 8 * c + 1 > hi[e]) e1 = 0.f;
            }
            add2f(ts0, ts1, e0, e1);
            __nv_bfloat162 p2 = __floats2bfloat162_rn(e0, e1);
            packed[2 * c + e] = *reinterpret_cast<uint32_t*>(&p2);
          }
          lsum[e] += ts0 + ts1;
        }
        // P over the first 32 columns of S, in this warp's 16 lanes: scores it has read
        tmem_st_frag32(my_s + (uint32_t)((n & 1) * A2_BN), packed);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full + grp * 2 + (n & 1));
      }
      // a row's sum lies in the threads of its quad
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        lsum[e] += __shfl_xor_sync(0xffffffffu, lsum[e], 1);
        lsum[e] += __shfl_xor_sync(0xffffffffu, lsum[e], 2);
      }
      float* xl = xm + grp * 128;
      float* xr = xm + 256 + grp * 128;                    // the rows' exponent references
      if (q4 == 0) {
        xl[wq * 32 + hb * 16 + (lane >> 2)] = lsum[0];
        xl[wq * 32 + hb * 16 + (lane >> 2) + 8] = lsum[1];
        xr[wq * 32 + hb * 16 + (lane >> 2)] = m_ref[0];
        xr[wq * 32 + hb * 16 + (lane >> 2) + 8] = m_ref[1];
      }
      // O leaves row by row: thread r of a quarter takes row r, each of the two warps of a
      // quarter one half of its columns
      const int half = hb;
      const int r = wq * 32 + lane;
      const int l = qb * 2 * A2_BM + grp * A2_BM + r;
      const bool valid = l < qlen;
      const uint32_t my_o = tmem_base + ((uint32_t)(wq * 32) << 16) +
                            (uint32_t)(256 + grp * 128 + half * OH);
      const int bar_id = 1 + grp;
      bool ok = alive && !*abort &&
                mbar_wait(my_o_done + ((my_tiles - 1) & 1), (uint32_t)((my_tiles - 1) >> 1) & 1u,
                          abort);
      ok = group_all(bar_id, ok);
      if (ok && splits > 1) {
        // unnormalised, for the merge: O in float, the reference and the sum beside it
        tc_fence_after();
        const size_t slot = ((size_t)(row0 + l) * nh + h) * splits + split;
        float* dst = part_o + slot * D + half * OH;
#pragma unroll 1
        for (int c0 = 0; c0 < OH; c0 += 32) {
          uint32_t w[32];
          tmem_ld32(my_o + c0, w);
          if (valid) {
#pragma unroll
            for (int c = 0; c < 32; c += 4)
              *reinterpret_cast<uint4*>(dst + c0 + c) = make_uint4(w[c], w[c + 1], w[c + 2], w[c + 3]);
          }
        }
        if (valid && half == 0) {
          part_ml[slot * 2] = xr[r];
          part_ml[slot * 2 + 1] = xl[r];
        }
      } else if (ok) {
        tc_fence_after();
        const float inv = 1.f / xl[r];
        __nv_bfloat16* dst = out + ((size_t)(row0 + l) * nh + h) * D + half * OH;
#pragma unroll 1
        for (int c0 = 0; c0 < OH; c0 += 32) {
          uint32_t w[32];
          tmem_ld32(my_o + c0, w);                         // the whole warp loads; valid rows store
          if (valid) {
#pragma unroll
            for (int c = 0; c < 32; c += 8) {
              uint4 o4;
              __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
              for (int j = 0; j < 4; ++j)
                o2[j] = __floats2bfloat162_rn(__uint_as_float(w[c + 2 * j]) * inv,
                                              __uint_as_float(w[c + 2 * j + 1]) * inv);
              *reinterpret_cast<uint4*>(dst + c0 + c) = o4;
            }
          }
        }
      }
      tc_fence_before();
    } else if (splits > 1 && (grp == 0 || active_b) && ((warp >> 2) & 1) == 0) {
      // no key tile of this share for the group's rows: a partial that the merge passes over
      const int l = qb * 2 * A2_BM + grp * A2_BM + (warp & 3) * 32 + lane;
      if (l < qlen) {
        const size_t slot = ((size_t)(row0 + l) * nh + h) * splits + split;
        part_ml[slot * 2] = -INFINITY;
        part_ml[slot * 2 + 1] = 0.f;
      }
    }
  }

  __syncthreads();
  if (*abort && threadIdx.x == 0) atomicOr(err, BF_ERR_WAIT);
  if (warp == A2_MMA_WARP) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
}

// The splits of a (query row, head) made one: out = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M),
// M the largest reference.  A warp per (row, head), a lane four of the 128 columns, the splits
// in ascending order.
__global__ void prefill_attention_merge_kernel(const float* __restrict__ part_o,
                                               const float* __restrict__ part_ml,
                                               const int* __restrict__ items,
                                               __nv_bfloat16* __restrict__ out, int nh, int splits) {
  const int* it = items + 4 * blockIdx.z;
  const int row0 = it[1], qlen = it[2];
  const int r = blockIdx.x * 4 + (threadIdx.x >> 5), h = blockIdx.y, lane = threadIdx.x & 31;
  if (r >= qlen) return;
  const size_t base = ((size_t)(row0 + r) * nh + h) * splits;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
  float L = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < splits; ++s) {
    const float m = part_ml[(base + s) * 2];
    if (m == -INFINITY) continue;                          // a share without keys for this row
    const float w = exp2f(m - M);
    L += part_ml[(base + s) * 2 + 1] * w;
    const float4 o = *reinterpret_cast<const float4*>(part_o + (base + s) * A2_D + lane * 4);
    acc.x += o.x * w;
    acc.y += o.y * w;
    acc.z += o.z * w;
    acc.w += o.w * w;
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  uint2 packed;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&packed);
  o2[0] = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
  o2[1] = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
  *reinterpret_cast<uint2*>(out + ((size_t)(row0 + r) * nh + h) * A2_D + lane * 4) = packed;
}

}  // namespace

// Arguments as bf_prefill_attention_umma, and: splits > 1 shares the keys of every block of 256
// queries out over that many CTAs (for few queries after many cached keys); part_o (float
// [total_rows, nh, splits, 128]) and part_ml (float [total_rows, nh, splits, 2]) take their
// partial results, which a second kernel merges.  Head size 128 only, pages of 8..64 keys that
// divide 64; cudaErrorInvalidValue otherwise (nothing launched).
BF_EXPORT int bf_prefill_attention_umma2(const void* q, const void* k_cache, const void* v_cache,
                                         const int* items, int n_items, int max_rows,
                                         int total_rows, const int* block_tables,
                                         int table_stride, void* out, int nh, int nkv, int d,
                                         int page_size, int num_pages, int window, float scale,
                                         int splits, float* part_o, float* part_ml, int* err,
                                         cudaStream_t stream) {
  if (n_items <= 0 || max_rows <= 0) return 0;
  if (splits < 1 || (splits > 1 && (!part_o || !part_ml))) return (int)cudaErrorInvalidValue;
  if (d != A2_D || nkv <= 0 || nh % nkv || page_size < 8 || page_size > A2_BN ||
      A2_BN % page_size || ((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) ||
      ((uintptr_t)v_cache & 15) || ((uintptr_t)out & 15))
    return (int)cudaErrorInvalidValue;
  CUtensorMap mq, mk, mv;
  int e = bf_make_tensor_map_bf16_2d(&mq, q, total_rows, (long long)nh * A2_D,
                                     (long long)nh * A2_D, A2_BM, 64);
  if (e) return e;
  const long long cache_rows = (long long)num_pages * nkv * page_size;
  e = bf_make_tensor_map_bf16_2d(&mk, k_cache, cache_rows, A2_D, A2_D, page_size, 64);
  if (e) return e;
  e = bf_make_tensor_map_bf16_2d(&mv, v_cache, cache_rows, A2_D, A2_D, page_size, 64);
  if (e) return e;
  CUtensorMap mkr, mvr;      // a whole tile of pages that follow one another
  e = bf_make_tensor_map_pages_bf16(&mkr, k_cache, num_pages, nkv, page_size, A2_D,
                                    A2_BN / page_size);
  if (e) return e;
  e = bf_make_tensor_map_pages_bf16(&mvr, v_cache, num_pages, nkv, page_size, A2_D,
                                    A2_BN / page_size);
  if (e) return e;
  // two Q tiles, the stages of K and V, the row sums, barriers
  const size_t smem = 1024 + (size_t)2 * 32768 + (size_t)2 * A2_STAGES * 16384 + 2048 + 256;
  auto kern = prefill_attention_umma2_kernel;
  static bool configured_on[BF_MAX_DEVICES];
  bool& configured = configured_on[bf_current_device()];
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)smem);
    if (ce != cudaSuccess) return (int)ce;
    configured = true;
  }
  dim3 grid(nh, n_items * splits, (max_rows + 2 * A2_BM - 1) / (2 * A2_BM));
  if (grid.y > 65535u || grid.z > 65535u) return (int)cudaErrorInvalidValue;
  kern<<<grid, A2_THREADS, smem, stream>>>(mq, mk, mv, mkr, mvr, items, block_tables, table_stride,
                                           (__nv_bfloat16*)out, nh, nkv, page_size, num_pages,
                                           window, scale * 1.4426950408889634f, splits, part_o, part_ml, err);
  if (splits > 1) {
    int st = bf_launch_status();
    if (st) return st;
    prefill_attention_merge_kernel<<<dim3((max_rows + 3) / 4, nh, n_items), 128, 0, stream>>>(
        part_o, part_ml, items, (__nv_bfloat16*)out, nh, splits);
  }
  return bf_launch_status();
}
