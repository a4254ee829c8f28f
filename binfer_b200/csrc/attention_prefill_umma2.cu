// Causal flash attention for prompt portions on the 5th-generation tensor cores, second
// arrangement: one CTA per SM that takes TWO query tiles (256 consecutive queries of one
// portion, one head) and walks the keys once for both.
//
// attention_prefill_umma.cu puts two independent CTAs of 128 queries on an SM.  Each fetches
// its own K and V tiles and, with shared memory for only two stages, the copies of tile n+1
// cannot start before tile n-1 is wholly consumed; the chain "P V done -> copies -> S ready"
// is what bounds it.  Here the two query tiles share one ring of K/V stages: the same shared
// memory gives three stages, every K/V tile is fetched once for 256 queries instead of twice,
// and sixteen softmax warps (four per scheduler) hide each other's latencies.
//
//   warp 16     TMA producer: both Q tiles once; per key tile one cp.async.bulk.tensor copy
//               per (page, 64 columns) of K and of V, three key tiles in flight;
//   warps 17,18 one thread each issues the tcgen05.mma of one query tile: per key tile
//               S = Q K^T (into one of two S buffers of its own in tensor memory, so the
//               product of tile n+1 runs under the softmax of tile n), then O += P V as the
//               probabilities arrive.  All 512 columns of tensor memory are in use: 4 x 64
//               for S, 2 x 128 for O;
//   warps 0-7   softmax of query tile A, warps 8-15 of query tile B; in each group two threads
//               per query row, exactly as in attention_prefill_umma.cu (exponent reference
//               that follows the maximum only when it has grown by more than 8, O in tensor
//               memory, rescaled only then).  P_A is written over the K tile (dead once both
//               S products are done: a barrier per stage says when S_B is); P_B has two
//               buffers of its own.
//
// Query tile A is the lower half of the 256 rows and needs up to two key tiles fewer than B
// (causal); its group then goes to its epilogue while B finishes.  A block whose second tile
// has no rows runs with group B idle.  Head size 128 only; the caller takes the first
// arrangement for head size 64 and for portions of at most 128 queries.
//
// Every mbarrier wait is bounded.  A barrier whose waiter could fall two phases behind exists
// once per parity of the tile number, so that its one-bit phase cannot alias: "P V of tile n
// done" (waited for only when O must be rescaled or a P buffer reused), and "P of tile n
// written" (a softmax group needs no answer from the MMA warp before it signals the next
// tile's P, while that warp may still be waiting for the other group's).  On a timeout
// the CTA sets BF_ERR_WAIT, all roles leave their loops, TMEM is freed and the CTA returns
// without storing.  No copy uses multicast.
#include <cuda.h>
#include <float.h>
#include <stdint.h>
#include <stdlib.h>

#include "common.cuh"
#include "tma_utils.cuh"
#include "umma_utils.cuh"

namespace {

constexpr int A2_BM = 128;       // queries per tile; two tiles per CTA
constexpr int A2_BN = 64;        // keys per tile
constexpr int A2_STAGES = 3;
constexpr int A2_THREADS = 608;  // sixteen softmax warps, the TMA warp, two MMA warps
constexpr int A2_TMA_WARP = 16;
constexpr int A2_MMA_WARP = 17;  // 17 issues for query tile A, 18 for tile B
constexpr int A2_D = 128;
constexpr int A2_STAGGER_CYCLES = 1200;

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
                               int num_pages, int window, float scale_log2, int stagger,
                               int p_tmem, int* __restrict__ err) {
  constexpr int D = A2_D;
  constexpr int HALVES = D / 64;
  constexpr int QHALF_BYTES = A2_BM * 128;               // 128 query rows of 128 bytes
  constexpr int KHALF_BYTES = A2_BN * 128;               // 64 key rows of 128 bytes
  constexpr int Q_BYTES = HALVES * QHALF_BYTES;          // one Q tile
  constexpr int KV_BYTES = HALVES * KHALF_BYTES;         // one K (or V) tile of 64 keys
  constexpr int P_BYTES = A2_BM * 128;                   // 128 queries x 64 keys (= KV_BYTES)
  constexpr int OH = D / 2;                              // O columns per softmax thread
  static_assert(P_BYTES == KV_BYTES, "P_A lies exactly over a K tile");
  extern __shared__ __align__(16) uint8_t smem_raw[];
  uint8_t* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* Qs = base;                                    // [2][Q_BYTES]
  uint8_t* Ks = Qs + 2 * Q_BYTES;                        // [STAGES][KV_BYTES]
  uint8_t* Vs = Ks + A2_STAGES * KV_BYTES;               // [STAGES][KV_BYTES]
  uint8_t* Pb = Vs + A2_STAGES * KV_BYTES;               // [2][P_BYTES]: P of query tile B
  float* xm = reinterpret_cast<float*>(Pb + 2 * P_BYTES);   // [2 groups][3][2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(xm + 2 * 3 * 256);
  uint64_t* q_full = bars;                     // [1]
  uint64_t* kv_full = bars + 1;                // [STAGES]
  uint64_t* kv_empty = kv_full + A2_STAGES;    // [STAGES]
  uint64_t* s_full = kv_empty + A2_STAGES;     // [group][2]: one per S buffer
  uint64_t* p_full = s_full + 4;               // [group][2], 256 arrivals: P of the tiles of that parity
  uint64_t* o_done = p_full + 4;               // [group][2]: P V of the tiles of that parity
  uint64_t* k_dead = o_done + 4;               // [STAGES]: S_B of the stage's tile is done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(k_dead + A2_STAGES);
  volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int* it = items + 4 * blockIdx.z;
  const int seq = it[0], row0 = it[1], qlen = it[2], pos0 = it[3];
  // the last query blocks see the most keys: they are launched first
  const int qb = (int)gridDim.x - 1 - (int)blockIdx.x, h = blockIdx.y;
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
  const int kt_first = j_lo / A2_BN;
  const int tiles_a = p_last_a / A2_BN - kt_first + 1;
  const int tiles = p_last / A2_BN - kt_first + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < A2_STAGES; ++s) {
      mbar_init(kv_full + s, 1);
      mbar_init(kv_empty + s, active_b ? 2 : 1);         // one arrival per MMA thread
      mbar_init(k_dead + s, 1);
    }
    for (int s = 0; s < 4; ++s) {
      mbar_init(s_full + s, 1);
      mbar_init(o_done + s, 1);
      mbar_init(p_full + s, 256);
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
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * Q_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int hh = 0; hh < HALVES; ++hh)
          tma_load_2d(Qs + t * Q_BYTES + hh * QHALF_BYTES, &map_q, q_full, h * D + hh * 64,
                      row0 + qb * 2 * A2_BM + t * A2_BM);
    }
    // the page ids of a tile are looked up one tile ahead of its copies
    auto lookup = [&](int n, bool& wanted) {
      const int jp = (kt_first + n) * A2_BN + lane * page_size;
      wanted = n < tiles && lane < pages && jp <= p_last && jp + page_size > j_lo;
      int page = 0;
      if (wanted) {
        page = table[jp / page_size];
        if (page < 0 || page >= num_pages) {
          atomicOr(err, BF_ERR_PAGE);
          page = 0;
        }
      }
      return page;
    };
    bool wanted_next;
    int page_next = lookup(0, wanted_next);
    for (int n = 0; n < tiles && !*abort; ++n) {
      const int st = n % A2_STAGES;
      const int page = page_next;
      const bool wanted = wanted_next;
      page_next = lookup(n + 1, wanted_next);
      bool ok = true;
      if (lane == 0 && n >= A2_STAGES)
        ok = mbar_wait(kv_empty + st, (uint32_t)(n / A2_STAGES - 1) & 1u, abort);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      // V rows of pages that are not fetched must read as zero
      uint8_t* vb = Vs + st * KV_BYTES;
      for (int pg = 0; pg < pages; ++pg) {
        const int jq = (kt_first + n) * A2_BN + pg * page_size;
        if (jq <= p_last && jq + page_size > j_lo) continue;
        for (int c = lane; c < page_size * 8 * HALVES; c += 32) {
          const int hh = c / (page_size * 8), rem = c - hh * page_size * 8;
          *reinterpret_cast<uint4*>(vb + hh * KHALF_BYTES + pg * page_size * 128 + rem * 16) =
              make_uint4(0u, 0u, 0u, 0u);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      const unsigned live = __ballot_sync(0xffffffffu, wanted);
      if (lane == 0)
        mbar_expect_tx(kv_full + st, (uint32_t)__popc(live) * page_size * D * 4);
      __syncwarp();
      // A tile whose pages lie one after the other in the pool (the pool hands them out
      // so) comes as one box of all its pages per half, instead of one box per page.
      const int page0 = __shfl_sync(0xffffffffu, page, 0);
      const bool run = pages > 1 && __all_sync(0xffffffffu, lane >= pages ||
                                                                (wanted && page == page0 + lane));
      if (run) {
        if (lane < 2 * HALVES) {
          const int hh = lane >> 1;
          if (lane & 1)
            bf_tma_load_4d(vb + hh * KHALF_BYTES, &map_v_run, kv_full + st, hh * 64, 0, g, page0);
          else
            bf_tma_load_4d(Ks + st * KV_BYTES + hh * KHALF_BYTES, &map_k_run, kv_full + st,
                           hh * 64, 0, g, page0);
        }
      } else if (wanted) {
        const int y = (page * nkv + g) * page_size;
#pragma unroll
        for (int hh = 0; hh < HALVES; ++hh) {
          tma_load_2d(Ks + st * KV_BYTES + hh * KHALF_BYTES + lane * page_size * 128, &map_k,
                      kv_full + st, hh * 64, y);
          tma_load_2d(vb + hh * KHALF_BYTES + lane * page_size * 128, &map_v, kv_full + st,
                      hh * 64, y);
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
    if (lane == 0 && my_tiles > 0) {
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
        if (grp == 1 && !p_tmem) umma_commit(k_dead + n % A2_STAGES);   // tile A may then write P over K
      };
      bool ok = mbar_wait(q_full, 0, abort) && mbar_wait(kv_full, 0, abort);
      // tile B starts about half a tile's softmax after tile A: the two groups then stay out
      // of step, one's exponentials under the other's loads, maxima and stores, instead of
      // queueing for the same unit at the same time.  (It cannot wait for A's first P instead:
      // A writes that over the K tile, which needs B's first product done.)
      if (ok && grp == 1 && tiles >= 8) {
        const long long t0 = clock64();
        while (clock64() - t0 < stagger) {
        }
      }
      if (ok) {
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
        const uint32_t p_addr = smem_u32(grp == 0 ? Ks + st * KV_BYTES : Pb + (n & 1) * P_BYTES);
        const uint32_t v_addr = smem_u32(Vs + st * KV_BYTES);
        const uint32_t d_addr = tmem_base + (uint32_t)(256 + grp * 128);
        if (p_tmem) {
          // P lies over the first 32 columns of the tile's S buffer, two keys a column
          const uint32_t p_tm = tmem_base + (uint32_t)(grp * 128 + (n & 1) * A2_BN);
#pragma unroll
          for (int k = 0; k < A2_BN / 16; ++k)
            umma_bf16_a_tmem(d_addr, p_tm + (uint32_t)(k * 8),
                             umma_desc_mn_sw128(v_addr + (uint32_t)(k * 2048), KHALF_BYTES),
                             idesc_o, (n > 0 || k > 0) ? 1u : 0u);
        } else {
#pragma unroll
          for (int k = 0; k < A2_BN / 16; ++k) {
            // 16 keys further: along K inside P's swizzled rows, two 8-row groups down in V
            umma_bf16(d_addr, umma_desc_k_sw128(p_addr + (uint32_t)(k * 32)),
                      umma_desc_mn_sw128(v_addr + (uint32_t)(k * 2048), KHALF_BYTES), idesc_o,
                      (n > 0 || k > 0) ? 1u : 0u);
          }
        }
        umma_commit(o_done + grp * 2 + (n & 1));
        umma_commit(kv_empty + st);          // this thread's share: K, V (and P_A) of the tile
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
      const int wq = warp & 3, half = (warp >> 2) & 1;
      const int r = wq * 32 + lane;                      // query row of the tile = TMEM lane
      const int l = qb * 2 * A2_BM + grp * A2_BM + r;    // index inside the portion
      const bool valid = l < qlen;
      const int pr = pos0 + l;
      const int jl = window > 0 ? max(0, pr - window + 1) : 0;
      const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
      const uint32_t my_s = tmem_base + lane_addr + (uint32_t)(grp * 128 + half * 32);
      const uint32_t my_o = tmem_base + lane_addr + (uint32_t)(256 + grp * 128 + half * OH);
      float* gx = xm + grp * 3 * 256;
      uint64_t* my_s_full = s_full + grp * 2;
      uint64_t* my_o_done = o_done + grp * 2;
      const int bar_id = 1 + grp;
      float m_ref = -INFINITY, lsum = 0.f;
      bool alive = true;
      int n = 0;
      for (; n < my_tiles; ++n) {
        const bool ok = !*abort && mbar_wait(my_s_full + (n & 1), (uint32_t)(n >> 1) & 1u, abort);
        tc_fence_after();
        uint32_t v[32];
        tmem_ld32(my_s + (uint32_t)((n & 1) * A2_BN), v);
        const int t_lo = (kt_first + n) * A2_BN + half * 32;   // first key of this thread's columns
        const bool need_mask = !valid || t_lo + 31 > pr || t_lo < jl;
        const int hi = valid ? pr - t_lo : -1;             // last visible column
        const int lo = jl - t_lo;                          // first visible column
        float t4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains, not one of 32
        if (need_mask) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j >= lo && j <= hi) t4[j & 3] = fmaxf(t4[j & 3], __uint_as_float(v[j]));
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) t4[j & 3] = fmaxf(t4[j & 3], __uint_as_float(v[j]));
        }
        float tmax = fmaxf(fmaxf(t4[0], t4[1]), fmaxf(t4[2], t4[3]));
        tmax *= scale_log2;                                // the scale is positive
        float* x = gx + (n & 1) * 256;
        x[half * 128 + r] = tmax;
        if (!group_all(bar_id, ok)) {
          alive = false;
          break;
        }
        tmax = fmaxf(tmax, x[(half ^ 1) * 128 + r]);       // both threads of the row now agree
        float factor = 1.f;
        bool rescale = false;
        if (tmax > m_ref + 8.f) {                          // also the first finite maximum
          rescale = m_ref != -INFINITY;                    // before it, O and the sum are zero
          factor = rescale ? exp2f(m_ref - tmax) : 0.f;
          m_ref = tmax;
        }
        if (n > 0 && __any_sync(0xffffffffu, rescale)) {
          // P V of the tile before must be complete; the warp goes on as one
          if (__all_sync(0xffffffffu, mbar_wait(my_o_done + ((n - 1) & 1),
                                                (uint32_t)((n - 1) >> 1) & 1u, abort))) {
            tc_fence_after();
            const float f = rescale ? factor : 1.f;
#pragma unroll 1
            for (int c0 = 0; c0 < OH; c0 += 32) {
              uint32_t w[32];
              tmem_ld32(my_o + c0, w);
#pragma unroll
              for (int j = 0; j < 32; ++j) w[j] = __float_as_uint(__uint_as_float(w[j]) * f);
              tmem_st32(my_o + c0, w);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          }
        }
        lsum *= factor;
        uint8_t* Ps = nullptr;
        if (p_tmem) {
          // nothing to wait for: the S buffer is this tile's own
        } else if (grp == 0) {
          Ps = Ks + ((n % A2_STAGES)) * KV_BYTES;          // over the K tile, dead once S_B is done too
          if (active_b)
            mbar_wait(k_dead + n % A2_STAGES, (uint32_t)(n / A2_STAGES) & 1u, abort);
        } else {
          Ps = Pb + (n & 1) * P_BYTES;
          // the buffer was read by P V of tile n - 2
          if (n >= 2) mbar_wait(my_o_done + (n & 1), (uint32_t)((n - 2) >> 1) & 1u, abort);
        }
        const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
        float tsum = 0.f;
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          float e0 = ex2_approx(fmaf(__uint_as_float(v[j]), scale_log2, -m_use));
          float e1 = ex2_approx(fmaf(__uint_as_float(v[j + 1]), scale_log2, -m_use));
          if (need_mask) {
            if (j < lo || j > hi) e0 = 0.f;
            if (j + 1 < lo || j + 1 > hi) e1 = 0.f;
          }
          tsum += e0 + e1;
          __nv_bfloat162 p2 = __floats2bfloat162_rn(e0, e1);
          packed[j >> 1] = *reinterpret_cast<uint32_t*>(&p2);
        }
        lsum += tsum;
        if (p_tmem) {
          // P over the first 32 columns of S (every thread of the row has read its S: the
          // barrier above lies between); 32 keys = 16 columns
          tmem_st16(tmem_base + lane_addr + (uint32_t)(grp * 128 + (n & 1) * A2_BN + half * 16),
                    packed);
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        } else {
          // 32 keys = four 16-byte chunks of this row
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const int c = half * 4 + q4;                   // chunk index along the 64 keys
            uint8_t* dst = Ps + r * 128 + ((c ^ (r & 7)) << 4);
            *reinterpret_cast<uint4*>(dst) = make_uint4(packed[4 * q4], packed[4 * q4 + 1],
                                                        packed[4 * q4 + 2], packed[4 * q4 + 3]);
          }
          // P is read by the tensor core through the async proxy
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        tc_fence_before();
        mbar_arrive(p_full + grp * 2 + (n & 1));
      }
      // the row's sum from both halves, then O
      bool ok = alive && !*abort &&
                mbar_wait(my_o_done + ((my_tiles - 1) & 1), (uint32_t)((my_tiles - 1) >> 1) & 1u,
                          abort);
      float* xl = gx + 512;
      xl[half * 128 + r] = lsum;
      ok = group_all(bar_id, ok);
      if (ok) {
        tc_fence_after();
        const float inv = 1.f / (xl[r] + xl[128 + r]);
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

}  // namespace

// Arguments as bf_prefill_attention_umma.  Head size 128 only, pages of 8..64 keys that
// divide 64; cudaErrorInvalidValue otherwise (nothing launched).
BF_EXPORT int bf_prefill_attention_umma2(const void* q, const void* k_cache, const void* v_cache,
                                         const int* items, int n_items, int max_rows,
                                         int total_rows, const int* block_tables,
                                         int table_stride, void* out, int nh, int nkv, int d,
                                         int page_size, int num_pages, int window, float scale,
                                         int* err, cudaStream_t stream) {
  if (n_items <= 0 || max_rows <= 0) return 0;
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
  // two Q tiles, three stages of K and V, two P buffers, the exchange arrays, barriers
  const size_t smem = 1024 + (size_t)2 * 32768 + (size_t)2 * A2_STAGES * 16384 +
                      (size_t)2 * 16384 + 2 * 3 * 1024 + 256;
  auto kern = prefill_attention_umma2_kernel;
  static bool configured_on[BF_MAX_DEVICES];
  bool& configured = configured_on[bf_current_device()];
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)smem);
    if (ce != cudaSuccess) return (int)ce;
    configured = true;
  }
  static const int p_tmem =
      getenv("BINFER_B200_ATTN_P_TMEM") ? atoi(getenv("BINFER_B200_ATTN_P_TMEM")) : 1;
  dim3 grid((max_rows + 2 * A2_BM - 1) / (2 * A2_BM), nh, n_items);
  kern<<<grid, A2_THREADS, smem, stream>>>(mq, mk, mv, mkr, mvr, items, block_tables, table_stride,
                                           (__nv_bfloat16*)out, nh, nkv, page_size, num_pages,
                                           window, scale * 1.4426950408889634f,
                                           A2_STAGGER_CYCLES, p_tmem, err);
  return bf_launch_status();
}
