// Causal flash attention for prompt portions on the 5th-generation tensor cores.
//
// A CTA takes 128 consecutive queries of one portion for one head and walks the keys in
// tiles of 64 (edges at multiples of 64 counted from position 0), every key and value
// coming from the paged bf16 cache.  Two CTAs share an SM, so that one's softmax runs
// while the other's products occupy the tensor cores:
//
//   warp 8      TMA producer: the Q tile once; per key tile one cp.async.bulk.tensor copy
//               per (page, 64 columns) of K and of V into 128-byte-swizzled shared memory,
//               two key tiles in flight;
//   warp 9      one thread issues tcgen05.mma: S = Q K^T (M = 128 queries, N = 64 keys,
//               K = head size) into one of two S buffers in tensor memory, and, once the
//               probabilities are written, O += P V (M = 128, N = head size, K = 64 keys;
//               V is read as stored, an MN-major operand).  O stays in tensor memory over
//               all key tiles;
//   warps 0-7   softmax, two threads per query row (row r = TMEM lane r; warps w and w + 4
//               read the same lanes): each reads 32 of the tile's 64 scores (tcgen05.ld),
//               masks, the two exchange their maxima through shared memory, write their
//               halves of P as bf16 into the swizzled A-operand tile (over the K tile, which
//               is dead by then, when the head size is 128) and keep their halves of the
//               row's sum.  The exponent's reference follows the running maximum only when
//               that has grown by more than 8; only then is O read, scaled and written
//               back (tcgen05.ld / st), each thread its half of the columns.
//
// S of the next tile is multiplied while the softmax warps work on this one.
// The reference's prefill attention is scalar, over whole prompts' fresh keys only
// (cuda/kernels/bf16_kernels.cu:873-1024); the engine's first kernel for this job is
// attention_prefill.cu (mma.sync), which stays for the sizes this one does not take:
// head sizes other than 64 and 128, pages that do not divide 64 or are shorter than 8.
//
// Pages wholly outside the tile's keys are not fetched; their V rows are zeroed (a zero
// probability times stale shared memory must not give a NaN).  Every mbarrier wait is
// bounded (about a second): on a timeout the CTA sets BF_ERR_WAIT, all roles leave their
// loops, TMEM is freed and the CTA returns without storing.  No copy uses multicast.
#include <cuda.h>
#include <float.h>
#include <stdint.h>

#include "common.cuh"
#include "tma_utils.cuh"
#include "umma_utils.cuh"

namespace {

constexpr int AU_BM = 128;       // queries per CTA
constexpr int AU_BN = 64;        // keys per tile
constexpr int AU_THREADS = 320;   // eight softmax warps, the TMA warp, the MMA warp
constexpr int AU_TMA_WARP = 8;
constexpr int AU_MMA_WARP = 9;

// Barrier among the 256 softmax threads that also ANDs a predicate.
__device__ __forceinline__ bool softmax_all(bool ok) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "barrier.cta.red.and.pred p, 1, 256, q;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)ok)
      : "memory");
  return r != 0;
}

template <int D>
__global__ void __launch_bounds__(AU_THREADS, 2)
prefill_attention_umma_kernel(const __grid_constant__ CUtensorMap map_q,
                              const __grid_constant__ CUtensorMap map_k,
                              const __grid_constant__ CUtensorMap map_v,
                              const __grid_constant__ CUtensorMap map_k_run,
                              const __grid_constant__ CUtensorMap map_v_run,
                              const int* __restrict__ items, const int* __restrict__ block_tables,
                              int table_stride, __nv_bfloat16* __restrict__ out, int nh, int nkv,
                              int page_size, int num_pages, int window, float scale_log2,
                              int* __restrict__ err) {
  constexpr int HALVES = D / 64;
  constexpr int QHALF_BYTES = AU_BM * 128;               // 128 query rows of 128 bytes
  constexpr int KHALF_BYTES = AU_BN * 128;               // 64 key rows of 128 bytes
  constexpr int Q_BYTES = HALVES * QHALF_BYTES;
  constexpr int KV_BYTES = HALVES * KHALF_BYTES;         // one K (or V) tile of 64 keys
  constexpr int P_BYTES = AU_BM * 128;                   // 128 queries x 64 keys
  constexpr bool P_OVER_K = KV_BYTES >= P_BYTES;         // P may lie over the dead K tile
  constexpr int TMEM_COLS = 256;                         // S twice 64 columns, O: D columns
  constexpr int OH = D / 2;                              // O columns per softmax thread
  extern __shared__ __align__(16) uint8_t smem_raw[];
  uint8_t* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* Qs = base;
  uint8_t* Ks = Qs + Q_BYTES;                            // [2][KV_BYTES]
  uint8_t* Vs = Ks + 2 * KV_BYTES;                       // [2][KV_BYTES]
  uint8_t* Psep = Vs + 2 * KV_BYTES;                     // used only when P cannot lie over K
  float* xm = reinterpret_cast<float*>(Psep + (P_OVER_K ? 0 : P_BYTES));   // [3][2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(xm + 3 * 256);
  uint64_t* q_full = bars;             // [1]
  uint64_t* kv_full = bars + 1;        // [2]
  uint64_t* kv_empty = bars + 3;       // [2]
  uint64_t* s_full = bars + 5;         // [2]  one per S buffer
  uint64_t* p_full = bars + 7;         // [2]  256 arrivals; one per parity of the tile number, so
                                       //      that the softmax threads cannot lap the MMA warp
  uint64_t* o_done = bars + 9;         // [1]  completes once per key tile, after its P V
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int* it = items + 4 * blockIdx.y;
  const int seq = it[0], row0 = it[1], qlen = it[2], pos0 = it[3];
  // the last query tiles see the most keys: they are launched first
  // (z, the slowest index of the hand-out, counts the query tiles down: the longest first)
  const int qt = (int)gridDim.z - 1 - (int)blockIdx.z, h = blockIdx.x;
  if (qt * AU_BM >= qlen) return;
  const int g = h / (nh / nkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int* table = block_tables + (size_t)seq * table_stride;
  const int pages = AU_BN / page_size;

  const int p_first = pos0 + qt * AU_BM;
  const int p_last = min(pos0 + qlen - 1, p_first + AU_BM - 1);
  const int j_lo = window > 0 ? max(0, p_first - window + 1) : 0;
  const int kt_first = j_lo / AU_BN, kt_last = p_last / AU_BN;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(kv_full + s, 1);
      mbar_init(kv_empty + s, 1);
      mbar_init(s_full + s, 1);
    }
    mbar_init(p_full, 256);
    mbar_init(p_full + 1, 256);
    mbar_init(o_done, 1);
    *abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == AU_MMA_WARP) {
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
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 2 * AU_BN;

  if (warp == AU_TMA_WARP) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
      for (int hh = 0; hh < HALVES; ++hh)
        tma_load_2d(Qs + hh * QHALF_BYTES, &map_q, q_full, h * D + hh * 64, row0 + qt * AU_BM);
    }
    uint32_t phase = 0;
    // the page ids of a tile are looked up one tile ahead of its copies
    auto lookup = [&](int kt, bool& wanted) {
      const int jp = kt * AU_BN + lane * page_size;
      wanted = kt <= kt_last && lane < pages && jp <= p_last && jp + page_size > j_lo;
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
    int page_next = lookup(kt_first, wanted_next);
    for (int kt = kt_first; kt <= kt_last && !*abort; ++kt) {
      const int buf = (kt - kt_first) & 1;
      const int page = page_next;
      const bool wanted = wanted_next;
      page_next = lookup(kt + 1, wanted_next);
      bool ok = true;
      if (lane == 0) ok = mbar_wait(kv_empty + buf, phase ^ 1, abort);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      // V rows of pages that are not fetched must read as zero
      uint8_t* vb = Vs + buf * KV_BYTES;
      for (int pg = 0; pg < pages; ++pg) {
        const int jq = kt * AU_BN + pg * page_size;
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
        mbar_expect_tx(kv_full + buf, (uint32_t)__popc(live) * page_size * D * 4);
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
            bf_tma_load_4d(vb + hh * KHALF_BYTES, &map_v_run, kv_full + buf, hh * 64, 0, g, page0);
          else
            bf_tma_load_4d(Ks + buf * KV_BYTES + hh * KHALF_BYTES, &map_k_run, kv_full + buf,
                           hh * 64, 0, g, page0);
        }
      } else if (wanted) {
        const int y = (page * nkv + g) * page_size;
#pragma unroll
        for (int hh = 0; hh < HALVES; ++hh) {
          tma_load_2d(Ks + buf * KV_BYTES + hh * KHALF_BYTES + lane * page_size * 128, &map_k,
                      kv_full + buf, hh * 64, y);
          tma_load_2d(vb + hh * KHALF_BYTES + lane * page_size * 128, &map_v, kv_full + buf,
                      hh * 64, y);
        }
      }
      if (buf == 1) phase ^= 1;
    }
  } else if (warp == AU_MMA_WARP) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // S: a = Q (K-major), b = K tile (K-major), N = 64 keys
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) |
                               ((uint32_t)(AU_BN >> 3) << 17) | ((uint32_t)(AU_BM >> 4) << 24);
      // O: a = P (K-major), b = V as stored (MN-major), N = head size
      const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                               ((uint32_t)(D >> 3) << 17) | ((uint32_t)(AU_BM >> 4) << 24);
      const uint32_t q_addr = smem_u32(Qs);
      auto issue_s = [&](int n) {                        // S of the n-th tile into S buffer n & 1
        const uint32_t k_addr = smem_u32(Ks + (n & 1) * KV_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t qo = (uint32_t)((k >> 2) * QHALF_BYTES + (k & 3) * 32);
          const uint32_t ko = (uint32_t)((k >> 2) * KHALF_BYTES + (k & 3) * 32);
          umma_bf16(tmem_s + (uint32_t)((n & 1) * AU_BN), umma_desc_k_sw128(q_addr + qo),
                    umma_desc_k_sw128(k_addr + ko), idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(s_full + (n & 1));
      };
      const int tiles = kt_last - kt_first + 1;
      bool ok = mbar_wait(q_full, 0, abort) && mbar_wait(kv_full, 0, abort);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int n = 0; n < tiles && ok; ++n) {
        const int buf = n & 1;
        if (n + 1 < tiles) {
          // S of the next tile runs under the softmax of this one; its buffer is free since
          // the softmax threads signalled P of the tile before this one
          if (!(ok = mbar_wait(kv_full + ((n + 1) & 1), ((n + 1) >> 1) & 1, abort))) break;
          tc_fence_after();
          issue_s(n + 1);
        }
        if (!(ok = mbar_wait(p_full + (n & 1), (uint32_t)(n >> 1) & 1u, abort))) break;
        tc_fence_after();
        const uint32_t p_addr = smem_u32(P_OVER_K ? Ks + buf * KV_BYTES : Psep);
        const uint32_t v_addr = smem_u32(Vs + buf * KV_BYTES);
#pragma unroll
        for (int k = 0; k < AU_BN / 16; ++k) {
          // 16 keys further: along K inside P's swizzled rows, two 8-row groups down in V
          umma_bf16(tmem_o, umma_desc_k_sw128(p_addr + (uint32_t)(k * 32)),
                    umma_desc_mn_sw128(v_addr + (uint32_t)(k * 2048), KHALF_BYTES), idesc_o,
                    (n > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(kv_empty + buf);       // K, V (and P) of this tile are free when done
        umma_commit(o_done);
      }
    }
  } else {
    // --------------------------------------------------------------------- softmax
    // Two threads per query row: warps 0-3 take keys 0..31 of a tile and the lower half of
    // O's columns, warps 4-7 keys 32..63 and the upper half (a warp reads the TMEM lanes
    // 32 * (warp % 4) onwards).  O stays in tensor memory across the tiles.  It, and the
    // running sum, refer to m_ref, which follows the running maximum only when that has
    // grown by more than 8 (a factor 256 in the probabilities, harmless in bf16 and float):
    // only then is O read, scaled and written back, and only by the warps that hold such a row.
    const int wq = warp & 3, half = warp >> 2;
    const int r = wq * 32 + lane;                        // query row of the tile = TMEM lane
    const int l = qt * AU_BM + r;                        // index inside the portion
    const bool valid = l < qlen;
    const int pr = pos0 + l;
    const int jl = window > 0 ? max(0, pr - window + 1) : 0;
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    const uint32_t my_o = tmem_o + lane_addr + (uint32_t)(half * OH);
    float m_ref = -INFINITY, lsum = 0.f;
    bool alive = true;
    int n = 0;
    for (int kt = kt_first; kt <= kt_last; ++kt, ++n) {
      const bool ok = !*abort && mbar_wait(s_full + (n & 1), (n >> 1) & 1, abort);
      tc_fence_after();
      uint32_t v[32];
      tmem_ld32(tmem_s + lane_addr + (uint32_t)((n & 1) * AU_BN + half * 32), v);
      const int t_lo = kt * AU_BN + half * 32;           // first key of this thread's columns
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
      float* x = xm + (n & 1) * 256;
      x[half * 128 + r] = tmax;
      if (!softmax_all(ok)) {
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
        if (__all_sync(0xffffffffu, mbar_wait(o_done, (n - 1) & 1, abort))) {
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
      if (!P_OVER_K && n > 0) mbar_wait(o_done, (n - 1) & 1, abort);   // P of the tile before was read
      const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
      uint8_t* Ps = P_OVER_K ? Ks + (n & 1) * KV_BYTES : Psep;
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
      // 32 keys = four 16-byte chunks of this row
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const int c = half * 4 + q4;                     // chunk index along the 64 keys
        uint8_t* dst = Ps + r * 128 + ((c ^ (r & 7)) << 4);
        *reinterpret_cast<uint4*>(dst) = make_uint4(packed[4 * q4], packed[4 * q4 + 1],
                                                    packed[4 * q4 + 2], packed[4 * q4 + 3]);
      }
      lsum += tsum;
      // P is read by the tensor core through the async proxy
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_before();
      mbar_arrive(p_full + (n & 1));
    }
    // the row's sum from both halves, then O
    bool ok = alive && !*abort && mbar_wait(o_done, (n - 1) & 1, abort);
    float* xl = xm + 512;
    xl[half * 128 + r] = lsum;
    ok = softmax_all(ok);
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

  __syncthreads();
  if (*abort && threadIdx.x == 0) atomicOr(err, BF_ERR_WAIT);
  if (warp == AU_MMA_WARP) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
}

template <int D>
int launch_umma(const void* q, const void* k_cache, const void* v_cache, const int* items,
                int n_items, int max_rows, int total_rows, const int* block_tables,
                int table_stride, void* out, int nh, int nkv, int page_size, int num_pages,
                int window, float scale, int* err, cudaStream_t stream) {
  CUtensorMap mq, mk, mv;
  int e = bf_make_tensor_map_bf16_2d(&mq, q, total_rows, (long long)nh * D, (long long)nh * D,
                                     AU_BM, 64);
  if (e) return e;
  const long long cache_rows = (long long)num_pages * nkv * page_size;
  e = bf_make_tensor_map_bf16_2d(&mk, k_cache, cache_rows, D, D, page_size, 64);
  if (e) return e;
  e = bf_make_tensor_map_bf16_2d(&mv, v_cache, cache_rows, D, D, page_size, 64);
  if (e) return e;
  CUtensorMap mkr, mvr;      // a whole tile of pages that follow one another
  e = bf_make_tensor_map_pages_bf16(&mkr, k_cache, num_pages, nkv, page_size, D,
                                    AU_BN / page_size);
  if (e) return e;
  e = bf_make_tensor_map_pages_bf16(&mvr, v_cache, num_pages, nkv, page_size, D,
                                    AU_BN / page_size);
  if (e) return e;
  constexpr int HALVES = D / 64;
  // Q, two stages of K and V, P apart only when it does not fit over a K tile, barriers
  const size_t smem = 1024 + (size_t)HALVES * 16384 + (size_t)4 * HALVES * 8192 +
                      (HALVES * 8192 >= 16384 ? 0 : 16384) + 3 * 1024 + 128;
  auto kern = prefill_attention_umma_kernel<D>;
  static bool configured_on[BF_MAX_DEVICES];
  bool& configured = configured_on[bf_current_device()];
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)smem);
    if (ce != cudaSuccess) return (int)ce;
    configured = true;
  }
  dim3 grid(nh, n_items, (max_rows + AU_BM - 1) / AU_BM);
  if (grid.y > 65535u || grid.z > 65535u) return (int)cudaErrorInvalidValue;
  kern<<<grid, AU_THREADS, smem, stream>>>(mq, mk, mv, mkr, mvr, items, block_tables, table_stride,
                                           (__nv_bfloat16*)out, nh, nkv, page_size, num_pages,
                                           window, scale * 1.4426950408889634f, err);
  return bf_launch_status();
}

}  // namespace

// Same arguments as bf_prefill_attention plus total_rows, the number of token rows of q (the
// extent of the Q tensor map).  Returns cudaErrorInvalidValue for head sizes and page sizes
// it does not take.
BF_EXPORT int bf_prefill_attention_umma(const void* q, const void* k_cache, const void* v_cache,
                                        const int* items, int n_items, int max_rows,
                                        int total_rows, const int* block_tables,
                                        int table_stride, void* out, int nh, int nkv, int d,
                                        int page_size, int num_pages, int window, float scale,
                                        int* err, cudaStream_t stream) {
  if (n_items <= 0 || max_rows <= 0) return 0;
  if (nkv <= 0 || nh % nkv || page_size < 8 || page_size > AU_BN || AU_BN % page_size ||
      ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) || ((uintptr_t)q & 15))
    return (int)cudaErrorInvalidValue;
  if (d == 128)
    return launch_umma<128>(q, k_cache, v_cache, items, n_items, max_rows, total_rows,
                            block_tables, table_stride, out, nh, nkv, page_size, num_pages,
                            window, scale, err, stream);
  if (d == 64)
    return launch_umma<64>(q, k_cache, v_cache, items, n_items, max_rows, total_rows,
                           block_tables, table_stride, out, nh, nkv, page_size, num_pages, window,
                           scale, err, stream);
  return (int)cudaErrorInvalidValue;
}

