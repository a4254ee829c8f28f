// Split-KV decode attention, third generation: one resident CTA per SM walks the work.
//
// The unit of work is the same as in attention_decode_tma.cu: (row, kv head, 128-key split),
// the kv head's query heads as the rows of the tensor-core tile, partial results to scratch,
// merged by decode_attention_merge_kernel.  What changes is who runs it.  There, every item
// is a CTA of its own whose life is a chain (look the pages up, fetch, compute, store) that
// nothing overlaps but the two other CTAs on the SM.  Here a CTA stays and takes items
// idx = blockIdx.x, blockIdx.x + gridDim.x, ...:
//
//   warp 0        producer.  Finds the item's row by bisection in a prefix sum kept in shared
//                 memory, looks its pages up and fetches the K tile (with the item's queries)
//                 and the V tile by TMA into a ring of tile slots, as far ahead as the ring
//                 allows, so the next items are in flight while this one is computed.
//   warps 1-4,    two consumer groups that take alternate items.  Inside a group each warp
//   warps 5-8     scores 32 of the 128 keys; the row maxima are exchanged through shared
//                 memory, so the probabilities of all four warps refer to one maximum and go,
//                 as bf16, into one [16, 128] tile; each warp then multiplies that tile with
//                 its quarter of V's columns and stores its quarter of the partial result
//                 straight from registers.
//
// Every tile is fetched whole: pages that lie outside the row's keys are replaced by page 0,
// the pool's scratch page, so a slot never holds stale bits, and a masked probability of
// zero always meets a finite V.  (The cache pool is allocated zeroed.)
//
// Takes head sizes 64, 128, 256, page sizes that divide 128 and are at least 8, up to 16
// query heads per kv head and up to DP_MAX_ROWS rows; the caller uses the second kernel for
// everything else.  All waits are bounded (about a second): the thread that gives up sets
// BF_ERR_WAIT, its group leaves together, and the others run into their own limits.
// No copy uses multicast.
#include <float.h>
#include <stdlib.h>

#include "common.cuh"
#include "mma_utils.cuh"
#include "tma_utils.cuh"

#define DP_SPLIT 128
#define DP_GROUPS 2
#define DP_THREADS (32 + DP_GROUPS * 128)
#define DP_MAX_ROWS 512
#define DP_MAX_SLOTS 8
#define DP_P_LD 136                        // bf16 elements per row of the probability tile

extern "C" int bf_decode_attention_merge(const float* part_o, const float* part_ml,
                                         const int* rows, const int* positions, void* out,
                                         int n_rows, int nh, int d, int window, int max_splits,
                                         cudaStream_t stream);

__device__ __forceinline__ int dp_sw_off(int r, int c) { return r * 64 + ((c ^ (r & 7)) << 3); }

__device__ __forceinline__ void dp_mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bf_smem_u32(bar)) : "memory");
}
// Barrier over `threads` threads that also tells every one of them whether all said ok.
__device__ __forceinline__ bool dp_group_all(int id, int threads, bool ok) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 p, %1, 0;\n\t"
      "barrier.cta.red.and.pred q, %2, %3, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)ok), "r"(id), "r"(threads)
      : "memory");
  return r != 0;
}
// Untiled bulk copy global -> shared; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void dp_bulk_load(void* smem_dst, const void* src, uint32_t bytes,
                                             uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(bf_smem_u32(smem_dst)),
      "l"(src), "r"(bytes), "r"(bf_smem_u32(bar))
      : "memory");
}

struct DpSmem {
  size_t bars, qbuf, pbuf, red, info, row_start, row_t, row_p, row_seq, total;
};
// Offsets from the 1024-byte aligned base; the same function lays shared memory out on the
// host (to size the launch) and in the kernel.
__host__ __device__ inline DpSmem dp_layout(int d, int slots, int groups, int G, int n_rows) {
  DpSmem s;
  const int qs = groups * ((slots / groups + 1) / 2);
  size_t o = (size_t)slots * DP_SPLIT * d * 2;
  s.bars = o;       o += 2 * DP_MAX_SLOTS * 8;
  s.qbuf = o;       o += (size_t)qs * G * d * 2;
  s.pbuf = o;       o += (size_t)DP_GROUPS * 2 * 16 * DP_P_LD * 2;
  s.red = o;        o += (size_t)DP_GROUPS * 2 * 2 * 64 * 4;
  s.info = o;       o += (size_t)qs * 8 * 4;
  s.row_start = o;  o += (size_t)(n_rows + 1) * 4;
  s.row_t = o;      o += (size_t)n_rows * 4;
  s.row_p = o;      o += (size_t)n_rows * 4;
  s.row_seq = o;    o += (size_t)n_rows * 4;
  s.total = o;
  return s;
}

struct DpItem {
  int r, g, split;
  int pg[4];                 // page ids of this lane's share of the tile (0: the scratch page)
};
// What the producer needs to fetch item `idx`: its row, kv head and split, and the ids of
// `pp` (at most 4) consecutive pages of its tile, those from logical page `first` of the
// tile on.  Pages outside the row's keys are replaced by page 0, the pool's scratch page.
// A tile's pages are looked up by pages / pp lanes, so that one round of lookups covers 8 to
// 32 items: with a lane per page it covered 4 items of eight 16-token pages, and the round's
// fixed cost (the bisection, the table's latency) showed in every item, 195 against 177 us at
// batch 64 for 16- against 64-token pages.
__device__ __forceinline__ DpItem dp_lookup(int idx, bool lane_on, int first, int pp, int total,
                                            int n_rows, int nkv, int page_size, int num_pages,
                                            int window, int table_stride, const int* row_start,
                                            const int* row_t, const int* row_p, const int* row_seq,
                                            const int* __restrict__ block_tables, int* err) {
  DpItem d = {0, 0, 0, {0, 0, 0, 0}};
  if (!lane_on || idx >= total) return d;
  int lo = 0, hi = n_rows - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (row_start[mid] <= idx) lo = mid; else hi = mid - 1;
  }
  const int rem = idx - row_start[lo];
  const int p = row_p[lo];
  const int j0 = window > 0 ? max(0, p - window + 1) : 0;
  d.r = lo;
  d.g = rem % nkv;
  d.split = j0 / DP_SPLIT + rem / nkv;
  const int* table = block_tables + (size_t)row_seq[lo] * table_stride;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int jp = d.split * DP_SPLIT + (first + e) * page_size;
    if (e < pp && jp <= p && jp + page_size > j0) d.pg[e] = table[jp / page_size];
  }
#pragma unroll
  for (int e = 0; e < 4; ++e)
    if (d.pg[e] < 0 || d.pg[e] >= num_pages) {
      atomicOr(err, BF_ERR_PAGE);
      d.pg[e] = 0;
    }
  return d;
}

template <int D>
__global__ void __launch_bounds__(DP_THREADS, 1)
decode_attention_persistent_kernel(const __grid_constant__ CUtensorMap map_k,
                                   const __grid_constant__ CUtensorMap map_v,
                                   const __grid_constant__ CUtensorMap map_k_run,
                                   const __grid_constant__ CUtensorMap map_v_run,
                                   const __nv_bfloat16* __restrict__ q,
                                   const int* __restrict__ rows,
                                   const int* __restrict__ seq_of_token,
                                   const int* __restrict__ positions,
                                   const int* __restrict__ block_tables, int table_stride,
                                   float* __restrict__ part_o, float* __restrict__ part_ml,
                                   int n_rows, int nh, int nkv, int page_size, int num_pages,
                                   int window, int max_splits, float scale_log2, int slots,
                                   int groups, int early, int* __restrict__ err) {
  constexpr int HALVES = D / 64;
  constexpr int HALF_ELEMS = DP_SPLIT * 64;
  constexpr int TILE_ELEMS = DP_SPLIT * D;
  constexpr uint32_t TILE_BYTES = TILE_ELEMS * 2;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned char* base = smem_raw + ((1024u - (bf_smem_u32(smem_raw) & 1023u)) & 1023u);
  const int G = nh / nkv;
  // Each consumer group has a ring of its own (spg slots, qsg query buffers): a slot is
  // then filled and read by the same parties in strict turn, which the one-bit phase of an
  // mbarrier needs.  (Were a slot shared, the group that reads its next fill could ask for
  // that phase while the fill before it is still in flight, and the parity would say yes.)
  const int spg = slots / groups, qsg = (spg + 1) / 2;
  const DpSmem L = dp_layout(D, slots, groups, G, n_rows);
  __nv_bfloat16* tiles = reinterpret_cast<__nv_bfloat16*>(base);
  uint64_t* full = reinterpret_cast<uint64_t*>(base + L.bars);
  uint64_t* empty = full + DP_MAX_SLOTS;
  __nv_bfloat16* qbuf = reinterpret_cast<__nv_bfloat16*>(base + L.qbuf);
  __nv_bfloat16* pbuf = reinterpret_cast<__nv_bfloat16*>(base + L.pbuf);
  float* red = reinterpret_cast<float*>(base + L.red);
  int* info = reinterpret_cast<int*>(base + L.info);
  int* row_start = reinterpret_cast<int*>(base + L.row_start);
  int* row_t = reinterpret_cast<int*>(base + L.row_t);
  int* row_p = reinterpret_cast<int*>(base + L.row_p);
  int* row_seq = reinterpret_cast<int*>(base + L.row_seq);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  BF_TRACE_POINT(10 * BF_TR_ATTN);
  bf_pdl_trigger();
  if (tid == 32) {
    for (int s = 0; s < slots; ++s) {
      bf_mbar_init(full + s, 1);
      bf_mbar_init(empty + s, 4);                        // the four warps of the group that read it
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // What follows reads the step's description (rows, positions, block tables) and, in the
  // producer, cache pages of keys that earlier steps wrote: none of it comes from the kernel
  // before this one, which writes this step's queries and this step's keys and values.  So it
  // runs ahead of the wait; only the queries and the splits that hold a row's newest key wait.
  if (warp == 0) {
    // items before each row: (splits the row's keys touch) x (kv heads), in row order
    int running = 0;
    for (int rb = 0; rb < n_rows; rb += 32) {
      const int r = rb + lane;
      int cnt = 0, t = 0, p = 0;
      if (r < n_rows) {
        t = rows ? rows[r] : r;
        p = positions[t];
        const int j0 = window > 0 ? max(0, p - window + 1) : 0;
        int last = p / DP_SPLIT;
        if (last >= max_splits) {        // splits without room in the scratch get no item
          atomicOr(err, BF_ERR_SPLITS);
          last = max_splits - 1;
        }
        cnt = max(0, last - j0 / DP_SPLIT + 1) * nkv;
      }
      int incl = cnt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      if (r < n_rows) {
        row_start[r] = running + incl - cnt;
        row_t[r] = t;
        row_p[r] = p;
        row_seq[r] = seq_of_token[t];
      }
      running += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) row_start[n_rows] = running;
  }
  __syncthreads();
  const int total = row_start[n_rows];
  const int pages = DP_SPLIT / page_size;
  if (warp != 0) bf_pdl_wait();                          // the producer waits further down

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    // Lookups go in batches: a tile has `pages` pages, so the warp's 32 lanes look the pages
    // of 32 / pages items up with one load each, and the batch after this one is looked up
    // before this one is issued: the table's latency is paid once per batch, and hidden.
    const int pp = pages < 4 ? pages : 4;                // pages a lane looks up
    const int per = pages / pp;                          // lanes per item: 1, 2 or 4
    const int nb = 32 / per;                             // items per batch (pages <= 16)
    const int sub = lane / per, first = (lane - sub * per) * pp;
    DpItem nxt = dp_lookup(blockIdx.x + sub * gridDim.x, sub < nb, first, pp, total, n_rows, nkv,
                           page_size, num_pages, window, table_stride, row_start, row_t, row_p,
                           row_seq, block_tables, err);
    bool failed = false;
    bool waited = false;
    if (!early) bf_pdl_wait(), waited = true;
    // the queries of the items issued before the wait are fetched right after it
    auto wait_then_queries = [&]() {
      bf_pdl_wait();
      BF_TRACE_POINT(10 * BF_TR_ATTN + 1);
      waited = true;
      if (lane == 0)
        for (int e = 0; e < groups * qsg; ++e) {
          int* inf = info + e * 8;
          if (inf[7]) {
            inf[7] = 0;
            dp_bulk_load(qbuf + (size_t)e * G * D,
                         q + ((size_t)inf[5] * nh + (size_t)inf[1] * G) * D,
                         (uint32_t)(G * D * 2), full + inf[6]);
          }
        }
      __syncwarp();
    };
    if (lane < groups * qsg) info[lane * 8 + 7] = 0;
    __syncwarp();
    for (int it0 = 0; !failed && blockIdx.x + it0 * gridDim.x < total; it0 += nb) {
      const DpItem cur = nxt;
      nxt = dp_lookup(blockIdx.x + (it0 + nb + sub) * gridDim.x, sub < nb, first, pp, total,
                      n_rows, nkv, page_size, num_pages, window, table_stride, row_start, row_t,
                      row_p, row_seq, block_tables, err);
      for (int j = 0; j < nb; ++j) {
        const int it = it0 + j;
        if (blockIdx.x + it * gridDim.x >= total) break;
        const int src = j * per;
        const int r = __shfl_sync(0xffffffffu, cur.r, src);
        const int g = __shfl_sync(0xffffffffu, cur.g, src);
        const int split = __shfl_sync(0xffffffffu, cur.split, src);
        // lane l < pages fetches page l of the tile: its id sits in lane src + l / pp, place l % pp
        int pid = 0;
        {
          const int holder = src + (lane < pages ? lane / pp : 0), place = lane % pp;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int v = __shfl_sync(0xffffffffu, cur.pg[e], holder);
            if (place == e) pid = v;
          }
        }
        const int y = (pid * nkv + g) * page_size;
        // the tile's pages lie side by side in the pool (what a prompt's pages do, and a
        // decoding request's where the pool could give it neighbours): one box for all of them
        const int y0 = __shfl_sync(0xffffffffu, y, 0);
        const bool run = pages > 1 && __all_sync(0xffffffffu, lane >= pages ||
                                                 y == y0 + lane * nkv * page_size);
        const int page0 = y0 / (nkv * page_size);
        const int pgrp = it % groups, k = it / groups;
        const int qi = pgrp * qsg + k % qsg;
        bool ok = true;
        // ahead of the wait: tiles of keys that earlier steps wrote, into slots never used
        if (!waited && ((2 * k + 1) / spg > 0 || split == row_p[r] / DP_SPLIT))
          wait_then_queries();
        {
          const int n = 2 * k, slot = pgrp * spg + n % spg, use = n / spg;
          if (use > 0) ok = bf_mbar_wait_bounded(empty + slot, (use - 1) & 1);
          if (!__all_sync(0xffffffffu, ok)) {
            failed = true;
            break;
          }
          if (lane == 0) {
            const int t = row_t[r];
            int* inf = info + qi * 8;
            inf[0] = r; inf[1] = g; inf[2] = split;
            bf_mbar_expect_tx(full + slot, TILE_BYTES + (uint32_t)(G * D * 2));
            if (waited) {
              dp_bulk_load(qbuf + (size_t)qi * G * D, q + ((size_t)t * nh + (size_t)g * G) * D,
                           (uint32_t)(G * D * 2), full + slot);
            } else {
              inf[5] = t; inf[6] = slot; inf[7] = 1;
            }
          }
          __syncwarp();
          if (run) {
            if (lane < HALVES)
              bf_tma_load_4d(tiles + (size_t)slot * TILE_ELEMS + lane * HALF_ELEMS, &map_k_run,
                             full + slot, lane * 64, 0, g, page0);
          } else if (lane < pages) {
            __nv_bfloat16* dst = tiles + (size_t)slot * TILE_ELEMS + lane * page_size * 64;
#pragma unroll
            for (int hh = 0; hh < HALVES; ++hh)
              bf_tma_load_2d(dst + hh * HALF_ELEMS, &map_k, full + slot, hh * 64, y);
          }
        }
        {
          const int n = 2 * k + 1, slot = pgrp * spg + n % spg, use = n / spg;
          if (use > 0) ok = bf_mbar_wait_bounded(empty + slot, (use - 1) & 1);
          if (!__all_sync(0xffffffffu, ok)) {
            failed = true;
            break;
          }
          if (lane == 0) bf_mbar_expect_tx(full + slot, TILE_BYTES);
          __syncwarp();
          if (run) {
            if (lane < HALVES)
              bf_tma_load_4d(tiles + (size_t)slot * TILE_ELEMS + lane * HALF_ELEMS, &map_v_run,
                             full + slot, lane * 64, 0, g, page0);
          } else if (lane < pages) {
            __nv_bfloat16* dst = tiles + (size_t)slot * TILE_ELEMS + lane * page_size * 64;
#pragma unroll
            for (int hh = 0; hh < HALVES; ++hh)
              bf_tma_load_2d(dst + hh * HALF_ELEMS, &map_v, full + slot, hh * 64, y);
          }
        }
      }
    }
    if (!waited) wait_then_queries();
    if (failed && lane == 0) atomicOr(err, BF_ERR_WAIT);
    BF_TRACE_POINT(10 * BF_TR_ATTN + 2);                 // the producer's end: all tiles requested
    return;
  }

  // -------------------------------------------------------------------- consumers
  const int cw = warp - 1, grp = cw >> 2, w = cw & 3;
  if (grp >= groups) return;
  const int bar_id = 1 + grp;
  const int r0 = lane >> 2, cq = (lane & 3) * 2;
  const int wkey = w * 32;
  int itg = 0;
  for (int it = grp;; it += groups, ++itg) {
    const int idx = blockIdx.x + it * gridDim.x;
    if (idx >= total) break;
    const int qi = grp * qsg + itg % qsg;
    const int nK = 2 * itg, slotK = grp * spg + nK % spg, nV = nK + 1, slotV = grp * spg + nV % spg;
    const __nv_bfloat16* Ks = tiles + (size_t)slotK * TILE_ELEMS;
    const __nv_bfloat16* Vs = tiles + (size_t)slotV * TILE_ELEMS;
    __nv_bfloat16* P = pbuf + (size_t)(grp * 2 + (itg & 1)) * 16 * DP_P_LD;
    float* red_m = red + (size_t)(grp * 2 + (itg & 1)) * 128;
    float* red_l = red_m + 64;

    const bool okK = bf_mbar_wait_bounded(full + slotK, (nK / spg) & 1);
    const int* inf = info + qi * 8;
    const int r = min(max(inf[0], 0), n_rows - 1), g = inf[1], split = inf[2];
    const int p = row_p[r], j0 = window > 0 ? max(0, p - window + 1) : 0;
    const int k_begin = split * DP_SPLIT;

    unsigned qa[D / 16][4];
    {
      const __nv_bfloat16* q0 = qbuf + (size_t)qi * G * D + (size_t)r0 * D;
      const __nv_bfloat16* q1 = q0 + (size_t)8 * D;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int c = ks * 16 + cq;
        qa[ks][0] = r0 < G ? *reinterpret_cast<const unsigned*>(q0 + c) : 0u;
        qa[ks][1] = r0 + 8 < G ? *reinterpret_cast<const unsigned*>(q1 + c) : 0u;
        qa[ks][2] = r0 < G ? *reinterpret_cast<const unsigned*>(q0 + c + 8) : 0u;
        qa[ks][3] = r0 + 8 < G ? *reinterpret_cast<const unsigned*>(q1 + c + 8) : 0u;
      }
    }
    float s[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
      for (int i = 0; i < 4; ++i) s[nt][i] = 0.f;
      const int krow = wkey + nt * 8 + (lane & 7);
#pragma unroll
      for (int ks = 0; ks < D / 16; ks += 2) {
        unsigned b[4];
        const int c = ks * 2 + (lane >> 3);
        ldmatrix_x4(b, Ks + (c >> 3) * HALF_ELEMS + dp_sw_off(krow, c & 7));
        mma_bf16_16816(s[nt], qa[ks], b[0], b[1]);
        mma_bf16_16816(s[nt], qa[ks + 1], b[2], b[3]);
      }
    }
    __syncwarp();
    if (lane == 0) dp_mbar_arrive(empty + slotK);        // K tile, queries and info are in registers

    float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int j = k_begin + wkey + nt * 8 + cq + (i & 1);
        s[nt][i] = (j >= j0 && j <= p) ? s[nt][i] * scale_log2 : -INFINITY;
      }
      m0 = fmaxf(m0, fmaxf(s[nt][0], s[nt][1]));
      m1 = fmaxf(m1, fmaxf(s[nt][2], s[nt][3]));
    }
    m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 1));
    m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 2));
    m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 1));
    m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 2));
    if ((lane & 3) == 0) {
      red_m[w * 16 + r0] = m0;
      red_m[w * 16 + r0 + 8] = m1;
    }
    if (!dp_group_all(bar_id, 128, okK)) {
      if ((tid & 127) == 32) atomicOr(err, BF_ERR_WAIT);
      break;
    }
    float M0 = -INFINITY, M1 = -INFINITY;
#pragma unroll
    for (int ww = 0; ww < 4; ++ww) {
      M0 = fmaxf(M0, red_m[ww * 16 + r0]);
      M1 = fmaxf(M1, red_m[ww * 16 + r0 + 8]);
    }
    const float u0 = M0 == -INFINITY ? 0.f : M0, u1 = M1 == -INFINITY ? 0.f : M1;
    float l0 = 0.f, l1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const float e0 = exp2f(s[nt][0] - u0), e1 = exp2f(s[nt][1] - u0);
      const float e2 = exp2f(s[nt][2] - u1), e3 = exp2f(s[nt][3] - u1);
      l0 += e0 + e1;
      l1 += e2 + e3;
      const int col = wkey + nt * 8 + cq;
      *reinterpret_cast<unsigned*>(P + r0 * DP_P_LD + col) = pack_bf16(e0, e1);
      *reinterpret_cast<unsigned*>(P + (r0 + 8) * DP_P_LD + col) = pack_bf16(e2, e3);
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if ((lane & 3) == 0) {
      red_l[w * 16 + r0] = l0;
      red_l[w * 16 + r0 + 8] = l1;
    }
    const bool okV = bf_mbar_wait_bounded(full + slotV, (nV / spg) & 1);
    if (!dp_group_all(bar_id, 128, okV)) {
      if ((tid & 127) == 32) atomicOr(err, BF_ERR_WAIT);
      break;
    }

    // this warp's quarter of the columns, over all 128 keys
    constexpr int CH = D / 32;                           // 16-byte column chunks per warp
    float o[CH][4];
#pragma unroll
    for (int dn = 0; dn < CH; ++dn)
#pragma unroll
      for (int i = 0; i < 4; ++i) o[dn][i] = 0.f;
#pragma unroll
    for (int kk = 0; kk < DP_SPLIT / 16; ++kk) {
      unsigned pa[4];
      ldmatrix_x4(pa, P + (lane & 15) * DP_P_LD + kk * 16 + (lane >> 4) * 8);
      const int m = lane >> 3;
      const int vrow = kk * 16 + (m & 1) * 8 + (lane & 7);
#pragma unroll
      for (int dn = 0; dn < CH; dn += 2) {
        unsigned b[4];
        const int c = w * CH + dn + (m >> 1);
        ldmatrix_x4_trans(b, Vs + (c >> 3) * HALF_ELEMS + dp_sw_off(vrow, c & 7));
        mma_bf16_16816(o[dn], pa, b[0], b[1]);
        mma_bf16_16816(o[dn + 1], pa, b[2], b[3]);
      }
    }
    __syncwarp();
    if (lane == 0) dp_mbar_arrive(empty + slotV);

    const size_t pb0 = ((size_t)r * nh + (size_t)g * G + r0) * max_splits + split;
    const size_t pb1 = pb0 + (size_t)8 * max_splits;
#pragma unroll
    for (int dn = 0; dn < CH; ++dn) {
      const int col = (w * CH + dn) * 8 + cq;
      if (r0 < G) *reinterpret_cast<float2*>(part_o + pb0 * D + col) = make_float2(o[dn][0], o[dn][1]);
      if (r0 + 8 < G)
        *reinterpret_cast<float2*>(part_o + pb1 * D + col) = make_float2(o[dn][2], o[dn][3]);
    }
    if (w == 0 && (lane & 3) == 0) {
      float L0 = 0.f, L1 = 0.f;
#pragma unroll
      for (int ww = 0; ww < 4; ++ww) {                   // fixed order: the sum does not depend on timing
        L0 += red_l[ww * 16 + r0];
        L1 += red_l[ww * 16 + r0 + 8];
      }
      if (r0 < G) {
        part_ml[pb0 * 2] = M0;
        part_ml[pb0 * 2 + 1] = L0;
      }
      if (r0 + 8 < G) {
        part_ml[pb1 * 2] = M1;
        part_ml[pb1 * 2 + 1] = L1;
      }
    }
  }
}

static int dp_sm_count() {
  static int counts[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (!counts[dev]) cudaDeviceGetAttribute(&counts[dev], cudaDevAttrMultiProcessorCount, dev);
  return counts[dev];
}

template <int D>
static int launch_persistent(const void* q, const void* k_cache, const void* v_cache,
                             const int* rows, const int* seq_of_token, const int* positions,
                             const int* block_tables, int table_stride, float* part_o,
                             float* part_ml, int n_rows, int nh, int nkv, int page_size,
                             int num_pages, int window, int max_splits, float scale, int* err,
                             cudaStream_t stream) {
  const int G = nh / nkv;
  const size_t limit = 227 * 1024;
  int slots = DP_MAX_SLOTS;
  int groups = DP_GROUPS;
  while (slots >= 2 && 1024 + dp_layout(D, slots, slots >= 4 ? 2 : 1, G, n_rows).total > limit)
    --slots;
  if (slots < 2) return (int)cudaErrorInvalidValue;
  if (slots < 4 || groups < 2) groups = 1;
  slots -= slots % groups;
  const size_t smem = 1024 + dp_layout(D, slots, groups, G, n_rows).total;
  CUtensorMap mk, mv;
  const long long cache_rows = (long long)num_pages * nkv * page_size;
  int e = bf_make_tensor_map_bf16_2d(&mk, k_cache, cache_rows, D, D, page_size, 64);
  if (e) return e;
  e = bf_make_tensor_map_bf16_2d(&mv, v_cache, cache_rows, D, D, page_size, 64);
  if (e) return e;
  // the same pages as a 4-d tensor, for tiles whose pages are neighbours in the pool
  CUtensorMap mkr, mvr;
  e = bf_make_tensor_map_pages_bf16(&mkr, k_cache, num_pages, nkv, page_size, D,
                                    DP_SPLIT / page_size);
  if (e) return e;
  e = bf_make_tensor_map_pages_bf16(&mvr, v_cache, num_pages, nkv, page_size, D,
                                    DP_SPLIT / page_size);
  if (e) return e;
  auto kern = decode_attention_persistent_kernel<D>;
  static bool configured_on[BF_MAX_DEVICES];
  bool& configured = configured_on[bf_current_device()];
  if (!configured) {
    cudaError_t ce =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)limit);
    if (ce != cudaSuccess) return (int)ce;
    configured = true;
  }
  const int sms = dp_sm_count();
  if (sms <= 0) return (int)cudaErrorInvalidValue;
  const long long most = (long long)n_rows * nkv * max_splits;
  const int grid = (int)(most < sms ? most : sms);
  return bf_launch_pdl(kern, dim3(grid), dim3(DP_THREADS), smem, stream, mk, mv, mkr, mvr,
                       (const __nv_bfloat16*)q, rows, seq_of_token, positions, block_tables,
                       table_stride, part_o, part_ml, n_rows, nh, nkv, page_size, num_pages,
                       window, max_splits, scale * 1.4426950408889634f, slots, groups,
                       getenv("BINFER_B200_ATTN_EARLY") ? atoi(getenv("BINFER_B200_ATTN_EARLY")) : 1,
                       err);
}

// Same arguments and result as bf_decode_attention.  Returns cudaErrorInvalidValue for what
// it does not take (see the head of this file); nothing has been launched then.
BF_EXPORT int bf_decode_attention_persistent(const void* q, const void* k_cache,
                                             const void* v_cache, const int* rows,
                                             const int* seq_of_token, const int* positions,
                                             const int* block_tables, int table_stride, void* out,
                                             float* part_o, float* part_ml, int n_rows, int nh,
                                             int nkv, int d, int page_size, int num_pages,
                                             int window, int max_splits, float scale, int* err,
                                             cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (nkv <= 0 || nh % nkv || nh / nkv > 16 || n_rows > DP_MAX_ROWS || page_size < 8 ||
      page_size > 128 || DP_SPLIT % page_size || ((uintptr_t)k_cache & 15) ||
      ((uintptr_t)v_cache & 15) || ((uintptr_t)q & 15))
    return (int)cudaErrorInvalidValue;
  int e;
#define DP_CASE(DD)                                                                          \
  case DD:                                                                                   \
    e = launch_persistent<DD>(q, k_cache, v_cache, rows, seq_of_token, positions,            \
                              block_tables, table_stride, part_o, part_ml, n_rows, nh, nkv,  \
                              page_size, num_pages, window, max_splits, scale, err, stream); \
    break
  switch (d) {
    DP_CASE(64);
    DP_CASE(128);
    DP_CASE(256);
    default:
      return (int)cudaErrorInvalidValue;
  }
#undef DP_CASE
  if (e) return e;
  return bf_decode_attention_merge(part_o, part_ml, rows, positions, out, n_rows, nh, d, window,
                                   max_splits, stream);
}

BF_TRACE_READER(bf_trace_read_attention_decode_persistent)
