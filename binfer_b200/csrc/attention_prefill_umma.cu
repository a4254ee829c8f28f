// Causal flash attention for prompt portions on the 5th-generation tensor cores.
//
// A CTA takes 128 consecutive queries of one portion for one head and walks the keys in
// tiles of 64 (edges at multiples of 64 counted from position 0), every key and value
// coming from the paged bf16 cache.  Two CTAs share an SM, so that one's softmax runs
// while the other's products occupy the tensor cores:
//
//   warp 4      TMA producer: the Q tile once; per key tile one cp.async.bulk.tensor copy
//               per (page, 64 columns) of K and of V into 128-byte-swizzled shared memory,
//               two key tiles in flight;
//   warp 5      one thread issues tcgen05.mma: S = Q K^T (M = 128 queries, N = 64 keys,
//               K = head size) into tensor memory, and, once the probabilities are written,
//               O_tile = P V (M = 128, N = head size, K = 64 keys; V is read as stored,
//               an MN-major operand);
//   warps 0-3   softmax: thread r owns query row r = TMEM lane r.  It reads its row of S
//               (tcgen05.ld), masks, keeps the running maximum and sum in float with exp2,
//               writes P as bf16 into the swizzled A-operand tile (over the K tile, which
//               is dead by then, when the head size is 128), then adds O_tile into its
//               float accumulators with the running rescale.
//
// S of the next tile is multiplied while the softmax warps still add O of this one.
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
constexpr int AU_THREADS = 192;

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 2^x by the special-function unit (x <= 0 here; -inf gives 0)
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// MN-major operand (rows = K index, 64 contiguous elements of the MN index per 128-byte row,
// 128-byte swizzle): 8-row groups 1024 bytes apart, 64-column blocks `lbo_bytes` apart.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

template <int D>
__global__ void __launch_bounds__(AU_THREADS, 2)
prefill_attention_umma_kernel(const __grid_constant__ CUtensorMap map_q,
                              const __grid_constant__ CUtensorMap map_k,
                              const __grid_constant__ CUtensorMap map_v,
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
  constexpr int TMEM_COLS = 256;                         // S: 64 columns, O tile: D columns
  extern __shared__ __align__(16) uint8_t smem_raw[];
  uint8_t* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* Qs = base;
  uint8_t* Ks = Qs + Q_BYTES;                            // [2][KV_BYTES]
  uint8_t* Vs = Ks + 2 * KV_BYTES;                       // [2][KV_BYTES]
  uint8_t* Psep = Vs + 2 * KV_BYTES;                     // used only when P cannot lie over K
  uint64_t* bars = reinterpret_cast<uint64_t*>(Psep + (P_OVER_K ? 0 : P_BYTES));
  uint64_t* q_full = bars;             // [1]
  uint64_t* kv_full = bars + 1;        // [2]
  uint64_t* kv_empty = bars + 3;       // [2]
  uint64_t* s_full = bars + 5;         // [1]
  uint64_t* p_full = bars + 6;         // [1]  128 arrivals
  uint64_t* o_full = bars + 7;         // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int* it = items + 4 * blockIdx.z;
  const int seq = it[0], row0 = it[1], qlen = it[2], pos0 = it[3];
  // the last query tiles see the most keys: they are launched first
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x, h = blockIdx.y;
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
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 128);
    mbar_init(o_full, 1);
    *abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
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
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + AU_BN;

  if (warp == 4) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
      for (int hh = 0; hh < HALVES; ++hh)
        tma_load_2d(Qs + hh * QHALF_BYTES, &map_q, q_full, h * D + hh * 64, row0 + qt * AU_BM);
    }
    uint32_t phase = 0;
    for (int kt = kt_first; kt <= kt_last && !*abort; ++kt) {
      const int buf = (kt - kt_first) & 1;
      bool ok = true;
      if (lane == 0) ok = mbar_wait(kv_empty + buf, phase ^ 1, abort);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      const int jp = kt * AU_BN + lane * page_size;
      const bool wanted = lane < pages && jp <= p_last && jp + page_size > j_lo;
      int page = 0;
      if (wanted) {
        page = table[jp / page_size];
        if (page < 0 || page >= num_pages) {
          atomicOr(err, BF_ERR_PAGE);
          page = 0;
        }
      }
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
      if (wanted) {
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
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // S: a = Q (K-major), b = K tile (K-major), N = 64 keys
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) |
                               ((uint32_t)(AU_BN >> 3) << 17) | ((uint32_t)(AU_BM >> 4) << 24);
      // O: a = P (K-major), b = V as stored (MN-major), N = head size
      const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                               ((uint32_t)(D >> 3) << 17) | ((uint32_t)(AU_BM >> 4) << 24);
      bool ok = mbar_wait(q_full, 0, abort);
      uint32_t kv_phase = 0, p_phase = 0;
      for (int kt = kt_first; kt <= kt_last && ok; ++kt) {
        const int buf = (kt - kt_first) & 1;
        if (!(ok = mbar_wait(kv_full + buf, kv_phase, abort))) break;
        tc_fence_after();
        const uint32_t q_addr = smem_u32(Qs), k_addr = smem_u32(Ks + buf * KV_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t qo = (uint32_t)((k >> 2) * QHALF_BYTES + (k & 3) * 32);
          const uint32_t ko = (uint32_t)((k >> 2) * KHALF_BYTES + (k & 3) * 32);
          umma_bf16(tmem_s, umma_desc_k_sw128(q_addr + qo), umma_desc_k_sw128(k_addr + ko),
                    idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        if (!(ok = mbar_wait(p_full, p_phase, abort))) break;
        p_phase ^= 1;
        tc_fence_after();
        const uint32_t p_addr = smem_u32(P_OVER_K ? Ks + buf * KV_BYTES : Psep);
        const uint32_t v_addr = smem_u32(Vs + buf * KV_BYTES);
#pragma unroll
        for (int k = 0; k < AU_BN / 16; ++k) {
          // 16 keys further: along K inside P's swizzled rows, two 8-row groups down in V
          umma_bf16(tmem_o, umma_desc_k_sw128(p_addr + (uint32_t)(k * 32)),
                    umma_desc_mn_sw128(v_addr + (uint32_t)(k * 2048), KHALF_BYTES), idesc_o,
                    k > 0 ? 1u : 0u);
        }
        umma_commit(kv_empty + buf);       // K, V (and P) of this tile are free when done
        umma_commit(o_full);
        if (buf == 1) kv_phase ^= 1;
      }
    }
  } else {
    // --------------------------------------------------------------------- softmax
    const int r = threadIdx.x;                           // query row of the tile = TMEM lane
    const int l = qt * AU_BM + r;                        // index inside the portion
    const bool valid = l < qlen;
    const int pr = pos0 + l;
    const int jl = window > 0 ? max(0, pr - window + 1) : 0;
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    float m = -INFINITY, lsum = 0.f;
    float acc[D];
#pragma unroll
    for (int i = 0; i < D; ++i) acc[i] = 0.f;
    uint32_t s_phase = 0, o_phase = 0;
    bool alive = true;
    for (int kt = kt_first; kt <= kt_last; ++kt) {
      const bool ok = alive && !*abort && mbar_wait(s_full, s_phase, abort);
      s_phase ^= 1;
      if (!epilogue_all(ok)) {
        alive = false;
        break;
      }
      tc_fence_after();
      uint8_t* Ps = P_OVER_K ? Ks + ((kt - kt_first) & 1) * KV_BYTES : Psep;
      const int t_lo = kt * AU_BN;
      const bool need_mask = !valid || t_lo + AU_BN - 1 > pr || t_lo < jl;
      // pass 1: the row's maximum over this tile.  (The chunk loops are kept rolled: fully
      // unrolled, the softmax no longer fits the instruction cache and runs many times slower.)
      const int hi = valid ? pr - t_lo : -1;             // last visible key of the tile
      const int lo = jl - t_lo;                          // first visible key of the tile
      float tmax = -INFINITY;
#pragma unroll 1
      for (int c0 = 0; c0 < AU_BN; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(tmem_s + lane_addr + c0, v);
        if (need_mask) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c0 + j >= lo && c0 + j <= hi) tmax = fmaxf(tmax, __uint_as_float(v[j]));
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) tmax = fmaxf(tmax, __uint_as_float(v[j]));
        }
      }
      tmax *= scale_log2;                                // the scale is positive
      const float m_new = fmaxf(m, tmax);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float corr = m == -INFINITY ? 0.f : exp2f(m - m_use);
      m = m_new;
      // pass 2: probabilities, their sum, and P as bf16 in the swizzled operand tile
      float tsum = 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < AU_BN; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(tmem_s + lane_addr + c0, v);
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          float e0 = ex2_approx(fmaf(__uint_as_float(v[j]), scale_log2, -m_use));
          float e1 = ex2_approx(fmaf(__uint_as_float(v[j + 1]), scale_log2, -m_use));
          if (need_mask) {
            if (c0 + j < lo || c0 + j > hi) e0 = 0.f;
            if (c0 + j + 1 < lo || c0 + j + 1 > hi) e1 = 0.f;
          }
          tsum += e0 + e1;
          __nv_bfloat162 p2 = __floats2bfloat162_rn(e0, e1);
          packed[j >> 1] = *reinterpret_cast<uint32_t*>(&p2);
        }
        // 32 keys = four 16-byte chunks of this row
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int c = (c0 >> 3) + q4;                  // chunk index along the 64 keys
          uint8_t* dst = Ps + r * 128 + ((c ^ (r & 7)) << 4);
          *reinterpret_cast<uint4*>(dst) = make_uint4(packed[4 * q4], packed[4 * q4 + 1],
                                                      packed[4 * q4 + 2], packed[4 * q4 + 3]);
        }
      }
      lsum = lsum * corr + tsum;
      // P is read by the tensor core through the async proxy
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_before();
      mbar_arrive(p_full);
      // O of this tile
      const bool ok2 = mbar_wait(o_full, o_phase, abort);
      o_phase ^= 1;
      if (!epilogue_all(ok2)) {
        alive = false;
        break;
      }
      tc_fence_after();
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(tmem_o + lane_addr + c0, v);
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[c0 + j] = acc[c0 + j] * corr + __uint_as_float(v[j]);
      }
      tc_fence_before();
    }
    if (alive && valid) {
      const float inv = 1.f / lsum;
      __nv_bfloat16* dst = out + ((size_t)(row0 + l) * nh + h) * D;
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 8) {
        uint4 o4;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          o2[j] = __floats2bfloat162_rn(acc[c0 + 2 * j] * inv, acc[c0 + 2 * j + 1] * inv);
        *reinterpret_cast<uint4*>(dst + c0) = o4;
      }
    }
  }

  __syncthreads();
  if (*abort && threadIdx.x == 0) atomicOr(err, BF_ERR_WAIT);
  if (warp == 5) {
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
  constexpr int HALVES = D / 64;
  // Q, two stages of K and V, P apart only when it does not fit over a K tile, barriers
  const size_t smem = 1024 + (size_t)HALVES * 16384 + (size_t)4 * HALVES * 8192 +
                      (HALVES * 8192 >= 16384 ? 0 : 16384) + 128;
  auto kern = prefill_attention_umma_kernel<D>;
  static bool configured = false;
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)smem);
    if (ce != cudaSuccess) return (int)ce;
    configured = true;
  }
  dim3 grid((max_rows + AU_BM - 1) / AU_BM, nh, n_items);
  kern<<<grid, AU_THREADS, smem, stream>>>(mq, mk, mv, items, block_tables, table_stride,
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

