// bf16 matrix product for many token rows (prefill) on pairs of SMs:
// out[t, f] = sum_k x[t, k] * w[f, k], float accumulation, bf16 or float out; or, in the
// gated form, act[t, o] = silu(g) * u with g = x . w[o], u = x . w[inter + o] (the stacked
// gate/up weight of the feed-forward, the activation in the epilogue).  The reference makes
// these products through cuBLAS and runs the activation as a kernel of its own
// (cuda/kernels/gemm.cu:244-267, cuda/kernels/bf16_kernels.cu:461-477).
//
// A cluster of two CTAs works on one tile of 256 token rows x BN feature rows with
// tcgen05.mma.cta_group::2: each CTA holds its own 128 token rows and HALF of the feature
// rows of every K slice in shared memory, the product reads both halves, and each CTA's
// tensor memory receives its 128 token rows x BN columns.  Per 64-deep K slice a CTA so
// fetches 16 KB + BN/2 x 128 bytes for 128 x BN x 64 products: half the shared-memory
// traffic per product of the one-CTA kernel (gemm_tcgen05.cu), which is what bounded that
// kernel at these sizes.
//
//   warp 0      TMA producer in both CTAs: its own token rows and its own half of the
//               feature rows, completion on the LEADER's (cluster rank 0) mbarrier of the
//               stage (cp.async.bulk.tensor ... .cta_group::2), which expects both CTAs' bytes;
//   warp 1      in the leader one thread issues the products and commits with
//               .multicast::cluster to both CTAs' barriers (stage free; accumulator complete);
//               in both CTAs the warp owns the tensor-memory allocation (two accumulators);
//   warps 2-5   epilogue in both CTAs: tcgen05.ld of the own 128 rows, conversion (or the
//               activation), 16-byte stores; then one arrival per warp on the leader's
//               "accumulator free" barrier.
//
// No load here uses multicast: each CTA fetches what it holds.  Every mbarrier wait is
// bounded (about a second); a CTA that gives up raises its own and its peer's abort flag,
// sets BF_ERR_WAIT, every role leaves its loop, and both CTAs meet at a cluster barrier
// before tensor memory is freed.
#include <cuda.h>
#include <stdint.h>
#include <stdlib.h>

#include "common.cuh"
#include "tma_utils.cuh"
#include "umma_utils.cuh"

namespace {

struct PairParams {
  int tokens, features, K;     // features: output columns (gated form: the activation's width)
  int tiles_t, tiles_f;        // tiles over tokens (256 each) and over accumulator columns
  int bn;                      // accumulator columns per tile: a multiple of 16 (gated: 64)
  int stages;
  int gated;                   // 1: w is [2 features, K], gate rows first
  int staged;                  // 1: results leave through shared memory and TMA stores
  int accumulate;              // 1: out (float) += the product
  long long ldo;               // row stride of the output, in elements
  int* err;
};

constexpr int PM = 256;                      // token rows per tile (128 per CTA)
constexpr int P_A_BYTES = 128 * BK * 2;      // a CTA's token rows of one K slice
constexpr int P_MAX_STAGES = 12;
constexpr int P_BAR_BYTES = 1024;
constexpr int P_THREADS = 192;
constexpr int P_OUT_BYTES = 128 * 128;       // a staged slab: a CTA's 128 rows x 64 bf16

__device__ __forceinline__ uint32_t pair_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t pair_map(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void pair_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// A tile into this CTA's shared memory; the bytes are counted on `bar_cluster_addr`, a
// shared::cluster address that may lie in the peer CTA.
__device__ __forceinline__ void pair_tma_load(void* smem_dst, const CUtensorMap* map,
                                              uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void pair_umma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives, once the products issued so far are done, on the barrier at this offset in both CTAs
__device__ __forceinline__ void pair_commit_both(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(smem_u32(bar)),
      "h"((uint16_t)3)
      : "memory");
}
__device__ __forceinline__ void pair_commit_own(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void pair_arrive_remote(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(
                   bar_cluster_addr)
               : "memory");
}
__device__ __forceinline__ float pair_silu(float g) { return __fdividef(g, 1.f + __expf(-g)); }

template <typename OutT>
__device__ __forceinline__ void pair_store16(OutT* dst, const uint32_t (&r)[16], bool vec,
                                             int valid, bool accumulate) {
  if constexpr (sizeof(OutT) == 4) {
    if (accumulate) {
#pragma unroll
      for (int jj = 0; jj < 16; ++jj)
        if (jj < valid) dst[jj] += __uint_as_float(r[jj]);
      return;
    }
  }
  if (vec && valid >= 16) {
    if constexpr (sizeof(OutT) == 2) {
      uint4 v0, v1;
      v0.x = pack_bf16x2(r[0], r[1]);   v0.y = pack_bf16x2(r[2], r[3]);
      v0.z = pack_bf16x2(r[4], r[5]);   v0.w = pack_bf16x2(r[6], r[7]);
      v1.x = pack_bf16x2(r[8], r[9]);   v1.y = pack_bf16x2(r[10], r[11]);
      v1.z = pack_bf16x2(r[12], r[13]); v1.w = pack_bf16x2(r[14], r[15]);
      reinterpret_cast<uint4*>(dst)[0] = v0;
      reinterpret_cast<uint4*>(dst)[1] = v1;
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q)
        reinterpret_cast<uint4*>(dst)[q] =
            make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
    }
  } else {
#pragma unroll
    for (int jj = 0; jj < 16; ++jj)
      if (jj < valid) bf_st(dst + jj, __uint_as_float(r[jj]));
  }
}

template <typename OutT>
__global__ void __launch_bounds__(P_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x,
                 const __grid_constant__ CUtensorMap map_w,
                 const __grid_constant__ CUtensorMap map_out, OutT* __restrict__ out,
                 const PairParams p) {
  constexpr int TMEM_COLS = 512;             // two accumulators of up to 256 columns
  extern __shared__ __align__(16) uint8_t smem_raw[];
  // Swizzled tiles must start on a 1024-byte boundary of the shared window, and the two CTAs'
  // layouts must be the same: the products address both with one descriptor.
  uint8_t* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(base);       // waited on in the leader only
  uint64_t* empty = full + P_MAX_STAGES;
  uint64_t* acc_full = empty + P_MAX_STAGES;                // [2]
  uint64_t* acc_empty = acc_full + 2;                       // [2], waited on in the leader only
  uint64_t* drain = acc_empty + 2;                          // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain + 1);
  volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* out_stage = base + P_BAR_BYTES;                  // [2] slabs on their way out
  uint8_t* tiles = out_stage + 2 * P_OUT_BYTES;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = pair_rank();
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int units = p.tiles_t * p.tiles_f;
  const int kc_total = (p.K + BK - 1) / BK;
  const int b_rows = p.bn >> 1;                             // feature rows this CTA holds
  const int stage_bytes = P_A_BYTES + b_rows * BK * 2;
  const int STAGES = p.stages;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full + a, 1);
      mbar_init(acc_empty + a, 8);           // one arrival per epilogue warp of both CTAs
    }
    mbar_init(drain, 1);
    *abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  pair_sync();                               // the peer's barriers exist before anything lands
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint32_t full_leader = pair_map(smem_u32(full), 0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = pair; u < units && ok && !*abort; u += pairs) {
        const int tt = u % p.tiles_t, tf = u / p.tiles_t;
        const int t0 = tt * PM + (int)rank * 128;
        for (int kc = 0; kc < kc_total; ++kc) {
          if (!mbar_wait(empty + stage, phase ^ 1, abort)) {
            ok = false;
            break;
          }
          uint8_t* dst = tiles + (size_t)stage * stage_bytes;
          const uint32_t bar = full_leader + 8u * (uint32_t)stage;
          if (rank == 0) mbar_expect_tx(full + stage, 2u * (uint32_t)stage_bytes);
          pair_tma_load(dst, &map_x, bar, kc * BK, t0);
          if (!p.gated) {
            pair_tma_load(dst + P_A_BYTES, &map_w, bar, kc * BK, tf * p.bn + (int)rank * b_rows);
          } else {
            // this CTA's columns: gate rows of its outputs, then the up rows of the same
            const int q = p.bn >> 2;
            const int o0 = tf * (p.bn >> 1) + (int)rank * q;
            pair_tma_load(dst + P_A_BYTES, &map_w, bar, kc * BK, o0);
            pair_tma_load(dst + P_A_BYTES + q * BK * 2, &map_w, bar, kc * BK, p.features + o0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      // every arrival that the leader's commits send to this CTA's barriers lands before it ends
      for (int s = 0; s < STAGES && ok && !*abort; ++s) {
        ok = mbar_wait(empty + stage, phase ^ 1, abort);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0 && rank == 0) {
      // c = float, a = b = bf16, both K-major, N = bn, M = 256 over the pair
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                             ((uint32_t)(p.bn >> 3) << 17) | ((uint32_t)(PM >> 4) << 24);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      for (int u = pair; u < units && !*abort; u += pairs) {
        if (!mbar_wait(acc_empty + acc, acc_phase ^ 1, abort)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * 256);
        bool ok = true;
        for (int kc = 0; kc < kc_total; ++kc) {
          if (!mbar_wait(full + stage, phase, abort)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + (size_t)stage * stage_bytes);
          const uint64_t a_desc = umma_desc_k_sw128(a_addr);
          const uint64_t b_desc = umma_desc_k_sw128(a_addr + P_A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            pair_umma(d_tmem, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc,
                      (kc > 0 || k > 0) ? 1u : 0u);
          pair_commit_both(empty + stage);     // both CTAs' producers may refill the stage
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        pair_commit_both(acc_full + acc);      // both CTAs' epilogues may read the accumulator
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // --------------------------------------------------------------- epilogue
    const int quarter = warp & 3;              // the TMEM lanes this warp may read
    const bool vec_ok = (p.ldo * sizeof(OutT)) % 16 == 0 && ((uintptr_t)out & 15) == 0;
    const uint32_t acc_empty_leader = pair_map(smem_u32(acc_empty), 0);
    int acc = 0;
    uint32_t acc_phase = 0;
    int n_stored = 0;                          // slabs handed to TMA stores so far
    for (int u = pair; u < units; u += pairs) {
      const int tt = u % p.tiles_t, tf = u / p.tiles_t;
      const bool ok = !*abort && mbar_wait(acc_full + acc, acc_phase, abort);
      if (!epilogue_all(ok)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * 256);
      const int row0 = tt * PM + (int)rank * 128 + quarter * 32;
      const int t = row0 + lane;               // token of this thread
      if (p.staged) {
        // 128 bytes of every row at a time (64 bf16 or 32 floats): into shared memory in the
        // 128-byte swizzle, out by one TMA store (or add) per slab: whole lines, the matrix's
        // edges cut by the copy.
        const int row = quarter * 32 + lane;
        constexpr int SLAB = 128 / (int)sizeof(OutT);
        const int slabs = p.gated ? 2 : p.bn / SLAB;
        for (int slab = 0; slab < slabs; ++slab) {
          uint8_t* buf = out_stage + (n_stored & 1) * P_OUT_BYTES;
          if (threadIdx.x == 64) bf_bulk_wait_read<1>();   // the store before last has read it
          epilogue_sync();
          if constexpr (sizeof(OutT) == 2) {
#pragma unroll
            for (int hs = 0; hs < 2; ++hs) {
              uint32_t r[32];
              if (!p.gated) {
                tmem_ld32(taddr + slab * 64 + hs * 32, r);
              } else {
                uint32_t up[32];
                const int col = slab * 128 + hs * 32;
                tmem_ld32(taddr + col, r);
                tmem_ld32(taddr + col + 64, up);
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  r[j] = __float_as_uint(pair_silu(__uint_as_float(r[j])) *
                                         __uint_as_float(up[j]));
              }
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 v;
                v.x = pack_bf16x2(r[8 * q], r[8 * q + 1]);
                v.y = pack_bf16x2(r[8 * q + 2], r[8 * q + 3]);
                v.z = pack_bf16x2(r[8 * q + 4], r[8 * q + 5]);
                v.w = pack_bf16x2(r[8 * q + 6], r[8 * q + 7]);
                const int chunk = hs * 4 + q;
                *reinterpret_cast<uint4*>(buf + row * 128 + ((chunk ^ (row & 7)) << 4)) = v;
              }
            }
          } else {
            uint32_t r[32];
            tmem_ld32(taddr + slab * 32, r);
#pragma unroll
            for (int q = 0; q < 8; ++q)
              *reinterpret_cast<uint4*>(buf + row * 128 + ((q ^ (row & 7)) << 4)) =
                  make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          epilogue_sync();
          if (threadIdx.x == 64) {
            const int x = p.gated ? tf * 128 + slab * 64 : tf * p.bn + slab * SLAB;
            const int y = tt * PM + (int)rank * 128;
            if (x < p.features && y < p.tokens) {
              if (p.accumulate)
                bf_tma_reduce_add_2d(&map_out, buf, x, y);
              else
                bf_tma_store_2d(&map_out, buf, x, y);
            }
            bf_bulk_commit();
          }
          ++n_stored;
        }
      } else if (row0 < p.tokens) {          // uniform per warp: tcgen05.ld is warp-wide
        if (!p.gated) {
          for (int c0 = 0; c0 < p.bn; c0 += 16) {
            uint32_t r[16];
            tmem_ld16(taddr + c0, r);
            const int f0 = tf * p.bn + c0;
            if (t < p.tokens && f0 < p.features)
              pair_store16(out + (size_t)t * p.ldo + f0, r, vec_ok, p.features - f0, p.accumulate != 0);
          }
        } else {
          const int q = p.bn >> 2;
          for (int half = 0; half < 2; ++half)
            for (int c0 = 0; c0 < q; c0 += 16) {
              uint32_t g[16], up[16];
              tmem_ld16_pair(taddr + half * 2 * q + c0, taddr + half * 2 * q + q + c0, g, up);
              const int o0 = tf * (p.bn >> 1) + half * q + c0;
              if (t < p.tokens && o0 < p.features) {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                  g[j] = __float_as_uint(pair_silu(__uint_as_float(g[j])) *
                                         __uint_as_float(up[j]));
                pair_store16(out + (size_t)t * p.ldo + o0, g, vec_ok, p.features - o0, false);
              }
            }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) pair_arrive_remote(acc_empty_leader + 8u * (uint32_t)acc);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if (threadIdx.x == 64) bf_bulk_wait_read<0>();   // shared memory stays until the stores read it
  }

  // ------------------------------------------------------------------ wind-down
  __syncthreads();
  if (*abort) {
    if (threadIdx.x == 0) {
      atomicOr(p.err, BF_ERR_WAIT);
      // the peer leaves its waits at once instead of running each of them out
      asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(
                       pair_map(smem_u32(const_cast<int*>(abort)), rank ^ 1u)),
                   "r"(1)
                   : "memory");
    }
    if (warp == 0 && lane == 0 && rank == 0) {
      // copies that were issued but never consumed: give each stage's barrier a bounded chance
      for (int s = 0; s < STAGES; ++s) {
        const long long t0 = clock64();
        while (!mbar_try_wait(full + s, 0) && !mbar_try_wait(full + s, 1) &&
               clock64() - t0 < WAIT_LIMIT_CYCLES / 16) {
        }
      }
    }
    if (warp == 1 && lane == 0 && rank == 0) {
      pair_commit_own(drain);                  // products still in flight
      const long long t0 = clock64();
      while (!mbar_try_wait(drain, 0) && clock64() - t0 < WAIT_LIMIT_CYCLES / 16) {
      }
    }
    __syncthreads();
  }
  tc_fence_before();
  pair_sync();                                 // neither CTA's memory goes while the other uses it
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
}

template <typename OutT>
int launch(const void* x, const void* w, OutT* out, PairParams p, long long ldx, long long ldw,
           int num_sms, cudaStream_t stream) {
  CUtensorMap mx, mw;
  int e = bf_make_tensor_map_bf16_2d(&mx, x, p.tokens, p.K, ldx, 128, BK);
  if (e) return e;
  const int w_rows = p.gated ? 2 * p.features : p.features;
  e = bf_make_tensor_map_bf16_2d(&mw, w, w_rows, p.K, ldw, p.gated ? p.bn / 4 : p.bn / 2, BK);
  if (e) return e;
  // Results leave through shared memory and TMA stores where the output's rows start on
  // 16-byte boundaries and the tile is cut into slabs of 128 bytes a row.
  CUtensorMap mo = mx;
  p.staged = 0;
  static const bool staged_ok =
      !getenv("BINFER_B200_PAIR_STAGED") || atoi(getenv("BINFER_B200_PAIR_STAGED")) != 0;
  if (staged_ok && (p.ldo * sizeof(OutT)) % 16 == 0 && ((uintptr_t)out & 15) == 0 &&
      (p.gated ? p.bn == 256 : p.bn % (128 / (int)sizeof(OutT)) == 0)) {
    e = bf_make_tensor_map_2d_store(&mo, out, p.tokens, p.features, p.ldo, 128, (int)sizeof(OutT));
    if (e) return e;
    p.staged = 1;
  }
  const size_t smem_max = 226 * 1024;
  const size_t stage_bytes = (size_t)P_A_BYTES + (size_t)(p.bn / 2) * BK * 2;
  const size_t fixed = 1024 /* alignment slack */ + P_BAR_BYTES + 2 * P_OUT_BYTES;
  int stages = (int)((smem_max - fixed) / stage_bytes);
  if (stages > P_MAX_STAGES) stages = P_MAX_STAGES;
  if (stages < 2) return (int)cudaErrorInvalidValue;
  p.stages = stages;
  const size_t smem = fixed + (size_t)stages * stage_bytes;
  auto kern = gemm_pair_kernel<OutT>;
  static bool configured_on[BF_MAX_DEVICES];
  bool& configured = configured_on[bf_current_device()];
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)smem_max);
    if (ce != cudaSuccess) return (int)ce;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(P_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const int units = p.tiles_t * p.tiles_f;
  const int pairs = units < num_sms / 2 ? units : num_sms / 2;
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cudaError_t ce = cudaLaunchKernelEx(&cfg, kern, mx, mw, mo, out, p);
  if (ce != cudaSuccess) return (int)ce;
  return bf_launch_status();
}

}  // namespace

// Accumulator columns per tile (a multiple of `step`, at most 256) for `tokens` x `columns`
// on num_sms / 2 pairs: the width that wastes least of the last wave of tiles, wider tiles
// preferred when there is little to choose (they reuse the token rows more).
BF_EXPORT int bf_gemm_pair_choose_bn(int tokens, int columns, int step, int num_sms) {
  const int tiles_t = (tokens + PM - 1) / PM;
  const int pairs = num_sms / 2 > 0 ? num_sms / 2 : 1;
  int best = step;
  double best_score = -1.0;
  for (int bn = 128; bn <= 256; bn += step) {
    if (bn % step) continue;
    const long long tiles = (long long)tiles_t * ((columns + bn - 1) / bn);
    const long long waves = (tiles + pairs - 1) / pairs;
    const double used = (double)columns / ((double)((columns + bn - 1) / bn) * bn);
    const double eff = used * (double)tiles / ((double)waves * pairs);
    const double score = eff * (0.8 + 0.2 * bn / 256.0);
    if (score > best_score) {
      best_score = score;
      best = bn;
    }
  }
  return best;
}

// out[tokens, features] = x[tokens, K] * w[features, K]^T in bf16 with float accumulation, on
// pairs of CTAs.  gated != 0: w is [2 features, K] (gate rows first) and out[t, o] =
// silu(x . w[o]) * (x . w[features + o]), bf16 only.  out_dtype: BF_DTYPE_BF16 or
// BF_DTYPE_F32.  accumulate != 0 (float out only): out += the product.  bn: accumulator
// columns per tile (0: chosen here).  Returns
// cudaErrorInvalidValue for shapes it does not take.
BF_EXPORT int bf_gemm_bf16_pair(const void* x, const void* w, void* out, int tokens, int features,
                                int K, long long ldx, long long ldw, long long ldo, int out_dtype,
                                int gated, int accumulate, int bn, int num_sms, int* err,
                                cudaStream_t stream) {
  if (tokens <= 0 || features <= 0) return 0;
  if (K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || num_sms < 2)
    return (int)cudaErrorInvalidValue;
  if (gated && out_dtype != BF_DTYPE_BF16) return (int)cudaErrorInvalidValue;
  if (accumulate && (gated || out_dtype != BF_DTYPE_F32)) return (int)cudaErrorInvalidValue;
  // (widths chosen here are multiples of 64: the slabs that leave through TMA stores)
  const int step = gated || bn <= 0 ? 64 : 16;
  const int columns = gated ? 2 * features : features;
  if (bn <= 0) bn = bf_gemm_pair_choose_bn(tokens, columns, step, num_sms);
  if (bn % step || bn > 256 || bn < step) return (int)cudaErrorInvalidValue;
  PairParams p;
  p.tokens = tokens;
  p.features = features;
  p.K = K;
  p.ldo = ldo;
  p.bn = bn;
  p.gated = gated ? 1 : 0;
  p.accumulate = accumulate ? 1 : 0;
  p.tiles_t = (tokens + PM - 1) / PM;
  p.tiles_f = (columns + bn - 1) / bn;
  p.stages = 0;
  p.err = err;
  return out_dtype == BF_DTYPE_F32
             ? launch<float>(x, w, (float*)out, p, ldx, ldw, num_sms, stream)
             : launch<__nv_bfloat16>(x, w, (__nv_bfloat16*)out, p, ldx, ldw, num_sms, stream);
}
