// bf16 matrix product on the 5th-generation tensor cores:
// out[t, f] = sum_k x[t, k] * w[f, k], float accumulation, bf16 or float out.
//
// Both operands are K-major ("[rows, K] row-major"), which is how the engine holds
// activations [tokens, K] and weights [features, K]; the reference makes the same
// product through cuBLAS (cuda/kernels/gemm.cu:244-267).  One persistent CTA per SM:
//
//   warp 0      TMA producer: per stage one cp.async.bulk.tensor load of a tile of
//               up to 128 token rows x 64 K and one of BN feature rows x 64 K (128-byte
//               swizzle) into a ring of shared-memory stages, completion on an
//               mbarrier per stage;
//   warp 1      one thread issues tcgen05.mma (M = 128, N = BN, K = 16, four per stage)
//               with the accumulator in tensor memory; tcgen05.commit hands the stage
//               back to the producer.  The warp also owns the TMEM allocation: two
//               accumulators, so the epilogue of one tile overlaps the products of the
//               next;
//   warps 2-5   epilogue: tcgen05.ld of the accumulator (one TMEM lane = one token per
//               thread), conversion, 16-byte stores.
//
// BN (16..256 in steps of 16) and the ring's depth are chosen per call, not per
// build: the instruction descriptor and the TMA box are runtime values.  With few
// tokens (decode) the product is bound by streaming the weights once, so BN is
// picked to give about one tile per SM (for instance 48 features for a 6144-wide
// projection), the token tile shrinks to the tokens present, and the ring holds
// dozens of small stages to keep enough bytes in flight.  The MMA still computes
// 128 token rows; rows beyond the tokens present read whatever lies behind the
// token tile in shared memory and produce values that are never stored.  With
// many tokens (prefill) BN is 256 and the stages are 48 KB.
//
// Every mbarrier wait is bounded (about a second); on a timeout the kernel sets
// BF_ERR_WAIT in the error word, every role leaves its loop, outstanding copies and
// products are waited for (bounded), TMEM is freed and the kernel returns.
//
// No TMA load here uses multicast; every load reads this GPU's own memory.
#include <cuda.h>
#include <stdint.h>

#include "common.cuh"
#include "tma_utils.cuh"

#include <stdlib.h>

#include "umma_utils.cuh"

namespace {

struct GemmParams {
  int tokens, features, K;
  int tiles_t, tiles_f;        // tiles over tokens (128 each) and over features (bn each)
  int bn;                      // feature rows per tile, multiple of 16
  int a_rows;                  // token rows fetched per tile, multiple of 8
  int mma_rows;                // M of the tcgen05.mma: 128, or 64 with at most 16 tokens
  int stages;
  long long ldo;               // row stride of the output, in elements
  int* err;
};

constexpr int MAX_STAGES = 32;
constexpr int BAR_BYTES = 1024;              // barriers and flags, in front of the ring
constexpr int TAIL_BYTES = 16 * 1024;        // the MMA reads 128 token rows whatever a_rows is

template <typename OutT>
__global__ void __launch_bounds__(192, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x,
                    const __grid_constant__ CUtensorMap map_w, OutT* __restrict__ out,
                    const GemmParams p) {
  constexpr int TMEM_COLS = 512;             // two accumulators of up to 256 columns
  extern __shared__ __align__(16) uint8_t smem_raw[];
  // swizzled tiles must start on a 1024-byte boundary of the shared window
  uint8_t* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(base);
  uint64_t* empty = full + MAX_STAGES;
  uint64_t* acc_full = empty + MAX_STAGES;                  // [2]
  uint64_t* acc_empty = acc_full + 2;                       // [2]
  uint64_t* drain = acc_empty + 2;                          // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain + 1);
  volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* tiles = base + BAR_BYTES;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int units = p.tiles_t * p.tiles_f;
  const int kc_total = (p.K + BK - 1) / BK;
  const int a_bytes = p.a_rows * BK * 2, b_bytes = p.bn * BK * 2;
  const int stage_bytes = a_bytes + b_bytes;
  const int STAGES = p.stages;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full + a, 1);
      mbar_init(acc_empty + a, 128);
    }
    mbar_init(drain, 1);
    *abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
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

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int u = blockIdx.x; u < units && !*abort; u += gridDim.x) {
        const int tt = u % p.tiles_t, tf = u / p.tiles_t;
        for (int kc = 0; kc < kc_total; ++kc) {
          if (!mbar_wait(empty + stage, phase ^ 1, abort)) break;
          uint8_t* dst = tiles + (size_t)stage * stage_bytes;
          mbar_expect_tx(full + stage, stage_bytes);
          tma_load_2d(dst, &map_x, full + stage, kc * BK, tt * BM);
          tma_load_2d(dst + a_bytes, &map_w, full + stage, kc * BK, tf * p.bn);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      // c = float, a = b = bf16, both K-major, N = bn, M = 128
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                             ((uint32_t)(p.bn >> 3) << 17) | ((uint32_t)(p.mma_rows >> 4) << 24);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      for (int u = blockIdx.x; u < units && !*abort; u += gridDim.x) {
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
          const uint64_t b_desc = umma_desc_k_sw128(a_addr + a_bytes);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // 16 bf16 = 32 bytes further along K inside the swizzled row: +2 in 16-byte units
            umma_bf16(d_tmem, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc,
                      (kc > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(empty + stage);          // the stage is free once these products are done
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(acc_full + acc);           // the accumulator is complete
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // --------------------------------------------------------------- epilogue
    const int quarter = warp & 3;              // the TMEM lanes this warp may read
    const int row_in_tile = quarter * 32 + lane;
    const bool vec_ok = (p.ldo * sizeof(OutT)) % 16 == 0 && ((uintptr_t)out & 15) == 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
      const int tt = u % p.tiles_t, tf = u / p.tiles_t;
      const bool ok = !*abort && mbar_wait(acc_full + acc, acc_phase, abort);
      if (!epilogue_all(ok)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * 256);
      const int t = tt * BM + row_in_tile;     // token of this thread
      const bool warp_has_rows = tt * BM + quarter * 32 < p.tokens;
      if (warp_has_rows) {                     // uniform per warp: tcgen05.ld is warp-wide
        for (int c0 = 0; c0 < p.bn; c0 += 16) {
          uint32_t r[16];
          tmem_ld16(taddr + c0, r);
          const int f0 = tf * p.bn + c0;
          if (t < p.tokens && f0 < p.features) {
            OutT* dst = out + (size_t)t * p.ldo + f0;
            if (vec_ok && f0 + 16 <= p.features) {
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
                if (f0 + jj < p.features) bf_st(dst + jj, __uint_as_float(r[jj]));
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(acc_empty + acc);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  // ------------------------------------------------------------------ wind-down
  __syncthreads();
  if (*abort) {
    if (threadIdx.x == 0) atomicOr(p.err, BF_ERR_WAIT);
    if (warp == 0 && lane == 0) {
      // copies that were issued but never consumed: give each stage's barrier a bounded chance
      for (int s = 0; s < STAGES; ++s) {
        const long long t0 = clock64();
        while (!mbar_try_wait(full + s, 0) && !mbar_try_wait(full + s, 1) &&
               clock64() - t0 < WAIT_LIMIT_CYCLES / 16) {
        }
      }
    }
    if (warp == 1 && lane == 0) {
      umma_commit(drain);                      // products still in flight
      const long long t0 = clock64();
      while (!mbar_try_wait(drain, 0) && clock64() - t0 < WAIT_LIMIT_CYCLES / 16) {
      }
    }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
}

// ------------------------------------------------------------------------ host side
// A [rows, K] bf16 row-major matrix, fetched in boxes of box_rows x 64 with the 128-byte swizzle.
int make_map(CUtensorMap* map, const void* base, int rows, int K, long long ld, int box_rows) {
  return bf_make_tensor_map_bf16_2d(map, base, rows, K, ld, box_rows, BK);
}

template <typename OutT>
int launch(const void* x, const void* w, OutT* out, GemmParams p, long long ldx, long long ldw,
           int num_sms, cudaStream_t stream) {
  CUtensorMap mx, mw;
  int e = make_map(&mx, x, p.tokens, p.K, ldx, p.a_rows);
  if (e) return e;
  e = make_map(&mw, w, p.features, p.K, ldw, p.bn);
  if (e) return e;
  const size_t smem_max = 226 * 1024;
  const size_t stage_bytes = (size_t)(p.a_rows + p.bn) * BK * 2;
  const size_t fixed = 1024 /* alignment slack */ + BAR_BYTES + TAIL_BYTES;
  int stages = (int)((smem_max - fixed) / stage_bytes);
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  if (stages < 2) return (int)cudaErrorInvalidValue;
  p.stages = stages;
  const size_t smem = fixed + (size_t)stages * stage_bytes;
  auto kern = gemm_tcgen05_kernel<OutT>;
  static bool configured_on[BF_MAX_DEVICES];
  bool& configured = configured_on[bf_current_device()];
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)smem_max);
    if (ce != cudaSuccess) return (int)ce;
    configured = true;
  }
  const int units = p.tiles_t * p.tiles_f;
  const int grid = units < num_sms ? units : num_sms;
  kern<<<grid, 192, smem, stream>>>(mx, mw, out, p);
  return bf_launch_status();
}

}  // namespace

// Feature rows per tile (a multiple of 16, at most 256) for `tokens` x `features`: the width
// that wastes least of the last wave of tiles over `num_sms` SMs, wider tiles preferred when
// there is little to choose (more so with many tokens, where reuse of the token tile pays).
BF_EXPORT int bf_gemm_choose_bn(int tokens, int features, int num_sms) {
  const int tiles_t = (tokens + BM - 1) / BM;
  const double width_weight = tokens > 128 ? 0.25 : 0.04;
  int best = 16;
  double best_score = -1.0;
  for (int bn = 16; bn <= 256; bn += 16) {
    const long long tiles = (long long)tiles_t * ((features + bn - 1) / bn);
    const long long waves = (tiles + num_sms - 1) / num_sms;
    const double eff = (double)tiles / ((double)waves * num_sms);
    const double score = eff * (1.0 - width_weight + width_weight * bn / 256.0);
    if (score > best_score) {
      best_score = score;
      best = bn;
    }
  }
  return best;
}

// out[tokens, features] = x[tokens, K] * w[features, K]^T in bf16 with float accumulation.
// out_dtype: BF_DTYPE_BF16 or BF_DTYPE_F32.  bn: feature rows per tile (0: chosen here).
// Returns cudaErrorInvalidValue for shapes it does not take (K % 8 != 0, misaligned bases).
BF_EXPORT int bf_gemm_bf16_tcgen05(const void* x, const void* w, void* out, int tokens,
                                   int features, int K, long long ldx, long long ldw,
                                   long long ldo, int out_dtype, int bn, int num_sms, int* err,
                                   cudaStream_t stream) {
  if (tokens <= 0 || features <= 0) return 0;
  if (K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15))
    return (int)cudaErrorInvalidValue;
  if (bn <= 0) bn = bf_gemm_choose_bn(tokens, features, num_sms);
  if (bn % 16 || bn > 256) return (int)cudaErrorInvalidValue;
  GemmParams p;
  p.tokens = tokens;
  p.features = features;
  p.K = K;
  p.ldo = ldo;
  p.bn = bn;
  p.tiles_t = (tokens + BM - 1) / BM;
  p.tiles_f = (features + bn - 1) / bn;
  p.a_rows = tokens >= BM ? BM : ((tokens + 7) / 8) * 8;
  // At most 16 tokens lie in tensor memory lanes 0..15 whether the product has 128 rows or
  // 64; 64 rows are half the tensor work per weight byte (a decode step runs at the board's
  // power limit, so that is clock: see gemm_tcgen05_cluster.cu).
  static const int rows =
      getenv("BINFER_B200_GEMM_MMA_ROWS") ? atoi(getenv("BINFER_B200_GEMM_MMA_ROWS")) : 64;
  p.mma_rows = rows == 64 && tokens <= 16 ? 64 : 128;
  p.stages = 0;
  p.err = err;
  return out_dtype == BF_DTYPE_F32
             ? launch<float>(x, w, (float*)out, p, ldx, ldw, num_sms, stream)
             : launch<__nv_bfloat16>(x, w, (__nv_bfloat16*)out, p, ldx, ldw, num_sms, stream);
}
