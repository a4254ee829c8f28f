// bf16 matrix product for few tokens (at most 64) against a weight too narrow to give every
// SM a tile: out[t, f] = sum_k x[t, k] * w[f, k], with the K range split over a thread-block
// cluster and the partial sums combined through distributed shared memory.
//
// Why: a tcgen05.mma with M = 128 occupies the tensor pipe for about 128 cycles however
// small N is, so a CTA only streams weights at the rate HBM can deliver when each product
// covers many weight rows (N = 192..256 feature rows = 6..8 KB per product).  A projection
// with 4096 or 6144 output features then has only 16 to 32 tiles for 148 SMs.  Here a
// cluster of C CTAs (2, 4 or 8) shares one tile: CTA r of the cluster multiplies the r-th
// part of the K range, so C times as many SMs stream.  The reference has no counterpart:
// it calls cuBLAS for every product (cuda/kernels/gemm.cu:244-267).
//
// Per CTA: warp 2 issues the TMA loads (token tile + BN x 64 weight tile per stage, 128-byte
// swizzle), warps 1 and 3 issue tcgen05.mma for the K steps in turn, each into a TMEM
// accumulator of its own, warp 0 (which may read TMEM lanes 0..31; the tokens are rows
// 0..15) reads and adds the accumulators.  Reduction: the tile's columns are cut
// into C slices; CTA r owns slice r.  Every CTA writes each slice of its partial sum into
// the owner's shared memory (st.shared::cluster), the cluster synchronises once
// (barrier.cluster), and each owner adds the C partials of its slice in ascending rank
// order and stores the result: one fixed order of summation, no atomics, no global
// workspace, and nothing spins on another CTA (the cluster barrier is the hardware's).
//
// mbarrier waits are bounded (about a second); on a timeout the CTA sets BF_ERR_WAIT,
// still contributes (zeros) and still joins the cluster barrier, frees TMEM and returns.
// No TMA load uses multicast; every load reads this GPU's own memory.
#include <cuda.h>
#include <stdint.h>
#include <stdlib.h>

#include "common.cuh"
#include "tma_utils.cuh"
#include "umma_utils.cuh"

namespace {

constexpr int CL_MAX_STAGES = 16;
constexpr int CL_MAX_TOKENS = 64;             // token rows: 16, 32 or 64 are fetched and reduced
constexpr int CL_BAR_BYTES = 512;

struct ClusterGemmParams {
  int tokens, features, K;
  int bn;                       // feature rows per tile (multiple of 16 * cluster)
  int cluster;                  // CTAs per tile
  int stages;
  int issuers;                  // threads that issue tcgen05.mma, 1 or 2
  int tok_rows;                 // token rows fetched and reduced: 16, 32 or 64 (>= tokens)
  int tmem_cols;                // tensor memory columns the CTA allocates (a power of two)
  int acc_stride;               // columns between the two issuers' accumulators
  long long ldo;
  int* err;
  // Fused "add into the residual stream and prepare the next norm" epilogue (resid != null):
  // resid[t, f] += sum; xt[t, f] = bf16(resid[t, f] * norm_w[f]); and this CTA's part of the
  // row's sum of squares goes to partials[t, blockIdx.x].  `out` is not written then.
  float* resid;
  const float* norm_w;
  __nv_bfloat16* xt;
  float* partials;
  long long ldr, ldxt;
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;"
               ::: "memory");
}
// address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b),
               "f"(c), "f"(d)
               : "memory");
}

template <typename OutT>
__global__ void __launch_bounds__(192, 1)
gemm_cluster_kernel(const __grid_constant__ CUtensorMap map_x,
                    const __grid_constant__ CUtensorMap map_w, OutT* __restrict__ out,
                    const ClusterGemmParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  BF_TRACE_POINT(10 * BF_TR_GEMM);
  bf_pdl_trigger();
  uint8_t* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(base);
  uint64_t* empty = full + CL_MAX_STAGES;
  uint64_t* acc_full = empty + CL_MAX_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // recv[rank][token][slice column]: partial sums sent to this CTA, as the owner of a slice
  float* recv = reinterpret_cast<float*>(base + CL_BAR_BYTES);
  const int slice = p.bn / p.cluster;                          // columns owned per CTA
  const int recv_bytes = p.cluster * p.tok_rows * slice * 4;
  uint8_t* tiles = base + CL_BAR_BYTES + ((recv_bytes + 1023) & ~1023);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)cluster_rank();
  const int tile = blockIdx.x / p.cluster;
  const int kc_total = (p.K + BK - 1) / BK;
  const int kc0 = (int)((long long)kc_total * rank / p.cluster);
  const int kc1 = (int)((long long)kc_total * (rank + 1) / p.cluster);
  const int a_bytes = p.tok_rows * BK * 2, b_bytes = p.bn * BK * 2;
  const int stage_bytes = a_bytes + b_bytes;
  const int STAGES = p.stages;
  const int TMEM_COLS = p.tmem_cols;                     // room for the issuers' accumulators

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    mbar_init(acc_full, min(p.issuers, max(kc1 - kc0, 1)));   // one arrival per issuing thread with work
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
  // Barriers and tensor memory are set up.  The weights do not depend on the kernel before
  // this one, so the first ring of weight tiles is asked for before waiting for it: when
  // this kernel was launched early (programmatic dependent launch) they stream in while the
  // predecessor finishes.  The activations are fetched after the wait.
  const int pre = min(STAGES, kc1 - kc0);
  if (warp == 2 && lane == 0) {
    for (int i = 0; i < pre; ++i) {
      mbar_expect_tx(full + i, stage_bytes);
      tma_load_2d(tiles + (size_t)i * stage_bytes + a_bytes, &map_w, full + i, (kc0 + i) * BK,
                  tile * p.bn);
    }
  }
  bf_pdl_wait();
  BF_TRACE_POINT(10 * BF_TR_GEMM + 1);

  if (warp == 2) {
    if (lane == 0) {
      for (int i = 0; i < pre; ++i)
        tma_load_2d(tiles + (size_t)i * stage_bytes, &map_x, full + i, (kc0 + i) * BK, 0);
      int stage = pre == STAGES ? 0 : pre;
      uint32_t phase = pre == STAGES ? 1 : 0;
      for (int kc = kc0 + pre; kc < kc1; ++kc) {
        if (!mbar_wait(empty + stage, phase ^ 1, abort)) break;
        uint8_t* dst = tiles + (size_t)stage * stage_bytes;
        mbar_expect_tx(full + stage, stage_bytes);
        tma_load_2d(dst, &map_x, full + stage, kc * BK, 0);
        tma_load_2d(dst + a_bytes, &map_w, full + stage, kc * BK, tile * p.bn);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1 || warp == 3) {   // (warp 4 idles; warp 5 reads token rows 32..63)
    // Two issuing threads, K steps in turn, an accumulator each (summed by the epilogue in
    // a fixed order): issuing a tcgen05.mma costs its thread about a hundred cycles whatever
    // the product's size, and with one thread that, not HBM, bounded the narrow projections.
    const int who = warp == 1 ? 0 : 1;
    if (lane == 0 && who < p.issuers && kc1 - kc0 > who) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                             ((uint32_t)(p.bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      const uint32_t acc = tmem_base + (uint32_t)(who * p.acc_stride);
      bool ok = true;
      for (int n = who; n < kc1 - kc0; n += p.issuers) {
        const int stage = n % STAGES;
        if (!mbar_wait(full + stage, (uint32_t)(n / STAGES) & 1u, abort)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(tiles + (size_t)stage * stage_bytes);
        const uint64_t a_desc = umma_desc_k_sw128(a_addr);
        const uint64_t b_desc = umma_desc_k_sw128(a_addr + a_bytes);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          umma_bf16(acc, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc,
                    (n > who || k > 0) ? 1u : 0u);
        umma_commit(empty + stage);
      }
      if (ok) umma_commit(acc_full);
    }
  } else if (warp == 0 || (warp == 5 && p.tok_rows > 32)) {
    // warp 0: TMEM lanes 0..31, warp 5 (more than 32 token rows): lanes 32..63; a lane holds
    // one token's row of the partial sum
    const int row = (warp == 0 ? 0 : 32) + lane;
    const uint32_t lanes = (uint32_t)(warp == 0 ? 0 : 32) << 16;
    bool have = kc1 > kc0;
    if (have) have = mbar_wait(acc_full, 0, abort);
    have = __all_sync(0xffffffffu, have);
    tc_fence_after();
    const uint32_t my_recv = smem_u32(recv);
    for (int c0 = 0; c0 < p.bn; c0 += 16) {
      uint32_t r[16];
      if (have) {
        tmem_ld16(tmem_base + lanes + c0, r);
        if (p.issuers == 2 && kc1 - kc0 >= 2) {          // the second issuer's share
          uint32_t r2[16];
          tmem_ld16(tmem_base + lanes + (uint32_t)p.acc_stride + c0, r2);
#pragma unroll
          for (int j = 0; j < 16; ++j)
            r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(r2[j]));
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) r[j] = 0u;     // no K steps here (or a timeout): send zeros
      }
      if (row < p.tok_rows) {
        const int owner = c0 / slice, col = c0 - owner * slice;
        const uint32_t dst = map_to_rank(
            my_recv + (uint32_t)(((rank * p.tok_rows + row) * slice + col) * 4), (uint32_t)owner);
#pragma unroll
        for (int q = 0; q < 4; ++q)
          st_cluster_v4(dst + 16 * q, __uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                        __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
      }
    }
    tc_fence_before();
  }

  // the fused epilogue's inputs do not depend on the product: they are asked for before the
  // cluster waits for its slowest member (up to four elements a thread; more are read later)
  float pre_r[4], pre_w[4];
  if (p.resid) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int idx = threadIdx.x + j * blockDim.x;
      const int t = idx / slice, col = idx - t * slice;
      const int f = tile * p.bn + rank * slice + col;
      const bool in = idx < p.tokens * slice && f < p.features;
      pre_r[j] = in ? p.resid[(size_t)t * p.ldr + f] : 0.f;
      pre_w[j] = in ? p.norm_w[f] : 0.f;
    }
  }

  // every thread of every CTA of the cluster: partials are in place after this
  cluster_sync_all();

  // this CTA's slice: add the partials in ascending rank order, store
  int j = 0;
  for (int idx = threadIdx.x; idx < p.tokens * slice; idx += blockDim.x, ++j) {
    const int t = idx / slice, col = idx - t * slice;
    float sum = 0.f;
    for (int r = 0; r < p.cluster; ++r) sum += recv[(r * p.tok_rows + t) * slice + col];
    const int f = tile * p.bn + rank * slice + col;
    if (!p.resid) {
      if (f < p.features) bf_st(out + (size_t)t * p.ldo + f, sum);
    } else {
      float x = 0.f;
      if (f < p.features) {
        float* rp = p.resid + (size_t)t * p.ldr + f;
        // (the selects keep pre_r and pre_w in registers)
        const float r0 = j == 0 ? pre_r[0] : j == 1 ? pre_r[1] : j == 2 ? pre_r[2] : pre_r[3];
        const float w0 = j == 0 ? pre_w[0] : j == 1 ? pre_w[1] : j == 2 ? pre_w[2] : pre_w[3];
        x = (j < 4 ? r0 : *rp) + sum;
        *rp = x;
        p.xt[(size_t)t * p.ldxt + f] = __float2bfloat16_rn(x * (j < 4 ? w0 : p.norm_w[f]));
      }
      recv[t * slice + col] = x * x;                     // rank 0's part of recv: read above, by this thread
    }
  }
  if (p.resid) {
    // one partial sum of squares per token and CTA, its columns added in ascending order
    __syncthreads();
    for (int t = threadIdx.x; t < p.tokens; t += blockDim.x) {
      float sq = 0.f;
      for (int col = 0; col < slice; ++col) sq += recv[t * slice + col];
      p.partials[(size_t)t * gridDim.x + blockIdx.x] = sq;
    }
  }

  __syncthreads();
  BF_TRACE_POINT(10 * BF_TR_GEMM + 2);
  if (*abort && threadIdx.x == 0) atomicOr(p.err, BF_ERR_WAIT);
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
  // no CTA may exit while a peer could still write into its shared memory: all writes
  // happened before the cluster barrier above, so nothing more is needed here
}

template <typename OutT>
int launch_cluster(const void* x, const void* w, OutT* out, ClusterGemmParams p, long long ldx,
                   long long ldw, cudaStream_t stream) {
  CUtensorMap mx, mw;
  p.tok_rows = p.tokens <= 16 ? 16 : p.tokens <= 32 ? 32 : 64;
  int e = bf_make_tensor_map_bf16_2d(&mx, x, p.tokens, p.K, ldx, p.tok_rows, BK);
  if (e) return e;
  e = bf_make_tensor_map_bf16_2d(&mw, w, p.features, p.K, ldw, p.bn, BK);
  if (e) return e;
  const size_t smem_max = 226 * 1024;
  const size_t stage_bytes = (size_t)(p.tok_rows + p.bn) * BK * 2;
  const size_t recv_bytes = ((size_t)p.tok_rows * p.bn * 4 + 1023) & ~(size_t)1023;
  // behind the last stage the MMA still reads 128 token rows' worth of shared memory
  const size_t fixed = 1024 + CL_BAR_BYTES + recv_bytes + 16 * 1024;
  int stages = (int)((smem_max - fixed) / stage_bytes);
  if (stages > CL_MAX_STAGES) stages = CL_MAX_STAGES;
  if (stages < 2) return (int)cudaErrorInvalidValue;
  p.stages = stages;
  static const int issuers = getenv("BINFER_B200_GEMM_ISSUERS") ? atoi(getenv("BINFER_B200_GEMM_ISSUERS")) : 2;
  p.issuers = issuers == 1 ? 1 : 2;
  int need = p.issuers * p.bn, cols = 32;
  while (cols < need) cols *= 2;
  p.tmem_cols = cols;
  p.acc_stride = p.bn;
  // Never less than 120 KB, so that two of these CTAs cannot share an SM: each allocates
  // tensor memory (which blocks while another CTA holds it) and then waits for its cluster,
  // and with two clusters' CTAs paired on the same SMs in opposite order that is a cycle.
  // (Seen once, with the shared memory capped at 110 KB for an experiment: the launch failed.)
  size_t smem = fixed + (size_t)stages * stage_bytes;
  if (smem < 120 * 1024) smem = 120 * 1024;
  auto kern = gemm_cluster_kernel<OutT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)smem_max);
    if (ce != cudaSuccess) return (int)ce;
    configured = true;
  }
  const int tiles = (p.features + p.bn - 1) / p.bn;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * p.cluster, 1, 1);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = p.cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = bf_pdl_enabled();
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  cudaError_t ce = cudaLaunchKernelEx(&cfg, kern, mx, mw, out, p);
  if (ce != cudaSuccess) return (int)ce;
  return bf_launch_status();
}

}  // namespace

// Tile width and cluster size for `features` x K on `num_sms` SMs.  Clusters of 4 measured
// best on a B200 (8 schedules worse, 2 leaves too few CTAs); a weight wide enough to give
// nearly every SM a tile of its own (the gate/up projection) takes "clusters" of one CTA,
// which is the same kernel without a split; the tile width (a multiple of
// 16 per CTA of the cluster, at most 256 feature rows) is the one that brings the number of
// CTAs closest to, and not above, the SM count, each CTA keeping at least 4 K-steps.
// Returns the number of CTAs, or 0 (outputs untouched) when no split is worth it.
BF_EXPORT int bf_gemm_cluster_plan(int features, int K, int num_sms, int* bn_out,
                                   int* cluster_out) {
  const int kc = (K + BK - 1) / BK;
  int best_ctas = 0, best_bn = 0, best_c = 0;
  const int order[3] = {4, 2, 1};
  for (int i = 0; i < 3; ++i) {
    const int c = order[i];
    if (kc / c < 4) continue;
    const int max_ctas = (num_sms / c) * c;
    for (int bn = 256; bn >= 64; bn -= 16) {
      if (bn % (16 * c)) continue;
      const int ctas = ((features + bn - 1) / bn) * c;
      if (ctas > max_ctas) continue;
      if (ctas > best_ctas) {
        best_ctas = ctas;
        best_bn = bn;
        best_c = c;
      }
    }
  }
  if (best_ctas == 0) return 0;
  *bn_out = best_bn;
  *cluster_out = best_c;
  return best_ctas;
}

// out[tokens, features] = x[tokens, K] * w[features, K]^T for tokens <= 64, the K range split
// over clusters of `cluster` CTAs.  bn: feature rows per tile, a multiple of 16 * cluster,
// at most 256.  Returns cudaErrorInvalidValue for what it does not take.
BF_EXPORT int bf_gemm_bf16_cluster(const void* x, const void* w, void* out, int tokens,
                                   int features, int K, long long ldx, long long ldw,
                                   long long ldo, int out_dtype, int bn, int cluster, int* err,
                                   cudaStream_t stream) {
  if (tokens <= 0 || features <= 0) return 0;
  if (tokens > CL_MAX_TOKENS || K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x & 15) ||
      ((uintptr_t)w & 15))
    return (int)cudaErrorInvalidValue;
  if ((cluster != 1 && cluster != 2 && cluster != 4 && cluster != 8) || bn <= 0 || bn > 256 ||
      bn % (16 * cluster))
    return (int)cudaErrorInvalidValue;
  ClusterGemmParams p;
  p.tokens = tokens;
  p.features = features;
  p.K = K;
  p.bn = bn;
  p.cluster = cluster;
  p.stages = 0;
  p.ldo = ldo;
  p.err = err;
  p.resid = nullptr;
  p.norm_w = nullptr;
  p.xt = nullptr;
  p.partials = nullptr;
  p.ldr = p.ldxt = 0;
  return out_dtype == BF_DTYPE_F32
             ? launch_cluster<float>(x, w, (float*)out, p, ldx, ldw, stream)
             : launch_cluster<__nv_bfloat16>(x, w, (__nv_bfloat16*)out, p, ldx, ldw, stream);
}

// The same product with the residual stream and the next norm in its epilogue:
//   resid[tokens, features] (float) += x * w^T;   xt = bf16(resid * norm_w)   (per feature);
//   partials[t, c] = CTA c's part of sum_f resid[t, f]^2,  c < the number of CTAs, which is
//   ceil(features / bn) * cluster and is returned in *n_partials.
// The norm's output is xt * rsqrt(sum_c partials[t, c] / features + eps): the factor is left
// to the kernel after the next product (BfRowScale).  No other output is written.
BF_EXPORT int bf_gemm_bf16_cluster_add_norm(const void* x, const void* w, int tokens, int features,
                                            int K, long long ldx, long long ldw, int bn,
                                            int cluster, float* resid, long long ldr,
                                            const float* norm_w, void* xt, long long ldxt,
                                            float* partials, int* n_partials, int* err,
                                            cudaStream_t stream) {
  if (tokens <= 0 || features <= 0) return 0;
  if (tokens > CL_MAX_TOKENS || K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x & 15) ||
      ((uintptr_t)w & 15) || !resid || !norm_w || !xt || !partials)
    return (int)cudaErrorInvalidValue;
  if ((cluster != 1 && cluster != 2 && cluster != 4 && cluster != 8) || bn <= 0 || bn > 256 ||
      bn % (16 * cluster))
    return (int)cudaErrorInvalidValue;
  ClusterGemmParams p;
  p.tokens = tokens;
  p.features = features;
  p.K = K;
  p.bn = bn;
  p.cluster = cluster;
  p.stages = 0;
  p.ldo = 0;
  p.err = err;
  p.resid = resid;
  p.norm_w = norm_w;
  p.xt = (__nv_bfloat16*)xt;
  p.partials = partials;
  p.ldr = ldr;
  p.ldxt = ldxt;
  if (n_partials) *n_partials = ((features + bn - 1) / bn) * cluster;
  return launch_cluster<__nv_bfloat16>(x, w, (__nv_bfloat16*)nullptr, p, ldx, ldw, stream);
}

BF_TRACE_READER(bf_trace_read_gemm_tcgen05_cluster)
