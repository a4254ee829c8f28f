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
// accumulator of its own, warps 0 and 4 (which may read TMEM lanes 0..31; the tokens are rows
// 0..15) read and add the accumulators, half of the tile's columns each.  Reduction: the
// tile's columns are cut into C slices; CTA r owns slice r.  Every CTA writes each slice of
// its partial sum into the owner's shared memory (st.shared::cluster, laid out so that the
// lanes of a store are neighbours there), the cluster synchronises once (barrier.cluster),
// and each owner adds the C partials of its slice in ascending rank order and stores the
// result: one fixed order of summation, no atomics, no global workspace, and nothing spins
// on another CTA (the cluster barrier is the hardware's).
//
// The product itself has 64 rows when there are at most 32 token rows, else 128.  What
// happens to the sums is the kernel's FORM, a template parameter: stored as they are; added into the float residual stream with
// the next RMSNorm prepared; (q/k/v projection) head norms, rotation and the store into the
// cache pages, the tile's rows shared out by token instead of by column; (gate/up
// projection, clusters of one CTA) the activation, from tensor memory straight to global
// memory.  Each form is described at its export below.
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
  int mma_rows;                 // M of the tcgen05.mma: 128, or 64 (at most 32 token rows)
  int tok_rows;                 // token rows fetched and reduced: 8, 16, 32 or 64 (>= tokens)
  int replicate;                // at most 8 tokens, shown in every lane quarter of tensor memory
  int async_send;               // partial sums by st.async onto the owner's mbarrier (not q/k/v)
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
  // Fused "head norms, rotation and store into the pages" epilogue of the q/k/v projection
  // (q_out != null): a tile's columns are whole heads (bn a multiple of d) and the tile's
  // rows are shared out by token, token t to CTA t % cluster, so that an owner holds whole
  // heads of its tokens.  `out` is not written then.
  const float* q_w;             // per-head norm weights, null: no norm
  const float* k_w;
  const float* inv_freq;        // rot_half rotation frequencies, null: no rotation
  const int* positions;
  const int* slots;             // place of each token in the pages; negative: store nothing
  __nv_bfloat16* q_out;         // [tokens, nh * d]
  __nv_bfloat16* k_cache;       // [pages, nkv, page_size, d]; null with nkv = 0
  __nv_bfloat16* v_cache;
  int nh, nkv, d, rot_half, page_size;
  long long num_slots;
  float head_eps;
  BfRowScale rs;                // factor on the rows of the product (the norm before it)
  // Fused SwiGLU of the stacked gate/up projection (act_out != null; one CTA a tile, no
  // split of K): w is [2 inter, K], gate rows first; the tile's first bn/2 weight rows are
  // the gate rows of outputs tile * bn/2 .., the others the up rows of the same outputs, so
  // that one accumulator holds both; act_out[t, o] = silu(f g) * (f u), f the row's factor
  // (rs), goes from tensor memory to global memory with no pass through shared memory.
  __nv_bfloat16* act_out;
  long long ldact;
  int inter;
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

// The same store, asynchronous: it counts its 16 bytes on the mbarrier `bar` of the CTA that
// holds `addr` (both addresses in the cluster's shared window), so the receiver knows when
// everything sent to it has landed without the whole cluster meeting at a barrier.
__device__ __forceinline__ void st_async_v4(uint32_t addr, uint32_t bar, float a, float b,
                                            float c, float d) {
  asm volatile(
      "st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];"
      ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---- the q/k/v form's epilogue: what a warp needs of a token, and the rotation
struct QkvToken {
  int slot;
  float factor;                 // of the norm before the projection
  float sn[4], cs[4];           // of the lane's rotation pairs (frequencies lane + 32 j)
};
__device__ __forceinline__ QkvToken qkv_token(const ClusterGemmParams& p, int t, int lane) {
  QkvToken k;
  const BfRowShare share = bf_row_fetch(p.rs, t, lane);
  k.slot = p.k_cache ? p.slots[t] : -1;
  const float pos = p.inv_freq ? (float)p.positions[t] : 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    k.sn[j] = 0.f;
    k.cs[j] = 1.f;
    if (lane + 32 * j < p.rot_half) sincosf(pos * p.inv_freq[lane + 32 * j], &k.sn[j], &k.cs[j]);
  }
  k.factor = bf_row_finish(p.rs, share);
  return k;
}
// a lane holds the head's elements lane + 32 j; element i < rot_half turns with element
// i + rot_half, which is M = rot_half / 32 places further in the same lane
template <int M>
__device__ __forceinline__ void rotate_pairs(float (&v)[8], const QkvToken& k) {
#pragma unroll
  for (int j = 0; j < M; ++j) {
    const float a = v[j], b = v[j + M];
    v[j] = a * k.cs[j] - b * k.sn[j];
    v[j + M] = a * k.sn[j] + b * k.cs[j];
  }
}

// One stage's weight rows: the tile's bn rows, or (SwiGLU form) bn/2 gate rows and the bn/2
// up rows of the same outputs, one behind the other (bn/2 is a multiple of 8, so the second
// box starts on a swizzle period).
template <bool SWIGLU>
__device__ __forceinline__ void load_weights(const ClusterGemmParams& p, const CUtensorMap* map_w,
                                             uint8_t* dst, uint64_t* bar, int k, int tile) {
  if (!SWIGLU) {
    tma_load_2d(dst, map_w, bar, k, tile * p.bn);
  } else {
    const int h = p.bn / 2;
    tma_load_2d(dst, map_w, bar, k, tile * h);
    tma_load_2d(dst + (size_t)h * BK * 2, map_w, bar, k, p.inter + tile * h);
  }
}
__device__ __forceinline__ float silu_fast(float g) { return __fdividef(g, 1.f + __expf(-g)); }

// The epilogue's form is a template parameter, so that each instance carries only its own
// code: with all four behind run-time tests the plain product was 3 % slower.
enum { FORM_PLAIN = 0, FORM_ADD_NORM = 1, FORM_QKV = 2, FORM_SWIGLU = 3 };

constexpr int CL_THREADS = 256;       // eight warps: the roles of warps 1 to 3, then the epilogue

template <typename OutT, int FORM>
__global__ void __launch_bounds__(CL_THREADS, 1)
gemm_cluster_kernel(const __grid_constant__ CUtensorMap map_x,
                    const __grid_constant__ CUtensorMap map_w, OutT* __restrict__ out,
                    const ClusterGemmParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  constexpr bool kNorm = FORM == FORM_ADD_NORM, kQkv = FORM == FORM_QKV, kAct = FORM == FORM_SWIGLU;
  BF_TRACE_POINT(10 * BF_TR_GEMM);
  bf_pdl_trigger();
  uint8_t* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(base);
  uint64_t* empty = full + CL_MAX_STAGES;
  uint64_t* acc_full = empty + CL_MAX_STAGES;
  uint64_t* landed = acc_full + 1;                         // the partial sums sent to this CTA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(landed + 1);
  volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // recv[rank][token][slice column]: partial sums sent to this CTA, as the owner of a slice
  float* recv = reinterpret_cast<float*>(base + CL_BAR_BYTES);
  const int slice = p.bn / p.cluster;                          // columns owned per CTA
  const int own_tokens = (p.tokens + p.cluster - 1) / p.cluster;   // (q/k/v form) per CTA
  const int recv_bytes = kAct ? 0
                         : kQkv ? p.cluster * own_tokens * p.bn * 4
                                   : p.cluster * p.tok_rows * slice * 4;
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
    mbar_init(landed, 1);
    *abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // what this CTA, as the owner of a slice, will be sent: every rank's rows of it
    if (p.async_send) mbar_expect_tx(landed, (uint32_t)(p.cluster * p.tokens * (p.bn / p.cluster) * 4));
  }
  // (the peers learn that this barrier exists: waited for before the first send, long after)
  if (p.async_send) cluster_arrive();
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
      load_weights<kAct>(p, &map_w, tiles + (size_t)i * stage_bytes + a_bytes, full + i, (kc0 + i) * BK,
                   tile);
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
        load_weights<kAct>(p, &map_w, dst + a_bytes, full + stage, kc * BK, tile);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1 || warp == 3) {
    // Two issuing threads, an accumulator each (summed by the epilogue in a fixed order):
    // issuing a tcgen05.mma costs its thread about a hundred cycles whatever the product's
    // size, and with one thread that, not HBM, bounded the narrow projections.
    // A ring slot belongs to one issuer for good (slot s to issuer s % 2), so that the thread
    // waits for every fill of its slots in turn.  An mbarrier's phase is one bit: with the K
    // steps dealt out in turn and an odd number of slots, a thread met only every second fill
    // of a slot, always with the same parity, and its wait for fill u + 2 passed while fill
    // u + 1 was still in flight whenever the copies of several later steps had overtaken it.
    // The product then read a slot that was being written and freed it under the copy: rare
    // with few K steps, an "unspecified launch failure" (or a wait that gave up) once in a
    // thousand launches with a hundred of them.
    const int who = warp == 1 ? 0 : 1;
    if (lane == 0 && who < p.issuers && kc1 - kc0 > who) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                             ((uint32_t)(p.bn >> 3) << 17) | ((uint32_t)(p.mma_rows >> 4) << 24);
      const uint32_t acc = tmem_base + (uint32_t)(who * p.acc_stride);
      bool ok = true, first = true;
      for (int n = 0; n < kc1 - kc0; ++n) {
        const int stage = n % STAGES;
        if (p.issuers == 2 && (stage & 1) != who) continue;
        if (!mbar_wait(full + stage, (uint32_t)(n / STAGES) & 1u, abort)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(tiles + (size_t)stage * stage_bytes);
        // (replicate: every 8-row group of the product reads the tile's eight token rows)
        const uint64_t a_desc = umma_desc_k_sw128_sbo(a_addr, p.replicate ? 0u : 1024u);
        const uint64_t b_desc = umma_desc_k_sw128(a_addr + a_bytes);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          umma_bf16(acc, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc,
                    (!first || k > 0) ? 1u : 0u);
        first = false;
        umma_commit(empty + stage);
      }
      if (ok) umma_commit(acc_full);
    }
  }
  __syncwarp();
  // The epilogue: every warp whose lane quarter holds token rows.  Warp w may read the tensor
  // memory lanes of quarter w % 4 only; the two warps of a quarter (w and w + 4) share the
  // tile's columns.  A lane holds one token's row of the partial sum: row = lane for a 128-row
  // product; a 64-row product keeps rows 16 q .. 16 q + 15 in the first 16 lanes of quarter q
  // (so 64 token rows use all four quarters, 16 of them only warps 0 and 4).  Warps 1 to 3
  // come here when the last load or product is issued.
  // With at most eight tokens every quarter holds them all (the product's 8-row groups read
  // the same eight rows), and the eight warps take the 16-column chunks in turn: the sums
  // leave tensor memory in a quarter of the time that two warps took (1.3 to 1.9 us of a
  // product's 7 to 35).
  const int quarter = warp & 3;
  const int per = p.mma_rows == 64 ? 16 : 32;            // rows a lane quarter holds
  if (p.async_send) cluster_wait();                      // every peer's landing barrier exists
  const uint32_t landed_addr = smem_u32(landed);
  if (p.replicate || quarter * per < p.tok_rows) {
    const int row = p.replicate ? (lane < 8 ? lane : 1 << 20)
                                : (lane < per ? quarter * per + lane : 1 << 20);
    const uint32_t lanes = (uint32_t)(quarter * 32) << 16;
    const int width = kAct ? p.bn / 2 : p.bn;          // columns to walk: outputs or sums
    const int chunks = (width + 15) / 16, half = (chunks + 1) / 2;
    const int c_begin = p.replicate ? warp * 16 : warp >= 4 ? half * 16 : 0;
    const int c_end = p.replicate || warp >= 4 ? chunks * 16 : half * 16;
    const int c_step = p.replicate ? 8 * 16 : 16;
    // (SwiGLU form) the factor of this lane's row, worked out while the products run
    float factor = 1.f;
    if (kAct && p.rs.partials)
      for (int t = p.replicate ? 0 : quarter * per;
           t < p.tokens && t < (p.replicate ? 8 : (quarter + 1) * per); ++t) {
        const float ft = bf_row_factor(p.rs, t, lane);
        if (t == row) factor = ft;
      }
    bool have = kc1 > kc0;
    if (have) have = mbar_wait(acc_full, 0, abort);
    have = __all_sync(0xffffffffu, have);
    tc_fence_after();
    BF_TRACE_POINT(10 * BF_TR_GEMM + 5);
    const uint32_t my_recv = smem_u32(recv);
    for (int c0 = c_begin; c0 < c_end && kAct; c0 += c_step) {
      // gate columns c0.., up columns bn/2 + c0.. of both issuers' accumulators
      const int h = p.bn / 2;
      uint32_t g[16], u[16];
      if (have) {
        const uint32_t at = tmem_base + lanes + (uint32_t)c0;
        if (p.issuers == 2 && kc1 - kc0 >= 2) {
          uint32_t g2[16], u2[16];
          tmem_ld16_pair(at, at + (uint32_t)p.acc_stride, g, g2);
          tmem_ld16_pair(at + (uint32_t)h, at + (uint32_t)(p.acc_stride + h), u, u2);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            g[j] = __float_as_uint(__uint_as_float(g[j]) + __uint_as_float(g2[j]));
            u[j] = __float_as_uint(__uint_as_float(u[j]) + __uint_as_float(u2[j]));
          }
        } else {
          tmem_ld16_pair(at, at + (uint32_t)h, g, u);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) g[j] = u[j] = 0u;   // a timeout (flagged): zeros
      }
      if (row < p.tokens) {
        const int o0 = tile * h + c0;                     // first output of the chunk
        uint32_t packed[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float a = silu_fast(__uint_as_float(g[2 * j]) * factor) *
                          (__uint_as_float(u[2 * j]) * factor);
          const float b = silu_fast(__uint_as_float(g[2 * j + 1]) * factor) *
                          (__uint_as_float(u[2 * j + 1]) * factor);
          packed[j] = pack_bf16x2(__float_as_uint(a), __float_as_uint(b));
        }
        __nv_bfloat16* dst = p.act_out + (size_t)row * p.ldact + o0;
        if (c0 + 16 <= h && o0 + 16 <= p.inter) {         // (16-byte aligned: o0 and ldact are multiples of 8)
          reinterpret_cast<uint4*>(dst)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          reinterpret_cast<uint4*>(dst)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (c0 + j < h && o0 + j < p.inter)
              dst[j] = reinterpret_cast<const __nv_bfloat16*>(packed)[j];
        }
      }
    }
    for (int c0 = c_begin; c0 < c_end && !kAct; c0 += c_step) {
      uint32_t r[16];
      if (have) {
        if (p.issuers == 2 && kc1 - kc0 >= 2) {          // with the second issuer's share
          uint32_t r2[16];
          tmem_ld16_pair(tmem_base + lanes + c0, tmem_base + lanes + (uint32_t)p.acc_stride + c0,
                         r, r2);
#pragma unroll
          for (int j = 0; j < 16; ++j)
            r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(r2[j]));
        } else {
          tmem_ld16(tmem_base + lanes + c0, r);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) r[j] = 0u;     // no K steps here (or a timeout): send zeros
      }
      if (kQkv) {
        // the token's owner gets its whole row: recv[rank][own token][column]
        if (row < p.tokens) {
          const int at = (rank * own_tokens + row / p.cluster) * p.bn + c0;
          const uint32_t dst =
              map_to_rank(my_recv + (uint32_t)(at * 4), (uint32_t)(row % p.cluster));
#pragma unroll
          for (int q = 0; q < 4; ++q)
            st_cluster_v4(dst + 16 * q, __uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                          __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
        }
      } else if (row < p.tokens) {                        // (rows beyond are padding: never read)
        // the owner of these 16 columns gets them as recv[rank][group of 4 columns][token][4]:
        // the lanes of one store are then neighbours in the owner's shared memory (with the
        // token's row contiguous instead, every lane's 16 bytes went to a line of their own,
        // and the send took 2.5 to 3.9 us of a product's 10 to 15)
        const int owner = c0 / slice, group = (c0 - owner * slice) / 4;
        const int at = ((rank * (slice / 4) + group) * p.tok_rows + row) * 4;
        const uint32_t dst = map_to_rank(my_recv + (uint32_t)(at * 4), (uint32_t)owner);
        if (p.async_send) {
          const uint32_t bar = map_to_rank(landed_addr, (uint32_t)owner);
#pragma unroll
          for (int q = 0; q < 4; ++q)
            st_async_v4(dst + (uint32_t)(q * p.tok_rows * 16), bar, __uint_as_float(r[4 * q]),
                        __uint_as_float(r[4 * q + 1]), __uint_as_float(r[4 * q + 2]),
                        __uint_as_float(r[4 * q + 3]));
        } else {
#pragma unroll
          for (int q = 0; q < 4; ++q)
            st_cluster_v4(dst + (uint32_t)(q * p.tok_rows * 16), __uint_as_float(r[4 * q]),
                          __uint_as_float(r[4 * q + 1]), __uint_as_float(r[4 * q + 2]),
                          __uint_as_float(r[4 * q + 3]));
        }
      }
    }
    tc_fence_before();
  }

  // The plain forms' work after the barrier: an item is 4 neighbouring columns of one token.
  // The fused epilogue's inputs do not depend on the product: those of a thread's first item
  // are asked for before the cluster waits for its slowest member (further items' later).
  const int groups = slice / 4;
  const int n_plain = kQkv || kAct ? 0 : p.tokens * groups;
  float pre_r[4] = {0.f, 0.f, 0.f, 0.f}, pre_w[4] = {0.f, 0.f, 0.f, 0.f};
  if (kNorm && (int)threadIdx.x < n_plain) {
    const int g = threadIdx.x / p.tokens, t = threadIdx.x - g * p.tokens;
    const int f = tile * p.bn + rank * slice + g * 4;
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (f + k < p.features) {
        pre_r[k] = p.resid[(size_t)t * p.ldr + f + k];
        pre_w[k] = p.norm_w[f + k];
      }
  }

  // the q/k/v form: a warp per token of this CTA, which walks the tile's heads; what the
  // warp's first token needs beside the product (its place, the row's factor, the sines) is
  // asked for before the cluster's barrier.  The warps take their turns in the order in which
  // they are free: 2 has issued its loads long before the sums are there, 5 idles unless there
  // are more than 32 token rows, 1 and 3 issue products to the end, 4 and 0 send.
  const int heads_per_tile = kQkv ? p.bn / p.d : 1;
  const int n_mine = kQkv && p.tokens > rank ? (p.tokens - rank + p.cluster - 1) / p.cluster : 0;
  const int turn = warp == 2 ? 0 : warp == 5 ? 1 : warp == 1 ? 2 : warp == 3 ? 3 : warp == 4 ? 4 : 5;
  const bool takes_turns = kQkv && warp < 6;             // (six warps walk the tokens)
  QkvToken tk;
  if (takes_turns && turn < n_mine) tk = qkv_token(p, turn * p.cluster + rank, lane);

  // every thread of every CTA of the cluster: partials are in place after this
  BF_TRACE_POINT(10 * BF_TR_GEMM + 3);
  if (p.async_send) {
    // this CTA's slice has landed (a wait that gives up is flagged at the end; zeros or
    // stale sums are then stored, as after any such wait)
    mbar_wait(landed, 0, abort);
  } else {
    cluster_sync_all();
  }
  BF_TRACE_POINT(10 * BF_TR_GEMM + 4);

  for (int it = turn * heads_per_tile; takes_turns && it < n_mine * heads_per_tile; ++it) {
    const int lt = it / heads_per_tile, hh = it - lt * heads_per_tile;
    if (hh == heads_per_tile - 1) it += 5 * heads_per_tile;      // on to the token 6 further
    const int t = lt * p.cluster + rank;
    if (lt != turn && hh == 0) tk = qkv_token(p, t, lane);
    const int head = tile * p.bn / p.d + hh;
    if (head >= p.nh + 2 * p.nkv) continue;
    const bool is_q = head < p.nh, is_k = !is_q && head < p.nh + p.nkv;
    if (!is_q && tk.slot < 0) continue;
    const int nj = p.d >> 5;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float sum = 0.f;
      if (j < nj)
        for (int r = 0; r < p.cluster; ++r)                // ascending rank: one fixed order
          sum += recv[(r * own_tokens + lt) * p.bn + hh * p.d + lane + 32 * j];
      v[j] = sum * tk.factor;
    }
    if (is_q || is_k) {
      const float* w = is_q ? p.q_w : p.k_w;
      if (w) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
        const float inv = rsqrtf(warp_sum(ss) / (float)p.d + p.head_eps);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j < nj) v[j] *= inv * w[lane + 32 * j];
      }
      switch (p.rot_half >> 5) {
        case 1: rotate_pairs<1>(v, tk); break;
        case 2: rotate_pairs<2>(v, tk); break;
        case 3: rotate_pairs<3>(v, tk); break;
        case 4: rotate_pairs<4>(v, tk); break;
        default: break;
      }
    }
    __nv_bfloat16* dst;
    if (is_q) {
      dst = p.q_out + ((size_t)t * p.nh + head) * p.d;
    } else {
      if ((long long)tk.slot >= p.num_slots) {
        if (lane == 0) atomicOr(p.err, BF_ERR_SLOT);
        continue;
      }
      const int h = is_k ? head - p.nh : head - p.nh - p.nkv;
      const int page = tk.slot / p.page_size, off = tk.slot - page * p.page_size;
      dst = (is_k ? p.k_cache : p.v_cache) + (((size_t)page * p.nkv + h) * p.page_size + off) * p.d;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j < nj) dst[lane + 32 * j] = __float2bfloat16_rn(v[j]);
  }

  // this CTA's slice: add the partials in ascending rank order, store
  for (int idx = threadIdx.x; idx < n_plain; idx += blockDim.x) {
    const int g = idx / p.tokens, t = idx - g * p.tokens;
    float sum[4] = {0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < p.cluster; ++r) {
      const float4 v =
          *reinterpret_cast<const float4*>(recv + ((r * groups + g) * p.tok_rows + t) * 4);
      sum[0] += v.x;
      sum[1] += v.y;
      sum[2] += v.z;
      sum[3] += v.w;
    }
    const int f = tile * p.bn + rank * slice + g * 4;
    if (!kNorm) {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (f + k < p.features) bf_st(out + (size_t)t * p.ldo + f + k, sum[k]);
    } else {
      const bool first = idx == (int)threadIdx.x;
      float sq[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float x = 0.f;
        if (f + k < p.features) {
          float* rp = p.resid + (size_t)t * p.ldr + f + k;
          x = (first ? pre_r[k] : *rp) + sum[k];
          *rp = x;
          p.xt[(size_t)t * p.ldxt + f + k] =
              __float2bfloat16_rn(x * (first ? pre_w[k] : p.norm_w[f + k]));
        }
        sq[k] = x * x;
      }
      // rank 0's part of recv, which this thread has read: now the squares
      *reinterpret_cast<float4*>(recv + (g * p.tok_rows + t) * 4) =
          make_float4(sq[0], sq[1], sq[2], sq[3]);
    }
  }
  if (kNorm) {
    // one partial sum of squares per token and CTA, its columns added in ascending order
    __syncthreads();
    for (int t = threadIdx.x; t < p.tokens; t += blockDim.x) {
      float sq = 0.f;
      for (int col = 0; col < slice; ++col) sq += recv[((col >> 2) * p.tok_rows + t) * 4 + (col & 3)];
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
  // no CTA may exit while a peer could still write into its shared memory: every write to
  // this CTA was counted on its landing barrier (or happened before the cluster barrier),
  // which it has waited for above, so nothing more is needed here
}

template <typename OutT, int FORM>
int launch_cluster(const void* x, const void* w, OutT* out, ClusterGemmParams p, long long ldx,
                   long long ldw, cudaStream_t stream) {
  CUtensorMap mx, mw;
  static const int rows = getenv("BINFER_B200_GEMM_MMA_ROWS") ? atoi(getenv("BINFER_B200_GEMM_MMA_ROWS")) : 64;
  static const int replicate = getenv("BINFER_B200_GEMM_REPLICATE") ? atoi(getenv("BINFER_B200_GEMM_REPLICATE")) : 1;
  p.mma_rows = rows == 64 ? 64 : 128;
  // (the q/k/v form shares its tile's rows out by token and is left as it was)
  p.replicate = replicate && p.tokens <= 8 && p.q_out == nullptr ? 1 : 0;
  static const int async_send = getenv("BINFER_B200_GEMM_ASYNC_SEND") ? atoi(getenv("BINFER_B200_GEMM_ASYNC_SEND")) : 1;
  p.async_send = async_send && p.q_out == nullptr && p.act_out == nullptr ? 1 : 0;
  p.tok_rows = p.replicate ? 8 : p.tokens <= 16 ? 16 : p.tokens <= 32 ? 32 : 64;
  int e = bf_make_tensor_map_bf16_2d(&mx, x, p.tokens, p.K, ldx, p.tok_rows, BK);
  if (e) return e;
  e = bf_make_tensor_map_bf16_2d(&mw, w, p.features, p.K, ldw, p.act_out ? p.bn / 2 : p.bn, BK);
  if (e) return e;
  const size_t smem_max = 226 * 1024;
  const size_t stage_bytes = (size_t)(p.tok_rows + p.bn) * BK * 2;
  const size_t recv_rows =
      p.act_out ? 0
      : p.q_out ? (size_t)p.cluster * ((p.tokens + p.cluster - 1) / p.cluster)
                : (size_t)p.tok_rows;
  const size_t recv_bytes = (recv_rows * p.bn * 4 + 1023) & ~(size_t)1023;
  // behind the last stage the MMA still reads 128 token rows' worth of shared memory
  const size_t fixed = 1024 + CL_BAR_BYTES + recv_bytes + 16 * 1024;
  int stages = (int)((smem_max - fixed) / stage_bytes);
  if (stages > CL_MAX_STAGES) stages = CL_MAX_STAGES;
  if (stages < 2) return (int)cudaErrorInvalidValue;
  static const int issuers = getenv("BINFER_B200_GEMM_ISSUERS") ? atoi(getenv("BINFER_B200_GEMM_ISSUERS")) : 2;
  p.issuers = issuers == 1 ? 1 : 2;
  // an even ring with two issuers: slot s belongs to issuer s % 2, so the K steps go to the
  // issuers strictly in turn
  static const int even = getenv("BINFER_B200_GEMM_EVEN_STAGES") ? atoi(getenv("BINFER_B200_GEMM_EVEN_STAGES")) : 1;
  if (even && p.issuers == 2) stages -= stages % 2;
  p.stages = stages;
  // With at most 32 token rows (a 64-row product keeps rows 0..15 in tensor memory lanes
  // 0..15 and rows 16..31 in lanes 32..47) a 64-row product does: half the tensor work per
  // weight byte.  The time of one product is
  // the same, but a decode step is long enough to run into the board's power limit, and with
  // 128-row products for 8 tokens the SM clock settled near 1750 MHz instead of 1965 (36
  // layers, batch 8: 4.28 against 4.12 ms a step with every projection on this kernel).
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
  auto kern = gemm_cluster_kernel<OutT, FORM>;
  static bool configured_on[BF_MAX_DEVICES];
  bool& configured = configured_on[bf_current_device()];
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)smem_max);
    if (ce != cudaSuccess) return (int)ce;
    configured = true;
  }
  const int tiles = (p.features + p.bn - 1) / p.bn;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * p.cluster, 1, 1);
  cfg.blockDim = dim3(CL_THREADS, 1, 1);
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
  static const int max_c = getenv("BINFER_B200_CLUSTER_MAX_C") ? atoi(getenv("BINFER_B200_CLUSTER_MAX_C")) : 4;
  for (int i = 0; i < 3; ++i) {
    const int c = order[i];
    if (c > max_c) continue;
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
  ClusterGemmParams p = {};
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
             ? launch_cluster<float, FORM_PLAIN>(x, w, (float*)out, p, ldx, ldw, stream)
             : launch_cluster<__nv_bfloat16, FORM_PLAIN>(x, w, (__nv_bfloat16*)out, p, ldx, ldw,
                                                         stream);
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
  ClusterGemmParams p = {};
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
  return launch_cluster<__nv_bfloat16, FORM_ADD_NORM>(x, w, (__nv_bfloat16*)nullptr, p, ldx, ldw,
                                                     stream);
}

// How many clusters of c CTAs of this kernel can be resident at once (0 on an error).
static int resident_clusters(int c) {
  static int known[9] = {-1, -1, -1, -1, -1, -1, -1, -1, -1};
  if (c < 1 || c > 8) return 0;
  if (known[c] >= 0) return known[c];
  auto kern = gemm_cluster_kernel<__nv_bfloat16, FORM_QKV>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) !=
      cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(c * 148, 1, 1);
  cfg.blockDim = dim3(CL_THREADS, 1, 1);
  cfg.dynamicSmemBytes = 200 * 1024;              // one CTA an SM, as every launch of it has
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = c;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int resident = 0;
  if (cudaOccupancyMaxActiveClusters(&resident, kern, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return known[c] = resident;
}

// Tile and cluster for the q/k/v form: tiles of whole heads (bn a multiple of d, at most 256),
// clusters of 1 to 8 CTAs that each keep at least 4 K-steps, all clusters resident at once
// (asked of the occupancy calculator: clusters do not straddle GPCs, so the SM count alone
// does not tell).  The narrowest tile that gives at least min_ctas CTAs, with the largest
// such cluster: the time after the last weight byte grows with the tile's width (one warp
// sends the sums), and measured on the 8B shape 96 CTAs of 128 rows (13.3 us) beat 128 of 192
// (13.7) and 120 of 256 (15.0 and more).  If no arrangement gives min_ctas: the one with the
// most CTAs.  Returns the number of CTAs or 0.  Needs a device.
BF_EXPORT int bf_gemm_cluster_qkv_plan(int features, int K, int d, int num_sms, int min_ctas,
                                       int* bn_out, int* cluster_out) {
  if (d <= 0 || d % 32 || d > 256) return 0;
  const int kc = (K + BK - 1) / BK;
  int best_ctas = 0, best_bn = 0, best_c = 0;
  for (int bn = d; bn <= 256; bn += d) {
    const int tiles = (features + bn - 1) / bn;
    for (int c = 8; c >= 1; --c) {
      const int ctas = tiles * c;
      if (kc / c < 4 || ctas > num_sms || ctas <= best_ctas) continue;
      if (resident_clusters(c) < tiles) continue;
      best_ctas = ctas;
      best_bn = bn;
      best_c = c;
      break;                                      // smaller clusters of this tile: fewer CTAs
    }
    if (best_ctas >= min_ctas && min_ctas > 0) break;
  }
  if (best_ctas == 0) return 0;
  *bn_out = best_bn;
  *cluster_out = best_c;
  return best_ctas;
}

// The q/k/v projection with what follows it in its epilogue: x[tokens, K] * w[features, K]^T,
// features = (nh + 2 nkv) * d (nkv = 0 and no caches: queries only); each row times the factor
// of the norm before it (row_partials, as in bf_qk_norm_rope_kv_write); q and k heads normed
// (q_w, k_w: null for none) and turned (inv_freq: rot_half frequencies, a multiple of 32, or
// null); q to q_out [tokens, nh * d], k and v into the pages at slots[t].  bn and cluster from
// bf_gemm_cluster_qkv_plan.  Returns cudaErrorInvalidValue for what it does not take.
BF_EXPORT int bf_gemm_bf16_cluster_qkv(
    const void* x, const void* w, int tokens, int features, int K, long long ldx, long long ldw,
    int bn, int cluster, const float* q_w, const float* k_w, const float* inv_freq, int rot_half,
    const int* positions, const int* slots, void* q_out, void* k_cache, void* v_cache, int nh,
    int nkv, int d, int page_size, long long num_slots, float eps, const float* row_partials,
    int row_count, int row_width, float row_eps, int* err, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (tokens > CL_MAX_TOKENS || K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x & 15) ||
      ((uintptr_t)w & 15) || !q_out || !positions)
    return (int)cudaErrorInvalidValue;
  if (d <= 0 || d % 32 || d > 256 || bn <= 0 || bn > 256 || bn % d || cluster < 1 || cluster > 8 ||
      nh <= 0 || nkv < 0 || features != (nh + 2 * nkv) * d)
    return (int)cudaErrorInvalidValue;
  if (inv_freq && (rot_half <= 0 || rot_half % 32 || 2 * rot_half > d))
    return (int)cudaErrorInvalidValue;
  if (nkv > 0 && (!k_cache || !v_cache || !slots || page_size <= 0))
    return (int)cudaErrorInvalidValue;
  // only arrangements whose clusters are all resident at once (the plan gives no other; one
  // that needed a second wave, 24 clusters of 6, ended in a launch failure when it was tried)
  if (resident_clusters(cluster) < (features + bn - 1) / bn) return (int)cudaErrorInvalidValue;
  ClusterGemmParams p = {};
  p.tokens = tokens;
  p.features = features;
  p.K = K;
  p.bn = bn;
  p.cluster = cluster;
  p.err = err;
  p.q_w = q_w;
  p.k_w = k_w;
  p.inv_freq = inv_freq;
  p.rot_half = inv_freq ? rot_half : 0;
  p.positions = positions;
  p.slots = slots;
  p.q_out = (__nv_bfloat16*)q_out;
  p.k_cache = nkv > 0 ? (__nv_bfloat16*)k_cache : nullptr;
  p.v_cache = nkv > 0 ? (__nv_bfloat16*)v_cache : nullptr;
  p.nh = nh;
  p.nkv = nkv;
  p.d = d;
  p.page_size = page_size > 0 ? page_size : 1;
  p.num_slots = num_slots;
  p.head_eps = eps;
  p.rs.partials = row_partials;
  p.rs.count = row_count;
  p.rs.inv_width = row_width > 0 ? 1.f / (float)row_width : 0.f;
  p.rs.eps = row_eps;
  return launch_cluster<__nv_bfloat16, FORM_QKV>(x, w, (__nv_bfloat16*)nullptr, p, ldx, ldw,
                                                     stream);
}

// Tile for the SwiGLU form: the narrowest tile (bn = 2 h weight rows for h outputs, h a multiple
// of 8, bn at most 256) that gives every output a CTA in one wave.  Returns the number of
// CTAs, or 0 where there is none (more than 128 outputs an SM).
BF_EXPORT int bf_gemm_swiglu_plan(int inter, int K, int num_sms, int* bn_out) {
  if (inter <= 0 || num_sms <= 0 || (K + BK - 1) / BK < 4) return 0;
  int h = (inter + num_sms - 1) / num_sms;
  h = (h + 7) / 8 * 8;
  if (h < 16) h = 16;
  if (2 * h > 256) return 0;
  *bn_out = 2 * h;
  return (inter + h - 1) / h;
}

// act[tokens, inter] = silu(f g) * (f u) with [g | u] = x[tokens, K] * w[2 inter, K]^T (gate
// rows first) and f the factor of the norm before the projection (row_partials as in
// bf_silu_mul_scaled; null: 1), as one kernel for at most 64 token rows.  bn from
// bf_gemm_swiglu_plan.  Returns cudaErrorInvalidValue for what it does not take.
BF_EXPORT int bf_gemm_bf16_swiglu(const void* x, const void* w, int tokens, int inter, int K,
                                  long long ldx, long long ldw, int bn, void* act,
                                  long long ldact, const float* row_partials, int row_count,
                                  int row_width, float row_eps, int* err, cudaStream_t stream) {
  if (tokens <= 0 || inter <= 0) return 0;
  if (tokens > CL_MAX_TOKENS || K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x & 15) ||
      ((uintptr_t)w & 15) || !act || ((uintptr_t)act & 15) || ldact % 8)
    return (int)cudaErrorInvalidValue;
  if (bn < 32 || bn > 256 || bn % 16) return (int)cudaErrorInvalidValue;
  ClusterGemmParams p = {};
  p.tokens = tokens;
  p.features = 2 * inter;
  p.K = K;
  p.bn = bn;
  p.cluster = 1;
  p.err = err;
  p.act_out = (__nv_bfloat16*)act;
  p.ldact = ldact;
  p.inter = inter;
  p.rs.partials = row_partials;
  p.rs.count = row_count;
  p.rs.inv_width = row_width > 0 ? 1.f / (float)row_width : 0.f;
  p.rs.eps = row_eps;
  return launch_cluster<__nv_bfloat16, FORM_SWIGLU>(x, w, (__nv_bfloat16*)nullptr, p, ldx, ldw,
                                                     stream);
}

BF_TRACE_READER(bf_trace_read_gemm_tcgen05_cluster)
