// Causal flash attention for prompt portions (rows that bring more than one token),
// reading every key and value from the paged bf16 cache.
//
// Grid (query tile, head, portion).  A CTA of 4 warps takes 64 consecutive queries
// of one portion for one head; each warp owns 16 query rows.  Keys are walked in
// tiles of 64 whose edges are multiples of 64 counted from position 0, fetched
// page by page with cp.async into a double-buffered shared-memory tile.  Scores and
// P.V run on mma.sync m16n8k16 (bf16 in, float accumulate); the softmax is online,
// in float, with exp2 and the scale folded in.  A query at absolute position p sees
// keys j in (p - window, p] (window 0: all j <= p): a portion that starts in the
// middle of a prompt reads the keys of earlier portions from their pages like any
// other key.
//
// The reference's prefill attention is a scalar kernel, one warp per query row, over
// the fresh keys of whole prompts only, one launch per sequence
// (cuda/kernels/bf16_kernels.cu:873-1024; src/engine/batched_engine.ts:1061-1090).
#include <float.h>

#include "common.cuh"
#include "mma_utils.cuh"

#define PF_BM 64
#define PF_BN 64
#define PF_THREADS 128

template <int D>
__global__ void __launch_bounds__(PF_THREADS)
prefill_attention_kernel(const __nv_bfloat16* __restrict__ q,
                         const __nv_bfloat16* __restrict__ k_cache,
                         const __nv_bfloat16* __restrict__ v_cache,
                         const int* __restrict__ items,   // [n, 4]: seq, first row, rows, first position
                         const int* __restrict__ block_tables, int table_stride,
                         __nv_bfloat16* __restrict__ out, int nh, int nkv, int page_size,
                         int num_pages, int window, float scale_log2, int* __restrict__ err) {
  constexpr int LD = D + 8;
  constexpr int CPK = D / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem_raw);        // [2][64][LD]
  __nv_bfloat16* Vs = Ks + 2 * PF_BN * LD;                               // [2][64][LD]
  long long* rowoff = reinterpret_cast<long long*>(Vs + 2 * PF_BN * LD); // [2][64]

  const int* it = items + 4 * blockIdx.z;
  const int seq = it[0], row0 = it[1], qlen = it[2], pos0 = it[3];
  // the last query tiles see the most keys: they are launched first
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x, h = blockIdx.y;
  if (qt * PF_BM >= qlen) return;
  const int g = h / (nh / nkv);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r0 = lane >> 2, cq = (lane & 3) * 2;
  const int* table = block_tables + (size_t)seq * table_stride;

  const int p_first = pos0 + qt * PF_BM;
  const int p_last = min(pos0 + qlen - 1, p_first + PF_BM - 1);
  const int j_lo = window > 0 ? max(0, p_first - window + 1) : 0;
  const int kt_first = j_lo / PF_BN, kt_last = p_last / PF_BN;

  // this thread's two query rows
  const int l0 = qt * PF_BM + warp * 16 + r0, l1 = l0 + 8;     // index inside the portion
  const bool v0 = l0 < qlen, v1 = l1 < qlen;
  const int pr0 = pos0 + l0, pr1 = pos0 + l1;                  // absolute positions
  const int jl0 = window > 0 ? max(0, pr0 - window + 1) : 0;
  const int jl1 = window > 0 ? max(0, pr1 - window + 1) : 0;

  unsigned qa[D / 16][4];
  {
    const __nv_bfloat16* q0 = q + ((size_t)(row0 + l0) * nh + h) * D;
    const __nv_bfloat16* q1 = q + ((size_t)(row0 + l1) * nh + h) * D;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int c = ks * 16 + cq;
      qa[ks][0] = v0 ? *reinterpret_cast<const unsigned*>(q0 + c) : 0u;
      qa[ks][1] = v1 ? *reinterpret_cast<const unsigned*>(q1 + c) : 0u;
      qa[ks][2] = v0 ? *reinterpret_cast<const unsigned*>(q0 + c + 8) : 0u;
      qa[ks][3] = v1 ? *reinterpret_cast<const unsigned*>(q1 + c + 8) : 0u;
    }
  }

  auto fetch = [&](int kt, int buf) {
    // where each key of the tile lives (threads 0..63), then the copies (all threads)
    if (tid < PF_BN) {
      const int j = kt * PF_BN + tid;
      long long off = -1;
      if (j >= j_lo && j <= p_last) {
        const int lp = j / page_size;
        const int page = table[lp];
        if (page < 0 || page >= num_pages) {
          atomicOr(err, BF_ERR_PAGE);
        } else {
          off = (((long long)page * nkv + g) * page_size + (j - lp * page_size)) * D;
        }
      }
      rowoff[buf * PF_BN + tid] = off;
    }
    __syncthreads();
    __nv_bfloat16* kd = Ks + (size_t)buf * PF_BN * LD;
    __nv_bfloat16* vd = Vs + (size_t)buf * PF_BN * LD;
    for (int c = tid; c < PF_BN * CPK; c += PF_THREADS) {
      const int key = c / CPK, part = c - key * CPK;
      const long long off = rowoff[buf * PF_BN + key];
      cp_async16(kd + key * LD + part * 8, off >= 0 ? k_cache + off + part * 8 : k_cache,
                 off >= 0 ? 16 : 0);
      cp_async16(vd + key * LD + part * 8, off >= 0 ? v_cache + off + part * 8 : v_cache,
                 off >= 0 ? 16 : 0);
    }
    cp_async_commit();
  };

  float m0 = -INFINITY, m1 = -INFINITY, s0 = 0.f, s1 = 0.f;
  float o[D / 8][4];
#pragma unroll
  for (int dn = 0; dn < D / 8; ++dn)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[dn][i] = 0.f;

  fetch(kt_first, 0);
  for (int kt = kt_first; kt <= kt_last; ++kt) {
    const int buf = (kt - kt_first) & 1;
    if (kt < kt_last) {
      fetch(kt + 1, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();                              // tile kt has landed for every thread
    const __nv_bfloat16* kb = Ks + (size_t)buf * PF_BN * LD;
    const __nv_bfloat16* vb = Vs + (size_t)buf * PF_BN * LD;

    float s[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int i = 0; i < 4; ++i) s[nt][i] = 0.f;
#pragma unroll
      for (int ks = 0; ks < D / 16; ks += 2) {
        unsigned b[4];
        ldmatrix_x4(b, kb + (nt * 8 + (lane & 7)) * LD + ks * 16 + (lane >> 3) * 8);
        mma_bf16_16816(s[nt], qa[ks], b[0], b[1]);
        mma_bf16_16816(s[nt], qa[ks + 1], b[2], b[3]);
      }
    }
    float t0 = -INFINITY, t1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int j = kt * PF_BN + nt * 8 + cq + i;
        s[nt][i] = (v0 && j >= jl0 && j <= pr0) ? s[nt][i] * scale_log2 : -INFINITY;
        s[nt][2 + i] = (v1 && j >= jl1 && j <= pr1) ? s[nt][2 + i] * scale_log2 : -INFINITY;
      }
      t0 = fmaxf(t0, fmaxf(s[nt][0], s[nt][1]));
      t1 = fmaxf(t1, fmaxf(s[nt][2], s[nt][3]));
    }
    t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 1));
    t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 2));
    t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 1));
    t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 2));
    const float n0 = fmaxf(m0, t0), n1 = fmaxf(m1, t1);
    const float u0 = n0 == -INFINITY ? 0.f : n0, u1 = n1 == -INFINITY ? 0.f : n1;
    const float c0 = m0 == -INFINITY ? 0.f : exp2f(m0 - u0);
    const float c1 = m1 == -INFINITY ? 0.f : exp2f(m1 - u1);
    m0 = n0;
    m1 = n1;
    float a0 = 0.f, a1 = 0.f;
    unsigned pa[4][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const float e0 = exp2f(s[nt][0] - u0), e1 = exp2f(s[nt][1] - u0);
      const float e2 = exp2f(s[nt][2] - u1), e3 = exp2f(s[nt][3] - u1);
      a0 += e0 + e1;
      a1 += e2 + e3;
      pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(e0, e1);
      pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(e2, e3);
    }
    s0 = s0 * c0 + a0;                            // per-thread partial row sums; reduced at the end
    s1 = s1 * c1 + a1;
#pragma unroll
    for (int dn = 0; dn < D / 8; ++dn) {
      o[dn][0] *= c0;
      o[dn][1] *= c0;
      o[dn][2] *= c1;
      o[dn][3] *= c1;
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
      for (int dn = 0; dn < D / 8; dn += 2) {
        unsigned b[4];
        const int m = lane >> 3;
        ldmatrix_x4_trans(b, vb + (kk * 16 + (m & 1) * 8 + (lane & 7)) * LD + (dn + (m >> 1)) * 8);
        mma_bf16_16816(o[dn], pa[kk], b[0], b[1]);
        mma_bf16_16816(o[dn + 1], pa[kk], b[2], b[3]);
      }
    }
    __syncthreads();                              // everyone is done with this buffer
  }
  s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
  s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
  s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
  s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
  const float i0 = v0 ? 1.f / s0 : 0.f, i1 = v1 ? 1.f / s1 : 0.f;
  __nv_bfloat16* o0 = out + ((size_t)(row0 + l0) * nh + h) * D;
  __nv_bfloat16* o1 = out + ((size_t)(row0 + l1) * nh + h) * D;
#pragma unroll
  for (int dn = 0; dn < D / 8; ++dn) {
    if (v0) *reinterpret_cast<unsigned*>(o0 + dn * 8 + cq) = pack_bf16(o[dn][0] * i0, o[dn][1] * i0);
    if (v1) *reinterpret_cast<unsigned*>(o1 + dn * 8 + cq) = pack_bf16(o[dn][2] * i1, o[dn][3] * i1);
  }
}

template <int D>
static int launch_prefill(const void* q, const void* k_cache, const void* v_cache, const int* items,
                          int n_items, int max_rows, const int* block_tables, int table_stride,
                          void* out, int nh, int nkv, int page_size, int num_pages, int window,
                          float scale, int* err, cudaStream_t stream) {
  constexpr int LD = D + 8;
  const size_t smem = (size_t)4 * PF_BN * LD * 2 + 2 * PF_BN * 8;
  auto kern = prefill_attention_kernel<D>;
  static bool configured_on[BF_MAX_DEVICES];
  bool& configured = configured_on[bf_current_device()];
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid((max_rows + PF_BM - 1) / PF_BM, nh, n_items);
  kern<<<grid, PF_THREADS, smem, stream>>>(
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, items,
      block_tables, table_stride, (__nv_bfloat16*)out, nh, nkv, page_size, num_pages, window,
      scale * 1.4426950408889634f, err);
  return bf_launch_status();
}

// items: int32 [n_items, 4] on the device: (request index in the block table, first token
// row, number of rows, absolute position of the first row).  max_rows: the largest row count.
// Returns cudaErrorInvalidValue for head sizes it does not take (take the generic kernel).
BF_EXPORT int bf_prefill_attention(const void* q, const void* k_cache, const void* v_cache,
                                   const int* items, int n_items, int max_rows,
                                   const int* block_tables, int table_stride, void* out, int nh,
                                   int nkv, int d, int page_size, int num_pages, int window,
                                   float scale, int* err, cudaStream_t stream) {
  if (n_items <= 0 || max_rows <= 0) return 0;
  if (nkv <= 0 || nh % nkv) return (int)cudaErrorInvalidValue;
#define BF_PF_CASE(DD)                                                                          \
  case DD:                                                                                      \
    return launch_prefill<DD>(q, k_cache, v_cache, items, n_items, max_rows, block_tables,      \
                              table_stride, out, nh, nkv, page_size, num_pages, window, scale,  \
                              err, stream)
  switch (d) {
    BF_PF_CASE(32);
    BF_PF_CASE(64);
    BF_PF_CASE(96);
    BF_PF_CASE(128);
    BF_PF_CASE(256);
    default:
      return (int)cudaErrorInvalidValue;
  }
#undef BF_PF_CASE
}
