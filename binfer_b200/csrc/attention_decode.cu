// Split-KV attention for single-token (decode) rows over the paged bf16 cache.
//
// Grid (split, kv_head, row).  A CTA takes the 128 keys [split*128, split*128+128)
// of one request for one kv head, and all query heads of that kv head's group
// together: the group's heads are the rows of the tensor-core tile, so every key
// and value byte is read from HBM once per group.  The reference's decode kernel
// is one block per (sequence, query head), reads each kv head once per query head
// and never splits the keys across blocks (cuda/kernels/paged_attention.cu:370-489).
//
// The whole 128-key K and V tile is fetched with cp.async in one go (64 KB for
// head size 128); three CTAs fit an SM, so one CTA's math overlaps another's
// loads.  Scores and P.V run on mma.sync m16n8k16 (bf16 in, float accumulate);
// softmax is float with exp2 and the scale folded in.  Each of the 4 warps owns 32
// keys; the warps' (max, sum, out) are merged in shared memory, and the CTA writes
// an unnormalised partial to scratch memory.  A second kernel merges the splits
// of a row in ascending order and normalises.  Which keys a warp and a split own
// depends only on the key's position, so the result for a row does not depend on
// the rest of the batch.
//
// Scratch: part_o float [rows, nh, max_splits, D], part_ml float [rows, nh, max_splits, 2].
#include <float.h>

#include <stdlib.h>

#include "common.cuh"
#include "mma_utils.cuh"

#define DEC_SPLIT 128
#define DEC_THREADS 128

template <int D>
__global__ void __launch_bounds__(DEC_THREADS)
decode_attention_split_kernel(const __nv_bfloat16* __restrict__ q,
                              const __nv_bfloat16* __restrict__ k_cache,
                              const __nv_bfloat16* __restrict__ v_cache,
                              const int* __restrict__ rows, const int* __restrict__ seq_of_token,
                              const int* __restrict__ positions,
                              const int* __restrict__ block_tables, int table_stride,
                              float* __restrict__ part_o, float* __restrict__ part_ml, int nh,
                              int nkv, int page_size, int num_pages, int window, int max_splits,
                              float scale_log2, int* __restrict__ err) {
  constexpr int LD = D + 8;            // padded row: ldmatrix rows fall in distinct banks
  constexpr int CPK = D / 8;           // 16-byte chunks per key
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* Vs = Ks + DEC_SPLIT * LD;
  long long* rowoff = reinterpret_cast<long long*>(Vs + DEC_SPLIT * LD);

  const int split = blockIdx.x, g = blockIdx.y, r = blockIdx.z;
  const int t = rows ? rows[r] : r;
  const int p = positions[t];
  const int j0 = window > 0 ? max(0, p - window + 1) : 0;
  const int k_begin = split * DEC_SPLIT;
  // the grid has max_splits splits: keys beyond them have nowhere to put their partial
  if (split == 0 && g == 0 && threadIdx.x == 0 && p / DEC_SPLIT >= max_splits)
    atomicOr(err, BF_ERR_SPLITS);
  if (k_begin > p || k_begin + DEC_SPLIT <= j0) return;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = nh / nkv;
  const int* table = block_tables + (size_t)seq_of_token[t] * table_stride;

  {  // where each key of the tile lives
    const int j = k_begin + tid;
    long long off = -1;
    if (j >= j0 && j <= p) {
      const int lp = j / page_size;
      const int page = table[lp];
      if (page < 0 || page >= num_pages) {
        atomicOr(err, BF_ERR_PAGE);
      } else {
        off = (((long long)page * nkv + g) * page_size + (j - lp * page_size)) * D;
      }
    }
    rowoff[tid] = off;
  }
  __syncthreads();
  for (int c = tid; c < DEC_SPLIT * CPK; c += DEC_THREADS) {
    const int key = c / CPK, part = c - key * CPK;
    const long long off = rowoff[key];
    cp_async16(Ks + key * LD + part * 8, off >= 0 ? k_cache + off + part * 8 : k_cache,
               off >= 0 ? 16 : 0);
  }
  cp_async_commit();
  for (int c = tid; c < DEC_SPLIT * CPK; c += DEC_THREADS) {
    const int key = c / CPK, part = c - key * CPK;
    const long long off = rowoff[key];
    cp_async16(Vs + key * LD + part * 8, off >= 0 ? v_cache + off + part * 8 : v_cache,
               off >= 0 ? 16 : 0);
  }
  cp_async_commit();

  const int r0 = lane >> 2, cq = (lane & 3) * 2;
  const int wkey = warp * 32;          // this warp's first key inside the tile
  bool first_block = true;

  for (int hb = 0; hb < G; hb += 16) {
    const int gblk = min(16, G - hb);
    // query fragments: rows = heads of the group, zero beyond the group
    unsigned qa[D / 16][4];
    {
      const __nv_bfloat16* q0 = q + ((size_t)t * nh + (size_t)g * G + hb + r0) * D;
      const __nv_bfloat16* q1 = q0 + (size_t)8 * D;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int c = ks * 16 + cq;
        qa[ks][0] = r0 < gblk ? *reinterpret_cast<const unsigned*>(q0 + c) : 0u;
        qa[ks][1] = r0 + 8 < gblk ? *reinterpret_cast<const unsigned*>(q1 + c) : 0u;
        qa[ks][2] = r0 < gblk ? *reinterpret_cast<const unsigned*>(q0 + c + 8) : 0u;
        qa[ks][3] = r0 + 8 < gblk ? *reinterpret_cast<const unsigned*>(q1 + c + 8) : 0u;
      }
    }
    if (first_block) {
      cp_async_wait<1>();
      __syncthreads();                 // every thread's K chunks have landed
    }
    float s[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
      for (int i = 0; i < 4; ++i) s[nt][i] = 0.f;
#pragma unroll
      for (int ks = 0; ks < D / 16; ks += 2) {
        unsigned b[4];
        ldmatrix_x4(b, Ks + (wkey + nt * 8 + (lane & 7)) * LD + ks * 16 + (lane >> 3) * 8);
        mma_bf16_16816(s[nt], qa[ks], b[0], b[1]);
        mma_bf16_16816(s[nt], qa[ks + 1], b[2], b[3]);
      }
    }
    // mask, scale, softmax over this warp's 32 keys
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
    const float u0 = m0 == -INFINITY ? 0.f : m0, u1 = m1 == -INFINITY ? 0.f : m1;
    float l0 = 0.f, l1 = 0.f;
    unsigned pa[2][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const float e0 = exp2f(s[nt][0] - u0), e1 = exp2f(s[nt][1] - u0);
      const float e2 = exp2f(s[nt][2] - u1), e3 = exp2f(s[nt][3] - u1);
      l0 += e0 + e1;
      l1 += e2 + e3;
      pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(e0, e1);
      pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(e2, e3);
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    if (first_block) {
      cp_async_wait<0>();
      __syncthreads();                 // V has landed
      first_block = false;
    }
    float o[D / 8][4];
#pragma unroll
    for (int dn = 0; dn < D / 8; ++dn)
#pragma unroll
      for (int i = 0; i < 4; ++i) o[dn][i] = 0.f;
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
      for (int dn = 0; dn < D / 8; dn += 2) {
        unsigned b[4];
        const int m = lane >> 3;
        ldmatrix_x4_trans(b, Vs + (wkey + kk * 16 + (m & 1) * 8 + (lane & 7)) * LD +
                                 (dn + (m >> 1)) * 8);
        mma_bf16_16816(o[dn], pa[kk], b[0], b[1]);
        mma_bf16_16816(o[dn + 1], pa[kk], b[2], b[3]);
      }
    }

    // merge the four warps' partials in shared memory.  With a single head block the K
    // tile is dead here (every warp passed the barrier between its score and its P.V
    // phase), so the merge buffer lies over it; with several head blocks the tiles are
    // read again, and the buffer sits behind them.
    float* red = G <= 16 ? reinterpret_cast<float*>(Ks)
                         : reinterpret_cast<float*>(rowoff + DEC_SPLIT);
    float* red_m = red;                       // [4][16]
    float* red_l = red + 64;                  // [4][16]
    float* red_o = red + 128;                 // [4][16][D]
    if ((lane & 3) == 0) {
      red_m[warp * 16 + r0] = m0;
      red_m[warp * 16 + r0 + 8] = m1;
      red_l[warp * 16 + r0] = l0;
      red_l[warp * 16 + r0 + 8] = l1;
    }
#pragma unroll
    for (int dn = 0; dn < D / 8; ++dn) {
      float* o0 = red_o + ((size_t)warp * 16 + r0) * D + dn * 8 + cq;
      float* o1 = o0 + (size_t)8 * D;
      o0[0] = o[dn][0];
      o0[1] = o[dn][1];
      o1[0] = o[dn][2];
      o1[1] = o[dn][3];
    }
    __syncthreads();
    for (int idx = tid; idx < gblk * D; idx += DEC_THREADS) {
      const int row = idx / D, col = idx - row * D;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) M = fmaxf(M, red_m[w * 16 + row]);
      float L = 0.f, O = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float mw = red_m[w * 16 + row];
        const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
        L += red_l[w * 16 + row] * f;
        O += red_o[((size_t)w * 16 + row) * D + col] * f;
      }
      const size_t base = ((size_t)r * nh + (size_t)g * G + hb + row) * max_splits + split;
      part_o[base * D + col] = O;
      if (col == 0) {
        part_ml[base * 2] = M;
        part_ml[base * 2 + 1] = L;
      }
    }
    __syncthreads();
  }
}

// Merge the splits of each (row, head) and normalise.  The kernel is all latency (a few KB
// from L2 per (row, head); 128 KB at 32 768 keys), so it is built around the number of
// dependent round trips and needs neither shared memory nor a block-wide barrier: a warp owns
// 16 (or 32) columns of one (row, head) for all of its splits.  Lane = (4 columns, one of 8 (or
// 4) classes of splits): the lane's splits are those with index = class mod 8.  First pass: every (m, l)
// pair of the lane's splits, up to 32 in flight at once (asked for, when there is no window,
// together with the row's position, whose value says which of them count), gives the
// maximum M over the classes by shuffles.  Second pass, 16 splits a lane at once: the pairs
// again (from L2) with the partial outputs, weights exp2(m - M), sums over the lane's splits
// in ascending order, then over the classes in one fixed tree.  32 splits (4096 keys) take
// two round trips, 256 splits three; the kernel before this one (a block per (row, head),
// a thread per column, 32 splits at once) took two and ten.
// Two shapes of it.  4 classes and 8 / 8 in flight (a block per (row, head), 40 registers)
// is the one for most steps.  8 classes and 32 / 16 in flight (two blocks per (row, head), 86
// registers) is launched where the rows' contexts may reach 16 384 keys (128 splits) and
// there are at most 1 024 (row, head) pairs: 29.8 against 39.5 us for one row of 32 768 keys,
// but 28.0 against 26.3 us for 8 rows of 4 096 and 188 against 177 us for 64 rows, where fewer
// of its blocks are resident beside the attention kernel's and they come in more waves.
// (row, head) pairs up to which the first shape is launched (BINFER_B200_MERGE_FEW_PAIRS)
static int merge_few_pairs() {
  static const int n = getenv("BINFER_B200_MERGE_FEW_PAIRS") ? atoi(getenv("BINFER_B200_MERGE_FEW_PAIRS")) : 1024;
  return n;
}
#define MERGE_FEW_PAIRS merge_few_pairs()
#define MERGE_MANY_SPLITS 128
template <int D, int MERGE_CLASSES, int UA, int UB>
__global__ void __launch_bounds__(128)
decode_attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                              const int* __restrict__ rows, const int* __restrict__ positions,
                              __nv_bfloat16* __restrict__ out, int nh, int window,
                              int max_splits) {
  BF_TRACE_POINT(10 * BF_TR_MERGE);
  bf_pdl_trigger();
  bf_pdl_wait();
  BF_TRACE_POINT(10 * BF_TR_MERGE + 1);
  const int r = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int CG = 32 / MERGE_CLASSES;                   // groups of 4 columns a warp covers
  const int cb = (blockIdx.z * 4 + warp) * CG * 4;         // the warp's first column
  if (cb >= D) return;
  const int cg = lane % CG, sc = lane / CG;                // column group of 4, class of splits
  const size_t base = ((size_t)r * nh + h) * max_splits;
  const float2* ml2 = reinterpret_cast<const float2*>(part_ml) + base;
  const int t = rows ? rows[r] : r;
  const float2 none = make_float2(-INFINITY, 0.f);

  // first pass, first chunk: asked for before the position is known where the first split is 0
  float2 first[UA];
  if (window <= 0) {
#pragma unroll
    for (int u = 0; u < UA; ++u) {
      const int i = sc + MERGE_CLASSES * u;
      first[u] = i < max_splits ? __ldcg(ml2 + i) : none;
    }
  }
  const int p = positions[t];
  const int j0 = window > 0 ? max(0, p - window + 1) : 0;
  // never beyond the scratch: the attention kernel has flagged a row that needs more splits
  const int s_first = j0 / DEC_SPLIT, n = min(p / DEC_SPLIT, max_splits - 1) - s_first + 1;
  const float2* ml = ml2 + s_first;
  float M = -INFINITY;
  for (int k0 = 0; k0 < n; k0 += MERGE_CLASSES * UA) {
    float2 v[UA];
#pragma unroll
    for (int u = 0; u < UA; ++u) {
      const int i = k0 + sc + MERGE_CLASSES * u;
      v[u] = i >= n ? none : (k0 == 0 && window <= 0) ? first[u] : __ldcg(ml + i);
    }
#pragma unroll
    for (int u = 0; u < UA; ++u) M = fmaxf(M, v[u].x);
  }
#pragma unroll
  for (int d = CG; d <= 16; d *= 2) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, d));

  float L = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  const float* po = part_o + (base + s_first) * D + cb + cg * 4;
  for (int k0 = 0; k0 < n; k0 += MERGE_CLASSES * UB) {
    float2 v[UB];
    float4 o[UB];
#pragma unroll
    for (int u = 0; u < UB; ++u) {
      const int i = k0 + sc + MERGE_CLASSES * u;
      v[u] = i < n ? __ldcg(ml + i) : none;
      o[u] = i < n ? __ldcg(reinterpret_cast<const float4*>(po + (size_t)i * D))
                   : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < UB; ++u) {
      const float w = v[u].x == -INFINITY ? 0.f : exp2f(v[u].x - M);
      L += v[u].y * w;
      acc.x += o[u].x * w;
      acc.y += o[u].y * w;
      acc.z += o[u].z * w;
      acc.w += o[u].w * w;
    }
  }
#pragma unroll
  for (int d = CG; d <= 16; d *= 2) {                       // over the classes: one fixed tree
    L += __shfl_xor_sync(0xffffffffu, L, d);
    acc.x += __shfl_xor_sync(0xffffffffu, acc.x, d);
    acc.y += __shfl_xor_sync(0xffffffffu, acc.y, d);
    acc.z += __shfl_xor_sync(0xffffffffu, acc.z, d);
    acc.w += __shfl_xor_sync(0xffffffffu, acc.w, d);
  }
  if (sc == 0) {
    const float inv = n > 0 ? 1.f / L : 0.f;
    uint2 packed;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&packed);
    o2[0] = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
    o2[1] = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(out + ((size_t)t * nh + h) * D + cb + cg * 4) = packed;
  }
}

template <int D>
static int launch_decode(const void* q, const void* k_cache, const void* v_cache, const int* rows,
                         const int* seq_of_token, const int* positions, const int* block_tables,
                         int table_stride, void* out, float* part_o, float* part_ml, int n_rows,
                         int nh, int nkv, int page_size, int num_pages, int window,
                         int max_splits, float scale, int* err, cudaStream_t stream) {
  constexpr int LD = D + 8;
  const size_t tiles = (size_t)2 * DEC_SPLIT * LD * 2 + DEC_SPLIT * 8;
  const size_t merge = (size_t)(128 + 4 * 16 * D) * 4;
  const size_t smem_max = tiles + merge;
  const size_t smem = nh / nkv <= 16 ? tiles : smem_max;
  auto kern = decode_attention_split_kernel<D>;
  static bool configured_on[BF_MAX_DEVICES];
  bool& configured = configured_on[bf_current_device()];
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem_max);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(max_splits, nkv, n_rows);
  kern<<<grid, DEC_THREADS, smem, stream>>>(
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, rows,
      seq_of_token, positions, block_tables, table_stride, part_o, part_ml, nh, nkv, page_size,
      num_pages, window, max_splits, scale * 1.4426950408889634f, err);
  int e = bf_launch_status();
  if (e) return e;
  if (n_rows * nh <= MERGE_FEW_PAIRS && max_splits >= MERGE_MANY_SPLITS)
    decode_attention_merge_kernel<D, 8, 32, 16><<<dim3(n_rows, nh, (D + 63) / 64), 128, 0, stream>>>(
      part_o, part_ml, rows, positions, (__nv_bfloat16*)out, nh, window, max_splits);
  else
    decode_attention_merge_kernel<D, 4, 8, 8><<<dim3(n_rows, nh, (D + 127) / 128), 128, 0, stream>>>(
      part_o, part_ml, rows, positions, (__nv_bfloat16*)out, nh, window, max_splits);
  return bf_launch_status();
}

// max_splits must be >= ceil(longest context / 128) of the rows given; a row that needs more
// sets BF_ERR_SPLITS in the error word, and the splits beyond the scratch are left out (no
// kernel reads or writes past part_o / part_ml).
// Returns cudaErrorInvalidValue for head sizes it does not take (take the generic kernel).
BF_EXPORT int bf_decode_attention(const void* q, const void* k_cache, const void* v_cache,
                                  const int* rows, const int* seq_of_token, const int* positions,
                                  const int* block_tables, int table_stride, void* out,
                                  float* part_o, float* part_ml, int n_rows, int nh, int nkv,
                                  int d, int page_size, int num_pages, int window, int max_splits,
                                  float scale, int* err, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (nkv <= 0 || nh % nkv) return (int)cudaErrorInvalidValue;
#define BF_DEC_CASE(DD)                                                                         \
  case DD:                                                                                      \
    return launch_decode<DD>(q, k_cache, v_cache, rows, seq_of_token, positions, block_tables,  \
                             table_stride, out, part_o, part_ml, n_rows, nh, nkv, page_size,    \
                             num_pages, window, max_splits, scale, err, stream)
  switch (d) {
    BF_DEC_CASE(32);
    BF_DEC_CASE(64);
    BF_DEC_CASE(96);
    BF_DEC_CASE(128);
    BF_DEC_CASE(256);
    default:
      return (int)cudaErrorInvalidValue;
  }
#undef BF_DEC_CASE
}

BF_EXPORT int bf_decode_attention_split_keys() { return DEC_SPLIT; }

// Only the second half: merge the partials that a split kernel left in scratch.
BF_EXPORT int bf_decode_attention_merge(const float* part_o, const float* part_ml, const int* rows,
                                        const int* positions, void* out, int n_rows, int nh, int d,
                                        int window, int max_splits, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
#define BF_MERGE_CASE(DD)                                                                     \
  case DD:                                                                                    \
    return n_rows * nh <= MERGE_FEW_PAIRS && max_splits >= MERGE_MANY_SPLITS                  \
               ? bf_launch_pdl(decode_attention_merge_kernel<DD, 8, 32, 16>,                  \
                               dim3(n_rows, nh, (DD + 63) / 64), dim3(128), 0, stream, part_o, \
                               part_ml, rows, positions, (__nv_bfloat16*)out, nh, window,     \
                               max_splits)                                                    \
               : bf_launch_pdl(decode_attention_merge_kernel<DD, 4, 8, 8>,                    \
                               dim3(n_rows, nh, (DD + 127) / 128), dim3(128), 0, stream,      \
                               part_o, part_ml, rows, positions, (__nv_bfloat16*)out, nh,     \
                               window, max_splits)
  switch (d) {
    BF_MERGE_CASE(32);
    BF_MERGE_CASE(64);
    BF_MERGE_CASE(96);
    BF_MERGE_CASE(128);
    BF_MERGE_CASE(256);
    default:
      return (int)cudaErrorInvalidValue;
  }
#undef BF_MERGE_CASE
}

// ------------------------------------------------------------------------------
// The same attention with its scratch inside the library (see the header for who
// needs this and for the rules of use).  Host code must not pass the array's
// name to a kernel: on the host that name is only a handle for the runtime.  Its
// device address is looked up once per device and kept.
#include "attention_decode_static.h"

static __device__ __align__(256) unsigned char bf_decode_static_scratch[BF_DECODE_STATIC_SCRATCH_BYTES];

#define BF_STATIC_MAX_DEVICES 64
static void* bf_decode_static_ptr[BF_STATIC_MAX_DEVICES];   // device address, per device

BF_EXPORT const char* bf_decode_attention_static_error(int code) {
  switch (code) {
    case 0: return "ok";
    case BF_STATIC_ERR_TOO_LARGE:
      return "n_rows * nh * max_splits * (d + 2) * 4 bytes exceeds the library's 8 MiB scratch "
             "array; use fewer rows or splits per call, or bf_decode_attention with scratch of "
             "your own";
    case BF_STATIC_ERR_HEAD_DIM: return "head size must be one of 32, 64, 96, 128, 256";
    case BF_STATIC_ERR_ARGUMENT: return "a required pointer is null or a size is not positive";
    case BF_STATIC_ERR_DEVICE: return "the current device index is beyond the 64 the library tracks";
    default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown code";
  }
}

BF_EXPORT int bf_decode_attention_static(const void* q, const void* k_cache, const void* v_cache,
                                         const int* rows, const int* seq_of_token,
                                         const int* positions, const int* block_tables,
                                         int table_stride, void* out, int n_rows, int nh, int nkv,
                                         int d, int page_size, int num_pages, int window,
                                         int max_splits, float scale, int* err,
                                         cudaStream_t stream) {
  if (!q || !k_cache || !v_cache || !seq_of_token || !positions || !block_tables || !out || !err)
    return BF_STATIC_ERR_ARGUMENT;
  if (n_rows <= 0 || nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0 || max_splits <= 0)
    return BF_STATIC_ERR_ARGUMENT;
  if (d != 32 && d != 64 && d != 96 && d != 128 && d != 256) return BF_STATIC_ERR_HEAD_DIM;
  const unsigned long long cells = (unsigned long long)n_rows * nh * max_splits;
  const unsigned long long need = cells * (unsigned long long)(d + 2) * sizeof(float);
  if (need > BF_DECODE_STATIC_SCRATCH_BYTES) return BF_STATIC_ERR_TOO_LARGE;

  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= BF_STATIC_MAX_DEVICES) return BF_STATIC_ERR_DEVICE;
  if (!bf_decode_static_ptr[dev]) {
    // once per device, with that device current: the array's address on this device
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, bf_decode_static_scratch);
    if (e != cudaSuccess) return (int)e;
    bf_decode_static_ptr[dev] = p;
  }
  float* part_o = reinterpret_cast<float*>(bf_decode_static_ptr[dev]);
  float* part_ml = part_o + cells * d;      // behind the outputs' partials; 8-byte aligned
  return bf_decode_attention(q, k_cache, v_cache, rows, seq_of_token, positions, block_tables,
                             table_stride, out, part_o, part_ml, n_rows, nh, nkv, d, page_size,
                             num_pages, window, max_splits, scale, err, stream);
}

BF_TRACE_READER(bf_trace_read_attention_decode)
