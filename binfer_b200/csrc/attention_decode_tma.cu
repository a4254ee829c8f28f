// Split-KV decode attention, second generation: K and V tiles come in by TMA.
//
// Same work split as attention_decode.cu (grid (128-key split, kv head, row), the group's
// query heads as the rows of the tensor-core tile, partials to scratch, merge kernel), but
// each (page, kv head) block of the cache, which is contiguous in memory, is fetched with
// one cp.async.bulk.tensor copy per 64 columns into a 128-byte-swizzled shared-memory tile,
// completion on an mbarrier.  A tile of 128 keys is 16 to 64 such copies instead of 8192
// 16-byte cp.async requests, which is what kept the first kernel at under half of the
// memory bandwidth.  ldmatrix reads the swizzled tile without bank conflicts, so the tile
// needs no padding.
//
// Takes head sizes 64, 128, 256 and page sizes that divide 128 and are at least 8; the
// caller uses the first kernel for everything else.
//
// Pages that lie wholly outside a row's keys are not fetched; their V rows are zeroed so
// that a zero probability times stale shared memory cannot give a NaN.
//
// The waits on the copies are bounded (about a second): on a timeout the CTA sets
// BF_ERR_WAIT and returns without storing.  No copy uses multicast.
#include <float.h>

#include "common.cuh"
#include "mma_utils.cuh"
#include "tma_utils.cuh"

#define DT_SPLIT 128
#define DT_THREADS 128

extern "C" int bf_decode_attention_merge(const float* part_o, const float* part_ml,
                                         const int* rows, const int* positions, void* out,
                                         int n_rows, int nh, int d, int window, int max_splits,
                                         cudaStream_t stream);

// element offset of 16-byte chunk `c` of row `r` inside a swizzled [128][64] bf16 half tile
__device__ __forceinline__ int sw_off(int r, int c) { return r * 64 + ((c ^ (r & 7)) << 3); }

template <int D>
__global__ void __launch_bounds__(DT_THREADS)
decode_attention_tma_kernel(const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v,
                            const __nv_bfloat16* __restrict__ q, const int* __restrict__ rows,
                            const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                            const int* __restrict__ block_tables, int table_stride,
                            float* __restrict__ part_o, float* __restrict__ part_ml, int nh, int nkv,
                            int page_size, int num_pages, int window, int max_splits,
                            float scale_log2, int* __restrict__ err) {
  constexpr int HALVES = D / 64;
  constexpr int HALF_ELEMS = DT_SPLIT * 64;             // 16 KB per half tile
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned char* base = smem_raw + ((1024u - (bf_smem_u32(smem_raw) & 1023u)) & 1023u);
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(base);
  __nv_bfloat16* Vs = Ks + HALVES * HALF_ELEMS;
  uint64_t* bars = reinterpret_cast<uint64_t*>(Vs + HALVES * HALF_ELEMS);   // [2]: K, V
  float* red_far = reinterpret_cast<float*>(bars + 2);                      // merge buffer if G > 16

  bf_pdl_trigger();
  bf_pdl_wait();
  const int split = blockIdx.x, g = blockIdx.y, r = blockIdx.z;
  const int t = rows ? rows[r] : r;
  const int p = positions[t];
  const int j0 = window > 0 ? max(0, p - window + 1) : 0;
  const int k_begin = split * DT_SPLIT;
  // the grid has max_splits splits: keys beyond them have nowhere to put their partial
  if (split == 0 && g == 0 && threadIdx.x == 0 && p / DT_SPLIT >= max_splits)
    atomicOr(err, BF_ERR_SPLITS);
  if (k_begin > p || k_begin + DT_SPLIT <= j0) return;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = nh / nkv;
  const int pages = DT_SPLIT / page_size;

  if (tid == 0) {
    bf_mbar_init(bars, 1);
    bf_mbar_init(bars + 1, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == 0) {
    // one lane per page of the tile: look the page up, then fetch its K and V blocks
    const int jp = k_begin + lane * page_size;
    const bool wanted = lane < pages && jp <= p && jp + page_size > j0;
    int page = 0;
    if (wanted) {
      page = block_tables[(size_t)seq_of_token[t] * table_stride + jp / page_size];
      if (page < 0 || page >= num_pages) {
        atomicOr(err, BF_ERR_PAGE);
        page = 0;                                        // the scratch page: valid memory
      }
    }
    const unsigned live = __ballot_sync(0xffffffffu, wanted);
    if (lane == 0) {
      const uint32_t bytes = (uint32_t)__popc(live) * page_size * D * 2;
      bf_mbar_expect_tx(bars, bytes);
      bf_mbar_expect_tx(bars + 1, bytes);
    }
    __syncwarp();
    if (wanted) {
      const int y = (page * nkv + g) * page_size;
#pragma unroll
      for (int hh = 0; hh < HALVES; ++hh)
        bf_tma_load_2d(Ks + hh * HALF_ELEMS + lane * page_size * 64, &map_k, bars, hh * 64, y);
#pragma unroll
      for (int hh = 0; hh < HALVES; ++hh)
        bf_tma_load_2d(Vs + hh * HALF_ELEMS + lane * page_size * 64, &map_v, bars + 1, hh * 64, y);
    }
  }
  // V rows of pages that are not fetched must read as zero
  for (int pg = 0; pg < pages; ++pg) {
    const int jp = k_begin + pg * page_size;
    if (jp <= p && jp + page_size > j0) continue;
    for (int c = tid; c < page_size * 8 * HALVES; c += DT_THREADS) {
      const int hh = c / (page_size * 8), rem = c - hh * page_size * 8;
      *reinterpret_cast<uint4*>(Vs + hh * HALF_ELEMS + (pg * page_size) * 64 + rem * 8) =
          make_uint4(0u, 0u, 0u, 0u);
    }
  }

  const int r0 = lane >> 2, cq = (lane & 3) * 2;
  const int wkey = warp * 32;
  bool first_block = true;

  for (int hb = 0; hb < G; hb += 16) {
    const int gblk = min(16, G - hb);
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
      const bool ok = bf_mbar_wait_bounded(bars, 0);
      if (!__syncthreads_and(ok)) {                      // uniform: every thread leaves or none
        if (tid == 0) atomicOr(err, BF_ERR_WAIT);
        return;
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
        const int c = ks * 2 + (lane >> 3);              // 16-byte chunk along the head
        ldmatrix_x4(b, Ks + (c >> 3) * HALF_ELEMS + sw_off(krow, c & 7));
        mma_bf16_16816(s[nt], qa[ks], b[0], b[1]);
        mma_bf16_16816(s[nt], qa[ks + 1], b[2], b[3]);
      }
    }
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
      const bool ok = bf_mbar_wait_bounded(bars + 1, 0);
      if (!__syncthreads_and(ok)) {
        if (tid == 0) atomicOr(err, BF_ERR_WAIT);
        return;
      }
      first_block = false;
    }
    float o[D / 8][4];
#pragma unroll
    for (int dn = 0; dn < D / 8; ++dn)
#pragma unroll
      for (int i = 0; i < 4; ++i) o[dn][i] = 0.f;
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
      const int m = lane >> 3;
      const int vrow = wkey + kk * 16 + (m & 1) * 8 + (lane & 7);
#pragma unroll
      for (int dn = 0; dn < D / 8; dn += 2) {
        unsigned b[4];
        const int c = dn + (m >> 1);
        ldmatrix_x4_trans(b, Vs + (c >> 3) * HALF_ELEMS + sw_off(vrow, c & 7));
        mma_bf16_16816(o[dn], pa[kk], b[0], b[1]);
        mma_bf16_16816(o[dn + 1], pa[kk], b[2], b[3]);
      }
    }

    // merge the four warps' partials; over the dead K tile when there is one head block
    float* red = G <= 16 ? reinterpret_cast<float*>(Ks) : red_far;
    float* red_m = red;
    float* red_l = red + 64;
    float* red_o = red + 128;
    if ((lane & 3) == 0) {
      red_m[warp * 16 + r0] = m0;
      red_m[warp * 16 + r0 + 8] = m1;
      red_l[warp * 16 + r0] = l0;
      red_l[warp * 16 + r0 + 8] = l1;
    }
    // only the rows of real heads are parked (rows r0 >= gblk are padding)
#pragma unroll
    for (int dn = 0; dn < D / 8; ++dn) {
      float* o0 = red_o + ((size_t)warp * 16 + r0) * D + dn * 8 + cq;
      if (r0 < gblk) {
        o0[0] = o[dn][0];
        o0[1] = o[dn][1];
      }
      if (r0 + 8 < gblk) {
        o0[(size_t)8 * D] = o[dn][2];
        o0[(size_t)8 * D + 1] = o[dn][3];
      }
    }
    __syncthreads();
    for (int idx = tid; idx < gblk * D; idx += DT_THREADS) {
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
      const size_t pb = ((size_t)r * nh + (size_t)g * G + hb + row) * max_splits + split;
      part_o[pb * D + col] = O;
      if (col == 0) {
        part_ml[pb * 2] = M;
        part_ml[pb * 2 + 1] = L;
      }
    }
    __syncthreads();
  }
}

template <int D>
static int launch_tma(const void* q, const void* k_cache, const void* v_cache, const int* rows,
                      const int* seq_of_token, const int* positions, const int* block_tables,
                      int table_stride, float* part_o, float* part_ml, int n_rows, int nh, int nkv,
                      int page_size, int num_pages, int window, int max_splits, float scale,
                      int* err, cudaStream_t stream) {
  CUtensorMap mk, mv;
  const long long cache_rows = (long long)num_pages * nkv * page_size;
  int e = bf_make_tensor_map_bf16_2d(&mk, k_cache, cache_rows, D, D, page_size, 64);
  if (e) return e;
  e = bf_make_tensor_map_bf16_2d(&mv, v_cache, cache_rows, D, D, page_size, 64);
  if (e) return e;
  const size_t tiles = (size_t)2 * DT_SPLIT * D * 2;
  const size_t merge = (size_t)(128 + 4 * 16 * D) * 4;
  const size_t smem_max = 1024 + tiles + 16 + merge;
  const size_t smem = nh / nkv <= 16 ? 1024 + tiles + 16 : smem_max;
  auto kern = decode_attention_tma_kernel<D>;
  static bool configured_on[BF_MAX_DEVICES];
  bool& configured = configured_on[bf_current_device()];
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)smem_max);
    if (ce != cudaSuccess) return (int)ce;
    configured = true;
  }
  dim3 grid(max_splits, nkv, n_rows);
  return bf_launch_pdl(kern, grid, dim3(DT_THREADS), smem, stream, mk, mv,
                       (const __nv_bfloat16*)q, rows, seq_of_token, positions, block_tables,
                       table_stride, part_o, part_ml, nh, nkv, page_size, num_pages, window,
                       max_splits, scale * 1.4426950408889634f, err);
}

// Same arguments and result as bf_decode_attention.  Returns cudaErrorInvalidValue for head
// sizes and page sizes it does not take.
BF_EXPORT int bf_decode_attention_tma(const void* q, const void* k_cache, const void* v_cache,
                                      const int* rows, const int* seq_of_token,
                                      const int* positions, const int* block_tables,
                                      int table_stride, void* out, float* part_o, float* part_ml,
                                      int n_rows, int nh, int nkv, int d, int page_size,
                                      int num_pages, int window, int max_splits, float scale,
                                      int* err, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (nkv <= 0 || nh % nkv || page_size < 8 || page_size > 128 || DT_SPLIT % page_size ||
      ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15))
    return (int)cudaErrorInvalidValue;
  int e;
  switch (d) {
    case 64:
      e = launch_tma<64>(q, k_cache, v_cache, rows, seq_of_token, positions, block_tables,
                         table_stride, part_o, part_ml, n_rows, nh, nkv, page_size, num_pages,
                         window, max_splits, scale, err, stream);
      break;
    case 128:
      e = launch_tma<128>(q, k_cache, v_cache, rows, seq_of_token, positions, block_tables,
                          table_stride, part_o, part_ml, n_rows, nh, nkv, page_size, num_pages,
                          window, max_splits, scale, err, stream);
      break;
    case 256:
      e = launch_tma<256>(q, k_cache, v_cache, rows, seq_of_token, positions, block_tables,
                          table_stride, part_o, part_ml, n_rows, nh, nkv, page_size, num_pages,
                          window, max_splits, scale, err, stream);
      break;
    default:
      return (int)cudaErrorInvalidValue;
  }
  if (e) return e;
  return bf_decode_attention_merge(part_o, part_ml, rows, positions, out, n_rows, nh, d, window,
                                   max_splits, stream);
}
