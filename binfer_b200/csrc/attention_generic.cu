// Generic causal attention over the paged cache: any number of query tokens per
// request, any head count, group size, page size and head size up to 256.
//
// One warp per (query token, query head).  The query sits at absolute position p
// of its request; its keys are j in (p - window, p] (window 0: j in [0, p]), read
// through the request's block table.  Keys are walked in tiles of 32 whose edges
// are multiples of 32 counted from position 0, so the order of every sum depends
// only on p and the window, never on how the tokens were cut into steps or on
// what else is in the batch.
//
// This kernel is the whole 32-bit path's attention and the fallback for sizes
// that the tuned kernels refuse.  Formulas: scores (q . k) * scale, online
// softmax in float, probabilities kept in float for the product with v
// (cuda/kernels/bf16_kernels.cu:909-973; cuda/kernels/paged_attention.cu:408-487).
// The reference reads prefill keys from the fresh projection, not the cache
// (src/engine/batched_engine.ts:1082-1086); here every key comes from the pages.
//
// It is also where changes to the scores live, for attention that has them (the tuned
// kernels take none): a soft cap s <- c tanh(s / c), a bias per distance s <- s +
// slope_h (j - p), and a sink, a logit per head that joins the softmax's denominator and
// carries no value.  All three are off with softcap 0 and null pointers.
#include <float.h>

#include "common.cuh"

#define ATT_MAX_ACC 8   // head_dim <= 32 * ATT_MAX_ACC

template <typename A>
__global__ void paged_attention_generic_kernel(
    const A* __restrict__ q, const A* __restrict__ k_cache, const A* __restrict__ v_cache,
    const int* __restrict__ seq_of_token, const int* __restrict__ positions,
    const int* __restrict__ block_tables, int table_stride, A* __restrict__ out, int nh, int nkv,
    int d, int page_size, int num_pages, int window, float scale, float softcap,
    const float* __restrict__ slopes, const float* __restrict__ sinks, int* __restrict__ err) {
  extern __shared__ float sh[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const int t = blockIdx.x;
  const int h = blockIdx.y * warps + warp;
  if (h >= nh) return;
  const int g = h / (nh / nkv);
  float* qs = sh + (size_t)warp * d;
  const A* qrow = q + ((size_t)t * nh + h) * d;
  for (int i = lane; i < d; i += 32) qs[i] = bf_ld(qrow + i) * scale;
  __syncwarp();

  const int p = positions[t];
  const int* table = block_tables + (size_t)seq_of_token[t] * table_stride;
  const int j0 = window > 0 ? max(0, p - window + 1) : 0;

  float m = -FLT_MAX, l = 0.f;
  float acc[ATT_MAX_ACC];
#pragma unroll
  for (int c = 0; c < ATT_MAX_ACC; ++c) acc[c] = 0.f;

  for (int tile = j0 >> 5; tile <= (p >> 5); ++tile) {
    const int j = (tile << 5) + lane;
    bool valid = j >= j0 && j <= p;
    long long row = 0;     // element offset of this lane's key/value row
    if (valid) {
      const int lp = j / page_size;
      const int page = table[lp];
      if (page < 0 || page >= num_pages) {
        atomicOr(err, BF_ERR_PAGE);
        valid = false;
      } else {
        row = (((long long)page * nkv + g) * page_size + (j - lp * page_size)) * d;
      }
    }
    float s = -FLT_MAX;
    if (valid) {
      const A* kr = k_cache + row;
      float a = 0.f;
#pragma unroll 8
      for (int i = 0; i < d; ++i) a += qs[i] * bf_ld(kr + i);
      if (softcap > 0.f) a = softcap * tanhf(a / softcap);
      if (slopes) a += slopes[h] * (float)(j - p);
      s = a;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);
    const float pj = valid ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(pj);
    m = m_new;
#pragma unroll
    for (int c = 0; c < ATT_MAX_ACC; ++c) acc[c] *= corr;
    const unsigned live = __ballot_sync(0xffffffffu, valid);
    for (int jj = 0; jj < 32; ++jj) {
      if (!((live >> jj) & 1u)) continue;
      const float pb = __shfl_sync(0xffffffffu, pj, jj);
      const long long rb = __shfl_sync(0xffffffffu, row, jj);
      const A* vr = v_cache + rb;
#pragma unroll
      for (int c = 0; c < ATT_MAX_ACC; ++c) {
        const int i = lane + 32 * c;
        if (i < d) acc[c] += pb * bf_ld(vr + i);
      }
    }
  }
  if (sinks) {                                  // the sink: in the denominator only
    const float m_new = fmaxf(m, sinks[h]);
    const float corr = expf(m - m_new);
    l = l * corr + expf(sinks[h] - m_new);
#pragma unroll
    for (int c = 0; c < ATT_MAX_ACC; ++c) acc[c] *= corr;
  }
  const float inv = 1.f / l;
  A* o = out + ((size_t)t * nh + h) * d;
#pragma unroll
  for (int c = 0; c < ATT_MAX_ACC; ++c) {
    const int i = lane + 32 * c;
    if (i < d) bf_st(o + i, acc[c] * inv);
  }
}

BF_EXPORT int bf_paged_attention_generic(
    const void* q, const void* k_cache, const void* v_cache, const int* seq_of_token,
    const int* positions, const int* block_tables, int table_stride, void* out, int T, int nh,
    int nkv, int d, int page_size, int num_pages, int window, float scale, float softcap,
    const float* slopes, const float* sinks, int act_dtype, int* err, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (d > 32 * ATT_MAX_ACC || nkv <= 0 || nh % nkv) return (int)cudaErrorInvalidValue;
  const int warps = 4;
  dim3 grid(T, (nh + warps - 1) / warps);
  const size_t smem = (size_t)warps * d * sizeof(float);
  if (act_dtype == BF_DTYPE_F32)
    paged_attention_generic_kernel<float><<<grid, warps * 32, smem, stream>>>(
        (const float*)q, (const float*)k_cache, (const float*)v_cache, seq_of_token, positions,
        block_tables, table_stride, (float*)out, nh, nkv, d, page_size, num_pages, window, scale,
        softcap, slopes, sinks, err);
  else
    paged_attention_generic_kernel<__nv_bfloat16><<<grid, warps * 32, smem, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
        seq_of_token, positions, block_tables, table_stride, (__nv_bfloat16*)out, nh, nkv, d,
        page_size, num_pages, window, scale, softcap, slopes, sinks, err);
  return bf_launch_status();
}
