// After the fused q/k/v projection: per-head RMSNorm of q and k, the rotation,
// and the write of k and v into their cache pages, in one pass over the row.
//
// The reference runs these as separate kernels and launches: two RMSNorm calls
// with rows = tokens * heads (src/engine/batched_engine.ts:834-839), a rotary
// kernel per sequence (:861-876; cuda/kernels/bf16_kernels.cu:133-185), and a
// cache scatter per sequence (:933-961; cuda/kernels/paged_attention.cu:590-609).
//
// Rotation: rotate-half pairs (i, i + rot/2), angle = position * inv_freq[i]
// formed in float, sin/cos by the accurate sincosf.  v is written as projected.
//
// Cache layout per layer execution: [page][kv_head][slot_in_page][d].  A token's
// place is `slot = page * page_size + slot_in_page`, given per token; a negative
// slot means "do not write".
#include "common.cuh"

template <typename A>
__global__ void qk_norm_rope_kv_write_kernel(
    const A* __restrict__ qkv, long long row_stride, const float* __restrict__ q_w,
    const float* __restrict__ k_w, const float* __restrict__ inv_freq, int rot_half,
    const int* __restrict__ positions, const int* __restrict__ slots, A* __restrict__ q_out,
    A* __restrict__ k_cache, A* __restrict__ v_cache, int nh, int nkv, int d, int page_size,
    long long num_slots, float eps, int* __restrict__ err) {
  extern __shared__ float sh[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const int t = blockIdx.x;
  const int hh = blockIdx.y * warps + warp;
  const int total = nh + 2 * nkv;
  if (hh >= total) return;
  float* x = sh + (size_t)warp * d;
  const A* src = qkv + (size_t)t * row_stride + (size_t)hh * d;
  float ss = 0.f;
  for (int i = lane; i < d; i += 32) {
    const float v = bf_ld(src + i);
    x[i] = v;
    ss += v * v;
  }
  __syncwarp();
  const bool is_q = hh < nh;
  const bool is_k = !is_q && hh < nh + nkv;
  if (is_q || is_k) {
    const float* w = is_q ? q_w : k_w;
    if (w) {
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / (float)d + eps);
      for (int i = lane; i < d; i += 32) x[i] = x[i] * inv * w[i];
      __syncwarp();
    }
    if (rot_half > 0) {
      const float p = (float)positions[t];
      for (int i = lane; i < rot_half; i += 32) {
        float s, c;
        sincosf(p * inv_freq[i], &s, &c);
        const float a = x[i], b = x[i + rot_half];
        x[i] = a * c - b * s;
        x[i + rot_half] = a * s + b * c;
      }
      __syncwarp();
    }
  }
  if (is_q) {
    A* dst = q_out + ((size_t)t * nh + hh) * d;
    for (int i = lane; i < d; i += 32) bf_st(dst + i, x[i]);
    return;
  }
  if (!k_cache) return;
  const int slot = slots[t];
  if (slot < 0) return;
  if ((long long)slot >= num_slots) {
    if (lane == 0) atomicOr(err, BF_ERR_SLOT);
    return;
  }
  const int h = is_k ? hh - nh : hh - nh - nkv;
  const int page = slot / page_size, off = slot - page * page_size;
  A* dst = (is_k ? k_cache : v_cache) + (((size_t)page * nkv + h) * page_size + off) * d;
  for (int i = lane; i < d; i += 32) bf_st(dst + i, x[i]);
}

BF_EXPORT int bf_qk_norm_rope_kv_write(
    const void* qkv, long long row_stride, const float* q_w, const float* k_w,
    const float* inv_freq, int rot_half, const int* positions, const int* slots, void* q_out,
    void* k_cache, void* v_cache, int T, int nh, int nkv, int d, int page_size,
    long long num_slots, float eps, int act_dtype, int* err, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (2 * rot_half > d) return (int)cudaErrorInvalidValue;
  const int warps = 4;
  const int total = nh + 2 * nkv;
  dim3 grid(T, (total + warps - 1) / warps);
  const size_t smem = (size_t)warps * d * sizeof(float);
  if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
  if (act_dtype == BF_DTYPE_F32)
    qk_norm_rope_kv_write_kernel<float><<<grid, warps * 32, smem, stream>>>(
        (const float*)qkv, row_stride, q_w, k_w, inv_freq, rot_half, positions, slots,
        (float*)q_out, (float*)k_cache, (float*)v_cache, nh, nkv, d, page_size, num_slots, eps,
        err);
  else
    qk_norm_rope_kv_write_kernel<__nv_bfloat16><<<grid, warps * 32, smem, stream>>>(
        (const __nv_bfloat16*)qkv, row_stride, q_w, k_w, inv_freq, rot_half, positions, slots,
        (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, nh, nkv, d,
        page_size, num_slots, eps, err);
  return bf_launch_status();
}
