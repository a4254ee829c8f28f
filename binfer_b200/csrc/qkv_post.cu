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
    long long num_slots, float eps, BfRowScale rs, int* __restrict__ err) {
  extern __shared__ float sh[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const int t = blockIdx.x;
  const int hh = blockIdx.y * warps + warp;
  const int total = nh + 2 * nkv;
  if (hh >= total) return;
  float* x = sh + (size_t)warp * d;
  const A* src = qkv + (size_t)t * row_stride + (size_t)hh * d;
  const float row_factor = bf_row_factor(rs, t, lane);
  float ss = 0.f;
  for (int i = lane; i < d; i += 32) {
    const float v = bf_ld(src + i) * row_factor;
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

// The common case in registers: bf16, head size 128, full rotation (64 pairs).  A block takes
// some of a token's heads (blockIdx.y; all of them when there are many tokens): the 64 sines
// and cosines of the token's position are computed once per block and shared by its heads;
// each warp then walks its heads, lane l holding elements 4l..4l+3, whose rotation partners
// sit in lane l ^ 16.  With few tokens every warp has one head: the kernel is then two
// dependent round trips long (position, then the head's values) instead of one per head.
__global__ void qk_norm_rope_kv_write_d128_kernel(
    const __nv_bfloat16* __restrict__ qkv, long long row_stride, const float* __restrict__ q_w,
    const float* __restrict__ k_w, const float* __restrict__ inv_freq,
    const int* __restrict__ positions, const int* __restrict__ slots,
    __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_cache,
    __nv_bfloat16* __restrict__ v_cache, int nh, int nkv, int page_size, long long num_slots,
    float eps, BfRowScale rs, int* __restrict__ err) {
  constexpr int D = 128;
  __shared__ float sn_s[64], cs_s[64];
  BF_TRACE_POINT(10 * BF_TR_QKNORM);
  bf_pdl_trigger();
  bf_pdl_wait();
  BF_TRACE_POINT(10 * BF_TR_QKNORM + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int t = blockIdx.x;
  const BfRowShare share = bf_row_fetch(rs, t, lane);    // in flight under the sines and cosines
  const int slot = k_cache ? slots[t] : -1;
  // so are the values of the warp's first head
  const int hh_first = blockIdx.y * warps + warp;
  uint2 raw_first = make_uint2(0u, 0u);
  if (hh_first < nh + 2 * nkv)
    raw_first = *reinterpret_cast<const uint2*>(qkv + (size_t)t * row_stride +
                                                (size_t)hh_first * D + lane * 4);
  if (threadIdx.x < 64) {
    float sn, cs;
    sincosf((float)positions[t] * inv_freq[threadIdx.x], &sn, &cs);
    sn_s[threadIdx.x] = sn;
    cs_s[threadIdx.x] = cs;
  }
  __syncthreads();
  const float row_factor = bf_row_finish(rs, share);
  const bool upper = lane >= 16;               // holds elements i + 64 of the pairs
  const int fi = (lane & 15) * 4;
  const float4 wq = q_w ? *reinterpret_cast<const float4*>(q_w + lane * 4) : make_float4(1, 1, 1, 1);
  const float4 wk = k_w ? *reinterpret_cast<const float4*>(k_w + lane * 4) : make_float4(1, 1, 1, 1);
  // what does not depend on the head stays in registers: the lane's sines and cosines, and
  // where the token's keys and values go
  float sn4[4], cs4[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    sn4[j] = sn_s[fi + j];
    cs4[j] = cs_s[fi + j];
  }
  const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot - page * page_size : 0;
  const size_t kv_base = ((size_t)page * nkv * page_size + off) * D + lane * 4;
  const size_t kv_head = (size_t)page_size * D;
  // A warp's heads are asked for six at a time, before the first of them is used: with one
  // load in flight per warp a block of 2048 tokens' worth moved 2 TB/s (25 us a layer).
  constexpr int AHEAD = 6;
  const int stride = gridDim.y * warps;
  uint2 ahead[AHEAD];
  for (int hh0 = hh_first; hh0 < nh + 2 * nkv; hh0 += AHEAD * stride) {
#pragma unroll
    for (int a = 0; a < AHEAD; ++a) {
      const int hh = hh0 + a * stride;
      ahead[a] = make_uint2(0u, 0u);
      if (hh == hh_first)
        ahead[a] = raw_first;
      else if (hh < nh + 2 * nkv && (hh < nh || slot >= 0))
        ahead[a] = *reinterpret_cast<const uint2*>(qkv + (size_t)t * row_stride +
                                                   (size_t)hh * D + lane * 4);
    }
#pragma unroll
    for (int n = 0; n < AHEAD; ++n) {
    const int hh = hh0 + n * stride;
    if (hh >= nh + 2 * nkv) break;
    const bool is_q = hh < nh, is_k = !is_q && hh < nh + nkv;
    if (!is_q && slot < 0) continue;
    const uint2 raw = ahead[n];
    const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 a = __bfloat1622float2(r2[0]), b = __bfloat1622float2(r2[1]);
    float x[4] = {a.x * row_factor, a.y * row_factor, b.x * row_factor, b.y * row_factor};
    if (is_q || is_k) {
      if (is_q ? q_w != nullptr : k_w != nullptr) {
        const float ss = warp_sum(x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3]);
        const float inv = rsqrtf(ss / (float)D + eps);
        const float4 w4 = is_q ? wq : wk;
        x[0] *= inv * w4.x;
        x[1] *= inv * w4.y;
        x[2] *= inv * w4.z;
        x[3] *= inv * w4.w;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float other = __shfl_xor_sync(0xffffffffu, x[j], 16);
        // lower half: x[i] cos - x[i+64] sin;  upper half: x[i] sin + x[i+64] cos
        x[j] = upper ? other * sn4[j] + x[j] * cs4[j] : x[j] * cs4[j] - other * sn4[j];
      }
    }
    uint2 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
    o2[0] = __floats2bfloat162_rn(x[0], x[1]);
    o2[1] = __floats2bfloat162_rn(x[2], x[3]);
    if (is_q) {
      *reinterpret_cast<uint2*>(q_out + ((size_t)t * nh + hh) * D + lane * 4) = o;
      continue;
    }
    if ((long long)slot >= num_slots) {
      if (lane == 0) atomicOr(err, BF_ERR_SLOT);
      continue;
    }
    const int h = is_k ? hh - nh : hh - nh - nkv;
    *reinterpret_cast<uint2*>((is_k ? k_cache : v_cache) + kv_base + (size_t)h * kv_head) = o;
    }
  }
}

BF_EXPORT int bf_qk_norm_rope_kv_write(
    const void* qkv, long long row_stride, const float* q_w, const float* k_w,
    const float* inv_freq, int rot_half, const int* positions, const int* slots, void* q_out,
    void* k_cache, void* v_cache, int T, int nh, int nkv, int d, int page_size,
    long long num_slots, float eps, int act_dtype, const float* row_partials, int row_count,
    int row_width, float row_eps, int* err, cudaStream_t stream) {
  if (T <= 0) return 0;
  // the rows of qkv may still lack a factor (see BfRowScale); it is applied as they are read
  const BfRowScale rs = {row_partials, row_count, row_width > 0 ? 1.f / (float)row_width : 0.f,
                         row_eps};
  if (2 * rot_half > d) return (int)cudaErrorInvalidValue;
  const int warps = 4;
  const int total = nh + 2 * nkv;
  dim3 grid(T, (total + warps - 1) / warps);
  if (act_dtype == BF_DTYPE_BF16 && d == 128 && rot_half == 64 && row_stride % 4 == 0 &&
      ((uintptr_t)qkv & 7) == 0 && ((uintptr_t)q_out & 7) == 0 && ((uintptr_t)k_cache & 7) == 0 &&
      ((uintptr_t)v_cache & 7) == 0 && ((uintptr_t)inv_freq & 15) == 0 &&
      ((uintptr_t)q_w & 15) == 0 && ((uintptr_t)k_w & 15) == 0) {
    const int block = total >= 16 ? 256 : 128;
    // few tokens: a warp per head; many: a block per token, which walks the heads (at 2048
    // tokens a warp per head measured a third slower: the sines are then computed six times).
    // At 2048 tokens the kernel is bound by issue, not memory (ncu: 13.1 M warp instructions,
    // issue slots 67 % busy, 18.5 us for 50 MB); most of them are a block's preamble, not the
    // heads' arithmetic: a variant with eight elements a lane and two heads a warp executed
    // 10.4 M and, with fewer warps resident, took 21.6 us.
    const int parts = T <= 64 ? (total * 32 + block - 1) / block : 1;
    return bf_launch_pdl(qk_norm_rope_kv_write_d128_kernel, dim3(T, parts), dim3(block), 0,
                         stream, (const __nv_bfloat16*)qkv,
                         row_stride, q_w, k_w, inv_freq, positions, slots, (__nv_bfloat16*)q_out,
                         (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, nh, nkv, page_size,
                         num_slots, eps, rs, err);
  }
  const size_t smem = (size_t)warps * d * sizeof(float);
  if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
  if (act_dtype == BF_DTYPE_F32)
    qk_norm_rope_kv_write_kernel<float><<<grid, warps * 32, smem, stream>>>(
        (const float*)qkv, row_stride, q_w, k_w, inv_freq, rot_half, positions, slots,
        (float*)q_out, (float*)k_cache, (float*)v_cache, nh, nkv, d, page_size, num_slots, eps,
        rs, err);
  else
    qk_norm_rope_kv_write_kernel<__nv_bfloat16><<<grid, warps * 32, smem, stream>>>(
        (const __nv_bfloat16*)qkv, row_stride, q_w, k_w, inv_freq, rot_half, positions, slots,
        (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, nh, nkv, d,
        page_size, num_slots, eps, rs, err);
  return bf_launch_status();
}

BF_TRACE_READER(bf_trace_read_qkv_post)
