// Embedding gather, fused residual-add + RMSNorm, SiLU-mul, residual add.
//
// The residual stream is float in both engine precisions: the sum over layers
// is formed in 32-bit, and only what feeds a matrix product is rounded to the
// activation type.  The reference rounds the stream to bf16 after every add
// (cuda/kernels/bf16_kernels.cu:504-517) and runs norm and add as separate
// kernels (src/engine/batched_engine.ts:1164-1178).
#include <stdlib.h>

#include "common.cuh"

static int g_pdl = -1;
int bf_pdl_enabled() {
  if (g_pdl < 0) {
    const char* e = getenv("BINFER_B200_PDL");
    g_pdl = (e && e[0] == '0') ? 0 : 1;
  }
  return g_pdl;
}
// 1: launch the decode step's short kernels with programmatic dependent launch (default);
// 0: ordinary launches.  The environment variable BINFER_B200_PDL=0 does the same.
BF_EXPORT void bf_set_pdl(int on) { g_pdl = on ? 1 : 0; }

// ------------------------------------------------------------------ embedding
// out[t, :] = table[ids[t], :] * scale   (cuda/kernels/bf16_kernels.cu:711-729,
// which does not check the id; here a bad id sets an error bit and yields zeros).
template <typename W>
__global__ void embed_gather_kernel(const W* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ out, int H, int vocab, float scale,
                                    int* __restrict__ err) {
  bf_pdl_trigger();
  bf_pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  float* o = out + (size_t)t * H;
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(err, BF_ERR_TOKEN_ID);
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = 0.f;
    return;
  }
  const W* row = table + (size_t)id * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = bf_ld(row + i) * scale;
}

BF_EXPORT int bf_embed_gather(const void* table, int table_dtype, const int* ids, float* out,
                              int T, int H, int vocab, float scale, int* err,
                              cudaStream_t stream) {
  if (T <= 0) return 0;
  const int threads = H >= 1024 ? 256 : 128;
  if (table_dtype == BF_DTYPE_F32)
    return bf_launch_pdl(embed_gather_kernel<float>, dim3(T), dim3(threads), 0, stream,
                         (const float*)table, ids, out, H, vocab, scale, err);
  return bf_launch_pdl(embed_gather_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream,
                       (const __nv_bfloat16*)table, ids, out, H, vocab, scale, err);
}

// -------------------------------------------------------- add + RMSNorm (fused)
// For output row i (source row r = rows ? rows[i] : i):
//   x = resid[r] + (delta ? delta[r] : 0);  if (write_back) resid[r] = x;
//   out[i] = x * rsqrt(mean(x^2) + eps) * w           (bf16_kernels.cu:40-84)
// One block per row; the row is kept in shared memory between the two passes.
template <typename A>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const A* __restrict__ delta,
                                   const float* __restrict__ w, A* __restrict__ out,
                                   const int* __restrict__ rows, int H, float eps,
                                   int write_back) {
  extern __shared__ float sh[];
  float* row = sh;            // H floats
  float* scratch = sh + H;    // 33 floats
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* x = resid + (size_t)r * H;
  const A* d = delta ? delta + (size_t)r * H : nullptr;
  float ss = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float v = x[c];
    if (d) v += bf_ld(d + c);
    row[c] = v;
    if (write_back && d) x[c] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)H + eps);
  A* o = out + (size_t)i * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x) bf_st(o + c, row[c] * inv * w[c]);
}

// The same for bf16 activations and H a multiple of 8: 8 elements per thread per trip, all
// loads of a trip issued before they are used, the row kept in registers between the passes.
template <int TRIPS>
__global__ void add_rmsnorm_bf16_vec_kernel(float* __restrict__ resid,
                                            const __nv_bfloat16* __restrict__ delta,
                                            const float* __restrict__ w,
                                            __nv_bfloat16* __restrict__ out,
                                            const int* __restrict__ rows, int H, float eps,
                                            int write_back) {
  __shared__ float scratch[33];
  BF_TRACE_POINT(10 * BF_TR_RMSNORM);
  bf_pdl_trigger();
  bf_pdl_wait();
  BF_TRACE_POINT(10 * BF_TR_RMSNORM + 1);
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* x = resid + (size_t)r * H;
  const __nv_bfloat16* d = delta ? delta + (size_t)r * H : nullptr;
  float v[TRIPS][8];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < TRIPS; ++k) {
    const int c = (k * blockDim.x + threadIdx.x) * 8;
    if (c < H) {
      const float4 a = *reinterpret_cast<const float4*>(x + c);
      const float4 b = *reinterpret_cast<const float4*>(x + c + 4);
      v[k][0] = a.x; v[k][1] = a.y; v[k][2] = a.z; v[k][3] = a.w;
      v[k][4] = b.x; v[k][5] = b.y; v[k][6] = b.z; v[k][7] = b.w;
      if (d) {
        const uint4 q = *reinterpret_cast<const uint4*>(d + c);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h[j]);
          v[k][2 * j] += f.x;
          v[k][2 * j + 1] += f.y;
        }
        if (write_back) {
          *reinterpret_cast<float4*>(x + c) = make_float4(v[k][0], v[k][1], v[k][2], v[k][3]);
          *reinterpret_cast<float4*>(x + c + 4) = make_float4(v[k][4], v[k][5], v[k][6], v[k][7]);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[k][j] * v[k][j];
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)H + eps);
  __nv_bfloat16* o = out + (size_t)i * H;
#pragma unroll
  for (int k = 0; k < TRIPS; ++k) {
    const int c = (k * blockDim.x + threadIdx.x) * 8;
    if (c < H) {
      const float4 wa = *reinterpret_cast<const float4*>(w + c);
      const float4 wb = *reinterpret_cast<const float4*>(w + c + 4);
      uint4 q;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
      h[0] = __floats2bfloat162_rn(v[k][0] * inv * wa.x, v[k][1] * inv * wa.y);
      h[1] = __floats2bfloat162_rn(v[k][2] * inv * wa.z, v[k][3] * inv * wa.w);
      h[2] = __floats2bfloat162_rn(v[k][4] * inv * wb.x, v[k][5] * inv * wb.y);
      h[3] = __floats2bfloat162_rn(v[k][6] * inv * wb.z, v[k][7] * inv * wb.w);
      *reinterpret_cast<uint4*>(o + c) = q;
    }
  }
}

BF_EXPORT int bf_add_rmsnorm(float* resid, const void* delta, const float* w, void* out,
                             const int* rows, int n_rows, int H, float eps, int act_dtype,
                             int write_back, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (act_dtype == BF_DTYPE_BF16 && H % 8 == 0 && H <= 8 * 256 * 4 &&
      ((uintptr_t)resid & 15) == 0 && ((uintptr_t)delta & 15) == 0 &&
      ((uintptr_t)w & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    const int threads = H >= 2048 ? 256 : 128;
    const int trips = (H / 8 + threads - 1) / threads;
    auto go = [&](auto kern) {
      return bf_launch_pdl(kern, dim3(n_rows), dim3(threads), 0, stream, resid,
                           (const __nv_bfloat16*)delta, w, (__nv_bfloat16*)out, rows, H, eps,
                           write_back);
    };
    if (trips <= 1) return go(add_rmsnorm_bf16_vec_kernel<1>);
    if (trips == 2) return go(add_rmsnorm_bf16_vec_kernel<2>);
    return go(add_rmsnorm_bf16_vec_kernel<4>);
  }
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  const size_t smem = (size_t)(H + 33) * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (act_dtype == BF_DTYPE_F32) {
    auto k = add_rmsnorm_kernel<float>;
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    k<<<n_rows, threads, smem, stream>>>(resid, (const float*)delta, w, (float*)out, rows, H,
                                         eps, write_back);
  } else {
    auto k = add_rmsnorm_kernel<__nv_bfloat16>;
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    k<<<n_rows, threads, smem, stream>>>(resid, (const __nv_bfloat16*)delta, w,
                                         (__nv_bfloat16*)out, rows, H, eps, write_back);
  }
  return bf_launch_status();
}

// --------------------------------------------------------------- residual add
// resid[t, :] += delta[t, :]   (used when an add cannot ride on a following norm)
template <typename A>
__global__ void residual_add_kernel(float* __restrict__ resid, const A* __restrict__ delta,
                                    size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += step) resid[i] += bf_ld(delta + i);
}

BF_EXPORT int bf_residual_add(float* resid, const void* delta, long long n, int act_dtype,
                              cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = 256;
  long long blocks = (n + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (act_dtype == BF_DTYPE_F32)
    residual_add_kernel<float><<<(int)blocks, threads, 0, stream>>>(resid, (const float*)delta,
                                                                    (size_t)n);
  else
    residual_add_kernel<__nv_bfloat16><<<(int)blocks, threads, 0, stream>>>(
        resid, (const __nv_bfloat16*)delta, (size_t)n);
  return bf_launch_status();
}

// ------------------------------------------------------------------- SiLU-mul
// out[t, c] = silu(gu[t, c]) * gu[t, I + c],  silu(g) = g / (1 + exp(-g))
// (cuda/kernels/bf16_kernels.cu:461-477; there gate and up are separate buffers,
// here they are the two halves of one fused projection's output row).
template <typename A>
__global__ void silu_mul_kernel(const A* __restrict__ gu, A* __restrict__ out, int T, int I) {
  const size_t n = (size_t)T * I;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += step) {
    const size_t t = i / I, c = i - t * I;
    const float g = bf_ld(gu + t * 2 * I + c);
    const float u = bf_ld(gu + t * 2 * I + I + c);
    bf_st(out + i, g / (1.f + expf(-g)) * u);
  }
}

// silu for the bf16 kernels: float arithmetic with the hardware's exp2 and reciprocal
// approximations (relative error about 2^-21, far inside the bf16 result's 2^-9).  With the
// accurate expf and division the bf16 kernel was bound by arithmetic, not by memory.
__device__ __forceinline__ float bf_silu_fast(float g) { return __fdividef(g, 1.f + __expf(-g)); }

// The same when the rows of gu still lack a factor (see BfRowScale).  I is at least 256, so
// the 32 chunks of a warp lie in at most two rows, whose factors the warp works out itself,
// its loads of the partial sums in flight together with its loads of gate and up.
__global__ void silu_mul_bf16_scaled_kernel(const __nv_bfloat16* __restrict__ gu,
                                            __nv_bfloat16* __restrict__ out, int T, int I,
                                            BfRowScale rs) {
  BF_TRACE_POINT(10 * BF_TR_SILU);
  bf_pdl_trigger();
  bf_pdl_wait();
  BF_TRACE_POINT(10 * BF_TR_SILU + 1);
  const int lane = threadIdx.x & 31;
  const int per_row = I / 8;
  const size_t n = (size_t)T * per_row;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  // whole warps stay in the loop together: the factor is a warp's work
  for (size_t i0 = (size_t)blockIdx.x * blockDim.x + (threadIdx.x & ~31); i0 < n; i0 += step) {
    const size_t i = i0 + lane;
    const bool on = i < n;
    const size_t t = on ? i / per_row : 0, c = on ? (i - t * per_row) * 8 : 0;
    uint4 g4 = make_uint4(0, 0, 0, 0), u4 = g4;
    if (on) {
      g4 = *reinterpret_cast<const uint4*>(gu + t * 2 * I + c);
      u4 = *reinterpret_cast<const uint4*>(gu + t * 2 * I + I + c);
    }
    const int t_lo = (int)(i0 / per_row);
    const size_t i_hi = i0 + 31 < n ? i0 + 31 : n - 1;
    const int t_hi = (int)(i_hi / per_row);
    const BfRowShare s_lo = bf_row_fetch(rs, t_lo, lane);
    float f = bf_row_finish(rs, s_lo);
    if (t_hi != t_lo) {                                  // uniform over the warp
      const float f_hi = bf_row_factor(rs, t_hi, lane);
      if ((int)t == t_hi) f = f_hi;
    }
    if (!on) continue;
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
      g.x *= f; g.y *= f; u.x *= f; u.y *= f;
      o2[j] = __floats2bfloat162_rn(bf_silu_fast(g.x) * u.x, bf_silu_fast(g.y) * u.y);
    }
    *reinterpret_cast<uint4*>(out + t * I + c) = o4;
  }
}

// bf16, I a multiple of 8: eight elements per thread with 16-byte loads and stores.
__global__ void silu_mul_bf16_vec_kernel(const __nv_bfloat16* __restrict__ gu,
                                         __nv_bfloat16* __restrict__ out, int T, int I) {
  BF_TRACE_POINT(10 * BF_TR_SILU);
  bf_pdl_trigger();
  bf_pdl_wait();
  BF_TRACE_POINT(10 * BF_TR_SILU + 1);
  const int per_row = I / 8;
  const size_t n = (size_t)T * per_row;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  // two chunks a trip, all four loads asked for before the first is used
  for (; i < n; i += 2 * step) {
    const size_t i2 = i + step;
    const bool two = i2 < n;
    const size_t t = i / per_row, c = (i - t * per_row) * 8;
    const size_t t2 = two ? i2 / per_row : t, c2 = two ? (i2 - t2 * per_row) * 8 : c;
    uint4 g4[2], u4[2];
    g4[0] = *reinterpret_cast<const uint4*>(gu + t * 2 * I + c);
    u4[0] = *reinterpret_cast<const uint4*>(gu + t * 2 * I + I + c);
    g4[1] = *reinterpret_cast<const uint4*>(gu + t2 * 2 * I + c2);
    u4[1] = *reinterpret_cast<const uint4*>(gu + t2 * 2 * I + I + c2);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      if (k == 1 && !two) break;
      const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4[k]);
      const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4[k]);
      uint4 o4;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
        o2[j] = __floats2bfloat162_rn(bf_silu_fast(g.x) * u.x, bf_silu_fast(g.y) * u.y);
      }
      *reinterpret_cast<uint4*>(out + (k ? t2 * I + c2 : t * I + c)) = o4;
    }
  }
}

// silu(f gate) * (f up) for bf16 rows that still lack the factor f (see BfRowScale): I a
// multiple of 8 and at least 256; cudaErrorInvalidValue otherwise.
BF_EXPORT int bf_silu_mul_scaled(const void* gu, void* out, int T, int I,
                                 const float* row_partials, int row_count, int row_width,
                                 float row_eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (I % 8 || I < 256 || ((uintptr_t)gu & 15) || ((uintptr_t)out & 15) ||
      !row_partials || row_count <= 0 || row_width <= 0)
    return (int)cudaErrorInvalidValue;
  const BfRowScale rs = {row_partials, row_count, 1.f / (float)row_width, row_eps};
  const int threads = 256;
  long long blocks = ((long long)T * (I / 8) + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return bf_launch_pdl(silu_mul_bf16_scaled_kernel, dim3((int)blocks), dim3(threads), 0, stream,
                       (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, T, I, rs);
}

BF_EXPORT int bf_silu_mul(const void* gu, void* out, int T, int I, int act_dtype,
                          cudaStream_t stream) {
  if (T <= 0) return 0;
  const int threads = 256;
  if (act_dtype == BF_DTYPE_BF16 && I % 8 == 0 && ((uintptr_t)gu & 15) == 0 &&
      ((uintptr_t)out & 15) == 0) {
    long long blocks = ((long long)T * (I / 8) + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    return bf_launch_pdl(silu_mul_bf16_vec_kernel, dim3((int)blocks), dim3(threads), 0, stream,
                         (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, T, I);
  }
  long long blocks = ((long long)T * I + threads - 1) / threads;
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (act_dtype == BF_DTYPE_F32)
    silu_mul_kernel<float><<<(int)blocks, threads, 0, stream>>>((const float*)gu, (float*)out,
                                                               T, I);
  else
    silu_mul_kernel<__nv_bfloat16><<<(int)blocks, threads, 0, stream>>>(
        (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, T, I);
  return bf_launch_status();
}

// ------------------------------------------------------------- token ids from the device
// dst[pairs[2i]] = src[pairs[2i+1]]: the ids that the last step sampled become this step's
// input tokens without a trip through the host.
__global__ void copy_ids_kernel(int* __restrict__ dst, const int* __restrict__ src,
                                const int* __restrict__ pairs, int n) {
  bf_pdl_trigger();
  bf_pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[pairs[2 * i]] = src[pairs[2 * i + 1]];
}

BF_EXPORT int bf_copy_ids(int* dst, const int* src, const int* pairs, int n, cudaStream_t stream) {
  if (n <= 0) return 0;
  copy_ids_kernel<<<(n + 127) / 128, 128, 0, stream>>>(dst, src, pairs, n);
  return bf_launch_status();
}

BF_TRACE_READER(bf_trace_read_elementwise)
