// Sampling from float logits on the device: repetition penalty, greedy argmax,
// temperature, top-k, top-p, and the draw.
//
// Order of operations as in the reference's CPU sampler (src/engine/sampler.ts:57-157):
// penalty on generated tokens (s > 0 ? s / pen : s * pen, once per occurrence),
// argmax if the temperature is 0, else divide by the temperature, keep the top_k
// largest, cut at the first prefix of descending probabilities whose sum reaches
// top_p, renormalise, and take the first kept token whose running probability
// exceeds a uniform number.  Two stated differences: the reference sorts the whole
// vocabulary on the host for every token (:87-93) and walks the kept tokens in
// descending order; here thresholds are found by bisection on the value, tokens
// tied with the threshold are all kept, and the draw walks the kept tokens in
// index order.  Argmax returns the lowest index among equal maxima (the
// reference's device argmax leaves that open, cuda/kernels/bf16_kernels.cu:1265-1353).
//
// The uniform number comes from the host, one per row, so a request draws the
// same tokens whatever else is in the batch.
#include <float.h>

#include "common.cuh"

#define SAMPLE_THREADS 1024

// ---------------------------------------------------------- repetition penalty
// items: (row, token, count) triples; logits[row, token] is penalised count times.
__global__ void repetition_penalty_kernel(float* __restrict__ logits, int V,
                                          const int* __restrict__ items, int n_items,
                                          const float* __restrict__ penalty) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_items) return;
  const int row = items[3 * i], tok = items[3 * i + 1], cnt = items[3 * i + 2];
  if (tok < 0 || tok >= V) return;
  const float pen = penalty[row];
  float s = logits[(size_t)row * V + tok];
  for (int c = 0; c < cnt; ++c) s = s > 0.f ? s / pen : s * pen;
  logits[(size_t)row * V + tok] = s;
}

BF_EXPORT int bf_repetition_penalty(float* logits, int V, const int* items, int n_items,
                                    const float* penalty, cudaStream_t stream) {
  if (n_items <= 0) return 0;
  repetition_penalty_kernel<<<(n_items + 127) / 128, 128, 0, stream>>>(logits, V, items, n_items,
                                                                      penalty);
  return bf_launch_status();
}

// --------------------------------------------------------------------- helpers
__device__ __forceinline__ unsigned ordered_key(float f) {
  const unsigned u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float block_sum_f(float v, float* scratch) {
  return block_sum(v, scratch);
}

__device__ __forceinline__ float block_max_f(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < (blockDim.x >> 5) ? scratch[lane] : -FLT_MAX;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  const float r = scratch[32];
  __syncthreads();
  return r;
}

// ------------------------------------------------------------------ the sampler
// One block per row.  logits [R, V] float; per row: temperature, top_k, top_p,
// uniform in [0, 1).  out[r] = chosen token id.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ uniform, int* __restrict__ out) {
  __shared__ float scratch[33];
  __shared__ float s_val[SAMPLE_THREADS / 32];
  __shared__ int s_idx[SAMPLE_THREADS / 32];
  __shared__ float s_prefix[SAMPLE_THREADS];
  __shared__ int s_choice;
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* x = logits + (size_t)r * V;
  const float T = temperature[r];

  if (T <= 0.f) {
    // greedy: the lowest index among the maxima
    float bv = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
      const float v = x[i];
      if (v > bv || (v == bv && i < bi) || bi == 0x7fffffff) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((tid & 31) == 0) { s_val[tid >> 5] = bv; s_idx[tid >> 5] = bi; }
    __syncthreads();
    if (tid < 32) {
      bv = tid < SAMPLE_THREADS / 32 ? s_val[tid] : -FLT_MAX;
      bi = tid < SAMPLE_THREADS / 32 ? s_idx[tid] : 0x7fffffff;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if (tid == 0) out[r] = bi;
    }
    return;
  }

  // scaled scores s_i = x_i / T; everything below is on s
  float m = -FLT_MAX;
  for (int i = tid; i < V; i += SAMPLE_THREADS) m = fmaxf(m, x[i] / T);
  m = block_max_f(m, scratch);

  unsigned keep_key = 0u;   // a token is kept when ordered_key(s_i) >= keep_key
  const int k = top_k[r];
  if (k > 0 && k < V) {
    // the largest key t with count(key >= t) >= k is the key of the k-th largest score
    unsigned t = 0u;
    for (int bit = 31; bit >= 0; --bit) {
      const unsigned cand = t | (1u << bit);
      float cnt = 0.f;
      for (int i = tid; i < V; i += SAMPLE_THREADS) cnt += ordered_key(x[i] / T) >= cand;
      cnt = block_sum_f(cnt, scratch);
      if (cnt >= (float)k) t = cand;
    }
    keep_key = t;
  }
  const float p = top_p[r];
  if (p < 1.f) {
    float z = 0.f;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
      const float s = x[i] / T;
      if (ordered_key(s) >= keep_key) z += expf(s - m);
    }
    z = block_sum_f(z, scratch);
    const float want = p * z;
    // the largest key t >= keep_key whose tokens (key >= t) hold at least p of the mass
    unsigned t = 0u;
    for (int bit = 31; bit >= 0; --bit) {
      const unsigned cand = t | (1u << bit);
      float mass = 0.f;
      for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const float s = x[i] / T;
        const unsigned key = ordered_key(s);
        if (key >= cand && key >= keep_key) mass += expf(s - m);
      }
      mass = block_sum_f(mass, scratch);
      if (mass >= want) t = cand;
    }
    if (t > keep_key) keep_key = t;
  }

  // the draw: contiguous chunk per thread, prefix over threads, walk inside one chunk
  const int chunk = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const int a = tid * chunk, b = min(V, a + chunk);
  float mine = 0.f;
  for (int i = a; i < b; ++i) {
    const float s = x[i] / T;
    if (ordered_key(s) >= keep_key) mine += expf(s - m);
  }
  s_prefix[tid] = mine;
  if (tid == 0) s_choice = -1;
  __syncthreads();
  if (tid == 0) {
    float run = 0.f;
    for (int i = 0; i < SAMPLE_THREADS; ++i) {   // exclusive prefix, in index order
      const float v = s_prefix[i];
      s_prefix[i] = run;
      run += v;
    }
    scratch[0] = run;
  }
  __syncthreads();
  const float total = scratch[0];
  const float target = uniform[r] * total;
  const float before = s_prefix[tid];
  if (mine > 0.f && before <= target && before + mine > target) {
    float run = before;
    int pick = -1, last = -1;
    for (int i = a; i < b; ++i) {
      const float s = x[i] / T;
      if (ordered_key(s) >= keep_key) {
        run += expf(s - m);
        last = i;
        if (run > target) { pick = i; break; }
      }
    }
    s_choice = pick >= 0 ? pick : last;
  }
  __syncthreads();
  if (s_choice < 0 && tid == 0) {
    // rounding left the target at or past the total: the last kept token
    int last = 0;
    for (int i = V - 1; i >= 0; --i)
      if (ordered_key(x[i] / T) >= keep_key) { last = i; break; }
    s_choice = last;
  }
  __syncthreads();
  if (tid == 0) out[r] = s_choice;
}

BF_EXPORT int bf_sample(const float* logits, int R, int V, const float* temperature,
                        const int* top_k, const float* top_p, const float* uniform, int* out,
                        cudaStream_t stream) {
  if (R <= 0) return 0;
  sample_kernel<<<R, SAMPLE_THREADS, 0, stream>>>(logits, V, temperature, top_k, top_p, uniform,
                                                  out);
  return bf_launch_status();
}
