// Shared helpers for the engine's CUDA kernels (sm_100a).
//
// Every launcher is a plain C function: raw device pointers, sizes, a stream; it
// returns the cudaError_t of the launch as an int (0 = ok).  Activations and
// cache pages are either float (dtype code 0) or __nv_bfloat16 (code 1); all
// arithmetic inside a kernel is float.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define BF_DTYPE_F32 0
#define BF_DTYPE_BF16 1

// Bits of the device error word that kernels set instead of faulting.
#define BF_ERR_TOKEN_ID 1      // token id outside the vocabulary
#define BF_ERR_SLOT 2          // cache slot outside the pool
#define BF_ERR_PAGE 4          // page id outside the pool
#define BF_ERR_WAIT 8          // a bounded wait gave up
#define BF_ERR_SPLITS 16       // a row's keys need more splits than the scratch has room for

#define BF_EXPORT extern "C" __attribute__((visibility("default")))

__device__ __forceinline__ float bf_ld(const float* p) { return *p; }
__device__ __forceinline__ float bf_ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void bf_st(float* p, float v) { *p = v; }
__device__ __forceinline__ void bf_st(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a whole block; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  float r = scratch[32];
  __syncthreads();
  return r;
}

static inline int bf_launch_status() { return (int)cudaGetLastError(); }

// Function attributes (the dynamic shared memory limit) belong to a device, so launchers keep
// their "configured" flag per device: index of the current one, clamped to the table.
#define BF_MAX_DEVICES 64
static inline int bf_current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return 0;
  return dev < BF_MAX_DEVICES ? dev : BF_MAX_DEVICES - 1;
}

// ---------------------------------------------------- programmatic dependent launch
// A kernel launched through bf_launch_pdl may be scheduled while its predecessor on the
// stream is still running (its blocks become resident, its prologue runs), which hides the
// launch latency between the short kernels of a decode step.  Such a kernel must call
// bf_pdl_wait() before it touches global memory that an earlier kernel writes or reads: the
// call returns when every earlier grid has completed and its writes are visible.  Every
// thread calls it, on every path, so that "this grid has completed" implies the same of all
// grids before it.  bf_pdl_trigger(), called first, lets the kernel after this one be
// scheduled in turn (it then sits in its own wait).  What a kernel does between the two
// (barrier and tensor-memory set-up, fetching weights, which no kernel of a step writes)
// overlaps the kernels before it.  Launched the ordinary way, both calls do nothing.
__device__ __forceinline__ void bf_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void bf_pdl_trigger() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

int bf_pdl_enabled();    // defined in elementwise.cu; switched by bf_set_pdl()

template <typename... KArgs, typename... Args>
static inline int bf_launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = bf_pdl_enabled();
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
  if (e != cudaSuccess) return (int)e;
  return bf_launch_status();
}

// ------------------------------------------------------------------ a row factor left out
// A product whose epilogue also adds into the residual stream and prepares the next norm's
// output (gemm_tcgen05_cluster.cu) cannot know the row's mean square, which spans all its
// CTAs.  It leaves x * w_norm and, per row, one partial sum of squares per CTA; the factor
// rsqrt(sum / width + eps) commutes with the product that follows, so the kernel after
// that product applies it.  `partials` is [rows, count]; a null pointer means no factor.
struct BfRowScale {
  const float* partials;
  int count;
  float inv_width, eps;
};
// By one warp, in two steps so that the loads of the first can be in flight under other
// work: every lane fetches its share (up to four values; a row has one partial per CTA of the
// product, 128 or so), then the shares are summed in one fixed order and every lane gets the
// factor.
struct BfRowShare {
  float v[4];
};
__device__ __forceinline__ BfRowShare bf_row_fetch(const BfRowScale& rs, int row, int lane) {
  BfRowShare sh = {{0.f, 0.f, 0.f, 0.f}};
  if (!rs.partials) return sh;
  const float* p = rs.partials + (size_t)row * rs.count;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (lane + 32 * j < rs.count) sh.v[j] = p[lane + 32 * j];
  for (int i = lane + 128; i < rs.count; i += 32) sh.v[0] += p[i];
  return sh;
}
__device__ __forceinline__ float bf_row_finish(const BfRowScale& rs, const BfRowShare& sh) {
  if (!rs.partials) return 1.f;
  const float s = warp_sum(((sh.v[0] + sh.v[1]) + sh.v[2]) + sh.v[3]);
  return rsqrtf(s * rs.inv_width + rs.eps);
}
__device__ __forceinline__ float bf_row_factor(const BfRowScale& rs, int row, int lane) {
  return bf_row_finish(rs, bf_row_fetch(rs, row, lane));
}

// ------------------------------------------------------------------- timeline of a step
// Built with -DBF_TRACE (BINFER_B200_TRACE=1 in the environment when the library is
// compiled; it goes to a build folder of its own), the decode step's kernels record the
// global timer when block 0 starts, when its dependency wait returns and when it ends.  Each
// source file keeps its own list and exports a reader; `python -m binfer_b200.microbench
// step_timeline` puts them in order.  Without the flag the macros are empty.
#ifdef BF_TRACE
#define BF_TRACE_EVENTS 8192
static __device__ unsigned long long bf_trace_time[BF_TRACE_EVENTS];
static __device__ int bf_trace_code[BF_TRACE_EVENTS];
static __device__ int bf_trace_count;
__device__ __forceinline__ void bf_trace_point(int code) {
  if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    const int i = atomicAdd(&bf_trace_count, 1);
    if (i < BF_TRACE_EVENTS) {
      bf_trace_time[i] = t;
      bf_trace_code[i] = code;
    }
  }
}
#define BF_TRACE_POINT(code) bf_trace_point(code)
// Copies this file's events out (times in ns, codes), empties the list, returns their number.
#define BF_TRACE_READER(name)                                                    \
  BF_EXPORT int name(unsigned long long* times, int* codes) {                    \
    int n = 0, zero = 0;                                                         \
    cudaMemcpyFromSymbol(&n, bf_trace_count, sizeof(int));                       \
    cudaMemcpyFromSymbol(times, bf_trace_time, sizeof(bf_trace_time));           \
    cudaMemcpyFromSymbol(codes, bf_trace_code, sizeof(bf_trace_code));           \
    cudaMemcpyToSymbol(bf_trace_count, &zero, sizeof(int));                      \
    return n < BF_TRACE_EVENTS ? n : BF_TRACE_EVENTS;                            \
  }
#else
#define BF_TRACE_POINT(code)
#define BF_TRACE_READER(name)
#endif
// kernel ids of the trace codes (code = 10 * id + phase; phase 0 start, 1 after the wait, 2 end;
// the cluster product also 5: its products are done, 3: its sums are sent, 4: the cluster's
// barrier is passed)
#define BF_TR_RMSNORM 1
#define BF_TR_SILU 2
#define BF_TR_QKNORM 3
#define BF_TR_ATTN 4
#define BF_TR_MERGE 5
#define BF_TR_GEMM 6
