// Host-side making of TMA tensor maps, and the device-side mbarrier / bulk-tensor-copy
// instructions that go with them.  The driver's encode function is looked up at run time
// (cudaGetDriverEntryPoint), so the library does not link against libcuda.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

typedef CUresult (*BfEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                    const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                    const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline BfEncodeTiledFn bf_encode_tiled() {
  static BfEncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<BfEncodeTiledFn>(p);
  }
  return fn;
}

// A [rows, cols] bf16 row-major matrix (row stride ld elements), fetched in boxes of
// box_rows x box_cols (box_cols * 2 bytes = 128) with the 128-byte swizzle; reads outside the
// matrix give zeros.  Returns 0 or a cudaError_t.
static inline int bf_make_tensor_map_bf16_2d(CUtensorMap* map, const void* base, long long rows,
                                             long long cols, long long ld, int box_rows,
                                             int box_cols) {
  BfEncodeTiledFn enc = bf_encode_tiled();
  if (!enc) return (int)cudaErrorNotSupported;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                   strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

// The same for writing: boxes of box_rows x 128 bytes (64 bf16 or 32 floats: elem_bytes 2 or 4)
// leave shared memory (128-byte swizzle) for a [rows, cols] matrix; what lies outside the
// matrix is not written.
static inline int bf_make_tensor_map_2d_store(CUtensorMap* map, void* base, long long rows,
                                              long long cols, long long ld, int box_rows,
                                              int elem_bytes) {
  BfEncodeTiledFn enc = bf_encode_tiled();
  if (!enc) return (int)cudaErrorNotSupported;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * elem_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map,
                   elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                   : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                   2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

// The paged cache [pages, heads, page_size, d] (bf16) as a 4-d tensor, fetched in boxes of
// `box_pages` whole pages of one head and 64 columns: {64, page_size, 1, box_pages}.  In
// shared memory the box is box_pages * page_size rows of 128 bytes, page after page, in the
// 128-byte swizzle: what box_pages separate boxes of the 2-d view above would leave, one
// behind the other (page_size is a multiple of 8, the swizzle's period in rows).  For pages
// that lie side by side in the pool: one instruction instead of one per page.
static inline int bf_make_tensor_map_pages_bf16(CUtensorMap* map, const void* base,
                                                long long pages, int heads, int page_size, int d,
                                                int box_pages) {
  BfEncodeTiledFn enc = bf_encode_tiled();
  if (!enc) return (int)cudaErrorNotSupported;
  const cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)page_size, (cuuint64_t)heads,
                              (cuuint64_t)pages};
  const cuuint64_t strides[3] = {(cuuint64_t)d * 2, (cuuint64_t)page_size * d * 2,
                                 (cuuint64_t)heads * page_size * d * 2};
  const cuuint32_t box[4] = {64u, (cuuint32_t)page_size, 1u, (cuuint32_t)box_pages};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims,
                   strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

#ifdef __CUDACC__
__device__ __forceinline__ uint32_t bf_smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void bf_mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bf_smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void bf_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bf_smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool bf_mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bf_smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Wait with a clock limit (about a second).  False when it gave up.
__device__ __forceinline__ bool bf_mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  if (bf_mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!bf_mbar_try_wait(bar, parity))
    if (clock64() - t0 > 2000000000LL) return false;
  return true;
}
__device__ __forceinline__ void bf_tma_load_2d(void* smem_dst, const CUtensorMap* map,
                                               uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];" ::"r"(bf_smem_u32(smem_dst)),
      "l"(map), "r"(bf_smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// A box from shared memory to the matrix, in this thread's current bulk group (x: column, a
// multiple of 8 elements; no coordinate negative).
__device__ __forceinline__ void bf_tma_store_2d(const CUtensorMap* map, const void* smem_src,
                                                int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   map),
               "r"(bf_smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
// The same, added to what the matrix holds (the element type is the map's).
__device__ __forceinline__ void bf_tma_reduce_add_2d(const CUtensorMap* map, const void* smem_src,
                                                     int x, int y) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::
          "l"(map),
      "r"(bf_smem_u32(smem_src)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void bf_bulk_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// until at most N of this thread's bulk groups have not yet read their shared memory
template <int N>
__device__ __forceinline__ void bf_bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// (x: column, a multiple of 8 elements = 16 bytes; the other coordinates have no rule)
__device__ __forceinline__ void bf_tma_load_4d(void* smem_dst, const CUtensorMap* map,
                                               uint64_t* bar, int x, int row, int head, int page) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(bf_smem_u32(smem_dst)),
      "l"(map), "r"(bf_smem_u32(bar)), "r"(x), "r"(row), "r"(head), "r"(page)
      : "memory");
}
#endif
