// TMA (cp.async.bulk.tensor) helpers: host-side tensor-map encoding through the driver entry
// point (no link-time dependency on libcuda) and device-side load / store wrappers.
// Only plain loads and stores are used: no multicast, no peer memory.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace based {
namespace tma {

// ---------------------------------------------------------------- host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// bf16 tensor [d3][d2][d1][d0] with d0 contiguous; strides of d1, d2, d3 in ELEMENTS (multiples of 8);
// box = box0 x box1 x 1 x 1, with 128-byte swizzle (box0 * 2 bytes <= 128) or, when sw128 is false,
// rows of box0 elements packed back to back.  Returns 0 on success.
inline int encode_bf16_4d(CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3,
                          int64_t s1, int64_t s2, int64_t s3, uint32_t box0, uint32_t box1, bool sw128) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -1;
  const cuuint64_t dims[4] = {d0, d1, d2, d3};
  const cuuint64_t strides[3] = {(cuuint64_t)s1 * 2, (cuuint64_t)s2 * 2, (cuuint64_t)s3 * 2};
  const cuuint32_t box[4] = {box0, box1, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, sw128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}
inline int encode_bf16_4d_sw128(CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3,
                                int64_t s1, int64_t s2, int64_t s3, uint32_t box0, uint32_t box1) {
  return encode_bf16_4d(map, base, d0, d1, d2, d3, s1, s2, s3, box0, box1, true);
}

// ---------------------------------------------------------------- device
__device__ __forceinline__ void mbar_expect_tx(uint32_t mbar_saddr, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}\n" ::"r"(mbar_saddr),
               "r"(bytes)
               : "memory");
}
// Tile load global -> shared; completion is signalled on the mbarrier in bytes.  The inner
// coordinate c0 times the element size must be a multiple of 16 bytes (here it is always 0 or
// a multiple of 64 elements); the other coordinates may be negative or past the end (zero fill).
__device__ __forceinline__ void load_4d(uint32_t dst_saddr, const CUtensorMap* map, uint32_t mbar_saddr, int c0, int c1,
                                        int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];\n" ::
          "r"(dst_saddr),
      "l"(map), "r"(mbar_saddr), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// Tile store shared -> global (rows past the tensor's extent are clipped); never started at a
// negative coordinate.
__device__ __forceinline__ void store_4d(const CUtensorMap* map, uint32_t src_saddr, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];\n" ::"l"(map),
               "r"(src_saddr), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];\n" ::"l"(map) : "memory");
}

// Byte offset of the 16-byte chunk `chunk` (0..7) of row `row` inside a 128-byte-swizzled tile
// whose rows are 128 bytes and whose base is 1024-byte aligned.
__device__ __forceinline__ uint32_t sw128_offset(int row, int chunk) {
  return (uint32_t)row * 128u + (uint32_t)((chunk ^ (row & 7)) << 4);
}

}  // namespace tma
}  // namespace based
