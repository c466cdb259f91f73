// TMA (cp.async.bulk.tensor) helpers: host-side tensor-map encoding through the driver entry
// point (no link-time dependency on libcuda) and device-side load / store wrappers.
// Only plain loads and stores are used: no multicast, no peer memory.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <mutex>

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

// bf16 rows of `groups * 8` contiguous elements, seen as [d4][d3][groups][rows][8]: the row is cut into 16-byte
// groups and the GROUP index becomes a tensor dimension outside the row index.  A box of
// 8 x box_rows x groups x 1 x 1 then lands in shared memory as [group][row][16 bytes] - the no-swizzle canonical
// layout of a UMMA operand (K-major with the k-halves as groups, or MN-major with 8-column groups) - in ONE copy.
// Strides of rows, d3, d4 in ELEMENTS (multiples of 8).  Rows past `rows` read as zero.  Returns 0 on success.
inline int encode_bf16_grouped_rows(CUtensorMap* map, const void* base, uint64_t groups, uint64_t rows, uint64_t d3,
                                    uint64_t d4, int64_t s_row, int64_t s3, int64_t s4, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -1;
  const cuuint64_t dims[5] = {8, rows, groups, d3, d4};
  const cuuint64_t strides[4] = {(cuuint64_t)s_row * 2, 16, (cuuint64_t)s3 * 2, (cuuint64_t)s4 * 2};
  const cuuint32_t box[5] = {8, box_rows, (cuuint32_t)groups, 1, 1};
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

// A few recently encoded tensor maps, keyed by everything that went into them.  Encoding costs a driver call per
// map; a generation loop or a benchmark calls with the same pointers and shapes again and again.
struct MapKey {
  const void* base;
  uint64_t dims[5];
  int64_t strides[4];
  uint32_t box[3];
  uint32_t kind;
};
class MapCache {
 public:
  // Returns true and fills *out when the key is cached.
  bool find(const MapKey& k, CUtensorMap* out) {
    std::lock_guard<std::mutex> lock(mu_);
    for (int i = 0; i < kSlots; ++i)
      if (used_[i] && memcmp(&keys_[i], &k, sizeof(MapKey)) == 0) {
        *out = maps_[i];
        return true;
      }
    return false;
  }
  void put(const MapKey& k, const CUtensorMap& m) {
    std::lock_guard<std::mutex> lock(mu_);
    keys_[next_] = k;
    maps_[next_] = m;
    used_[next_] = true;
    next_ = (next_ + 1) % kSlots;
  }

 private:
  static constexpr int kSlots = 32;
  std::mutex mu_;
  MapKey keys_[kSlots];
  CUtensorMap maps_[kSlots];
  bool used_[kSlots] = {};
  int next_ = 0;
};
inline MapKey make_key(const void* base, uint64_t a, uint64_t b, uint64_t c, uint64_t d, uint64_t e, int64_t s0,
                       int64_t s1, int64_t s2, int64_t s3, uint32_t b0, uint32_t b1, uint32_t b2, uint32_t kind) {
  MapKey k;
  memset(&k, 0, sizeof(k));  // padding bytes take part in the comparison
  k.base = base;
  k.dims[0] = a; k.dims[1] = b; k.dims[2] = c; k.dims[3] = d; k.dims[4] = e;
  k.strides[0] = s0; k.strides[1] = s1; k.strides[2] = s2; k.strides[3] = s3;
  k.box[0] = b0; k.box[1] = b1; k.box[2] = b2;
  k.kind = kind;
  return k;
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
__device__ __forceinline__ void load_5d(uint32_t dst_saddr, const CUtensorMap* map, uint32_t mbar_saddr, int c0, int c1,
                                        int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];\n" ::
          "r"(dst_saddr),
      "l"(map), "r"(mbar_saddr), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
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
