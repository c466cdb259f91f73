// Pieces shared by the two tensor-core kernels of the Taylor linear-attention prefill:
// chunk geometry, the symmetry-packed feature map phi' in bf16x2 arithmetic, the map from the
// reference's 273-feature layout to the packed one, and the kernel parameter block.
#pragma once

#include "common.cuh"
#include "tcgen05.cuh"

#include <cuda.h>

#include <type_traits>

namespace based {
namespace tcp {

using namespace tc;

constexpr int C = 128;     // tokens per chunk
constexpr int DR = 160;    // packed + padded feature count
// threads per CTA: 4 expansion warps (0-3), 4 polynomial / state-drain warps (4-7), 4 output warps (8-11),
// the MMA warp (12), the TMA producer warp (13; one thread issues the copies), 2 spare warps.  A compute warp w reaches TMEM lanes 32*(w%4)..+31.
constexpr int NT = 512;
constexpr int W_OUT = 8, W_MMA = 12, W_LOAD = 13;

constexpr int STAGE_STRIDE_F = 164;  // floats per row of the final fp32 staging (conflict-free 16 B stores)

template <int G0, int G1, typename F>
__device__ __forceinline__ void static_for(F&& f) {
  if constexpr (G0 < G1) {
    f(std::integral_constant<int, G0>{});
    static_for<G0 + 1, G1>(f);
  }
}

// ---------------------------------------------------------------- packed feature map, bf16x2 arithmetic
// Feature order of phi' (160 features = 80 bf16x2 words; u = x/2, c = 1/sqrt2):
//   0        : 1            (features 1..7 are zero padding)
//   8  + i   : u_i                                  i = 0..15      (= x_i / 2)
//   24 + a   : c * u_a^2                            a = 0..15      (= x_a^2 / (4 sqrt2))
//   40 + m   : u_{2m} u_{2m+1}                      m = 0..7
//   48 + 4*blk(m,n) + 2*(a&1) + (b&1) : u_a u_b     a in pair m, b in pair n, m < n,
//                                                   blk(m,n) = 7m - m(m-1)/2 + (n - m - 1)
// Off-diagonal products appear once with weight 1/4 = sqrt2 * 1/(4 sqrt2), so that
// phi'(q).phi'(k) = 1 + s + s^2/2 (s = q.k/4) exactly as for the 273-feature map.
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;\n" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t fma_bf16x2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
// pair-block number blk = 0..27 -> (m, n), m < n
__host__ __device__ constexpr int blk_m(int blk) {
  int m = 0;
  while (blk >= 7 - m) { blk -= 7 - m; ++m; }
  return m;
}
__host__ __device__ constexpr int blk_n(int blk) {
  int m = 0;
  while (blk >= 7 - m) { blk -= 7 - m; ++m; }
  return m + 1 + blk;
}
constexpr uint32_t kHalf2 = 0x3F003F00u;    // (0.5, 0.5)
constexpr uint32_t kRsqrt2_2 = 0x3F353F35u; // (0.70703125, 0.70703125): bf16(1/sqrt2)
constexpr uint32_t kOneLo = 0x00003F80u;    // (1.0, 0)

// Expands one token: X = the 16 raw bf16 values as 8 packed words.  emit(G, w0, w1, w2, w3) is
// called for G = 0..19 in order with the four words of feature group G (features 8G .. 8G+7).
template <typename Emit>
__device__ __forceinline__ void expand_packed(const uint32_t (&X)[8], Emit&& emit) {
  uint32_t U[8];
#pragma unroll
  for (int m = 0; m < 8; ++m) U[m] = mul_bf16x2(X[m], kHalf2);
  emit(std::integral_constant<int, 0>{}, kOneLo, 0u, 0u, 0u);
  emit(std::integral_constant<int, 1>{}, U[0], U[1], U[2], U[3]);
  emit(std::integral_constant<int, 2>{}, U[4], U[5], U[6], U[7]);
  {
    uint32_t d[8];
#pragma unroll
    for (int m = 0; m < 8; ++m) d[m] = mul_bf16x2(mul_bf16x2(U[m], U[m]), kRsqrt2_2);
    emit(std::integral_constant<int, 3>{}, d[0], d[1], d[2], d[3]);
    emit(std::integral_constant<int, 4>{}, d[4], d[5], d[6], d[7]);
  }
  {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)  // (u_{4j} u_{4j+1}, u_{4j+2} u_{4j+3})
      w[j] = mul_bf16x2(__byte_perm(U[2 * j], U[2 * j + 1], 0x5410), __byte_perm(U[2 * j], U[2 * j + 1], 0x7632));
    emit(std::integral_constant<int, 5>{}, w[0], w[1], w[2], w[3]);
  }
  // cross blocks (m < n), two blocks (four words) per group
  static_for<0, 14>([&](auto GG) {
    constexpr int g = decltype(GG)::value;
    constexpr int m0 = blk_m(2 * g), n0 = blk_n(2 * g), m1 = blk_m(2 * g + 1), n1 = blk_n(2 * g + 1);
    const uint32_t w0 = mul_bf16x2(__byte_perm(U[m0], 0, 0x1010), U[n0]);
    const uint32_t w1 = mul_bf16x2(__byte_perm(U[m0], 0, 0x3232), U[n0]);
    const uint32_t w2 = mul_bf16x2(__byte_perm(U[m1], 0, 0x1010), U[n1]);
    const uint32_t w3 = mul_bf16x2(__byte_perm(U[m1], 0, 0x3232), U[n1]);
    emit(std::integral_constant<int, 6 + g>{}, w0, w1, w2, w3);
  });
}

// Index of full feature f (0..272) in the packed vector, and whether it is an off-diagonal
// second-order term (whose packed value is sqrt2 times the full-map value).
__device__ __forceinline__ int packed_index(int f, bool& offdiag) {
  offdiag = false;
  if (f == 0) return 0;
  if (f < 17) return 8 + (f - 1);
  const int g = f - 17, i = g >> 4, j = g & 15;
  const int a = min(i, j), b = max(i, j);
  if (a == b) return 24 + a;
  offdiag = true;
  const int m = a >> 1, n = b >> 1;
  if (m == n) return 40 + m;
  const int blk = 7 * m - (m * (m - 1)) / 2 + (n - m - 1);
  return 48 + 4 * blk + 2 * (a & 1) + (b & 1);
}

struct Params {
  CUtensorMap mq, mk, mv;   // q, k: [B][H][2 k-halves][L][8]; v: [B][H][dv/8 groups][L][8]; box = 128 tokens
  const __nv_bfloat16 *q, *k, *v;
  __nv_bfloat16* y;
  void *kv_state, *k_state;
  int H, L, dv, state_bf16;
  Strides3 sq, sk, sv, sy;
  float eps;
  unsigned int* status;
  // Sequence split.  The sequence is cut into nseg segments of seg_chunks chunks and the grid is
  // (batch x head) x grid_segs CTAs, one segment each.
  //   mode 0: grid_segs = nseg = 1, the whole sequence in one CTA.
  //   mode 1: segments 0 .. nseg-2 only accumulate their own state^T (packed features, fp32) and
  //           write it to seg_state[bh][seg][dv+1][160]; no outputs.
  //   mode 2: every segment computes its outputs; segment s > 0 starts from seg_state[bh][s-1],
  //           which by then holds the sum over the segments before it (see segment_scan_kernel);
  //           the last segment writes kv_state / k_state.
  int mode, nseg, grid_segs, seg_chunks;
  float* seg_state;
};
constexpr int MODE_WHOLE = 0, MODE_SEG_STATE = 1, MODE_SEG_OUTPUT = 2;

}  // namespace tcp
}  // namespace based
