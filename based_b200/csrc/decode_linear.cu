// Linear layers of a decode step: y[M, N] = x[M, K] W[N, K]^T (+ bias) for a handful of rows
// (M = batch of single tokens), bf16 in, fp32 accumulation, with the elementwise step that
// follows the projection in the Based blocks fused into the epilogue:
//   PLAIN   y = x W^T + b                                   (out_proj, fc2, Wqkv, q/k/v projections)
//   SWIGLU  out = (x W1^T) * act(x W2^T), W = [W1; W2]      fc1 + `y * act(gate)` of GatedMlp.forward
//                                                           (based/models/mlp.py:141-154)
//   CONV    u = x W^T + b, [u1 | u2] = u; the BaseConv decode step on u1 (shift the [B, d, k] state,
//           append, dot with the taps), silu, gate by u2       in_proj + ShortConvolution.step + gate
//                                                           (based/models/mixers/convolution.py:88-109, :205-211)
// With M <= 16 the work is reading W once: HBM-bound (2 bytes per weight, 2 M flops per weight).
// A warp owns 8 output columns (one n8 tile of mma.sync.m16n8k16; M = 16 is exactly the tile
// height) and a quarter of K; the four warps of a block reduce through shared memory.  Each lane
// reads 16 contiguous bytes of one weight row per step -- the K order inside a 32-wide block is
// permuted identically for x and W, which a dot product does not notice -- so a warp's load
// covers 8 rows x 64 bytes, and x (a few KB, L1/L2 resident) is read the same way.
#include "common.cuh"

namespace based {
namespace {

constexpr int WARPS = 4;  // split of K inside a block
enum Epi { EPI_PLAIN = 0, EPI_SWIGLU = 1, EPI_CONV = 2 };

struct LinParams {
  const __nv_bfloat16 *x, *w, *bias;
  __nv_bfloat16* out;
  int M, N, K;          // N = rows of W (PLAIN: outputs; SWIGLU / CONV: 2 x outputs)
  int64_t sx, so;       // row strides of x and out
  int act;              // SWIGLU: 0 silu, 1 sigmoid
  // CONV
  __nv_bfloat16* state;            // [M, N/2, ck]
  const void *cw, *cb;             // taps [N/2, ck], bias [N/2] or null
  int ck, cw_bf16;
};

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float sigmoid_f(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ float ld_w(const void* p, int bf16, int i) {
  return bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]) : static_cast<const float*>(p)[i];
}

// NTILE = 1: one n8 tile per warp; 2: two tiles, columns n0.. and n0 + N/2.. (the two halves an epilogue combines)
// grid = (outputs / 8, ceil(M / 16)), block = WARPS x 32
template <int NTILE, int EPI>
__global__ void __launch_bounds__(WARPS * 32) decode_linear_kernel(const LinParams p) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * 8, m0 = blockIdx.y * 16;
  const int half = p.N / 2;
  // K slice of this warp, in blocks of 32
  const int kblocks = p.K / 32, per = (kblocks + WARPS - 1) / WARPS;
  const int kb0 = warp * per, kb1 = min(kb0 + per, kblocks);
  const int r0 = m0 + g, r1 = m0 + g + 8;
  const bool v0 = r0 < p.M, v1 = r1 < p.M;
  const __nv_bfloat16* xa = p.x + (int64_t)(v0 ? r0 : 0) * p.sx + 8 * t;
  const __nv_bfloat16* xb = p.x + (int64_t)(v1 ? r1 : 0) * p.sx + 8 * t;
  const __nv_bfloat16* wr[NTILE];
#pragma unroll
  for (int i = 0; i < NTILE; ++i) wr[i] = p.w + (int64_t)(n0 + g + i * half) * p.K + 8 * t;
  float acc[NTILE][4];
#pragma unroll
  for (int i = 0; i < NTILE; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;
  constexpr int U = 4;  // K blocks per round: their loads are issued together
  const uint4 zero = make_uint4(0, 0, 0, 0);
  for (int kb = kb0; kb < kb1; kb += U) {
    uint4 wv[U][NTILE], a0[U], a1[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const bool ok = kb + u < kb1;
      const int ko = (kb + u) * 32;
#pragma unroll
      for (int i = 0; i < NTILE; ++i) wv[u][i] = ok ? __ldg(reinterpret_cast<const uint4*>(wr[i] + ko)) : zero;
      a0[u] = (ok && v0) ? __ldg(reinterpret_cast<const uint4*>(xa + ko)) : zero;
      a1[u] = (ok && v1) ? __ldg(reinterpret_cast<const uint4*>(xb + ko)) : zero;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t fa[4] = {a0[u].x, a1[u].x, a0[u].y, a1[u].y};
      const uint32_t fb[4] = {a0[u].z, a1[u].z, a0[u].w, a1[u].w};
#pragma unroll
      for (int i = 0; i < NTILE; ++i) {
        mma_16816(acc[i], fa, wv[u][i].x, wv[u][i].y);
        mma_16816(acc[i], fb, wv[u][i].z, wv[u][i].w);
      }
    }
  }
  // ---- reduce the K slices
  __shared__ float red[WARPS][NTILE][4][32];
#pragma unroll
  for (int i = 0; i < NTILE; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) red[warp][i][e][lane] = acc[i][e];
  __syncthreads();
  if (warp != 0) return;
#pragma unroll
  for (int i = 0; i < NTILE; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) s += red[w][i][e][lane];
      acc[i][e] = s;
    }
  // this lane holds rows r0 (e = 0, 1) and r1 (e = 2, 3), columns c0 = n0 + 2t and c0 + 1 of each tile
  const int c0 = n0 + 2 * t;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int row = e < 2 ? r0 : r1, col = c0 + (e & 1);
    if (row >= p.M) continue;
    if (EPI == EPI_PLAIN) {
      float y = acc[0][e];
      if (p.bias) y += __bfloat162float(p.bias[col]);
      p.out[(int64_t)row * p.so + col] = __float2bfloat16_rn(y);
    } else if (EPI == EPI_SWIGLU) {
      float y = acc[0][e], gt = acc[NTILE - 1][e];
      if (p.bias) { y += __bfloat162float(p.bias[col]); gt += __bfloat162float(p.bias[col + half]); }
      y = bf16_round(y); gt = bf16_round(gt);  // fc1's output is a bf16 tensor in the unfused sequence
      const float s = sigmoid_f(gt);
      p.out[(int64_t)row * p.so + col] = __float2bfloat16_rn(y * (p.act == 0 ? gt * s : s));
    } else {
      float u1 = acc[0][e], u2 = acc[NTILE - 1][e];
      if (p.bias) { u1 += __bfloat162float(p.bias[col]); u2 += __bfloat162float(p.bias[col + half]); }
      const __nv_bfloat16 u1b = __float2bfloat16_rn(u1);
      u2 = bf16_round(u2);
      __nv_bfloat16* st = p.state + ((int64_t)row * half + col) * p.ck;
      float c = p.cb ? ld_w(p.cb, p.cw_bf16, col) : 0.f;
      for (int j = 0; j + 1 < p.ck; ++j) {
        const __nv_bfloat16 h = st[j + 1];
        st[j] = h;
        c = fmaf(ld_w(p.cw, p.cw_bf16, col * p.ck + j), __bfloat162float(h), c);
      }
      st[p.ck - 1] = u1b;
      c = fmaf(ld_w(p.cw, p.cw_bf16, col * p.ck + p.ck - 1), __bfloat162float(u1b), c);
      p.out[(int64_t)row * p.so + col] = __float2bfloat16_rn(c * sigmoid_f(c) * u2);
    }
  }
}

}  // namespace

int launch_decode_linear(const void* x, const void* w, const void* bias, void* out, int M, int N, int K, int64_t sx,
                         int64_t so, int epilogue, int act, void* conv_state, const void* conv_weight,
                         const void* conv_bias, int conv_k, int conv_w_dtype, cudaStream_t stream) {
  if (K % 32 != 0 || sx % 8 != 0 || !aligned16(x) || !aligned16(w)) return BASED_ERR_ALIGN;
  const int outputs = epilogue == EPI_PLAIN ? N : N / 2;
  if (outputs % 8 != 0 || (epilogue != EPI_PLAIN && N % 2 != 0)) return BASED_ERR_SHAPE;
  LinParams p{static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
              static_cast<const __nv_bfloat16*>(bias), static_cast<__nv_bfloat16*>(out), M, N, K, sx, so, act,
              static_cast<__nv_bfloat16*>(conv_state), conv_weight, conv_bias, conv_k, conv_w_dtype == BASED_BF16};
  const dim3 grid(outputs / 8, (M + 15) / 16);
  if (epilogue == EPI_PLAIN) decode_linear_kernel<1, EPI_PLAIN><<<grid, WARPS * 32, 0, stream>>>(p);
  else if (epilogue == EPI_SWIGLU) decode_linear_kernel<2, EPI_SWIGLU><<<grid, WARPS * 32, 0, stream>>>(p);
  else if (epilogue == EPI_CONV) decode_linear_kernel<2, EPI_CONV><<<grid, WARPS * 32, 0, stream>>>(p);
  else return BASED_ERR_SHAPE;
  return (int)cudaGetLastError();
}

}  // namespace based
