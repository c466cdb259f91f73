// The two elementwise / row-wise steps that sit between the mixers and the GEMMs of a block:
//
//  * residual add + RMSNorm in one pass: z = x + residual; residual_out = z; out = z * rstd(z) * w + b.
//    Replaces the Triton kernel behind RMSNorm.forward / rms_norm_fn as Block.forward and
//    GPTModel.forward call it with prenorm=True (based/ops/triton/layer_norm.py:926-953, semantics
//    restated in rms_norm_ref :74-125; call sites based/models/block.py:134-163 and
//    based/models/gpt.py:696-733).
//  * gated activation of the MLP: out = y * act(gate) with (y, gate) the two halves of fc1's output.
//    Replaces `y, gate = y.chunk(2, dim=-1); y = swiglu(gate, y)` / F.glu in GatedMlp.forward
//    (based/models/mlp.py:141-154), where the reference uses flash-attn's jiterator swiglu.
//
// Both are HBM-bound; 16-byte vector accesses, fp32 arithmetic, one read of every input.
#include "common.cuh"

namespace based {
namespace {

template <typename T>
struct V16;  // 16 bytes of T <-> floats
template <>
struct V16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& v, float (&x)[4]) {
    x[0] = __uint_as_float(v.x); x[1] = __uint_as_float(v.y); x[2] = __uint_as_float(v.z); x[3] = __uint_as_float(v.w);
  }
  static __device__ __forceinline__ void load(const float* p, float (&x)[4]) {
    unpack(*reinterpret_cast<const uint4*>(p), x);
  }
  static __device__ __forceinline__ void store(float* p, const float (&x)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
  }
};
template <>
struct V16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& v, float (&x)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      x[2 * i] = __uint_as_float(w[i] << 16);
      x[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  }
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&x)[8]) {
    unpack(*reinterpret_cast<const uint4*>(p), x);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&x)[8]) {
    uint4 v;
    uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = v;
  }
};

// 8 consecutive values of a tensor of runtime dtype (two 16-byte loads when it is fp32)
__device__ __forceinline__ void load8(const void* base, int bf16, int64_t idx, float (&x)[8]) {
  if (bf16) {
    V16<__nv_bfloat16>::load(static_cast<const __nv_bfloat16*>(base) + idx, x);
  } else {
    float a[4], b[4];
    V16<float>::load(static_cast<const float*>(base) + idx, a);
    V16<float>::load(static_cast<const float*>(base) + idx + 4, b);
#pragma unroll
    for (int i = 0; i < 4; ++i) { x[i] = a[i]; x[4 + i] = b[i]; }
  }
}
__device__ __forceinline__ void store8(void* base, int bf16, int64_t idx, const float (&x)[8]) {
  if (bf16) {
    V16<__nv_bfloat16>::store(static_cast<__nv_bfloat16*>(base) + idx, x);
  } else {
    const float a[4] = {x[0], x[1], x[2], x[3]}, b[4] = {x[4], x[5], x[6], x[7]};
    V16<float>::store(static_cast<float*>(base) + idx, a);
    V16<float>::store(static_cast<float*>(base) + idx + 4, b);
  }
}

struct NormParams {
  const void *x, *residual, *weight, *bias;
  void *out, *residual_out;
  int64_t M, sx, sr, so, sro;  // rows and row strides (elements)
  int D, io_bf16, res_bf16, w_bf16, round_input;
  float eps;
};

constexpr int NORM_THREADS = 128;

// One row per block; thread t owns the 8-value groups t, t + 128, ... (VPT of them, in registers
// between the reduction and the scaling, so the row is read once).
template <int VPT>
__global__ void __launch_bounds__(NORM_THREADS) add_rmsnorm_kernel(const NormParams p) {
  const int64_t row = blockIdx.x;
  const int ngroups = p.D >> 3;
  float z[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int g = threadIdx.x + v * NORM_THREADS;
    if (g < ngroups) {
      load8(p.x, p.io_bf16, row * p.sx + 8 * g, z[v]);
      if (p.residual) {
        float r[8];
        load8(p.residual, p.res_bf16, row * p.sr + 8 * g, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) z[v][i] += r[i];
      }
      if (p.residual_out) {
        store8(p.residual_out, p.res_bf16, row * p.sro + 8 * g, z[v]);
        if (p.res_bf16) {  // the norm sees the residual stream as it is stored
#pragma unroll
          for (int i = 0; i < 8; ++i) z[v][i] = __bfloat162float(__float2bfloat16_rn(z[v][i]));
        }
      }
      if (p.round_input && p.io_bf16) {  // the norm sees z cast to the activation dtype
#pragma unroll
        for (int i = 0; i < 8; ++i) z[v][i] = __bfloat162float(__float2bfloat16_rn(z[v][i]));
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) ss = fmaf(z[v][i], z[v][i], ss);
    }
  }
  __shared__ float part[NORM_THREADS / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < NORM_THREADS / 32; ++w) tot += part[w];
  const float rstd = rsqrtf(tot / (float)p.D + p.eps);
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int g = threadIdx.x + v * NORM_THREADS;
    if (g < ngroups) {
      float w[8], o[8];
      load8(p.weight, p.w_bf16, 8 * g, w);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = z[v][i] * rstd * w[i];
      if (p.bias) {
        load8(p.bias, p.w_bf16, 8 * g, w);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] += w[i];
      }
      store8(p.out, p.io_bf16, row * p.so + 8 * g, o);
    }
  }
}

struct ActParams {
  const void *y, *gate;
  void* out;
  int64_t M, sy, sg, so;
  int F, act;
};

__device__ __forceinline__ float act_fn(float g, int act) {
  const float s = __fdividef(1.0f, 1.0f + __expf(-g));  // sigmoid
  return act == 0 ? g * s : s;                            // 0: silu, 1: sigmoid
}

// One row per block; thread t owns the 16-byte vectors t, t + 128, ... of the row (VPT of them): a
// warp's accesses are contiguous, all loads of a thread are issued before any arithmetic.
template <typename T, int VPT>
__global__ void __launch_bounds__(NORM_THREADS) gated_act_kernel(const ActParams p) {
  constexpr int N = V16<T>::N;
  const int nvec = p.F / N;
  const int64_t row = blockIdx.x;
  const T* y = static_cast<const T*>(p.y) + row * p.sy;
  const T* gate = static_cast<const T*>(p.gate) + row * p.sg;
  T* out = static_cast<T*>(p.out) + row * p.so;
  uint4 a[VPT], g[VPT];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int c = threadIdx.x + v * NORM_THREADS;
    if (c < nvec) {
      a[v] = *reinterpret_cast<const uint4*>(y + c * N);
      g[v] = *reinterpret_cast<const uint4*>(gate + c * N);
    }
  }
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int c = threadIdx.x + v * NORM_THREADS;
    if (c < nvec) {
      float x[N], h[N];
      V16<T>::unpack(a[v], x);
      V16<T>::unpack(g[v], h);
#pragma unroll
      for (int e = 0; e < N; ++e) x[e] *= act_fn(h[e], p.act);
      V16<T>::store(out + c * N, x);
    }
  }
}

}  // namespace

int launch_add_rmsnorm(const void* x, const void* residual, const void* weight, const void* bias, void* out,
                       void* residual_out, int64_t M, int D, int64_t sx, int64_t sr, int64_t so, int64_t sro, float eps,
                       int io_dtype, int res_dtype, int w_dtype, int round_input, cudaStream_t stream) {
  if (D % 8 != 0 || D > 8 * NORM_THREADS * 8) return BASED_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(out) || !aligned16(weight) || (residual && !aligned16(residual)) ||
      (residual_out && !aligned16(residual_out)) || (bias && !aligned16(bias)))
    return BASED_ERR_ALIGN;
  if (sx % 8 || so % 8 || (residual && sr % 8) || (residual_out && sro % 8)) return BASED_ERR_ALIGN;
  if (M > 2147483647LL) return BASED_ERR_TOO_LARGE;
  NormParams p{x, residual, weight, bias, out, residual_out, M, sx, sr, so, sro, D,
               io_dtype == BASED_BF16, res_dtype == BASED_BF16, w_dtype == BASED_BF16, round_input != 0, eps};
  const int groups = D / 8, vpt = (groups + NORM_THREADS - 1) / NORM_THREADS;
  const unsigned grid = (unsigned)M;
  if (vpt <= 1) add_rmsnorm_kernel<1><<<grid, NORM_THREADS, 0, stream>>>(p);
  else if (vpt <= 2) add_rmsnorm_kernel<2><<<grid, NORM_THREADS, 0, stream>>>(p);
  else if (vpt <= 4) add_rmsnorm_kernel<4><<<grid, NORM_THREADS, 0, stream>>>(p);
  else add_rmsnorm_kernel<8><<<grid, NORM_THREADS, 0, stream>>>(p);
  return (int)cudaGetLastError();
}

int launch_gated_act(const void* y, const void* gate, void* out, int64_t M, int F, int64_t sy, int64_t sg, int64_t so,
                     int act, int io_dtype, cudaStream_t stream) {
  const int N = io_dtype == BASED_BF16 ? 8 : 4;
  if (F % N != 0) return BASED_ERR_SHAPE;
  if (!aligned16(y) || !aligned16(gate) || !aligned16(out) || sy % N || sg % N || so % N) return BASED_ERR_ALIGN;
  if (M > 2147483647LL) return BASED_ERR_TOO_LARGE;
  const int nvec = F / N, vpt = (nvec + NORM_THREADS - 1) / NORM_THREADS;
  if (vpt > 16) return BASED_ERR_SHAPE;  // F up to 16384 (bf16) / 8192 (fp32)
  ActParams p{y, gate, out, M, sy, sg, so, F, act};
  const unsigned grid = (unsigned)M;
#define BASED_LAUNCH_ACT(T)                                                                      \
  do {                                                                                           \
    if (vpt <= 1) gated_act_kernel<T, 1><<<grid, NORM_THREADS, 0, stream>>>(p);                  \
    else if (vpt <= 2) gated_act_kernel<T, 2><<<grid, NORM_THREADS, 0, stream>>>(p);             \
    else if (vpt <= 4) gated_act_kernel<T, 4><<<grid, NORM_THREADS, 0, stream>>>(p);             \
    else if (vpt <= 8) gated_act_kernel<T, 8><<<grid, NORM_THREADS, 0, stream>>>(p);             \
    else gated_act_kernel<T, 16><<<grid, NORM_THREADS, 0, stream>>>(p);                          \
  } while (0)
  if (io_dtype == BASED_BF16) BASED_LAUNCH_ACT(__nv_bfloat16);
  else BASED_LAUNCH_ACT(float);
#undef BASED_LAUNCH_ACT
  return (int)cudaGetLastError();
}

}  // namespace based
