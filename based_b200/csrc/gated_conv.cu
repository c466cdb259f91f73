// Gated short causal convolution of the BaseConv mixer: v = silu(conv_k(u1) [+ bias]) * u2.
//
// Replaces ShortConvolution.forward / .step (based/models/mixers/convolution.py:47-109: depthwise
// nn.Conv1d with padding k-1 truncated to the sequence, the [B, d, k] state of the last k inputs)
// together with the silu and the gate of BaseConv.forward (:205-211), which the reference runs as
// separate torch ops (or hands to the external causal_conv1d kernels, :9-13, :76-83).
//
// HBM-bound elementwise work: per (token, channel) one u1 and one u2 element in, one out.  A
// thread owns one 16-byte vector of channels and walks a tile of tokens with the k-1 previous
// inputs in registers, so u1 is read once (plus k-1 halo rows per tile); a warp's accesses are
// 512 contiguous bytes per row.
#include "common.cuh"

namespace based {
namespace {

template <typename T>
struct Vec;  // 16 bytes of T
template <>
struct Vec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float (&x)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&x)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
  }
};
template <>
struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&x)[8]) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      x[2 * i] = __uint_as_float(w[i] << 16);
      x[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
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

__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T>
__device__ __forceinline__ T from_f(float x);
template <>
__device__ __forceinline__ float from_f<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float load_w(const void* w, int w_bf16, int i) {
  return w_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(w)[i]) : static_cast<const float*>(w)[i];
}
__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }

struct ConvParams {
  const void *u1, *u2, *weight, *bias;
  void *v, *state;
  int B, L, di, w_bf16;
  Strides2 s1, s2, sv;  // .b = batch stride, .h = token stride (elements)
};

constexpr int TL = 32;  // tokens per block
constexpr int NTH = 128;

// grid = (ceil(di / (N * NTH)), ceil(L / TL), B)
template <typename T, int K>
__global__ void __launch_bounds__(NTH) gated_conv_prefill_kernel(const ConvParams p) {
  constexpr int N = Vec<T>::N;
  const int ch = (blockIdx.x * NTH + threadIdx.x) * N;
  if (ch >= p.di) return;
  const int b = blockIdx.z, l0 = blockIdx.y * TL, l1 = min(l0 + TL, p.L);
  const T* u1 = static_cast<const T*>(p.u1) + b * p.s1.b + ch;
  const T* u2 = static_cast<const T*>(p.u2) + b * p.s2.b + ch;
  T* v = static_cast<T*>(p.v) + b * p.sv.b + ch;
  float w[N][K], bias[N];
#pragma unroll
  for (int i = 0; i < N; ++i) {
#pragma unroll
    for (int j = 0; j < K; ++j) w[i][j] = load_w(p.weight, p.w_bf16, (ch + i) * K + j);
    bias[i] = p.bias ? load_w(p.bias, p.w_bf16, ch + i) : 0.f;
  }
  // hist[j] = input of token l - (K-1) + j; the halo before the tile (zeros before the sequence)
  float hist[K][N];
#pragma unroll
  for (int j = 0; j < K - 1; ++j) {
    const int l = l0 - (K - 1) + j;
    if (l >= 0) {
      Vec<T>::load(u1 + (int64_t)l * p.s1.h, hist[j]);
    } else {
#pragma unroll
      for (int i = 0; i < N; ++i) hist[j][i] = 0.f;
    }
  }
  constexpr int U = 4;  // tokens per round: their loads are issued together
  for (int l = l0; l < l1; l += U) {
    float a[U][N], g[U][N];
#pragma unroll
    for (int r = 0; r < U; ++r) {
      if (l + r < l1) {
        Vec<T>::load(u1 + (int64_t)(l + r) * p.s1.h, a[r]);
        Vec<T>::load(u2 + (int64_t)(l + r) * p.s2.h, g[r]);
      }
    }
#pragma unroll
    for (int r = 0; r < U; ++r) {
      if (l + r < l1) {
#pragma unroll
        for (int i = 0; i < N; ++i) hist[K - 1][i] = a[r][i];
        float o[N];
#pragma unroll
        for (int i = 0; i < N; ++i) {
          float c = bias[i];
#pragma unroll
          for (int j = 0; j < K; ++j) c = fmaf(w[i][j], hist[j][i], c);
          o[i] = silu(c) * g[r][i];
        }
        Vec<T>::store(v + (int64_t)(l + r) * p.sv.h, o);
#pragma unroll
        for (int j = 0; j < K - 1; ++j)
#pragma unroll
          for (int i = 0; i < N; ++i) hist[j][i] = hist[j + 1][i];
      }
    }
  }
  // the block with the last token leaves the state: the last K inputs, oldest first, zeros when
  // the sequence is shorter than K
  if (p.state != nullptr && l1 == p.L) {
    T* st = static_cast<T*>(p.state) + ((int64_t)b * p.di + ch) * K;
#pragma unroll
    for (int j = 0; j < K; ++j) {
      const int l = p.L - K + j;
      float x[N];
      if (l >= 0) {
        Vec<T>::load(u1 + (int64_t)l * p.s1.h, x);
      } else {
#pragma unroll
        for (int i = 0; i < N; ++i) x[i] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < N; ++i) st[i * K + j] = from_f<T>(x[i]);
    }
  }
}

// One decode step: thread per (batch, channel); the state row of a channel is K contiguous elements.
template <typename T, int K>
__global__ void __launch_bounds__(256) gated_conv_step_kernel(const ConvParams p) {
  const int idx = blockIdx.x * 256 + threadIdx.x;
  if (idx >= p.B * p.di) return;
  const int b = idx / p.di, ch = idx - b * p.di;
  T* st = static_cast<T*>(p.state) + (int64_t)idx * K;
  float h[K];
#pragma unroll
  for (int j = 0; j < K - 1; ++j) h[j] = to_f(st[j + 1]);
  const T x = static_cast<const T*>(p.u1)[b * p.s1.b + ch];  // kept in its own precision, as the reference stores it
  h[K - 1] = to_f(x);
  float c = p.bias ? load_w(p.bias, p.w_bf16, ch) : 0.f;
#pragma unroll
  for (int j = 0; j < K; ++j) c = fmaf(load_w(p.weight, p.w_bf16, ch * K + j), h[j], c);
#pragma unroll
  for (int j = 0; j < K - 1; ++j) st[j] = from_f<T>(h[j]);
  st[K - 1] = x;
  const float g = to_f(static_cast<const T*>(p.u2)[b * p.s2.b + ch]);
  static_cast<T*>(p.v)[b * p.sv.b + ch] = from_f<T>(silu(c) * g);
}

template <typename T>
int launch_prefill_t(const ConvParams& p, int k, cudaStream_t stream) {
  constexpr int N = Vec<T>::N;
  const dim3 grid((p.di / N + NTH - 1) / NTH, (p.L + TL - 1) / TL, p.B);
  switch (k) {
    case 1: gated_conv_prefill_kernel<T, 1><<<grid, NTH, 0, stream>>>(p); break;
    case 2: gated_conv_prefill_kernel<T, 2><<<grid, NTH, 0, stream>>>(p); break;
    case 3: gated_conv_prefill_kernel<T, 3><<<grid, NTH, 0, stream>>>(p); break;
    case 4: gated_conv_prefill_kernel<T, 4><<<grid, NTH, 0, stream>>>(p); break;
    default: return BASED_ERR_SHAPE;
  }
  return (int)cudaGetLastError();
}
template <typename T>
int launch_step_t(const ConvParams& p, int k, cudaStream_t stream) {
  const int grid = (int)(((int64_t)p.B * p.di + 255) / 256);
  switch (k) {
    case 1: gated_conv_step_kernel<T, 1><<<grid, 256, 0, stream>>>(p); break;
    case 2: gated_conv_step_kernel<T, 2><<<grid, 256, 0, stream>>>(p); break;
    case 3: gated_conv_step_kernel<T, 3><<<grid, 256, 0, stream>>>(p); break;
    case 4: gated_conv_step_kernel<T, 4><<<grid, 256, 0, stream>>>(p); break;
    default: return BASED_ERR_SHAPE;
  }
  return (int)cudaGetLastError();
}

}  // namespace

int launch_gated_conv_prefill(const void* u1, const void* u2, void* v, void* state, const void* weight,
                              const void* bias, int B, int L, int di, int k, Strides2 s1, Strides2 s2, Strides2 sv,
                              int io_dtype, int w_dtype, cudaStream_t stream) {
  const int N = io_dtype == BASED_BF16 ? 8 : 4;
  if (di % N != 0) return BASED_ERR_SHAPE;
  if (!aligned16(u1) || !aligned16(u2) || !aligned16(v)) return BASED_ERR_ALIGN;
  const int64_t all[] = {s1.b, s1.h, s2.b, s2.h, sv.b, sv.h};
  for (int64_t s : all)
    if (s % N != 0) return BASED_ERR_ALIGN;  // 16-byte vector accesses on every row
  if (B > 65535 || (L + TL - 1) / TL > 65535) return BASED_ERR_TOO_LARGE;
  ConvParams p{u1, u2, weight, bias, v, state, B, L, di, w_dtype == BASED_BF16, s1, s2, sv};
  return io_dtype == BASED_BF16 ? launch_prefill_t<__nv_bfloat16>(p, k, stream) : launch_prefill_t<float>(p, k, stream);
}

int launch_gated_conv_step(const void* u1, const void* u2, void* y, void* state, const void* weight, const void* bias,
                           int B, int di, int k, int64_t s1, int64_t s2, int64_t sy, int io_dtype, int w_dtype,
                           cudaStream_t stream) {
  ConvParams p{u1, u2, weight, bias, y, state, B, 1, di, w_dtype == BASED_BF16, {s1, 0}, {s2, 0}, {sy, 0}};
  return io_dtype == BASED_BF16 ? launch_step_t<__nv_bfloat16>(p, k, stream) : launch_step_t<float>(p, k, stream);
}

}  // namespace based
