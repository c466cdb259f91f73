// Gated short causal convolution of the BaseConv mixer: v = silu(conv_k(u1) [+ bias]) * u2.
//
// Replaces ShortConvolution.forward / .step (based/models/mixers/convolution.py:47-109: depthwise
// nn.Conv1d with padding k-1 truncated to the sequence, the [B, d, k] state of the last k inputs)
// together with the silu and the gate of BaseConv.forward (:205-211), which the reference runs as
// separate torch ops (or hands to the external causal_conv1d kernels, :9-13, :76-83).
//
// HBM-bound elementwise work: per (token, channel) one u1 and one u2 element in, one out.  A
// thread owns three consecutive tokens of one 16-byte vector of channels; a warp's accesses are
// 512 contiguous bytes per row, and the k-1 rows before a thread's first token are rows its
// neighbour loads as well (L1/L2 hits).
#include "common.cuh"

namespace based {
namespace {

template <typename T>
struct Vec;  // 16 bytes of T
template <>
struct Vec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& v, float (&x)[4]) {
    x[0] = __uint_as_float(v.x); x[1] = __uint_as_float(v.y); x[2] = __uint_as_float(v.z); x[3] = __uint_as_float(v.w);
  }
  static __device__ __forceinline__ void store(float* p, const float (&x)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
  }
};
template <>
struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& v, float (&x)[8]) {
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
__device__ __forceinline__ float silu(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

struct ConvParams {
  const void *u1, *u2, *weight, *bias;
  void *v, *state;
  int B, L, di, w_bf16;
  Strides2 s1, s2, sv;  // .b = batch stride, .h = token stride (elements)
};

constexpr int TT = 3;     // consecutive tokens per thread (measured: 3 -> 0.79 of HBM peak, 4 -> 0.76, 5 -> 0.68)
constexpr int TY = 2;     // token groups per block (threadIdx.y)
constexpr int NTH = 128;  // channel vectors per block (threadIdx.x)

// The N * K taps of N consecutive channels, [channel][tap] as the weight tensor stores them.
template <int N, int K>
__device__ __forceinline__ void load_taps(const void* weight, int w_bf16, int ch, float (&w)[N][K]) {
  if (w_bf16 && (N * K * 2) % 16 == 0) {  // whole 16-byte vectors (ch is a multiple of N)
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(weight) + (int64_t)ch * K);
    float flat[N * K];
#pragma unroll
    for (int q = 0; q < N * K / 8; ++q) {
      const uint4 x = __ldg(src + q);
      const uint32_t r[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        flat[8 * q + 2 * e] = __uint_as_float(r[e] << 16);
        flat[8 * q + 2 * e + 1] = __uint_as_float(r[e] & 0xFFFF0000u);
      }
    }
#pragma unroll
    for (int i = 0; i < N; ++i)
#pragma unroll
      for (int j = 0; j < K; ++j) w[i][j] = flat[i * K + j];
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i)
#pragma unroll
      for (int j = 0; j < K; ++j) w[i][j] = load_w(weight, w_bf16, (ch + i) * K + j);
  }
}

// One thread per (TT consecutive tokens, 16-byte vector of channels).  All its loads -- the K-1
// rows before its first token, TT rows of u1, TT rows of u2 -- are issued before any arithmetic
// and stay packed in registers until used, so a thread keeps 2 TT + K - 1 16-byte loads in flight
// with a small register count; there is no loop-carried state.
// grid = (ceil(di / (N * NTH)), ceil(L / (TT * TY)), B), block = (NTH, TY)
template <typename T, int K>
__global__ void __launch_bounds__(NTH * TY, 3) gated_conv_prefill_kernel(const ConvParams p) {
  constexpr int N = Vec<T>::N;
  const int ch = (blockIdx.x * NTH + threadIdx.x) * N;
  const int l0 = (blockIdx.y * TY + threadIdx.y) * TT, b = blockIdx.z;
  if (ch >= p.di || l0 >= p.L) return;
  const T* u1 = static_cast<const T*>(p.u1) + b * p.s1.b + ch;
  const T* u2 = static_cast<const T*>(p.u2) + b * p.s2.b + ch;
  // rows[r] = packed input of token l0 - (K-1) + r (zeros outside the sequence); gate[t] of token l0 + t
  uint4 rows[K - 1 + TT], gate[TT];
#pragma unroll
  for (int r = 0; r < K - 1 + TT; ++r) {
    const int l = l0 - (K - 1) + r;
    rows[r] = (l >= 0 && l < p.L) ? *reinterpret_cast<const uint4*>(u1 + (int64_t)l * p.s1.h) : make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int t = 0; t < TT; ++t)
    gate[t] = (l0 + t < p.L) ? *reinterpret_cast<const uint4*>(u2 + (int64_t)(l0 + t) * p.s2.h) : make_uint4(0, 0, 0, 0);
  float w[N][K], bias[N];
  load_taps<N, K>(p.weight, p.w_bf16, ch, w);
#pragma unroll
  for (int i = 0; i < N; ++i) bias[i] = p.bias ? load_w(p.bias, p.w_bf16, ch + i) : 0.f;
  T* v = static_cast<T*>(p.v) + b * p.sv.b + ch;
#pragma unroll
  for (int t = 0; t < TT; ++t) {
    if (l0 + t < p.L) {
      float c[N], x[N];
#pragma unroll
      for (int i = 0; i < N; ++i) c[i] = bias[i];
#pragma unroll
      for (int j = 0; j < K; ++j) {
        Vec<T>::unpack(rows[t + j], x);
#pragma unroll
        for (int i = 0; i < N; ++i) c[i] = fmaf(w[i][j], x[i], c[i]);
      }
      Vec<T>::unpack(gate[t], x);
#pragma unroll
      for (int i = 0; i < N; ++i) c[i] = silu(c[i]) * x[i];
      Vec<T>::store(v + (int64_t)(l0 + t) * p.sv.h, c);
    }
  }
  // the thread that holds the last token leaves the state: the last K inputs, oldest first
  // (zeros when L < K); rows[] already has them
  if (p.state != nullptr && l0 + TT >= p.L) {
    T* st = static_cast<T*>(p.state) + ((int64_t)b * p.di + ch) * K;
    const int tl = p.L - 1 - l0;  // this thread's index of the last token, 0 .. TT-1
#pragma unroll
    for (int t = 0; t < TT; ++t) {
      if (t == tl) {
#pragma unroll
        for (int j = 0; j < K; ++j) {
          float x[N];
          Vec<T>::unpack(rows[t + j], x);
#pragma unroll
          for (int i = 0; i < N; ++i) st[i * K + j] = from_f<T>(x[i]);
        }
      }
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
  const dim3 grid((p.di / N + NTH - 1) / NTH, (p.L + TT * TY - 1) / (TT * TY), p.B), block(NTH, TY);
  switch (k) {
    case 1: gated_conv_prefill_kernel<T, 1><<<grid, block, 0, stream>>>(p); break;
    case 2: gated_conv_prefill_kernel<T, 2><<<grid, block, 0, stream>>>(p); break;
    case 3: gated_conv_prefill_kernel<T, 3><<<grid, block, 0, stream>>>(p); break;
    case 4: gated_conv_prefill_kernel<T, 4><<<grid, block, 0, stream>>>(p); break;
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
  if (B > 65535 || (L + TT * TY - 1) / (TT * TY) > 65535) return BASED_ERR_TOO_LARGE;
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
