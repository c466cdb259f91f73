// Shared helpers for the based_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "based_b200.h"

namespace based {

constexpr int kFeatureDim = 16;                 // d
constexpr int kExpandedDim = BASED_EXPANDED_DIM;  // D = 1 + d + d*d

// Constants of the Taylor map for d = 16 (linear_attention.py:62-64):
//   first order  x / d^(1/4)            = x * 0.5
//   second order x_i x_j / (sqrt2 * sqrt d) = x_i x_j * 0.17677669...
constexpr float kC1 = 0.5f;
constexpr float kC2 = 0.17677669529663687f;

struct Strides3 { int64_t b, h, l; };
struct Strides2 { int64_t b, h; };

template <typename T> __device__ __forceinline__ float to_float(T x);
template <> __device__ __forceinline__ float to_float<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// phi(x)[f] for f in [0, 273) from the 16 raw values in x[] (any indexable of float).
template <typename X>
__device__ __forceinline__ float taylor_feature(const X& x, int f) {
  if (f == 0) return 1.0f;
  if (f <= kFeatureDim) return x[f - 1] * kC1;
  const int g = f - 1 - kFeatureDim;
  return x[g >> 4] * x[g & 15] * kC2;
}

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

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Launchers implemented one per .cu file; all return a cudaError_t-compatible int (0 = ok).
int launch_linattn_decode(const void* q, const void* k, const void* v, void* y, void* kv_state, void* k_state,
                          int B, int H, int dv, Strides2 sq, Strides2 sk, Strides2 sv, Strides2 sy,
                          int io_dtype, int state_dtype, float eps, cudaStream_t stream);

int launch_linattn_prefill_simt(const void* q, const void* k, const void* v, void* y, void* kv_state, void* k_state,
                                int B, int H, int L, int dv, Strides3 sq, Strides3 sk, Strides3 sv, Strides3 sy,
                                int io_dtype, int state_dtype, float eps, cudaStream_t stream);

int launch_linattn_prefill_tc(const void* q, const void* k, const void* v, void* y, void* kv_state, void* k_state,
                              int B, int H, int L, int dv, Strides3 sq, Strides3 sk, Strides3 sv, Strides3 sy,
                              int state_dtype, float eps, int nseg, void* scratch, size_t scratch_bytes,
                              cudaStream_t stream);
int launch_linattn_prefill_tc_static(const void* q, const void* k, const void* v, void* y, void* kv_state,
                                     void* k_state, int B, int H, int L, int dv, Strides3 sq, Strides3 sk,
                                     Strides3 sv, Strides3 sy, int state_dtype, float eps, int nseg,
                                     cudaStream_t stream);
int linattn_prefill_tc_auto_segments(int B, int H, int L);
size_t linattn_prefill_tc_scratch_bytes(int B, int H, int L, int dv, int nseg);

int launch_gated_conv_prefill(const void* u1, const void* u2, void* v, void* state, const void* weight,
                              const void* bias, int B, int L, int di, int k, Strides2 s1, Strides2 s2, Strides2 sv,
                              int io_dtype, int w_dtype, cudaStream_t stream);
int launch_gated_conv_step(const void* u1, const void* u2, void* y, void* state, const void* weight, const void* bias,
                           int B, int di, int k, int64_t s1, int64_t s2, int64_t sy, int io_dtype, int w_dtype,
                           cudaStream_t stream);

int launch_add_rmsnorm(const void* x, const void* residual, const void* weight, const void* bias, void* out,
                       void* residual_out, int64_t M, int D, int64_t sx, int64_t sr, int64_t so, int64_t sro, float eps,
                       int io_dtype, int res_dtype, int w_dtype, int round_input, cudaStream_t stream);
int launch_gated_act(const void* y, const void* gate, void* out, int64_t M, int F, int64_t sy, int64_t sg, int64_t so,
                     int act, int io_dtype, cudaStream_t stream);

int launch_rotary_qkv_cache(void* qkv, int B, int L, int H, int hd, int64_t sb, int64_t sl, int64_t s3, int64_t sh,
                            const void* rcos, const void* rsin, void* cache, int64_t cb, int64_t cl,
                            cudaStream_t stream);
int launch_decode_linear(const void* x, const void* w, const void* bias, void* out, int M, int N, int K, int64_t sx,
                         int64_t so, int epilogue, int act, void* conv_state, const void* conv_weight,
                         const void* conv_bias, int conv_k, int conv_w_dtype, cudaStream_t stream);

int launch_tp_outproj_allreduce(const void* const* x, const void* const* w, const void* bias, void* const* out,
                                void* const* workspaces, int M, int N, int K, int64_t sx, int64_t so, int Mmax,
                                int rank, int world, int emulate, cudaStream_t stream);
size_t tp_outproj_workspace_bytes(int world, int Mmax, int N);
int read_tp_status(unsigned int* out, int reset);      // fused output projection + all-reduce

int read_tc_status(unsigned int* out, int reset);      // linear-attention prefill kernel
int read_tc_status_swa(unsigned int* out, int reset);  // sliding-window prefill kernel

int launch_swa_prefill_simt(const void* q, const void* k, const void* v, void* o, int B, int L, int H, int hd,
                            Strides3 sq, Strides3 sk, Strides3 sv, Strides3 so, int window_left, float scale,
                            int io_dtype, cudaStream_t stream);

int launch_swa_prefill_tc(const void* q, const void* k, const void* v, void* o, int B, int L, int H, int hd,
                          Strides3 sq, Strides3 sk, Strides3 sv, Strides3 so, int window_left, float scale,
                          cudaStream_t stream);

int launch_rotary(void* x, int B, int L, int H, Strides3 sx, const void* rcos, const void* rsin, int rotary_dim,
                  const int32_t* offsets, int offset_scalar, int io_dtype, cudaStream_t stream);

int launch_swa_decode(const void* q, const void* k_new, const void* v_new, void* o, void* kv_cache,
                      const int32_t* cache_seqlens, int cache_seqlen_scalar, const void* rotary_cos,
                      const void* rotary_sin, int rotary_dim, int B, int H, int hd, int max_seqlen,
                      Strides2 sq, Strides2 sk, Strides2 sv, Strides2 so, int window_left, float scale,
                      int io_dtype, cudaStream_t stream);

}  // namespace based
