// Recurrent decode step of Taylor linear attention: feature map, rank-1 state update and
// normalised readout in ONE pass over the state (HBM-bound: the state is read once and
// written once).
//
// Replaces TaylorExp.forward on q, k (based/models/mixers/linear_attention.py:67-75, called
// at :139) and LinearAttention.recurrent_forward (:230-251) up to out_proj.
//
// State layout (unchanged from the reference, linear_attention.py:261-266):
//   kv_state [B, H, 1, dv, 273]  feature index fastest, k_state [B, H, 1, 1, 273].
// One row of 273 elements is not 16-byte aligned, but RPG = 16/sizeof(state) consecutive rows
// are exactly 273 sixteen-byte vectors.  A warp owns such a row group: 128-bit coalesced
// loads, FMA, 128-bit stores, and a per-row dot product with phi(q) reduced by shuffles.
#include "common.cuh"

namespace based {
namespace {

// CTA size: 192 threads (three CTAs per SM, 96 registers) when there are many (batch, head) blocks -- measured
// 0.1052 ms against 0.1091 ms at B=256, H=16, fp32 state -- and 256 threads (two per SM) when there are few, where
// one block's latency is what counts (B=16, H=16, bf16 state: 10.6 us against 17.3 us).
constexpr int kTab = 288;     // table length: 273 + wrap-around + padding, multiple of 4
constexpr int kVecPerGroup = kExpandedDim;  // 273 vectors of 16 B per row group
constexpr int kIters = (kVecPerGroup + 31) / 32;  // 9

template <typename ST> struct VecOps;
template <> struct VecOps<float> {
  static constexpr int kVec = 4;
  static __device__ __forceinline__ void unpack(const uint4& r, float* e) {
    e[0] = __uint_as_float(r.x); e[1] = __uint_as_float(r.y);
    e[2] = __uint_as_float(r.z); e[3] = __uint_as_float(r.w);
  }
  static __device__ __forceinline__ uint4 pack(const float* e) {
    return make_uint4(__float_as_uint(e[0]), __float_as_uint(e[1]), __float_as_uint(e[2]), __float_as_uint(e[3]));
  }
  static __device__ __forceinline__ float round(float x) { return x; }
};
template <> struct VecOps<__nv_bfloat16> {
  static constexpr int kVec = 8;
  static __device__ __forceinline__ void unpack(const uint4& r, float* e) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      e[2 * i] = __uint_as_float(w[i] << 16);
      e[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ uint4 pack(const float* e) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // inputs are already rounded to bf16, so truncation is exact
      w[i] = (__float_as_uint(e[2 * i]) >> 16) | (__float_as_uint(e[2 * i + 1]) & 0xffff0000u);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  static __device__ __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
};

template <typename IO, typename ST, int kThreads>
__global__ void __launch_bounds__(kThreads, kThreads <= 192 ? 3 : 2)
linattn_decode_kernel(const IO* __restrict__ q, const IO* __restrict__ k, const IO* __restrict__ v,
                      IO* __restrict__ y, ST* __restrict__ kv_state, ST* __restrict__ k_state,
                      int H, int dv, Strides2 sq, Strides2 sk, Strides2 sv, Strides2 sy, float eps) {
  using VO = VecOps<ST>;
  constexpr int VEC = VO::kVec;
  constexpr int RPG = VEC;  // rows per 16-byte-aligned group
  constexpr int kWarps = kThreads / 32;

  // s_t*[s][i] = phi[(i + s) % 273]: four shifted copies so that phi[f0 .. f0+VEC) can be
  // fetched with aligned 128-bit shared loads whatever f0 mod 4 is.
  __shared__ __align__(16) float s_tq[4][kTab];
  __shared__ __align__(16) float s_tk[4][kTab];
  __shared__ float s_x[2][kFeatureDim];
  __shared__ float s_v[128];
  __shared__ float s_num[128];
  __shared__ float s_den;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int bh = blockIdx.x;
  const int b = bh / H, h = bh - b * H;

  if (tid < kFeatureDim) {
    s_x[0][tid] = to_float(q[b * sq.b + h * sq.h + tid]);
  } else if (tid < 2 * kFeatureDim) {
    s_x[1][tid - kFeatureDim] = to_float(k[b * sk.b + h * sk.h + tid - kFeatureDim]);
  } else if (tid - 2 * kFeatureDim < dv) {
    s_v[tid - 2 * kFeatureDim] = to_float(v[b * sv.b + h * sv.h + tid - 2 * kFeatureDim]);
  }
  __syncthreads();
  for (int idx = tid; idx < 2 * 4 * kTab; idx += kThreads) {
    const int which = idx / (4 * kTab);
    const int rem = idx - which * 4 * kTab;
    const int s = rem / kTab, i = rem - s * kTab;
    int f = i + s;
    if (f >= kExpandedDim) f -= kExpandedDim;
    const float val = taylor_feature(s_x[which], f);
    if (which == 0) s_tq[s][i] = val; else s_tk[s][i] = val;
  }
  __syncthreads();

  // k_state: last warp, scalar accesses (a 273-element row is only element-aligned).
  if (warp == kWarps - 1) {
    ST* ks = k_state + (size_t)bh * kExpandedDim;
    float den = 0.f;
#pragma unroll
    for (int n = 0; n < kIters; ++n) {
      const int f = lane + 32 * n;
      if (f < kExpandedDim) {
        const float nw = VO::round(to_float(ks[f]) + s_tk[0][f]);
        ks[f] = from_float<ST>(nw);
        den += s_tq[0][f] * nw;
      }
    }
    den = warp_sum(den);
    if (lane == 0) s_den = den;
  }

  const int ngroups = dv / RPG;
  for (int g = warp; g < ngroups; g += kWarps) {
    uint4* base = reinterpret_cast<uint4*>(kv_state + ((size_t)bh * dv + (size_t)g * RPG) * kExpandedDim);
    uint4 r[kIters];
#pragma unroll
    for (int n = 0; n < kIters; ++n) {
      const int idx = lane + 32 * n;
      if (idx < kVecPerGroup) r[n] = __ldcs(base + idx);
    }
    float acc[RPG];
#pragma unroll
    for (int rr = 0; rr < RPG; ++rr) acc[rr] = 0.f;
#pragma unroll
    for (int n = 0; n < kIters; ++n) {
      const int idx = lane + 32 * n;
      if (idx < kVecPerGroup) {
        const int e0 = idx * VEC;
        const int row0 = e0 / kExpandedDim;
        const int f0 = e0 - row0 * kExpandedDim;
        const int s = f0 & 3, i = f0 - s;
        float pk[VEC], pq[VEC], e[VEC];
#pragma unroll
        for (int c4 = 0; c4 < VEC / 4; ++c4) {
          const float4 a = *reinterpret_cast<const float4*>(&s_tk[s][i + 4 * c4]);
          const float4 bq = *reinterpret_cast<const float4*>(&s_tq[s][i + 4 * c4]);
          pk[4 * c4] = a.x; pk[4 * c4 + 1] = a.y; pk[4 * c4 + 2] = a.z; pk[4 * c4 + 3] = a.w;
          pq[4 * c4] = bq.x; pq[4 * c4 + 1] = bq.y; pq[4 * c4 + 2] = bq.z; pq[4 * c4 + 3] = bq.w;
        }
        VO::unpack(r[n], e);
        const int rbase = g * RPG + row0;
        const float v0 = s_v[rbase];
        const float v1 = s_v[min(rbase + 1, dv - 1)];
        const int cwrap = kExpandedDim - f0;  // elements c >= cwrap belong to row0 + 1
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int c = 0; c < VEC; ++c) {
          const bool hi = c >= cwrap;
          const float nw = VO::round(fmaf(pk[c], hi ? v1 : v0, e[c]));
          e[c] = nw;
          const float contrib = pq[c] * nw;
          a0 += hi ? 0.f : contrib;
          a1 += hi ? contrib : 0.f;
        }
        __stcs(base + idx, VO::pack(e));
#pragma unroll
        for (int rr = 0; rr < RPG; ++rr) {
          acc[rr] += (row0 == rr) ? a0 : 0.f;
          acc[rr] += (row0 + 1 == rr) ? a1 : 0.f;
        }
      }
    }
#pragma unroll
    for (int rr = 0; rr < RPG; ++rr) {
      const float t = warp_sum(acc[rr]);
      if (lane == 0) s_num[g * RPG + rr] = t;
    }
  }
  __syncthreads();
  if (tid < dv) {
    y[b * sy.b + h * sy.h + tid] = from_float<IO>(s_num[tid] / (s_den + eps));
  }
}

template <typename IO, typename ST>
int launch_typed(const void* q, const void* k, const void* v, void* y, void* kv_state, void* k_state, int B, int H,
                 int dv, Strides2 sq, Strides2 sk, Strides2 sv, Strides2 sy, float eps, cudaStream_t stream) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if ((long long)B * H >= 6LL * sms) {  // at least two waves of three CTAs per SM
    linattn_decode_kernel<IO, ST, 192><<<B * H, 192, 0, stream>>>(
        static_cast<const IO*>(q), static_cast<const IO*>(k), static_cast<const IO*>(v), static_cast<IO*>(y),
        static_cast<ST*>(kv_state), static_cast<ST*>(k_state), H, dv, sq, sk, sv, sy, eps);
  } else {
    linattn_decode_kernel<IO, ST, 256><<<B * H, 256, 0, stream>>>(
        static_cast<const IO*>(q), static_cast<const IO*>(k), static_cast<const IO*>(v), static_cast<IO*>(y),
        static_cast<ST*>(kv_state), static_cast<ST*>(k_state), H, dv, sq, sk, sv, sy, eps);
  }
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

int launch_linattn_decode(const void* q, const void* k, const void* v, void* y, void* kv_state, void* k_state,
                          int B, int H, int dv, Strides2 sq, Strides2 sk, Strides2 sv, Strides2 sy,
                          int io_dtype, int state_dtype, float eps, cudaStream_t stream) {
  using bf16 = __nv_bfloat16;
  if (io_dtype == BASED_BF16 && state_dtype == BASED_F32)
    return launch_typed<bf16, float>(q, k, v, y, kv_state, k_state, B, H, dv, sq, sk, sv, sy, eps, stream);
  if (io_dtype == BASED_BF16 && state_dtype == BASED_BF16)
    return launch_typed<bf16, bf16>(q, k, v, y, kv_state, k_state, B, H, dv, sq, sk, sv, sy, eps, stream);
  if (io_dtype == BASED_F32 && state_dtype == BASED_F32)
    return launch_typed<float, float>(q, k, v, y, kv_state, k_state, B, H, dv, sq, sk, sv, sy, eps, stream);
  if (io_dtype == BASED_F32 && state_dtype == BASED_BF16)
    return launch_typed<float, bf16>(q, k, v, y, kv_state, k_state, B, H, dv, sq, sk, sv, sy, eps, stream);
  return BASED_ERR_DTYPE;
}

}  // namespace based
