// Causal Taylor linear attention over a whole sequence, CUDA-core version with fp32
// arithmetic throughout.  It is the fp32-I/O path (tf32/bf16 tensor-core operands cannot
// hold 1e-4 relative error) and the reference point for the tensor-core kernel.
//
// Replaces LinearAttention.parallel_forward's "quadratic" branch
// (based/models/mixers/linear_attention.py:171-182) and the state hand-off (:220-222) in
// O(L) memory: the sequence is walked in blocks of T tokens; within a block the causal part
// uses phi(q).phi(k) = 1 + s + s^2/2 (s = q.k/4), across blocks the [273 x dv] state is
// carried in registers.
//
// One CTA per (batch, head).  Thread (j, g) with j < dv, g < 4 owns state column j for the
// features [g*69, g*69+69); one extra warp owns k_state.
#include "common.cuh"

namespace based {
namespace {

constexpr int G = 4;         // feature groups
constexpr int FPG = 69;      // features per group (4 * 69 = 276 >= 273)
constexpr int DP = G * FPG;  // padded feature count, 276

template <int T>
struct SmemLayout {
  // all offsets in floats
  int q, k, v, phiq, phik, p, part, den, total;
  __host__ __device__ explicit SmemLayout(int dv) {
    int o = 0;
    q = o; o += T * kFeatureDim;
    k = o; o += T * kFeatureDim;
    v = o; o += T * dv;
    phiq = o; o += DP * T;   // [f][t]
    phik = o; o += DP * T;   // [f][t]
    p = o; o += T * T;       // [t][s]
    part = o; o += G * T * dv;  // [g][t][j]
    den = o; o += T;
    total = o;
  }
};

// T = tokens per block step; MAXT = thread-count bound (sets the register budget).
template <typename IO, typename ST, int T, int MAXT>
__global__ void __launch_bounds__(MAXT)
linattn_prefill_simt_kernel(const IO* __restrict__ q, const IO* __restrict__ k, const IO* __restrict__ v,
                            IO* __restrict__ y, ST* __restrict__ kv_state, ST* __restrict__ k_state, int H, int L,
                            int dv, Strides3 sq, Strides3 sk, Strides3 sv, Strides3 sy, float eps) {
  extern __shared__ __align__(16) float smem[];
  const SmemLayout<T> lay(dv);
  float* s_q = smem + lay.q;
  float* s_k = smem + lay.k;
  float* s_v = smem + lay.v;
  float* s_phiq = smem + lay.phiq;
  float* s_phik = smem + lay.phik;
  float* s_p = smem + lay.p;
  float* s_part = smem + lay.part;
  float* s_den = smem + lay.den;

  const int tid = threadIdx.x, nthreads = blockDim.x;
  const int bh = blockIdx.x, b = bh / H, h = bh - b * H;
  const int nkv = G * dv;                 // threads that own kv_state columns
  const bool is_kv = tid < nkv;
  const bool is_ks = tid >= nkv;          // the trailing warp
  const int j = is_kv ? tid % dv : 0;
  const int g = is_kv ? tid / dv : 0;
  const int lane = tid & 31;

  const IO* qb = q + b * sq.b + h * sq.h;
  const IO* kb = k + b * sk.b + h * sk.h;
  const IO* vb = v + b * sv.b + h * sv.h;
  IO* yb = y + b * sy.b + h * sy.h;

  float S[FPG];
#pragma unroll
  for (int i = 0; i < FPG; ++i) S[i] = 0.f;
  float ks[9];
#pragma unroll
  for (int i = 0; i < 9; ++i) ks[i] = 0.f;

  for (int t0 = 0; t0 < L; t0 += T) {
    const int nt = min(T, L - t0);
    // ---- load the block (zero-filled past the end) ----
    for (int i = tid; i < T * kFeatureDim; i += nthreads) {
      const int t = i >> 4, c = i & 15;
      const bool ok = t < nt;
      s_q[i] = ok ? to_float(qb[(int64_t)(t0 + t) * sq.l + c]) : 0.f;
      s_k[i] = ok ? to_float(kb[(int64_t)(t0 + t) * sk.l + c]) : 0.f;
    }
    for (int i = tid; i < T * dv; i += nthreads) {
      const int t = i / dv, c = i - t * dv;
      s_v[i] = (t < nt) ? to_float(vb[(int64_t)(t0 + t) * sv.l + c]) : 0.f;
    }
    __syncthreads();
    // ---- feature maps (tokens past the end get phi(k) = 0 so they never reach the state) ----
    for (int i = tid; i < DP * T; i += nthreads) {
      const int f = i / T, t = i - f * T;
      float pq = 0.f, pk = 0.f;
      if (f < kExpandedDim && t < nt) {
        pq = taylor_feature(s_q + t * kFeatureDim, f);
        pk = taylor_feature(s_k + t * kFeatureDim, f);
      }
      s_phiq[i] = pq;
      s_phik[i] = pk;
    }
    for (int i = tid; i < T * T; i += nthreads) {
      const int t = i / T, s = i - t * T;
      float p = 0.f;
      if (s <= t && t < nt) {
        float dot = 0.f;
#pragma unroll
        for (int c = 0; c < kFeatureDim; ++c) dot = fmaf(s_q[t * kFeatureDim + c], s_k[s * kFeatureDim + c], dot);
        const float x = dot * 0.25f;
        p = 1.f + x + 0.5f * x * x;
      }
      s_p[i] = p;
    }
    __syncthreads();
    // ---- inter-block readout against the carried state, then state update ----
    if (is_kv) {
      float acc[T];
#pragma unroll
      for (int t = 0; t < T; ++t) acc[t] = 0.f;
      float vr[T];
#pragma unroll
      for (int t = 0; t < T; ++t) vr[t] = s_v[t * dv + j];
      const float4* pq4 = reinterpret_cast<const float4*>(s_phiq + (size_t)g * FPG * T);
      const float4* pk4 = reinterpret_cast<const float4*>(s_phik + (size_t)g * FPG * T);
#pragma unroll
      for (int fi = 0; fi < FPG; ++fi) {
        float s = S[fi];
        float upd = 0.f;
#pragma unroll
        for (int t4 = 0; t4 < T / 4; ++t4) {
          const float4 a = pq4[fi * (T / 4) + t4];
          acc[4 * t4 + 0] = fmaf(a.x, s, acc[4 * t4 + 0]);
          acc[4 * t4 + 1] = fmaf(a.y, s, acc[4 * t4 + 1]);
          acc[4 * t4 + 2] = fmaf(a.z, s, acc[4 * t4 + 2]);
          acc[4 * t4 + 3] = fmaf(a.w, s, acc[4 * t4 + 3]);
          const float4 c = pk4[fi * (T / 4) + t4];
          upd = fmaf(c.x, vr[4 * t4 + 0], upd);
          upd = fmaf(c.y, vr[4 * t4 + 1], upd);
          upd = fmaf(c.z, vr[4 * t4 + 2], upd);
          upd = fmaf(c.w, vr[4 * t4 + 3], upd);
        }
        S[fi] = s + upd;
      }
#pragma unroll
      for (int t = 0; t < T; ++t) s_part[(g * T + t) * dv + j] = acc[t];
    } else if (is_ks) {
      float acc[T];
#pragma unroll
      for (int t = 0; t < T; ++t) acc[t] = 0.f;
#pragma unroll
      for (int n = 0; n < 9; ++n) {
        const int f = lane + 32 * n;  // < 288; rows >= 276 are outside the tables
        if (f < DP) {
          float upd = 0.f;
#pragma unroll
          for (int t = 0; t < T; ++t) {
            acc[t] = fmaf(s_phiq[f * T + t], ks[n], acc[t]);
            upd += s_phik[f * T + t];
          }
          ks[n] += upd;
        }
      }
#pragma unroll
      for (int t = 0; t < T; ++t) {
        const float r = warp_sum(acc[t]);
        if (lane == 0) s_den[t] = r;
      }
    }
    __syncthreads();
    // ---- combine: inter-block partials + causal intra-block part, normalise, store ----
    for (int i = tid; i < nt * dv; i += nthreads) {
      const int t = i / dv, c = i - t * dv;
      float num = 0.f;
#pragma unroll
      for (int gg = 0; gg < G; ++gg) num += s_part[(gg * T + t) * dv + c];
      float den = s_den[t];
      for (int s = 0; s <= t; ++s) {
        const float p = s_p[t * T + s];
        num = fmaf(p, s_v[s * dv + c], num);
        den += p;
      }
      yb[(int64_t)(t0 + t) * sy.l + c] = from_float<IO>(num / (den + eps));
    }
    __syncthreads();
  }

  if (kv_state != nullptr && is_kv) {
    ST* dst = kv_state + ((size_t)bh * dv + j) * kExpandedDim;
#pragma unroll
    for (int fi = 0; fi < FPG; ++fi) {
      const int f = g * FPG + fi;
      if (f < kExpandedDim) dst[f] = from_float<ST>(S[fi]);
    }
  }
  if (k_state != nullptr && is_ks) {
    ST* dst = k_state + (size_t)bh * kExpandedDim;
#pragma unroll
    for (int n = 0; n < 9; ++n) {
      const int f = lane + 32 * n;
      if (f < kExpandedDim) dst[f] = from_float<ST>(ks[n]);
    }
  }
}

template <typename IO, typename ST, int T, int MAXT>
int launch_cfg(const void* q, const void* k, const void* v, void* y, void* kv_state, void* k_state, int B, int H,
               int L, int dv, Strides3 sq, Strides3 sk, Strides3 sv, Strides3 sy, float eps, cudaStream_t stream) {
  const SmemLayout<T> lay(dv);
  const size_t smem = (size_t)lay.total * sizeof(float);
  auto kern = linattn_prefill_simt_kernel<IO, ST, T, MAXT>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  kern<<<B * H, G * dv + 32, smem, stream>>>(static_cast<const IO*>(q), static_cast<const IO*>(k),
                                            static_cast<const IO*>(v), static_cast<IO*>(y),
                                            static_cast<ST*>(kv_state), static_cast<ST*>(k_state), H, L, dv, sq, sk,
                                            sv, sy, eps);
  return (int)cudaGetLastError();
}

template <typename IO, typename ST>
int launch_typed(const void* q, const void* k, const void* v, void* y, void* kv_state, void* k_state, int B, int H,
                 int L, int dv, Strides3 sq, Strides3 sk, Strides3 sv, Strides3 sy, float eps,
                 cudaStream_t stream) {
  if (dv <= 64) return launch_cfg<IO, ST, 16, 288>(q, k, v, y, kv_state, k_state, B, H, L, dv, sq, sk, sv, sy, eps, stream);
  return launch_cfg<IO, ST, 8, 544>(q, k, v, y, kv_state, k_state, B, H, L, dv, sq, sk, sv, sy, eps, stream);
}

}  // namespace

int launch_linattn_prefill_simt(const void* q, const void* k, const void* v, void* y, void* kv_state, void* k_state,
                                int B, int H, int L, int dv, Strides3 sq, Strides3 sk, Strides3 sv, Strides3 sy,
                                int io_dtype, int state_dtype, float eps, cudaStream_t stream) {
  using bf16 = __nv_bfloat16;
  if (io_dtype == BASED_F32 && state_dtype == BASED_F32)
    return launch_typed<float, float>(q, k, v, y, kv_state, k_state, B, H, L, dv, sq, sk, sv, sy, eps, stream);
  if (io_dtype == BASED_BF16 && state_dtype == BASED_F32)
    return launch_typed<bf16, float>(q, k, v, y, kv_state, k_state, B, H, L, dv, sq, sk, sv, sy, eps, stream);
  if (io_dtype == BASED_BF16 && state_dtype == BASED_BF16)
    return launch_typed<bf16, bf16>(q, k, v, y, kv_state, k_state, B, H, L, dv, sq, sk, sv, sy, eps, stream);
  if (io_dtype == BASED_F32 && state_dtype == BASED_BF16)
    return launch_typed<float, bf16>(q, k, v, y, kv_state, k_state, B, H, L, dv, sq, sk, sv, sy, eps, stream);
  return BASED_ERR_DTYPE;
}

}  // namespace based
