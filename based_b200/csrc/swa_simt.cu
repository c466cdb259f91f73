// Sliding-window causal softmax attention on CUDA cores: the prefill kernel used for fp32 I/O
// and as the reference point of the tensor-core kernel, and the decode-step kernel (RoPE on
// q/k at the new position, append to the KV cache, attend over <= window_left+1 cached keys),
// which is latency/bandwidth-bound and needs no tensor cores.
//
// Semantics follow the reference's calls into flash-attn:
//   prefill  based/models/mixers/slide_attention.py:100-106, :206-213
//            (causal=True, window_size=(window_left, 0): keys [i - window_left, i])
//   decode   slide_attention.py:414-427, :471-481 (append at cache_seqlens, then attend)
//   RoPE     based/ops/triton/rotary.py:75-105 (non-interleaved halves, fp32 math)
#include "common.cuh"

namespace based {
namespace {

constexpr int kWarpsPerBlock = 4;
constexpr int kMaxHd = 128;
constexpr int kMaxKeysPerLane = 9;  // supports window_left + 1 <= 288

// One warp per query.  Lane l scores keys lo + l, lo + l + 32, ...; then the lanes switch to
// owning output channels for the weighted sum of value rows.
template <typename IO>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
swa_prefill_simt_kernel(const IO* __restrict__ q, const IO* __restrict__ k, const IO* __restrict__ v,
                        IO* __restrict__ o, int L, int H, int hd, Strides3 sq, Strides3 sk, Strides3 sv,
                        Strides3 so, int window_left, float scale) {
  __shared__ float s_q[kWarpsPerBlock][kMaxHd];
  __shared__ float s_p[kWarpsPerBlock][kMaxKeysPerLane * 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i = blockIdx.x * kWarpsPerBlock + warp;  // query position
  const int h = blockIdx.y, b = blockIdx.z;
  if (i >= L) return;
  const IO* qp = q + b * sq.b + (int64_t)i * sq.l + h * sq.h;
  for (int c = lane; c < hd; c += 32) s_q[warp][c] = to_float(qp[c]);
  __syncwarp();
  const int lo = max(0, i - window_left);
  const int nk = i - lo + 1;
  float sc[kMaxKeysPerLane];
  float m = -INFINITY;
#pragma unroll
  for (int n = 0; n < kMaxKeysPerLane; ++n) {
    const int jj = lane + 32 * n;
    sc[n] = -INFINITY;
    if (jj < nk) {
      const IO* kp = k + b * sk.b + (int64_t)(lo + jj) * sk.l + h * sk.h;
      float dot = 0.f;
      for (int c = 0; c < hd; ++c) dot = fmaf(s_q[warp][c], to_float(kp[c]), dot);
      sc[n] = dot * scale;
      m = fmaxf(m, sc[n]);
    }
  }
  m = warp_max(m);
  float sum = 0.f;
#pragma unroll
  for (int n = 0; n < kMaxKeysPerLane; ++n) {
    const int jj = lane + 32 * n;
    if (jj < nk) {
      const float p = __expf(sc[n] - m);
      s_p[warp][jj] = p;
      sum += p;
    }
  }
  sum = warp_sum(sum);
  __syncwarp();
  const float inv = 1.f / sum;
  for (int c = lane; c < hd; c += 32) {
    float acc = 0.f;
    for (int jj = 0; jj < nk; ++jj) {
      acc = fmaf(s_p[warp][jj], to_float(v[b * sv.b + (int64_t)(lo + jj) * sv.l + h * sv.h + c]), acc);
    }
    o[b * so.b + (int64_t)i * so.l + h * so.h + c] = from_float<IO>(acc * inv);
  }
}

// dot product of a cached key row with the query held in shared memory (fp32); 16-byte loads
__device__ __forceinline__ float dot_row(const __nv_bfloat16* kc, const float* sq, int hd) {
  float dot = 0.f;
  for (int c = 0; c < hd; c += 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(kc + c);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      dot = fmaf(sq[c + 2 * i], __uint_as_float(w[i] << 16), dot);
      dot = fmaf(sq[c + 2 * i + 1], __uint_as_float(w[i] & 0xFFFF0000u), dot);
    }
  }
  return dot;
}
__device__ __forceinline__ float dot_row(const float* kc, const float* sq, int hd) {
  float dot = 0.f;
  for (int c = 0; c < hd; c += 4) {
    const float4 v = *reinterpret_cast<const float4*>(kc + c);
    dot = fmaf(sq[c], v.x, dot);
    dot = fmaf(sq[c + 1], v.y, dot);
    dot = fmaf(sq[c + 2], v.z, dot);
    dot = fmaf(sq[c + 3], v.w, dot);
  }
  return dot;
}
// two adjacent value columns of a cached row
__device__ __forceinline__ float2 load2(const __nv_bfloat16* p) {
  const uint32_t w = *reinterpret_cast<const uint32_t*>(p);
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}
__device__ __forceinline__ float2 load2(const float* p) { return *reinterpret_cast<const float2*>(p); }

// One warp per (batch, head).  hd is a multiple of 8 and the cache 16-byte aligned (checked by the launcher).
template <typename IO>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
swa_decode_kernel(const IO* __restrict__ q, const IO* __restrict__ k_new, const IO* __restrict__ v_new,
                  IO* __restrict__ o, IO* __restrict__ kv_cache, const int32_t* __restrict__ cache_seqlens,
                  int cache_seqlen_scalar, const IO* __restrict__ rcos, const IO* __restrict__ rsin, int rotary_dim,
                  int BH, int H, int hd, int max_seqlen, Strides2 sq, Strides2 sk, Strides2 sv, Strides2 so,
                  int window_left, float scale) {
  __shared__ float s_q[kWarpsPerBlock][kMaxHd];
  __shared__ float s_k[kWarpsPerBlock][kMaxHd];
  __shared__ float s_p[kWarpsPerBlock][kMaxKeysPerLane * 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.x * kWarpsPerBlock + warp;
  if (bh >= BH) return;
  const int b = bh / H, h = bh - b * H;
  const int pos = cache_seqlens ? cache_seqlens[b] : cache_seqlen_scalar;
  if (pos < 0 || pos >= max_seqlen) return;  // nothing sensible to do; the host validates the scalar case
  const IO* qp = q + b * sq.b + h * sq.h;
  const IO* kp = k_new + b * sk.b + h * sk.h;
  const IO* vp = v_new + b * sv.b + h * sv.h;
  for (int c = lane; c < hd; c += 32) {
    s_q[warp][c] = to_float(qp[c]);
    s_k[warp][c] = to_float(kp[c]);
  }
  __syncwarp();
  const size_t row = (size_t)2 * H * hd;  // elements per cached position
  IO* cache_b = kv_cache + (size_t)b * max_seqlen * row;
  IO* knew = cache_b + (size_t)pos * row + (size_t)h * hd;
  IO* vnew = knew + (size_t)H * hd;
  // RoPE in fp32, result rounded to the I/O dtype like the reference kernel's store.
  const int half = rcos ? rotary_dim / 2 : 0;
  float qr[kMaxHd / 32], kr[kMaxHd / 32];
#pragma unroll
  for (int n = 0; n < kMaxHd / 32; ++n) {
    const int c = lane + 32 * n;
    if (c < hd) {
      float qv = s_q[warp][c], kv = s_k[warp][c];
      if (c < 2 * half) {
        const int cc = c < half ? c : c - half;
        const float cs = to_float(rcos[(size_t)pos * half + cc]);
        const float sn = to_float(rsin[(size_t)pos * half + cc]);
        if (c < half) {
          qv = s_q[warp][c] * cs - s_q[warp][c + half] * sn;
          kv = s_k[warp][c] * cs - s_k[warp][c + half] * sn;
        } else {
          qv = s_q[warp][c - half] * sn + s_q[warp][c] * cs;
          kv = s_k[warp][c - half] * sn + s_k[warp][c] * cs;
        }
      }
      qr[n] = to_float(from_float<IO>(qv));
      kr[n] = to_float(from_float<IO>(kv));
    }
  }
  __syncwarp();
#pragma unroll
  for (int n = 0; n < kMaxHd / 32; ++n) {
    const int c = lane + 32 * n;
    if (c < hd) {
      s_q[warp][c] = qr[n];
      knew[c] = from_float<IO>(kr[n]);
      vnew[c] = vp[c];
    }
  }
  __syncwarp();  // orders this warp's cache writes before its reads below
  const int lo = max(0, pos - window_left);
  const int nk = pos - lo + 1;
  float sc[kMaxKeysPerLane];
  float m = -INFINITY;
#pragma unroll
  for (int n = 0; n < kMaxKeysPerLane; ++n) {
    const int jj = lane + 32 * n;
    sc[n] = -INFINITY;
    if (jj < nk) {
      const IO* kc = cache_b + (size_t)(lo + jj) * row + (size_t)h * hd;
      sc[n] = dot_row(kc, s_q[warp], hd) * scale;
      m = fmaxf(m, sc[n]);
    }
  }
  m = warp_max(m);
  float sum = 0.f;
#pragma unroll
  for (int n = 0; n < kMaxKeysPerLane; ++n) {
    const int jj = lane + 32 * n;
    if (jj < nk) {
      const float p = __expf(sc[n] - m);
      s_p[warp][jj] = p;
      sum += p;
    }
  }
  sum = warp_sum(sum);
  __syncwarp();
  const float inv = 1.f / sum;
  // a lane owns two adjacent value columns; sixteen (then four) rows per round so that their loads overlap
  for (int c = 2 * lane; c < hd; c += 64) {
    const IO* vc = cache_b + (size_t)lo * row + (size_t)(H + h) * hd + c;
    float a0 = 0.f, a1 = 0.f;
    int jj = 0;
    for (; jj + 16 <= nk; jj += 16) {  // sixteen rows in flight: the loop is latency-bound
      float2 x[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) x[u] = load2(vc + (size_t)(jj + u) * row);
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        a0 = fmaf(s_p[warp][jj + u], x[u].x, a0);
        a1 = fmaf(s_p[warp][jj + u], x[u].y, a1);
      }
    }
    for (; jj + 4 <= nk; jj += 4) {
      float2 x[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) x[u] = load2(vc + (size_t)(jj + u) * row);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        a0 = fmaf(s_p[warp][jj + u], x[u].x, a0);
        a1 = fmaf(s_p[warp][jj + u], x[u].y, a1);
      }
    }
    for (; jj < nk; ++jj) {
      const float2 x = load2(vc + (size_t)jj * row);
      a0 = fmaf(s_p[warp][jj], x.x, a0);
      a1 = fmaf(s_p[warp][jj], x.y, a1);
    }
    IO* op = o + b * so.b + h * so.h + c;
    op[0] = from_float<IO>(a0 * inv);
    op[1] = from_float<IO>(a1 * inv);
  }
}

// In-place non-interleaved RoPE on x [B, L, H, hd]: one thread per rotated pair.
template <typename IO>
__global__ void rotary_kernel(IO* __restrict__ x, int L, int H, Strides3 sx, const IO* __restrict__ rcos,
                              const IO* __restrict__ rsin, int half, const int32_t* __restrict__ offsets,
                              int offset_scalar, long long total) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int c = (int)(idx % half);
  long long r = idx / half;
  const int h = (int)(r % H); r /= H;
  const int l = (int)(r % L);
  const int b = (int)(r / L);
  const int pos = l + (offsets ? offsets[b] : offset_scalar);
  IO* px = x + b * sx.b + (int64_t)l * sx.l + h * sx.h;
  const float cs = to_float(rcos[(size_t)pos * half + c]), sn = to_float(rsin[(size_t)pos * half + c]);
  const float x0 = to_float(px[c]), x1 = to_float(px[c + half]);
  px[c] = from_float<IO>(x0 * cs - x1 * sn);
  px[c + half] = from_float<IO>(x0 * sn + x1 * cs);
}

// The same with 16-byte accesses: one thread per group of 8 (bf16) / 4 (fp32) rotated pairs.
template <typename IO>
__global__ void rotary_vec_kernel(IO* __restrict__ x, int L, int H, Strides3 sx, const IO* __restrict__ rcos,
                                  const IO* __restrict__ rsin, int half, const int32_t* __restrict__ offsets,
                                  int offset_scalar, long long total) {
  constexpr int N = 16 / sizeof(IO);
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int groups = half / N;
  const int c = (int)(idx % groups) * N;
  long long r = idx / groups;
  const int h = (int)(r % H); r /= H;
  const int l = (int)(r % L);
  const int b = (int)(r / L);
  const int pos = l + (offsets ? offsets[b] : offset_scalar);
  IO* px = x + b * sx.b + (int64_t)l * sx.l + h * sx.h + c;
  union V { uint4 u; IO e[N]; } x0, x1, cs, sn;
  x0.u = *reinterpret_cast<const uint4*>(px);
  x1.u = *reinterpret_cast<const uint4*>(px + half);
  cs.u = __ldg(reinterpret_cast<const uint4*>(rcos + (size_t)pos * half + c));
  sn.u = __ldg(reinterpret_cast<const uint4*>(rsin + (size_t)pos * half + c));
#pragma unroll
  for (int i = 0; i < N; ++i) {
    const float a = to_float(x0.e[i]), bb = to_float(x1.e[i]), cc = to_float(cs.e[i]), ss = to_float(sn.e[i]);
    x0.e[i] = from_float<IO>(a * cc - bb * ss);
    x1.e[i] = from_float<IO>(a * ss + bb * cc);
  }
  *reinterpret_cast<uint4*>(px) = x0.u;
  *reinterpret_cast<uint4*>(px + half) = x1.u;
}

// Prompt pass of the sliding-window mixer on the packed projection qkv [B, L, 3, H, hd] (bf16): q and k rotated in
// place (whole head, non-interleaved), and the rotated k and v written to the layer's cache [*, max_seqlen, 2, H, hd]
// in the same pass.  One thread per 16-byte piece: q and k pieces carry a rotated pair of 8-element groups, v pieces
// a plain copy.  Pieces per head: hd/16 (q) + hd/16 (k) + hd/8 (v) = hd/4.
__global__ void __launch_bounds__(256)
rotary_qkv_cache_kernel(__nv_bfloat16* __restrict__ qkv, int L, int H, int hd, int64_t sb, int64_t sl, int64_t s3,
                        int64_t sh, const __nv_bfloat16* __restrict__ rcos, const __nv_bfloat16* __restrict__ rsin,
                        __nv_bfloat16* __restrict__ cache, int64_t cb, int64_t cl, long long total) {
  using IO = __nv_bfloat16;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int half = hd / 2, gq = half / 8, per_head = 2 * gq + hd / 8;
  const int piece = (int)(idx % per_head);
  long long r = idx / per_head;
  const int h = (int)(r % H); r /= H;
  const int l = (int)(r % L);
  const int b = (int)(r / L);
  IO* base = qkv + b * sb + (int64_t)l * sl + h * sh;
  IO* crow = cache + b * cb + (int64_t)l * cl + (int64_t)h * hd;  // k part; the v part is H * hd further
  if (piece >= 2 * gq) {  // v: copy
    const int c = (piece - 2 * gq) * 8;
    *reinterpret_cast<uint4*>(crow + (int64_t)H * hd + c) = *reinterpret_cast<const uint4*>(base + 2 * s3 + c);
    return;
  }
  const int part = piece / gq, c = (piece - part * gq) * 8;  // part 0 = q, 1 = k
  IO* px = base + part * s3 + c;
  union V { uint4 u; IO e[8]; } x0, x1, cs, sn;
  x0.u = *reinterpret_cast<const uint4*>(px);
  x1.u = *reinterpret_cast<const uint4*>(px + half);
  cs.u = __ldg(reinterpret_cast<const uint4*>(rcos + (size_t)l * half + c));
  sn.u = __ldg(reinterpret_cast<const uint4*>(rsin + (size_t)l * half + c));
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float a = to_float(x0.e[i]), bb = to_float(x1.e[i]), cc = to_float(cs.e[i]), ss = to_float(sn.e[i]);
    x0.e[i] = from_float<IO>(a * cc - bb * ss);
    x1.e[i] = from_float<IO>(a * ss + bb * cc);
  }
  *reinterpret_cast<uint4*>(px) = x0.u;
  *reinterpret_cast<uint4*>(px + half) = x1.u;
  if (part == 1) {
    *reinterpret_cast<uint4*>(crow + c) = x0.u;
    *reinterpret_cast<uint4*>(crow + c + half) = x1.u;
  }
}

}  // namespace

int launch_rotary_qkv_cache(void* qkv, int B, int L, int H, int hd, int64_t sb, int64_t sl, int64_t s3, int64_t sh,
                            const void* rcos, const void* rsin, void* cache, int64_t cb, int64_t cl,
                            cudaStream_t stream) {
  if (hd % 16 != 0) return BASED_ERR_SHAPE;
  const int64_t strides[] = {sb, sl, s3, sh, cb, cl};
  for (int64_t s : strides)
    if (s % 8 != 0) return BASED_ERR_ALIGN;
  if (!aligned16(qkv) || !aligned16(rcos) || !aligned16(rsin) || !aligned16(cache)) return BASED_ERR_ALIGN;
  const long long total = (long long)B * L * H * (hd / 4);
  if (total == 0) return 0;
  const long long blocks = (total + 255) / 256;
  if (blocks > 2147483647LL) return BASED_ERR_TOO_LARGE;
  rotary_qkv_cache_kernel<<<(unsigned)blocks, 256, 0, stream>>>(
      static_cast<__nv_bfloat16*>(qkv), L, H, hd, sb, sl, s3, sh, static_cast<const __nv_bfloat16*>(rcos),
      static_cast<const __nv_bfloat16*>(rsin), static_cast<__nv_bfloat16*>(cache), cb, cl, total);
  return (int)cudaGetLastError();
}

int launch_rotary(void* x, int B, int L, int H, Strides3 sx, const void* rcos, const void* rsin, int rotary_dim,
                  const int32_t* offsets, int offset_scalar, int io_dtype, cudaStream_t stream) {
  const int half = rotary_dim / 2;
  const int threads = 256;
  if (io_dtype != BASED_BF16 && io_dtype != BASED_F32) return BASED_ERR_DTYPE;
  {
    // 16-byte path when every access it makes is aligned
    const int N = io_dtype == BASED_BF16 ? 8 : 4;
    if (half % N == 0 && sx.b % N == 0 && sx.l % N == 0 && sx.h % N == 0 && aligned16(x) && aligned16(rcos) &&
        aligned16(rsin)) {
      const long long total = (long long)B * L * H * (half / N);
      if (total == 0) return 0;
      const long long blocks = (total + threads - 1) / threads;
      if (blocks > 2147483647LL) return BASED_ERR_TOO_LARGE;
      if (io_dtype == BASED_BF16) {
        using T = __nv_bfloat16;
        rotary_vec_kernel<T><<<(unsigned)blocks, threads, 0, stream>>>(
            static_cast<T*>(x), L, H, sx, static_cast<const T*>(rcos), static_cast<const T*>(rsin), half, offsets,
            offset_scalar, total);
      } else {
        rotary_vec_kernel<float><<<(unsigned)blocks, threads, 0, stream>>>(
            static_cast<float*>(x), L, H, sx, static_cast<const float*>(rcos), static_cast<const float*>(rsin), half,
            offsets, offset_scalar, total);
      }
      return (int)cudaGetLastError();
    }
  }
  const long long total = (long long)B * L * H * half;
  if (total == 0) return 0;
  const long long blocks = (total + threads - 1) / threads;
  if (blocks > 2147483647LL) return BASED_ERR_TOO_LARGE;
  if (io_dtype == BASED_BF16) {
    using T = __nv_bfloat16;
    rotary_kernel<T><<<(unsigned)blocks, threads, 0, stream>>>(static_cast<T*>(x), L, H, sx, static_cast<const T*>(rcos),
                                                              static_cast<const T*>(rsin), half, offsets,
                                                              offset_scalar, total);
  } else if (io_dtype == BASED_F32) {
    rotary_kernel<float><<<(unsigned)blocks, threads, 0, stream>>>(
        static_cast<float*>(x), L, H, sx, static_cast<const float*>(rcos), static_cast<const float*>(rsin), half,
        offsets, offset_scalar, total);
  } else {
    return BASED_ERR_DTYPE;
  }
  return (int)cudaGetLastError();
}

int launch_swa_prefill_simt(const void* q, const void* k, const void* v, void* o, int B, int L, int H, int hd,
                            Strides3 sq, Strides3 sk, Strides3 sv, Strides3 so, int window_left, float scale,
                            int io_dtype, cudaStream_t stream) {
  if (window_left + 1 > kMaxKeysPerLane * 32) return BASED_ERR_TOO_LARGE;
  const dim3 grid((L + kWarpsPerBlock - 1) / kWarpsPerBlock, H, B);
  if (io_dtype == BASED_BF16) {
    using T = __nv_bfloat16;
    swa_prefill_simt_kernel<T><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v), static_cast<T*>(o), L, H, hd,
        sq, sk, sv, so, window_left, scale);
  } else if (io_dtype == BASED_F32) {
    swa_prefill_simt_kernel<float><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        static_cast<const float*>(q), static_cast<const float*>(k), static_cast<const float*>(v),
        static_cast<float*>(o), L, H, hd, sq, sk, sv, so, window_left, scale);
  } else {
    return BASED_ERR_DTYPE;
  }
  return (int)cudaGetLastError();
}

int launch_swa_decode(const void* q, const void* k_new, const void* v_new, void* o, void* kv_cache,
                      const int32_t* cache_seqlens, int cache_seqlen_scalar, const void* rotary_cos,
                      const void* rotary_sin, int rotary_dim, int B, int H, int hd, int max_seqlen, Strides2 sq,
                      Strides2 sk, Strides2 sv, Strides2 so, int window_left, float scale, int io_dtype,
                      cudaStream_t stream) {
  if (window_left + 1 > kMaxKeysPerLane * 32) return BASED_ERR_TOO_LARGE;
  if (!aligned16(kv_cache) || hd % 8 != 0) return BASED_ERR_ALIGN;  // 16-byte reads of cached rows
  const int BH = B * H;
  const int grid = (BH + kWarpsPerBlock - 1) / kWarpsPerBlock;
  if (io_dtype == BASED_BF16) {
    using T = __nv_bfloat16;
    swa_decode_kernel<T><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        static_cast<const T*>(q), static_cast<const T*>(k_new), static_cast<const T*>(v_new), static_cast<T*>(o),
        static_cast<T*>(kv_cache), cache_seqlens, cache_seqlen_scalar, static_cast<const T*>(rotary_cos),
        static_cast<const T*>(rotary_sin), rotary_dim, BH, H, hd, max_seqlen, sq, sk, sv, so, window_left, scale);
  } else if (io_dtype == BASED_F32) {
    swa_decode_kernel<float><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        static_cast<const float*>(q), static_cast<const float*>(k_new), static_cast<const float*>(v_new),
        static_cast<float*>(o), static_cast<float*>(kv_cache), cache_seqlens, cache_seqlen_scalar,
        static_cast<const float*>(rotary_cos), static_cast<const float*>(rotary_sin), rotary_dim, BH, H, hd,
        max_seqlen, sq, sk, sv, so, window_left, scale);
  } else {
    return BASED_ERR_DTYPE;
  }
  return (int)cudaGetLastError();
}

}  // namespace based
