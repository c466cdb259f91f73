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
//
// Two kernels.  The staged one (linattn_decode_staged_kernel) is persistent: one CTA per SM
// walks over (batch, head) blocks; the whole [dv, 273] state block of an item (70 KB at dv = 64,
// fp32) is brought into shared memory by ONE bulk async copy (cp.async.bulk, completion on an
// mbarrier), updated in place there, and written back by ONE bulk store, with three blocks in
// rotation per CTA (one being loaded, one computed on, one being stored).  The copies are issued
// by a single thread and need no registers, so ~140 KB per SM are in flight all the time and no
// warp ever waits on a global load.  The direct kernel (linattn_decode_kernel) streams the state
// through registers, one CTA per item; it serves shapes whose blocks do not fit in shared memory
// three (or two) times.
#include "common.cuh"
#include "tcgen05.cuh"

namespace based {

__device__ unsigned int g_decode_status = 0;  // ORed with a code when a bounded wait expires

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
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

template <typename IO, typename ST>
__global__ void __launch_bounds__(kThreads, 2)
linattn_decode_kernel(const IO* __restrict__ q, const IO* __restrict__ k, const IO* __restrict__ v,
                      IO* __restrict__ y, ST* __restrict__ kv_state, ST* __restrict__ k_state,
                      int H, int dv, Strides2 sq, Strides2 sk, Strides2 sv, Strides2 sy, float eps) {
  using VO = VecOps<ST>;
  constexpr int VEC = VO::kVec;
  constexpr int RPG = VEC;  // rows per 16-byte-aligned group

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

// ------------------------------------------------------------------------------------------------
// Staged persistent kernel.  A (batch, head) block is moved in `ppb` pieces of whole row groups
// (35 KB at dv = 64, fp32) so that six pieces rotate through shared memory: one being updated, one
// being stored, the others in flight.  Shared memory: NSTAGE pieces | tables | small vectors | barriers.
struct StagedParams {
  const void *q, *k, *v;
  void *y, *kv_state, *k_state;
  int H, dv, blocks, nstage, ppb, groups_per_piece;
  uint32_t piece_bytes;
  Strides2 sq, sk, sv, sy;
  float eps;
  unsigned int* status;
};

__device__ __forceinline__ void bulk_load(uint32_t dst_saddr, const void* gsrc, uint32_t bytes, uint32_t mbar_saddr) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst_saddr),
               "l"(gsrc), "r"(bytes), "r"(mbar_saddr)
               : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t mbar_saddr, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}\n" ::"r"(mbar_saddr),
               "r"(bytes)
               : "memory");
}
// at most two committed bulk stores still read their shared-memory source
__device__ __forceinline__ void bulk_wait_read_2() { asm volatile("cp.async.bulk.wait_group.read 2;\n" ::: "memory"); }
constexpr int kStoreSlack = 2;  // a stage is reloaded only when two newer stores have been issued after its own

// Measured at B=256, H=16, dv=64, fp32 state: see the launcher.
constexpr int kStagedThreads = 512;  // one CTA per SM: sixteen warps share the in-place update of a piece
constexpr int kStagedWarps = kStagedThreads / 32;
constexpr int kMaxStages = 8;

template <typename IO, typename ST>
__global__ void __launch_bounds__(kStagedThreads, 1) linattn_decode_staged_kernel(const StagedParams p) {
  using VO = VecOps<ST>;
  constexpr int VEC = VO::kVec;
  constexpr int RPG = VEC;
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int dv = p.dv, NS = p.nstage, PPB = p.ppb;
  const uint32_t pc = p.piece_bytes;
  // layout
  uint8_t* tabs = smem + (size_t)NS * pc;
  float (*s_tq)[kTab] = reinterpret_cast<float (*)[kTab]>(tabs);
  float (*s_tk)[kTab] = reinterpret_cast<float (*)[kTab]>(tabs + 4 * kTab * sizeof(float));
  float* s_x = reinterpret_cast<float*>(tabs + 8 * kTab * sizeof(float));  // [2][16]
  float* s_v = s_x + 2 * kFeatureDim;                                      // [128]
  float* s_num = s_v + 128;                                                // [128]
  float* s_den = s_num + 128;                                              // [1] (+3 pad)
  float* s_part = s_den + 4;                                               // [2 * units], units <= 32 * kIters
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_part + 2 * 32 * kIters);  // [kMaxStages] full barriers
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + kMaxStages);
  const uint32_t sb = tc::smem_u32(smem), bar0 = tc::smem_u32(bars);

  const IO* q = static_cast<const IO*>(p.q);
  const IO* k = static_cast<const IO*>(p.k);
  const IO* v = static_cast<const IO*>(p.v);
  IO* y = static_cast<IO*>(p.y);
  uint8_t* kv_bytes = static_cast<uint8_t*>(p.kv_state);
  ST* k_state = static_cast<ST*>(p.k_state);

  if (tid == 0) {
    for (int i = 0; i < NS; ++i) tc::mbar_init(bar0 + 8 * i, 1);
    *abort_flag = 0;
    tc::fence_mbar_init();
  }
  __syncthreads();
  // blocks of this CTA: blockIdx.x, + gridDim.x, ...; its pieces are numbered j = block_index * PPB + piece;
  // piece j uses stage j % NS, phase (j / NS) & 1.  Pieces of a block are contiguous in memory.
  const int first = blockIdx.x, step = gridDim.x;
  const int nblk = first < p.blocks ? (p.blocks - first + step - 1) / step : 0;
  const int npieces = nblk * PPB;
  auto piece_gptr = [&](int j) {
    const int bi = j / PPB, pi = j - bi * PPB;
    return kv_bytes + ((size_t)(first + bi * step) * PPB + pi) * pc;
  };
  auto issue_load = [&](int j) {  // thread 0 only
    const uint32_t bar = bar0 + 8 * (j % NS);
    mbar_expect_tx(bar, pc);
    bulk_load(sb + (j % NS) * pc, piece_gptr(j), pc, bar);
  };
  if (tid == 0)
    for (int j = 0; j < NS - kStoreSlack && j < npieces; ++j) issue_load(j);

  const int units = p.groups_per_piece * kIters;  // one unit = one warp-wide pass over 32 sixteen-byte vectors
  for (int j = 0; j < npieces; ++j) {
    const int bi = j / PPB, pi = j - bi * PPB;
    const int bh = first + bi * step;
    const int b = bh / p.H, h = bh - b * p.H;
    if (pi == 0) {
      // ---- this block's q, k, v, k_state row and the shifted feature tables (while its pieces are in flight)
      if (tid < kFeatureDim) {
        s_x[tid] = to_float(q[b * p.sq.b + h * p.sq.h + tid]);
      } else if (tid < 2 * kFeatureDim) {
        s_x[tid] = to_float(k[b * p.sk.b + h * p.sk.h + tid - kFeatureDim]);
      } else if (tid - 2 * kFeatureDim < dv) {
        s_v[tid - 2 * kFeatureDim] = to_float(v[b * p.sv.b + h * p.sv.h + tid - 2 * kFeatureDim]);
      }
      float ksr[kIters];
      if (warp == kStagedWarps - 1) {
        const ST* ks = k_state + (size_t)bh * kExpandedDim;
#pragma unroll
        for (int n = 0; n < kIters; ++n) {
          const int f = lane + 32 * n;
          ksr[n] = f < kExpandedDim ? to_float(ks[f]) : 0.f;
        }
      }
      __syncthreads();
      for (int idx = tid; idx < 2 * 4 * kTab; idx += kStagedThreads) {
        const int which = idx / (4 * kTab);
        const int rem = idx - which * 4 * kTab;
        const int s = rem / kTab, i = rem - s * kTab;
        int f = i + s;
        if (f >= kExpandedDim) f -= kExpandedDim;
        const float val = taylor_feature(s_x + which * kFeatureDim, f);
        if (which == 0) s_tq[s][i] = val; else s_tk[s][i] = val;
      }
      __syncthreads();
      if (warp == kStagedWarps - 1) {
        ST* ks = k_state + (size_t)bh * kExpandedDim;
        float den = 0.f;
#pragma unroll
        for (int n = 0; n < kIters; ++n) {
          const int f = lane + 32 * n;
          if (f < kExpandedDim) {
            const float nw = VO::round(ksr[n] + s_tk[0][f]);
            ks[f] = from_float<ST>(nw);
            den += s_tq[0][f] * nw;
          }
        }
        den = warp_sum(den);
        if (lane == 0) *s_den = den;
      }
    }
    // ---- the piece has landed?
    tc::mbar_wait_bounded(bar0 + 8 * (j % NS), (uint32_t)((j / NS) & 1), abort_flag, p.status, 0x10000u);
    uint8_t* piece = smem + (size_t)(j % NS) * pc;
    const int row_base = pi * p.groups_per_piece * RPG;  // first row of the piece within the block
#ifdef BASED_DEC_SKIP_COMPUTE
    for (int u = warp; u < 0; u += kStagedWarps) {
#else
    for (int u = warp; u < units; u += kStagedWarps) {
#endif
      const int g = u / kIters, n = u - g * kIters;
      const int idx = lane + 32 * n;
      uint4* base = reinterpret_cast<uint4*>(piece + (size_t)g * RPG * kExpandedDim * sizeof(ST));
      // the 32 vectors of a unit touch at most two rows of the group: r_first and r_first + 1
      const int r_first = (32 * n * VEC) / kExpandedDim;
      float a_lo = 0.f, a_hi = 0.f;
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
        VO::unpack(base[idx], e);
        const int rbase = row_base + g * RPG + row0;
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
        base[idx] = VO::pack(e);
        if (row0 == r_first) { a_lo = a0; a_hi = a1; } else { a_hi = a0; /* a1 is zero: a unit spans two rows */ }
      }
      a_lo = warp_sum(a_lo);
      a_hi = warp_sum(a_hi);
      if (lane == 0) {
        s_part[2 * u] = a_lo;
        s_part[2 * u + 1] = a_hi;
      }
    }
    tc::fence_proxy_async();  // this thread's shared-memory writes, before the bulk store reads them
    __syncthreads();
    // row sums of this piece, partials added in a fixed order (deterministic): row rr of group g gets the
    // low part of the units that start in it and the high part of the units that start in the row before
    if (tid < p.groups_per_piece * RPG) {
      const int g = tid / RPG, rr = tid - g * RPG;
      float t = 0.f;
#pragma unroll
      for (int n = 0; n < kIters; ++n) {
        const int rf = (32 * n * VEC) / kExpandedDim;
        if (rf == rr) t += s_part[2 * (g * kIters + n)];
        if (rf + 1 == rr) t += s_part[2 * (g * kIters + n) + 1];
      }
      s_num[row_base + tid] = t;
    }
    if (tid == 0) {
      tc::bulk_store(piece_gptr(j), sb + (j % NS) * pc, pc);
      tc::bulk_commit();
      // piece j + NS - 2 goes to the stage piece j - 2 was stored from: that store has had two pieces' time to
      // read its source, so this wait does not normally block
      if (j + NS - kStoreSlack < npieces) {
        bulk_wait_read_2();
        issue_load(j + NS - kStoreSlack);
      }
    }
    if (pi == PPB - 1) {
      __syncthreads();  // the row sums of the last piece
      if (tid < dv) y[b * p.sy.b + h * p.sy.h + tid] = from_float<IO>(s_num[tid] / (*s_den + p.eps));
    }
    // the __syncthreads of the next block's set-up order these reads of s_num / s_den before their next writes
  }
  if (tid == 0) tc::bulk_wait_all();
}

// Which kernel serves shapes both can run.  Measured at B=256, H=16, dv=64, fp32 state (CUDA events, 300 steps):
// direct 0.109 ms; staged 0.132 ms with three 70 KB stages, 0.199 ms with six 35 KB stages (the copy pipeline
// alone, update skipped: 0.095 / 0.135 ms).  The direct kernel therefore stays the default.
#ifndef BASED_PREFER_STAGED
#define BASED_PREFER_STAGED 0
#endif
constexpr bool kPreferStaged = BASED_PREFER_STAGED != 0;

template <typename IO, typename ST>
int launch_staged(const void* q, const void* k, const void* v, void* y, void* kv_state, void* k_state, int B, int H,
                  int dv, Strides2 sq, Strides2 sk, Strides2 sv, Strides2 sy, float eps, cudaStream_t stream) {
  constexpr int RPG = VecOps<ST>::kVec;
  const size_t group_bytes = (size_t)RPG * kExpandedDim * sizeof(ST);  // 273 sixteen-byte vectors
  const int ngroups = dv / RPG;
  const size_t extra = 8 * kTab * sizeof(float) + (2 * kFeatureDim + 128 + 128 + 4 + 2 * 32 * kIters) * sizeof(float) +
                       kMaxStages * 8 + 16;
  int dev = 0, smem_max = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return BASED_ERR_IMPL;
  // pieces per block: the fewest that give pieces of at most ~36 KB made of whole row groups
  int ppb = 1;
  while (ppb < ngroups && (ngroups % ppb != 0 || (ngroups / ppb) * group_bytes > 36 * 1024)) ++ppb;
  const int gpp = ngroups / ppb;
  const size_t pc = gpp * group_bytes;
  if (ngroups % ppb != 0 || pc > 64 * 1024 || gpp > 32 || !aligned16(kv_state)) return BASED_ERR_IMPL;
  int nstage = (int)(((size_t)smem_max - extra) / pc);
  if (nstage > kMaxStages) nstage = kMaxStages;
  if (nstage < kStoreSlack + 2) return BASED_ERR_IMPL;
  StagedParams p{q, k, v, y, kv_state, k_state, H, dv, B * H, nstage, ppb, gpp, (uint32_t)pc, sq, sk, sv, sy, eps, nullptr};
  cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p.status), g_decode_status);
  if (e != cudaSuccess) return (int)e;
  const int smem = (int)(nstage * pc + extra);
  e = cudaFuncSetAttribute(linattn_decode_staged_kernel<IO, ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  const int grid = B * H < sms ? B * H : sms;
  linattn_decode_staged_kernel<IO, ST><<<grid, kStagedThreads, smem, stream>>>(p);
  return static_cast<int>(cudaGetLastError());
}

template <typename IO, typename ST>
int launch_typed(const void* q, const void* k, const void* v, void* y, void* kv_state, void* k_state, int B, int H,
                 int dv, Strides2 sq, Strides2 sk, Strides2 sv, Strides2 sy, float eps, cudaStream_t stream) {
  // the staged kernel when the state block fits in shared memory at least twice, and there is more than one
  // block per SM to rotate through; else the direct one
  {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && B * H >= 2 * sms &&
        kPreferStaged) {
      const int rc = launch_staged<IO, ST>(q, k, v, y, kv_state, k_state, B, H, dv, sq, sk, sv, sy, eps, stream);
      if (rc != BASED_ERR_IMPL) return rc;
    }
  }
  linattn_decode_kernel<IO, ST><<<B * H, kThreads, 0, stream>>>(
      static_cast<const IO*>(q), static_cast<const IO*>(k), static_cast<const IO*>(v), static_cast<IO*>(y),
      static_cast<ST*>(kv_state), static_cast<ST*>(k_state), H, dv, sq, sk, sv, sy, eps);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

int read_decode_status(unsigned int* out, int reset) {
  unsigned int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_decode_status, sizeof(v));
  if (e != cudaSuccess) return (int)e;
  if (out) *out = v;
  if (reset && v != 0) {
    v = 0;
    e = cudaMemcpyToSymbol(g_decode_status, &v, sizeof(v));
  }
  return (int)e;
}

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
