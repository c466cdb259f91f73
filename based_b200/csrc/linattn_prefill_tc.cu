// Causal Taylor linear attention over a whole sequence on the sm_100a tensor cores
// (tcgen05.mma, accumulators in TMEM), bf16 I/O.
//
// Replaces LinearAttention.parallel_forward's "quadratic" branch
// (based/models/mixers/linear_attention.py:171-182) and the state hand-off (:220-222), the job
// the reference hands to causal_dot_product (train/csrc/causal_dot_prod/causal_attention_cuda.cu)
// or to external fused kernels (linear_attention.py:154-167, :199-215).
//
// One CTA per (batch, head) walks the sequence in chunks of 128 tokens.  Per chunk:
//   S   = Q K^T                          (M128 N128 K16)      -> TMEM
//   P   = causal(1 + S/4 + (S/4)^2/2)    CUDA cores, S is phi(q).phi(k) in closed form
//   O   = P V'                           (M128 N=NV K128)      A = P in TMEM (bf16)
//   O  += phi'(Q) State                  (M128 N=NV K160)      A = phi'(Q) in TMEM, B = bf16 state in smem
//   St += V'^T phi'(K)                   (M128 N160 K128)      St = state^T, fp32 in TMEM for the whole sequence
// where V' = [V | 1 | 0...] (NV = dv + 16 columns): the ones column makes column dv of O the
// normaliser and row dv of St the k_state, so no separate reductions are needed.
//
// phi' is the SYMMETRY-PACKED Taylor map: 1, x_i/2, and the 136 products x_i x_j (i <= j) with
// weight 1/(4 sqrt2) on the diagonal and 1/4 off it, 153 features padded to 160.  phi'(q).phi'(k)
// equals phi(q).phi(k) of the 273-feature map exactly; the 273-wide reference layout is restored
// only when the final state is written.
#include "common.cuh"
#include "tcgen05.cuh"

#include <type_traits>

namespace based {

__device__ unsigned int g_tc_status = 0;  // ORed with a code when a bounded wait expires

namespace {

using namespace tc;

constexpr int C = 128;     // tokens per chunk
constexpr int DR = 160;    // packed + padded feature count
constexpr int NT = 256;    // threads per CTA

// shared memory map (bytes)
constexpr int SM_Q = 0;                    // 2 stages x 4096   K-major [128 tok x 16]
constexpr int SM_K = 8192;                 // 2 stages x 4096
constexpr int SM_V = 16384;                // 2 stages x 32768  MN-major [16 groups of 8 cols][128 tok][16 B]
constexpr int SM_PHIK = SM_V + 65536;      // 40960             MN-major [20 groups of 8 feats][128 tok][16 B]
constexpr int SM_STB = SM_PHIK + 40960;    // 40960             K-major  [20 k-units][128 rows][16 B]
constexpr int SM_BAR = SM_STB + 40960;     // barriers, TMEM base, abort flag
constexpr int SM_TOTAL = SM_BAR + 64;
constexpr int STAGE_STRIDE_F = 164;        // floats per row of the final fp32 staging (conflict-free 16 B stores)
static_assert(SM_V + C * STAGE_STRIDE_F * 4 <= SM_BAR, "final staging must fit below the barriers");

// TMEM columns (32-bit each), 512 allocated
constexpr uint32_t TM_ST = 0;     // state^T accumulator: lanes = V' column, 160 feature columns, fp32
constexpr uint32_t TM_S = 160;    // S fp32 (128 cols), overwritten in place by P bf16 (64 cols)
constexpr uint32_t TM_O = 288;    // O accumulator, NV <= 128 columns
constexpr uint32_t TM_PQ = 416;   // phi'(Q) bf16, 80 columns
constexpr uint32_t TM_COLS = 512;

__host__ __device__ constexpr int pair_row(int p) {
  int a = 0;
  while (p >= 16 - a) { p -= 16 - a; ++a; }
  return a;
}
__host__ __device__ constexpr int pair_col(int p) {
  int a = 0;
  while (p >= 16 - a) { p -= 16 - a; ++a; }
  return a + p;
}

// Packed feature F (0..159) of x[16].
template <int F>
__device__ __forceinline__ float packed_feature(const float (&x)[16]) {
  if constexpr (F == 0) {
    return 1.0f;
  } else if constexpr (F <= 16) {
    return x[F - 1] * kC1;
  } else if constexpr (F < 153) {
    constexpr int a = pair_row(F - 17), b = pair_col(F - 17);
    if constexpr (a == b) return x[a] * x[a] * kC2;
    else return x[a] * x[b] * 0.25f;
  } else {
    return 0.0f;
  }
}
// Features 8G .. 8G+7 as four packed bf16x2 words.
template <int G>
__device__ __forceinline__ void packed_group(const float (&x)[16], uint32_t* out) {
  out[0] = pack_bf16(packed_feature<8 * G + 0>(x), packed_feature<8 * G + 1>(x));
  out[1] = pack_bf16(packed_feature<8 * G + 2>(x), packed_feature<8 * G + 3>(x));
  out[2] = pack_bf16(packed_feature<8 * G + 4>(x), packed_feature<8 * G + 5>(x));
  out[3] = pack_bf16(packed_feature<8 * G + 6>(x), packed_feature<8 * G + 7>(x));
}

template <int G0, int G1, typename F>
__device__ __forceinline__ void static_for(F&& f) {
  if constexpr (G0 < G1) {
    f(std::integral_constant<int, G0>{});
    static_for<G0 + 1, G1>(f);
  }
}

// Index of full feature f (0..272) in the packed vector, and whether it is an off-diagonal
// second-order term (whose packed value is sqrt2 times the full-map value).
__device__ __forceinline__ int packed_index(int f, bool& offdiag) {
  offdiag = false;
  if (f < 17) return f;
  const int g = f - 17, i = g >> 4, j = g & 15;
  const int a = min(i, j), b = max(i, j);
  offdiag = a != b;
  return 17 + a * 16 - (a * (a - 1)) / 2 + (b - a);
}

__device__ __forceinline__ void unpack8(const uint4& u, float* x) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    x[2 * i] = __uint_as_float(w[i] << 16);
    x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

struct Params {
  const __nv_bfloat16 *q, *k, *v;
  __nv_bfloat16* y;
  void *kv_state, *k_state;
  int H, L, dv, state_bf16;
  Strides3 sq, sk, sv, sy;
  float eps;
  unsigned int* status;
};

__global__ void __launch_bounds__(NT, 1) linattn_prefill_tc_kernel(const Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sb = smem_u32(smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int qd = warp & 3;   // TMEM lane quadrant this warp can reach
  const int hf = warp >> 2;  // which half of the column work this warp takes
  const int t = qd * 32 + lane;  // token within the chunk == TMEM lane
  const int bh = blockIdx.x, b = bh / p.H, h = bh - b * p.H;
  const int dv = p.dv, NV = dv + 16, L = p.L;

  const uint32_t bar_s = sb + SM_BAR, bar_o = sb + SM_BAR + 8, bar_st = sb + SM_BAR + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM_BAR + 24);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM_BAR + 28);

  const __nv_bfloat16* qb = p.q + b * p.sq.b + h * p.sq.h;
  const __nv_bfloat16* kb = p.k + b * p.sk.b + h * p.sk.h;
  const __nv_bfloat16* vb = p.v + b * p.sv.b + h * p.sv.h;
  __nv_bfloat16* yb = p.y + b * p.sy.b + h * p.sy.h;

  // ------------------------------------------------------------------ set-up
  if (tid == 0) {
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    mbar_init(bar_st, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  __syncwarp();
  if (warp == 0) tmem_alloc(smem_u32(tmem_slot), TM_COLS);
  // V' stages: zero everything once; the column groups above dv stay constant for the whole
  // kernel (group dv/8 = [1,0,...,0] per token, the rest 0), the groups below are refilled.
  for (int i = tid; i < 65536 / 16; i += NT) reinterpret_cast<uint4*>(smem + SM_V)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();
  if (tid < C) {
    const uint32_t off = (dv >> 3) * 2048 + (tid >> 3) * 128 + (tid & 7) * 16;
    const uint4 one = make_uint4(0x00003F80u, 0, 0, 0);  // bf16 1.0 in element 0
    *reinterpret_cast<uint4*>(smem + SM_V + off) = one;
    *reinterpret_cast<uint4*>(smem + SM_V + 32768 + off) = one;
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tlane = tmem + ((uint32_t)(qd * 32) << 16);  // this warp's lane window, column 0

  const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
  const uint32_t idesc_o_pv = make_idesc_bf16(128, NV, 0, 1);   // A = P (TMEM), B = V' MN-major
  const uint32_t idesc_o_st = make_idesc_bf16(128, NV, 0, 0);   // A = phi'(Q) (TMEM), B = state K-major
  const uint32_t idesc_st = make_idesc_bf16(128, DR, 1, 1);     // A = V'^T MN-major, B = phi'(K) MN-major

  const int nchunks = (L + C - 1) / C;
  const int vpieces = C * (dv >> 3);

  auto issue_loads = [&](int c, int stage) {
    const int tok0 = c * C;
    {
      const int tk = tid >> 1, half = tid & 1;
      const bool ok = tok0 + tk < L;
      const int64_t row = ok ? tok0 + tk : 0;
      const uint32_t off = stage * 4096 + (tk >> 3) * 256 + half * 128 + (tk & 7) * 16;
      cp_async16(sb + SM_Q + off, qb + row * p.sq.l + half * 8, ok);
      cp_async16(sb + SM_K + off, kb + row * p.sk.l + half * 8, ok);
    }
    const int gpt = dv >> 3;  // 16-byte pieces per token
    for (int i = tid; i < vpieces; i += NT) {
      const int tk = i / gpt, g = i - tk * gpt;
      const bool ok = tok0 + tk < L;
      const int64_t row = ok ? tok0 + tk : 0;
      cp_async16(sb + SM_V + stage * 32768 + g * 2048 + (tk >> 3) * 128 + (tk & 7) * 16, vb + row * p.sv.l + g * 8,
                 ok);
    }
  };

  issue_loads(0, 0);
  cp_async_commit();

  for (int c = 0; c < nchunks; ++c) {
    const int stage = c & 1;
    const uint32_t par = c & 1;
    const bool last = c + 1 == nchunks;
    const bool valid = c * C + t < L;

    // (A) chunk c's q/k/v have landed; everything written by the previous iteration
    //     (bf16 state in smem, TMEM reads) is ordered before this chunk's MMAs.
    cp_async_wait_all();
    fence_proxy_async();
    fence_before_sync();
    __syncthreads();
    fence_after_sync();

    if (tid == 0) {
      const uint64_t da = make_smem_desc(sb + SM_Q + stage * 4096, 128, 256);
      const uint64_t db = make_smem_desc(sb + SM_K + stage * 4096, 128, 256);
      mma_ss(tmem + TM_S, da, db, idesc_s, 0);
      mma_commit(bar_s);
    }
    __syncwarp();
    if (!last) issue_loads(c + 1, stage ^ 1);
    cp_async_commit();

    // ---- feature expansion: half 0 -> phi'(Q) into TMEM, half 1 -> phi'(K) into smem ----
    {
      float x[16];
      const uint8_t* src = smem + (hf == 0 ? SM_Q : SM_K) + stage * 4096 + (t >> 3) * 256 + (t & 7) * 16;
      unpack8(*reinterpret_cast<const uint4*>(src), x);
      unpack8(*reinterpret_cast<const uint4*>(src + 128), x + 8);
      if (hf == 0) {
        static_for<0, 10>([&](auto G2) {
          uint32_t r[8];
          packed_group<2 * decltype(G2)::value>(x, r);
          packed_group<2 * decltype(G2)::value + 1>(x, r + 4);
          tmem_st8(tlane + TM_PQ + 8 * decltype(G2)::value, r);
        });
      } else {
        uint8_t* dst = smem + SM_PHIK + (t >> 3) * 128 + (t & 7) * 16;
        static_for<0, 20>([&](auto G) {
          uint32_t r[4];
          packed_group<decltype(G)::value>(x, r);
          // tokens past the end contribute nothing to the state
          const uint4 val = valid ? make_uint4(r[0], r[1], r[2], r[3]) : make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(dst + decltype(G)::value * 2048) = val;
        });
      }
    }

    // ---- P = causal(1 + x + x^2/2), x = S/4: read S, block barrier, overwrite in place ----
    mbar_wait_bounded(bar_s, par, abort_flag, p.status, 1u);
    fence_after_sync();
    uint32_t sreg[2][32];
    tmem_ld32(tlane + TM_S + hf * 64, sreg[0]);
    tmem_ld32(tlane + TM_S + hf * 64 + 32, sreg[1]);
    tmem_ld_wait();
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
#pragma unroll
    for (int piece = 0; piece < 2; ++piece) {
      uint32_t pk[16];
      const int s0 = hf * 64 + piece * 32;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float pv[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float xx = __uint_as_float(sreg[piece][2 * i + e]) * 0.25f;
          const float val = fmaf(xx, fmaf(xx, 0.5f, 1.0f), 1.0f);
          pv[e] = (s0 + 2 * i + e <= t) ? val : 0.0f;
        }
        pk[i] = pack_bf16(pv[0], pv[1]);
      }
      tmem_st16(tlane + TM_S + (s0 >> 1), pk);
    }
    tmem_st_wait();
    fence_proxy_async();  // phi'(K) smem writes -> async proxy
    fence_before_sync();
    __syncthreads();

    // ---- MMAs of the chunk ----
    if (tid == 0) {
      fence_after_sync();
      const uint32_t vbase = sb + SM_V + stage * 32768;
#pragma unroll 1
      for (int j = 0; j < C / 16; ++j)  // O = P V'
        mma_ts(tmem + TM_O, tmem + TM_S + 8 * j, make_smem_desc(vbase + j * 256, 128, 2048), idesc_o_pv, j > 0);
      if (c > 0) {
#pragma unroll 1
        for (int j = 0; j < DR / 16; ++j)  // O += phi'(Q) State
          mma_ts(tmem + TM_O, tmem + TM_PQ + 8 * j, make_smem_desc(sb + SM_STB + j * 4096, 2048, 128), idesc_o_st,
                 1);
      }
      mma_commit(bar_o);
#pragma unroll 1
      for (int j = 0; j < C / 16; ++j)  // St += V'^T phi'(K)
        mma_ss(tmem + TM_ST, make_smem_desc(vbase + j * 256, 128, 2048),
               make_smem_desc(sb + SM_PHIK + j * 256, 128, 2048), idesc_st, (c > 0 || j > 0) ? 1u : 0u);
      mma_commit(bar_st);
    }
    __syncwarp();

    // ---- epilogue: y = O[:, :dv] / (O[:, dv] + eps) ----
    mbar_wait_bounded(bar_o, par, abort_flag, p.status, 2u);
    fence_after_sync();
    {
      uint32_t dreg;
      tmem_ld1(tlane + TM_O + dv, dreg);
      tmem_ld_wait();
      const float inv = 1.0f / (__uint_as_float(dreg) + p.eps);
      const int j0 = hf * (dv >> 1);
      __nv_bfloat16* yrow = yb + (int64_t)(c * C + t) * p.sy.l + j0;
      for (int i = 0; i < (dv >> 4); ++i) {
        uint32_t r[8];
        tmem_ld8(tlane + TM_O + j0 + 8 * i, r);
        tmem_ld_wait();
        if (valid) {
          uint4 o;
          o.x = pack_bf16(__uint_as_float(r[0]) * inv, __uint_as_float(r[1]) * inv);
          o.y = pack_bf16(__uint_as_float(r[2]) * inv, __uint_as_float(r[3]) * inv);
          o.z = pack_bf16(__uint_as_float(r[4]) * inv, __uint_as_float(r[5]) * inv);
          o.w = pack_bf16(__uint_as_float(r[6]) * inv, __uint_as_float(r[7]) * inv);
          *reinterpret_cast<uint4*>(yrow + 8 * i) = o;
        }
      }
    }

    // ---- state: fp32 TMEM -> bf16 smem operand for the next chunk, or fp32 staging at the end ----
    mbar_wait_bounded(bar_st, par, abort_flag, p.status, 4u);
    fence_after_sync();
    if (!last) {
#pragma unroll 1
      for (int i = 0; i < 5; ++i) {
        uint32_t r[16];
        const int col = hf * 80 + 16 * i;
        tmem_ld16(tlane + TM_ST + col, r);
        tmem_ld_wait();
        uint4 lo, hi;
        lo.x = pack_bf16(__uint_as_float(r[0]), __uint_as_float(r[1]));
        lo.y = pack_bf16(__uint_as_float(r[2]), __uint_as_float(r[3]));
        lo.z = pack_bf16(__uint_as_float(r[4]), __uint_as_float(r[5]));
        lo.w = pack_bf16(__uint_as_float(r[6]), __uint_as_float(r[7]));
        hi.x = pack_bf16(__uint_as_float(r[8]), __uint_as_float(r[9]));
        hi.y = pack_bf16(__uint_as_float(r[10]), __uint_as_float(r[11]));
        hi.z = pack_bf16(__uint_as_float(r[12]), __uint_as_float(r[13]));
        hi.w = pack_bf16(__uint_as_float(r[14]), __uint_as_float(r[15]));
        uint8_t* dst = smem + SM_STB + (col >> 3) * 2048 + t * 16;
        *reinterpret_cast<uint4*>(dst) = lo;
        *reinterpret_cast<uint4*>(dst + 2048) = hi;
      }
    } else if (p.kv_state != nullptr) {
      float* stg = reinterpret_cast<float*>(smem + SM_V) + t * STAGE_STRIDE_F;
#pragma unroll 1
      for (int i = 0; i < 5; ++i) {
        uint32_t r[16];
        const int col = hf * 80 + 16 * i;
        tmem_ld16(tlane + TM_ST + col, r);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 4; ++e)
          *reinterpret_cast<uint4*>(stg + col + 4 * e) = make_uint4(r[4 * e], r[4 * e + 1], r[4 * e + 2], r[4 * e + 3]);
      }
    }
  }

  // ------------------------------------------------------------------ final state, reference layout
  fence_before_sync();
  __syncthreads();
  if (p.kv_state != nullptr) {
    const float* stg = reinterpret_cast<const float*>(smem + SM_V);
    const int total = (dv + 1) * kExpandedDim;
    for (int e = tid; e < total; e += NT) {
      const int n = e / kExpandedDim, f = e - n * kExpandedDim;
      bool offdiag;
      const int idx = packed_index(f, offdiag);
      float val = stg[n * STAGE_STRIDE_F + idx];
      if (offdiag) val *= 0.70710678118654752f;
      if (n < dv) {
        const size_t o = (size_t)bh * dv * kExpandedDim + e;
        if (p.state_bf16) static_cast<__nv_bfloat16*>(p.kv_state)[o] = __float2bfloat16_rn(val);
        else static_cast<float*>(p.kv_state)[o] = val;
      } else {
        const size_t o = (size_t)bh * kExpandedDim + f;
        if (p.state_bf16) static_cast<__nv_bfloat16*>(p.k_state)[o] = __float2bfloat16_rn(val);
        else static_cast<float*>(p.k_state)[o] = val;
      }
    }
  }
  __syncthreads();
  if (warp == 0) {
    fence_after_sync();
    tmem_dealloc(tmem, TM_COLS);
  }
}

}  // namespace

int read_tc_status(unsigned int* out, int reset) {
  unsigned int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(v));
  if (e != cudaSuccess) return (int)e;
  if (out) *out = v;
  if (reset && v != 0) {
    v = 0;
    e = cudaMemcpyToSymbol(g_tc_status, &v, sizeof(v));
  }
  return (int)e;
}

int launch_linattn_prefill_tc(const void* q, const void* k, const void* v, void* y, void* kv_state, void* k_state,
                              int B, int H, int L, int dv, Strides3 sq, Strides3 sk, Strides3 sv, Strides3 sy,
                              int state_dtype, float eps, cudaStream_t stream) {
  // Requirements of this kernel; the caller may fall back to the CUDA-core kernel on ERR_IMPL.
  if (dv > 112) return BASED_ERR_IMPL;  // V' = dv + 16 columns must fit the 128 TMEM lanes
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(y)) return BASED_ERR_IMPL;
  const int64_t all[] = {sq.b, sq.h, sq.l, sk.b, sk.h, sk.l, sv.b, sv.h, sv.l, sy.b, sy.h, sy.l};
  for (int64_t s : all)
    if (s % 8 != 0) return BASED_ERR_IMPL;  // 16-byte vector accesses on every row
  Params p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k = static_cast<const __nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.y = static_cast<__nv_bfloat16*>(y);
  p.kv_state = kv_state;
  p.k_state = k_state;
  p.H = H; p.L = L; p.dv = dv;
  p.state_bf16 = state_dtype == BASED_BF16;
  p.sq = sq; p.sk = sk; p.sv = sv; p.sy = sy;
  p.eps = eps;
  cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p.status), g_tc_status);
  if (e != cudaSuccess) return (int)e;
  e = cudaFuncSetAttribute(linattn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_TOTAL);
  if (e != cudaSuccess) return (int)e;
  linattn_prefill_tc_kernel<<<B * H, NT, SM_TOTAL, stream>>>(p);
  return (int)cudaGetLastError();
}

}  // namespace based
