// Causal sliding-window softmax attention over a whole sequence on the sm_100a tensor cores
// (tcgen05.mma, accumulators in TMEM), bf16 I/O: a banded, one-pass flash-style kernel.
//
// Replaces the flash-attn calls of the reference's SlidingAttention
// (based/models/mixers/slide_attention.py:100-106, :206-213: causal=True,
// window_size=(window_left, 0), i.e. query i attends keys [i - window_left, i]).
//
// One CTA of 128 threads owns a tile of 128 queries of one (batch, head) and the
// NK = 128 + window_left keys that any of them can see:
//   S = Q K^T            (M128, N = NK, K = head_dim)          -> TMEM, fp32
//   P = exp2(scale*(S - rowmax)) under the band mask           CUDA cores, one thread per query
//       row; all keys of a row are present, so the softmax is exact in one pass; P (bf16)
//       overwrites S in place and becomes the A operand
//   O = P V              (M128, N = head_dim, K = NK)          -> TMEM
//   out = O / rowsum
// TMEM lanes are private to the warp that owns the rows, so the S -> P rewrite needs no
// block-wide barrier.  With window 64 and head_dim 64 a CTA needs 256 TMEM columns and 64 KB
// of shared memory, so two CTAs share an SM and overlap each other's load / MMA / softmax.
#include "common.cuh"
#include "tcgen05.cuh"

namespace based {

__device__ unsigned int g_tc_status_swa = 0;

namespace {

using namespace tc;

constexpr int TQ = 128;  // queries per tile
constexpr int NT = 128;  // threads per CTA

struct Params {
  const __nv_bfloat16 *q, *k, *v;
  __nv_bfloat16* o;
  int L, H, hd, W, tiles_per_seq, tmem_cols;
  Strides3 sq, sk, sv, so;
  float scale_log2e;
  unsigned int* status;
};

__global__ void __launch_bounds__(NT) swa_prefill_tc_kernel(const Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sb = smem_u32(smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int hd = p.hd, W = p.W, NK = TQ + W, L = p.L;
  int tile = blockIdx.x;
  const int ti = tile % p.tiles_per_seq; tile /= p.tiles_per_seq;
  const int h = tile % p.H, b = tile / p.H;
  const int t0 = ti * TQ;          // first query of the tile
  const int k0 = t0 - W;           // position of key column 0 (may be negative)

  // shared memory: Q K-major [hd/8 units][128 rows][16 B]; K K-major [hd/8][NK][16 B];
  // V MN-major [hd/8 groups][NK keys][16 B]
  const uint32_t q_bytes = (uint32_t)hd * 256, kv_bytes = (uint32_t)hd * NK * 2;
  const uint32_t SM_Q = 0, SM_K = q_bytes, SM_V = q_bytes + kv_bytes, SM_BAR = q_bytes + 2 * kv_bytes;
  const uint32_t bar_s = sb + SM_BAR, bar_o = sb + SM_BAR + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM_BAR + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM_BAR + 20);

  if (tid == 0) {
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  __syncwarp();
  if (warp == 0) tmem_alloc(smem_u32(tmem_slot), p.tmem_cols);

  // ---- loads: 16-byte pieces straight into the operand layouts, zero-filled outside [0, L) ----
  const int upr = hd >> 3;  // 16-byte units per row
  {
    const __nv_bfloat16* qb = p.q + b * p.sq.b + h * p.sq.h;
    for (int i = tid; i < TQ * upr; i += NT) {
      const int r = i / upr, u = i - r * upr;
      const bool ok = t0 + r < L;
      cp_async16(sb + SM_Q + u * 2048 + r * 16, qb + (int64_t)(ok ? t0 + r : 0) * p.sq.l + u * 8, ok);
    }
    const __nv_bfloat16* kb = p.k + b * p.sk.b + h * p.sk.h;
    const __nv_bfloat16* vb = p.v + b * p.sv.b + h * p.sv.h;
    for (int i = tid; i < NK * upr; i += NT) {
      const int r = i / upr, u = i - r * upr;
      const int pos = k0 + r;
      const bool ok = pos >= 0 && pos < L;
      const int64_t row = ok ? pos : 0;
      cp_async16(sb + SM_K + u * (NK * 16) + r * 16, kb + row * p.sk.l + u * 8, ok);
      cp_async16(sb + SM_V + u * (NK * 16) + r * 16, vb + row * p.sv.l + u * 8, ok);
    }
  }
  cp_async_commit();
  cp_async_wait_all();
  fence_proxy_async();
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tlane = tmem + ((uint32_t)(warp * 32) << 16);
  const uint32_t TM_S = 0, TM_O = (uint32_t)NK;

  // ---- S = Q K^T ----
  if (tid == 0) {
    const uint32_t idesc = make_idesc_bf16(128, NK, 0, 0);
    for (int ks = 0; ks < (hd >> 4); ++ks) {
      const uint64_t da = make_smem_desc(sb + SM_Q + ks * 4096, 2048, 128);
      const uint64_t db = make_smem_desc(sb + SM_K + ks * (NK * 32), NK * 16, 128);
      mma_ss(tmem + TM_S, da, db, idesc, ks > 0);
    }
    mma_commit(bar_s);
  }
  __syncwarp();

  // ---- softmax of row t over the band; this warp's rows only need W + 32 key columns ----
  const int t = tid;                       // query row == TMEM lane
  const int c_lo = warp * 32;              // first key column any row of this warp can see
  const int npieces = (W + 32) >> 5;
  // valid columns of row t: [t, t + W]  (column c holds key position k0 + c = t0 + c - W)
  const int v_lo = max(t, -k0), v_hi = t + W;
  mbar_wait_bounded(bar_s, 0, abort_flag, p.status, 16u);
  fence_after_sync();
  float m = -INFINITY;
  for (int pc = 0; pc < npieces; ++pc) {
    uint32_t r[32];
    tmem_ld32(tlane + TM_S + c_lo + 32 * pc, r);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int c = c_lo + 32 * pc + i;
      if (c >= v_lo && c <= v_hi) m = fmaxf(m, __uint_as_float(r[i]));
    }
  }
  const float msc = m * p.scale_log2e;
  float sum = 0.f;
  for (int pc = 0; pc < npieces; ++pc) {
    uint32_t r[32];
    tmem_ld32(tlane + TM_S + c_lo + 32 * pc, r);
    tmem_ld_wait();
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float e[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int c = c_lo + 32 * pc + 2 * i + j;
        const float val = exp2f(fmaf(__uint_as_float(r[2 * i + j]), p.scale_log2e, -msc));
        e[j] = (c >= v_lo && c <= v_hi) ? val : 0.f;
      }
      pk[i] = pack_bf16(e[0], e[1]);
      // the normaliser sums what the MMA will see: the bf16-rounded probabilities
      sum += __uint_as_float(pk[i] << 16) + __uint_as_float(pk[i] & 0xffff0000u);
    }
    tmem_st16(tlane + TM_S + ((c_lo + 32 * pc) >> 1), pk);
  }
  // zero the P columns of keys this warp's rows cannot see
  {
    uint32_t z[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) z[i] = 0;
    const int p_lo = c_lo >> 1, p_hi = (c_lo + 32 * npieces) >> 1;  // data columns [p_lo, p_hi)
    for (int c = 0; c < (NK >> 1); c += 16)
      if (c < p_lo || c >= p_hi) tmem_st16(tlane + TM_S + c, z);
  }
  tmem_st_wait();
  fence_before_sync();
  __syncthreads();

  // ---- O = P V ----
  if (tid == 0) {
    fence_after_sync();
    const uint32_t idesc = make_idesc_bf16(128, hd, 0, 1);
    for (int ks = 0; ks < (NK >> 4); ++ks)
      mma_ts(tmem + TM_O, tmem + TM_S + 8 * ks, make_smem_desc(sb + SM_V + ks * 256, 128, NK * 16), idesc, ks > 0);
    mma_commit(bar_o);
  }
  __syncwarp();

  // ---- epilogue ----
  mbar_wait_bounded(bar_o, 0, abort_flag, p.status, 32u);
  fence_after_sync();
  {
    const float inv = 1.0f / sum;
    const bool valid = t0 + t < L;
    __nv_bfloat16* orow = p.o + b * p.so.b + (int64_t)(t0 + t) * p.so.l + h * p.so.h;
    for (int i = 0; i < (hd >> 4); ++i) {
      uint32_t r[16];
      tmem_ld16(tlane + TM_O + 16 * i, r);
      tmem_ld_wait();
      if (valid) {
        uint4 lo, hi;
        lo.x = pack_bf16(__uint_as_float(r[0]) * inv, __uint_as_float(r[1]) * inv);
        lo.y = pack_bf16(__uint_as_float(r[2]) * inv, __uint_as_float(r[3]) * inv);
        lo.z = pack_bf16(__uint_as_float(r[4]) * inv, __uint_as_float(r[5]) * inv);
        lo.w = pack_bf16(__uint_as_float(r[6]) * inv, __uint_as_float(r[7]) * inv);
        hi.x = pack_bf16(__uint_as_float(r[8]) * inv, __uint_as_float(r[9]) * inv);
        hi.y = pack_bf16(__uint_as_float(r[10]) * inv, __uint_as_float(r[11]) * inv);
        hi.z = pack_bf16(__uint_as_float(r[12]) * inv, __uint_as_float(r[13]) * inv);
        hi.w = pack_bf16(__uint_as_float(r[14]) * inv, __uint_as_float(r[15]) * inv);
        *reinterpret_cast<uint4*>(orow + 16 * i) = lo;
        *reinterpret_cast<uint4*>(orow + 16 * i + 8) = hi;
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    fence_after_sync();
    tmem_dealloc(tmem, p.tmem_cols);
  }
}

}  // namespace

int read_tc_status_swa(unsigned int* out, int reset) {
  unsigned int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_tc_status_swa, sizeof(v));
  if (e != cudaSuccess) return (int)e;
  if (out) *out = v;
  if (reset && v != 0) {
    v = 0;
    e = cudaMemcpyToSymbol(g_tc_status_swa, &v, sizeof(v));
  }
  return (int)e;
}

int launch_swa_prefill_tc(const void* q, const void* k, const void* v, void* o, int B, int L, int H, int hd,
                          Strides3 sq, Strides3 sk, Strides3 sv, Strides3 so, int window_left, float scale,
                          cudaStream_t stream) {
  // Requirements of this kernel; the caller may fall back to the CUDA-core kernel on ERR_IMPL.
  if (window_left % 32 != 0 || window_left > 128) return BASED_ERR_IMPL;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o)) return BASED_ERR_IMPL;
  const int64_t all[] = {sq.b, sq.h, sq.l, sk.b, sk.h, sk.l, sv.b, sv.h, sv.l, so.b, so.h, so.l};
  for (int64_t s : all)
    if (s % 8 != 0) return BASED_ERR_IMPL;
  const int NK = TQ + window_left;
  const int tiles_per_seq = (L + TQ - 1) / TQ;
  const long long tiles = (long long)B * H * tiles_per_seq;
  if (tiles > 2147483647LL) return BASED_ERR_TOO_LARGE;
  Params p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k = static_cast<const __nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.o = static_cast<__nv_bfloat16*>(o);
  p.L = L; p.H = H; p.hd = hd; p.W = window_left; p.tiles_per_seq = tiles_per_seq;
  p.tmem_cols = (NK + hd <= 256) ? 256 : 512;
  p.sq = sq; p.sk = sk; p.sv = sv; p.so = so;
  p.scale_log2e = scale * 1.4426950408889634f;
  cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p.status), g_tc_status_swa);
  if (e != cudaSuccess) return (int)e;
  const int smem = hd * 256 + 2 * hd * NK * 2 + 64;
  e = cudaFuncSetAttribute(swa_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  swa_prefill_tc_kernel<<<(unsigned)tiles, NT, smem, stream>>>(p);
  return (int)cudaGetLastError();
}

}  // namespace based
