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

#ifdef BASED_TC_TRACE
// Debug build only: cycles per phase summed over all CTAs (thread 0), and the CTA count.
__device__ unsigned long long g_swa_trace[16];
#define SWA_TR(slot) do { if (tid == 0) { const long long now_ = clock64(); atomicAdd(&g_swa_trace[slot], (unsigned long long)(now_ - tr_t)); tr_t = now_; } } while (0)
#else
#define SWA_TR(slot)
#endif

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

#ifdef BASED_TC_TRACE
  long long tr_t = clock64();
#endif
  if (tid == 0) {
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }

  // ---- loads: 16-byte pieces straight into the operand layouts, zero-filled outside [0, L) ----
  const int upr = hd >> 3;  // 16-byte units per row
  {
    // piece i = tid + 128 n  ->  row i / upr, unit i % upr, advanced incrementally
    const int dq = NT / upr, dr = NT % upr;
    const __nv_bfloat16* qb = p.q + b * p.sq.b + h * p.sq.h;
    {
      int r = tid / upr, u = tid - r * upr;
      for (int n = 0; n < upr; ++n) {  // 128 rows x upr units / 128 threads
        const bool ok = t0 + r < L;
        cp_async16(sb + SM_Q + u * 2048 + r * 16, ok ? qb + (int64_t)(t0 + r) * p.sq.l + u * 8 : qb, ok);
        r += dq; u += dr;
        if (u >= upr) { u -= upr; ++r; }
      }
    }
    const __nv_bfloat16* kb = p.k + b * p.sk.b + h * p.sk.h;
    const __nv_bfloat16* vb = p.v + b * p.sv.b + h * p.sv.h;
    {
      int r = tid / upr, u = tid - r * upr;
      const int total = (NK * upr) / NT;  // NK is a multiple of 32, so NK * upr is a multiple of 128
      for (int n = 0; n < total; ++n) {
        const int pos = k0 + r;
        const bool ok = pos >= 0 && pos < L;
        const uint32_t off = u * (NK * 16) + r * 16;
        cp_async16(sb + SM_K + off, ok ? kb + (int64_t)pos * p.sk.l + u * 8 : kb, ok);
        cp_async16(sb + SM_V + off, ok ? vb + (int64_t)pos * p.sv.l + u * 8 : vb, ok);
        r += dq; u += dr;
        if (u >= upr) { u -= upr; ++r; }
      }
    }
  }
  cp_async_commit();
  SWA_TR(0);  // set-up + load issue
  // TMEM is allocated only now: when more CTAs are resident than TMEM can serve, the extra
  // CTA blocks here with its loads already in flight.
  __syncwarp();
  if (warp == 0) tmem_alloc(smem_u32(tmem_slot), p.tmem_cols);
  SWA_TR(10);  // TMEM allocation
  cp_async_wait_all();
  fence_proxy_async();
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  SWA_TR(1);  // load wait
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
  const int c_lo = warp * 32;              // first key column any row of this warp can see
  const int npieces = (W + 32) >> 5;
  // valid columns of row t: [t, t + W]  (column c holds key position k0 + c = t0 + c - W)
  // Relative to this warp's first column c_lo = 32*warp, row `lane` sees columns [lane, lane + W]:
  // in the first 32-column piece that is i >= lane, in the last one i <= lane, and everything in
  // between is visible.  Only the first tile of a sequence also has keys before position 0.
  const int first_col = -k0 - c_lo;  // columns below this (relative) are before the sequence start
  mbar_wait_bounded(bar_s, 0, abort_flag, p.status, 16u);
  fence_after_sync();
  SWA_TR(2);  // S MMA
  // Visibility of the 32 columns of piece pc for this row as a bit mask (bit i = column i),
  // so the inner loops are branch-free selects.
  auto piece_mask = [&](int pc) -> uint32_t {
    int lo = (pc == 0) ? lane : 0;
    const int hi = (pc == npieces - 1) ? lane : 31;
    lo = max(lo, first_col - 32 * pc);
    if (lo > hi) return 0u;
    return (0xFFFFFFFFu << lo) & (0xFFFFFFFFu >> (31 - hi));
  };
  float m = -INFINITY;
  for (int pc = 0; pc < npieces; ++pc) {
    uint32_t r[32];
    SWA_TR(3);
    tmem_ld32(tlane + TM_S + c_lo + 32 * pc, r);
    tmem_ld_wait();
    SWA_TR(9);  // TMEM load round trips of the max pass
    const uint32_t mask = piece_mask(pc);
#pragma unroll
    for (int i = 0; i < 32; ++i) m = fmaxf(m, (mask & (1u << i)) ? __uint_as_float(r[i]) : -INFINITY);
  }
  SWA_TR(3);  // max pass
  const float msc = m * p.scale_log2e;
  float sum = 0.f;
  for (int pc = 0; pc < npieces; ++pc) {
    uint32_t r[32];
    tmem_ld32(tlane + TM_S + c_lo + 32 * pc, r);
    tmem_ld_wait();
    const uint32_t mask = piece_mask(pc);
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float e[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int ii = 2 * i + j;
        float val;
        asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(val) : "f"(fmaf(__uint_as_float(r[ii]), p.scale_log2e, -msc)));
        e[j] = (mask & (1u << ii)) ? val : 0.f;
      }
      pk[i] = pack_bf16(e[0], e[1]);
      // the normaliser sums what the MMA will see: the bf16-rounded probabilities
      sum += __uint_as_float(pk[i] << 16) + __uint_as_float(pk[i] & 0xffff0000u);
    }
    tmem_st16(tlane + TM_S + ((c_lo + 32 * pc) >> 1), pk);
  }
  SWA_TR(4);  // exp pass
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
  SWA_TR(5);  // zero fill + barrier

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
  SWA_TR(6);  // PV MMA
  {
    // Each thread parks its normalised row in this warp's 32-row staging tile (the K operand
    // buffer, free since S was computed); the warp then copies the tile out with every store
    // instruction covering whole 128-byte lines.
    const float inv = 1.0f / sum;
    const int yrow_bytes = hd * 2 + 16;  // the pad keeps the per-row 16-byte stores conflict free
    uint8_t* ytile = smem + SM_K + (warp * 32) * yrow_bytes;
    uint8_t* yrow_s = ytile + lane * yrow_bytes;
    for (int i = 0; i < (hd >> 4); ++i) {
      uint32_t r[16];
      tmem_ld16(tlane + TM_O + 16 * i, r);
      tmem_ld_wait();
      uint4 lo, hi;
      lo.x = pack_bf16(__uint_as_float(r[0]) * inv, __uint_as_float(r[1]) * inv);
      lo.y = pack_bf16(__uint_as_float(r[2]) * inv, __uint_as_float(r[3]) * inv);
      lo.z = pack_bf16(__uint_as_float(r[4]) * inv, __uint_as_float(r[5]) * inv);
      lo.w = pack_bf16(__uint_as_float(r[6]) * inv, __uint_as_float(r[7]) * inv);
      hi.x = pack_bf16(__uint_as_float(r[8]) * inv, __uint_as_float(r[9]) * inv);
      hi.y = pack_bf16(__uint_as_float(r[10]) * inv, __uint_as_float(r[11]) * inv);
      hi.z = pack_bf16(__uint_as_float(r[12]) * inv, __uint_as_float(r[13]) * inv);
      hi.w = pack_bf16(__uint_as_float(r[14]) * inv, __uint_as_float(r[15]) * inv);
      *reinterpret_cast<uint4*>(yrow_s + 32 * i) = lo;
      *reinterpret_cast<uint4*>(yrow_s + 32 * i + 16) = hi;
    }
    __syncwarp();
    SWA_TR(7);  // O -> staging
    const int tok_w = t0 + warp * 32;
    __nv_bfloat16* otok = p.o + b * p.so.b + (int64_t)tok_w * p.so.l + h * p.so.h;
    const int dq = 32 / upr, dr = 32 % upr;
    int r = lane / upr, cc = lane - r * upr;
    for (int n0 = 0; n0 < upr; n0 += 4) {
      uint4 val[4];
      int rr[4], cq[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        rr[u] = r; cq[u] = cc;
        if (n0 + u < upr) val[u] = *reinterpret_cast<const uint4*>(ytile + r * yrow_bytes + cc * 16);
        r += dq; cc += dr;
        if (cc >= upr) { cc -= upr; ++r; }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (n0 + u < upr && tok_w + rr[u] < L)
          *reinterpret_cast<uint4*>(otok + (int64_t)rr[u] * p.so.l + cq[u] * 8) = val[u];
    }
  }
  SWA_TR(8);  // copy-out
  fence_before_sync();
  __syncthreads();
#ifdef BASED_TC_TRACE
  if (tid == 0) atomicAdd(&g_swa_trace[15], 1ull);
#endif
  if (warp == 0) {
    fence_after_sync();
    tmem_dealloc(tmem, p.tmem_cols);
  }
}

}  // namespace

#ifdef BASED_TC_TRACE
extern "C" int based_swa_trace_read(unsigned long long* out, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(out, g_swa_trace, sizeof(unsigned long long) * 16);
  if (e == cudaSuccess && reset) {
    unsigned long long z[16] = {0};
    e = cudaMemcpyToSymbol(g_swa_trace, z, sizeof(z));
  }
  return (int)e;
}
#endif

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
