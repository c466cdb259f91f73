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
// block-wide barrier.  Q, K, V tiles arrive by TMA (128-byte swizzle, zero fill outside the
// sequence) and the output tile leaves by TMA, so no thread spends instructions on copies.
// With window 64 and head_dim 64 a CTA needs 256 TMEM columns and 65 KB of shared memory: three
// CTAs fit an SM; TMEM serves two, the third waits in tcgen05.alloc with its loads in flight.
#include "common.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

#include <mutex>

namespace based {

__device__ unsigned int g_tc_status_swa = 0;


namespace {

using namespace tc;

constexpr int TQ = 128;  // queries per tile
constexpr int NT = 128;  // threads per CTA

struct Params {
  CUtensorMap mq, mk, mv, mo;  // [B][H][L][hd] views, box = (<= 64 columns) x (rows), 128-byte swizzle
  int L, H, hd, W, tiles_per_seq, tmem_cols;
  float scale_log2e;
  unsigned int* status;
};

__global__ void __launch_bounds__(NT) swa_prefill_tc_kernel(const __grid_constant__ Params p) {
  extern __shared__ uint8_t smem_raw[];
  // the swizzled tiles need a 1024-byte aligned base
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t sb = smem_u32(smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int hd = p.hd, W = p.W, NK = TQ + W;
  // head index fastest: CTAs that run at the same time then read the SAME token rows of the packed projection
  // (H x 128 contiguous bytes per row and part) instead of one 128-byte piece out of every row's 6 KB
  int tile = blockIdx.x;
  const int h = tile % p.H; tile /= p.H;
  const int ti = tile % p.tiles_per_seq, b = tile / p.tiles_per_seq;
  const int t0 = ti * TQ;          // first query of the tile
  const int k0 = t0 - W;           // position of key column 0 (may be negative)

  // shared memory: per 64-column atom a of the head dimension, a 128-byte-swizzled tile with
  // 128-byte rows: Q[a] 128 rows, K[a] and V[a] NK rows.  The output tile reuses Q's space.
  const int natom = (hd + 63) >> 6;
  const uint32_t q_atom = TQ * 128, kv_atom = (uint32_t)NK * 128;
  const uint32_t SM_Q = 0, SM_K = natom * q_atom, SM_V = SM_K + natom * kv_atom, SM_BAR = SM_V + natom * kv_atom;
  const uint32_t bar_qk = sb + SM_BAR, bar_v = sb + SM_BAR + 8, bar_s = sb + SM_BAR + 16, bar_o = sb + SM_BAR + 24;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM_BAR + 32);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM_BAR + 36);

  if (tid == 0) {
    mbar_init(bar_qk, 1);
    mbar_init(bar_v, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async();
    // ---- loads: one TMA tile per operand and column atom; rows outside [0, L) read as zero ----
    // every box is 64 columns wide (columns past hd are out of bounds: zero-filled, and counted)
    tma::mbar_expect_tx(bar_qk, (uint32_t)natom * 128u * (TQ + NK));
    tma::mbar_expect_tx(bar_v, (uint32_t)natom * 128u * NK);
    for (int a = 0; a < natom; ++a) {
      tma::load_4d(sb + SM_Q + a * q_atom, &p.mq, bar_qk, 64 * a, t0, h, b);
      tma::load_4d(sb + SM_K + a * kv_atom, &p.mk, bar_qk, 64 * a, k0, h, b);
    }
    for (int a = 0; a < natom; ++a) tma::load_4d(sb + SM_V + a * kv_atom, &p.mv, bar_v, 64 * a, k0, h, b);
  }
  // TMEM is allocated only now: when more CTAs are resident than TMEM can serve, the extra
  // CTA blocks here with its loads already in flight.
  __syncwarp();
  if (warp == 0) tmem_alloc(smem_u32(tmem_slot), p.tmem_cols);
  fence_before_sync();
  __syncthreads();  // barriers initialised, TMEM base published
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tlane = tmem + ((uint32_t)(warp * 32) << 16);
  const uint32_t TM_S = 0, TM_O = (uint32_t)NK;

  // ---- S = Q K^T as soon as Q and K have landed (V may still be in flight) ----
  // Warp 0 runs the issue loops converged and one elected lane issues: the descriptors are then values the compiler
  // can keep in uniform registers, instead of being moved there, several moves per MMA, by a single diverged lane.
  const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem, 0);
  const bool leader = warp == 0 && elect_one_sync();
  if (warp == 0) {
    mbar_wait_bounded(bar_qk, 0, abort_flag, p.status, 64u);
    fence_after_sync();
    const uint32_t idesc = make_idesc_bf16(128, NK, 0, 0);
    int first = 1;
    for (int a = 0; a < natom; ++a) {
      const int ksteps = (min(64, hd - 64 * a)) >> 4;
      for (int ks = 0; ks < ksteps; ++ks) {  // a K-step of 16 elements = 32 bytes inside the swizzled row
        const uint64_t da = make_smem_desc_sw128(sb + SM_Q + a * q_atom + ks * 32, 16, 1024);
        const uint64_t db = make_smem_desc_sw128(sb + SM_K + a * kv_atom + ks * 32, 16, 1024);
        if (leader) mma_ss(tmem_u + TM_S, da, db, idesc, first ? 0u : 1u);
        first = 0;
      }
    }
    if (leader) mma_commit(bar_s);
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
  // Visibility of the 32 columns of piece pc for this row as a bit mask (bit i = column i),
  // so the inner loops are branch-free selects.
  auto piece_mask = [&](int pc) -> uint32_t {
    int lo = (pc == 0) ? lane : 0;
    const int hi = (pc == npieces - 1) ? lane : 31;
    lo = max(lo, first_col - 32 * pc);
    if (lo > hi) return 0u;
    return (0xFFFFFFFFu << lo) & (0xFFFFFFFFu >> (31 - hi));
  };
  // one probability pair -> bf16x2, and what the MMA will see of it added to the normaliser.  The row is one
  // thread's work, and a tile's life is mostly this thread's dependent chain: the running maximum and the running
  // sum are kept in four independent lanes each, so that neither is a chain of 96 dependent operations.
  float sum4[4] = {0.f, 0.f, 0.f, 0.f};
  auto exp_piece = [&](const uint32_t (&r)[32], uint32_t mask, float msc, int pc) {
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
      sum4[i & 3] += __uint_as_float(pk[i] << 16) + __uint_as_float(pk[i] & 0xffff0000u);
    }
    tmem_st16(tlane + TM_S + ((c_lo + 32 * pc) >> 1), pk);
  };
  auto max_piece = [&](const uint32_t (&r)[32], uint32_t mask, float m) {
    float m4[4] = {m, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < 32; ++i) m4[i & 3] = fmaxf(m4[i & 3], (mask & (1u << i)) ? __uint_as_float(r[i]) : -INFINITY);
    return fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
  };
  if (npieces <= 3) {
    // window <= 64: the row's 96 scores stay in registers between the max and the exponentials, so S is read from
    // TMEM once, with all loads in flight together
    uint32_t r0[32], r1[32], r2[32];
    tmem_ld32(tlane + TM_S + c_lo, r0);
    if (npieces > 1) tmem_ld32(tlane + TM_S + c_lo + 32, r1);
    if (npieces > 2) tmem_ld32(tlane + TM_S + c_lo + 64, r2);
    tmem_ld_wait();
    const uint32_t m0 = piece_mask(0), m1 = npieces > 1 ? piece_mask(1) : 0u, m2 = npieces > 2 ? piece_mask(2) : 0u;
    float m = max_piece(r0, m0, -INFINITY);
    if (npieces > 1) m = max_piece(r1, m1, m);
    if (npieces > 2) m = max_piece(r2, m2, m);
    const float msc = m * p.scale_log2e;
    exp_piece(r0, m0, msc, 0);
    if (npieces > 1) exp_piece(r1, m1, msc, 1);
    if (npieces > 2) exp_piece(r2, m2, msc, 2);
  } else {
    float m = -INFINITY;
    for (int pc = 0; pc < npieces; ++pc) {
      uint32_t r[32];
      tmem_ld32(tlane + TM_S + c_lo + 32 * pc, r);
      tmem_ld_wait();
      m = max_piece(r, piece_mask(pc), m);
    }
    const float msc = m * p.scale_log2e;
    for (int pc = 0; pc < npieces; ++pc) {
      uint32_t r[32];
      tmem_ld32(tlane + TM_S + c_lo + 32 * pc, r);
      tmem_ld_wait();
      exp_piece(r, piece_mask(pc), msc, pc);
    }
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
  if (warp == 0) {
    mbar_wait_bounded(bar_v, 0, abort_flag, p.status, 128u);
    fence_after_sync();
    // V tiles are MN-major: 64-column atoms kv_atom apart (LBO), groups of 8 keys 1024 B apart (SBO)
    const uint32_t idesc = make_idesc_bf16(128, hd, 0, 1);
    for (int ks = 0; ks < (NK >> 4); ++ks) {
      const uint64_t dvd = make_smem_desc_sw128(sb + SM_V + ks * 2048, kv_atom, 1024);
      if (leader) mma_ts(tmem_u + TM_O, tmem_u + TM_S + 8 * ks, dvd, idesc, ks > 0);
    }
    if (leader) mma_commit(bar_o);
  }
  __syncwarp();

  // ---- epilogue ----
  mbar_wait_bounded(bar_o, 0, abort_flag, p.status, 32u);
  fence_after_sync();
  {
    // Each thread writes its normalised row into the output tile (Q's space, free since S was
    // computed) in the 128-byte-swizzled layout; one thread then hands the tile to the TMA unit,
    // which clips rows past the end of the sequence.
    const float inv = 1.0f / ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
    const int t = tid;
    // four 16-column pieces per round: their TMEM loads are in flight together
    auto put = [&](int i, const uint32_t (&r)[16]) {
      uint4 lo, hi;
      lo.x = pack_bf16(__uint_as_float(r[0]) * inv, __uint_as_float(r[1]) * inv);
      lo.y = pack_bf16(__uint_as_float(r[2]) * inv, __uint_as_float(r[3]) * inv);
      lo.z = pack_bf16(__uint_as_float(r[4]) * inv, __uint_as_float(r[5]) * inv);
      lo.w = pack_bf16(__uint_as_float(r[6]) * inv, __uint_as_float(r[7]) * inv);
      hi.x = pack_bf16(__uint_as_float(r[8]) * inv, __uint_as_float(r[9]) * inv);
      hi.y = pack_bf16(__uint_as_float(r[10]) * inv, __uint_as_float(r[11]) * inv);
      hi.z = pack_bf16(__uint_as_float(r[12]) * inv, __uint_as_float(r[13]) * inv);
      hi.w = pack_bf16(__uint_as_float(r[14]) * inv, __uint_as_float(r[15]) * inv);
      uint8_t* atom = smem + SM_Q + (i >> 2) * q_atom;  // 16 columns = 2 chunks; 4 such pieces per 64-column atom
      *reinterpret_cast<uint4*>(atom + tma::sw128_offset(t, 2 * (i & 3))) = lo;
      *reinterpret_cast<uint4*>(atom + tma::sw128_offset(t, 2 * (i & 3) + 1)) = hi;
    };
    const int np = hd >> 4;
    for (int i0 = 0; i0 < np; i0 += 4) {
      uint32_t ra[16], rb[16], rc[16], rd[16];
      tmem_ld16(tlane + TM_O + 16 * i0, ra);
      if (i0 + 1 < np) tmem_ld16(tlane + TM_O + 16 * (i0 + 1), rb);
      if (i0 + 2 < np) tmem_ld16(tlane + TM_O + 16 * (i0 + 2), rc);
      if (i0 + 3 < np) tmem_ld16(tlane + TM_O + 16 * (i0 + 3), rd);
      tmem_ld_wait();
      put(i0, ra);
      if (i0 + 1 < np) put(i0 + 1, rb);
      if (i0 + 2 < np) put(i0 + 2, rc);
      if (i0 + 3 < np) put(i0 + 3, rd);
    }
    fence_proxy_async();  // generic-proxy writes -> visible to the TMA unit
    __syncthreads();
    if (tid == 0) {
      for (int a = 0; a < natom; ++a) tma::store_4d(&p.mo, sb + SM_Q + a * q_atom, 64 * a, t0, h, b);
      bulk_commit();
      bulk_wait_read_all();  // shared memory must stay intact until the TMA unit has read it
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
    if (s % 8 != 0 || s <= 0) return BASED_ERR_IMPL;  // TMA strides: positive multiples of 16 bytes
  const int NK = TQ + window_left;
  const int tiles_per_seq = (L + TQ - 1) / TQ;
  const long long tiles = (long long)B * H * tiles_per_seq;
  if (tiles > 2147483647LL) return BASED_ERR_TOO_LARGE;
  Params p;
  // tensor maps over [B][H][L][hd] (dims innermost first: hd, L, H, B); a batch or head extent of 1
  // may come with any stride, so give those a harmless one.  Maps are cached by pointer and geometry.
  static tma::MapCache cache;
  auto fix = [&](int64_t s, int extent) { return extent == 1 ? (int64_t)8 : s; };
  auto get_map = [&](CUtensorMap* out, const void* base, Strides3 s, int rows) -> int {
    const tma::MapKey key = tma::make_key(base, (uint64_t)hd, (uint64_t)L, (uint64_t)H, (uint64_t)B, 0, s.l, fix(s.h, H),
                                          fix(s.b, B), 0, 64, (uint32_t)rows, 0, 4);
    if (cache.find(key, out)) return 0;
    if (tma::encode_bf16_4d_sw128(out, base, hd, L, H, B, s.l, fix(s.h, H), fix(s.b, B), 64, rows)) return BASED_ERR_IMPL;
    cache.put(key, *out);
    return 0;
  };
  if (get_map(&p.mq, q, sq, TQ) || get_map(&p.mk, k, sk, NK) || get_map(&p.mv, v, sv, NK) || get_map(&p.mo, o, so, TQ))
    return BASED_ERR_IMPL;
  p.L = L; p.H = H; p.hd = hd; p.W = window_left; p.tiles_per_seq = tiles_per_seq;
  p.tmem_cols = (NK + hd <= 256) ? 256 : 512;
  p.scale_log2e = scale * 1.4426950408889634f;
  const int natom = (hd + 63) / 64;
  const int smem = natom * (TQ + 2 * NK) * 128 + 64 + 1024;  // + slack to align the tiles to 1024 bytes
  {
    // once per device: the status word's address and the largest shared-memory size this kernel is launched with
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static unsigned int* status[kMaxDevices] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return BASED_ERR_TOO_LARGE;
    std::lock_guard<std::mutex> lock(mu);
    if (status[dev] == nullptr) {
      unsigned int* addr = nullptr;
      e = cudaGetSymbolAddress(reinterpret_cast<void**>(&addr), g_tc_status_swa);
      if (e != cudaSuccess) return (int)e;
      const int max_smem = 2 * (TQ + 2 * (TQ + 128)) * 128 + 64 + 1024;   // head_dim 128, window 128
      e = cudaFuncSetAttribute(swa_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
      if (e != cudaSuccess) return (int)e;
      status[dev] = addr;
    }
    p.status = status[dev];
  }
  swa_prefill_tc_kernel<<<(unsigned)tiles, NT, smem, stream>>>(p);
  return (int)cudaGetLastError();
}

}  // namespace based
