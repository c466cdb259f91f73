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
#include "linattn_tc_shared.cuh"
#include "tma.cuh"

#include <mutex>
#include <type_traits>

namespace based {

__device__ unsigned int g_tc_status = 0;  // ORed with a code when a bounded wait expires

// Built-in workspace of the allocation-free sequence-split entry point: per-segment states,
// (batch x head) x (segments - 1) x (dv + 1) x 160 floats.  Every word the kernels read was
// written earlier in the same call, so nothing here has to start at zero.
static __device__ __align__(256) unsigned char g_static_scratch[BASED_STATIC_SCRATCH_BYTES];

namespace {

using namespace tc;
using namespace tcp;


// Shared memory map (bytes).  One stage = Q [2 k-halves][128 tok][16 B] K-major (4096) + K (4096) +
// V' MN-major [dv/8 + 1 groups of 8 columns][128 tok][16 B]: the columns of V, then the group that starts with
// the ones column.  The MMAs address NV/8 = dv/8 + 2 groups (N must be a multiple of 16) and the state-update
// MMA reads V'^T as an M = 128 operand, i.e. 16 groups from the stage's V' base: the groups past dv/8 + 1 are
// whatever follows in shared memory.  They only feed accumulator columns / lanes > dv + 8 of O and of the
// state, which nobody reads (a column of an MMA result depends on that column of its B operand alone).
struct Smem {
  int nstage, npk, stage_bytes, phik, stb, stb_bytes, ystage, yrow_bytes, bar, total;
  __host__ __device__ explicit Smem(int dv) {
    const int nv = dv + 16;
    nstage = dv <= 64 ? 3 : 2;     // what fits in 227 KB
    npk = dv <= 64 ? 2 : 1;        // phi'(K) buffers
    stage_bytes = 8192 + ((dv >> 3) + 1) * 2048;
    phik = nstage * stage_bytes;   // npk x 40960  MN-major [20 groups of 8 feats][128 tok][16 B]
    stb = phik + npk * 40960;      // 2 x stb_bytes: bf16 state, K-major [20 k-units][NV rows][16 B], double-buffered
    stb_bytes = nv * 320;
    ystage = stb + 2 * stb_bytes;  // output tile [128 rows][32 columns bf16 + 16 B pad], one round of the epilogue
    yrow_bytes = 64 + 16;          // the pad makes the per-row 16-byte stores bank-conflict free
    bar = ystage + C * yrow_bytes; // mbarriers, TMEM base, abort flag
    total = bar + 256;
  }
};

// TMEM columns (32-bit each), 512 allocated
constexpr uint32_t TM_ST = 0;     // state^T accumulator: lanes = V' column, 160 feature columns, fp32
constexpr uint32_t TM_S = 160;    // S fp32 (128 cols); with NV > 80 overwritten in place by P bf16 (64 cols)
constexpr uint32_t TM_O = 288;    // O accumulator, NV <= 128 columns
constexpr uint32_t TM_PQ = 416;   // phi'(Q) bf16, 80 columns (NV > 80)
// With NV <= 80 (dv <= 64) the O accumulator leaves room for P in columns of its own, 368-431, and phi'(Q) moves
// to 432-511: the pieces of P right of the diagonal, which are zeros, are then written once instead of once per
// chunk (S(c+1) no longer overwrites them), and P's stores cannot land on S columns another warp has yet to read.
constexpr uint32_t TM_P_SEP = 368, TM_PQ_SEP = 432;
constexpr uint32_t TM_COLS = 512;

// mbarrier slots (8 bytes each) from Smem::bar
//   B_FULL             per stage: tile landed (TMA transaction bytes)
//   B_EMPTY            per stage, state-only mode: the update that read the tile has completed      (commit)
//   B_S_DONE           S(c) = Q K^T complete                                   (tcgen05.commit)
//   B_A_READY          P(c) written AND O free (O(c-1) read out) AND tile c+1 landed   (poly warps + output warps)
//   B_XQ_READY         phi'(Q_c) written (phase c)                                   (expansion warps)
//   B_XK_READY[2]      phi'(K_c) written, and the raw q of chunk c taken into registers (buffer c % NPK, phase
//                      c / NPK: one barrier per phi'(K) buffer, because the expansion warps may run a whole
//                      buffer ahead of the MMA thread and a waiter must never fall two phases behind)
//   B_O_DONE           readout of chunk c complete: O(c) final, phi'(Q_c) consumed   (commit)
//   B_STB_READY        bf16 copy of the state after chunk c written (drain warps)
//   B_PK_FREE[2]       state update of chunk c complete (buffer c % NPK, phase c / NPK): its phi'(K) buffer is
//                      free again, and the state may be drained                     (commit)
// The MMA thread pays for every commit and every wait with idle tensor cycles, so the main loop has three of each.
//   B_INIT             carried-in state preloaded (sequence split)      B_FIN   last update complete (state-only mode)
enum Bar { B_FULL = 0, B_EMPTY = 3, B_S_DONE = 6, B_A_READY, B_XQ_READY, B_XK_READY, B_XK_READY1, B_O_DONE, B_STB_READY, B_PK_FREE,
           B_PK_FREE1, B_INIT, B_FIN, B_COUNT };

// P(c) = causal(1 + s/4 + s^2/32), evaluated in bf16x2 (two FMAs per pair), in place over S, for the 32-column
// pieces [p0, p1) of this warp's 32 rows; pieces right of the diagonal block (> qd) are zeros, no load.
// P is half as wide as S: piece k of P lands on S columns [16k, 16k + 16), i.e. inside S piece k / 2.  One warp
// going through its pieces in ascending order never overwrites what it has not read.  When two warps share a
// quadrant (pieces [0, 2) and [2, 4)), the second one's first store lands inside S piece 1, which belongs to
// the first warp: the first warp arrives on a named barrier once it has piece 1 in registers (share == 1), the
// second waits there before its first store (share == 2).
// A function of its own, not inlined: two roles call it, and the kernel's hot code has to stay inside the SM's
// instruction cache.
__device__ __noinline__ void poly_pieces(uint32_t tlane, uint32_t tm_p, bool zeros, int qd, int lane, int p0, int p1,
                                         int share) {
  constexpr uint32_t k1 = 0x3F803F80u, kq = 0x3E803E80u, k32 = 0x3D003D00u;  // (1,1) (1/4,1/4) (1/32,1/32)
#pragma unroll 1
  for (int piece = p0; piece < p1; ++piece) {
    if (piece <= qd) {
      uint32_t sreg[32], pk[16];
      tmem_ld32(tlane + TM_S + piece * 32, sreg);
      tmem_ld_wait();
      if (share == 1 && piece == 1) asm volatile("bar.arrive 1, 64;\n" ::: "memory");
      if (piece < qd) {   // left of the diagonal block: every column is visible
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const uint32_t w = pack_bf16(__uint_as_float(sreg[2 * i]), __uint_as_float(sreg[2 * i + 1]));
          pk[i] = fma_bf16x2(w, fma_bf16x2(w, k32, kq), k1);
        }
      } else {            // the diagonal block: columns 0..lane of this piece are visible
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const uint32_t w = pack_bf16(__uint_as_float(sreg[2 * i]), __uint_as_float(sreg[2 * i + 1]));
          const uint32_t pv = fma_bf16x2(w, fma_bf16x2(w, k32, kq), k1);
          const uint32_t mask = (2 * i + 1 <= lane) ? 0xFFFFFFFFu : ((2 * i <= lane) ? 0x0000FFFFu : 0u);
          pk[i] = pv & mask;
        }
      }
      if (share == 2 && piece == p0) asm volatile("bar.sync 1, 64;\n" ::: "memory");
      tmem_st16(tlane + tm_p + piece * 16, pk);
    } else if (zeros) {
      uint32_t z[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) z[i] = 0;
      tmem_st16(tlane + tm_p + piece * 16, z);
    }
  }
}

// Per 128-token chunk c the MMA thread issues, in this order,
//   PV(c):  O  = P(c) V'(c)                    8 MMAs  M128 N=NV  K16   A = P in TMEM
//   S(c+1)                                     1 MMA   M128 N128  K16
//   R(c):   O += phi'(Q_c) State(c-1)          10 MMAs M128 N=NV  K16   A = phi'(Q) in TMEM, B = bf16 state (smem)
//   U(c+1): St^T += V'(c+1)^T phi'(K_{c+1})    8 MMAs  M128 N160  K16   (the state update runs ONE CHUNK AHEAD)
// so that the output warps read O(c) while U(c+1) keeps the tensor pipe busy, the polynomial of chunk c+1 runs
// under R(c) and U(c+1), the expansions run a step ahead, and the only chain carried from chunk to chunk is
// U(c) -> drain (fp32 state -> bf16 operand) -> U(c+1): the drain reads the accumulator that U(c+1) writes.
//
// Two properties of the SM shaped the code as much as the schedule did:
//  * The 16 warps run five different programs, and what they execute per chunk has to stay inside the SM's
//    instruction cache: misses go to a cache shared by all SMs of a GPC, and with every SM running this kernel
//    that cache saturates - the same CTA ran 1.6x slower with 128 CTAs on the chip than with 16.  Hence the rolled
//    output rounds, the polynomial as one function shared by its two callers, and no variant code in the loops.
//  * The MMA thread's own instructions between two MMAs are idle tensor time (an issue blocks until the pipe
//    accepts it, so the thread cannot run ahead): its MMA loops are unrolled and it has three waits and three
//    commits per chunk.
__global__ void __launch_bounds__(NT, 1) linattn_prefill_tc_kernel(const __grid_constant__ Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sb = smem_u32(smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int qd = warp & 3;       // TMEM lane quadrant this warp can reach
  const int t = qd * 32 + lane;  // token within the chunk == TMEM lane (compute warps)
  const int bh = blockIdx.x / p.grid_segs, seg = blockIdx.x - bh * p.grid_segs;
  const int b = bh / p.H, h = bh - b * p.H;
  const int dv = p.dv, NV = dv + 16;
  const Smem lay(dv);
  // This CTA's tokens: tok_base .. tok_base + L - 1 (L counts from the segment's first token).
  const int tok_base = seg * p.seg_chunks * C;
  const int L = p.L - tok_base;
  const int nchunks = min(p.seg_chunks, (L + C - 1) / C);
  const int mode = p.mode;
  const bool has_init = mode == MODE_SEG_OUTPUT && seg > 0;
  const bool write_state = mode != MODE_SEG_STATE && seg == p.nseg - 1 && p.kv_state != nullptr;
  const bool q3_has_state = 96 < NV;          // TMEM lanes 96..127 hold state rows (dv > 80)
  const int NS = lay.nstage, NPK = lay.npk;

  auto bar = [&](int i) { return sb + lay.bar + 8 * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + lay.bar + 8 * B_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + lay.bar + 8 * B_COUNT + 4);
  auto wait = [&](int i, uint32_t parity, unsigned int code) {
    mbar_wait_bounded(bar(i), parity & 1u, abort_flag, p.status, code);
  };
  auto wait1 = [&](int i, uint32_t parity, unsigned int code) {   // by one lane of a diverged warp
    mbar_wait_bounded<false>(bar(i), parity & 1u, abort_flag, p.status, code);
  };

  // One thread feeds the stages: Q and K land as [k-half][token][16 B], V' as [8-column group][token][16 B] - the
  // no-swizzle UMMA layouts - by one cp.async.bulk.tensor each (the tensor maps cut a row into 16-byte groups and
  // put the group index outside the token index).  Tokens past the end of the sequence are zero-filled by the
  // copy unit.  Chunk j goes to stage j % NS once the MMAs that read chunk j - NS have completed.
  const bool need_q = mode != MODE_SEG_STATE;
  auto issue_tile = [&](int j) {
    const int st = j % NS;
    const uint32_t base = sb + st * lay.stage_bytes;
    const int tok = tok_base + j * C;
    tma::mbar_expect_tx(bar(B_FULL + st), (need_q ? 8192u : 4096u) + (uint32_t)dv * 256u);
    if (need_q) tma::load_5d(base, &p.mq, bar(B_FULL + st), 0, tok, 0, h, b);
    tma::load_5d(base + 4096, &p.mk, bar(B_FULL + st), 0, tok, 0, h, b);
    tma::load_5d(base + 8192, &p.mv, bar(B_FULL + st), 0, tok, 0, h, b);
  };

  // ------------------------------------------------------------------ set-up (by the producer thread, which then
  // requests the first tiles at once: they travel while TMEM is allocated and the constants are written)
  if (tid == W_LOAD * 32) {
    for (int i = 0; i < 3; ++i) { mbar_init(bar(B_FULL + i), 1); mbar_init(bar(B_EMPTY + i), 1); }
    mbar_init(bar(B_S_DONE), 1);
    mbar_init(bar(B_O_DONE), 1);
    // polynomial warps: 4 (one per quadrant), 5 when quadrant 3 is shared by two warps; + 4 output warps
    mbar_init(bar(B_A_READY), 4 + (q3_has_state ? 4 : 5));
    mbar_init(bar(B_XQ_READY), 4);
    mbar_init(bar(B_XK_READY), 4);
    mbar_init(bar(B_XK_READY1), 4);
    mbar_init(bar(B_STB_READY), 4);
    mbar_init(bar(B_PK_FREE), 1);
    mbar_init(bar(B_PK_FREE + 1), 1);
    mbar_init(bar(B_INIT), 4);
    mbar_init(bar(B_FIN), 1);
    *abort_flag = 0;
    fence_mbar_init();
    for (int j = 0; j < min(NS, nchunks); ++j) issue_tile(j);
  }
  __syncwarp();
  if (warp == 0) tmem_alloc(smem_u32(tmem_slot), TM_COLS);
  // V' column group dv/8 (the ones column, then zeros) is constant for the whole kernel.
  for (int i = tid; i < NS * C; i += NT) {
    const int st = i / C, tk = i - st * C;
    *reinterpret_cast<uint4*>(smem + st * lay.stage_bytes + 8192 + (dv >> 3) * 2048 + tk * 16) =
        make_uint4(0x00003F80u, 0, 0, 0);  // bf16 1.0 in element 0
  }
  fence_proxy_async();
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_v = tmem;
  const uint32_t tlane = tmem + ((uint32_t)(qd * 32) << 16);  // this warp's lane window, column 0

  // the polynomial of chunk c by this warp (pieces [p0, p1)), then one arrival on B_A_READY - which, with three
  // stages, also vouches for tile c + 1 having landed (it was requested two chunks earlier), so that the MMA thread
  // need not test that barrier itself; with two stages the tile is requested only after this arrival, and the MMA
  // thread waits for it where it needs it
  const bool full_via_a = NS >= 3;
  const bool p_separate = NV <= 80;
  const uint32_t tm_p = p_separate ? TM_P_SEP : TM_S, tm_pq = p_separate ? TM_PQ_SEP : TM_PQ;
  auto make_p = [&](int c, int p0, int p1, int share, bool producer) {
    wait(B_S_DONE, c, 0x400u);
    fence_after_sync();
    // S(c) is complete, hence so is P(c-1) V'(c-1), issued before it: the MMAs are done with the stage of chunk
    // c - 1, and so are the expansion warps (see their loop).  Its refill starts here, ahead of the polynomial.
    if (producer && lane == 0 && c >= 1 && c + NS - 1 < nchunks) issue_tile(c + NS - 1);
    __syncwarp();
    poly_pieces(tlane, tm_p, !p_separate || c == 0, qd, lane, p0, p1, share);
    tmem_st_wait();
    fence_before_sync();
    if (full_via_a && c + 1 < nchunks) wait(B_FULL + (c + 1) % NS, (c + 1) / NS, 0x403u);
    __syncwarp();
    if (lane == 0) mbar_arrive(bar(B_A_READY));
  };

  if (warp >= W_LOAD) {
    // ================================================================ polynomial warps of quadrants 1-3; warp 13's
    // lane 0 is also the TMA producer
    if (mode == MODE_SEG_STATE) {
      if (warp == W_LOAD && lane == 0)
        for (int j = min(NS, nchunks); j < nchunks; ++j) {
          if (j >= NS) wait1(B_EMPTY + j % NS, j / NS - 1, 0x100u);   // the update that read tile j - NS is complete
          issue_tile(j);
        }
    } else {
      // quadrant 3 is shared with warp 7 when that warp has no state rows to drain
      const bool shared_q3 = qd == 3 && !q3_has_state;
      const int p0 = shared_q3 ? 2 : 0;
      for (int c = 0; c < nchunks; ++c) {
        make_p(c, p0, 4, shared_q3 ? 2 : 0, warp == W_LOAD);
      }
    }
  } else if (warp == W_MMA) {
    // ================================================================ MMA issue.  The WHOLE warp runs the loop and the waits,
    // converged, and one elected lane issues the MMAs and the commits: every operand of an MMA is then a value the
    // compiler can see to be the same in all lanes (the TMEM base is broadcast by a shuffle for that reason), so
    // the descriptors are built and kept in uniform registers instead of being moved there, several moves per MMA,
    // by a single diverged lane - whose own instructions between two MMAs are idle tensor time.
    {
      const uint32_t tmem = __shfl_sync(0xffffffffu, tmem_v, 0);
      const bool leader = elect_one_sync();
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_o_pv = make_idesc_bf16(128, NV, 0, 1);   // A = P (TMEM), B = V' MN-major
      const uint32_t idesc_o_st = make_idesc_bf16(128, NV, 0, 0);   // A = phi'(Q) (TMEM), B = state K-major
      const uint32_t idesc_st = make_idesc_bf16(128, DR, 1, 1);     // A = V'^T MN-major, B = phi'(K) MN-major
      // Descriptors differ between K-steps only in the start address (bits 0-13, units of 16 B).
      const uint64_t d_q = make_smem_desc(sb, 2048, 128);                // + stage offset; k-halves 2048 B apart
      const uint64_t d_k = make_smem_desc(sb + 4096, 2048, 128);
      const uint64_t d_v = make_smem_desc(sb + 8192, 128, 2048);         // + stage offset, + 16 per K-step
      const uint64_t d_pk = make_smem_desc(sb + lay.phik, 128, 2048);    // + buffer offset, + 16 per K-step
      const uint64_t d_stb = make_smem_desc(sb + lay.stb, NV * 16, 128); // + buffer offset, + 2 NV per K-step
      const uint32_t stage_units = (uint32_t)lay.stage_bytes >> 4, stb_units = (uint32_t)lay.stb_bytes >> 4;
      const uint32_t stb_step = 2 * NV;
      // U(c): St^T (+)= V'(c)^T phi'(K_c)
      auto issue_update = [&](int c, bool acc0) {
        const uint64_t dv_c = d_v + (c % NS) * stage_units, d_pk_c = d_pk + (c % NPK) * (40960 >> 4);
        if (leader) {
#pragma unroll
          for (int j = 0; j < C / 16; ++j)
            mma_ss(tmem + TM_ST, dv_c + 16 * j, d_pk_c + 16 * j, idesc_st, (acc0 || j > 0) ? 1u : 0u);
        }
      };
      if (mode == MODE_SEG_STATE) {
        // state only: St += V'(c)^T phi'(K_c) for every chunk of the segment
        for (int c = 0; c < nchunks; ++c) {
          wait(B_FULL + c % NS, c / NS, 0x210u);
          wait(B_XK_READY + c % NPK, c / NPK, 0x211u);
          fence_after_sync();
          issue_update(c, c > 0);
          if (leader) {
            mma_commit(bar(B_EMPTY + c % NS));
            mma_commit(bar(B_PK_FREE + c % NPK));
          }
        }
        if (leader) mma_commit(bar(B_FIN));
      } else {
        wait(B_FULL + 0, 0, 0x200u);
        fence_after_sync();
        if (leader) {
          mma_ss(tmem + TM_S, d_q, d_k, idesc_s, 0);
          mma_commit(bar(B_S_DONE));
        }
        wait(B_XK_READY, 0, 0x208u);                      // phi'(K_0)
        if (has_init) wait(B_INIT, 0, 0x207u);            // state^T and its bf16 copy were preloaded
        fence_after_sync();
        issue_update(0, has_init);
        if (leader) mma_commit(bar(B_PK_FREE + 0));
        for (int c = 0; c < nchunks; ++c) {
          const int st = c % NS;
          // PV(c): needs P(c) and a free O; the same barrier covers tile c + 1
          wait(B_A_READY, c, 0x201u);
          fence_after_sync();
          {
            const uint64_t dv_c = d_v + st * stage_units;
            if (leader) {
#pragma unroll
              for (int j = 0; j < C / 16; ++j)
                mma_ts(tmem + TM_O, tmem + tm_p + 8 * j, dv_c + 16 * j, idesc_o_pv, j > 0);
            }
          }
          // S(c+1): issued behind the P(c) reads above; the tensor core executes MMAs in issue order
          if (c + 1 < nchunks) {
            if (!full_via_a) {
              wait(B_FULL + (c + 1) % NS, (c + 1) / NS, 0x203u);
              fence_after_sync();
            }
            const uint32_t so = ((c + 1) % NS) * stage_units;
            if (leader) {
              mma_ss(tmem + TM_S, d_q + so, d_k + so, idesc_s, 0);
              mma_commit(bar(B_S_DONE));
            }
          }
          // R(c): O(c) += phi'(Q_c) State(c-1).  The bf16 state of chunk c-1 sits in buffer (c-1) & 1 and was
          // awaited before U(c) was issued (see below); a carried-in state was preloaded into buffer 1.
          wait(B_XQ_READY, c, 0x204u);                    // phi'(Q_c)
          fence_after_sync();
          if (c > 0 || has_init) {
            const uint64_t d_stb_c = d_stb + ((c + 1) & 1) * stb_units;
            if (leader) {
#pragma unroll
              for (int j = 0; j < DR / 16; ++j)
                mma_ts(tmem + TM_O, tmem + tm_pq + 8 * j, d_stb_c + stb_step * j, idesc_o_st, 1);
            }
          }
          if (leader) mma_commit(bar(B_O_DONE));
          // U(c+1): must not start before the drain of State(c) has read the accumulator
          if (c + 1 < nchunks) {
            wait(B_STB_READY, c, 0x205u);
            wait(B_XK_READY + (c + 1) % NPK, (c + 1) / NPK, 0x206u);   // phi'(K_{c+1})
            fence_after_sync();
            issue_update(c + 1, true);
            if (leader) mma_commit(bar(B_PK_FREE + (c + 1) % NPK));
          }
        }
        if (leader) mma_commit(bar(B_FIN));   // every MMA is complete: the stages may be reused for the final state
      }
    }
  } else if (warp < 4) {
    // ================================================================ expansion warps: phi'(K) -> smem, phi'(Q) -> TMEM
    auto load_x = [&](int c, int off, uint32_t (&X)[8]) {
      const uint8_t* stg = smem + (c % NS) * lay.stage_bytes + off + t * 16;   // [k-half][token][16 B]
      const uint4 a = *reinterpret_cast<const uint4*>(stg), bq = *reinterpret_cast<const uint4*>(stg + 2048);
      X[0] = a.x; X[1] = a.y; X[2] = a.z; X[3] = a.w; X[4] = bq.x; X[5] = bq.y; X[6] = bq.z; X[7] = bq.w;
    };
    auto expand_k = [&](int c) {
      wait(B_FULL + c % NS, c / NS, 0x300u);
      uint32_t X[8];
      load_x(c, 4096, X);
      const bool valid = c * C + t < L;
      if (!valid) {  // tokens past the end contribute nothing to the state: phi'(K) = 0, also the constant
#pragma unroll
        for (int m = 0; m < 8; ++m) X[m] = 0;
      }
      const uint32_t one = valid ? 0xFFFFFFFFu : 0u;
      // the phi'(K) buffer is free once the state update that read it (NPK chunks ago) has completed
      const int pkb = c % NPK;
      if (c >= NPK) wait(B_PK_FREE + pkb, c / NPK - 1, 0x302u);
      uint8_t* dst = smem + lay.phik + pkb * 40960 + t * 16;
      expand_packed(X, [&](auto G, uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3) {
        constexpr int g = decltype(G)::value;
        if constexpr (g == 0) w0 &= one;
        *reinterpret_cast<uint4*>(dst + g * 2048) = make_uint4(w0, w1, w2, w3);
      });
      fence_proxy_async();
    };
    // phi'(Q_c) from the raw q held in X (taken from the stage one step earlier, see below)
    auto expand_q = [&](int c, const uint32_t (&X)[8]) {
      if (c > 0) wait(B_O_DONE, c - 1, 0x301u);  // the previous phi'(Q) has been consumed
      fence_after_sync();
      uint32_t hold[4];
      expand_packed(X, [&](auto G, uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3) {
        constexpr int g = decltype(G)::value;
        if constexpr ((g & 1) == 0) {
          hold[0] = w0; hold[1] = w1; hold[2] = w2; hold[3] = w3;
        } else {
          const uint32_t r[8] = {hold[0], hold[1], hold[2], hold[3], w0, w1, w2, w3};
          tmem_st8(tlane + tm_pq + 4 * (g - 1), r);
        }
      });
      tmem_st_wait();
      fence_before_sync();
    };
    // phi'(Q_c) goes first in a step and is announced on its own: it only waits for the readout of chunk c - 1, and
    // the readout of chunk c needs nothing else from these warps, while phi'(K_{c+1}) also needs tile c + 1, the
    // youngest load in flight, and is only needed by the state update at the end of the MMA thread's step.  The
    // raw q of chunk c + 1 is taken into registers BEFORE the arrival for phi'(K_{c+1}), so that once the MMA
    // thread has seen that arrival nothing on the CUDA cores reads tile c + 1's q or k any more - the producer
    // relies on it when it refills a stage.  Step -1 only expands phi'(K_0); the state-only mode has no phi'(Q).
    // (One loop for both modes, so that each expansion exists once in the kernel's code: the less code lies between
    // the hot loops, the fewer instruction-cache misses reach the GPC's shared cache.)
    const bool with_q = mode != MODE_SEG_STATE;
    uint32_t XQ[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
    for (int c = -1; c < nchunks; ++c) {
      if (with_q && c >= 0) {
        expand_q(c, XQ);
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_XQ_READY));
      }
      if (c + 1 < nchunks) {
        expand_k(c + 1);                                 // waits for tile c + 1
        if (with_q) load_x(c + 1, 0, XQ);
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_XK_READY + (c + 1) % NPK));
      }
    }
  } else if (warp >= W_OUT && warp < W_MMA) {
    // ================================================================ output warps: O -> y
    __nv_bfloat16* yb = p.y + b * p.sy.b + h * p.sy.h + (int64_t)tok_base * p.sy.l;
    // 16 fp32 accumulator columns -> 8 packed bf16 pairs, scaled by the row's normaliser
    auto pack16 = [&](const uint32_t (&r)[16], float sc, uint32_t* o) {
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = pack_bf16(__uint_as_float(r[2 * e]) * sc, __uint_as_float(r[2 * e + 1]) * sc);
    };
    auto free_o = [&]() {   // the last TMEM read of O(c) is done: the next chunk may overwrite it
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_A_READY));
    };
    if (mode != MODE_SEG_STATE) {
      if (lane == 0) mbar_arrive(bar(B_A_READY));          // O is free before the first chunk
      // Each thread parks 32 columns of its normalised row in this warp's 32-row staging tile; the warp then copies
      // the tile out with every store instruction covering whole 64-byte row segments (row-per-thread stores would
      // touch 32 different lines per instruction).
      uint8_t* ytile = smem + lay.ystage + (qd * 32) * lay.yrow_bytes;
      uint8_t* yrow_s = ytile + lane * lay.yrow_bytes;
      const int n16 = dv >> 4;
      const int nrd = (n16 + 1) >> 1;                // rounds of 32 columns
      for (int c = 0; c < nchunks; ++c) {
        wait(B_O_DONE, c, 0x401u);
        fence_after_sync();
        const int tok_w = c * C + qd * 32;           // first token of this warp's tile
        __nv_bfloat16* ytok = yb + (int64_t)tok_w * p.sy.l;
        uint32_t dreg;
        tmem_ld1(tlane + TM_O + dv, dreg);           // the row's normaliser; completes with the first round's loads
        float inv = 0.f;
        // one round: 32 (or 16) normalised columns -> staging tile -> global, whole 64-byte row segments per store
        auto round_out = [&](int rd, bool two, const uint32_t (&r0)[16], const uint32_t (&r1)[16]) {
          uint32_t pk[16];
          pack16(r0, inv, pk);
          *reinterpret_cast<uint4*>(yrow_s) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          *reinterpret_cast<uint4*>(yrow_s + 16) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
          if (two) {
            pack16(r1, inv, pk + 8);
            *reinterpret_cast<uint4*>(yrow_s + 32) = make_uint4(pk[8], pk[9], pk[10], pk[11]);
            *reinterpret_cast<uint4*>(yrow_s + 48) = make_uint4(pk[12], pk[13], pk[14], pk[15]);
          }
          __syncwarp();
          // 16-byte pieces of the tile: ppr per row; piece idx = lane + 32 n -> row idx / ppr, piece idx % ppr
          const int ppr = two ? 4 : 2, sh = two ? 2 : 1;
#pragma unroll 1
          for (int n = 0; n < ppr; ++n) {
            const int idx = lane + 32 * n, r = idx >> sh, cc = idx & (ppr - 1);
            const uint4 val = *reinterpret_cast<const uint4*>(ytile + r * lay.yrow_bytes + cc * 16);
            if (tok_w + r < L) *reinterpret_cast<uint4*>(ytok + (int64_t)r * p.sy.l + 32 * rd + cc * 8) = val;
          }
          __syncwarp();  // the tile is rewritten in the next round
        };
        if (n16 == 4) {
          // dv = 64: all of O(c) into registers first, so that the accumulator is free again as early as possible
          uint32_t r0[16], r1[16], r2[16], r3[16];
          tmem_ld16(tlane + TM_O, r0);
          tmem_ld16(tlane + TM_O + 16, r1);
          tmem_ld16(tlane + TM_O + 32, r2);
          tmem_ld16(tlane + TM_O + 48, r3);
          tmem_ld_wait();
          free_o();
          inv = 1.0f / (__uint_as_float(dreg) + p.eps);
          round_out(0, true, r0, r1);
          round_out(1, true, r2, r3);
          continue;
        }
        // y = O[:, :dv] / (O[:, dv] + eps), 32 columns per round.  The loop is kept rolled: this kernel's hot
        // code has to stay inside the SM's instruction cache.
#pragma unroll 1
        for (int rd = 0; rd < nrd; ++rd) {
          const bool two = 2 * rd + 1 < n16;
          uint32_t r0[16], r1[16];
          tmem_ld16(tlane + TM_O + 32 * rd, r0);
          if (two) tmem_ld16(tlane + TM_O + 32 * rd + 16, r1);
          tmem_ld_wait();
          if (rd == 0) inv = 1.0f / (__uint_as_float(dreg) + p.eps);
          if (rd == nrd - 1) free_o();               // that was the last read of O(c)
          round_out(rd, two, r0, r1);
        }
      }
    }
  } else {
    // ================================================================ state-drain warps (4-7); warp 4 also evaluates
    // the polynomial of quadrant 0 (its rows see one 32-column piece), warp 7 half of quadrant 3's when it has no
    // state rows to drain
    auto cvt16 = [&](const uint32_t (&r)[16], uint4& lo, uint4& hi) {
      lo.x = pack_bf16(__uint_as_float(r[0]), __uint_as_float(r[1]));
      lo.y = pack_bf16(__uint_as_float(r[2]), __uint_as_float(r[3]));
      lo.z = pack_bf16(__uint_as_float(r[4]), __uint_as_float(r[5]));
      lo.w = pack_bf16(__uint_as_float(r[6]), __uint_as_float(r[7]));
      hi.x = pack_bf16(__uint_as_float(r[8]), __uint_as_float(r[9]));
      hi.y = pack_bf16(__uint_as_float(r[10]), __uint_as_float(r[11]));
      hi.z = pack_bf16(__uint_as_float(r[12]), __uint_as_float(r[13]));
      hi.w = pack_bf16(__uint_as_float(r[14]), __uint_as_float(r[15]));
    };
    // final fp32 state^T -> shared memory at offset 0 (every MMA and every other warp's use of the stages is
    // over by then).  The TMEM loads are warp-collective, so every lane issues them; only rows < NV are kept.
    auto stage_state = [&]() {
      float* stg = reinterpret_cast<float*>(smem) + t * STAGE_STRIDE_F;
#pragma unroll 1
      for (int i = 0; i < 10; ++i) {
        uint32_t r[16];
        tmem_ld16(tlane + TM_ST + 16 * i, r);
        tmem_ld_wait();
        if (t < NV) {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            *reinterpret_cast<uint4*>(stg + 16 * i + 4 * e) = make_uint4(r[4 * e], r[4 * e + 1], r[4 * e + 2], r[4 * e + 3]);
        }
      }
    };
    // bf16 copy of 32 feature columns of this thread's state row into operand buffer `buf`
    auto store_stb = [&](int buf, int i, const uint32_t (&r0)[16], const uint32_t (&r1)[16]) {
      uint4 a0, a1, b0, b1;
      cvt16(r0, a0, a1);
      cvt16(r1, b0, b1);
      if (t < NV) {  // rows >= NV of the B operand do not exist (N = NV)
        uint8_t* dst = smem + lay.stb + buf * lay.stb_bytes + (4 * i) * (NV * 16) + t * 16;
        *reinterpret_cast<uint4*>(dst) = a0;
        *reinterpret_cast<uint4*>(dst + NV * 16) = a1;
        *reinterpret_cast<uint4*>(dst + 2 * NV * 16) = b0;
        *reinterpret_cast<uint4*>(dst + 3 * NV * 16) = b1;
      }
    };
    const bool my_rows = qd * 32 < NV;                       // warp-uniform: this quadrant holds state rows
    // polynomial pieces [0, pp1) of this warp: all of quadrant 0 (one piece to evaluate, three to clear), the first
    // two of quadrant 3 when warp 15 shares it
    const int pp1 = qd == 0 ? 4 : ((qd == 3 && !q3_has_state) ? 2 : 0);
    if (mode == MODE_SEG_STATE) {
      wait(B_FIN, 0, 0x410u);
      fence_after_sync();
      stage_state();
    } else {
      const int share = (qd == 3 && pp1 > 0) ? 1 : 0;
      if (pp1 > 0) make_p(0, 0, pp1, share, false);
      if (has_init) {
        // Preload state^T (fp32, TMEM) and its bf16 operand copy (buffer 1) with the sum over the earlier segments.
        const float* src = p.seg_state + ((size_t)bh * (p.nseg - 1) + (seg - 1)) * (size_t)((dv + 1) * DR) + (size_t)t * DR;
        const bool row = t <= dv;
#pragma unroll 1
        for (int i = 0; i < 5; ++i) {
          uint32_t r0[16], r1[16];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint4 x = row ? __ldg(reinterpret_cast<const uint4*>(src + 32 * i + 4 * e)) : make_uint4(0, 0, 0, 0);
            const uint4 y2 = row ? __ldg(reinterpret_cast<const uint4*>(src + 32 * i + 16 + 4 * e)) : make_uint4(0, 0, 0, 0);
            r0[4 * e] = x.x; r0[4 * e + 1] = x.y; r0[4 * e + 2] = x.z; r0[4 * e + 3] = x.w;
            r1[4 * e] = y2.x; r1[4 * e + 1] = y2.y; r1[4 * e + 2] = y2.z; r1[4 * e + 3] = y2.w;
          }
          tmem_st16(tlane + TM_ST + 32 * i, r0);
          tmem_st16(tlane + TM_ST + 32 * i + 16, r1);
          store_stb(1, i, r0, r1);
        }
        tmem_st_wait();
        fence_proxy_async();
        fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_INIT));
      }
      for (int c = 0; c < nchunks; ++c) {
        const bool last = c + 1 == nchunks;
        // ---- state after chunk c: fp32 TMEM -> bf16 smem operand (buffer c & 1), or fp32 staging at the end ----
        wait(B_PK_FREE + c % NPK, c / NPK, 0x402u);   // the state update of chunk c is complete
        fence_after_sync();
        if (!last) {
          if (my_rows) {
            // 32 feature columns per round trip, the next round's loads in flight while this one is converted
            uint32_t ra[16], rb[16], rc[16], rd[16];
            tmem_ld16(tlane + TM_ST, ra);
            tmem_ld16(tlane + TM_ST + 16, rb);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 5; ++i) {
              if (i & 1) {
                if (i < 4) { tmem_ld16(tlane + TM_ST + 32 * (i + 1), ra); tmem_ld16(tlane + TM_ST + 32 * (i + 1) + 16, rb); }
                store_stb(c & 1, i, rc, rd);
              } else {
                if (i < 4) { tmem_ld16(tlane + TM_ST + 32 * (i + 1), rc); tmem_ld16(tlane + TM_ST + 32 * (i + 1) + 16, rd); }
                store_stb(c & 1, i, ra, rb);
              }
              if (i < 4) tmem_ld_wait();
            }
          }
          fence_proxy_async();
          fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(B_STB_READY));
          if (pp1 > 0) make_p(c + 1, 0, pp1, share, false);
        } else if (write_state) {
          wait(B_FIN, 0, 0x404u);   // the last chunk's P V' and readout still read the stages and the operand buffers
          fence_after_sync();
          stage_state();
        }
      }
    }
  }

  // ------------------------------------------------------------------ final state, reference layout
  fence_before_sync();
  __syncthreads();
  if (mode == MODE_SEG_STATE) {
    // packed fp32 rows 0..dv, as they are
    const float* stg = reinterpret_cast<const float*>(smem);
    float* dst = p.seg_state + ((size_t)bh * (p.nseg - 1) + seg) * (size_t)((dv + 1) * DR);
    for (int e = tid; e < (dv + 1) * (DR / 4); e += NT) {
      const int n = e / (DR / 4), f4 = e - n * (DR / 4);
      reinterpret_cast<float4*>(dst)[e] = *reinterpret_cast<const float4*>(stg + n * STAGE_STRIDE_F + 4 * f4);
    }
  } else if (write_state) {
    const float* stg = reinterpret_cast<const float*>(smem);
    // thread f walks the dv + 1 rows of feature f: its place in the packed vector is worked out once, and a warp's
    // stores of one row are contiguous
    for (int f = tid; f < kExpandedDim; f += NT) {
      bool offdiag;
      const int idx = packed_index(f, offdiag);
      const float scale = offdiag ? 0.70710678118654752f : 1.0f;
      const size_t kv0 = (size_t)bh * dv * kExpandedDim + f;
#pragma unroll 4
      for (int n = 0; n < dv; ++n) {
        const float val = stg[n * STAGE_STRIDE_F + idx] * scale;
        const size_t o = kv0 + (size_t)n * kExpandedDim;
        if (p.state_bf16) static_cast<__nv_bfloat16*>(p.kv_state)[o] = __float2bfloat16_rn(val);
        else static_cast<float*>(p.kv_state)[o] = val;
      }
      const float val = stg[dv * STAGE_STRIDE_F + idx] * scale;
      const size_t o = (size_t)bh * kExpandedDim + f;
      if (p.state_bf16) static_cast<__nv_bfloat16*>(p.k_state)[o] = __float2bfloat16_rn(val);
      else static_cast<float*>(p.k_state)[o] = val;
    }
  }
  __syncthreads();
  if (warp == 0) {
    fence_after_sync();
    tmem_dealloc(tmem, TM_COLS);
  }
}

// In place over the segments of one (batch, head): x[s] <- x[0] + ... + x[s], so that slot s holds
// the state at the start of segment s + 1.  grid = (ceil(per / 256), batch x head).
__global__ void __launch_bounds__(256) segment_scan_kernel(float* __restrict__ x, int nslots, int per) {
  const int e = blockIdx.x * 256 + threadIdx.x;
  if (e >= per) return;
  float* col = x + (size_t)blockIdx.y * nslots * per + e;
  float acc = col[0];
  for (int s = 1; s < nslots; ++s) {
    acc += col[(size_t)s * per];
    col[(size_t)s * per] = acc;
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

// Segment plan for a split of about `want` segments: whole chunks per segment, no empty segment.
static void plan_segments(int L, int want, int* nseg, int* seg_chunks) {
  const int chunks = (L + C - 1) / C;
  want = want < 1 ? 1 : (want > chunks ? chunks : want);
  *seg_chunks = (chunks + want - 1) / want;
  *nseg = (chunks + *seg_chunks - 1) / *seg_chunks;
}

int linattn_prefill_tc_auto_segments(int B, int H, int L) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return 1;
  const int64_t bh = (int64_t)B * H;
  const int chunks = (L + C - 1) / C;
  if (bh <= 0 || bh * 2 > sms || chunks < 8) return 1;  // the grid already fills the machine, or nothing to split
  int want = (int)(sms / bh);
  if (want > chunks / 4) want = chunks / 4;             // at least four chunks per segment
  int nseg, seg_chunks;
  plan_segments(L, want, &nseg, &seg_chunks);
  return nseg;
}

size_t linattn_prefill_tc_scratch_bytes(int B, int H, int L, int dv, int nseg) {
  int n, sc;
  plan_segments(L, nseg, &n, &sc);
  return (size_t)B * H * (n - 1) * (dv + 1) * DR * sizeof(float);
}

// Once per device: the address of the status word and the kernel's shared-memory limit (both are properties of
// the device's primary context and stay valid for its lifetime).
struct DeviceInit {
  bool done = false;
  unsigned int* status = nullptr;
};
static int device_init(unsigned int** status) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static DeviceInit init[kMaxDevices];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return BASED_ERR_TOO_LARGE;
  std::lock_guard<std::mutex> lock(mu);
  if (!init[dev].done) {
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&init[dev].status), g_tc_status);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(linattn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem(112).total > Smem(64).total ? Smem(112).total : Smem(64).total);
    if (e != cudaSuccess) return (int)e;
    init[dev].done = true;
  }
  *status = init[dev].status;
  return 0;
}

// Tensor map of a [B][H][L][row] operand whose rows (`groups` x 8 bf16) are cut into 16-byte groups; cached.
static int grouped_map(CUtensorMap* out, const void* base, int groups, int L, int H, int B, Strides3 s) {
  static tma::MapCache cache;
  // an extent of 1 may come with any stride: give it a harmless one
  const int64_t sh = H == 1 ? 8 : s.h, sbb = B == 1 ? 8 : s.b, sl = L == 1 ? 8 * groups : s.l;
  if (sh <= 0 || sbb <= 0 || sl <= 0) return BASED_ERR_IMPL;
  const tma::MapKey key = tma::make_key(base, 8, (uint64_t)L, (uint64_t)groups, (uint64_t)H, (uint64_t)B, sl, 8, sh, sbb, 8, C,
                                        (uint32_t)groups, 5);
  if (cache.find(key, out)) return 0;
  if (tma::encode_bf16_grouped_rows(out, base, (uint64_t)groups, (uint64_t)L, (uint64_t)H, (uint64_t)B, sl, sh, sbb, C))
    return BASED_ERR_IMPL;
  cache.put(key, *out);
  return 0;
}

int launch_linattn_prefill_tc(const void* q, const void* k, const void* v, void* y, void* kv_state, void* k_state,
                              int B, int H, int L, int dv, Strides3 sq, Strides3 sk, Strides3 sv, Strides3 sy,
                              int state_dtype, float eps, int nseg, void* scratch, size_t scratch_bytes,
                              cudaStream_t stream) {
  // Requirements of this kernel; the caller may fall back to the CUDA-core kernel on ERR_IMPL.
  if (dv > 112) return BASED_ERR_IMPL;  // V' = dv + 16 columns must fit the 128 TMEM lanes
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(y)) return BASED_ERR_IMPL;
  const int64_t all[] = {sq.b, sq.h, sq.l, sk.b, sk.h, sk.l, sv.b, sv.h, sv.l, sy.b, sy.h, sy.l};
  for (int64_t s : all)
    if (s % 8 != 0) return BASED_ERR_IMPL;  // 16-byte vector accesses on every row
  Params p;
  int rc = grouped_map(&p.mq, q, 2, L, H, B, sq);
  if (rc == 0) rc = grouped_map(&p.mk, k, 2, L, H, B, sk);
  if (rc == 0) rc = grouped_map(&p.mv, v, dv / 8, L, H, B, sv);
  if (rc != 0) return rc;
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
  rc = device_init(&p.status);
  if (rc != 0) return rc;
  const Smem lay(dv);
  int seg_chunks;
  plan_segments(L, nseg, &nseg, &seg_chunks);
  p.nseg = nseg;
  p.seg_chunks = seg_chunks;
  p.seg_state = static_cast<float*>(scratch);
  auto launch_outputs = [&](int grid) -> int {
    linattn_prefill_tc_kernel<<<grid, NT, lay.total, stream>>>(p);
    return (int)cudaGetLastError();
  };
  if (nseg == 1) {
    p.mode = MODE_WHOLE;
    p.grid_segs = 1;
    return launch_outputs(B * H);
  }
  // Three launches: per-segment states, their running sum, then the outputs of every segment.
  if ((int64_t)B * H * nseg > 0x7fffffff) return BASED_ERR_SHAPE;
  if (scratch == nullptr || !aligned16(scratch) ||
      scratch_bytes < (size_t)B * H * (nseg - 1) * (dv + 1) * DR * sizeof(float))
    return BASED_ERR_SCRATCH;
  const int per = (dv + 1) * DR;
  p.mode = MODE_SEG_STATE;
  p.grid_segs = nseg - 1;
  linattn_prefill_tc_kernel<<<B * H * (nseg - 1), NT, lay.total, stream>>>(p);
  if (nseg > 2)
    segment_scan_kernel<<<dim3((per + 255) / 256, B * H), 256, 0, stream>>>(p.seg_state, nseg - 1, per);
  p.mode = MODE_SEG_OUTPUT;
  p.grid_segs = nseg;
  return launch_outputs(B * H * nseg);
}

int launch_linattn_prefill_tc_static(const void* q, const void* k, const void* v, void* y, void* kv_state,
                                     void* k_state, int B, int H, int L, int dv, Strides3 sq, Strides3 sk,
                                     Strides3 sv, Strides3 sy, int state_dtype, float eps, int nseg,
                                     cudaStream_t stream) {
  if (linattn_prefill_tc_scratch_bytes(B, H, L, dv, nseg) > (size_t)BASED_STATIC_SCRATCH_BYTES)
    return BASED_ERR_TOO_LARGE;
  // The symbol's address, resolved once per device (each device has its own copy of the array).
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static void* addr[kMaxDevices] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return BASED_ERR_TOO_LARGE;
  void* scratch;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (addr[dev] == nullptr) {
      e = cudaGetSymbolAddress(&addr[dev], g_static_scratch);
      if (e != cudaSuccess) {
        addr[dev] = nullptr;
        return (int)e;
      }
    }
    scratch = addr[dev];
  }
  return launch_linattn_prefill_tc(q, k, v, y, kv_state, k_state, B, H, L, dv, sq, sk, sv, sy, state_dtype, eps, nseg,
                                   scratch, BASED_STATIC_SCRATCH_BYTES, stream);
}

}  // namespace based
