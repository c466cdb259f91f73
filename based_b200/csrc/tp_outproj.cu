// Row-parallel output projection of a decode step fused with the tensor-parallel all-reduce:
//   out[M, N] = sum over ranks r of  x_r[M, K_r] W_r[N, K_r]^T   (+ bias, added once)
// in ONE kernel per rank.  Each rank computes its partial tile on the tensor cores (mma.sync: M <= 64
// rows of single tokens, the product is bound by reading W_r once, as in decode_linear.cu), PUSHES
// the fp32 tile into every rank's receive buffer with plain peer stores over NVLink, publishes a
// per-tile flag, waits (bounded) for the same tile from every rank, and adds the partials in rank
// order - so every rank computes bit-identical sums - before rounding to bf16 once.
//
// Models RowParallelLinear.forward of the reference (based/ops/fused_dense.py:239-246: local GEMM,
// then all_reduce of the [B, L, d_model] output), which runs as a cuBLAS GEMM followed by a NCCL
// all-reduce; at decode sizes (229 KB at B = 64, d_model = 1792) both are latency-bound launches.
// No TMA, no multicast, no library kernel touches peer memory: only st/ld.global on mapped peer
// addresses.
//
// Receive workspace of one rank (symmetric: same layout on every rank, zero-filled once):
//   [0, 256)                         control: word 0 = epoch of the NEXT call, word 1 = finished-block ticket
//   [256, 256 + 2*W*T*4)             flags[parity][src rank][tile]   (uint32: the epoch whose data is complete;
//                                    a tile = 8 output columns, all rows)
//   then                             data[parity][src rank][Mmax rows][N] fp32
// with W = world size, T = tile count.  The epoch lives on the device and is advanced by the last
// block of a launch, so a captured launch can be replayed; parity = epoch & 1 alternates two sets of
// buffers, which is enough because a rank cannot finish call e + 1 before every rank has finished
// call e (it needs their tiles of call e + 1, pushed by kernels that run after their call e).
#include "common.cuh"

#include <mutex>

namespace based {

__device__ unsigned int g_tp_status = 0;  // ORed with a code when a bounded wait expires

namespace {

constexpr int WARPS = 8;     // the K slice of a rank is split over the warps: one round of loads in flight per warp
constexpr int kMaxWorld = 8;
constexpr int kCtrlBytes = 256;

struct TpParams {
  const __nv_bfloat16* x[kMaxWorld];    // one entry in real use (index 0); one per emulated rank otherwise
  const __nv_bfloat16* w[kMaxWorld];
  __nv_bfloat16* out[kMaxWorld];
  unsigned char* ws[kMaxWorld];         // every rank's workspace, as mapped into THIS process
  const __nv_bfloat16* bias;            // [N] or null; added by every rank after the sum (the sum is replicated)
  int M, N, K, Mmax, world, rank, emulate;
  int64_t sx, so;
  unsigned int* status;
  long long max_wait_cycles;
};

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned int ld_relaxed_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// data written by a peer: read past L1 (a line of the previous use of this buffer may still sit there)
__device__ __forceinline__ float2 ld_peer_written(const float* p) {
  float2 v;
  asm volatile("ld.relaxed.sys.global.v2.f32 {%0, %1}, [%2];\n" : "=f"(v.x), "=f"(v.y) : "l"(p) : "memory");
  return v;
}

__host__ __device__ inline size_t flags_offset() { return kCtrlBytes; }
__host__ __device__ inline size_t data_offset(int world, int tiles) {
  return (kCtrlBytes + (size_t)2 * world * tiles * 4 + 255) / 256 * 256;
}

constexpr int kMaxRowTiles = 4;   // 16-row tiles per block: max_rows <= 64

// grid = (N / 8, 1, ranks emulated in this launch (1 in real use)); block = WARPS x 32.  A block owns 8 output
// columns for ALL rows: its weight rows are read once and applied to every 16-row tile.
__global__ void __launch_bounds__(WARPS * 32) tp_outproj_allreduce_kernel(const TpParams p) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int slot = p.emulate ? (int)blockIdx.z : 0;          // which of the pointer sets this block uses
  const int rank = p.emulate ? (int)blockIdx.z : p.rank;
  const int n0 = blockIdx.x * 8;
  const int tiles = gridDim.x, tile = blockIdx.x;
  const int mtiles = (p.M + 15) >> 4;
  unsigned char* my_ws = p.ws[rank];
  unsigned int* ctrl = reinterpret_cast<unsigned int*>(my_ws);
  // The epoch of this call: written by the last block of the previous launch on this GPU (1 after the workspace was
  // prepared), so the kernel boundary already orders it.  ONE thread reads it: an acquire at system scope by every
  // thread of every block costs each warp a system-wide fence, and those queue up per SM.
  __shared__ unsigned int s_epoch;
  if (threadIdx.x == 0) s_epoch = ld_relaxed_sys(ctrl);
  __syncthreads();
  const unsigned int epoch = s_epoch;
  const int parity = epoch & 1u;

  // ---- partial products of this rank: all rows, columns n0..n0+7, over the rank's K slice (split over the warps)
  const int kblocks = p.K / 32, per = (kblocks + WARPS - 1) / WARPS;
  const int kb0 = warp * per, kb1 = min(kb0 + per, kblocks);
  const __nv_bfloat16* wr = p.w[slot] + (int64_t)(n0 + g) * p.K + 8 * t;
  const __nv_bfloat16* xr = p.x[slot] + 8 * t;
  float acc[kMaxRowTiles][4];
#pragma unroll
  for (int m = 0; m < kMaxRowTiles; ++m)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[m][e] = 0.f;
  constexpr int U = 4;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  for (int kb = kb0; kb < kb1; kb += U) {
    uint4 wv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) wv[u] = (kb + u < kb1) ? __ldg(reinterpret_cast<const uint4*>(wr + (kb + u) * 32)) : zero;
#pragma unroll
    for (int m = 0; m < kMaxRowTiles; ++m) {
      if (m < mtiles) {
        const int r0 = 16 * m + g, r1 = r0 + 8;
        const bool v0 = r0 < p.M, v1 = r1 < p.M;
        uint4 a0[U], a1[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const bool ok = kb + u < kb1;
          const int ko = (kb + u) * 32;
          a0[u] = (ok && v0) ? __ldg(reinterpret_cast<const uint4*>(xr + (int64_t)r0 * p.sx + ko)) : zero;
          a1[u] = (ok && v1) ? __ldg(reinterpret_cast<const uint4*>(xr + (int64_t)r1 * p.sx + ko)) : zero;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const uint32_t fa[4] = {a0[u].x, a1[u].x, a0[u].y, a1[u].y};
          const uint32_t fb[4] = {a0[u].z, a1[u].z, a0[u].w, a1[u].w};
          mma_16816(acc[m], fa, wv[u].x, wv[u].y);
          mma_16816(acc[m], fb, wv[u].z, wv[u].w);
        }
      }
    }
  }
  __shared__ float red[WARPS][kMaxRowTiles][4][32];
  __shared__ int s_ok;
#pragma unroll
  for (int m = 0; m < kMaxRowTiles; ++m)
#pragma unroll
    for (int e = 0; e < 4; ++e) red[warp][m][e][lane] = acc[m][e];
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  // From here warp m owns row tile m (rows 16m .. 16m+15) of the block's 8 columns: the four warps push, wait and
  // add side by side, so the chain of NVLink round trips a block goes through is as short as one tile's.
  static_assert(kMaxRowTiles <= WARPS, "one warp per row tile");
  const int m = warp < kMaxRowTiles ? warp : 0;
  const bool have = warp < kMaxRowTiles && warp < mtiles;
  float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
#pragma unroll
    for (int w = 0; w < WARPS; ++w) part[e] += red[w][m][e][lane];
  }
  // this lane holds rows 16m + g (part 0, 1) and 16m + g + 8 (part 2, 3), columns c0 and c0 + 1
  const int c0 = n0 + 2 * t;
  const int r0 = 16 * m + g, r1 = r0 + 8;
  const bool v0 = have && r0 < p.M, v1 = have && r1 < p.M;
  const size_t doff = data_offset(p.world, tiles);
  const size_t slab = (size_t)p.Mmax * p.N;                               // floats per (parity, src rank)
  const size_t my_slab = ((size_t)parity * p.world + rank) * slab;
  // ---- push the tile column into every rank's receive buffer (own included), then publish its flag there
  for (int d = 0; d < p.world; ++d) {
    const int dst = (rank + d) % p.world;                                  // spread the first stores over the peers
    float* data = reinterpret_cast<float*>(p.ws[dst] + doff) + my_slab;
    if (v0) *reinterpret_cast<float2*>(data + (size_t)r0 * p.N + c0) = make_float2(part[0], part[1]);
    if (v1) *reinterpret_cast<float2*>(data + (size_t)r1 * p.N + c0) = make_float2(part[2], part[3]);
  }
  // The block's stores are ordered before the flags by the barrier (all threads) followed by ONE release at system
  // scope per flag (release is cumulative over what the barrier ordered before it): a system-wide fence by every
  // thread instead cost 6 us per call.
  __syncthreads();
  if (threadIdx.x < p.world) {
    const int lane_rank = threadIdx.x;
    const int dst = (rank + lane_rank) % p.world;
    unsigned int* flags = reinterpret_cast<unsigned int*>(p.ws[dst] + flags_offset());
    st_release_sys(flags + ((size_t)parity * p.world + rank) * tiles + tile, epoch);
    // ---- wait for this tile column from every rank (thread s watches source rank s), bounded:
    // relaxed polls (a load each), then ONE acquire that orders the reads of the partials behind the flag
    const unsigned int* flag =
        reinterpret_cast<const unsigned int*>(my_ws + flags_offset()) + ((size_t)parity * p.world + lane_rank) * tiles + tile;
    if (ld_relaxed_sys(flag) != epoch) {
      const long long t0 = clock64();
      while (ld_relaxed_sys(flag) != epoch) {
        if (clock64() - t0 > p.max_wait_cycles) {
          s_ok = 0;
          if (p.status) atomicOr(p.status, 0x1000u | (unsigned)lane_rank);
          break;
        }
        __nanosleep(32);
      }
    }
    (void)ld_acquire_sys(flag);
  }
  __syncthreads();
  const bool ok = s_ok != 0;
  // ---- sum the partials in rank order (all loads first, then the adds), add the bias, round once
  const float* mine = reinterpret_cast<const float*>(my_ws + doff) + (size_t)parity * p.world * slab;
  float2 in0[kMaxWorld], in1[kMaxWorld];
#pragma unroll
  for (int src = 0; src < kMaxWorld; ++src) {
    in0[src] = make_float2(0.f, 0.f);
    in1[src] = make_float2(0.f, 0.f);
    if (src < p.world) {
      const float* data = mine + (size_t)src * slab;
      if (v0) in0[src] = ld_peer_written(data + (size_t)r0 * p.N + c0);
      if (v1) in1[src] = ld_peer_written(data + (size_t)r1 * p.N + c0);
    }
  }
  float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int src = 0; src < kMaxWorld; ++src) {
    if (src < p.world) { sum[0] += in0[src].x; sum[1] += in0[src].y; sum[2] += in1[src].x; sum[3] += in1[src].y; }
  }
  if (p.bias) {
    const float b0 = __bfloat162float(p.bias[c0]), b1 = __bfloat162float(p.bias[c0 + 1]);
    sum[0] += b0; sum[1] += b1; sum[2] += b0; sum[3] += b1;
  }
  if (!ok) { sum[0] = sum[1] = sum[2] = sum[3] = __int_as_float(0x7fc00000); }   // a partial never came: NaN, not a silent sum
  __nv_bfloat16* out = p.out[slot];
  if (v0) *reinterpret_cast<__nv_bfloat162*>(out + (int64_t)r0 * p.so + c0) = __floats2bfloat162_rn(sum[0], sum[1]);
  if (v1) *reinterpret_cast<__nv_bfloat162*>(out + (int64_t)r1 * p.so + c0) = __floats2bfloat162_rn(sum[2], sum[3]);
  // ---- the last block of this rank's launch advances the epoch for the next call
  __syncthreads();
  // (nothing of this block has to be ordered before the count: the next launch starts after this one has ended)
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(ctrl + 1, 1u);
    if (done == (unsigned)tiles - 1) {
      ctrl[1] = 0;
      st_release_sys(ctrl, epoch + 1u);
    }
  }
}

}  // namespace

int read_tp_status(unsigned int* out, int reset) {
  unsigned int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_tp_status, sizeof(v));
  if (e != cudaSuccess) return (int)e;
  if (out) *out = v;
  if (reset && v != 0) {
    v = 0;
    e = cudaMemcpyToSymbol(g_tp_status, &v, sizeof(v));
  }
  return (int)e;
}

size_t tp_outproj_workspace_bytes(int world, int Mmax, int N) {
  if (world < 1 || world > kMaxWorld || Mmax < 1 || N < 8 || N % 8 != 0) return 0;
  if (Mmax > 16 * kMaxRowTiles) return 0;
  const int tiles = N / 8;
  return data_offset(world, tiles) + (size_t)2 * world * Mmax * N * sizeof(float);
}

int launch_tp_outproj_allreduce(const void* const* x, const void* const* w, const void* bias, void* const* out,
                                void* const* workspaces, int M, int N, int K, int64_t sx, int64_t so, int Mmax,
                                int rank, int world, int emulate, cudaStream_t stream) {
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) return BASED_ERR_SHAPE;
  if (M < 1 || M > Mmax || Mmax > 16 * kMaxRowTiles || N % 8 != 0 || K % 32 != 0 || sx % 8 != 0 || so % 2 != 0)
    return BASED_ERR_SHAPE;
  TpParams p;
  const int sets = emulate ? world : 1;
  for (int i = 0; i < kMaxWorld; ++i) { p.x[i] = nullptr; p.w[i] = nullptr; p.out[i] = nullptr; p.ws[i] = nullptr; }
  for (int i = 0; i < sets; ++i) {
    if (!x[i] || !w[i] || !out[i]) return BASED_ERR_NULL;
    if (!aligned16(x[i]) || !aligned16(w[i]) || (reinterpret_cast<uintptr_t>(out[i]) & 3u)) return BASED_ERR_ALIGN;
    p.x[i] = static_cast<const __nv_bfloat16*>(x[i]);
    p.w[i] = static_cast<const __nv_bfloat16*>(w[i]);
    p.out[i] = static_cast<__nv_bfloat16*>(out[i]);
  }
  for (int i = 0; i < world; ++i) {
    if (!workspaces[i]) return BASED_ERR_NULL;
    if (reinterpret_cast<uintptr_t>(workspaces[i]) & 255u) return BASED_ERR_ALIGN;
    p.ws[i] = static_cast<unsigned char*>(workspaces[i]);
  }
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.M = M; p.N = N; p.K = K; p.Mmax = Mmax; p.world = world; p.rank = rank; p.emulate = emulate ? 1 : 0;
  p.sx = sx; p.so = so;
  p.max_wait_cycles = 2000000000LL;
  // Once per device: the status word's address, the SM count and how many blocks of this kernel an SM holds.
  constexpr int kMaxDevices = 64;
  struct DeviceInfo { bool done = false; unsigned int* status = nullptr; int sms = 0, per_sm = 0; };
  static std::mutex mu;
  static DeviceInfo info[kMaxDevices];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return BASED_ERR_TOO_LARGE;
  int sms = 0, per_sm = 0;
  {
    std::lock_guard<std::mutex> lock(mu);
    DeviceInfo& di = info[dev];
    if (!di.done) {
      if ((e = cudaGetSymbolAddress(reinterpret_cast<void**>(&di.status), g_tp_status)) != cudaSuccess) return (int)e;
      if ((e = cudaDeviceGetAttribute(&di.sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
      if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&di.per_sm, tp_outproj_allreduce_kernel, WARPS * 32, 0)) !=
          cudaSuccess)
        return (int)e;
      di.done = true;
    }
    p.status = di.status;
    sms = di.sms;
    per_sm = di.per_sm;
  }
  const dim3 grid(N / 8, 1, sets);
  // Blocks wait for blocks of other ranks that handle the same tile: every block of the launch must be resident.
  if ((long long)grid.x * grid.y * grid.z > (long long)per_sm * sms) return BASED_ERR_TOO_LARGE;
  if (emulate) {
    // several ranks inside one launch wait on one another: co-residency must be guaranteed, not just likely
    void* args[] = {&p};
    e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(tp_outproj_allreduce_kernel), grid, dim3(WARPS * 32), args, 0,
                                    stream);
    return (int)e;
  }
  tp_outproj_allreduce_kernel<<<grid, WARPS * 32, 0, stream>>>(p);
  return (int)cudaGetLastError();
}

}  // namespace based
