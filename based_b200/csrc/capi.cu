// extern "C" entry points: host-side argument validation, then dispatch to the launchers.
// Nothing here allocates device memory.  The launches are asynchronous; the one call that waits for the device
// is based_read_status (a blocking copy of the status words).
#include "common.cuh"

using namespace based;

namespace {

bool dtype_ok(int dt) { return dt == BASED_F32 || dt == BASED_BF16; }
size_t dtype_size(int dt) { return dt == BASED_F32 ? 4 : 2; }
Strides3 s3(const int64_t* s) { return Strides3{s[0], s[1], s[2]}; }       // given as (batch, head, seq)
Strides3 s3_blh(const int64_t* s) { return Strides3{s[0], s[2], s[1]}; }   // given as (batch, seq, head)
Strides2 s2(const int64_t* s) { return Strides2{s[0], s[1]}; }

}  // namespace

extern "C" {

int based_b200_version(void) { return 1; }

const char* based_error_string(int code) {
  switch (code) {
    case BASED_OK: return "ok";
    case BASED_ERR_NULL: return "a required pointer is NULL";
    case BASED_ERR_SHAPE: return "unsupported shape";
    case BASED_ERR_DTYPE: return "unsupported dtype";
    case BASED_ERR_ALIGN: return "pointer or stride not aligned as required";
    case BASED_ERR_IMPL: return "requested implementation cannot run these arguments";
    case BASED_ERR_TOO_LARGE: return "size exceeds a fixed capacity";
    case BASED_ERR_SCRATCH: return "workspace is NULL, misaligned or too small";
    default: break;
  }
  if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
  return "unknown error";
}

int based_read_status(unsigned int* out, int reset) {
  unsigned int a = 0, b = 0, c = 0;
  int rc = read_tc_status(&a, reset);
  if (rc == 0) rc = read_tc_status_swa(&b, reset);
  if (rc == 0) rc = read_tp_status(&c, reset);
  if (out) *out = a | b | c;
  return rc;
}

}  // extern "C"

namespace {

// Checks shared by the whole-sequence entry points.  Returns kDone when the call is already complete
// (nothing to compute), 0 to go on, a negative code to reject.
constexpr int kDone = 0x40000000;  // not a cudaError_t value
int prefill_preamble(const void* q, const void* k, const void* v, void* y, void* kv_state, void* k_state, int B,
                     int H, int L, int d, int dv, const int64_t* q_strides, const int64_t* k_strides,
                     const int64_t* v_strides, const int64_t* y_strides, int io_dtype, int state_dtype,
                     cudaStream_t st) {
  if (!q || !k || !v || !y || !q_strides || !k_strides || !v_strides || !y_strides) return BASED_ERR_NULL;
  if ((kv_state == nullptr) != (k_state == nullptr)) return BASED_ERR_NULL;
  if (!dtype_ok(io_dtype) || !dtype_ok(state_dtype)) return BASED_ERR_DTYPE;
  if (B < 0 || H < 0 || L < 0 || d != kFeatureDim || dv < 16 || dv > 128 || dv % 16 != 0) return BASED_ERR_SHAPE;
  if ((int64_t)B * H > 2147483647LL) return BASED_ERR_TOO_LARGE;
  if (B == 0 || H == 0) return kDone;
  if (L == 0) {
    // empty sequence: the states are the empty sums
    if (kv_state) {
      const size_t es = dtype_size(state_dtype);
      cudaError_t e = cudaMemsetAsync(kv_state, 0, (size_t)B * H * dv * kExpandedDim * es, st);
      if (e == cudaSuccess) e = cudaMemsetAsync(k_state, 0, (size_t)B * H * kExpandedDim * es, st);
      return e == cudaSuccess ? kDone : (int)e;
    }
    return kDone;
  }
  return 0;
}

}  // namespace

extern "C" {

int based_linattn_prefill(const void* q, const void* k, const void* v, void* y, void* kv_state, void* k_state,
                          int B, int H, int L, int d, int dv, const int64_t q_strides[3],
                          const int64_t k_strides[3], const int64_t v_strides[3], const int64_t y_strides[3],
                          int io_dtype, int state_dtype, float eps, int impl, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int pre = prefill_preamble(q, k, v, y, kv_state, k_state, B, H, L, d, dv, q_strides, k_strides, v_strides,
                                   y_strides, io_dtype, state_dtype, st);
  if (pre != 0) return pre == kDone ? BASED_OK : pre;
  // AUTO: the tensor-core kernel when it accepts the arguments (bf16 I/O, its alignment
  // rules), else the CUDA-core kernel.  Both are GPU kernels; there is no host path.
  const bool autosel = impl == BASED_IMPL_AUTO;
  if (autosel) impl = (io_dtype == BASED_BF16) ? BASED_IMPL_TCGEN05 : BASED_IMPL_SIMT;
  if (impl == BASED_IMPL_TCGEN05) {
    if (io_dtype != BASED_BF16) return BASED_ERR_IMPL;
    const int rc = launch_linattn_prefill_tc(q, k, v, y, kv_state, k_state, B, H, L, dv, s3(q_strides),
                                             s3(k_strides), s3(v_strides), s3(y_strides), state_dtype, eps, 1,
                                             nullptr, 0, st);
    if (!(autosel && rc == BASED_ERR_IMPL)) return rc;
    impl = BASED_IMPL_SIMT;
  }
  if (impl != BASED_IMPL_SIMT) return BASED_ERR_IMPL;
  return launch_linattn_prefill_simt(q, k, v, y, kv_state, k_state, B, H, L, dv, s3(q_strides), s3(k_strides),
                                     s3(v_strides), s3(y_strides), io_dtype, state_dtype, eps, st);
}

int based_linattn_prefill_segments(int B, int H, int L) {
  if (B <= 0 || H <= 0 || L <= 0) return 1;
  return linattn_prefill_tc_auto_segments(B, H, L);
}

size_t based_linattn_prefill_scratch_bytes(int B, int H, int L, int dv, int nseg) {
  if (B <= 0 || H <= 0 || L <= 0 || dv <= 0 || nseg <= 1) return 0;
  return linattn_prefill_tc_scratch_bytes(B, H, L, dv, nseg);
}

int based_linattn_prefill_split(const void* q, const void* k, const void* v, void* y, void* kv_state,
                                void* k_state, int B, int H, int L, int d, int dv, const int64_t q_strides[3],
                                const int64_t k_strides[3], const int64_t v_strides[3],
                                const int64_t y_strides[3], int state_dtype, float eps, int nseg, void* scratch,
                                size_t scratch_bytes, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (nseg < 1) return BASED_ERR_SHAPE;
  const int pre = prefill_preamble(q, k, v, y, kv_state, k_state, B, H, L, d, dv, q_strides, k_strides, v_strides,
                                   y_strides, BASED_BF16, state_dtype, st);
  if (pre != 0) return pre == kDone ? BASED_OK : pre;
  return launch_linattn_prefill_tc(q, k, v, y, kv_state, k_state, B, H, L, dv, s3(q_strides), s3(k_strides),
                                   s3(v_strides), s3(y_strides), state_dtype, eps, nseg, scratch, scratch_bytes, st);
}

int based_linattn_prefill_split_static(const void* q, const void* k, const void* v, void* y, void* kv_state,
                                       void* k_state, int B, int H, int L, int d, int dv,
                                       const int64_t q_strides[3], const int64_t k_strides[3],
                                       const int64_t v_strides[3], const int64_t y_strides[3], int state_dtype,
                                       float eps, int nseg, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (nseg < 1) return BASED_ERR_SHAPE;
  const int pre = prefill_preamble(q, k, v, y, kv_state, k_state, B, H, L, d, dv, q_strides, k_strides, v_strides,
                                   y_strides, BASED_BF16, state_dtype, st);
  if (pre != 0) return pre == kDone ? BASED_OK : pre;
  return launch_linattn_prefill_tc_static(q, k, v, y, kv_state, k_state, B, H, L, dv, s3(q_strides), s3(k_strides),
                                          s3(v_strides), s3(y_strides), state_dtype, eps, nseg, st);
}

int based_linattn_decode(const void* q, const void* k, const void* v, void* y, void* kv_state, void* k_state,
                         int B, int H, int d, int dv, const int64_t q_strides[2], const int64_t k_strides[2],
                         const int64_t v_strides[2], const int64_t y_strides[2], int io_dtype, int state_dtype,
                         float eps, void* stream) {
  if (!q || !k || !v || !y || !kv_state || !k_state || !q_strides || !k_strides || !v_strides || !y_strides)
    return BASED_ERR_NULL;
  if (!dtype_ok(io_dtype) || !dtype_ok(state_dtype)) return BASED_ERR_DTYPE;
  const int rows_per_group = state_dtype == BASED_F32 ? 4 : 8;
  if (B < 0 || H < 0 || d != kFeatureDim || dv < rows_per_group || dv > 128 || dv % rows_per_group != 0)
    return BASED_ERR_SHAPE;
  if ((int64_t)B * H > 2147483647LL) return BASED_ERR_TOO_LARGE;
  if (!aligned16(kv_state)) return BASED_ERR_ALIGN;
  if (B == 0 || H == 0) return BASED_OK;
  return launch_linattn_decode(q, k, v, y, kv_state, k_state, B, H, dv, s2(q_strides), s2(k_strides),
                               s2(v_strides), s2(y_strides), io_dtype, state_dtype, eps,
                               static_cast<cudaStream_t>(stream));
}

int based_swa_prefill(const void* q, const void* k, const void* v, void* o, int B, int L, int H, int hd,
                      const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                      const int64_t o_strides[3], int window_left, float softmax_scale, int io_dtype, int impl,
                      void* stream) {
  if (!q || !k || !v || !o || !q_strides || !k_strides || !v_strides || !o_strides) return BASED_ERR_NULL;
  if (!dtype_ok(io_dtype)) return BASED_ERR_DTYPE;
  if (B < 0 || H < 0 || L < 0 || hd < 16 || hd > 128 || hd % 16 != 0 || window_left < 0) return BASED_ERR_SHAPE;
  if (H > 65535 || B > 65535) return BASED_ERR_TOO_LARGE;
  if (B == 0 || H == 0 || L == 0) return BASED_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool autosel = impl == BASED_IMPL_AUTO;
  if (autosel) impl = (io_dtype == BASED_BF16) ? BASED_IMPL_TCGEN05 : BASED_IMPL_SIMT;
  if (impl == BASED_IMPL_TCGEN05) {
    if (io_dtype != BASED_BF16) return BASED_ERR_IMPL;
    const int rc = launch_swa_prefill_tc(q, k, v, o, B, L, H, hd, s3_blh(q_strides), s3_blh(k_strides), s3_blh(v_strides),
                                         s3_blh(o_strides), window_left, softmax_scale, st);
    if (!(autosel && rc == BASED_ERR_IMPL)) return rc;
    impl = BASED_IMPL_SIMT;
  }
  if (impl != BASED_IMPL_SIMT) return BASED_ERR_IMPL;
  return launch_swa_prefill_simt(q, k, v, o, B, L, H, hd, s3_blh(q_strides), s3_blh(k_strides), s3_blh(v_strides),
                                 s3_blh(o_strides), window_left, softmax_scale, io_dtype, st);
}

int based_rotary_apply(void* x, int B, int L, int H, int hd, const int64_t x_strides[3], const void* rotary_cos,
                       const void* rotary_sin, int rotary_dim, const int32_t* seqlen_offsets, int seqlen_offset_scalar,
                       int io_dtype, void* stream) {
  if (!x || !x_strides || !rotary_cos || !rotary_sin) return BASED_ERR_NULL;
  if (!dtype_ok(io_dtype)) return BASED_ERR_DTYPE;
  if (B < 0 || L < 0 || H < 0 || hd <= 0 || rotary_dim <= 0 || rotary_dim > hd || rotary_dim % 2 != 0 ||
      seqlen_offset_scalar < 0)
    return BASED_ERR_SHAPE;
  return launch_rotary(x, B, L, H, s3_blh(x_strides), rotary_cos, rotary_sin, rotary_dim, seqlen_offsets,
                       seqlen_offset_scalar, io_dtype, static_cast<cudaStream_t>(stream));
}

int based_swa_decode(const void* q, const void* k_new, const void* v_new, void* o, void* kv_cache,
                     const int32_t* cache_seqlens, int cache_seqlen_scalar, const void* rotary_cos,
                     const void* rotary_sin, int rotary_dim, int B, int H, int hd, int max_seqlen,
                     const int64_t q_strides[2], const int64_t k_strides[2], const int64_t v_strides[2],
                     const int64_t o_strides[2], int window_left, float softmax_scale, int io_dtype, void* stream) {
  if (!q || !k_new || !v_new || !o || !kv_cache || !q_strides || !k_strides || !v_strides || !o_strides)
    return BASED_ERR_NULL;
  if ((rotary_cos == nullptr) != (rotary_sin == nullptr)) return BASED_ERR_NULL;
  if (!dtype_ok(io_dtype)) return BASED_ERR_DTYPE;
  if (B < 0 || H < 0 || hd < 16 || hd > 128 || hd % 16 != 0 || window_left < 0 || max_seqlen <= 0)
    return BASED_ERR_SHAPE;
  if (rotary_cos && (rotary_dim <= 0 || rotary_dim > hd || rotary_dim % 2 != 0)) return BASED_ERR_SHAPE;
  if (!cache_seqlens && (cache_seqlen_scalar < 0 || cache_seqlen_scalar >= max_seqlen)) return BASED_ERR_SHAPE;
  if (B == 0 || H == 0) return BASED_OK;
  return launch_swa_decode(q, k_new, v_new, o, kv_cache, cache_seqlens, cache_seqlen_scalar, rotary_cos, rotary_sin,
                           rotary_dim, B, H, hd, max_seqlen, s2(q_strides), s2(k_strides), s2(v_strides),
                           s2(o_strides), window_left, softmax_scale, io_dtype,
                           static_cast<cudaStream_t>(stream));
}

int based_gated_conv_prefill(const void* u1, const void* u2, void* v, void* state, const void* weight,
                             const void* bias, int B, int L, int di, int k, const int64_t u1_strides[2],
                             const int64_t u2_strides[2], const int64_t v_strides[2], int io_dtype, int w_dtype,
                             void* stream) {
  if (!u1 || !u2 || !v || !weight || !u1_strides || !u2_strides || !v_strides) return BASED_ERR_NULL;
  if (!dtype_ok(io_dtype) || !dtype_ok(w_dtype)) return BASED_ERR_DTYPE;
  if (B < 0 || L < 0 || di <= 0 || k < 1 || k > 4) return BASED_ERR_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (B == 0) return BASED_OK;
  if (L == 0) {  // nothing to compute; the state of an empty prompt is all zeros
    if (state) return (int)cudaMemsetAsync(state, 0, (size_t)B * di * k * dtype_size(io_dtype), st);
    return BASED_OK;
  }
  return launch_gated_conv_prefill(u1, u2, v, state, weight, bias, B, L, di, k, s2(u1_strides), s2(u2_strides),
                                   s2(v_strides), io_dtype, w_dtype, st);
}

int based_gated_conv_step(const void* u1, const void* u2, void* y, void* state, const void* weight, const void* bias,
                          int B, int di, int k, int64_t u1_batch_stride, int64_t u2_batch_stride,
                          int64_t y_batch_stride, int io_dtype, int w_dtype, void* stream) {
  if (!u1 || !u2 || !y || !state || !weight) return BASED_ERR_NULL;
  if (!dtype_ok(io_dtype) || !dtype_ok(w_dtype)) return BASED_ERR_DTYPE;
  if (B < 0 || di <= 0 || k < 1 || k > 4) return BASED_ERR_SHAPE;
  if ((int64_t)B * di > 2147483647LL) return BASED_ERR_TOO_LARGE;
  if (B == 0) return BASED_OK;
  return launch_gated_conv_step(u1, u2, y, state, weight, bias, B, di, k, u1_batch_stride, u2_batch_stride,
                                y_batch_stride, io_dtype, w_dtype, static_cast<cudaStream_t>(stream));
}

int based_add_rmsnorm(const void* x, const void* residual, const void* weight, const void* bias, void* out,
                      void* residual_out, int64_t M, int D, int64_t x_row_stride, int64_t residual_row_stride,
                      int64_t out_row_stride, int64_t residual_out_row_stride, float eps, int io_dtype, int res_dtype,
                      int w_dtype, int round_input, void* stream) {
  if (!x || !weight || !out) return BASED_ERR_NULL;
  if (!dtype_ok(io_dtype) || !dtype_ok(res_dtype) || !dtype_ok(w_dtype)) return BASED_ERR_DTYPE;
  if (M < 0 || D <= 0) return BASED_ERR_SHAPE;
  if (M == 0) return BASED_OK;
  return launch_add_rmsnorm(x, residual, weight, bias, out, residual_out, M, D, x_row_stride, residual_row_stride,
                            out_row_stride, residual_out_row_stride, eps, io_dtype, res_dtype, w_dtype, round_input,
                            static_cast<cudaStream_t>(stream));
}

int based_gated_act(const void* y, const void* gate, void* out, int64_t M, int F, int64_t y_row_stride,
                    int64_t gate_row_stride, int64_t out_row_stride, int act, int io_dtype, void* stream) {
  if (!y || !gate || !out) return BASED_ERR_NULL;
  if (!dtype_ok(io_dtype)) return BASED_ERR_DTYPE;
  if (M < 0 || F <= 0 || (act != BASED_ACT_SILU && act != BASED_ACT_SIGMOID)) return BASED_ERR_SHAPE;
  if (M == 0) return BASED_OK;
  return launch_gated_act(y, gate, out, M, F, y_row_stride, gate_row_stride, out_row_stride, act, io_dtype,
                          static_cast<cudaStream_t>(stream));
}

int based_decode_linear(const void* x, const void* w, const void* bias, void* out, int M, int N, int K,
                        int64_t x_row_stride, int64_t out_row_stride, int epilogue, int act, void* conv_state,
                        const void* conv_weight, const void* conv_bias, int conv_k, int conv_w_dtype, void* stream) {
  if (!x || !w || !out) return BASED_ERR_NULL;
  if (M < 0 || N <= 0 || K <= 0 || M > 65535 * 16) return BASED_ERR_SHAPE;
  if (epilogue == BASED_EPI_GATED && act != BASED_ACT_SILU && act != BASED_ACT_SIGMOID) return BASED_ERR_SHAPE;
  if (epilogue == BASED_EPI_CONV) {
    if (!conv_state || !conv_weight) return BASED_ERR_NULL;
    if (conv_k < 1 || conv_k > 8) return BASED_ERR_SHAPE;
    if (!dtype_ok(conv_w_dtype)) return BASED_ERR_DTYPE;
  }
  if (M == 0) return BASED_OK;
  return launch_decode_linear(x, w, bias, out, M, N, K, x_row_stride, out_row_stride, epilogue, act, conv_state,
                              conv_weight, conv_bias, conv_k, conv_w_dtype, static_cast<cudaStream_t>(stream));
}

int based_rotary_qkv_cache(void* qkv, int B, int L, int H, int hd, const int64_t qkv_strides[4],
                           const void* rotary_cos, const void* rotary_sin, void* kv_cache,
                           const int64_t cache_strides[2], void* stream) {
  if (!qkv || !qkv_strides || !rotary_cos || !rotary_sin || !kv_cache || !cache_strides) return BASED_ERR_NULL;
  if (B < 0 || L < 0 || H < 0 || hd < 16 || hd > 256) return BASED_ERR_SHAPE;
  return launch_rotary_qkv_cache(qkv, B, L, H, hd, qkv_strides[0], qkv_strides[1], qkv_strides[2], qkv_strides[3],
                                 rotary_cos, rotary_sin, kv_cache, cache_strides[0], cache_strides[1],
                                 static_cast<cudaStream_t>(stream));
}

size_t based_tp_outproj_workspace_bytes(int world, int max_rows, int N) {
  return tp_outproj_workspace_bytes(world, max_rows, N);
}

int based_tp_outproj_workspace_init(void* workspace, size_t bytes, void* stream) {
  if (!workspace) return BASED_ERR_NULL;
  if (bytes < 256 || (reinterpret_cast<uintptr_t>(workspace) & 255u)) return BASED_ERR_SCRATCH;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(workspace, 0, bytes, st);
  if (e != cudaSuccess) return (int)e;
  // epoch of the first call = 1: the zero-filled flags then read as "nothing has arrived"
  e = cudaMemsetAsync(workspace, 1, 1, st);   // little-endian word 0 becomes 0x00000001
  return (int)e;
}

int based_tp_outproj_allreduce(const void* x, const void* w, const void* bias, void* out, int M, int N, int K,
                               int64_t x_row_stride, int64_t out_row_stride, void* const* workspaces, int max_rows,
                               int rank, int world, void* stream) {
  if (!x || !w || !out || !workspaces) return BASED_ERR_NULL;
  const void* xs[1] = {x};
  const void* ws[1] = {w};
  void* os[1] = {out};
  return launch_tp_outproj_allreduce(xs, ws, bias, os, workspaces, M, N, K, x_row_stride, out_row_stride, max_rows, rank,
                                     world, 0, static_cast<cudaStream_t>(stream));
}

int based_tp_outproj_allreduce_emulated(const void* const* x, const void* const* w, const void* bias, void* const* out,
                                        int M, int N, int K, int64_t x_row_stride, int64_t out_row_stride,
                                        void* const* workspaces, int max_rows, int world, void* stream) {
  if (!x || !w || !out || !workspaces) return BASED_ERR_NULL;
  return launch_tp_outproj_allreduce(x, w, bias, out, workspaces, M, N, K, x_row_stride, out_row_stride, max_rows, 0,
                                     world, 1, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
