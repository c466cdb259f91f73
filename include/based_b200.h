/*
 * based_b200 — C ABI of the B200 (sm_100a) kernels for the Based hot path:
 * Taylor-feature-map linear attention (prefill + recurrent decode step),
 * sliding-window softmax attention (prefill + decode step), the gated short
 * convolution of the BaseConv mixer (prefill + decode step), and the residual-add +
 * RMSNorm and gated-MLP activation that sit between the mixers and the GEMMs.
 *
 * Conventions shared by every entry point
 * ---------------------------------------
 *  - All tensor arguments are DEVICE pointers owned by the caller.  The library
 *    never allocates, frees or keeps device memory between calls.
 *  - Strides are in ELEMENTS; the innermost (feature / head_dim) stride of every
 *    tensor must be 1, as the reference's own CUDA op requires
 *    (train/csrc/causal_dot_prod/causal_attention_cuda.cu:774-777).
 *  - `stream` is a cudaStream_t passed as void*; launches are asynchronous on it,
 *    so the calls can be captured in a CUDA graph the way
 *    based/generation.py:689-739 captures a decode step.
 *  - The current CUDA device must be the one that owns the pointers.
 *  - Return value: 0 = ok; negative = argument rejected on the host before any
 *    launch (BASED_ERR_*); positive = a cudaError_t from the launch.  No entry
 *    point throws, aborts or traps.
 */
#ifndef BASED_B200_H
#define BASED_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BASED_OK 0
#define BASED_ERR_NULL (-1)      /* a required pointer is NULL */
#define BASED_ERR_SHAPE (-2)     /* unsupported size (see each entry point) */
#define BASED_ERR_DTYPE (-3)     /* unknown dtype code / unsupported combination */
#define BASED_ERR_ALIGN (-4)     /* pointer or stride not aligned as required */
#define BASED_ERR_IMPL (-5)      /* requested implementation cannot run these arguments */
#define BASED_ERR_TOO_LARGE (-6) /* size exceeds a fixed capacity */
#define BASED_ERR_SCRATCH (-7)   /* caller-provided workspace is NULL, misaligned or too small */

/* dtype codes */
#define BASED_F32 0
#define BASED_BF16 1

/* implementation selectors */
#define BASED_IMPL_AUTO 0
#define BASED_IMPL_SIMT 1    /* CUDA-core kernel, fp32 arithmetic throughout */
#define BASED_IMPL_TCGEN05 2 /* tcgen05 tensor-core kernel (bf16 operands, fp32 accumulation) */

/* Width of the expanded feature vector for feature_dim 16: 1 + 16 + 256. */
#define BASED_EXPANDED_DIM 273

int based_b200_version(void);
const char* based_error_string(int code);

/*
 * Device-side status word of the tensor-core kernels.  Every wait inside those kernels is
 * bounded (about a second); a wait that expires ORs a code into this word and lets the kernel
 * run to its end with meaningless results instead of hanging.  This call synchronises with
 * the device (cudaMemcpyFromSymbol), stores the word in *out and clears it when reset != 0.
 * 0 means no wait has expired since the last reset.  No counterpart in the reference, whose
 * kernels have no in-kernel waits.
 */
int based_read_status(unsigned int* out, int reset);

/*
 * Causal linear attention with the 2nd-order Taylor feature map, whole sequence.
 *
 * Replaces the body of LinearAttention.parallel_forward
 * (based/models/mixers/linear_attention.py:169-183: feature map, tril(phi(q)phi(k)^T) v,
 * normaliser) and the state hand-off (:220-222), i.e. the job the reference gives to
 * causal_dot_product(q, k, v) (train/csrc/causal_dot_prod/causal_attention_cuda.cu:1273-1285)
 * plus the torch ops around it.
 *
 *   q, k      [B, H, L, 16]   raw (un-expanded) queries / keys
 *   v         [B, H, L, dv]
 *   y         [B, H, L, dv]   normalised output, before the 'b h l d -> b l (h d)' rearrange
 *   kv_state  [B, H, 1, dv, 273] contiguous, or NULL   (final sum_t phi(k_t) v_t^T, feature index fastest)
 *   k_state   [B, H, 1, 1, 273]  contiguous, or NULL   (final sum_t phi(k_t))
 *   *_strides (batch, head, seq) element strides of q, k, v, y
 *   io_dtype  dtype of q, k, v, y;  state_dtype dtype of kv_state / k_state
 *   d must be 16; dv a multiple of 16 in [16, 128].
 *   impl: AUTO picks TCGEN05 for bf16 I/O and SIMT for fp32 I/O.
 */
int based_linattn_prefill(const void* q, const void* k, const void* v, void* y,
                          void* kv_state, void* k_state,
                          int B, int H, int L, int d, int dv,
                          const int64_t q_strides[3], const int64_t k_strides[3],
                          const int64_t v_strides[3], const int64_t y_strides[3],
                          int io_dtype, int state_dtype, float eps, int impl, void* stream);

/*
 * The same computation with the SEQUENCE split into `nseg` segments, for long sequences with few
 * (batch x head) pairs, where based_linattn_prefill would occupy only B*H of the GPU's SMs.
 * Three launches on `stream`: each segment's own state sum_t phi(k_t) [v_t, 1]^T (fp32), the
 * running sum of those over the segments, and then every segment's outputs starting from the
 * state before it.  The reference has no counterpart: its chunked forms
 * (based/models/mixers/linear_attention.py:154-167) walk the sequence serially per head.
 *
 *   bf16 q, k, v, y only (the tcgen05 kernel); dv a multiple of 16 in [16, 112];
 *   every stride a multiple of 8 elements, q/k/v/y 16-byte aligned (else BASED_ERR_IMPL).
 *   nseg      requested segment count (>= 1).  Segments hold a whole number of 128-token chunks,
 *             so the count actually used is ceil(chunks / ceil(chunks / nseg)) <= nseg;
 *             nseg == 1 is exactly based_linattn_prefill with TCGEN05.
 *   scratch   device workspace of at least based_linattn_prefill_scratch_bytes(B, H, L, dv, nseg)
 *             bytes, 16-byte aligned; every byte the kernels read is written by them first, so it
 *             needs no initialisation.  It must not be shared by calls that can overlap.
 *             May be NULL when the size is 0.
 * based_linattn_prefill_segments returns the count this library would pick for the current
 * device (1 = do not split: B*H already covers at least half of the SMs, or L < 1024).
 */
int based_linattn_prefill_segments(int B, int H, int L);
size_t based_linattn_prefill_scratch_bytes(int B, int H, int L, int dv, int nseg);
int based_linattn_prefill_split(const void* q, const void* k, const void* v, void* y,
                                void* kv_state, void* k_state,
                                int B, int H, int L, int d, int dv,
                                const int64_t q_strides[3], const int64_t k_strides[3],
                                const int64_t v_strides[3], const int64_t y_strides[3],
                                int state_dtype, float eps, int nseg,
                                void* scratch, size_t scratch_bytes, void* stream);

/*
 * based_linattn_prefill_split without a workspace argument and without any allocation: the
 * per-segment states live in an array built into the library, BASED_STATIC_SCRATCH_BYTES
 * (8 MiB) of device memory on every GPU that loads the library, held until the process exits.
 * No counterpart in the reference.  It is for callers that cannot call cudaMalloc (or an
 * allocating library routine) where they run: a serving loop whose memory plan is fixed at
 * start-up, a callback that runs while the framework's allocator is locked, a real-time path
 * that may not take the driver's allocation lock.
 *
 *  - Arguments and results are those of based_linattn_prefill_split (bit-identical outputs).
 *  - A call whose based_linattn_prefill_scratch_bytes(B, H, L, dv, nseg) exceeds
 *    BASED_STATIC_SCRATCH_BYTES returns BASED_ERR_TOO_LARGE before any launch.
 *  - Nothing in the array has to start at zero and no call leaves state behind in it: every
 *    word a call reads, it has written first.
 *  - The first call on each device, with that device current, looks up the array's device
 *    address (cudaGetSymbolAddress, return code checked) and the kernel's launch attributes and
 *    keeps them; make that first call before any stream capture begins.  The address belongs
 *    to the device's primary context: it is not valid across a cudaDeviceReset.
 *  - All calls on one device share the one array: two calls that can run at the same time
 *    (different streams) race on it.  Order them on one stream, or give the overlapping ones
 *    their own workspace through based_linattn_prefill_split.
 */
#define BASED_STATIC_SCRATCH_BYTES (8 * 1024 * 1024)
int based_linattn_prefill_split_static(const void* q, const void* k, const void* v, void* y,
                                       void* kv_state, void* k_state,
                                       int B, int H, int L, int d, int dv,
                                       const int64_t q_strides[3], const int64_t k_strides[3],
                                       const int64_t v_strides[3], const int64_t y_strides[3],
                                       int state_dtype, float eps, int nseg, void* stream);

/*
 * One recurrent decode step; updates kv_state and k_state IN PLACE.
 *
 * Replaces TaylorExp.forward on q and k (linear_attention.py:139) followed by
 * LinearAttention.recurrent_forward (:230-251) up to, not including, out_proj:
 *   kv_state += phi(k) v^T ; k_state += phi(k) ;
 *   y = (phi(q) . kv_state) / (phi(q) . k_state + eps).
 *
 *   q, k      [B, H, 16]  raw; v, y [B, H, dv]; *_strides = (batch, head) element strides
 *   kv_state  [B, H, 1, dv, 273], k_state [B, H, 1, 1, 273], contiguous, 16-byte aligned
 *   dv a multiple of 8 (fp32 state) / 16 (bf16 state), at most 128.
 */
int based_linattn_decode(const void* q, const void* k, const void* v, void* y,
                         void* kv_state, void* k_state,
                         int B, int H, int d, int dv,
                         const int64_t q_strides[2], const int64_t k_strides[2],
                         const int64_t v_strides[2], const int64_t y_strides[2],
                         int io_dtype, int state_dtype, float eps, void* stream);

/*
 * Causal sliding-window softmax attention over a whole sequence.
 *
 * Replaces flash_attn_qkvpacked_func / flash_attn_kvpacked_func as called with
 * causal=True, window_size=(window_left, 0) at
 * based/models/mixers/slide_attention.py:100-106 and :206-213: query i attends keys
 * [i - window_left, i].
 *
 *   q, k, v, o  [B, L, H, hd]; *_strides = (batch, seq, head) element strides
 *               (q, k, v may point into one packed [B, L, 3, H, hd] tensor)
 *   hd a multiple of 16 in [16, 128]; window_left >= 0.
 *   io_dtype BASED_BF16 or BASED_F32 (fp32 runs the SIMT kernel only).
 */
int based_swa_prefill(const void* q, const void* k, const void* v, void* o,
                      int B, int L, int H, int hd,
                      const int64_t q_strides[3], const int64_t k_strides[3],
                      const int64_t v_strides[3], const int64_t o_strides[3],
                      int window_left, float softmax_scale, int io_dtype, int impl, void* stream);

/*
 * In-place rotary position embedding (non-interleaved: halves split at rotary_dim/2,
 * o0 = x0 cos - x1 sin, o1 = x0 sin + x1 cos, fp32 math) on x [B, L, H, hd].
 *
 * Replaces the rotary kernel the reference applies to q and k of the packed qkv before
 * prefill attention (slide_attention.py:553-556; formula based/ops/triton/rotary.py:75-105).
 * Token l of sample b uses table row l + seqlen_offsets[b] (device int32 [B]) or
 * l + seqlen_offset_scalar when seqlen_offsets is NULL.
 *   x_strides = (batch, seq, head); rotary_cos/sin [rows, rotary_dim/2] in io_dtype.
 */
int based_rotary_apply(void* x, int B, int L, int H, int hd, const int64_t x_strides[3],
                       const void* rotary_cos, const void* rotary_sin, int rotary_dim,
                       const int32_t* seqlen_offsets, int seqlen_offset_scalar,
                       int io_dtype, void* stream);

/*
 * One sliding-window decode step against the full-length KV cache.
 *
 * Replaces flash_attn_with_kvcache as called at slide_attention.py:414-427 and
 * :471-481: optionally rotate q and k_new at the new position (non-interleaved
 * RoPE), append k_new / v_new to the cache at that position, attend over cache
 * positions [pos - window_left, pos].
 *
 *   q, k_new, v_new, o  [B, H, hd]; *_strides = (batch, head)
 *   kv_cache            [B, max_seqlen, 2, H, hd] contiguous (slide_attention.py:374-377)
 *   cache_seqlens       device int32 [B] (tokens already cached = position of the new
 *                       token), or NULL to use cache_seqlen_scalar for every sample
 *   rotary_cos/sin      [>= max position + 1, rotary_dim / 2] in io_dtype, or NULL
 */
int based_swa_decode(const void* q, const void* k_new, const void* v_new, void* o,
                     void* kv_cache, const int32_t* cache_seqlens, int cache_seqlen_scalar,
                     const void* rotary_cos, const void* rotary_sin, int rotary_dim,
                     int B, int H, int hd, int max_seqlen,
                     const int64_t q_strides[2], const int64_t k_strides[2],
                     const int64_t v_strides[2], const int64_t o_strides[2],
                     int window_left, float softmax_scale, int io_dtype, void* stream);

/*
 * Gated short causal convolution of the BaseConv mixer, whole sequence:
 *   v[b, l, c] = silu(sum_j weight[c, j] * u1[b, l - (k-1) + j, c] + bias[c]) * u2[b, l, c]
 * with zeros before the start of the sequence.
 *
 * Replaces ShortConvolution.forward (based/models/mixers/convolution.py:47-86: depthwise
 * nn.Conv1d, padding k-1, truncated to the sequence; state fill :63-67) plus the silu and the
 * gate of BaseConv.forward (:205-211), the site where the reference optionally calls the
 * external causal_conv1d_fn (:76-83).
 *
 *   u1, u2, v  [B, L, di]; *_strides = (batch, seq) element strides, channel stride 1
 *              (u1 and u2 are normally the two halves of in_proj's output [B, L, 2*di])
 *   weight     [di, k] (conv.weight with its singleton dim dropped), bias [di] or NULL;
 *              both of dtype w_dtype
 *   state      [B, di, k] contiguous in io_dtype, or NULL: receives the last k inputs u1,
 *              oldest first, zeros in front when L < k (what the decode step continues from)
 *   k in [1, 4]; di a multiple of 8 (bf16) / 4 (fp32); u1, u2, v 16-byte aligned with
 *   strides that are multiples of 8 / 4 elements.
 */
int based_gated_conv_prefill(const void* u1, const void* u2, void* v, void* state,
                             const void* weight, const void* bias,
                             int B, int L, int di, int k,
                             const int64_t u1_strides[2], const int64_t u2_strides[2],
                             const int64_t v_strides[2],
                             int io_dtype, int w_dtype, void* stream);

/*
 * One decode step of the same op; updates `state` IN PLACE (shift left by one, append u1).
 *
 * Replaces ShortConvolution.step (convolution.py:88-109) plus silu and gate (:208-211).
 * The reference's torch step (:104-107) does not add the convolution bias; it has none with
 * the default conv_bias=False.  Here a non-NULL bias is added, as in the whole-sequence call.
 *
 *   u1, u2, y [B, di] with the given batch strides (channel stride 1); state [B, di, k].
 */
int based_gated_conv_step(const void* u1, const void* u2, void* y, void* state,
                          const void* weight, const void* bias,
                          int B, int di, int k,
                          int64_t u1_batch_stride, int64_t u2_batch_stride, int64_t y_batch_stride,
                          int io_dtype, int w_dtype, void* stream);

/*
 * Residual add + RMSNorm in one pass over [M, D] rows:
 *   z = x + residual;  residual_out = z;  out = z / sqrt(mean(z^2) + eps) * weight + bias.
 *
 * Replaces RMSNorm.forward / rms_norm_fn with prenorm=True, the Triton kernel that
 * Block.forward and GPTModel.forward call (based/ops/triton/layer_norm.py:926-953; semantics
 * restated by rms_norm_ref :74-125; call sites based/models/block.py:134-163,
 * based/models/gpt.py:696-733).
 *
 *   x, out        [M, D] in io_dtype; residual (or NULL), residual_out (or NULL) [M, D] in
 *                 res_dtype -- BASED_F32 is the reference's residual_in_fp32=True;
 *                 *_row_stride in elements, inner stride 1
 *   weight, bias  [D] in w_dtype; bias may be NULL
 *   The norm is taken of z as residual_out stores it (rounded to bf16 when res_dtype is bf16 and
 *   residual_out is given).  round_input != 0 additionally rounds z to io_dtype before the norm:
 *   that is what the blocks compute when they run the unfused sequence
 *   `residual = x + residual; hidden = norm(residual.to(weight.dtype))` (block.py:134-137) with
 *   an fp32 residual stream and bf16 activations.
 *   D a multiple of 8, at most 8192; pointers 16-byte aligned, row strides multiples of 8.
 *   fp32 arithmetic.
 */
int based_add_rmsnorm(const void* x, const void* residual, const void* weight, const void* bias,
                      void* out, void* residual_out,
                      int64_t M, int D,
                      int64_t x_row_stride, int64_t residual_row_stride,
                      int64_t out_row_stride, int64_t residual_out_row_stride,
                      float eps, int io_dtype, int res_dtype, int w_dtype, int round_input, void* stream);

/* activation selectors of based_gated_act */
#define BASED_ACT_SILU 0    /* SwiGLU: y * silu(gate) */
#define BASED_ACT_SIGMOID 1 /* GLU:    y * sigmoid(gate) */

/*
 * Gated activation of the MLP: out[m, f] = y[m, f] * act(gate[m, f]).
 *
 * Replaces `y, gate = y.chunk(2, dim=-1); y = swiglu(gate, y)` (flash-attn's jiterator op) and
 * F.glu in GatedMlp.forward (based/models/mlp.py:141-154).  y and gate are normally the two
 * halves of fc1's output [M, 2F]: pass both pointers with the same row stride 2F.
 *   F a multiple of 8 (bf16) / 4 (fp32), at most 16384 / 8192; pointers 16-byte aligned; row strides multiples of 8 / 4.
 */
int based_gated_act(const void* y, const void* gate, void* out,
                    int64_t M, int F,
                    int64_t y_row_stride, int64_t gate_row_stride, int64_t out_row_stride,
                    int act, int io_dtype, void* stream);

/*
 * Prompt pass of the sliding-window mixer, before attention: rotary embedding (non-interleaved, whole
 * head, positions 0 .. L-1) applied in place to q and k of the packed projection qkv [B, L, 3, H, hd],
 * and the rotated k and the v written into the layer's KV cache in the same pass.
 *
 * Replaces `self.rotary_emb(qkv, ...)` followed by the cache fill `_update_kv_cache(kv, ...)`
 * (based/models/mixers/slide_attention.py:553-556, :255-281), two passes over k and v in the reference.
 *
 *   qkv_strides   (batch, seq, part, head) element strides of qkv, hd contiguous; bf16
 *   rotary_cos/sin [>= L, hd/2] bf16, contiguous
 *   kv_cache      points at the first cache row to fill; layout [.., max_seqlen, 2, H, hd] with
 *                 cache_strides = (batch, seq) element strides and (2, H, hd) contiguous; bf16
 *   hd a multiple of 16; all strides multiples of 8; pointers 16-byte aligned.
 */
int based_rotary_qkv_cache(void* qkv, int B, int L, int H, int hd, const int64_t qkv_strides[4],
                           const void* rotary_cos, const void* rotary_sin,
                           void* kv_cache, const int64_t cache_strides[2], void* stream);

/* epilogue selectors of based_decode_linear */
#define BASED_EPI_PLAIN 0  /* out[M, N]   = x W^T + bias */
#define BASED_EPI_GATED 1  /* out[M, N/2] = (x W1^T + b1) * act(x W2^T + b2), W = [W1; W2], act as in based_gated_act */
#define BASED_EPI_CONV 2   /* out[M, N/2] = silu(conv_step(u1)) * u2 with [u1 | u2] = x W^T + bias */

/*
 * A linear layer on the few rows of a decode step (one token per sequence), bf16, with the
 * elementwise step that follows it in the Based blocks fused into the epilogue.
 *
 * Replaces, for single-token steps, nn.Linear calls of the mixers and the MLP
 * (based/models/mixers/linear_attention.py:126-128, :251; slide_attention.py:544, :599;
 * convolution.py:205, :212; based/models/mlp.py:142, :155) together with
 *   GATED: `y, gate = y.chunk(2, dim=-1); y = y * act(gate)` (mlp.py:146-154)
 *   CONV:  ShortConvolution.step + silu + gate (convolution.py:88-109, :205-211); `conv_state`
 *          [M, N/2, conv_k] (bf16) is updated in place, taps conv_weight [N/2, conv_k] and
 *          conv_bias [N/2] (or NULL) are in conv_w_dtype
 * which the reference runs as separate cuBLAS and elementwise launches.
 *
 *   x [M, K], W [N, K] (nn.Linear layout, contiguous), bias [N] or NULL, out as above; all bf16;
 *   row strides in elements.  K a multiple of 32; the number of outputs a multiple of 8;
 *   x and W 16-byte aligned, x_row_stride a multiple of 8.  Built for M <= 16 (weights are read
 *   once per 16 rows); larger M works and re-reads W from L2 per 16 rows.
 */
int based_decode_linear(const void* x, const void* w, const void* bias, void* out,
                        int M, int N, int K, int64_t x_row_stride, int64_t out_row_stride,
                        int epilogue, int act,
                        void* conv_state, const void* conv_weight, const void* conv_bias,
                        int conv_k, int conv_w_dtype, void* stream);

/*
 * Tensor-parallel decode step: row-parallel output projection fused with the all-reduce that follows it.
 *
 *   out[M, N] = sum over ranks r of x_r[M, K] W_r[N, K]^T (+ bias)        bf16 in / out, fp32 partials and sum
 *
 * Modelled on RowParallelLinear.forward (based/ops/fused_dense.py:239-246: local GEMM, then all_reduce of the
 * [B, L, d_model] output), the layer the head-sharded variant of LinearAttention / SlidingAttention ends with
 * (out_proj, based/models/mixers/linear_attention.py:252, slide_attention.py:599).  The reference's mixers have no
 * tensor parallelism; the unfused form here is a cuBLAS GEMM followed by ncclAllReduce.  One kernel per rank:
 * the rank's partial tile is pushed into EVERY rank's receive workspace with plain stores to peer memory (NVLink),
 * a per-tile flag follows, each rank then waits (bounded, ~1 s, reported through based_read_status; the affected
 * outputs become NaN) for the same tile of every rank and adds the partials in rank order, so all ranks hold
 * bit-identical results.  Built for decode sizes (M <= max_rows <= 64 single-token rows), where the collective is
 * latency-bound; prompt-size outputs stay on NCCL.
 *
 *   workspaces[world]  device pointers to every rank's workspace AS MAPPED IN THIS PROCESS (peer mappings from
 *                      CUDA IPC or a symmetric-memory allocator); entry `rank` is this rank's own.  Each is
 *                      based_tp_outproj_workspace_bytes(world, max_rows, N) bytes, 256-byte aligned, prepared ONCE with
 *                      based_tp_outproj_workspace_init (on its owner, before any rank's first call), and must not be
 *                      used by two calls that overlap in time.  The call counter lives in the workspace and is
 *                      advanced by the kernel, so a captured launch can be replayed.
 *   max_rows           (<= 64) fixes the workspace layout: the same value on every rank and every call.
 *   N a multiple of 8, K a multiple of 32, x and W 16-byte aligned, x_row_stride a multiple of 8, out_row_stride
 *   even; world <= 8.  Every rank must make the call (same M, N) at about the same time, like any collective.
 *   Returns BASED_ERR_TOO_LARGE when the launch could not be fully resident (its blocks wait for their
 *   counterparts on the other ranks).
 */
size_t based_tp_outproj_workspace_bytes(int world, int max_rows, int N);
int based_tp_outproj_workspace_init(void* workspace, size_t bytes, void* stream);
int based_tp_outproj_allreduce(const void* x, const void* w, const void* bias, void* out,
                               int M, int N, int K, int64_t x_row_stride, int64_t out_row_stride,
                               void* const* workspaces, int max_rows, int rank, int world, void* stream);
/*
 * The same kernel with all `world` ranks inside ONE cooperative launch on one GPU (x, w, out: one pointer per rank;
 * workspaces: all local).  For checking the exchange protocol where fewer GPUs than ranks are at hand; two separate
 * launches that wait on one another must never share a GPU.  No counterpart in the reference.
 */
int based_tp_outproj_allreduce_emulated(const void* const* x, const void* const* w, const void* bias, void* const* out,
                                        int M, int N, int K, int64_t x_row_stride, int64_t out_row_stride,
                                        void* const* workspaces, int max_rows, int world, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BASED_B200_H */
