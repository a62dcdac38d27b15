/*
 * spsattn.h — C ABI of libspsattn.so: the SPS Transformer attention hot path
 * (prefill attention over the doubled input/<predict> sequence, segmented decode
 * attention over the persistent KV cache plus the predict ring, and the decode
 * KV-cache update) as hand-written sm_100a CUDA.
 *
 * Conventions
 *   - every pointer named "device" is a CUDA device pointer on the current device;
 *     the library never allocates device memory (workspaces are caller-owned);
 *   - `stream` is a cudaStream_t passed as void* (NULL = default stream); all work is
 *     enqueued on it and the call returns without synchronising;
 *   - return value: 0 ok; <0 argument error found on the host before any launch
 *     (spsattn_strerror explains); >0 CUDA runtime / driver error code;
 *   - kernels never trap: a bounded wait that expires writes a non-zero code into
 *     the caller's `device_status` word (may be NULL) and the block returns.
 *
 * Reference interface each entry point stands in for (paths inside lil-lab/sps):
 *   spsattn_prefill_fwd      src/modeling/models/attention/triton_sps_flash_attention.py:491-620 (wrapper)
 *                            and :147-269 (_attn_fwd_sps); the reverse and standard variants
 *                            triton_reverse_sps_flash_attention.py:242-331, triton_full_flash_attention.py:204-283
 *   spsattn_prefill_bwd      triton_sps_flash_attention.py:623-720 (backward wrapper), :272-488
 *                            (_attn_bwd_preprocess, _sps_bwd_dkdv_kernel, _sps_bwd_dq_kernel)
 *   spsattn_decode_fwd       src/modeling/models/utils/decode_attention.py:483-594 (q=2), :393-480 (q=1)
 *   spsattn_kv_update        src/modeling/models/utils/decode_attention_fast.py:139-221
 *   spsattn_fill_decode_caches  src/modeling/models/reverse_sps/inference.py:568-613
 *   spsattn_rope_cast, spsattn_qkv_rope_cast
 *                            src/modeling/models/model.py:201-230 + sps/core.py:45-55
 *   spsattn_decode_step      one layer of src/modeling/models/reverse_sps/inference.py:322-362 (attention)
 *                            + :169-238 (cache update) in two launches
 *   spsattn_add_rmsnorm, spsattn_swiglu
 *                            src/modeling/models/model.py:101-132, :304-314, :324-327
 */
#ifndef SPSATTN_H_
#define SPSATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SPSATTN_DTYPE_BF16 0
#define SPSATTN_DTYPE_FP16 1
#define SPSATTN_DTYPE_FP32 2   /* accepted only where an entry point says so */

/* which key parity of the doubled sequence is persistent (window-exempt) */
#define SPSATTN_PARITY_EVEN 0   /* SPS: input token slot            (triton_sps_flash_attention.py:97) */
#define SPSATTN_PARITY_ODD 1    /* Reverse-SPS / Delayed-State      (triton_reverse_sps_flash_attention.py:123) */
#define SPSATTN_PARITY_NONE (-1) /* Standard: causal + document mask (triton_full_flash_attention.py:95-104) */

#define SPSATTN_NO_WINDOW (-2147483647 - 1) /* persistent_window: no persistent-key window */

/* mask_flags */
#define SPSATTN_FLAG_PERSISTENT_Q_SKIPS_TEMPORARY 1 /* rows of persistent parity see no temporary keys */

/* error codes (<0) */
#define SPSATTN_ERR_ARG (-1)        /* null pointer, bad enum, bad size */
#define SPSATTN_ERR_HEAD_DIM (-2)   /* head_dim not supported by this entry point */
#define SPSATTN_ERR_ALIGN (-3)      /* pointer or stride not 16-byte aligned */
#define SPSATTN_ERR_WORKSPACE (-4)  /* workspace missing or too small */
#define SPSATTN_ERR_ODD_LENGTH (-5) /* doubled sequence length must be even */
#define SPSATTN_ERR_DRIVER (-6)     /* tensor-map encoder unavailable */
#define SPSATTN_ERR_TOO_LARGE (-7)  /* size beyond a documented maximum */
#define SPSATTN_ERR_SCRATCH_LIMIT (-8) /* needs more scratch than the built-in static buffer holds */

/* device_status codes written by kernels (0 = ok) */
#define SPSATTN_STATUS_WAIT_EXPIRED 1

const char* spsattn_strerror(int code);
int spsattn_version(void);

/* ---------------------------------------------------------------------------------------------
 * Prefill: O = softmax(mask(Q K^T * sm_scale)) V over [B, H, N, D] row-major contiguous tensors.
 *
 * Visibility of key row j to query row i (tok = row / 2), the reference rule
 * (triton_sps_flash_attention.py:81-111):
 *     j <= i  AND  doc[b][i] == doc[b][j] (if doc_ids given)
 *     AND ( j%2 == persistent_parity ? (persistent_window unset OR tok_i - tok_j <= persistent_window OR i == j)
 *                                    : tok_i - tok_j <= temporary_window )
 * With SPSATTN_PARITY_NONE only the causal and document terms apply.  Rows with no visible key
 * produce 0.  doc_ids: [B, N] int64 (doc_is_i64 = 1) or int32, element strides given; NULL = none.
 * lse (nullable, [B, H, N] fp32) receives log2(sum_j exp2(score_ij * sm_scale * log2 e)), the
 * reference's M tensor (:265-267).  N must be even unless parity is NONE.  D in {64, 128} run on
 * the tcgen05/TMA kernel; D in {16, 32, 256} run on a plain CUDA-core kernel.  sm_scale > 0.
 * workspace: at least spsattn_prefill_workspace_bytes(B, H, N, D) bytes of device memory,
 * 256-byte aligned, private to this call until it completes.
 * ------------------------------------------------------------------------------------------- */
size_t spsattn_prefill_workspace_bytes(int B, int H, int N, int D);

int spsattn_prefill_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                        const void* doc_ids, int doc_is_i64, int64_t doc_stride_b, int64_t doc_stride_t,
                        int B, int H, int N, int D, int dtype, float sm_scale,
                        int persistent_parity, int temporary_window, int persistent_window,
                        int mask_flags,
                        void* workspace, size_t workspace_bytes,
                        int* device_status, void* stream);

/* Same computation on operands that are not dense [B, H, N, D] blocks: element (b, h, n, d) of an
 * operand lives at  strides[0]*b + strides[1]*h + strides[2]*n + d  (elements; d contiguous, every
 * stride a multiple of 8 and >= D).  The reference's model code hands its kernels transposed views
 * of token-major [B, N, H, D] projections (src/modeling/models/sps/core.py:45-55) and transposes
 * the result back (:79); with strides the kernel reads and writes those layouts in place — q, k, v
 * even straight out of a fused [B, N, 3*H*D] projection buffer — so the .contiguous() copies of
 * triton_sps_flash_attention.py:504-506 disappear.  D in {64, 128}; the other head dims need dense
 * operands. */
int spsattn_prefill_fwd_strided(const void* q, const void* k, const void* v, void* o, float* lse,
                                const int64_t* q_strides, const int64_t* k_strides,
                                const int64_t* v_strides, const int64_t* o_strides,
                                const void* doc_ids, int doc_is_i64, int64_t doc_stride_b,
                                int64_t doc_stride_t,
                                int B, int H, int N, int D, int dtype, float sm_scale,
                                int persistent_parity, int temporary_window, int persistent_window,
                                int mask_flags,
                                void* workspace, size_t workspace_bytes,
                                int* device_status, void* stream);

/* Backward of spsattn_prefill_fwd (the training path): dq, dk, dv from d_o, with the
 * probabilities recomputed from `lse` as written by the forward call on the same q, k, v, mask and
 * sm_scale (the reference's backward, triton_sps_flash_attention.py:623-720, does the same with
 * its M tensor).  All tensors dense [B, H, N, D] of `dtype`; `o` is the forward output; lse is
 * [B, H, N] fp32.  Launches (after the document pre-passes, if ids are given): delta = rowsum(d_o * o), then dk / dv (one block per 128-token
 * key tile of each parity stream, visiting only the query tiles that can see it), then dq (one
 * block per 128-row query tile, visiting the key tiles the forward visits).  D in {64, 128};
 * N <= 65536.  workspace: spsattn_prefill_bwd_workspace_bytes(B, H, N, D) bytes, 256-byte aligned. */
size_t spsattn_prefill_bwd_workspace_bytes(int B, int H, int N, int D);

int spsattn_prefill_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                        const float* lse, void* dq, void* dk, void* dv,
                        const void* doc_ids, int doc_is_i64, int64_t doc_stride_b, int64_t doc_stride_t,
                        int B, int H, int N, int D, int dtype, float sm_scale,
                        int persistent_parity, int temporary_window, int persistent_window,
                        int mask_flags,
                        void* workspace, size_t workspace_bytes,
                        int* device_status, void* stream);

/* The same on operands that are not dense blocks (the token-major views the reference's modules
 * pass, src/modeling/models/sps/core.py:45-55, and the gradients autograd hands back for them):
 * `strides` holds eight (batch, head, row) triples in elements, in the order q, k, v, o, d_o, dq,
 * dk, dv; rows are D contiguous elements, every stride a multiple of 8 and >= D.  The reference's
 * backward copies all of them first (triton_sps_flash_attention.py:629-633). */
int spsattn_prefill_bwd_strided(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                const float* lse, void* dq, void* dk, void* dv, const int64_t* strides,
                                const void* doc_ids, int doc_is_i64, int64_t doc_stride_b,
                                int64_t doc_stride_t,
                                int B, int H, int N, int D, int dtype, float sm_scale,
                                int persistent_parity, int temporary_window, int persistent_window,
                                int mask_flags,
                                void* workspace, size_t workspace_bytes,
                                int* device_status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Decode: nq (1 or 2) queries per (sequence, head) over up to 3 length-masked KV segments plus up
 * to 2 single-token "current" K/V entries; fp32 output [S, nq, H, D].
 *
 * Segment table (the reference's KVSegment, decode_attention.py:21-32, generalised so a packed
 * cache needs no copy): key row r of (sequence s, head h) lives at element offset
 *     (seq_offset ? seq_offset[s] : s * seq_stride) + h * head_stride + r * row_stride
 * from k / v, rows are D contiguous elements, and rows [0, min(len, max_rows)) are live, where
 * len = lengths[s] (lengths_per_head = 0) or lengths[s * H + h] (= 1), int64 on the device.
 * query_mask bit i set: query slot i scans this segment / sees this extra entry.  The reference's
 * q=2 call is segments {ring, retained} with query_mask 3, extras {current normal: 3, current
 * predict: 2} (decode_attention.py:309-361).  No visible key => output 0 (:363-366).
 * ------------------------------------------------------------------------------------------- */
typedef struct spsattn_segment {
  const void* k;              /* device */
  const void* v;              /* device */
  const int64_t* seq_offset;  /* device [S] element offsets, or NULL */
  int64_t seq_stride;         /* elements, used when seq_offset is NULL */
  int64_t head_stride;        /* elements */
  int64_t row_stride;         /* elements, >= D */
  const int64_t* lengths;     /* device [S] or [S*H] */
  int32_t lengths_per_head;   /* 0 or 1 */
  int32_t max_rows;           /* host cap on rows scanned: min(storage, max_len_cap) */
  uint32_t query_mask;
  uint32_t reserved;
} spsattn_segment;

typedef struct spsattn_extra {
  const void* k; /* device [S, H, D] contiguous */
  const void* v; /* device [S, H, D] contiguous */
  uint32_t query_mask;
  uint32_t reserved;
} spsattn_extra;

size_t spsattn_decode_workspace_bytes(int S, int H, int D, int nq, const spsattn_segment* segs,
                                      int n_segments);

/* q: device [S, nq, H, D] contiguous, dtype as given; out: device fp32 [S, nq, H, D].
 * D multiple of 8, 8 <= D <= 256.  Split-K over each (sequence, head): partial (max, sum,
 * accumulator) records go to `workspace`, then a merge pass writes `out`. */
int spsattn_decode_fwd(const void* q, int nq, float* out,
                       const spsattn_segment* segs, int n_segments,
                       const spsattn_extra* extras, int n_extras,
                       int S, int H, int D, int dtype, float sm_scale,
                       void* workspace, size_t workspace_bytes,
                       int* device_status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Allocation-free decode (no counterpart in the reference: its wrappers allocate freely through
 * torch).  Same computation, arguments and result as spsattn_decode_fwd, but the split-K records
 * go to a buffer that is compiled into the library instead of a caller-supplied workspace, so the
 * call needs no device allocation from anybody.  It is meant for hosts that cannot allocate at
 * the point where they decode: a serving process whose cache manager has already claimed all of
 * device memory for its own arena (a fresh cudaMalloc would fail or shrink the arena), a step
 * loop that must not hit cudaMalloc's device-wide synchronisation, or a binding that reaches the
 * library through an FFI and has no allocator to hand over.
 *
 * Limit: the records of one call, spsattn_decode_workspace_bytes(...), must fit in
 * SPSATTN_NOALLOC_SCRATCH_BYTES (16 MiB; the benchmark's 128-sequence step needs 9.3 MiB).  A larger
 * problem is refused with SPSATTN_ERR_SCRATCH_LIMIT before anything is launched: split the
 * sequences over several calls or use spsattn_decode_fwd.  Every GPU that loads the library
 * carries the 16 MiB until the process exits.
 *
 * Every call looks up the buffer's device address on the current device (the device must be
 * current, as for every call), so the address is never stale after a device reset; the first
 * call on a device also sets the library's code up there: make that first call outside any
 * stream capture.  All calls on a
 * device share the one buffer: calls that can overlap on the GPU (different streams, no ordering
 * between them) race on it and must be serialised by the caller.  The buffer keeps the previous
 * call's records; nothing in it has to start at zero, because a call only reads records it has
 * written itself.  The entry point calls no cudaMalloc / cudaFree and no allocating library routine.
 * ------------------------------------------------------------------------------------------- */
#define SPSATTN_NOALLOC_SCRATCH_BYTES (16u << 20)

int spsattn_decode_fwd_noalloc(const void* q, int nq, float* out,
                               const spsattn_segment* segs, int n_segments,
                               const spsattn_extra* extras, int n_extras,
                               int S, int H, int D, int dtype, float sm_scale,
                               int* device_status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * One layer of an SPS-family decode step in a single launch: the segmented attention of
 * spsattn_decode_fwd, merged by the last block of each (sequence, head) instead of a second
 * kernel, with the cache update of spsattn_kv_update folded into that merge, and the output written
 * in the type the output projection consumes.  Stands in for the pair of calls the reference makes
 * per layer and token (reverse_sps/inference.py:434-477: _attend_pair_from_decode_state, then
 * _update_normal_memory + _update_predict_memory -> fused_sps_kv_update).
 *
 * `append` (NULL = attention only) names the ring and the retained cache of this layer, which
 * must be the buffers the segments read, and this step's K/V rows for them.  The attention sees
 * the caches as they are before the update; afterwards, for every active sequence, the rows are
 * stored and the counters advanced exactly as spsattn_kv_update does.  A (sequence, head) is
 * updated only after all of its blocks have read the counters and finished reading its rows; the
 * per-sequence ring counters only after all heads of the sequence have.  No block waits for another.
 * out_dtype: SPSATTN_DTYPE_FP32, or the queries' 16-bit type.  16-bit caches only.
 *
 * Workspace: spsattn_decode_step_workspace_bytes; its last (S*H + S) * 4 bytes (rounded up to 256)
 * are completion tickets that must be ZERO before the first call that uses the buffer — zero the
 * whole workspace once after allocating it — and are left zero by every call that completes, so
 * the same buffer serves every later call on the same stream without further clearing.
 * ------------------------------------------------------------------------------------------- */
typedef struct spsattn_kv_append {
  void* nw_k;               /* device ring      [S, H, window_storage, D] */
  void* nw_v;
  int64_t* nw_len;          /* device [S] */
  int64_t* nw_pos;          /* device [S] */
  void* br_k;               /* device retained  [S, H, retained_storage, D] */
  void* br_v;
  int64_t* br_len;          /* device [S, H] */
  const void* k_window;     /* device [S, H, D]: this step's row for the ring */
  const void* v_window;
  const void* k_retained;   /* device [S, H, D]: this step's row for the retained cache */
  const void* v_retained;
  const int8_t* active;     /* device [S] */
  int32_t window_storage;
  int32_t retained_storage;
  int32_t window_tokens;    /* <= 0: no ring (ring pointers may be NULL) */
  int32_t reserved;
} spsattn_kv_append;

size_t spsattn_decode_step_workspace_bytes(int S, int H, int D, int nq, const spsattn_segment* segs,
                                           int n_segments);

int spsattn_decode_step(const void* q, int nq, void* out, int out_dtype,
                        const spsattn_segment* segs, int n_segments,
                        const spsattn_extra* extras, int n_extras,
                        const spsattn_kv_append* append_or_null,
                        int S, int H, int D, int dtype, float sm_scale,
                        void* workspace, size_t workspace_bytes,
                        int* device_status, void* stream);

/* Test hook: which kernel spsattn_decode_step uses.  0 = automatic (the tensor-core kernel when
 * head_dim is 64 or 128, no segment is packed through seq_offset and there are at least 444
 * (sequence, head, long segment) triples, else the CUDA-core kernel),
 * 1 = always the CUDA-core kernel, 2 = the tensor-core kernel (head_dim 64 or 128, no packed
 * segment) or SPSATTN_ERR_ARG.  Process-wide. */
int spsattn_debug_decode_path(int path);

/* Test hook: which tensor-core prefill kernel serves head_dim 64.  0 = automatic (today the
 * 64-key-tile kernel with P through shared memory, three blocks per SM, which also serves
 * head_dim 128 and measures faster), 1 = that kernel, forced, 2 = the persistent kernel with
 * 128-key tiles, P kept in tensor memory and a hand-pipelined softmax (two blocks per SM drawing
 * work items from a counter).  All apply the same plan and the same visibility rule and are held
 * to the same parity tests.  Process-wide.  No counterpart in the reference. */
int spsattn_debug_prefill_path(int path);

/* Test hook for the bounded waits of the kernels: launches one warp that waits on a barrier
 * nobody arrives at (no copy or tensor-core operation in flight), with a limit of `limit_ns`
 * nanoseconds (at most 1e9).  The wait gives up, writes SPSATTN_STATUS_WAIT_EXPIRED to
 * *device_status as the attention kernels do, sets device_result[0] = 1 (when given) and the
 * block ends normally.  While the status word is non-zero the tensor-core attention kernels
 * return without computing; the caller clears it.  No counterpart in the reference. */
int spsattn_debug_wait_expiry(int* device_status, unsigned long long limit_ns, int* device_result,
                              void* stream);

/* ---------------------------------------------------------------------------------------------
 * Decode KV-cache update, in place (decode_attention_fast.py:34-136): for every active sequence
 * insert k_window/v_window into the ring [S,H,window_storage,D] at `pos` when the ring is full
 * (len >= window_tokens) else at `len`, then pos = (pos+1) % window_tokens or len += 1; append
 * k_retained/v_retained to the retained cache [S,H,retained_storage,D] at len[s,h] when in
 * bounds and increment it.  window_tokens <= 0: retained part only (ring pointers may be NULL).
 * nw_len, nw_pos: int64 [S]; br_len: int64 [S,H]; active: int8 [S]; new K/V [S,H,D] in the
 * cache dtype (elem_bytes 2 or 4).
 * ------------------------------------------------------------------------------------------- */
int spsattn_kv_update(void* nw_k, void* nw_v, int64_t* nw_len, int64_t* nw_pos,
                      void* br_k, void* br_v, int64_t* br_len,
                      const void* k_window, const void* v_window,
                      const void* k_retained, const void* v_retained,
                      const int8_t* active,
                      int S, int H, int D, int window_storage, int retained_storage,
                      int window_tokens, int elem_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Rotary embedding + cast for q or k (rotate = 1) or plain cast for v (rotate = 0), writing the
 * 16-bit operand the attention kernels read (src/modeling/models/model.py:201-230 followed by the
 * bf16 cast of src/modeling/models/sps/core.py:53-55).  x: [B, N, H, D] view, x_dtype 0 bf16,
 * 1 fp16, 2 fp32, strides in elements (D contiguous).  freqs_cis: complex64 as (cos, sin) float
 * pairs, [N, D/2] (freqs_stride_b = 0) or [B, N, D/2] (freqs_stride_b = N * D/2, in complex
 * elements).  Adjacent elements (2i, 2i+1) form the complex number that is multiplied by
 * freqs_cis[n, i] in fp32.  out: 16-bit rows with its own strides.  D multiple of 8.
 * ------------------------------------------------------------------------------------------- */
int spsattn_rope_cast(const void* x, int x_dtype, int64_t x_stride_b, int64_t x_stride_n,
                      int64_t x_stride_h, const float* freqs_cis, int64_t freqs_stride_b,
                      void* out, int out_dtype, int64_t out_stride_b, int64_t out_stride_n,
                      int64_t out_stride_h, int B, int N, int H, int D, int rotate, void* stream);

/* ---------------------------------------------------------------------------------------------
 * The same for a fused q/k/v projection in one launch (sps/core.py:45-55 splits c_attn's output
 * into thirds, rotates q and k, casts all three).  x: [B, N, n_groups * heads_per_group, D] view;
 * the heads are split into n_groups (1..6) consecutive groups and group g is written to
 * groups[g].out with its own strides, rotated when groups[g].rotate is set, cast otherwise.
 * (A decode step passes the [S, 2, 3C] projection of a token pair as N = 1 with six groups.)
 * ------------------------------------------------------------------------------------------- */
typedef struct spsattn_rope_group {
  void* out;           /* device, 16-bit rows */
  int64_t stride_b;    /* elements */
  int64_t stride_n;
  int64_t stride_h;
  int32_t rotate;
  int32_t reserved;
} spsattn_rope_group;

int spsattn_qkv_rope_cast(const void* x, int x_dtype, int64_t x_stride_b, int64_t x_stride_n,
                          int64_t x_stride_h, const float* freqs_cis, int64_t freqs_stride_b,
                          const spsattn_rope_group* groups, int n_groups, int out_dtype,
                          int B, int N, int heads_per_group, int D, void* stream);

/* ---------------------------------------------------------------------------------------------
 * The element-wise passes of a decoder block around the attention call, so that a generation
 * step is a fixed chain of launches (model.py:101-132 RMSNorm, :324-327 residual adds, :304-314
 * SwiGLU MLP).  dtype: SPSATTN_DTYPE_BF16 (every intermediate rounded to bf16 where the
 * reference's bf16 tensors round) or SPSATTN_DTYPE_FP32.
 *
 * spsattn_add_rmsnorm: x [rows, C] += delta (when delta is not NULL; x is updated in place),
 * then y = cast(x_f32 * rsqrt(mean(x_f32^2) + eps)) * weight (when y is not NULL).
 * spsattn_swiglu: y [rows, I] = silu(gate_up[:, :I]) * gate_up[:, I:], gate_up [rows, 2I].
 * ------------------------------------------------------------------------------------------- */
int spsattn_add_rmsnorm(void* x, const void* delta_or_null, const void* weight, void* y_or_null,
                        int dtype, long long rows, int C, float eps, void* stream);

int spsattn_swiglu(const void* gate_up, void* y, int dtype, long long rows, int I, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Prefill -> decode hand-over for one layer (src/modeling/models/reverse_sps/inference.py:568-613,
 * there a Python loop over batch rows with host syncs): for every batch row the tokens selected by
 * doc_mask [B, T] (bytes; the prompt's last document) are compacted in order; the K/V rows of
 * parity `retained_slot` of those tokens go to the retained cache [B,H,retained_storage,D] rows
 * 0..doc_len-1 and br_len[b,:] = doc_len; the rows of parity `window_slot` of the last
 * min(window_tokens, doc_len) of them go to the ring [B,H,window_storage,D] rows 0.., with
 * nw_len[b] = that count and nw_pos[b] = 0.  Rows without a selected token are left untouched.
 * k, v: [B, 2T, H, D] 16-bit elements in the cache dtype, strides in elements (D contiguous,
 * multiples of 8), T < 32768.  window_tokens <= 0: retained part only.
 * ------------------------------------------------------------------------------------------- */
int spsattn_fill_decode_caches(const void* k, const void* v, int64_t stride_b, int64_t stride_n,
                               int64_t stride_h, const uint8_t* doc_mask,
                               void* br_k, void* br_v, int64_t* br_len,
                               void* nw_k, void* nw_v, int64_t* nw_len, int64_t* nw_pos,
                               int B, int T, int H, int D, int retained_storage, int window_storage,
                               int window_tokens, int retained_slot, int window_slot, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Test hook: the boolean visibility the prefill kernels apply, evaluated on the device with the
 * same per-row key-interval arithmetic (and the same document pre-pass) the kernels use, written
 * as bytes [B, N, N].  For bit-exact mask checks at small N (N <= 4096).
 * ------------------------------------------------------------------------------------------- */
int spsattn_debug_visibility(uint8_t* vis, const void* doc_ids, int doc_is_i64,
                             int64_t doc_stride_b, int64_t doc_stride_t, int B, int N,
                             int persistent_parity, int temporary_window, int persistent_window,
                             int mask_flags, void* workspace, size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SPSATTN_H_ */
