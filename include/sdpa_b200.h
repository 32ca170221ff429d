/*
 * sdpa_b200.h - C ABI of libsdpa_b200.so: scaled-dot-product attention forward, backward
 * and split-KV decode for NVIDIA B200 (sm_100a), written to stand where torch_mlu binds
 * Cambricon's closed attention library.
 *
 * What each entry point replaces in the reference (paths inside Cambricon/torch_mlu):
 *   sdpa_b200_fwd            <- mha_varlen_fwd, i.e. cnnlFlashAttentionForward_v2
 *                               torch_mlu/csrc/aten/operators/cnnl/internal/FlashAttention_internal.cpp:57-267
 *                               (declared cnnl_internal.h:1461-1476)
 *   sdpa_b200_bwd            <- mha_varlen_bwd, i.e. cnnlFlashAttentionBackward
 *                               .../internal/FlashAttention_internal.cpp:269-483 (cnnl_internal.h:1478-1495)
 *   sdpa_b200_*_workspace_bytes
 *                            <- cnnlGetFlashAttention{Forward,Backward}WorkspaceSize_v2
 *                               .../internal/FlashAttention_internal.cpp:215-230, 437-447
 *   sdpa_b200_status_string  <- TORCH_CNNL_CHECK's status-to-text, torch_mlu/csrc/aten/utils/exceptions.h:77-83
 *   sdpa_b200_dropout_keep_mask[_varlen]
 *                            <- the Philox state the reference hands to its kernel (cnnlRandGenerator / seed, offset,
 *                               .../internal/FlashAttention_internal.cpp:190-214): here the pattern itself, as bits
 *   bias / dbias fields      <- the attn_bias and grad_bias descriptors of mem_eff_fwd / mem_eff_bwd
 *                               (.../internal/FlashAttention_internal.cpp:485-904)
 *
 * Conventions
 *   - Plain C: pointers, sizes, one POD struct. No C++ or torch types cross this boundary.
 *   - Every pointer in sdpa_b200_params is a DEVICE pointer on the caller's current device.
 *   - The caller owns every buffer including the workspace; the library allocates no device
 *     memory and keeps no per-call state.
 *   - Calls enqueue work on `stream` and return without synchronising.
 *   - Errors are integer status codes; nothing throws, aborts or traps the device. A kernel
 *     whose internal wait runs out writes SDPA_B200_DEVICE_TIMEOUT into the first word of
 *     the workspace; sdpa_b200_read_device_status() fetches it (it synchronises the stream).
 *   - Layout: element strides for (batch, head, row); the head_dim stride must be 1.
 *       dense   : cu_seqlens_* == NULL, batch b / head h / row r of q lives at
 *                 q + b*q_batch_stride + h*q_head_stride + r*q_row_stride (any BHLD/BLHD view)
 *       varlen  : cu_seqlens_q/k are int32[batch+1] exclusive prefix sums; tensors are packed
 *                 [total_tokens, heads, head_dim]; *_batch_stride is ignored and row r of
 *                 sequence b is token cu_seqlens[b] + r.
 *   - lse (natural-log logsumexp of scale*QK^T over the visible keys, fp32):
 *       dense   : [batch, heads_q, seqlen_q] contiguous
 *       varlen  : [heads_q, total_q] contiguous (the buffer mha_varlen_fwd allocates,
 *                 FlashAttention_internal.cpp:129)
 *     A row with no visible key gets out = 0 and lse = +inf.
 *   - Causal masking is bottom-right aligned: key j is visible to query i when
 *     j <= i + seqlen_k - seqlen_q (the reference test oracle's rule,
 *     test/torch_ops/test_scaled_dot_product_attention.py:69). With seqlen_q == seqlen_k it is
 *     the usual lower triangle.
 *   - GQA/MQA: heads_q % heads_kv == 0; query head h reads KV head h / (heads_q/heads_kv)
 *     (FlashAttention_internal.cpp:117-124).
 */
#ifndef SDPA_B200_H_
#define SDPA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SDPA_B200_VERSION 108

#if defined(__GNUC__)
#define SDPA_B200_API __attribute__((visibility("default")))
#else
#define SDPA_B200_API
#endif

/* status codes */
enum {
  SDPA_B200_OK = 0,
  SDPA_B200_INVALID_ARG = 1,    /* null pointer, bad shape, bad stride/alignment, workspace too small */
  SDPA_B200_UNSUPPORTED = 2,    /* valid request this build has no kernel for (dtype, head_dim > 128 with a bias, decode with bias) */
  SDPA_B200_LAUNCH_FAILED = 3,  /* CUDA reported an error while configuring or launching */
  SDPA_B200_DEVICE_TIMEOUT = 4, /* a bounded wait inside a kernel ran out (read back from workspace) */
  SDPA_B200_NO_DEVICE = 5       /* not an sm_100 device / no CUDA driver */
};

enum { SDPA_B200_BF16 = 0, SDPA_B200_F16 = 1 }; /* element type of q, k, v, out and gradients (the reference
                                                   takes the same two: sdp_utils.h:433-455) */

/* kernel selection for the forward entry point */
enum {
  SDPA_B200_KERNEL_AUTO = 0,    /* decode when max_seqlen_q is small, prefill otherwise */
  SDPA_B200_KERNEL_PREFILL = 1, /* TMA + tcgen05 tile kernel */
  SDPA_B200_KERNEL_DECODE = 2   /* split-KV streaming kernel */
};

typedef struct sdpa_b200_params {
  /* inputs */
  const void* q; /* bf16 */
  const void* k;
  const void* v;
  /* forward outputs (inputs of backward) */
  void* out;  /* bf16, same shape as q */
  float* lse; /* fp32, layout above */
  /* backward only */
  const void* dout; /* bf16, same shape/strides family as out */
  void* dq;         /* bf16, shape of q */
  void* dk;         /* bf16, shape of k */
  void* dv;         /* bf16, shape of v */

  /* varlen: device int32[batch+1]; NULL for dense */
  const int32_t* cu_seqlens_q;
  const int32_t* cu_seqlens_k;

  int32_t batch;
  int32_t heads_q;
  int32_t heads_kv;
  int32_t head_dim;     /* a multiple of 8, at most 256 (SDPA_B200_KERNEL_DECODE: 64 or 128; with a bias: at most 128) */
  int32_t max_seqlen_q; /* dense: seqlen_q */
  int32_t max_seqlen_k; /* dense: seqlen_k */
  int32_t total_q;      /* varlen: rows of q/out; dense: ignored */
  int32_t total_k;      /* varlen: rows of k/v;   dense: ignored */

  /* element strides; head_dim stride is 1 */
  int64_t q_batch_stride, q_head_stride, q_row_stride;
  int64_t k_batch_stride, k_head_stride, k_row_stride;
  int64_t v_batch_stride, v_head_stride, v_row_stride;
  int64_t o_batch_stride, o_head_stride, o_row_stride;
  /* backward */
  int64_t do_batch_stride, do_head_stride, do_row_stride;
  int64_t dq_batch_stride, dq_head_stride, dq_row_stride;
  int64_t dk_batch_stride, dk_head_stride, dk_row_stride;
  int64_t dv_batch_stride, dv_head_stride, dv_row_stride;

  float softmax_scale; /* > 0; the reference default is 1/sqrt(head_dim), sdp_utils.h:40-47 */
  float dropout_p;     /* 0, or inside (0, 1) together with keep_rows / keep_cols */
  int32_t is_causal;
  int32_t dtype;      /* SDPA_B200_BF16 or SDPA_B200_F16 */
  int32_t kernel;     /* SDPA_B200_KERNEL_* (forward only) */
  int32_t num_splits; /* decode: 0 = choose; otherwise the number of KV splits */
  /* Dropout keep-masks written by sdpa_b200_dropout_keep_mask() (dense) or ..._varlen() (packed) for the same
   * batch, heads_q and sequence lengths; both NULL when dropout_p == 0. The forward reads keep_rows; the
   * backward reads both. */
  const uint32_t* keep_rows;
  const uint32_t* keep_cols;
  /* Additive attention bias of the memory-efficient operators (mem_eff_fwd / mem_eff_bwd,
   * FlashAttention_internal.cpp:485-904): out = softmax(scale * q k^T + bias) v. NULL = none. Same 16-bit
   * type as q; element strides for (batch, head, query row), 0 for a broadcast dimension; the key stride is 1.
   * Rows start 16-byte aligned (row stride a multiple of 8, or 0) and are readable up to the next multiple of
   * 8 keys. With packed (varlen) q / k / v the bias stays a [batch, heads_q, max_seqlen_q, max_seqlen_k] tensor:
   * sequence b reads bias[b, h, i, j] for its query i and key j counted from the start of the sequence. The
   * same holds for dbias and bias_t. */
  const void* bias;
  int64_t bias_batch_stride, bias_head_stride, bias_row_stride;
  /* Backward: gradient of the bias, [batch, heads_q, seqlen_q, dbias_row_stride >= seqlen_k rounded up to 8],
   * same type, or NULL. Elements the causal mask hides are not written: clear the buffer first. */
  void* dbias;
  int64_t dbias_batch_stride, dbias_head_stride, dbias_row_stride;
  /* Backward, optional: the same bias with keys and queries exchanged, [batch, heads_q, seqlen_k, seqlen_q]
   * with unit query stride and the rules of `bias` for alignment and padding (strides for batch, head, key row).
   * The dK/dV kernel, whose threads own keys, then reads 16 bytes at a time instead of two. Not needed when the
   * bias does not depend on the query (bias_row_stride == 0). NULL = not given. */
  const void* bias_t;
  int64_t bias_t_batch_stride, bias_t_head_stride, bias_t_row_stride;
  /* Backward: 0 = the fused kernel, which forms every tile's scores once and adds its dQ contributions into an
   * fp32 workspace with floating-point reductions whose order varies between launches (dK and dV are still summed
   * in a fixed order); non-zero = separate dK/dV and dQ kernels with fixed summation order throughout, so that the
   * same call gives the same bits every time, at about 1.4x the time. A call with a bias always takes the second
   * path. Ignored by the forward. */
  int32_t deterministic;
  /* Forward (tile kernel): number of SMs the persistent kernel leaves free, for a kernel that is to run beside it on
   * another stream - a collective that reassembles the previous step's outputs, say. 0 = one CTA on every SM, which
   * keeps any other kernel out until the CTAs leave. At least one SM is always used. */
  int32_t sm_margin;
  /* Optional device word (4-byte aligned) that collects kernel status across calls: a kernel whose bounded wait
   * runs out stores SDPA_B200_DEVICE_TIMEOUT there. The library never clears it, so one word can watch a whole
   * stream of calls whose workspaces come and go; read it with sdpa_b200_read_device_status and clear it
   * yourself. NULL = the first word of the call's workspace, cleared at the start of each call. */
  uint32_t* device_status;
} sdpa_b200_params;

SDPA_B200_API int sdpa_b200_version(void);
SDPA_B200_API const char* sdpa_b200_status_string(int status);
/* Text of the last error raised on the calling thread (what was wrong and where). */
SDPA_B200_API const char* sdpa_b200_last_error(void);

/* Workspace size the matching call needs for these params (>= 256 bytes; 256-byte aligned
 * base required). */
SDPA_B200_API int sdpa_b200_fwd_workspace_bytes(const sdpa_b200_params* p, size_t* bytes);
SDPA_B200_API int sdpa_b200_bwd_workspace_bytes(const sdpa_b200_params* p, size_t* bytes);

/* out, lse <- attention(q, k, v). `stream` is a cudaStream_t passed as void*. */
SDPA_B200_API int sdpa_b200_fwd(const sdpa_b200_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* dq, dk, dv <- backward(dout, q, k, v, out, lse). */
SDPA_B200_API int sdpa_b200_bwd(const sdpa_b200_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* Synchronises `stream`, reads the status word a kernel may have left in `workspace` (or in the word given as
 * sdpa_b200_params.device_status) and returns it in *device_status (SDPA_B200_OK or SDPA_B200_DEVICE_TIMEOUT). */
SDPA_B200_API int sdpa_b200_read_device_status(const void* workspace, void* stream, int* device_status);

/* Self-test of the time-out path every kernel of this library shares: launches one warp that waits, for at most
 * `budget_us` microseconds, on a shared-memory barrier nobody will ever arrive on - no copy or MMA is in flight -
 * then gives up exactly as the attention kernels do: it stores SDPA_B200_DEVICE_TIMEOUT into *device_status and
 * returns normally, leaving the context usable. No counterpart in the reference, whose vendor kernels report
 * nothing back from the device. */
SDPA_B200_API int sdpa_b200_selftest_wait_timeout(uint32_t* device_status, uint32_t budget_us, void* stream);

/* Split-KV decode (dense tensors, seqlen_q == 1) for callers that cannot allocate device memory
 * where they call it - inside an allocator or memory-pool callback, or after the process has
 * frozen its memory plan. No counterpart in the reference: its attention calls always take a
 * workspace from the caching allocator (FlashAttention_internal.cpp:215-230). The caller passes
 * inputs and outputs only; the split partials live in a fixed SDPA_B200_STATIC_SCRATCH_BYTES
 * array inside the library (held by every GPU that loads it). Requests whose partials
 * (batch * heads_q * splits * 516 bytes) exceed it are refused with SDPA_B200_INVALID_ARG. The
 * first call on each device looks the array's address up; make it outside stream capture. Calls
 * that overlap on one GPU race on the shared array - order them on one stream. */
#define SDPA_B200_STATIC_SCRATCH_BYTES (16u << 20)
SDPA_B200_API int sdpa_b200_decode_static(const sdpa_b200_params* p, void* stream);

/* Folds one partial attention result into an fp32 accumulator by the logsumexp rule (the combine
 * step of ring / context-parallel prefill; no counterpart in the reference, whose attention is
 * single-device):  lse' = log(exp(lse_acc) + exp(lse_part)),
 *                  o_acc' = o_acc*exp(lse_acc - lse') + o_part*exp(lse_part - lse').
 * o_acc [batch, heads, rows, head_dim] fp32 and lse_acc / lse_part [batch, heads, rows] fp32 are
 * contiguous; o_part is bf16 or f16 (`dtype`) with the given element strides (the `out` of
 * sdpa_b200_fwd).
 * Start an accumulator with lse_acc = -inf (o_acc may be uninitialised). */
SDPA_B200_API int sdpa_b200_merge_partial(float* o_acc, float* lse_acc, const void* o_part, const float* lse_part,
                                          int32_t batch, int32_t heads, int32_t rows, int32_t head_dim,
                                          int32_t dtype, int64_t part_batch_stride, int64_t part_head_stride,
                                          int64_t part_row_stride, void* stream);

/* Dropout pattern for one attention call, one bit per (query, key) pair, drawn from Philox4x32-10 with the
 * given seed and offset (the reference draws it inside its device kernel from such a pair,
 * FlashAttention_internal.cpp:190-214, and returns the pair so that the backward pass can repeat it; here the
 * caller generates the masks again from the pair before calling sdpa_b200_bwd, or keeps them).
 *   keep_rows: uint32 [batch*heads][Lq_pad][Lk_pad/32], bit (k & 31) of word (q, k >> 5) set = pair kept
 *   keep_cols: uint32 [batch*heads][Lk_pad][Lq_pad/32], bit (q & 31) of word (k, q >> 5): the transpose
 * Lq_pad / Lk_pad are the lengths rounded up to a multiple of 128; `heads` is heads_q. A pair is dropped with
 * probability round(dropout_p * 256) / 256; kept probabilities are scaled by 1 / (1 - dropout_p) in the
 * attention kernels. With `is_causal` (the bottom-right
 * aligned mask of the attention calls) 128 x 128 tiles that the mask hides completely are filled with zeros
 * instead of random bits; a call made with is_causal must be given masks made with it or without it, never the
 * other way round. */
SDPA_B200_API int sdpa_b200_dropout_keep_mask(uint64_t seed, uint64_t offset, float dropout_p, int32_t batch,
                                              int32_t heads, int32_t seqlen_q, int32_t seqlen_k, int32_t is_causal,
                                              uint32_t* keep_rows, uint32_t* keep_cols, void* stream);

/* The same pattern for packed (varlen) tensors: sequence b of the batch gets the bits batch index b would get
 * in the dense form, addressed by packed token index:
 *   keep_rows: uint32 [heads][total_q + 128][Lk_pad/32], row = packed query index, bit = key position inside
 *              the query's sequence;   keep_cols: uint32 [heads][total_k + 128][Lq_pad/32], the transpose.
 * Lq_pad / Lk_pad are max_seqlen_q / max_seqlen_k rounded up to 128. Both arrays must arrive zero-filled: only
 * words an attention kernel reads are written. */
SDPA_B200_API int sdpa_b200_dropout_keep_mask_varlen(uint64_t seed, uint64_t offset, float dropout_p, int32_t batch,
                                                     int32_t heads, const int32_t* cu_seqlens_q,
                                                     const int32_t* cu_seqlens_k, int32_t total_q, int32_t total_k,
                                                     int32_t max_seqlen_q, int32_t max_seqlen_k, int32_t is_causal,
                                                     uint32_t* keep_rows, uint32_t* keep_cols, void* stream);

/* Writes sdpa_b200_params.bias_t for a bias given as in sdpa_b200_params (16-bit elements, element strides, unit
 * key stride, row_stride != 0): out is [batch][heads][seqlen_k][out_row_stride], contiguous, out_row_stride a
 * multiple of 8 that holds seqlen_q; the padding is zero-filled. Pass batch = 1 (heads = 1) for a bias that is
 * broadcast along that dimension and give bias_t the stride 0 there. */
SDPA_B200_API int sdpa_b200_transpose_bias(const void* bias, int64_t batch_stride, int64_t head_stride, int64_t row_stride,
                                           int32_t batch, int32_t heads, int32_t seqlen_q, int32_t seqlen_k, void* out,
                                           int64_t out_row_stride, void* stream);

/* How many of this library's kernels the calling process has launched so far. */
SDPA_B200_API uint64_t sdpa_b200_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* SDPA_B200_H_ */
