/*
 * fdma.h -- C ABI of libfdma_sm100.so: dynamic-mask attention for NVIDIA B200 (sm_100a).
 *
 * The library replaces the pybind11 module `flash_sparse_attn_cuda` of SmallDoges/flash-dmattn
 * (csrc/flash_sparse_attn/flash_api.cpp:1270-1276: `fwd`, `bwd`) and the ATen calls inside
 * flash_sparse_attn/utils/mask.py:76-120 (`topk_mask`) with plain-C entry points:
 * POD parameter blocks, raw device pointers, element strides, an explicit CUDA stream.
 *
 * Rules common to every entry point
 *  - Nothing here allocates or frees device memory unless its comment says so. The caller owns
 *    inputs, outputs and the scratch buffer (`workspace`), whose size comes from the matching
 *    *_workspace_bytes() call, and keeps them alive until the stream work has finished.
 *  - All work is enqueued on `stream` (a cudaStream_t passed as void*); no hidden synchronisation.
 *  - Return value: 0 on success, a negative fdma_status, or a positive cudaError_t value.
 *    fdma_strerror() turns either into text. Nothing throws and nothing calls exit().
 *  - Strides are in ELEMENTS of the tensor's dtype. The innermost (head-dim / key) stride is 1.
 *    A stride of 0 means "broadcast along that dimension" (the reference does the same,
 *    flash_api.cpp:79-82, :90-91).
 */
#ifndef FDMA_H_
#define FDMA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FDMA_VERSION 10100 /* 1.1.0: fdma_fwd_params grew by mask_bits / tile_activity, fdma_mask_params by bits / activity */

enum fdma_dtype { FDMA_BF16 = 0, FDMA_FP16 = 1, FDMA_FP32 = 2 };

enum fdma_status {
  FDMA_OK = 0,
  FDMA_ERR_BAD_ARG = -1,       /* NULL pointer, negative size, inconsistent heads ...           */
  FDMA_ERR_UNSUPPORTED = -2,   /* head dim > 256 or not a multiple of 8, dtype not handled ...  */
  FDMA_ERR_WORKSPACE = -3,     /* workspace missing or smaller than *_workspace_bytes()         */
  FDMA_ERR_ARCH = -4,          /* device is not compute capability 10.x                         */
  FDMA_ERR_DRIVER = -5,        /* tensor-map encode entry point unavailable                     */
  FDMA_ERR_TIMEOUT = -6,       /* a bounded in-kernel wait gave up (reported by fdma_last_kernel_status) */
  FDMA_ERR_TOO_LARGE = -7      /* static-scratch variant: problem exceeds the compiled-in limit  */
};

/* Which kernel family the launcher picks. AUTO: the row-gather decode kernel for single-query calls
 * (seqlen_q == 1, head dim 64/128/256), tcgen05/TMA kernels where shape and alignment allow, the
 * CUDA-core kernels otherwise. The other values force one family (tests use them); forcing a family
 * on a shape it does not handle returns FDMA_ERR_UNSUPPORTED. */
enum fdma_path { FDMA_PATH_AUTO = 0, FDMA_PATH_SIMT = 1, FDMA_PATH_TCGEN05 = 2, FDMA_PATH_DECODE = 3 };

/*
 * Forward: O = softmax(scale * Q K^T + bias, masked) V, LSE = logsumexp of the masked scores.
 * Replaces `mha_fwd` (flash_api.cpp:351-554) + `set_params_fprop` (:24-153) and the kernels behind
 * `run_mha_fwd` (:251-267). Tensor meaning follows Flash_fwd_params (src/flash.h:80-160):
 *   q (B,Sq,H,d)  k,v (B,Sk,Hk,d)  out (B,Sq,H,d)  lse (B,H,Sq) fp32 contiguous
 *   mask: bool bytes ({B|1},{H|Hk|1},{Sq|1},Sk...) , bias: dtype of q, same broadcast rules.
 * mask/bias rows must be readable up to round_up(Sk,128) keys (the Python layer pads them the way
 * flash_sparse_attn_interface.py:420-430 does); keys >= Sk are ignored.
 * Causal alignment is bottom-right: key k is visible to query q iff k <= q + Sk - Sq (src/mask.h:39).
 * Rows with no visible key give O = 0 and LSE = +inf (src/softmax.h:211-214).
 */
typedef struct fdma_fwd_params {
  const void* q;
  const void* k;
  const void* v;
  const void* mask; /* may be NULL: nothing masked  */
  const void* bias; /* may be NULL: zero bias       */
  void* out;
  float* lse;
  int64_t q_batch_stride, q_row_stride, q_head_stride;
  int64_t k_batch_stride, k_row_stride, k_head_stride;
  int64_t v_batch_stride, v_row_stride, v_head_stride;
  int64_t o_batch_stride, o_row_stride, o_head_stride;
  int64_t mask_batch_stride, mask_head_stride, mask_row_stride;
  int64_t bias_batch_stride, bias_head_stride, bias_row_stride;
  int32_t b, seqlen_q, seqlen_k, h, h_k, h_mask, h_bias, d;
  int32_t dtype;     /* fdma_dtype of q/k/v/out/bias: BF16 or FP16 */
  int32_t is_causal; /* ignored (treated as 0) when seqlen_q == 1, flash_api.cpp:441 */
  float softmax_scale;
  int32_t path;      /* fdma_path */
  void* workspace;
  size_t workspace_bytes;
  /* Optional key positions, for K/V that were compacted to the kept keys (fdma_compact_gather): int32
   * ({B|1}, h_pos, Sk), ascending along the key dimension, h_pos in {1, h_k, h}. NULL: key k sits at position k.
   * When given, the causal test of key k is key_pos[k] <= q + causal_shift (causal_shift = original Sk - Sq);
   * is_causal = 0 ignores both. No counterpart in the reference's CUDA backend (its Triton prototype
   * flash_dmattn_triton.py:49-211 gathers keys the same way). */
  const int32_t* key_pos;
  int64_t key_pos_batch_stride, key_pos_head_stride;
  int32_t h_pos;
  int32_t causal_shift;
  /* Optional bit-packed per-query mask (what fdma_create_mask writes through fdma_mask_params::bits, together with
   * the tile activity below): non-zero mask_bits says that `mask` points to uint32 words -- bit (k & 31) of word
   * k >> 5 of a row is key k -- and that the three mask strides count WORDS; a row holds round_up(Sk,128)/32 words
   * (bits of keys >= Sk are zero), base and strides multiples of 16 bytes. One eighth of the bool tensor's bytes on
   * every pass of the forward and the backward. Taken by the tcgen05 kernels for masks with one row per query
   * (mask_row_stride != 0; forward at d = 64 / 128 / 256, backward at d = 128) and only together with
   * tile_activity; every other combination returns FDMA_ERR_UNSUPPORTED, and the caller expands the bits to bytes.
   * No counterpart in the reference (its mask is always a bool tensor, flash_api.cpp:388-391). */
  int32_t mask_bits;
  int32_t reserved;
  /* Optional, per-query masks: one byte per 128 x 128 tile, (B, h_mask, ceil(Sq/128), ceil(Sk/128)) contiguous,
   * non-zero iff the tile holds a kept element (tiles wholly beyond the causal limit may be marked either way).
   * When given, the kernels use it instead of deriving it from the mask into the workspace first. */
  const uint8_t* tile_activity;
} fdma_fwd_params;

size_t fdma_fwd_workspace_bytes(const fdma_fwd_params* p);
int fdma_fwd(const fdma_fwd_params* p, void* stream);

/*
 * Backward: dQ, dK, dV and dBias for the forward above, given dOut, Out and LSE.
 * Replaces `mha_bwd` (flash_api.cpp:792-1050) + `set_params_dgrad` (:155-249), the three launches of
 * run_flash_bwd_seqk_parallel (src/flash_bwd_launch_template.h:71-117) and the at::sum_out
 * reductions over the query-head group and broadcast dimensions (flash_api.cpp:1027-1047), which
 * happen inside the kernels here.
 *   dq like q, dk/dv like k/v (already summed over the H/Hk query heads that share a kv head),
 *   dbias has the SHAPE OF BIAS (strides given), already summed over every dimension in which
 *   bias is broadcast (batch, head group, query).  dbias may be NULL (no bias gradient wanted).
 * Outputs are overwritten; they need not be zeroed by the caller.
 */
typedef struct fdma_bwd_params {
  fdma_fwd_params f; /* q,k,v,mask,bias,out,lse + geometry exactly as given to fdma_fwd */
  const void* dout;  /* (B,Sq,H,d) */
  int64_t do_batch_stride, do_row_stride, do_head_stride;
  void* dq;
  void* dk;
  void* dv;
  void* dbias; /* may be NULL */
  int64_t dq_batch_stride, dq_row_stride, dq_head_stride;
  int64_t dk_batch_stride, dk_row_stride, dk_head_stride;
  int64_t dv_batch_stride, dv_row_stride, dv_head_stride;
  int64_t dbias_batch_stride, dbias_head_stride, dbias_row_stride;
  int32_t dbias_b, dbias_h, dbias_rows; /* extents of dbias dims 0..2 (1 where bias is broadcast) */
  int32_t dbias_keys;                   /* extent of the key dimension of dbias (>= Sk)          */
  int32_t deterministic;                /* flash_api.cpp:809. Non-zero: the tensor-core backward kernels sum dQ in
                                           64-bit fixed point (order-independent, bit-identical between runs; about 40 %
                                           slower). The CUDA-core backward computes each dQ row in one warp (fixed order) but
                                           sums dK, dV and dBias with fp32 atomics. On the tensor-core kernels dK, dV and
                                           dBias (except dBias shared across batch / kv heads) have a fixed summation
                                           order in both modes */
  int32_t reserved;
  float* softmax_d; /* optional out, may be NULL: D = rowsum(dOut o Out) as fp32 (B, H, round_up(Sq,128)) contiguous,
                       zeros in the padding columns -- the `softmax_d` tensor mha_bwd returns (flash_api.cpp:952,
                       :1049) */
} fdma_bwd_params;

size_t fdma_bwd_workspace_bytes(const fdma_bwd_params* p);
int fdma_bwd(const fdma_bwd_params* p, void* stream);

/*
 * create_mask: bool mask of the `window` largest bias entries along the key dimension of each row.
 * Replaces `topk_mask` / `relu_mask` / `block_smooth` of flash_sparse_attn/utils/mask.py:47-160
 * (torch.topk + scatter_ there). Output rows follow the broadcast of bias and pre-mask shapes.
 *   value(row,k) = premask(row,k) ? bias(row,k) : min_value
 *   kind TOPK : out = 1 for the `window` largest values of the row, except where value == min_value
 *               (mask.py:102-110). Equal values at the selection threshold are taken in ascending
 *               key order.
 *   kind RELU : out = value > 0 (mask.py:147-149)
 *   block_size > 1: afterwards each block of `block_size` keys (and the shorter tail block) is set
 *               to "more than half of the block was selected" (mask.py:47-73).
 * Rows are indexed (b, h, r) over out_b x out_h x out_rows; bias / premask strides may be 0.
 */
enum fdma_mask_kind { FDMA_MASK_TOPK = 0, FDMA_MASK_RELU = 1 };

typedef struct fdma_mask_params {
  const void* bias;
  const void* premask; /* bool bytes, may be NULL */
  void* out;           /* bool bytes, contiguous (out_b,out_h,out_rows,keys) */
  int64_t bias_batch_stride, bias_head_stride, bias_row_stride;
  int64_t pm_batch_stride, pm_head_stride, pm_row_stride;
  int32_t out_b, out_h, out_rows, keys;
  int32_t window;
  int32_t dtype;      /* fdma_dtype of bias: BF16, FP16 or FP32 */
  int32_t kind;       /* fdma_mask_kind */
  int32_t block_size; /* 0 or 1: no smoothing */
  float min_value;    /* the caller's min_dtype (mask.py:171) */
  /* Optional position output (kind TOPK, no block smoothing): the selection written directly as the sorted index
   * list that the reference builds with topk + sort in `topk_indices` (mask.py:20-44), without the bool tensor in
   * between. key_pos (rows, capacity) int32 receives the ascending positions of the selected keys of each row
   * (rows = out_b*out_h*out_rows, in that order), INT32_MAX in the unused slots; count (rows) their number;
   * slot_mask (rows, capacity) bool bytes, if given, slot < count. capacity >= min(window, keys). With key_pos
   * given, `out` may be NULL (no bool mask is written). These are exactly the tensors fdma_compact_index derives
   * from a bool mask, so fdma_gather_rows / fdma_fwd_params::key_pos take them as they are. */
  int32_t* key_pos;
  int32_t* count;
  void* slot_mask;
  int32_t capacity;
  int32_t reserved;
  /* Optional bit-packed output for per-query masks (kind TOPK, no block smoothing, 16-bit bias rows of at most 32768
   * keys with keys % 8 == 0): `bits` (out_b, out_h, out_rows, round_up(keys,128)/32) uint32, contiguous, bit (k & 31)
   * of word k >> 5 = key k selected, and `activity` (out_b, out_h, ceil(out_rows/128), ceil(keys/128)) bytes, 1 for
   * every 128 x 128 tile that holds a selected key and 0 otherwise. The kernel writes the bits of keys [0, keys) of
   * every row and `activity` in full; when keys is not a multiple of 128 the caller zero-fills `bits` first (the
   * padding bits of each row's last words must read 0). With `bits` given, `out` may be NULL. These
   * are the tensors fdma_fwd_params takes as mask (mask_bits = 1) and tile_activity. Other configurations return
   * FDMA_ERR_UNSUPPORTED. */
  uint32_t* bits;
  uint8_t* activity;
} fdma_mask_params;

int fdma_create_mask(const fdma_mask_params* p, void* stream);

/* Text for a status returned by any call above (fdma_status or cudaError_t). Never NULL. */
const char* fdma_strerror(int status);

/* FDMA_VERSION the library was built from. */
int fdma_version(void);

/*
 * The tcgen05 kernels bound every wait on an mbarrier; a wait that runs out records a code in a
 * per-device status word instead of hanging. This call copies the word to the host (it
 * synchronises `stream`), clears it, and returns 0 or FDMA_ERR_TIMEOUT. `detail`, if not NULL,
 * receives the raw code (which wait gave up).
 */
int fdma_last_kernel_status(void* stream, int32_t* detail);

/*
 * Non-blocking look at the same condition on the CURRENT device: a kernel whose wait gives up also stores its code
 * into 4 bytes of page-locked host memory (allocated once per device by the first tcgen05 launch there), which this
 * call reads without touching the GPU. Returns 0 or FDMA_ERR_TIMEOUT; clears nothing (fdma_last_kernel_status
 * does). A host layer can call it at the entry of every operator call and learn of a timed-out earlier kernel
 * whose results must not be trusted. No counterpart in the reference.
 */
int fdma_poll_kernel_status(int32_t* detail);

/*
 * Self-test of the bounded wait (no counterpart in the reference): one small CTA allocates tensor memory and
 * waits on an mbarrier that nothing arrives on, with a limit of `limit_us` microseconds (1 .. 1 000 000). The wait
 * gives up, records code 901 in the status word, and the CTA frees its tensor memory and returns; *result_dev
 * (device int) becomes 1 when every thread saw the wait fail. The next fdma_last_kernel_status call returns
 * FDMA_ERR_TIMEOUT with detail 901. It cannot hang: the only wait in it is the bounded one.
 */
int fdma_selftest_wait_timeout(uint32_t limit_us, int* result_dev, void* stream);

/*
 * Forward pass with library-owned scratch. It has no counterpart in the reference (whose C++ side allocates
 * its own temporaries with torch::empty). Same arguments, results and status codes as fdma_fwd, except that
 * p->workspace / p->workspace_bytes are ignored: whatever scratch fdma_fwd_workspace_bytes(p) asks for lives in a
 * fixed 1 MiB array inside the library (fdma_static_scratch_limit() returns that size). It exists for hosts
 * that cannot supply scratch at call time -- engines that partition device memory once at start-up and give
 * their operators no allocator, or loops where a device allocation is not acceptable. It allocates and frees
 * nothing. Two kinds of call need scratch, and the limit applies to each as fdma_fwd_workspace_bytes reports it
 * (query it first to know):
 *   - a per-query mask: one activity byte per 128x128 tile, B * h_mask * ceil(Sq/128) * ceil(Sk/128) bytes;
 *   - a single-query call (seqlen_q == 1, with or without a mask) on the row-gather decode kernel: per-split
 *     partials B * H * splits * 8 * (d + 2) * 4 bytes (splits >= 1, chosen from Sk and the SM count), e.g. 1.02 MiB --
 *     over the limit -- at B * H = 256, d = 128 with one split.
 * A call needing more than the limit returns FDMA_ERR_TOO_LARGE and launches nothing. The first call on each
 * device resolves the array's address: issue it outside any stream capture. Calls share the array; calls whose
 * GPU work overlaps in time race and must be serialised by the caller.
 */
int fdma_fwd_static_scratch(const fdma_fwd_params* p, void* stream);
size_t fdma_static_scratch_limit(void);

/*
 * Key compaction for row-broadcast masks (no counterpart in the reference's CUDA backend; its Triton prototype
 * gathers the top-k keys the same way, flash_sparse_attn/flash_dmattn_triton.py:49-211). When all queries of a
 * (batch, head) keep the same W of Sk keys, attention over the W gathered keys equals attention over all Sk keys,
 * provided the causal test uses the keys' original positions (fdma_fwd_params::key_pos).
 *
 * fdma_compact_index: for every mask row writes the ascending positions of its kept keys into
 * key_pos[row][0..count), INT32_MAX into the remaining slots, the number of kept keys into count[row] (which
 * may exceed `capacity`: positions beyond the capacity are dropped, the caller must check), and, when mask_out is
 * given, slot < count into mask_out[row][slot].
 */
typedef struct fdma_compact_params {
  const void* mask;                 /* bool bytes (b_mask, h_mask, seqlen_k), keys contiguous */
  int64_t mask_batch_stride, mask_head_stride;
  int32_t b_mask, h_mask, seqlen_k, capacity;
  int32_t* key_pos;                 /* out, dense (b_mask, h_mask, capacity) */
  int32_t* count;                   /* out, dense (b_mask, h_mask) */
  void* mask_out;                   /* out or NULL, dense bool bytes (b_mask, h_mask, capacity) */
} fdma_compact_params;
int fdma_compact_index(const fdma_compact_params* p, void* stream);

/*
 * fdma_gather_rows: dst[b][slot][h][:] = src[b][key_pos[b][h / (heads / h_pos)][slot]][h][:], zeros in slots whose
 * position is outside [0, rows_full). src is (b, rows_full, heads, row_elems), dst (b, capacity, heads,
 * row_elems); strides in elements, the innermost dimension is contiguous. A (B, H, 1, Sk) bias is passed as
 * row_elems = 1, row stride 1, head stride = its head stride.
 * fdma_scatter_rows: the inverse for gradients: dst (b, rows_full, heads, row_elems) is zero-filled, then
 * dst[b][key_pos[..][slot]][h][:] = src[b][slot][h][:] for the filled slots.
 */
typedef struct fdma_rows_params {
  const void* src;
  void* dst;
  const int32_t* key_pos;
  int64_t key_pos_batch_stride, key_pos_head_stride; /* batch stride 0 for a batch-broadcast list */
  int64_t src_batch_stride, src_row_stride, src_head_stride;
  int64_t dst_batch_stride, dst_row_stride, dst_head_stride;
  int32_t b, heads, h_pos, rows_full, capacity, row_elems;
  int32_t dtype;                    /* FDMA_BF16 or FDMA_FP16 */
  int32_t reserved_;
} fdma_rows_params;
int fdma_gather_rows(const fdma_rows_params* p, void* stream);
int fdma_scatter_rows(const fdma_rows_params* p, void* stream);

/*
 * fdma_merge_partials: folds a partial attention result computed over a subset of the keys into a running result,
 * with the rule of the reference's split-KV combine kernel (src/flash_fwd_kernel.h:1695-1727):
 *   lse' = log(exp(lse_acc) + exp(lse_part)),  acc' = exp(lse_acc - lse') acc + exp(lse_part - lse') part.
 * acc (B,Sq,H,d) fp32 contiguous and lse_acc (B,H,Sq) fp32 are updated in place; start them at 0 and -inf.
 * part is a 16-bit forward output (strides in elements), lse_part its LSE, where +inf (the forward's value for a row
 * without a visible key) counts as "no contribution". d a multiple of 8, at most 256; 16-byte aligned rows.
 */
typedef struct fdma_merge_params {
  float* acc;
  float* lse_acc;
  const void* part;
  const float* lse_part;
  int64_t part_batch_stride, part_row_stride, part_head_stride;
  int32_t b, seqlen_q, h, d;
  int32_t dtype; /* fdma_dtype of part: BF16 or FP16 */
  int32_t reserved;
} fdma_merge_params;
int fdma_merge_partials(const fdma_merge_params* p, void* stream);

/*
 * Measurement hook (no counterpart in the reference, which is timed from Python with wall clocks,
 * benchmarks/forward_performance.py:388-399). The NEXT fdma_fwd or fdma_bwd call made by this host thread
 * records `start_event` immediately before and `stop_event` immediately after its main attention kernel
 * (not the small pre/post kernels), on the stream given to that call, then forgets both. Events are
 * cudaEvent_t handles created by the caller with timing enabled. Pass NULLs to cancel.
 */
void fdma_time_next_kernel(void* start_event, void* stop_event);

#ifdef __cplusplus
}
#endif
#endif /* FDMA_H_ */
