/*
 * fa8_b200.h - C ABI of the B200 (sm_100a) FP8 flash-attention forward.
 *
 * This is the boundary a foreign-language binding loads (libfa8_b200.so):
 * plain pointers and sizes, a CUDA stream handle passed as void*, an int
 * status as the return value.  No C++ or torch types cross it.
 *
 * It replaces the host entry of the reference extension,
 *   std::vector<torch::Tensor> flash_attention_v2_cutlass(q, k, v, is_causal,
 *   softmax_scale)            (include/attention_api.h:10-11,
 *                              csrc/flash_attention.cu:639-668),
 * i.e. set_params_fprop (csrc/flash_attention.cu:277-318), the dtype/head_dim/
 * causal dispatch (:618-637, csrc/static_switch.h) and run_flash_fwd (:586-610).
 * Differences, all deliberate:
 *   - the output is fp16 (the reference stores e4m3, :656 and :556-557);
 *   - the kernel is launched on the caller's stream and the call does not
 *     synchronise the device (the reference uses stream 0 and calls
 *     cudaDeviceSynchronize, :608-609 and :663-665);
 *   - errors come back as codes (the reference prints and exit()s,
 *     include/attention_api.cuh:20-29);
 *   - arguments are validated (the reference checks only device/contiguity,
 *     include/attention_api.cuh:12-18).
 */
#ifndef FA8_B200_H_
#define FA8_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FA8_OK 0
#define FA8_ERR_BAD_ARG (-1)        /* null pointer, non-positive size, misaligned pointer, bad scale */
#define FA8_ERR_UNSUPPORTED (-2)    /* shape or layout outside what the kernel implements */
#define FA8_ERR_CUDA (-3)           /* a CUDA runtime/driver call failed; see fa8_last_error_detail */
#define FA8_ERR_DEVICE_TIMEOUT (-4) /* a bounded wait inside the kernel expired (status word != 0) */

/* Layout of V.  The reference requires the caller to pass V transposed,
 * [batch, heads, head_dim, seqlen] (test.py:71, csrc/flash_attention.cu:376-379). */
#define FA8_V_TRANSPOSED 0 /* [batch, heads, head_dim, seqlen], seqlen contiguous (reference layout) */
#define FA8_V_NATURAL 1    /* [batch, heads, seqlen, head_dim], head_dim contiguous */

#define FA8_FP8_E4M3 0
#define FA8_FP8_E5M2 1

/* Arguments of one forward call; mirrors the live fields of the reference's
 * Flash_fwd_params (csrc/flash.h:6-61).  All tensors are contiguous device
 * memory, 16-byte aligned. */
typedef struct fa8_fwd_params {
  const void* q;   /* e4m3 [batch, heads, seqlen, head_dim] */
  const void* k;   /* e4m3 [batch, heads, seqlen, head_dim] */
  const void* v;   /* e4m3, layout given by v_layout */
  void* o;         /* fp16 [batch, heads, seqlen, head_dim], written by the call */
  int32_t batch;
  int32_t heads;
  int32_t seqlen;    /* query rows per head (and key rows unless seqlen_k says otherwise); any positive
                        length, except that the key/value length must be a multiple of 16 when V is
                        passed transposed (its rows are then that many bytes long) */
  int32_t head_dim;  /* a multiple of 32 up to 256, the reference's eight buckets (csrc/static_switch.h:
                        50-77); kernels exist for 64, 128 and 256, the others run zero-padded on the
                        next one up */
  float softmax_scale; /* > 0; P = exp(softmax_scale * (S - rowmax)) */
  int32_t is_causal;   /* 0/1; mask is lower-triangular including the diagonal (test.py:25-33) */
  int32_t v_layout;    /* FA8_V_TRANSPOSED or FA8_V_NATURAL */
  float o_scale;       /* O is multiplied by this; 1.0f reproduces the reference; a caller with
                          per-tensor scaled inputs folds V's descale here and Q's and K's into
                          softmax_scale */
  int32_t* status_word; /* optional device int32, zero before the call; the kernel stores a
                           non-zero code there if one of its bounded waits runs out, and CTAs that
                           find it non-zero return without writing O.  NULL = a word the library
                           keeps per device.  Either way the failure also reaches the host through
                           a flag of the library's own, see fa8_fwd. */
  float* softmax_lse;   /* optional device fp32 [batch, heads, seqlen]: log(sum_j exp(softmax_scale *
                           s_ij)) per query row, written when not NULL.  The reference carries the
                           pointer (softmax_lse_ptr, csrc/flash.h:56) but never fills it
                           (csrc/flash_attention.cu:310-311 passes nullptr). */
  int32_t heads_kv;     /* heads of K and V (grouped-query attention): 0 or `heads` = one K/V head per
                           query head, otherwise a divisor of `heads`; query head h reads K/V head
                           h / (heads / heads_kv).  K and V are then [batch, heads_kv, ...].  The
                           reference reserves k_head / h_h_k_ratio for this (csrc/flash.h:36-45) but
                           its kernel ignores them (csrc/flash_attention.cu:364-379). */
  const float* descale_q; /* optional device floats: x_true = descale * x_e4m3 per tensor.  When given, */
  const float* descale_k; /* the kernel multiplies softmax_scale by descale_q * descale_k and O by     */
  const float* descale_v; /* descale_v itself, so the outputs of fa8_quantize_e4m3 can be used without */
                          /* a device-to-host round trip.  The reference has no descale arguments        */
                          /* (include/attention_api.h:10-11).                                            */
  int32_t fp8_format;   /* FA8_FP8_E4M3 (0) or FA8_FP8_E5M2: element format of Q, K and V alike; P is
                           re-quantised to the same format.  The reference switches on the input dtype
                           the same way (FP8_SWITCH, csrc/flash_attention.cu:308,631). */
  int32_t seqlen_k;     /* rows of K and V per head when they differ from `seqlen` (cross attention,
                           a prompt attending to a longer cache); 0 = seqlen.  A multiple of 16 when V
                           is transposed, otherwise any positive length.  The
                           causal mask stays aligned top-left (key index <= query index), as in the
                           reference (csrc/flash_attention.cu:24-71); the reference carries q_seqlen and
                           k_seqlen separately (csrc/flash.h) but its test only runs them equal. */
  int32_t descale_per_head; /* 0: descale_q/k/v point to one float each (per tensor).  1: to arrays, one
                               float per (batch, head) for Q ([batch*heads]) and per (batch, K/V head)
                               for K and V ([batch*heads_kv]), as fa8_quantize_e4m3_segments writes them. */
} fa8_fwd_params;

/* Enqueues the forward on `cuda_stream` (a cudaStream_t; NULL = default stream)
 * of the current device.  Returns FA8_OK when the launch was accepted.  Replaces
 * flash_attention_v2_cutlass (csrc/flash_attention.cu:639-668).
 *
 * Failure reporting without a synchronisation: a kernel whose bounded wait ran out also stores
 * its code in a word of pinned host memory the library owns.  Every call looks at that word
 * first; if an earlier launch on this device left a code there, the call returns
 * FA8_ERR_DEVICE_TIMEOUT (fa8_last_error_detail names the code), enqueues nothing but the
 * clearing of the status words, and the call after it starts clean.  So a caller that never
 * calls fa8_check_status still hears of a failed launch, at the latest from the first call made
 * after that launch ended (the reference exits the process, include/attention_api.cuh:20-29).
 * The first call on a device allocates that word (one cudaHostAlloc of four bytes). */
int fa8_fwd(const fa8_fwd_params* params, void* cuda_stream);

/* Reads a status word back after synchronising `cuda_stream`: FA8_OK,
 * FA8_ERR_DEVICE_TIMEOUT (code copied to *code_out if not NULL) or FA8_ERR_CUDA.
 * status_word NULL = the library's own word of the current device, which is cleared once
 * its code has been reported; a caller's word is left for the caller to clear.
 * Replaces the reference's cudaDeviceSynchronize + CUDA_ERROR_CHECK
 * (csrc/flash_attention.cu:663-665). */
int fa8_check_status(const int32_t* status_word, void* cuda_stream, int32_t* code_out);

#define FA8_DTYPE_FP16 0
#define FA8_DTYPE_BF16 1

/* Per-tensor quantisation of `n` contiguous fp16 / bf16 values to e4m3, enqueued on
 * `cuda_stream`: *amax = max |src|, dst = e4m3(src * 448 / amax) (round-to-nearest-even,
 * saturating), *descale = amax / 448 (descale may be NULL).  src and dst 16-byte aligned
 * device memory, amax and descale device floats.  This is the step the reference's callers do
 * with torch before the operator (test.py:12-23, 68-70: cast to float8_e4m3fn); here it is two
 * HBM-bound kernels (5 bytes of traffic per element). */
int fa8_quantize_e4m3(const void* src, int32_t src_dtype, void* dst, int64_t n, float* amax,
                      float* descale, void* cuda_stream);

/* The same for `n_seg` equal contiguous segments of `seg_len` values (a multiple of 8), each
 * with its own scale: amax[s], descale[s] for s < n_seg (<= 65535).  With seg_len = seqlen *
 * head_dim and n_seg = batch * heads this is per-head quantisation of a [batch, heads, seqlen,
 * head_dim] tensor, matching descale_per_head of fa8_fwd_params. */
int fa8_quantize_e4m3_segments(const void* src, int32_t src_dtype, void* dst, int64_t seg_len,
                               int32_t n_seg, float* amax, float* descale, void* cuda_stream);

/* The same per-segment quantisation for callers that cannot allocate (it has no counterpart in the
 * reference, whose callers cast with torch, test.py:20-22).  fa8_quantize_e4m3_segments wants
 * a device buffer for the per-segment maxima even from a caller that only needs the descales.
 * Code that runs where device memory must not be requested - a plug-in inside a framework that has
 * frozen its memory plan, a callback on a serving path whose allocator is off limits, a region
 * that is being captured into a graph, where cudaMalloc is an error - has no such buffer to give.
 * Here the maxima live in a file-scope device array of the library: FA8_NOALLOC_MAX_SEGMENTS
 * floats (16 KB), present on every GPU that loads the library until the process ends.  The call
 * allocates nothing, neither with cudaMalloc nor through any library: it clears the n_seg entries it
 * needs (stream-ordered) and enqueues the two passes on `cuda_stream`; src, dst and descale are the
 * caller's, as before (descale must not be NULL: it is the only way the scales come out).
 *   - n_seg above FA8_NOALLOC_MAX_SEGMENTS is refused with FA8_ERR_UNSUPPORTED (the detail
 *     string names both numbers); seg_len a multiple of 8 unless n_seg is 1.
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress, once
 *     per device, with that device current): make that first call outside any stream capture.
 *   - Every call on a device uses the same array, which keeps the last call's maxima: two calls
 *     that overlap on the GPU (different streams, no ordering between them) race on it.  Calls on
 *     one stream, or ordered by events, are safe. */
#define FA8_NOALLOC_MAX_SEGMENTS 4096
int fa8_quantize_e4m3_segments_noalloc(const void* src, int32_t src_dtype, void* dst, int64_t seg_len,
                                       int32_t n_seg, float* descale, void* cuda_stream);

/* Failure-detection self-test (no counterpart in the reference, whose only error path is
 * exit(), include/attention_api.cuh:20-29): enqueues a one-warp kernel that waits on a barrier
 * nobody completes, using the same bounded wait as the attention kernel.  After `limit_us`
 * microseconds (1..1000000) the wait gives up, the kernel stores 0x7e57 in *status_word and
 * returns; fa8_check_status then reports FA8_ERR_DEVICE_TIMEOUT (and so does the next fa8_fwd
 * on the device, if that comes first) and the CUDA context stays usable.  status_word NULL =
 * the library's own word.  Nothing faults, traps or hangs. */
int fa8_selftest_expired_wait(int32_t* status_word, uint32_t limit_us, void* cuda_stream);

/* Says whether fa8_fwd implements this shape: FA8_OK or FA8_ERR_UNSUPPORTED.  `seqlen_k` is
 * the key/value length (the query length is free).  Replaces the head_dim switch of the
 * reference (csrc/static_switch.h:50-77). */
int fa8_supported(int32_t seqlen_k, int32_t head_dim, int32_t v_layout);

/* How fa8_fwd would cut a problem of `slices` = batch * heads slices into work items on a GPU
 * with `sm_count` SMs (host arithmetic; no GPU needed, nothing is launched).  Replaces the
 * reference's grid calculation, (seqlen / 64, batch * heads) CTAs of one 64-row tile each
 * (csrc/flash_attention.cu:586-610): here the grid is one CTA per SM and a CTA works through
 * items of 256 query rows (two 128-row tiles side by side; one tile at head dims above 128);
 * a causal unit pairs item f with item n-1-f of a slice so that all units cost the same.
 * Problems that would leave more than half of the SMs idle are cut finer: items of 128 rows,
 * or causal items as units of their own.  Results do not depend on the plan.
 * plan[0] = query rows per item, plan[1] = 1 if causal items are paired, plan[2] = items per
 * slice, plan[3] = units (the grid is min(units, sm_count) CTAs).  seqlen_k 0 = seqlen. */
int fa8_work_plan(int32_t slices, int32_t seqlen, int32_t seqlen_k, int32_t head_dim, int32_t is_causal,
                  int32_t sm_count, int32_t plan[4]);

/* Static text for a return code.  Replaces the message printed by CUDA_ERROR_CHECK
 * (include/attention_api.cuh:20-29). */
const char* fa8_error_string(int code);

/* Text of the last CUDA failure seen by the calling thread (empty string if none). */
const char* fa8_last_error_detail(void);

/* ABI version of this header: major*100 + minor (101 added softmax_lse, 102 heads_kv, 103 the
 * descale pointers and fa8_quantize_e4m3, 104 fp8_format, 105 seqlen_k, 106 descale_per_head and
 * fa8_quantize_e4m3_segments, 107 the library-owned status word and host-side failure flag,
 * sequence lengths free of the multiple-of-16 rule except for transposed V, 108
 * fa8_quantize_e4m3_segments_noalloc, 109 fa8_work_plan; new fields go at the end of
 * fa8_fwd_params). */
int fa8_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FA8_B200_H_ */
