/* fa_b200.h — C ABI of the B200 (sm_100a) FlashAttention-forward library `libfa_b200.so`.
 *
 * Plain pointers and sizes only: every pointer is a DEVICE pointer unless its comment says host.
 * No entry point allocates device memory, synchronises the stream, or throws; each returns 0
 * (FA_OK) or one of the FA_ERR_* codes below, and launches on the stream it is given.
 * The library never computes on the CPU: without a usable sm_100 device every compute entry point
 * returns FA_ERR_NO_DEVICE.
 *
 * These entry points sit directly under the torch-op boundary of the reference
 * (`fwd` / `get_scheduler_metadata`, kernels/fa4_blackwell.cu:10187-10205); citations below name the
 * reference function each one replaces.
 */
#ifndef FA_B200_H_
#define FA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* fa_stream_t; /* == cudaStream_t */

enum {
  FA_OK = 0,
  FA_ERR_UNSUPPORTED = 1,   /* configuration outside the supported envelope ("unsupported") */
  FA_ERR_BAD_ARG = 2,       /* inconsistent or missing argument */
  FA_ERR_WORKSPACE = 3,     /* workspace too small */
  FA_ERR_NO_DEVICE = 4,     /* no sm_100 device / driver entry point missing */
  FA_ERR_LAUNCH = 5,        /* a CUDA call failed; see fa_b200_last_cuda_error() */
  FA_ERR_DEVICE_TIMEOUT = 6, /* a bounded device-side wait ran out (read from the status word) */
  FA_ERR_STATIC_LIMIT = 7,   /* problem needs more scratch than the built-in array of fa_b200_decode_fwd_static */
  FA_ERR_BAD_METADATA = 8    /* scheduler_metadata was made for another problem (read from the status word) */
};

/* FA_DT_FP32 is an OUTPUT type only: `out` then receives the normalised result in fp32 (the form a partial
 * result travels in before fa_b200_combine merges it; see fa_b200_combine_strided). */
enum { FA_DT_BF16 = 0, FA_DT_FP16 = 1, FA_DT_FP8_E4M3 = 2, FA_DT_FP32 = 3 };

/* FaFwdParams.flags */
enum {
  /* The caller promises that the first 256 bytes of `workspace` are zero when the call runs on its stream:
   * zeroed once after allocation and since then used only by this library, one call at a time (every
   * successful call leaves them zero again).  The library then issues no memset for them. */
  FA_FLAG_WORKSPACE_CLEAN = 1
};

/* Which kernel family to use. AUTO routes by shape; the others force one family (testing, A/B). */
enum { FA_ROUTE_AUTO = 0, FA_ROUTE_PREFILL_TC = 1, FA_ROUTE_DECODE = 2, FA_ROUTE_GENERAL = 3 };

/* One attention-forward problem. Strides are in ELEMENTS.  K/V rows that a page or a tile holds beyond a
 * sequence's end (the tail of its last page, the next sequence's rows) get weight zero, but they are still
 * multiplied: they must hold finite values (as with the page-granular loads of the reference,
 * kernels/fa4_blackwell.cu:8913-8916). Replaces the argument list of
 * `mha_fwd` (kernels/fa4_blackwell.cu:10081-10094) after tensor unpacking. */
typedef struct FaFwdParams {
  /* ---- tensors ---- */
  const void* q;            /* (total_q, hq, hd) */
  const void* k;            /* non-paged (total_k, hkv, hd); paged (num_pages, page_size, hkv, hd) */
  const void* v;            /* non-paged (total_k, hkv, hdv); paged (num_pages, page_size, hkv, hdv) */
  void* out;                /* (total_q, hq, hdv); element type out_dtype (q's type, bf16 for e4m3 q, or FA_DT_FP32) */
  float* lse;               /* (hq, total_q) fp32, natural log; -inf for rows that see nothing */
  int64_t q_row_stride, q_head_stride;
  int64_t k_row_stride, k_head_stride, k_page_stride; /* row = one token; page stride only when paged */
  int64_t v_row_stride, v_head_stride, v_page_stride;
  int64_t o_row_stride, o_head_stride;
  const int32_t* cu_seqlens_q;  /* (batch+1), required */
  const int32_t* cu_seqlens_k;  /* (batch+1), non-paged */
  const int32_t* seqused_k;     /* (batch), paged (optional override when non-paged) */
  const int32_t* page_table;    /* (batch, page_table_stride) physical page of each logical page, or NULL */
  const int32_t* leftpad_k;     /* (batch) keys with index < leftpad_k[b] are ignored, or NULL */
  const float* q_descale;       /* fp8: (batch, hkv) via the two strides below, or NULL */
  const float* k_descale;
  const float* v_descale;
  const float* s_aux;           /* (hq) fp32 sink logits or NULL */
  const int32_t* scheduler_metadata; /* output of fa_b200_get_scheduler_metadata for this problem, or NULL.
                                      * The kernels compare its header (batch, tiles, splits, route) with the
                                      * call before they index it; a mismatch ends the call without output and
                                      * fa_b200_check_status returns FA_ERR_BAD_METADATA.  Calls that the
                                      * general kernel serves do not read it at all. */
  /* ---- sizes ---- */
  int32_t batch, total_q, total_k, hq, hkv, hd, hdv;
  int32_t max_seqlen_q, max_seqlen_k;      /* upper bounds known on the host (any upper bound is valid: the
                                            * kernels read the true lengths from cu_seqlens / seqused_k) */
  int32_t page_size, num_pages, page_table_stride;
  int32_t descale_batch_stride, descale_head_stride; /* 0,0 broadcasts a scalar */
  int32_t q_dtype, kv_dtype, out_dtype;    /* FA_DT_* */
  /* ---- semantics ---- */
  float softmax_scale;
  float softcap;                           /* 0 = off */
  int32_t is_causal;                       /* bottom-right aligned: qpos = seqlen_k - seqlen_q + row */
  int32_t window_left, window_right;       /* -1 = unbounded */
  /* ---- scheduling ---- */
  int32_t num_splits;                      /* 0 = heuristic, 1 = never split, >1 = at most that many */
  int32_t sm_margin;                       /* SMs to leave free */
  int32_t route;                           /* FA_ROUTE_* */
  int32_t scheduler_metadata_len;          /* int32 words behind scheduler_metadata (0 = not stated); a length
                                            * that differs from fa_b200_scheduler_metadata_len of this problem
                                            * is refused on the host with FA_ERR_BAD_METADATA */
  int32_t flags;                           /* FA_FLAG_* */
} FaFwdParams;

/* Bytes of scratch fa_b200_fwd needs for `p` (split partials, work list, status word). Host-only
 * arithmetic. The caller allocates it (256-byte aligned) and may reuse it across calls on one stream.
 * Replaces the per-call `at::empty` scratch of `launch_ws_paged` (kernels/fa4_blackwell.cu:9737-9738). */
size_t fa_b200_fwd_workspace_bytes(const FaFwdParams* p);

/* Attention forward. Replaces `mha_fwd`'s routing and launches (kernels/fa4_blackwell.cu:10138-10169:
 * launch_ws / launch_paged_maybe_split / launch, and combine_kernel 5964-5985 after a split launch). */
int fa_b200_fwd(const FaFwdParams* p, void* workspace, size_t workspace_bytes, fa_stream_t stream);

/* The split count fa_b200_fwd will use for `p` (>= 1). Host-only arithmetic; restates the role of the
 * split heuristic in `launch_ws_paged` (kernels/fa4_blackwell.cu:9721-9735). */
int fa_b200_num_splits(const FaFwdParams* p);

/* Scheduler metadata. Replaces `mha_fwd_get_scheduler_metadata` (kernels/fa4_blackwell.cu:10175-10183,
 * a stub there). The arguments mirror that op's. */
typedef struct FaSchedParams {
  const int32_t* seqused_k;     /* (batch) or NULL */
  const int32_t* cu_seqlens_q;  /* (batch+1) or NULL => every sequence has max_seqlen_q rows */
  const int32_t* cu_seqlens_k;  /* (batch+1) or NULL */
  const int32_t* leftpad_k;     /* (batch) or NULL */
  int32_t batch, max_seqlen_q, max_seqlen_k, hq, hkv, hd, hdv;
  int32_t qkv_dtype;            /* FA_DT_* */
  int32_t page_size;            /* 0 = not paged */
  int32_t is_causal, window_left, window_right, has_softcap;
  int32_t num_splits, sm_margin;
} FaSchedParams;

/* Number of int32 words of the metadata tensor for `p` (host arithmetic). */
int fa_b200_scheduler_metadata_len(const FaSchedParams* p);
/* Fills `out_dev` (device, fa_b200_scheduler_metadata_len words) on `stream`. */
int fa_b200_get_scheduler_metadata(const FaSchedParams* p, int32_t* out_dev, fa_stream_t stream);

/* LSE-weighted merge of `nsplits` partial results; also the merge step of the multi-GPU KV-range
 * sharding. Replaces `combine_kernel` (kernels/fa4_blackwell.cu:5964-5985).
 *   o_part   (nsplits, total_q, hq, hdv) fp32, each split normalised by its own denominator
 *   lse_part (nsplits, hq, total_q)      fp32 natural log, -inf for a split that saw no key
 *   s_aux    (hq) fp32 sink logits or NULL (the sink joins exactly once, here)
 *   out      (total_q, hq, hdv) with the given strides, out_dtype FA_DT_BF16/FP16
 *   lse      (hq, total_q) fp32 */
int fa_b200_combine(const float* o_part, const float* lse_part, int32_t nsplits, int32_t total_q,
                    int32_t hq, int32_t hdv, const float* s_aux, void* out, int64_t o_row_stride,
                    int64_t o_head_stride, int32_t out_dtype, float* lse, fa_stream_t stream);

/* The same merge reading the partials where a gather left them: split s begins `o_split_stride` /
 * `lse_split_stride` floats after split s-1 (a packed per-rank buffer [O_r | LSE_r] gathered from N ranks has
 * both strides equal to the buffer length).  No counterpart in the reference (single GPU). */
int fa_b200_combine_strided(const float* o_part, const float* lse_part, int64_t o_split_stride,
                            int64_t lse_split_stride, int32_t nsplits, int32_t total_q, int32_t hq, int32_t hdv,
                            const float* s_aux, void* out, int64_t o_row_stride, int64_t o_head_stride,
                            int32_t out_dtype, float* lse, fa_stream_t stream);

/* Appends the new keys / values of this step to a paged cache, in place, and applies the rotary position embedding to
 * them and to the queries: the step in front of the attention call when the op is given `k_new` / `v_new` /
 * `rotary_cos` / `rotary_sin`.  Those arguments exist in the op's schema (kernels/fa4_blackwell.cu:10188-10196), but the
 * reference pins them to None (bench/scenarios.py:915-921) and has no kernel for them; the behaviour here is the op's
 * documented one: new key i of sequence b lands at key index seqused_k[b] + i and is rotated at position r_b + i,
 * r_b = seqlens_rotary[b] if given else seqused_k[b]; query i is rotated at r_b + i when q_positions_advance is set
 * (causal or windowed attention) and at r_b otherwise; `rotary_interleaved` pairs dimensions (2j, 2j+1), else
 * (j, j + rotary_dim/2); dimensions >= rotary_dim pass through.  All arithmetic is fp32 with separately rounded
 * products and sums, results rounded to the element type.  Strides in ELEMENTS. */
typedef struct FaAppendParams {
  const void* k_new;             /* (total_new, hkv, hd), element type kv_dtype */
  const void* v_new;             /* (total_new, hkv, hdv) */
  void* k_cache;                 /* (num_pages, page_size, hkv, hd), written in place */
  void* v_cache;                 /* (num_pages, page_size, hkv, hdv) */
  const void* q;                 /* (total_q, hq, hd), element type q_dtype; read only when a rotary table is given */
  void* q_out;                   /* (total_q, hq, hd) rotated copy of q (must not alias q); NULL without rotary */
  const void* rotary_cos;        /* (seqlen_ro, rotary_dim/2) of q_dtype, or NULL: no rotation */
  const void* rotary_sin;
  const int32_t* cu_seqlens_k_new; /* (batch+1) */
  const int32_t* cu_seqlens_q;     /* (batch+1); needed with rotary */
  const int32_t* seqused_k;        /* (batch) keys in the cache before the call */
  int32_t* seqused_k_out;          /* (batch) keys after it: seqused_k + new keys (must not alias seqused_k) */
  const int32_t* page_table;       /* (batch, page_table_stride) */
  const int32_t* seqlens_rotary;   /* (batch) or NULL */
  int64_t kn_row_stride, kn_head_stride, vn_row_stride, vn_head_stride;
  int64_t k_row_stride, k_head_stride, k_page_stride, v_row_stride, v_head_stride, v_page_stride;
  int64_t q_row_stride, q_head_stride, qo_row_stride, qo_head_stride;
  int32_t batch, total_new, total_q, hq, hkv, hd, hdv;
  int32_t page_size, page_table_stride;
  int32_t rotary_dim;              /* multiple of 16, <= hd */
  int32_t rotary_interleaved, q_positions_advance;
  int32_t q_dtype, kv_dtype;       /* FA_DT_*; rotary needs 16-bit q and k_new of the same type; an e4m3 cache takes
                                    * e4m3 k_new / v_new without rotation of the keys */
} FaAppendParams;
int fa_b200_append_kv(const FaAppendParams* p, fa_stream_t stream);
size_t fa_b200_sizeof_append_params(void);

/* Reads the device status word of a workspace after synchronising `stream` (the only entry point that
 * synchronises). Returns FA_OK, FA_ERR_DEVICE_TIMEOUT with *detail = (role<<24 | block) of the first
 * wait that gave up, or FA_ERR_BAD_METADATA when a kernel refused the scheduler metadata. The reference has
 * no counterpart: its device waits are unbounded (kernels/fa4_blackwell.cu:5732). */
int fa_b200_check_status(void* workspace, fa_stream_t stream, uint32_t* detail /* host, may be NULL */);

/* Self-test of the bounded-wait machinery: launches ONE thread block that waits, with the same wait routine
 * the attention kernels use, on a barrier nobody ever arrives at, for at most `max_cycles` SM clock cycles
 * (clamped to [1e4, 1e8]).  The wait gives up, records the time-out in the status word at the start of
 * `workspace` (>= 256 bytes, zeroed on `stream` by this call) and the kernel returns by itself; nothing is in
 * flight and nothing faults.  fa_b200_check_status then reports FA_ERR_DEVICE_TIMEOUT.  No counterpart in the
 * reference. */
int fa_b200_selftest_timeout(void* workspace, int64_t max_cycles, fa_stream_t stream);

/* Paged decode without any allocation, for callers that cannot obtain device memory at call time: an
 * inference worker that handed every free byte of HBM to its KV-cache pool at start-up (a later cudaMalloc
 * fails, or stalls the device while the driver looks for room), or a host written in another language that
 * holds no device allocator at all.  It is fa_b200_fwd restricted to the decode route, with the scratch
 * (status word, work counter, work list, split partials) living in an array compiled into this library
 * instead of a caller-supplied workspace.  The caller still passes inputs and outputs in `p`.
 *   - The array is FA_B200_STATIC_SCRATCH_BYTES (8 MiB) per GPU, held by every GPU that loads the library
 *     until the process exits.  A problem whose scratch (fa_b200_fwd_workspace_bytes) exceeds it returns
 *     FA_ERR_STATIC_LIMIT; a shape the decode route does not take returns FA_ERR_UNSUPPORTED.
 *   - The first call on each device looks the array's device address up (with that device current); make that
 *     first call before any stream capture begins.
 *   - All calls on one GPU share the array and find the previous call's contents in it; the words that must
 *     start at zero are cleared on `stream` at every call.  Two calls that overlap on the GPU (different
 *     streams, no ordering between them) race on it: order them.
 *   - fa_b200_check_status does not apply (there is no workspace pointer to hand it).
 * Has no counterpart in the reference, which allocates its scratch with at::empty on every call. */
#define FA_B200_STATIC_SCRATCH_BYTES (8u << 20)
int fa_b200_decode_fwd_static(const FaFwdParams* p, fa_stream_t stream);

const char* fa_b200_strerror(int code);      /* host string */
const char* fa_b200_last_cuda_error(void);   /* host string of the last failed CUDA call on this thread */
int fa_b200_version(void);
/* sizeof(FaFwdParams) / sizeof(FaSchedParams) as this library was compiled: lets a foreign-function
 * binding verify its own struct layout before the first call. No counterpart in the reference. */
size_t fa_b200_sizeof_fwd_params(void);
size_t fa_b200_sizeof_sched_params(void);

#ifdef __cplusplus
}
#endif
#endif /* FA_B200_H_ */
