// fa_internal.h — structures shared by the host planner and the kernels (not part of the C ABI).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fa_b200.h"
#include "fa_sched.h"

namespace fa {

struct DeviceStatus;

// Kernel-side view of one problem: FaFwdParams plus what the planner derived.
struct KParams {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  float* lse;
  float* o_part;      // (nsplits, total_q, hq, hdv) fp32 when nsplits > 1
  float* lse_part;    // (nsplits, hq, total_q) fp32 when nsplits > 1
  const int32_t* cu_q;
  const int32_t* cu_k;
  const int32_t* seqused_k;
  const int32_t* page_table;
  const int32_t* leftpad_k;
  const float* q_descale;
  const float* k_descale;
  const float* v_descale;
  const float* s_aux;
  const int32_t* work;      // scheduler metadata / work list (layout in fa_sched.h), or null
  SchedExpect work_expect;  // header values `work` must carry
  int32_t* counters;        // zero at kernel start: [0] = persistent work counter, [1] = CTAs that have finished;
                            // the last CTA to finish sets both back to zero
  DeviceStatus* status;
  int64_t q_row_stride, q_head_stride;
  int64_t k_row_stride, k_head_stride, k_page_stride;
  int64_t v_row_stride, v_head_stride, v_page_stride;
  int64_t o_row_stride, o_head_stride;
  int32_t batch, total_q, total_k, num_pages, hq, hkv, rep, hd, hdv;
  int32_t max_seqlen_q, max_seqlen_k;
  int32_t page_size, page_shift /* log2(page_size) or -1 */, page_table_stride;
  int32_t descale_batch_stride, descale_head_stride;
  int32_t q_fp8, kv_fp8;
  int32_t is_causal, window_left, window_right;
  int32_t nsplits;
  int32_t out_f32;     // `out` is fp32 (FA_DT_FP32) instead of the 16-bit type of the kernel
  float scale;         // softmax_scale
  float softcap;       // 0 = off
};

// ------------------------------------------------------------------------------------------
// Index arithmetic shared by every kernel and restated on the CPU in oracle/sched_oracle.py.
// ------------------------------------------------------------------------------------------

// Key-block range [lo, hi) a tile of query positions [qp_min, qp_max] has to visit, in blocks of `tn`
// keys, given the sequence's key count, its leftpad, causal flag and window.
__host__ __device__ inline void nblock_range(int seqlen_k, int leftpad, int qp_min, int qp_max, int is_causal,
                                             int win_l, int win_r, int tn, int* lo, int* hi) {
  int nblocks = (seqlen_k + tn - 1) / tn;
  int n_lo = 0, n_hi = nblocks;
  if (is_causal) n_hi = min(n_hi, max(qp_max, -1) / tn + (qp_max >= 0 ? 1 : 0));
  if (win_r >= 0) {
    int last = qp_max + win_r;
    n_hi = min(n_hi, last >= 0 ? last / tn + 1 : 0);
  }
  if (win_l >= 0) {
    int first = qp_min - win_l;
    if (first > 0) n_lo = first / tn;
  }
  if (leftpad > 0) n_lo = max(n_lo, leftpad / tn);
  if (n_lo > n_hi) n_lo = n_hi;
  *lo = n_lo;
  *hi = n_hi;
}

// Sub-range of [lo, hi) owned by split `s` of `nsplits`: contiguous chunks of ceil(total / nsplits).
__host__ __device__ inline void split_range(int lo, int hi, int s, int nsplits, int* slo, int* shi) {
  int tot = hi - lo;
  int per = (tot + nsplits - 1) / nsplits;
  int a = lo + s * per, b = lo + (s + 1) * per;
  *slo = a < hi ? a : hi;
  *shi = b < hi ? b : hi;
}

// launchers (each returns a cudaError_t-compatible int; 0 = success)
int launch_general(const KParams& kp, int dtype /*FA_DT_BF16|FP16 compute type*/, int out_dtype, int num_sms,
                   cudaStream_t stream);
int launch_combine(const float* o_part, const float* lse_part, int nsplits, int total_q, int hq, int hdv,
                   const float* s_aux, void* out, int64_t o_row_stride, int64_t o_head_stride, int out_dtype,
                   float* lse, cudaStream_t stream);

}  // namespace fa
