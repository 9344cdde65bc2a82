// fa_capi.cu — the C ABI (include/fa_b200.h): validation, planning, workspace carving, routing.
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "fa_internal.h"
#include "fa_sched.h"
#include "ptx.cuh"

namespace fa {

int launch_sched(const FaSchedParams& sp, const Plan& pl, int32_t* out_dev, int32_t* zero_words, cudaStream_t stream,
                 int row_class = 0, int class_rows = 0);
int launch_selftest_timeout(DeviceStatus* status, long long max_cycles, cudaStream_t stream);
int launch_append_kv(const FaAppendParams& p, int num_sms, cudaStream_t stream);
int launch_depage(const KParams& kp, int kpad, void* k_out, void* v_out, int32_t* cu_out, int num_sms, cudaStream_t stream);
int launch_combine_strided(const float* o_part, const float* lse_part, int64_t o_split_stride, int64_t lse_split_stride,
                           int nsplits, int total_q, int hq, int hdv, const float* s_aux, void* out,
                           int64_t o_row_stride, int64_t o_head_stride, int out_dtype, float* lse, cudaStream_t stream);
int launch_decode(const KParams& kp, const Plan& pl, int compute_dtype, cudaStream_t stream);
int launch_prefill_tc(const KParams& kp, const Plan& pl, int compute_dtype, cudaStream_t stream);
bool prefill_tc_supported(const PlanInput& in);
bool prefill_tc_single_tile(int hd, int hdv);
bool decode_supported(const PlanInput& in);
bool prefill_tc_layout_ok(const FaFwdParams* p);

static thread_local char g_last_cuda_error[256] = "";

static int cuda_fail(cudaError_t e, const char* what) {
  snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "%s: %s", what, cudaGetErrorString(e));
  return FA_ERR_LAUNCH;
}
int note_cuda_error(int e, const char* what) {   // used by launchers that return raw cudaError_t values
  if (e == 0) return FA_OK;
  if (e < 0) { snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "%s: no kernel instance", what); return FA_ERR_UNSUPPORTED; }
  return cuda_fail((cudaError_t)e, what);
}

// ---- per-device facts, queried once ----
struct DevInfo { int ok; int sms; int cc_major; };
static DevInfo g_dev[64];
static std::atomic<int> g_dev_init[64];
static std::mutex g_dev_mu;

static const DevInfo* device_info() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (g_dev_init[dev].load(std::memory_order_acquire) == 0) {
    std::lock_guard<std::mutex> lk(g_dev_mu);
    if (g_dev_init[dev].load(std::memory_order_relaxed) == 0) {
      DevInfo d{0, 0, 0};
      cudaDeviceProp prop;
      if (cudaGetDeviceProperties(&prop, dev) == cudaSuccess) {
        d.sms = prop.multiProcessorCount;
        d.cc_major = prop.major;
        d.ok = (prop.major == 10);
      }
      g_dev[dev] = d;
      g_dev_init[dev].store(1, std::memory_order_release);
    }
  }
  return &g_dev[dev];
}

static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Windows that cannot mask anything are dropped (kernels/fa4_blackwell.cu:10148-10153): under causal any
// right window is implied; a left window of at least max_seqlen_k - 1 keys never cuts.
static void normalize_window(int is_causal, int max_seqlen_k, int* wl, int* wr) {
  if (is_causal && *wr >= 0) *wr = -1;
  if (*wl >= 0 && max_seqlen_k > 0 && *wl >= max_seqlen_k - 1) *wl = -1;
  if (*wr >= 0 && max_seqlen_k > 0 && *wr >= max_seqlen_k - 1) *wr = -1;
}

// ------------------------------------------------------------------------------------------------
// plan: route, tile geometry, split count.  Pure host arithmetic on shape facts, so that
// get_scheduler_metadata and fwd agree.  Restated in oracle/sched_oracle.py.
// ------------------------------------------------------------------------------------------------
Plan make_plan(const PlanInput& in) {
  Plan pl{};
  pl.err = FA_OK;
  pl.num_sms = in.num_sms_device - (in.sm_margin > 0 ? in.sm_margin : 0);
  if (pl.num_sms < 1) pl.num_sms = 1;
  if (in.hkv <= 0 || in.hq % in.hkv != 0 || in.batch < 0 || in.hd <= 0 || in.hdv <= 0 || in.max_seqlen_q <= 0) {
    pl.err = FA_ERR_BAD_ARG;
    return pl;
  }
  const int rep = in.hq / in.hkv;
  int route = in.route;
  const bool tc_ok = prefill_tc_supported(in) && in.tc_layout_ok, dec_ok = decode_supported(in);
  if (route == FA_ROUTE_AUTO) {
    if (dec_ok && in.max_seqlen_q * rep <= kDecodeMaxRows) route = FA_ROUTE_DECODE;
    else if (tc_ok) route = FA_ROUTE_PREFILL_TC;
    else route = FA_ROUTE_GENERAL;
  }
  if ((route == FA_ROUTE_PREFILL_TC && !tc_ok) || (route == FA_ROUTE_DECODE && !(dec_ok && in.max_seqlen_q * rep <= kDecodeMaxRows))) {
    pl.err = FA_ERR_UNSUPPORTED;
    return pl;
  }
  pl.route = route;
  if (route == FA_ROUTE_PREFILL_TC) {
    pl.tile_m = prefill_tc_single_tile(in.hd, in.hdv) ? 128 : 256; pl.tile_n = 128; pl.rows_per_token = 1;
  } else if (route == FA_ROUTE_DECODE) {
    pl.tile_m = 16; pl.tile_n = 64; pl.rows_per_token = rep;
  } else {
    if (in.hd > 256 || in.hdv > 256 || in.hd % 8 != 0 || in.hdv % 8 != 0) { pl.err = FA_ERR_UNSUPPORTED; return pl; }
    pl.tile_m = 64; pl.tile_n = 64; pl.rows_per_token = rep;
  }
  pl.max_mtiles = ceil_div(in.max_seqlen_q * pl.rows_per_token, pl.tile_m);

  // split count
  const int max_nb = in.max_seqlen_k > 0 ? ceil_div(in.max_seqlen_k, pl.tile_n) : 1;
  const long heads = pl.rows_per_token > 1 ? in.hkv : in.hq;
  const long ctas = (long)in.batch * heads * pl.max_mtiles;
  int s = 1;
  if (route == FA_ROUTE_PREFILL_TC || in.num_splits == 1) {   // the tensor-core prefill route never splits
    s = 1;
  } else if (in.num_splits > 1) {
    s = in.num_splits < max_nb ? in.num_splits : max_nb;
  } else if (route != FA_ROUTE_PREFILL_TC && ctas > 0 && ctas * 2 <= pl.num_sms && max_nb >= 8) {
    long want = pl.num_sms / ctas;
    long cap = max_nb / 4;
    s = (int)(want < cap ? want : cap);
    if (s > 64) s = 64;
  }
  if (s < 1) s = 1;
  pl.nsplits = s;
  return pl;
}

static PlanInput plan_input(const FaFwdParams* p, int num_sms) {
  PlanInput in{};
  in.batch = p->batch; in.max_seqlen_q = p->max_seqlen_q; in.max_seqlen_k = p->max_seqlen_k;
  in.hq = p->hq; in.hkv = p->hkv; in.hd = p->hd; in.hdv = p->hdv;
  in.q_dtype = p->q_dtype; in.kv_dtype = p->kv_dtype;
  in.page_size = p->page_table ? p->page_size : 0;
  in.is_causal = p->is_causal; in.window_left = p->window_left; in.window_right = p->window_right;
  normalize_window(in.is_causal, in.max_seqlen_k, &in.window_left, &in.window_right);
  in.has_softcap = p->softcap > 0.f;
  in.num_splits = p->out_dtype == FA_DT_FP32 ? 1 : p->num_splits;   // fp32 output is itself the partial form
  in.sm_margin = p->sm_margin; in.route = p->route;
  in.num_sms_device = num_sms;
  in.tc_layout_ok = prefill_tc_layout_ok(p) ? 1 : 0;
  return in;
}
static PlanInput plan_input(const FaSchedParams* p, int num_sms) {
  PlanInput in{};
  in.batch = p->batch; in.max_seqlen_q = p->max_seqlen_q; in.max_seqlen_k = p->max_seqlen_k;
  in.hq = p->hq; in.hkv = p->hkv; in.hd = p->hd; in.hdv = p->hdv;
  in.q_dtype = p->qkv_dtype; in.kv_dtype = p->qkv_dtype;
  in.page_size = p->page_size;
  in.is_causal = p->is_causal; in.window_left = p->window_left; in.window_right = p->window_right;
  normalize_window(in.is_causal, in.max_seqlen_k, &in.window_left, &in.window_right);
  in.has_softcap = p->has_softcap;
  in.num_splits = p->num_splits; in.sm_margin = p->sm_margin; in.route = FA_ROUTE_AUTO;
  in.num_sms_device = num_sms;
  in.tc_layout_ok = 1;
  return in;
}

// A batch that mixes decode-shaped sequences (a few query rows) with prefill-shaped ones: when both kernels take the
// shape and the sequences are ragged enough (the mean query length is under a quarter of the maximum), one call runs
// BOTH kernels, each over its own work list (the reference splits such a batch into two launches as well,
// kernels/fa4_blackwell.cu:9995-10021).  Decided from host-side facts only; a list for either kernel may turn out empty.
static bool mixed_batch(const FaFwdParams* p, const PlanInput& in, const Plan& pl) {
  if (p->route != FA_ROUTE_AUTO || pl.route != FA_ROUTE_PREFILL_TC || p->scheduler_metadata != nullptr) return false;
  if (p->batch < 2 || !decode_supported(in) || p->out_dtype == FA_DT_FP32) return false;
  return (long long)p->total_q * 4 < (long long)p->batch * p->max_seqlen_q;
}
static Plan decode_part_plan(const PlanInput& in, const Plan& pl) {
  Plan d = pl;
  d.route = FA_ROUTE_DECODE;
  d.tile_m = 16; d.tile_n = 64; d.rows_per_token = in.hq / in.hkv;
  d.max_mtiles = kDecodeMaxRows / 16;
  d.nsplits = 1;
  return d;
}

// De-paging.  A prefill over pages of 1 .. 16 keys pays for its small copies in every query tile that reads a key
// block (the tensor-core kernel runs at 500 - 900 TFLOP/s there against ~1150 over contiguous keys).  Where the keys
// are read often enough - ceil(max_seqlen_q / 256) x (q heads per kv head) tiles per block, at least 4 - and the
// batch's keys fit a bounded scratch, one pass copies every sequence's K and V rows out of the pages into contiguous
// slabs of `kpad` rows in the workspace and the kernel runs on those with its contiguous-K/V producer (the
// reference's route for page sizes its paged kernel has no producer for, kernels/fa4_blackwell.cu:9352-9378,
// 9638-9679).  Decided from host-side facts only.
constexpr size_t kDepageMaxBytes = (size_t)256 << 20;
static bool depage_plan(const FaFwdParams* p, const Plan& pl, int* kpad, size_t* k_bytes, size_t* v_bytes) {
  if (pl.route != FA_ROUTE_PREFILL_TC || !p->page_table) return false;
  const int ps = p->page_size;
  if (!(ps == 1 || ps == 2 || ps == 4 || ps == 8 || ps == 16)) return false;
  if ((long long)ceil_div(p->max_seqlen_q, 256) * (p->hq / p->hkv) < 4) return false;
  const size_t esz = p->kv_dtype == FA_DT_FP8_E4M3 ? 1 : 2;
  const size_t rows = (size_t)p->batch * (size_t)((p->max_seqlen_k + 127) / 128 * 128);
  const size_t kb = rows * p->hkv * p->hd * esz, vb = rows * p->hkv * p->hdv * esz;
  if (kb + vb > kDepageMaxBytes) return false;
  *kpad = (p->max_seqlen_k + 127) / 128 * 128;
  *k_bytes = align_up(kb, 256);
  *v_bytes = align_up(vb, 256);
  return true;
}

// ---- workspace layout ----
struct WsLayout {
  size_t header;      // DeviceStatus @0, counters @64
  size_t dp_cu_off, dp_k_off, dp_v_off, dp_k_bytes;   // de-paged K/V slabs and their row offsets (dp_k_bytes 0: none)
  int dp_kpad;
  size_t work_off, work_bytes;
  size_t work2_off, work2_bytes;   // mixed batches: the prefill kernel's list
  size_t lse_off, lse_bytes;
  size_t o_off, o_bytes;
  size_t total;
};
static WsLayout ws_layout(const FaFwdParams* p, const Plan& pl) {
  WsLayout w{};
  w.header = 256;
  size_t off = w.header;
  w.work_off = off;
  w.work_bytes = (pl.route == FA_ROUTE_DECODE && p->scheduler_metadata == nullptr)
                     ? align_up((size_t)sched_len(pl, p->batch) * 4, 256) : 0;
  off += w.work_bytes;
  if (pl.route == FA_ROUTE_PREFILL_TC && p->scheduler_metadata == nullptr && p->batch >= 2) {
    // room for the two lists of a mixed batch (whether the call is one is decided from the same facts in fa_b200_fwd)
    const PlanInput in = plan_input(p, pl.num_sms);
    if (mixed_batch(p, in, pl)) {
      w.work_off = off;
      w.work_bytes = align_up((size_t)sched_len(decode_part_plan(in, pl), p->batch) * 4, 256);
      off += w.work_bytes;
      w.work2_off = off;
      w.work2_bytes = align_up((size_t)sched_len(pl, p->batch) * 4, 256);
      off += w.work2_bytes;
    }
  }
  if (w.work2_bytes == 0) {
    size_t kb = 0, vb = 0;
    int kpad = 0;
    if (depage_plan(p, pl, &kpad, &kb, &vb)) {
      w.dp_kpad = kpad;
      w.dp_cu_off = off;
      off += align_up((size_t)(p->batch + 1) * 4, 256);
      w.dp_k_off = off;
      w.dp_k_bytes = kb;
      off += kb;
      w.dp_v_off = off;
      off += vb;
    }
  }
  if (pl.nsplits > 1) {
    w.lse_off = off;
    w.lse_bytes = align_up((size_t)pl.nsplits * p->hq * p->total_q * 4, 256);
    off += w.lse_bytes;
    w.o_off = off;
    w.o_bytes = align_up((size_t)pl.nsplits * p->total_q * p->hq * p->hdv * 4, 256);
    off += w.o_bytes;
  }
  w.total = off;
  return w;
}

static int validate(const FaFwdParams* p) {
  if (!p || !p->cu_seqlens_q) return FA_ERR_BAD_ARG;
  // tensors without elements have no address: queries are needed only if there is a query row, keys only if a
  // contiguous K/V holds a key
  if (p->total_q > 0 && (!p->q || !p->out || !p->lse)) return FA_ERR_BAD_ARG;
  if ((p->page_table || p->total_k > 0) && (!p->k || !p->v)) return FA_ERR_BAD_ARG;
  if (p->page_table) {
    if (!p->seqused_k || p->page_size <= 0) return FA_ERR_BAD_ARG;
  } else if (!p->cu_seqlens_k) {
    return FA_ERR_BAD_ARG;
  }
  if (p->batch < 0 || p->total_q < 0 || p->hq <= 0 || p->hkv <= 0 || p->hq % p->hkv) return FA_ERR_BAD_ARG;
  if (p->max_seqlen_q <= 0 && p->total_q > 0) return FA_ERR_BAD_ARG;
  const bool q8 = p->q_dtype == FA_DT_FP8_E4M3, kv8 = p->kv_dtype == FA_DT_FP8_E4M3;
  if (p->q_dtype < 0 || p->q_dtype > 2 || p->kv_dtype < 0 || p->kv_dtype > 2) return FA_ERR_BAD_ARG;
  if (!kv8 && p->kv_dtype != p->q_dtype) return FA_ERR_UNSUPPORTED;          // bf16 Q with fp16 KV etc.
  if (p->out_dtype != FA_DT_FP32 && p->out_dtype != (q8 ? FA_DT_BF16 : p->q_dtype)) return FA_ERR_UNSUPPORTED;
  if (p->hd % 8 || p->hdv % 8) return FA_ERR_UNSUPPORTED;
  const int64_t strides[] = {p->q_row_stride, p->q_head_stride, p->k_row_stride, p->k_head_stride,
                             p->v_row_stride, p->v_head_stride, p->o_row_stride, p->o_head_stride,
                             p->page_table ? p->k_page_stride : 0, p->page_table ? p->v_page_stride : 0};
  for (int64_t s : strides) if (s % 8) return FA_ERR_UNSUPPORTED;
  const uintptr_t ptrs[] = {(uintptr_t)p->q, (uintptr_t)p->k, (uintptr_t)p->v, (uintptr_t)p->out};
  for (uintptr_t a : ptrs) if (a % 16) return FA_ERR_UNSUPPORTED;
  return FA_OK;
}

// The call as the kernels get it: unchanged, or (a contiguous K/V without a single key) re-addressed for the
// general kernel, see fa_b200_fwd.
static const FaFwdParams* without_keys(const FaFwdParams* p, FaFwdParams* tmp) {
  if (p->page_table || p->total_k != 0 || p->total_q <= 0 || !p->q) return p;
  *tmp = *p;
  tmp->k = tmp->v = p->q;
  tmp->route = FA_ROUTE_GENERAL;
  tmp->num_splits = 1;
  tmp->scheduler_metadata = nullptr;
  return tmp;
}

}  // namespace fa

using namespace fa;

extern "C" {

int fa_b200_version(void) { return 1; }
size_t fa_b200_sizeof_fwd_params(void) { return sizeof(FaFwdParams); }
size_t fa_b200_sizeof_sched_params(void) { return sizeof(FaSchedParams); }

const char* fa_b200_strerror(int code) {
  switch (code) {
    case FA_OK: return "ok";
    case FA_ERR_UNSUPPORTED: return "unsupported configuration";
    case FA_ERR_BAD_ARG: return "bad argument";
    case FA_ERR_WORKSPACE: return "workspace too small";
    case FA_ERR_NO_DEVICE: return "no sm_100 CUDA device";
    case FA_ERR_LAUNCH: return "CUDA call failed";
    case FA_ERR_DEVICE_TIMEOUT: return "a device-side wait timed out";
    case FA_ERR_STATIC_LIMIT: return "problem needs more scratch than the 8 MiB built into fa_b200_decode_fwd_static";
    case FA_ERR_BAD_METADATA: return "scheduler_metadata does not belong to this problem (length or header mismatch)";
    default: return "unknown error";
  }
}
const char* fa_b200_last_cuda_error(void) { return g_last_cuda_error; }

size_t fa_b200_fwd_workspace_bytes(const FaFwdParams* p_in) {
  if (!p_in) return 0;
  FaFwdParams no_keys;
  const FaFwdParams* p = without_keys(p_in, &no_keys);
  const DevInfo* di = device_info();
  Plan pl = make_plan(plan_input(p, di && di->sms > 0 ? di->sms : 148));
  if (pl.err != FA_OK) return 256;
  return ws_layout(p, pl).total;
}

int fa_b200_num_splits(const FaFwdParams* p) {
  if (!p) return 1;
  const DevInfo* di = device_info();
  Plan pl = make_plan(plan_input(p, di && di->sms > 0 ? di->sms : 148));
  return pl.err == FA_OK ? pl.nsplits : 1;
}

int fa_b200_fwd(const FaFwdParams* p_in, void* workspace, size_t workspace_bytes, fa_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  int rc = validate(p_in);
  if (rc != FA_OK) return rc;
  // A contiguous K/V without a single key: every row sees nothing (zeros, LSE of the sink alone or -inf).  The
  // general kernel writes that without touching K or V; it is given the query tensor as a stand-in address.
  if (p_in->total_q == 0 || p_in->batch == 0) {
    // no query row: nothing to write, but fa_b200_check_status must find a clean status word afterwards
    if (workspace && workspace_bytes >= 256 && !(p_in->flags & FA_FLAG_WORKSPACE_CLEAN)) {
      cudaError_t ce = cudaMemsetAsync(workspace, 0, 256, stream);
      if (ce != cudaSuccess) return cuda_fail(ce, "cudaMemsetAsync(workspace header)");
    }
    return FA_OK;
  }
  FaFwdParams no_keys;
  const FaFwdParams* p = without_keys(p_in, &no_keys);
  const DevInfo* di = device_info();
  if (!di || !di->ok) return FA_ERR_NO_DEVICE;
  PlanInput in = plan_input(p, di->sms);
  Plan pl = make_plan(in);
  if (pl.err != FA_OK) return pl.err;
  WsLayout w = ws_layout(p, pl);
  if (!workspace || workspace_bytes < w.total || ((uintptr_t)workspace % 256)) return FA_ERR_WORKSPACE;
  if (p->total_q == 0 || p->batch == 0) return FA_OK;

  // Only the decode and the tensor-core prefill kernels read the metadata; the general kernel has no use for it, and
  // a list made for one of the other two (the metadata call knows a single element type: 16-bit queries over an
  // e4m3 cache with many rows are planned there as a tensor-core prefill, here as the general route) is then left
  // unread rather than refused.
  const bool md_read = pl.route == FA_ROUTE_DECODE || pl.route == FA_ROUTE_PREFILL_TC;
  if (md_read && p->scheduler_metadata && p->scheduler_metadata_len > 0 &&
      p->scheduler_metadata_len != sched_len(pl, p->batch))
    return FA_ERR_BAD_METADATA;

  char* ws = (char*)workspace;
  // The header (status word, work counters) must be zero when the kernels start.  A caller that keeps it clean
  // (FA_FLAG_WORKSPACE_CLEAN) saves the memset: the kernels leave the counters at zero when they finish.
  const bool clean = (p->flags & FA_FLAG_WORKSPACE_CLEAN) != 0;
  // (on the decode route without caller metadata the work-list kernel runs first and clears the header itself)
  const bool sched_first = pl.route == FA_ROUTE_DECODE && p->scheduler_metadata == nullptr;
  if (!clean && !sched_first) {
    cudaError_t ce = cudaMemsetAsync(ws, 0, w.header, stream);
    if (ce != cudaSuccess) return cuda_fail(ce, "cudaMemsetAsync(workspace header)");
  }

  KParams kp{};
  kp.q = p->q; kp.k = p->k; kp.v = p->v; kp.out = p->out; kp.lse = p->lse;
  kp.cu_q = p->cu_seqlens_q; kp.cu_k = p->cu_seqlens_k; kp.seqused_k = p->seqused_k;
  kp.page_table = p->page_table; kp.leftpad_k = p->leftpad_k;
  kp.q_descale = p->q_descale; kp.k_descale = p->k_descale; kp.v_descale = p->v_descale;
  kp.s_aux = p->s_aux;
  kp.status = (DeviceStatus*)ws;
  kp.counters = (int32_t*)(ws + 64);
  kp.q_row_stride = p->q_row_stride; kp.q_head_stride = p->q_head_stride;
  kp.k_row_stride = p->k_row_stride; kp.k_head_stride = p->k_head_stride; kp.k_page_stride = p->k_page_stride;
  kp.v_row_stride = p->v_row_stride; kp.v_head_stride = p->v_head_stride; kp.v_page_stride = p->v_page_stride;
  kp.o_row_stride = p->o_row_stride; kp.o_head_stride = p->o_head_stride;
  kp.batch = p->batch; kp.total_q = p->total_q; kp.total_k = p->total_k; kp.num_pages = p->num_pages; kp.hq = p->hq; kp.hkv = p->hkv; kp.rep = p->hq / p->hkv;
  kp.hd = p->hd; kp.hdv = p->hdv;
  kp.max_seqlen_q = p->max_seqlen_q; kp.max_seqlen_k = p->max_seqlen_k;
  kp.page_size = p->page_table ? p->page_size : 0;
  kp.page_shift = -1;
  if (kp.page_size > 0 && (kp.page_size & (kp.page_size - 1)) == 0) {
    int s = 0; while ((1 << s) < kp.page_size) ++s; kp.page_shift = s;
  }
  kp.page_table_stride = p->page_table_stride;
  kp.descale_batch_stride = p->descale_batch_stride; kp.descale_head_stride = p->descale_head_stride;
  kp.q_fp8 = p->q_dtype == FA_DT_FP8_E4M3; kp.kv_fp8 = p->kv_dtype == FA_DT_FP8_E4M3;
  kp.is_causal = in.is_causal; kp.window_left = in.window_left; kp.window_right = in.window_right;
  kp.nsplits = pl.nsplits;
  kp.out_f32 = p->out_dtype == FA_DT_FP32;
  kp.work_expect = SchedExpect{p->batch, pl.nsplits, pl.tile_m, pl.tile_n, pl.max_mtiles, pl.rows_per_token, pl.route};
  kp.scale = p->softmax_scale; kp.softcap = p->softcap;
  if (pl.nsplits > 1) { kp.lse_part = (float*)(ws + w.lse_off); kp.o_part = (float*)(ws + w.o_off); }

  const int compute_dtype = p->q_dtype == FA_DT_FP16 ? FA_DT_FP16 : FA_DT_BF16;

  if (pl.route == FA_ROUTE_DECODE) {
    const int32_t* work = p->scheduler_metadata;
    if (!work) {
      FaSchedParams sp{};
      sp.seqused_k = p->seqused_k; sp.cu_seqlens_q = p->cu_seqlens_q; sp.cu_seqlens_k = p->cu_seqlens_k;
      sp.leftpad_k = p->leftpad_k; sp.batch = p->batch; sp.max_seqlen_q = p->max_seqlen_q;
      sp.max_seqlen_k = p->max_seqlen_k; sp.hq = p->hq; sp.hkv = p->hkv; sp.hd = p->hd; sp.hdv = p->hdv;
      sp.is_causal = in.is_causal; sp.window_left = in.window_left; sp.window_right = in.window_right;
      rc = note_cuda_error(launch_sched(sp, pl, (int32_t*)(ws + w.work_off), clean ? nullptr : (int32_t*)ws, stream),
                           "sched_kernel");
      if (rc != FA_OK) return rc;
      work = (const int32_t*)(ws + w.work_off);
    }
    kp.work = work;
    rc = note_cuda_error(launch_decode(kp, pl, compute_dtype, stream), "decode kernel");
  } else if (pl.route == FA_ROUTE_PREFILL_TC && w.work2_bytes > 0) {
    // mixed batch: two work lists, the decode kernel over the short sequences, then the prefill kernel over the rest
    FaSchedParams sp{};
    sp.seqused_k = p->seqused_k; sp.cu_seqlens_q = p->cu_seqlens_q; sp.cu_seqlens_k = p->cu_seqlens_k;
    sp.leftpad_k = p->leftpad_k; sp.batch = p->batch; sp.max_seqlen_q = p->max_seqlen_q;
    sp.max_seqlen_k = p->max_seqlen_k; sp.hq = p->hq; sp.hkv = p->hkv; sp.hd = p->hd; sp.hdv = p->hdv;
    sp.is_causal = in.is_causal; sp.window_left = in.window_left; sp.window_right = in.window_right;
    const Plan pd = decode_part_plan(in, pl);
    int32_t* list_d = (int32_t*)(ws + w.work_off);
    int32_t* list_p = (int32_t*)(ws + w.work2_off);
    rc = note_cuda_error(launch_sched(sp, pd, list_d, nullptr, stream, 1, kDecodeMaxRows), "sched_kernel");
    if (rc == FA_OK) rc = note_cuda_error(launch_sched(sp, pl, list_p, nullptr, stream, 2, kDecodeMaxRows), "sched_kernel");
    if (rc != FA_OK) return rc;
    KParams kd = kp;
    kd.work = list_d;
    kd.nsplits = 1;
    kd.work_expect = SchedExpect{p->batch, 1, pd.tile_m, pd.tile_n, pd.max_mtiles, pd.rows_per_token, pd.route};
    rc = note_cuda_error(launch_decode(kd, pd, compute_dtype, stream), "decode kernel");
    if (rc != FA_OK) return rc;
    kp.work = list_p;
    rc = note_cuda_error(launch_prefill_tc(kp, pl, compute_dtype, stream), "tcgen05 prefill kernel");
  } else if (pl.route == FA_ROUTE_PREFILL_TC) {
    kp.work = p->scheduler_metadata;   // optional: the sorted (batch, tile) list replaces the arithmetic order
    if (w.dp_k_bytes > 0) {
      // small pages, keys read many times: copy them out of the pages once, then run over contiguous K/V
      void* ks = ws + w.dp_k_off;
      void* vs = ws + w.dp_v_off;
      int32_t* cu = (int32_t*)(ws + w.dp_cu_off);
      rc = note_cuda_error(launch_depage(kp, w.dp_kpad, ks, vs, cu, pl.num_sms, stream), "de-paging kernel");
      if (rc != FA_OK) return rc;
      kp.k = ks; kp.v = vs;
      kp.k_row_stride = (int64_t)p->hkv * p->hd; kp.k_head_stride = p->hd; kp.k_page_stride = 0;
      kp.v_row_stride = (int64_t)p->hkv * p->hdv; kp.v_head_stride = p->hdv; kp.v_page_stride = 0;
      kp.page_table = nullptr; kp.page_size = 0; kp.page_shift = -1; kp.page_table_stride = 0; kp.num_pages = 0;
      kp.cu_k = cu;                              // slab b starts at row b * kpad; lengths still come from seqused_k
      kp.total_k = p->batch * w.dp_kpad;
    }
    rc = note_cuda_error(launch_prefill_tc(kp, pl, compute_dtype, stream), "tcgen05 prefill kernel");
  } else {
    rc = note_cuda_error(launch_general(kp, compute_dtype, p->out_dtype, pl.num_sms, stream), "general kernel");
  }
  if (rc != FA_OK) return rc;

  if (pl.nsplits > 1) {
    rc = note_cuda_error(launch_combine(kp.o_part, kp.lse_part, pl.nsplits, p->total_q, p->hq, p->hdv, p->s_aux,
                                        p->out, p->o_row_stride, p->o_head_stride, p->out_dtype, p->lse, stream),
                         "combine kernel");
  }
  return rc;
}

// ---- decode without allocation: scratch in a device array that is part of this library's image ----
// In host code `g_static_scratch` is only a handle for the symbol, not a device address: the address is looked up
// once per device with cudaGetSymbolAddress and that pointer is what the kernels receive.
static __device__ __align__(256) unsigned char g_static_scratch[FA_B200_STATIC_SCRATCH_BYTES];
static void* g_static_scratch_addr[64];
static std::atomic<int> g_static_scratch_ready[64];

int fa_b200_decode_fwd_static(const FaFwdParams* p, fa_stream_t stream) {
  int rc = validate(p);
  if (rc != FA_OK) return rc;
  const DevInfo* di = device_info();
  if (!di || !di->ok) return FA_ERR_NO_DEVICE;
  Plan pl = make_plan(plan_input(p, di->sms));
  if (pl.err != FA_OK) return pl.err;
  if (pl.route != FA_ROUTE_DECODE) return FA_ERR_UNSUPPORTED;
  if (ws_layout(p, pl).total > (size_t)FA_B200_STATIC_SCRATCH_BYTES) return FA_ERR_STATIC_LIMIT;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FA_ERR_NO_DEVICE;
  if (g_static_scratch_ready[dev].load(std::memory_order_acquire) == 0) {
    std::lock_guard<std::mutex> lk(g_dev_mu);
    if (g_static_scratch_ready[dev].load(std::memory_order_relaxed) == 0) {
      void* addr = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&addr, g_static_scratch);   // this device's copy of the array
      if (e != cudaSuccess || addr == nullptr) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
      g_static_scratch_addr[dev] = addr;
      g_static_scratch_ready[dev].store(1, std::memory_order_release);
    }
  }
  FaFwdParams q = *p;
  q.route = FA_ROUTE_DECODE;
  return fa_b200_fwd(&q, g_static_scratch_addr[dev], (size_t)FA_B200_STATIC_SCRATCH_BYTES, stream);
}

int fa_b200_scheduler_metadata_len(const FaSchedParams* p) {
  if (!p) return 0;
  const DevInfo* di = device_info();
  Plan pl = make_plan(plan_input(p, di && di->sms > 0 ? di->sms : 148));
  if (pl.err != FA_OK) return kSchedHeader;
  return sched_len(pl, p->batch);
}

int fa_b200_get_scheduler_metadata(const FaSchedParams* p, int32_t* out_dev, fa_stream_t stream) {
  if (!p || !out_dev) return FA_ERR_BAD_ARG;
  const DevInfo* di = device_info();
  if (!di || !di->ok) return FA_ERR_NO_DEVICE;
  PlanInput in = plan_input(p, di->sms);
  Plan pl = make_plan(in);
  if (pl.err != FA_OK) return pl.err;
  FaSchedParams sp = *p;
  sp.window_left = in.window_left; sp.window_right = in.window_right;
  return note_cuda_error(launch_sched(sp, pl, out_dev, nullptr, (cudaStream_t)stream), "sched_kernel");
}

int fa_b200_combine(const float* o_part, const float* lse_part, int32_t nsplits, int32_t total_q, int32_t hq,
                    int32_t hdv, const float* s_aux, void* out, int64_t o_row_stride, int64_t o_head_stride,
                    int32_t out_dtype, float* lse, fa_stream_t stream) {
  if (!o_part || !lse_part || !out || !lse || nsplits < 1 || hdv % 4 || o_row_stride % 4 || o_head_stride % 4)
    return FA_ERR_BAD_ARG;
  if (out_dtype != FA_DT_BF16 && out_dtype != FA_DT_FP16) return FA_ERR_UNSUPPORTED;
  const DevInfo* di = device_info();
  if (!di || !di->ok) return FA_ERR_NO_DEVICE;
  return note_cuda_error(launch_combine(o_part, lse_part, nsplits, total_q, hq, hdv, s_aux, out, o_row_stride,
                                        o_head_stride, out_dtype, lse, (cudaStream_t)stream),
                         "combine kernel");
}

int fa_b200_combine_strided(const float* o_part, const float* lse_part, int64_t o_split_stride,
                            int64_t lse_split_stride, int32_t nsplits, int32_t total_q, int32_t hq, int32_t hdv,
                            const float* s_aux, void* out, int64_t o_row_stride, int64_t o_head_stride,
                            int32_t out_dtype, float* lse, fa_stream_t stream) {
  if (!o_part || !lse_part || !out || !lse || nsplits < 1 || hdv % 4 || o_row_stride % 4 || o_head_stride % 4 ||
      o_split_stride % 4 || ((uintptr_t)o_part % 16))
    return FA_ERR_BAD_ARG;
  if (out_dtype != FA_DT_BF16 && out_dtype != FA_DT_FP16) return FA_ERR_UNSUPPORTED;
  const DevInfo* di = device_info();
  if (!di || !di->ok) return FA_ERR_NO_DEVICE;
  return note_cuda_error(launch_combine_strided(o_part, lse_part, o_split_stride, lse_split_stride, nsplits, total_q,
                                                hq, hdv, s_aux, out, o_row_stride, o_head_stride, out_dtype, lse,
                                                (cudaStream_t)stream),
                         "combine kernel");
}

size_t fa_b200_sizeof_append_params(void) { return sizeof(FaAppendParams); }

int fa_b200_append_kv(const FaAppendParams* p, fa_stream_t stream) {
  if (!p || !p->k_cache || !p->v_cache || !p->cu_seqlens_k_new || !p->seqused_k || !p->seqused_k_out || !p->page_table ||
      p->seqused_k_out == p->seqused_k)
    return FA_ERR_BAD_ARG;
  if (p->batch < 0 || p->total_new < 0 || p->hkv <= 0 || p->page_size <= 0) return FA_ERR_BAD_ARG;
  // (a step that appends no key at all - an empty k_new has no address - still rotates the queries and writes the counts)
  if (p->total_new > 0 && (!p->k_new || !p->v_new)) return FA_ERR_BAD_ARG;
  const bool kv8 = p->kv_dtype == FA_DT_FP8_E4M3;
  if (p->kv_dtype < 0 || p->kv_dtype > 2 || p->q_dtype < 0 || p->q_dtype > 1) return FA_ERR_UNSUPPORTED;
  const int esz = kv8 ? 1 : 2, epc = 16 / esz;   // elements per 16-byte chunk
  if (p->hd % epc || p->hdv % epc) return FA_ERR_UNSUPPORTED;
  const int64_t st[] = {p->kn_row_stride, p->kn_head_stride, p->vn_row_stride, p->vn_head_stride, p->k_row_stride,
                        p->k_head_stride, p->k_page_stride, p->v_row_stride, p->v_head_stride, p->v_page_stride};
  for (int64_t s : st) if (s % epc) return FA_ERR_UNSUPPORTED;
  const uintptr_t ptrs[] = {(uintptr_t)p->k_new, (uintptr_t)p->v_new, (uintptr_t)p->k_cache, (uintptr_t)p->v_cache};
  for (uintptr_t a : ptrs) if (a % 16) return FA_ERR_UNSUPPORTED;
  if (p->rotary_cos) {
    if (!p->rotary_sin || !p->cu_seqlens_q) return FA_ERR_BAD_ARG;
    if (p->total_q > 0 && (!p->q || !p->q_out || p->q_out == p->q)) return FA_ERR_BAD_ARG;   // (no query rows: no addresses)
    if (kv8 || p->kv_dtype != p->q_dtype) return FA_ERR_UNSUPPORTED;       // keys are rotated in the query type
    if (p->rotary_dim <= 0 || p->rotary_dim % 16 || p->rotary_dim > p->hd || p->hd % 8) return FA_ERR_UNSUPPORTED;
    if (p->q_row_stride % 8 || p->q_head_stride % 8 || p->qo_row_stride % 8 || p->qo_head_stride % 8 ||
        ((uintptr_t)p->q % 16) || ((uintptr_t)p->q_out % 16) || ((uintptr_t)p->rotary_cos % 16) || ((uintptr_t)p->rotary_sin % 16))
      return FA_ERR_UNSUPPORTED;
  }
  const DevInfo* di = device_info();
  if (!di || !di->ok) return FA_ERR_NO_DEVICE;
  if (p->batch == 0) return FA_OK;
  return note_cuda_error(launch_append_kv(*p, di->sms, (cudaStream_t)stream), "append kernel");
}

int fa_b200_selftest_timeout(void* workspace, int64_t max_cycles, fa_stream_t stream_) {
  if (!workspace || ((uintptr_t)workspace % 16)) return FA_ERR_BAD_ARG;
  const DevInfo* di = device_info();
  if (!di || !di->ok) return FA_ERR_NO_DEVICE;
  cudaStream_t stream = (cudaStream_t)stream_;
  cudaError_t ce = cudaMemsetAsync(workspace, 0, 256, stream);
  if (ce != cudaSuccess) return cuda_fail(ce, "cudaMemsetAsync(workspace header)");
  long long c = max_cycles < 10000 ? 10000 : (max_cycles > 100000000 ? 100000000 : max_cycles);
  return note_cuda_error(launch_selftest_timeout((DeviceStatus*)workspace, c, stream), "self-test kernel");
}

int fa_b200_check_status(void* workspace, fa_stream_t stream, uint32_t* detail) {
  if (!workspace) return FA_ERR_BAD_ARG;
  cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSynchronize");
  DeviceStatus st;
  e = cudaMemcpy(&st, workspace, sizeof(st), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpy(status)");
  if (detail) *detail = st.detail;
  if (st.error == 0) return FA_OK;
  return st.error == DEV_ERR_BAD_INDEX ? FA_ERR_BAD_METADATA : FA_ERR_DEVICE_TIMEOUT;
}

}  // extern "C"
