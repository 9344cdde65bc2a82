// fa_combine.cu — split-KV merge and the scheduler-metadata kernel.
#include "fa_internal.h"
#include "fa_sched.h"
#include "ptx.cuh"

namespace fa {

constexpr float kLog2eC = 1.4426950408889634f;
constexpr float kLn2C = 0.6931471805599453f;

// ------------------------------------------------------------------------------------------------
// LSE-weighted merge of split partials (the maths of kernels/fa4_blackwell.cu:5964-5985): one thread
// per (q row, head, 4 consecutive output columns); float4 reads of o_part, 8-byte stores of out.
// A split whose lse is -inf contributes exactly 0 even if its partial was never written.
// Split s starts o_split_stride / lse_split_stride floats after split s-1, so partials can be merged where a
// gather left them (one packed [O | LSE] buffer per rank).
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) combine_kernel(const float* __restrict__ o_part,
                                                      const float* __restrict__ lse_part, int64_t o_split_stride,
                                                      int64_t lse_split_stride, int nsplits, int total_q,
                                                      int hq, int hdv, const float* __restrict__ s_aux,
                                                      T* __restrict__ out, int64_t o_row_stride,
                                                      int64_t o_head_stride, float* __restrict__ lse) {
  const int vec = hdv >> 2;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)total_q * hq * vec) return;
  const int dv = (int)(idx % vec) * 4;
  const int64_t qh = idx / vec;
  const int h = (int)(qh % hq);
  const int64_t qi = qh / hq;

  float g = -INFINITY;
  const int64_t lse_idx = (int64_t)h * total_q + qi;
  const int64_t o_idx = (qi * hq + h) * hdv + dv;
  for (int s = 0; s < nsplits; ++s) g = fmaxf(g, lse_part[s * lse_split_stride + lse_idx]);
  const bool has_sink = s_aux != nullptr;
  const float sk = has_sink ? s_aux[h] : -INFINITY;
  g = fmaxf(g, sk);
  T* op = out + qi * o_row_stride + (int64_t)h * o_head_stride + dv;
  if (g == -INFINITY) {
    *reinterpret_cast<uint2*>(op) = make_uint2(0u, 0u);
    if (dv == 0) lse[(int64_t)h * total_q + qi] = -INFINITY;
    return;
  }
  float L = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < nsplits; ++s) {
    const float ls = lse_part[s * lse_split_stride + lse_idx];
    if (ls > -INFINITY) {
      const float w = ex2((ls - g) * kLog2eC);
      const float4 o = *reinterpret_cast<const float4*>(o_part + s * o_split_stride + o_idx);
      L += w;
      acc.x += w * o.x; acc.y += w * o.y; acc.z += w * o.z; acc.w += w * o.w;
    }
  }
  if (has_sink) L += ex2((sk - g) * kLog2eC);
  const float inv = L > 0.f ? 1.f / L : 0.f;
  uint2 packed;
  packed.x = pack2<T>(acc.x * inv, acc.y * inv);
  packed.y = pack2<T>(acc.z * inv, acc.w * inv);
  *reinterpret_cast<uint2*>(op) = packed;
  if (dv == 0) lse[(int64_t)h * total_q + qi] = g + lg2(L) * kLn2C;
}

int launch_combine_strided(const float* o_part, const float* lse_part, int64_t o_split_stride, int64_t lse_split_stride,
                           int nsplits, int total_q, int hq, int hdv, const float* s_aux, void* out,
                           int64_t o_row_stride, int64_t o_head_stride, int out_dtype, float* lse, cudaStream_t stream) {
  if (hdv % 4 != 0) return -1;
  const int64_t n = (int64_t)total_q * hq * (hdv / 4);
  if (n == 0) return 0;
  const int threads = 256;
  const unsigned blocks = (unsigned)((n + threads - 1) / threads);
  if (out_dtype == FA_DT_FP16)
    combine_kernel<__half><<<blocks, threads, 0, stream>>>(o_part, lse_part, o_split_stride, lse_split_stride, nsplits,
                                                            total_q, hq, hdv, s_aux, (__half*)out, o_row_stride,
                                                            o_head_stride, lse);
  else
    combine_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(o_part, lse_part, o_split_stride, lse_split_stride,
                                                                   nsplits, total_q, hq, hdv, s_aux,
                                                                   (__nv_bfloat16*)out, o_row_stride, o_head_stride, lse);
  return (int)cudaGetLastError();
}

int launch_combine(const float* o_part, const float* lse_part, int nsplits, int total_q, int hq, int hdv,
                   const float* s_aux, void* out, int64_t o_row_stride, int64_t o_head_stride, int out_dtype,
                   float* lse, cudaStream_t stream) {
  return launch_combine_strided(o_part, lse_part, (int64_t)total_q * hq * hdv, (int64_t)hq * total_q, nsplits, total_q,
                                hq, hdv, s_aux, out, o_row_stride, o_head_stride, out_dtype, lse, stream);
}

// ------------------------------------------------------------------------------------------------
// Scheduler metadata: per (batch, m_tile) key-block range, sorted longest-first (layout in fa_sched.h).
// One CTA; the slots are sorted in shared memory (bitonic network over 32-bit keys: block count in the high
// bits, descending; slot index in the low 13 bits, ascending), at most kSchedSortMax slots.
// ------------------------------------------------------------------------------------------------
struct SchedArgs {
  const int32_t* seqused_k;
  const int32_t* cu_q;
  const int32_t* cu_k;
  const int32_t* leftpad_k;
  int32_t batch, max_seqlen_q, max_seqlen_k;
  int32_t is_causal, window_left, window_right;
  int32_t tile_m, tile_n, rows_per_token, max_mtiles, nsplits, route;
  int32_t sorted;          // E <= kSchedSortMax and every block count fits the key (host decision, fa_sched.h)
  int32_t sort_n;          // power of two >= E
  int32_t* zero_words;     // when not null: 64 words (a workspace header) this kernel clears for the kernel after it
  int32_t row_class;       // 0: every sequence; 1: only sequences with at most class_rows packed query rows per kv head
  int32_t class_rows;      //    (the decode kernel's share of a mixed batch); 2: only the others (the prefill kernel's)
  int32_t class_rep;       // q heads per kv head, for the row count of the class test
};

__device__ __forceinline__ bool sched_entry(const SchedArgs& a, int e, int* b_out, int* mt_out, int* lo, int* hi) {
  const int b = e / a.max_mtiles, mt = e % a.max_mtiles;
  const int seqlen_q = a.cu_q ? a.cu_q[b + 1] - a.cu_q[b] : a.max_seqlen_q;
  const int seqlen_k = a.seqused_k ? a.seqused_k[b] : (a.cu_k ? a.cu_k[b + 1] - a.cu_k[b] : a.max_seqlen_k);
  const int leftpad = a.leftpad_k ? a.leftpad_k[b] : 0;
  const int rows_total = seqlen_q * a.rows_per_token;
  const int row0 = mt * a.tile_m;
  *b_out = b;
  *mt_out = mt;
  if (row0 >= rows_total) { *lo = 0; *hi = 0; return false; }
  if (a.row_class != 0) {
    const bool small = seqlen_q * a.class_rep <= a.class_rows;
    if (small != (a.row_class == 1)) { *lo = 0; *hi = 0; return false; }
  }
  const int tok_min = row0 / a.rows_per_token;
  const int tok_max = min(seqlen_q - 1, (row0 + a.tile_m - 1) / a.rows_per_token);
  nblock_range(seqlen_k, leftpad, seqlen_k - seqlen_q + tok_min, seqlen_k - seqlen_q + tok_max, a.is_causal,
               a.window_left, a.window_right, a.tile_n, lo, hi);
  return true;
}

__global__ void __launch_bounds__(1024) sched_kernel(const SchedArgs a, int32_t* __restrict__ out) {
  extern __shared__ uint32_t s_key[];   // sort keys, sort_n of them
  __shared__ int s_valid;
  const int E = a.batch * a.max_mtiles;
  const int tid = threadIdx.x, nt = blockDim.x;
  const bool sorted = a.sorted != 0;
  if (a.zero_words != nullptr && tid < 64) a.zero_words[tid] = 0;
  if (tid == 0) s_valid = 0;
  __syncthreads();
  if (!sorted) {
    for (int e = tid; e < E; e += nt) {
      int b, mt, lo, hi;
      const bool ok = sched_entry(a, e, &b, &mt, &lo, &hi);
      out[kSchedHeader + 4 * e + 0] = ok ? b : -1;
      out[kSchedHeader + 4 * e + 1] = ok ? mt : -1;
      out[kSchedHeader + 4 * e + 2] = lo;
      out[kSchedHeader + 4 * e + 3] = hi;
    }
  } else {
    const int N = a.sort_n;
    int nvalid = 0;
    for (int e = tid; e < N; e += nt) {
      uint32_t key = 0xffffffffu;               // padding and slots without rows sort last
      if (e < E) {
        int b, mt, lo, hi;
        if (sched_entry(a, e, &b, &mt, &lo, &hi)) {
          key = ((uint32_t)(kSchedCountMax - (hi - lo)) << kSchedSlotBits) | (uint32_t)e;
          ++nvalid;
        }
      }
      s_key[e] = key;
    }
    atomicAdd(&s_valid, nvalid);
    __syncthreads();
    for (int k = 2; k <= N; k <<= 1) {
      for (int j = k >> 1; j > 0; j >>= 1) {
        for (int i = tid; i < N; i += nt) {
          const int ixj = i ^ j;
          if (ixj > i) {
            const uint32_t x = s_key[i], y = s_key[ixj];
            const bool up = (i & k) == 0;
            if ((x > y) == up) { s_key[i] = y; s_key[ixj] = x; }
          }
        }
        __syncthreads();
      }
    }
    const int V = s_valid;
    for (int i = tid; i < E; i += nt) {
      int b = -1, mt = -1, lo = 0, hi = 0;
      if (i < V) sched_entry(a, (int)(s_key[i] & ((1u << kSchedSlotBits) - 1u)), &b, &mt, &lo, &hi);
      out[kSchedHeader + 4 * i + 0] = b;
      out[kSchedHeader + 4 * i + 1] = mt;
      out[kSchedHeader + 4 * i + 2] = lo;
      out[kSchedHeader + 4 * i + 3] = hi;
    }
  }
  __syncthreads();
  if (tid < kSchedHeader) {
    int32_t v = 0;
    switch (tid) {
      case 0: v = kSchedMagic; break;
      case 1: v = kSchedVersion; break;
      case 2: v = a.batch; break;
      case 3: v = a.nsplits; break;
      case 4: v = a.tile_m; break;
      case 5: v = a.tile_n; break;
      case 6: v = sorted ? s_valid : E; break;
      case 7: v = a.max_mtiles; break;
      case 8: v = a.rows_per_token; break;
      case 9: v = a.route; break;
      case 10: v = sorted ? 1 : 0; break;
      default: v = 0;
    }
    out[tid] = v;
  }
}

// Bounded-wait self-test: one warp waits on a barrier that nobody arrives at; the wait gives up after
// `max_cycles`, the time-out is recorded in the status word, and the kernel returns.
__global__ void __launch_bounds__(32) selftest_timeout_kernel(DeviceStatus* status, long long max_cycles) {
  __shared__ __align__(8) unsigned long long s_bar;
  __shared__ int s_abort;
  const uint32_t bar = smem_u32(&s_bar);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    s_abort = 0;
    mbar_fence_init();
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    if (!wait_or_abort(bar, 0, &s_abort, max_cycles)) report_error(status, DEV_ERR_TIMEOUT, 7u /* self-test role */);
  }
}

int launch_selftest_timeout(DeviceStatus* status, long long max_cycles, cudaStream_t stream) {
  selftest_timeout_kernel<<<1, 32, 0, stream>>>(status, max_cycles);
  return (int)cudaGetLastError();
}

int launch_sched(const FaSchedParams& sp, const Plan& pl, int32_t* out_dev, int32_t* zero_words, cudaStream_t stream,
                 int row_class, int class_rows) {
  SchedArgs a;
  a.seqused_k = sp.seqused_k; a.cu_q = sp.cu_seqlens_q; a.cu_k = sp.cu_seqlens_k; a.leftpad_k = sp.leftpad_k;
  a.batch = sp.batch; a.max_seqlen_q = sp.max_seqlen_q; a.max_seqlen_k = sp.max_seqlen_k;
  a.is_causal = sp.is_causal; a.window_left = sp.window_left; a.window_right = sp.window_right;
  a.tile_m = pl.tile_m; a.tile_n = pl.tile_n; a.rows_per_token = pl.rows_per_token;
  a.max_mtiles = pl.max_mtiles; a.nsplits = pl.nsplits; a.route = pl.route;
  const int E = sp.batch * pl.max_mtiles;
  a.sorted = sched_is_sorted(E, sp.max_seqlen_k, pl.tile_n) ? 1 : 0;
  a.sort_n = 1;
  while (a.sort_n < E) a.sort_n <<= 1;
  a.zero_words = zero_words;
  a.row_class = row_class; a.class_rows = class_rows; a.class_rep = sp.hkv > 0 ? sp.hq / sp.hkv : 1;
  const size_t smem = a.sorted ? (size_t)a.sort_n * sizeof(uint32_t) : 0;
  const int threads = (a.sorted && a.sort_n < 1024) ? (a.sort_n < 64 ? 64 : a.sort_n) : 1024;
  sched_kernel<<<1, threads, smem, stream>>>(a, out_dev);
  return (int)cudaGetLastError();
}

}  // namespace fa
