// fa_append.cu — the step in front of attention in a serving loop: append the new keys / values of this step to
// the paged cache (in place) and apply the rotary position embedding to them and to the queries.
//
// One launch, memory-bound: a group of (row bytes / 16) threads moves one (token, head) row, 16 bytes per thread.
//   K rows:  k_new[token, head] --rotary--> k_cache[page_table[b][(n + i) / page] * page + (n + i) % page, head]
//   V rows:  v_new[token, head] ----------> v_cache[same row, head]
//   Q rows:  q[token, head]     --rotary--> q_out[token, head]            (only when a rotary table is given)
// with n = seqused_k[b] (keys already cached) and i the index of the new token inside its sequence.  The kernel
// also writes seqused_k_out[b] = n + (number of new tokens of b), the key count the attention call then uses.
// Rotary (the op's documented behaviour): the new key i of sequence b is rotated at position r_b + i, r_b =
// seqlens_rotary[b] if given, else seqused_k[b]; query i at r_b + i when the attention is causal or windowed, at r_b
// otherwise.  Interleaved pairs dimensions (2j, 2j+1); otherwise (j, j + rotary_dim/2).  The products and the sum
// are rounded separately in fp32 (no fused multiply-add), so the result is bit-identical to the same arithmetic
// written out in any fp32 library.
//
// The reference pins these arguments of the op to None (bench/scenarios.py:915-921); there is no counterpart kernel.
#include "fa_internal.h"
#include "ptx.cuh"

namespace fa {

struct AppendArgs {
  FaAppendParams p;
  int64_t k_rows, v_rows, q_rows;   // (token, head) rows of each kind
  int k_tpr, v_tpr, q_tpr;          // threads per row
  int esz;                          // bytes per element
};

// batch index of packed token `tok` (cu is ascending, cu[batch] = total)
__device__ __forceinline__ int find_batch(const int32_t* cu, int batch, int tok) {
  int lo = 0, hi = batch - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu[mid] <= tok) lo = mid; else hi = mid - 1;
  }
  return lo;
}

template <typename T>
__device__ __forceinline__ float2 unpack2(uint32_t v);
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t v) {
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t v) {
  return __half22float2(*reinterpret_cast<const __half2*>(&v));
}

// Rotates the 8 elements `x` (dimensions e0 .. e0+7 of one row, e0 + 8 <= rotary_dim) at position `pos`.
template <typename T>
__device__ __forceinline__ uint4 rotate8(uint4 x, const T* row, int e0, const FaAppendParams& p, int pos) {
  const int half = p.rotary_dim >> 1;
  const T* cs = reinterpret_cast<const T*>(p.rotary_cos) + (int64_t)pos * half;
  const T* sn = reinterpret_cast<const T*>(p.rotary_sin) + (int64_t)pos * half;
  uint32_t in[4] = {x.x, x.y, x.z, x.w}, out[4];
  if (p.rotary_interleaved) {
    // pairs (e0 + 2i, e0 + 2i + 1) share table entry e0/2 + i: four entries = 8 bytes
    const uint2 c4 = *reinterpret_cast<const uint2*>(cs + (e0 >> 1));
    const uint2 s4 = *reinterpret_cast<const uint2*>(sn + (e0 >> 1));
    const uint32_t cw[2] = {c4.x, c4.y}, sw[2] = {s4.x, s4.y};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 v = unpack2<T>(in[i]);
      const float2 c2 = unpack2<T>(cw[i >> 1]), s2 = unpack2<T>(sw[i >> 1]);
      const float c = (i & 1) ? c2.y : c2.x, s = (i & 1) ? s2.y : s2.x;
      const float r0 = __fsub_rn(__fmul_rn(v.x, c), __fmul_rn(v.y, s));
      const float r1 = __fadd_rn(__fmul_rn(v.x, s), __fmul_rn(v.y, c));
      out[i] = pack2<T>(r0, r1);
    }
  } else {
    // dimension e pairs with e + half (first half) or e - half (second half); the partner chunk is read from the row
    const bool first = e0 < half;
    const int t0 = first ? e0 : e0 - half;          // table index of the chunk's first element
    const uint4 pr = *reinterpret_cast<const uint4*>(row + (first ? e0 + half : e0 - half));
    const uint4 c8 = *reinterpret_cast<const uint4*>(cs + t0);
    const uint4 s8 = *reinterpret_cast<const uint4*>(sn + t0);
    const uint32_t pw[4] = {pr.x, pr.y, pr.z, pr.w}, cw[4] = {c8.x, c8.y, c8.z, c8.w}, sw[4] = {s8.x, s8.y, s8.z, s8.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 v = unpack2<T>(in[i]), q = unpack2<T>(pw[i]), c = unpack2<T>(cw[i]), s = unpack2<T>(sw[i]);
      float r0, r1;
      if (first) {   // x1' = x1 c - x2 s
        r0 = __fsub_rn(__fmul_rn(v.x, c.x), __fmul_rn(q.x, s.x));
        r1 = __fsub_rn(__fmul_rn(v.y, c.y), __fmul_rn(q.y, s.y));
      } else {       // x2' = x1 s + x2 c   (x1 is the partner)
        r0 = __fadd_rn(__fmul_rn(q.x, s.x), __fmul_rn(v.x, c.x));
        r1 = __fadd_rn(__fmul_rn(q.y, s.y), __fmul_rn(v.y, c.y));
      }
      out[i] = pack2<T>(r0, r1);
    }
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}

template <typename T>
__global__ void __launch_bounds__(256) append_kv_kernel(const AppendArgs a) {
  const FaAppendParams& p = a.p;
  const int64_t k_threads = a.k_rows * a.k_tpr, v_threads = a.v_rows * a.v_tpr, q_threads = a.q_rows * a.q_tpr;
  const int64_t total = k_threads + v_threads + q_threads;
  const bool rot = p.rotary_cos != nullptr;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    if (idx < k_threads + v_threads) {
      const bool is_k = idx < k_threads;
      const int64_t j = is_k ? idx : idx - k_threads;
      const int tpr = is_k ? a.k_tpr : a.v_tpr;
      const int64_t row = j / tpr;
      const int c = (int)(j - row * tpr);                 // 16-byte chunk of the row
      const int tok = (int)(row / p.hkv), h = (int)(row - (int64_t)tok * p.hkv);
      const int b = find_batch(p.cu_seqlens_k_new, p.batch, tok);
      const int i = tok - p.cu_seqlens_k_new[b];
      const int n = p.seqused_k[b];
      const int kidx = n + i;
      const int lp = kidx / p.page_size;
      const int64_t page = p.page_table[(int64_t)b * p.page_table_stride + lp];
      const int64_t prow = kidx - lp * p.page_size;
      if (is_k && h == 0 && c == 0 && i == 0) p.seqused_k_out[b] = n + (p.cu_seqlens_k_new[b + 1] - p.cu_seqlens_k_new[b]);
      const unsigned char* src = reinterpret_cast<const unsigned char*>(is_k ? p.k_new : p.v_new) +
                                 ((int64_t)tok * (is_k ? p.kn_row_stride : p.vn_row_stride) +
                                  (int64_t)h * (is_k ? p.kn_head_stride : p.vn_head_stride)) * a.esz;
      unsigned char* dst = reinterpret_cast<unsigned char*>(is_k ? p.k_cache : p.v_cache) +
                           (page * (is_k ? p.k_page_stride : p.v_page_stride) + prow * (is_k ? p.k_row_stride : p.v_row_stride) +
                            (int64_t)h * (is_k ? p.k_head_stride : p.v_head_stride)) * a.esz;
      uint4 x = *reinterpret_cast<const uint4*>(src + c * 16);
      if (is_k && rot && c * 8 < p.rotary_dim) {
        const int pos = (p.seqlens_rotary ? p.seqlens_rotary[b] : n) + i;
        x = rotate8<T>(x, reinterpret_cast<const T*>(src), c * 8, p, pos);
      }
      *reinterpret_cast<uint4*>(dst + c * 16) = x;
    } else {
      const int64_t j = idx - k_threads - v_threads;
      const int64_t row = j / a.q_tpr;
      const int c = (int)(j - row * a.q_tpr);
      const int tok = (int)(row / p.hq), h = (int)(row - (int64_t)tok * p.hq);
      const int b = find_batch(p.cu_seqlens_q, p.batch, tok);
      const int i = tok - p.cu_seqlens_q[b];
      const T* src = reinterpret_cast<const T*>(p.q) + (int64_t)tok * p.q_row_stride + (int64_t)h * p.q_head_stride;
      T* dst = reinterpret_cast<T*>(p.q_out) + (int64_t)tok * p.qo_row_stride + (int64_t)h * p.qo_head_stride;
      uint4 x = *reinterpret_cast<const uint4*>(src + c * 8);
      if (c * 8 < p.rotary_dim) {
        const int pos = (p.seqlens_rotary ? p.seqlens_rotary[b] : p.seqused_k[b]) + (p.q_positions_advance ? i : 0);
        x = rotate8<T>(x, src, c * 8, p, pos);
      }
      *reinterpret_cast<uint4*>(dst + c * 8) = x;
    }
  }
  // sequences without new tokens still get their (unchanged) key count
  if (blockIdx.x == 0) {
    for (int b = threadIdx.x; b < p.batch; b += blockDim.x)
      if (p.cu_seqlens_k_new[b + 1] == p.cu_seqlens_k_new[b]) p.seqused_k_out[b] = p.seqused_k[b];
  }
}

int launch_append_kv(const FaAppendParams& p, int num_sms, cudaStream_t stream) {
  AppendArgs a;
  a.p = p;
  a.esz = p.kv_dtype == FA_DT_FP8_E4M3 ? 1 : 2;
  a.k_rows = (int64_t)p.total_new * p.hkv;
  a.v_rows = a.k_rows;
  a.k_tpr = p.hd * a.esz / 16;
  a.v_tpr = p.hdv * a.esz / 16;
  const bool rot = p.rotary_cos != nullptr;
  a.q_rows = rot ? (int64_t)p.total_q * p.hq : 0;
  a.q_tpr = p.hd * 2 / 16;
  const int64_t total = a.k_rows * a.k_tpr + a.v_rows * a.v_tpr + a.q_rows * a.q_tpr;
  int64_t blocks = (total + 255) / 256;
  if (blocks < 1) blocks = 1;                       // the key counts are still written
  const int64_t cap = (int64_t)num_sms * 8;
  if (blocks > cap) blocks = cap;
  if (p.q_dtype == FA_DT_FP16) append_kv_kernel<__half><<<(unsigned)blocks, 256, 0, stream>>>(a);
  else append_kv_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>(a);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------
// De-paging: every sequence's K and V rows out of the page pool into contiguous slabs of `kpad` rows (slab b starts
// at row b * kpad), 16 bytes per thread, a row's chunks on consecutive threads.  Rows from the sequence's end to
// the end of its last 128-key block are written as zeros: the attention kernel loads whole blocks and gives those
// rows weight zero, which needs finite values there.  Also writes the slabs' row offsets (batch + 1 words).
struct DepageArgs {
  const unsigned char* k;
  const unsigned char* v;
  unsigned char* k_out;
  unsigned char* v_out;
  const int32_t* page_table;
  const int32_t* seqused_k;
  int32_t* cu_out;
  int64_t k_page_bytes, k_row_bytes, k_head_bytes, v_page_bytes, v_row_bytes, v_head_bytes;
  int batch, kpad, hkv, page_shift, page_table_stride;
  int k_hchunks, v_hchunks;      // 16-byte chunks per head of a K / V row
};

__global__ void __launch_bounds__(256) depage_kernel(const DepageArgs a) {
  const int b = blockIdx.y;
  if (blockIdx.x == 0 && b == 0 && threadIdx.x <= a.batch) a.cu_out[threadIdx.x] = threadIdx.x * a.kpad;
  if (blockIdx.x == 0 && b == 0)
    for (int i = threadIdx.x + 256; i <= a.batch; i += 256) a.cu_out[i] = i * a.kpad;
  const int used = a.seqused_k[b];
  const int rows = min((used + 127) / 128 * 128, a.kpad);
  const int kc = a.hkv * a.k_hchunks, vc = a.hkv * a.v_hchunks, rc = kc + vc;     // chunks per (K row + V row)
  const int64_t total = (int64_t)rows * rc;
  const int32_t* pt = a.page_table + (int64_t)b * a.page_table_stride;
  const int pmask = (1 << a.page_shift) - 1;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
    const int r = (int)(i / rc), c = (int)(i - (int64_t)r * rc);
    const bool is_v = c >= kc;
    const int cc = is_v ? c - kc : c;
    const int hch = is_v ? a.v_hchunks : a.k_hchunks;
    const int h = cc / hch, w = cc - h * hch;
    int4 val = make_int4(0, 0, 0, 0);
    if (r < used) {
      const int pid = pt[r >> a.page_shift], slot = r & pmask;
      const unsigned char* src = is_v ? a.v + pid * a.v_page_bytes + slot * a.v_row_bytes + h * a.v_head_bytes
                                      : a.k + pid * a.k_page_bytes + slot * a.k_row_bytes + h * a.k_head_bytes;
      val = *reinterpret_cast<const int4*>(src + (int64_t)w * 16);
    }
    unsigned char* dst = is_v ? a.v_out + ((int64_t)b * a.kpad + r) * ((int64_t)vc * 16)
                              : a.k_out + ((int64_t)b * a.kpad + r) * ((int64_t)kc * 16);
    *reinterpret_cast<int4*>(dst + (int64_t)cc * 16) = val;
  }
}

int launch_depage(const KParams& kp, int kpad, void* k_out, void* v_out, int32_t* cu_out, int num_sms, cudaStream_t stream) {
  const int esz = kp.kv_fp8 ? 1 : 2;
  DepageArgs a;
  a.k = reinterpret_cast<const unsigned char*>(kp.k);
  a.v = reinterpret_cast<const unsigned char*>(kp.v);
  a.k_out = reinterpret_cast<unsigned char*>(k_out);
  a.v_out = reinterpret_cast<unsigned char*>(v_out);
  a.page_table = kp.page_table;
  a.seqused_k = kp.seqused_k;
  a.cu_out = cu_out;
  a.k_page_bytes = kp.k_page_stride * esz; a.k_row_bytes = kp.k_row_stride * esz; a.k_head_bytes = kp.k_head_stride * esz;
  a.v_page_bytes = kp.v_page_stride * esz; a.v_row_bytes = kp.v_row_stride * esz; a.v_head_bytes = kp.v_head_stride * esz;
  a.batch = kp.batch; a.kpad = kpad; a.hkv = kp.hkv; a.page_shift = kp.page_shift; a.page_table_stride = kp.page_table_stride;
  a.k_hchunks = kp.hd * esz / 16; a.v_hchunks = kp.hdv * esz / 16;
  if (kp.page_shift < 0 || kp.hd * esz % 16 || kp.hdv * esz % 16 || kp.batch <= 0) return (int)cudaErrorInvalidValue;
  const int64_t per_seq = (int64_t)kpad * kp.hkv * (a.k_hchunks + a.v_hchunks);
  int64_t bx = (per_seq + 256 * 8 - 1) / (256 * 8);        // about eight chunks per thread
  const int64_t cap = (int64_t)num_sms * 16 / kp.batch + 1;
  if (bx > cap) bx = cap;
  if (bx < 1) bx = 1;
  depage_kernel<<<dim3((unsigned)bx, (unsigned)kp.batch), 256, 0, stream>>>(a);
  return (int)cudaGetLastError();
}

}  // namespace fa
