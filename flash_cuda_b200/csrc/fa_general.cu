// fa_general.cu — the any-shape attention-forward kernel (warp-level mma.sync, 64x64 tiles).
//
// Role: the route for shapes outside the envelopes of the tcgen05 prefill kernel and the paged-decode
// kernel (odd page sizes, head dims 96/256, ...), the role `fwd_kernel` plays in the reference
// (kernels/fa4_blackwell.cu:5805-5959).  It implements the complete semantics of the op: varlen,
// paged or contiguous KV, GQA/MQA (rows of one KV head packed into the M tile), causal with
// bottom-right alignment, two-sided window, softcap, per-batch leftpad, fp8 inputs with descales,
// sink, head_dim_v != head_dim, split-KV partials.
#include "fa_internal.h"
#include "ptx.cuh"

namespace fa {
namespace general {

constexpr int BM = 64, BN = 64, NTHREADS = 128, PAD = 8;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

template <typename T>
__device__ __forceinline__ void store8(T* dst, uint4 v) { *reinterpret_cast<uint4*>(dst) = v; }

// 8 consecutive elements starting at `src` (16-bit types: one 16-byte load; fp8: one 8-byte load + convert)
template <typename T>
__device__ __forceinline__ uint4 load8(const void* base, int64_t elem_off, bool fp8) {
  uint4 r;
  if (!fp8) {
    r = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(base) + elem_off);
  } else {
    uint2 x = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(base) + elem_off);
    e4m3x4_to<T>(x.x, r.x, r.y);
    e4m3x4_to<T>(x.y, r.z, r.w);
  }
  return r;
}

template <typename T, int HD, int HDV>
__global__ void __launch_bounds__(NTHREADS) fwd_general_kernel(const KParams p) {
  constexpr int LDQ = HD + PAD, LDV = HDV + PAD;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* sQ = reinterpret_cast<T*>(smem_raw);
  T* sK = sQ + BM * LDQ;
  T* sV = sK + BN * LDQ;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // grid: x = (split * batch + b) * mtiles + m tile (x has the 2^31 range; y and z stop at 65535), y = kv head
  const int mtiles = (p.max_seqlen_q * p.rep + BM - 1) / BM;
  const int mt = blockIdx.x % mtiles, hk = blockIdx.y;
  const int bz = blockIdx.x / mtiles;
  const int b = bz % p.batch, split = bz / p.batch;
  const int rep = p.rep;

  const int q0 = p.cu_q[b];
  const int seqlen_q = p.cu_q[b + 1] - q0;
  const int k0 = p.page_table ? 0 : p.cu_k[b];
  const int seqlen_k = p.seqused_k ? p.seqused_k[b] : (p.cu_k[b + 1] - p.cu_k[b]);
  const int leftpad = p.leftpad_k ? p.leftpad_k[b] : 0;
  const int rows_total = seqlen_q * rep;      // packed rows of this (batch, kv head)
  const int row0 = mt * BM;
  if (row0 >= rows_total) return;

  // descales
  float sc = p.scale, vds = 1.f;
  {
    const int di = b * p.descale_batch_stride + hk * p.descale_head_stride;
    if (p.q_descale) sc *= p.q_descale[di];
    if (p.k_descale) sc *= p.k_descale[di];
    if (p.v_descale) vds = p.v_descale[di];
  }
  const bool has_cap = p.softcap > 0.f;
  const float y_scale = has_cap ? p.softcap * kLog2e : sc * kLog2e;   // multiplies tanh(.) or the raw score
  const float cap_in = has_cap ? sc / p.softcap : 0.f;

  // ---- Q tile -> smem (rows beyond the sequence and columns beyond hd are zero) ----
  for (int i = tid; i < BM * (HD / 8); i += NTHREADS) {
    const int r = i / (HD / 8), c = (i % (HD / 8)) * 8;
    const int R = row0 + r;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (R < rows_total && c < p.hd) {
      const int token = R / rep, head = hk * rep + R % rep;
      val = load8<T>(p.q, (int64_t)(q0 + token) * p.q_row_stride + (int64_t)head * p.q_head_stride + c, p.q_fp8);
    }
    store8(sQ + r * LDQ + c, val);
  }

  // ---- key-block range of this tile / split ----
  const int tok_min = row0 / rep;
  const int tok_max = min(seqlen_q - 1, (row0 + BM - 1) / rep);
  const int qp_min = seqlen_k - seqlen_q + tok_min, qp_max = seqlen_k - seqlen_q + tok_max;
  int n_lo, n_hi;
  nblock_range(seqlen_k, leftpad, qp_min, qp_max, p.is_causal, p.window_left, p.window_right, BN, &n_lo, &n_hi);
  if (p.nsplits > 1) split_range(n_lo, n_hi, split, p.nsplits, &n_lo, &n_hi);

  // this thread's two rows
  const int r_a = warp * 16 + (lane >> 2), r_b = r_a + 8;
  const int R_a = row0 + r_a, R_b = row0 + r_b;
  const int qp_a = seqlen_k - seqlen_q + R_a / rep, qp_b = seqlen_k - seqlen_q + R_b / rep;
  // valid key interval per row: [lo, hi]
  int lo_a = leftpad, lo_b = leftpad, hi_a = seqlen_k - 1, hi_b = seqlen_k - 1;
  if (p.is_causal) { hi_a = min(hi_a, qp_a); hi_b = min(hi_b, qp_b); }
  if (p.window_right >= 0) { hi_a = min(hi_a, qp_a + p.window_right); hi_b = min(hi_b, qp_b + p.window_right); }
  if (p.window_left >= 0) { lo_a = max(lo_a, qp_a - p.window_left); lo_b = max(lo_b, qp_b - p.window_left); }

  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
  float o[HDV / 8][4];
#pragma unroll
  for (int i = 0; i < HDV / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

  const uint32_t sQ_u = smem_u32(sQ), sK_u = smem_u32(sK), sV_u = smem_u32(sV);

  for (int nb = n_lo; nb < n_hi; ++nb) {
    const int key0 = nb * BN;
    __syncthreads();   // previous block's smem reads are done (and Q stores are visible on the first pass)
    // ---- K, V tiles -> smem ----
    for (int i = tid; i < BN * (HD / 8); i += NTHREADS) {
      const int r = i / (HD / 8), c = (i % (HD / 8)) * 8;
      const int kk = key0 + r;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (kk < seqlen_k && c < p.hd) {
        int64_t off;
        if (p.page_table) {
          const int pg = p.page_table[(int64_t)b * p.page_table_stride + kk / p.page_size];
          off = (int64_t)pg * p.k_page_stride + (int64_t)(kk % p.page_size) * p.k_row_stride;
        } else {
          off = (int64_t)(k0 + kk) * p.k_row_stride;
        }
        val = load8<T>(p.k, off + (int64_t)hk * p.k_head_stride + c, p.kv_fp8);
      }
      store8(sK + r * LDQ + c, val);
    }
    for (int i = tid; i < BN * (HDV / 8); i += NTHREADS) {
      const int r = i / (HDV / 8), c = (i % (HDV / 8)) * 8;
      const int kk = key0 + r;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (kk < seqlen_k && c < p.hdv) {
        int64_t off;
        if (p.page_table) {
          const int pg = p.page_table[(int64_t)b * p.page_table_stride + kk / p.page_size];
          off = (int64_t)pg * p.v_page_stride + (int64_t)(kk % p.page_size) * p.v_row_stride;
        } else {
          off = (int64_t)(k0 + kk) * p.v_row_stride;
        }
        val = load8<T>(p.v, off + (int64_t)hk * p.v_head_stride + c, p.kv_fp8);
      }
      store8(sV + r * LDV + c, val);
    }
    __syncthreads();

    // ---- S = Q K^T (16 rows x 64 keys per warp) ----
    float s[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      uint32_t a[4];
      {
        const int r = warp * 16 + (lane & 15), c = ks * 16 + (lane >> 4) * 8;
        ldmatrix_x4(a, sQ_u + (uint32_t)(r * LDQ + c) * 2u);
      }
#pragma unroll
      for (int np = 0; np < BN / 16; ++np) {
        uint32_t bfr[4];
        const int mat = lane >> 3;
        const int r = np * 16 + (mat >> 1) * 8 + (lane & 7), c = ks * 16 + (mat & 1) * 8;
        ldmatrix_x4(bfr, sK_u + (uint32_t)(r * LDQ + c) * 2u);
        mma_16816<T>(s[2 * np], a, bfr[0], bfr[1]);
        mma_16816<T>(s[2 * np + 1], a, bfr[2], bfr[3]);
      }
    }

    // ---- scale / softcap / mask, online softmax ----
    float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kk = key0 + nt * 8 + 2 * (lane & 3) + (e & 1);
        const bool row_b = e >= 2;
        float y = s[nt][e];
        y = has_cap ? tanhf(y * cap_in) * y_scale : y * y_scale;
        const bool ok = row_b ? (kk >= lo_b && kk <= hi_b) : (kk >= lo_a && kk <= hi_a);
        y = ok ? y : -INFINITY;
        s[nt][e] = y;
        if (row_b) mx_b = fmaxf(mx_b, y); else mx_a = fmaxf(mx_a, y);
      }
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
    const float ms_a = (mn_a == -INFINITY) ? 0.f : mn_a, ms_b = (mn_b == -INFINITY) ? 0.f : mn_b;
    const float corr_a = ex2(m_a - ms_a), corr_b = ex2(m_b - ms_b);   // ex2(-inf) = 0 on the first block
    m_a = mn_a; m_b = mn_b;
    float ps_a = 0.f, ps_b = 0.f;
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
      s[nt][0] = ex2(s[nt][0] - ms_a); s[nt][1] = ex2(s[nt][1] - ms_a);
      s[nt][2] = ex2(s[nt][2] - ms_b); s[nt][3] = ex2(s[nt][3] - ms_b);
      ps_a += s[nt][0] + s[nt][1];
      ps_b += s[nt][2] + s[nt][3];
    }
    l_a = l_a * corr_a + ps_a;
    l_b = l_b * corr_b + ps_b;
#pragma unroll
    for (int i = 0; i < HDV / 8; ++i) { o[i][0] *= corr_a; o[i][1] *= corr_a; o[i][2] *= corr_b; o[i][3] *= corr_b; }

    // ---- O += P V ----
#pragma unroll
    for (int kk16 = 0; kk16 < BN / 16; ++kk16) {
      uint32_t a[4];
      a[0] = pack2<T>(s[2 * kk16][0], s[2 * kk16][1]);
      a[1] = pack2<T>(s[2 * kk16][2], s[2 * kk16][3]);
      a[2] = pack2<T>(s[2 * kk16 + 1][0], s[2 * kk16 + 1][1]);
      a[3] = pack2<T>(s[2 * kk16 + 1][2], s[2 * kk16 + 1][3]);
#pragma unroll
      for (int np = 0; np < HDV / 16; ++np) {
        uint32_t bfr[4];
        const int mat = lane >> 3;
        const int r = kk16 * 16 + (mat & 1) * 8 + (lane & 7), c = np * 16 + (mat >> 1) * 8;
        ldmatrix_x4_trans(bfr, sV_u + (uint32_t)(r * LDV + c) * 2u);
        mma_16816<T>(o[2 * np], a, bfr[0], bfr[1]);
        mma_16816<T>(o[2 * np + 1], a, bfr[2], bfr[3]);
      }
    }
  }

  // ---- epilogue ----
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);

#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int R = half ? R_b : R_a;
    float m = half ? m_b : m_a, l = half ? l_b : l_a;
    if (R >= rows_total) continue;
    const int token = R / rep, head = hk * rep + R % rep;
    const int64_t qi = q0 + token;
    if (p.nsplits > 1) {
      // partial: normalised by this split's own denominator; the sink joins in the combine
      const float inv = l > 0.f ? vds / l : 0.f;
      float* op = p.o_part + (((int64_t)split * p.total_q + qi) * p.hq + head) * p.hdv;
#pragma unroll
      for (int nt = 0; nt < HDV / 8; ++nt) {
        const int c = nt * 8 + 2 * (lane & 3);
        if (c < p.hdv) *reinterpret_cast<float2*>(op + c) = make_float2(o[nt][2 * half] * inv, o[nt][2 * half + 1] * inv);
      }
      if ((lane & 3) == 0)
        p.lse_part[((int64_t)split * p.hq + head) * p.total_q + qi] = l > 0.f ? (m + lg2(l)) * kLn2 : -INFINITY;
    } else {
      float osc = 1.f;
      if (p.s_aux) {
        const float ys = p.s_aux[head] * kLog2e;
        const float mn = fmaxf(m, ys);
        osc = (m == -INFINITY) ? 0.f : ex2(m - mn);
        l = l * osc + ex2(ys - mn);
        m = mn;
      }
      const float inv = l > 0.f ? osc * vds / l : 0.f;
      if (p.out_f32) {
        float* of = reinterpret_cast<float*>(p.out) + qi * p.o_row_stride + (int64_t)head * p.o_head_stride;
#pragma unroll
        for (int nt = 0; nt < HDV / 8; ++nt) {
          const int c = nt * 8 + 2 * (lane & 3);
          if (c < p.hdv) *reinterpret_cast<float2*>(of + c) = make_float2(o[nt][2 * half] * inv, o[nt][2 * half + 1] * inv);
        }
      } else {
        T* op = reinterpret_cast<T*>(p.out) + qi * p.o_row_stride + (int64_t)head * p.o_head_stride;
#pragma unroll
        for (int nt = 0; nt < HDV / 8; ++nt) {
          const int c = nt * 8 + 2 * (lane & 3);
          if (c < p.hdv)
            *reinterpret_cast<uint32_t*>(op + c) = pack2<T>(o[nt][2 * half] * inv, o[nt][2 * half + 1] * inv);
        }
      }
      if ((lane & 3) == 0) p.lse[(int64_t)head * p.total_q + qi] = l > 0.f ? (m + lg2(l)) * kLn2 : -INFINITY;
    }
  }
}

template <typename T, int HD, int HDV>
static int launch_t(const KParams& kp, cudaStream_t stream) {
  const size_t smem = (size_t)(BM * (HD + PAD) + BN * (HD + PAD) + BN * (HDV + PAD)) * sizeof(T);
  auto kern = fwd_general_kernel<T, HD, HDV>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int mtiles = (kp.max_seqlen_q * kp.rep + BM - 1) / BM;
  if (kp.hkv > 65535 || (long long)mtiles * kp.batch * kp.nsplits > 2147483647ll) return -1;
  dim3 grid((unsigned)(mtiles * kp.batch * kp.nsplits), kp.hkv, 1);
  kern<<<grid, NTHREADS, smem, stream>>>(kp);
  return (int)cudaGetLastError();
}

template <typename T>
static int launch_hd(const KParams& kp, cudaStream_t stream) {
  const int hd = kp.hd, hdv = kp.hdv;
  if (hd <= 64 && hdv <= 64) return launch_t<T, 64, 64>(kp, stream);
  if (hd <= 128 && hdv <= 128) return launch_t<T, 128, 128>(kp, stream);
  if (hd <= 192 && hdv <= 128) return launch_t<T, 192, 128>(kp, stream);
  if (hd <= 256 && hdv <= 256) return launch_t<T, 256, 256>(kp, stream);
  return -1;
}

}  // namespace general

// compute type: fp16 inputs -> fp16 MMA; bf16 and fp8 inputs -> bf16 MMA (fp8 values are exact in bf16)
int launch_general(const KParams& kp, int dtype, int /*out_dtype*/, int /*num_sms*/, cudaStream_t stream) {
  if (dtype == FA_DT_FP16) return general::launch_hd<__half>(kp, stream);
  return general::launch_hd<__nv_bfloat16>(kp, stream);
}

}  // namespace fa
