// fa_decode.cu — paged-KV decode: a bandwidth-bound streaming kernel.
//
// Work item = (batch entry and 16-row tile, kv head, split).  The `rep * q_len` query rows that share one KV head
// are packed into 16-row MMA tiles: with up to 16 rows every K/V byte is read from HBM once per kv head, with
// more rows (up to 64) once per tile.  Persistent CTAs
// (one per SM) pull work items longest-first from the scheduler metadata through an atomic counter.
//
//   warp 4      producer: resolves page-table entries (32 at a time, one coalesced load) and streams whole
//               pages with TMA 2-D boxes over the page pool viewed as [num_pages * page_size, hkv * hd] into a
//               ring of 32 KB stages (64 keys of 16-bit K+V, or 128 keys of e4m3 K+V; 128-byte swizzle).  The ring runs on across
//               work-item boundaries; each stage carries a small descriptor (work id, first key, flags).  Pages
//               of 1, 2 or 4 keys are fetched with cp.async, 16 bytes per lane, into the same swizzled layout.
//   warps 0-3   consumers: each takes a quarter of the stage's keys: S = Q K^T and O += P V with warp-level
//               MMA (ldmatrix from the swizzled stage), a private online softmax, and at the end of the work
//               item a cross-warp merge through shared memory.
// The tensor cores are incidental here: the roofline is HBM, the design goal is bytes in flight.
//
// Plays the role of `fwd_kernel_ws_paged` + `launch_ws_paged` of the reference
// (kernels/fa4_blackwell.cu:8774-9103, 9605-9993), with per-batch leftpad and fp8 KV (descale folded in).
#include <cuda.h>

#include <atomic>
#include <mutex>

#include "fa_internal.h"
#include "fa_sched.h"
#include "ptx.cuh"

namespace fa {
namespace dec {

constexpr int TN = 64;                 // keys per scheduler block (metadata unit); a stage holds TNS keys
// Consumer warps per CTA.  A 16-bit cache runs one CTA per SM; an e4m3 cache runs TWO (half-size stages): every
// consumer warp works on every stage, so one CTA's stage rate is bounded by the latency of one warp's
// ldmatrix -> widen -> MMA -> softmax -> MMA chain, and with twice the keys per byte that chain, not HBM, was the
// limit; a second CTA's chain runs beside it.
constexpr int ncons_for(int) { return 4; }
constexpr int ctas_per_sm(int esz) { return esz == 1 ? 2 : 1; }
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
enum Role : unsigned { ROLE_PRODUCER = 5, ROLE_CONSUMER = 6 };
enum : int { F_FIRST = 1, F_LAST = 2, F_EMPTY = 4 };

struct DecArgs {
  KParams kp;
  int total_work;     // num_work * hkv * nsplits
  int box_rows;       // rows per TMA box = min(page_size, 64); 1 in gather mode
  int kv_total_rows;
  int gather;         // pages of 1, 2 or 4 keys: rows are fetched 16 bytes per lane with cp.async
};

template <int ESZ, int NST, int HD, int HDV, int TNS_>
struct Smem {
  static constexpr int TNS = TNS_;                  // keys per stage (64, or 128: two independent 16-key chains per warp)
  static constexpr int NC = ncons_for(ESZ);         // consumer warps; 16 keys per warp and stage either way
  static constexpr int kKBytes = TNS * HD * ESZ, kVBytes = TNS * HDV * ESZ;
  static constexpr int kStage = kKBytes + kVBytes;
  static constexpr int kRing = NST * kStage;
  static constexpr int kInfoOff = kRing;                       // NST x int4
  static constexpr int kBarOff = kInfoOff + NST * 16;          // full[NST], empty[NST]
  static constexpr int kMiscOff = kBarOff + 2 * NST * 8;       // abort flags
  static constexpr int kScrOff = (kMiscOff + 16 + 15) / 16 * 16;
  static constexpr int kLdO = HDV + 4;
  static constexpr int kScrBytes = NC * 16 * kLdO * 4 + 3 * NC * 16 * 4;
  static constexpr int kBytes = kScrOff + kScrBytes;
};

template <int NC>
__device__ __forceinline__ void bar_consumers() { asm volatile("bar.sync 1, %0;" ::"n"(NC * 32) : "memory"); }

struct WorkItem {
  int b, mt, hk, split, lo, hi;   // mt: which 16 of the rep*q_len packed rows; key-block range [lo, hi) in units of TN keys
  int seqlen_q, seqlen_k, q0, k0, leftpad;   // k0: first row of this sequence in a contiguous (unpaged) K/V
  bool valid;
  bool bad;     // the entry names a batch or a key range that this problem does not have
};

// Entry e of the work list -> work item.  The list may come from the caller: an entry is used only if its batch
// index and key-block range lie inside this problem (else `bad`, and nothing is dereferenced with it).
__device__ __forceinline__ WorkItem decode_work(const KParams& p, int w) {
  WorkItem it;
  const int per_entry = p.hkv * p.nsplits;
  const int e = w / per_entry, rem = w - e * per_entry;
  it.hk = rem / p.nsplits;
  it.split = rem - it.hk * p.nsplits;
  const int32_t* ent = p.work + kSchedHeader + 4 * e;
  it.b = ent[0];
  it.mt = ent[1] > 0 ? ent[1] : 0;
  it.valid = it.b >= 0;
  it.bad = false;
  it.lo = it.hi = 0;
  it.seqlen_q = it.seqlen_k = it.q0 = it.k0 = it.leftpad = 0;
  if (it.valid) {
    if (it.b >= p.batch || it.mt >= p.work_expect.max_mtiles) { it.valid = false; it.bad = true; return it; }
    it.q0 = p.cu_q[it.b];
    it.seqlen_q = p.cu_q[it.b + 1] - it.q0;
    it.k0 = p.page_table ? 0 : p.cu_k[it.b];
    it.seqlen_k = p.seqused_k ? p.seqused_k[it.b] : (p.cu_k[it.b + 1] - p.cu_k[it.b]);
    it.leftpad = p.leftpad_k ? p.leftpad_k[it.b] : 0;
    const int n_lo = ent[2], n_hi = ent[3];
    if (n_lo < 0 || n_hi < n_lo || (int64_t)n_hi * TN > (int64_t)it.seqlen_k + TN - 1) { it.valid = false; it.bad = true; return it; }
    split_range(n_lo, n_hi, it.split, p.nsplits, &it.lo, &it.hi);
  }
  return it;
}

// The cp.async producer's copies of one operand (K or V) of a stage: TNS rows of CPR 16-byte chunks, row r from
// pool row yr[r / 32] of lane r % 32, written where a 128-byte-swizzled TMA box would have put them (column block
// ch / 8 of the stage, row r, chunk (ch % 8) ^ (r % 8)).
template <int CPR, int TNS>
__device__ __forceinline__ void copy_rows(uint32_t dst0, const unsigned char* src0, uint32_t pitch,
                                          const int (&yr)[TNS / 32], int lane) {
  if constexpr (32 % CPR == 0) {
    // RPI rows per instruction; row r = i * RPI + hb, and (r & 7) = ((i * RPI) & 7) ^ hb because the low bits of
    // i * RPI are clear: the swizzle term splits into a lane constant and an immediate
    constexpr int RPI = 32 / CPR;
    const int hb = lane / CPR, ch = lane - hb * CPR;
    const uint32_t dl = dst0 + (uint32_t)(ch >> 3) * (TNS * 128) + (uint32_t)hb * 128u;
    const uint32_t xs = (uint32_t)(((ch & 7) ^ hb) << 4);
    const unsigned char* sl = src0 + ch * 16;
    // the row numbers of eight copies are fetched first: a shuffle followed at once by its copy would cost the
    // shuffle's latency per copy (the statements are not reordered)
    constexpr int G = 8;
    static_assert((TNS / RPI) % G == 0, "whole groups");
#pragma unroll
    for (int i0 = 0; i0 < TNS / RPI; i0 += G) {
      int y[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const int i = i0 + g;
        y[g] = __shfl_sync(0xffffffffu, yr[(i * RPI) >> 5], ((i * RPI) & 31) + hb);
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const int i = i0 + g;
        cp_async16(dl + (uint32_t)(i * RPI) * 128u + (xs ^ (uint32_t)(((i * RPI) & 7) << 4)),
                   sl + (uint64_t)(uint32_t)y[g] * pitch, 16u);
      }
    }
  } else {
    constexpr int N = TNS * CPR / 32, G = 8;
    static_assert(N % G == 0, "whole groups");
#pragma unroll
    for (int i0 = 0; i0 < N; i0 += G) {
      int y[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const int i = i0 + g, r = (i * 32 + lane) / CPR;
        y[g] = __shfl_sync(0xffffffffu, yr[(i * 32 / CPR) >> 5], r & 31);
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const int q = (i0 + g) * 32 + lane, r = q / CPR, ch = q - r * CPR;
        cp_async16(dst0 + (uint32_t)(ch >> 3) * (TNS * 128) + (uint32_t)r * 128u + (uint32_t)(((ch & 7) ^ (r & 7)) << 4),
                   src0 + (uint64_t)(uint32_t)y[g] * pitch + ch * 16, 16u);
      }
    }
  }
}

// T = MMA element type (bf16 / fp16); KV8 = the cache holds e4m3 bytes.
template <typename T, bool KV8, int NST, int HD, int HDV, int CPS, int TNS_>
__global__ void __launch_bounds__((ncons_for(KV8 ? 1 : 2) + 1) * 32, CPS)
fwd_decode_kernel(const DecArgs a, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v) {
  constexpr int ESZ = KV8 ? 1 : 2;
  static_assert(!KV8 || (HD == 128 && HDV == 128), "an e4m3 cache row must fill one 128-byte swizzle row");
  static_assert(HD % 64 == 0 && HDV % 64 == 0, "whole 128-byte column blocks");
  using SM = Smem<ESZ, NST, HD, HDV, TNS_>;
  static_assert(!(TNS_ != 64 && !KV8), "the 16-bit consumers take 16 keys per warp and stage");
  // 16-bit cache: m16n8k16 MMA in the cache's type.  e4m3 cache: the bytes are widened to fp16 in registers (exact,
  // one conversion per two elements) and fed to the fp16 m16n8k16 MMA; Q rows are scaled into fp16 range with a
  // per-row factor (undone in the softmax scale), P is fp16.  (The warp-level e4m3 MMA is not used: on sm_100a
  // it runs on the fp16 sub-pipe with both operands unpacked again for every instruction, which measured
  // 4 x the instructions of this path's 16-bit sibling per key.)
  using TM = typename std::conditional<KV8, __half, T>::type;
  constexpr int TNS = SM::TNS;            // keys per stage
  constexpr int NC = SM::NC;
  constexpr int WK = TNS / NC;            // keys per consumer warp and stage: 16
  constexpr int NT = WK / 8;              // 8-key MMA column tiles per warp
  const KParams& p = a.kp;
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* sm = smem_dyn + (base - raw);
  const uint32_t bar_full = base + SM::kBarOff, bar_empty = bar_full + 8 * NST;
  volatile int* s_info = reinterpret_cast<volatile int*>(sm + SM::kInfoOff);   // 4 ints per stage
  volatile int* s_abort = reinterpret_cast<volatile int*>(sm + SM::kMiscOff);
  float* s_o = reinterpret_cast<float*>(sm + SM::kScrOff);
  float* s_m = s_o + NC * 16 * SM::kLdO;
  float* s_l = s_m + NC * 16;
  float* s_lr = s_l + NC * 16;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    // cp.async stages complete on 33 arrivals: one per producer lane when its copies have landed, one from lane 0
    // after it has written the stage's descriptor
    for (int s = 0; s < NST; ++s) { mbar_init(bar_full + 8 * s, a.gather ? 33 : 1); mbar_init(bar_empty + 8 * s, NC); }
    s_abort[0] = 0; s_abort[1] = 0;
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == NC) {
    // ============================================ producer ============================================
    if (lane == 0) { tma_prefetch_desc(&map_k); tma_prefetch_desc(&map_v); }
    uint32_t cnt = 0;
    bool ok = true;
    const bool paged = p.page_table != nullptr;
    const int ps = paged ? p.page_size : TNS;   // contiguous K/V: "pages" of one stage, at rows k0 + key (page_shift is -1 then)
    const int boxes = TNS / a.box_rows;         // TMA boxes per stage and 128-byte column block
    // the list's header must describe this call before any entry is read
    int total_work = a.total_work;
    if (!sched_header_matches(p.work, p.work_expect)) {
      if (lane == 0) report_error(p.status, DEV_ERR_BAD_INDEX, ROLE_PRODUCER);
      total_work = 0;
    }
    bool first_ticket = true;
    // a stage that carries no copies: lane 0 has written its descriptor
    auto publish_plain = [&](uint32_t s) {
      if (a.gather) mbar_arrive(bar_full + 8 * s);
      if (lane == 0) mbar_arrive(bar_full + 8 * s);
    };
    while (ok) {
      int w = 0;
      if (first_ticket) w = (int)blockIdx.x;     // a CTA's first work id is its block index, later ones are tickets
      else if (lane == 0) w = (int)gridDim.x + atomicAdd(p.counters, 1);
      if (!first_ticket) w = __shfl_sync(0xffffffffu, w, 0);
      first_ticket = false;
      if (w >= total_work) break;
      const WorkItem it = decode_work(p, w);
      if (it.bad) {
        if (lane == 0) report_error(p.status, DEV_ERR_BAD_INDEX, ROLE_PRODUCER);
        break;
      }
      if (!it.valid) continue;
      if (it.lo >= it.hi) {   // nothing to stream: one descriptor-only stage so that the output still gets written
        const uint32_t s = cnt % NST;
        ok = wait_or_abort(bar_empty + 8 * s, ((cnt / NST) & 1) ^ 1, s_abort);
        if (!ok) break;
        if (lane == 0) { s_info[4 * s] = w; s_info[4 * s + 1] = 0; s_info[4 * s + 2] = F_FIRST | F_LAST | F_EMPTY; }
        publish_plain(s);
        ++cnt;
        continue;
      }
      const int npages = (it.seqlen_k + ps - 1) / ps;
      int cache_first = -1, cache_id = 0;       // 32 page-table entries, one per lane
      const int key_end = it.hi * TN;
      if (a.gather) {
        // Pages of 1, 2 or 4 keys, 16 bytes per lane: lane g looks up the physical rows of keys g, g + 32, .. of
        // a stage (one stage ahead, so that the lookups are in flight while the current stage is issued), then the
        // warp walks the stage's 16-byte chunks in row order, CPR consecutive lanes on one row, and writes them
        // where the swizzled TMA box would have put them.  The TMA unit retires about one copy per 100 cycles
        // whatever its size; these copies go through the load/store path instead (the reference's route for page
        // size 1, kernels/fa4_blackwell.cu:8936-8947).  Keys beyond the sequence fetch pool row 0 and are masked
        // by the consumers.
        const int32_t* pt = p.page_table + (int64_t)it.b * p.page_table_stride;
        constexpr int RG = TNS / 32;
        auto lookup = [&](int key0, int (&yr)[RG]) {
#pragma unroll
          for (int u = 0; u < RG; ++u) {
            const int kk = key0 + 32 * u + lane;
            yr[u] = 0;
            if (kk < it.seqlen_k && kk < key_end) {
              const int lp = kk >> p.page_shift;
              yr[u] = (pt[lp] << p.page_shift) + (kk - (lp << p.page_shift));
            }
          }
        };
        const unsigned char* kb = reinterpret_cast<const unsigned char*>(p.k) + (int64_t)it.hk * HD * ESZ;
        const unsigned char* vb = reinterpret_cast<const unsigned char*>(p.v) + (int64_t)it.hk * HDV * ESZ;
        const uint32_t kpitch = (uint32_t)(p.k_row_stride * ESZ), vpitch = (uint32_t)(p.v_row_stride * ESZ);
        int ynext[RG];
        lookup(it.lo * TN, ynext);
        for (int key0 = it.lo * TN; key0 < key_end && ok; key0 += TNS) {
          int ycur[RG];
#pragma unroll
          for (int u = 0; u < RG; ++u) ycur[u] = ynext[u];
          if (key0 + TNS < key_end) lookup(key0 + TNS, ynext);
          const uint32_t s = cnt % NST;
          ok = wait_or_abort(bar_empty + 8 * s, ((cnt / NST) & 1) ^ 1, s_abort);
          if (!ok) break;
          const uint32_t kdst = base + s * SM::kStage, vdst = kdst + SM::kKBytes;
          if (lane == 0) {
            int flags = 0;
            if (key0 == it.lo * TN) flags |= F_FIRST;
            if (key0 + TNS >= key_end) flags |= F_LAST;
            s_info[4 * s] = w; s_info[4 * s + 1] = key0; s_info[4 * s + 2] = flags;
            mbar_arrive(bar_full + 8 * s);
          }
          copy_rows<HD * ESZ / 16, TNS>(kdst, kb, kpitch, ycur, lane);
          copy_rows<HDV * ESZ / 16, TNS>(vdst, vb, vpitch, ycur, lane);
          cp_async_arrive_noinc(bar_full + 8 * s);
          ++cnt;
        }
        continue;
      }
      for (int key0 = it.lo * TN; key0 < key_end && ok; key0 += TNS) {
        const int lp0 = key0 / ps;              // first logical page of this stage
        if (paged && (cache_first < 0 || lp0 < cache_first || lp0 + boxes > cache_first + 32)) {
          cache_first = lp0;
          const int lp = lp0 + lane;
          cache_id = lp < npages ? p.page_table[(int64_t)it.b * p.page_table_stride + lp] : -1;
        }
        const uint32_t s = cnt % NST;
        ok = wait_or_abort(bar_empty + 8 * s, ((cnt / NST) & 1) ^ 1, s_abort);
        if (!ok) break;
        const uint32_t kdst = base + s * SM::kStage, vdst = kdst + SM::kKBytes;
        if (lane == 0) {
          int flags = 0;
          if (key0 == it.lo * TN) flags |= F_FIRST;
          if (key0 + TNS >= key_end) flags |= F_LAST;
          s_info[4 * s] = w; s_info[4 * s + 1] = key0; s_info[4 * s + 2] = flags;
          mbar_expect_tx(bar_full + 8 * s, SM::kStage);
        }
        // one copy per (box, 128-byte column block, K or V); the lanes share them out
        constexpr int EPB = KV8 ? 128 : 64;              // elements per 128-byte column block
        constexpr int KCB = HD / EPB, VCB = HDV / EPB, OPB = KCB + VCB;
        const int nops = boxes * OPB;
        for (int o0 = 0; o0 < nops; o0 += 32) {
          const int o = o0 + lane;
          const bool act = o < nops;
          const int j = act ? o / OPB : 0, c = o - j * OPB;
          const int kk = key0 + j * a.box_rows;
          const int lp = p.page_shift >= 0 ? (kk >> p.page_shift) : kk / ps;
          const int pid = paged ? __shfl_sync(0xffffffffu, cache_id, (lp - cache_first) & 31) : 0;
          if (act) {
            int y = a.kv_total_rows;                 // out of range: TMA fills zeros
            if (kk < it.seqlen_k && kk < key_end && pid >= 0) y = paged ? pid * ps + (kk - lp * ps) : it.k0 + kk;
            const uint32_t roff = (uint32_t)(j * a.box_rows) * 128u;
            if (c < KCB) tma_load_2d(kdst + c * (TNS * 128) + roff, &map_k, it.hk * HD + c * EPB, y, bar_full + 8 * s);
            else tma_load_2d(vdst + (c - KCB) * (TNS * 128) + roff, &map_v, it.hk * HDV + (c - KCB) * EPB, y, bar_full + 8 * s);
          }
        }
        ++cnt;
      }
    }
    if (!ok) { if (lane == 0) { report_error(p.status, DEV_ERR_TIMEOUT, ROLE_PRODUCER); s_abort[0] = 1; } }
    if (ok) {   // end-of-stream marker
      const uint32_t s = cnt % NST;
      if (wait_or_abort(bar_empty + 8 * s, ((cnt / NST) & 1) ^ 1, s_abort)) {
        if (lane == 0) s_info[4 * s] = -1;
        publish_plain(s);
        ++cnt;
      }
    }
    // every copy issued must have landed before the CTA may leave
    if (lane == 0) {
      for (uint32_t s = 0; s < (uint32_t)NST; ++s)
        if (cnt > s) wait_or_abort(bar_full + 8 * s, ((cnt - 1 - s) / NST) & 1, s_abort + 1);
      counters_release(p.counters);   // this CTA takes no more tickets
    }
  } else {
    // ============================================ consumers ===========================================
    const int g = lane >> 2, tq = lane & 3;
    const int rep = p.rep;
    uint32_t cnt = 0;
    bool ok = true;
    uint32_t qf[HD / 16][4];   // A operand of 8 k-steps of 16
    float qs_a = 1.f, qs_b = 1.f;   // e4m3 Q: 1 / (row quantisation scale), folded into the logit scale
    float o[HDV / 8][4];
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    float lr_a = 0.f, lr_b = 0.f;   // e4m3 cache: sums of the ROUNDED probabilities (normalise O); l_* stay exact for the LSE
    int lo_a = 0, hi_a = -1, lo_b = 0, hi_b = -1, lo_max = 0, hi_min = -1;
    float c_mul = 0.f, cap_in = 0.f, vds = 1.f;
    WorkItem it{};
    const bool has_cap = p.softcap > 0.f;

    while (true) {
      const uint32_t s = cnt % NST;
      ok = wait_or_abort(bar_full + 8 * s, (cnt / NST) & 1, s_abort);
      if (!ok) { report_error(p.status, DEV_ERR_TIMEOUT, ROLE_CONSUMER); s_abort[0] = 1; break; }
      const int4 info = make_int4(s_info[4 * s], s_info[4 * s + 1], s_info[4 * s + 2], 0);
      if (info.x < 0) break;
      const int key0 = info.y, flags = info.z;
      if (flags & F_FIRST) {
        it = decode_work(p, info.x);
        const int rows_total = it.seqlen_q * rep;
        // Q fragments straight from global memory (rows g and g+8 of the packed tile)
        if constexpr (!KV8) {
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {      // A operand of m16n8k16: columns ks*16 + 2*tq (+8)
              const int R = it.mt * 16 + g + (e & 1) * 8;
              const int c = ks * 16 + 2 * tq + (e >> 1) * 8;
              uint32_t v = 0;
              if (R < rows_total) {
                const int token = R / rep, head = it.hk * rep + R % rep;
                v = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const T*>(p.q) +
                                                       (int64_t)(it.q0 + token) * p.q_row_stride +
                                                       (int64_t)head * p.q_head_stride + c);
              }
              qf[ks][e] = v;
            }
          }
        } else {
          // A operand of m16n8k16 in fp16.  The K bytes reach a lane as 4 consecutive head-dim positions of one key
          // (see the QK loop), so k-step ks contracts positions 16ks + {4tq, 4tq+1 | 4tq+2, 4tq+3} in its two halves;
          // Q is gathered in the same order (a sum does not care about the order of its terms).  Each row is
          // scaled so that its largest magnitude is 256 before conversion to fp16.
          float qv[2][HD / 16][4];
          float amax[2] = {0.f, 0.f};
#pragma unroll
          for (int rr = 0; rr < 2; ++rr) {
            const int R = it.mt * 16 + g + rr * 8;
            const bool live = R < rows_total;
            const int token = R / rep, head = it.hk * rep + R % rep;
            const T* qrow = reinterpret_cast<const T*>(p.q) + (int64_t)(it.q0 + (live ? token : 0)) * p.q_row_stride +
                            (int64_t)(live ? head : 0) * p.q_head_stride;
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
              uint2 raw = make_uint2(0u, 0u);
              if (live) raw = *reinterpret_cast<const uint2*>(qrow + ks * 16 + 4 * tq);
              float f[4];
              if (std::is_same<T, __nv_bfloat16>::value) {
                f[0] = __uint_as_float(raw.x << 16); f[1] = __uint_as_float(raw.x & 0xffff0000u);
                f[2] = __uint_as_float(raw.y << 16); f[3] = __uint_as_float(raw.y & 0xffff0000u);
              } else {
                const float2 lo2 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
                const float2 hi2 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                f[0] = lo2.x; f[1] = lo2.y; f[2] = hi2.x; f[3] = hi2.y;
              }
#pragma unroll
              for (int j = 0; j < 4; ++j) { qv[rr][ks][j] = f[j]; amax[rr] = fmaxf(amax[rr], fabsf(f[j])); }
            }
          }
#pragma unroll
          for (int rr = 0; rr < 2; ++rr) {
            amax[rr] = fmaxf(amax[rr], __shfl_xor_sync(0xffffffffu, amax[rr], 1));
            amax[rr] = fmaxf(amax[rr], __shfl_xor_sync(0xffffffffu, amax[rr], 2));
          }
          const float sq_a = amax[0] > 0.f ? 256.f / amax[0] : 1.f, sq_b = amax[1] > 0.f ? 256.f / amax[1] : 1.f;
          qs_a = 1.f / sq_a; qs_b = 1.f / sq_b;
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {
            qf[ks][0] = pack2<__half>(qv[0][ks][0] * sq_a, qv[0][ks][1] * sq_a);
            qf[ks][1] = pack2<__half>(qv[1][ks][0] * sq_b, qv[1][ks][1] * sq_b);
            qf[ks][2] = pack2<__half>(qv[0][ks][2] * sq_a, qv[0][ks][3] * sq_a);
            qf[ks][3] = pack2<__half>(qv[1][ks][2] * sq_b, qv[1][ks][3] * sq_b);
          }
        }
        float sc = p.scale;
        vds = 1.f;
        const int di = it.b * p.descale_batch_stride + it.hk * p.descale_head_stride;
        if (p.q_descale) sc *= p.q_descale[di];
        if (p.k_descale) sc *= p.k_descale[di];
        if (p.v_descale) vds = p.v_descale[di];
        c_mul = has_cap ? p.softcap * kLog2e : sc * kLog2e;
        cap_in = has_cap ? sc / p.softcap : 0.f;
        const int off = it.seqlen_k - it.seqlen_q;
        const int rb = it.mt * 16;                   // first packed row of this work item
        const int qp_a = off + (rb + g) / rep, qp_b = off + (rb + g + 8) / rep;
        lo_a = lo_b = it.leftpad;
        hi_a = hi_b = min(it.seqlen_k, it.hi * TN) - 1;   // keys past this split's range are not ours
        if (p.is_causal) { hi_a = min(hi_a, qp_a); hi_b = min(hi_b, qp_b); }
        if (p.window_right >= 0) { hi_a = min(hi_a, qp_a + p.window_right); hi_b = min(hi_b, qp_b + p.window_right); }
        if (p.window_left >= 0) { lo_a = max(lo_a, qp_a - p.window_left); lo_b = max(lo_b, qp_b - p.window_left); }
        // bounds valid for all 16 rows (rows past rows_total included: conservative)
        const int qp_lo = off + rb / rep, qp_hi = off + (rb + 15) / rep;
        lo_max = it.leftpad; hi_min = min(it.seqlen_k, it.hi * TN) - 1;
        if (p.is_causal) hi_min = min(hi_min, qp_lo);
        if (p.window_right >= 0) hi_min = min(hi_min, qp_lo + p.window_right);
        if (p.window_left >= 0) lo_max = max(lo_max, qp_hi - p.window_left);
        m_a = m_b = -INFINITY; l_a = l_b = 0.f; lr_a = lr_b = 0.f;
#pragma unroll
        for (int i = 0; i < HDV / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
      }

      if (!(flags & F_EMPTY)) {
        const uint32_t kb = base + s * SM::kStage, vb = kb + SM::kKBytes;
        const int mat = lane >> 3, l7 = lane & 7;
        float sacc[NT][4];
#pragma unroll
        for (int i = 0; i < NT; ++i) { sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f; }
        if constexpr (!KV8) {
          const uint32_t krow = kb + (uint32_t)(warp * WK + (mat >> 1) * 8 + l7) * 128u;
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {
            uint32_t bfr[4];
            const uint32_t chunk = (uint32_t)((ks * 2 + (mat & 1)) & 7);
            ldmatrix_x4(bfr, krow + (ks >> 2) * (TNS * 128) + ((chunk ^ (uint32_t)l7) << 4));
            mma_16816<TM>(sacc[0], qf[ks], bfr[0], bfr[1]);
            mma_16816<TM>(sacc[1], qf[ks], bfr[2], bfr[3]);
          }
        } else {
          // e4m3 rows are 128 bytes: one swizzle row per key.  ldmatrix moves 16-byte chunks, so lane (g, tq)
          // receives bytes 4tq..4tq+3 of key g; widened to two fp16 pairs they are the B operand of one k-step.
#pragma unroll
          for (int hf = 0; hf < WK / 16; ++hf) {
            const uint32_t krow = kb + (uint32_t)(warp * WK + hf * 16 + (mat >> 1) * 8 + l7) * 128u;
#pragma unroll
            for (int k32 = 0; k32 < HD / 32; ++k32) {
              uint32_t raw4[4];
              const uint32_t chunk = (uint32_t)(k32 * 2 + (mat & 1));
              ldmatrix_x4(raw4, krow + ((chunk ^ (uint32_t)l7) << 4));
              uint32_t b[4][2];
#pragma unroll
              for (int m = 0; m < 4; ++m) e4m3x4_to<__half>(raw4[m], b[m][0], b[m][1]);
              mma_16816<__half>(sacc[2 * hf], qf[2 * k32], b[0][0], b[0][1]);
              mma_16816<__half>(sacc[2 * hf], qf[2 * k32 + 1], b[1][0], b[1][1]);
              mma_16816<__half>(sacc[2 * hf + 1], qf[2 * k32], b[2][0], b[2][1]);
              mma_16816<__half>(sacc[2 * hf + 1], qf[2 * k32 + 1], b[3][0], b[3][1]);
            }
          }
        }
        // ---- mask + online softmax over this warp's keys ----
        const int kbase = key0 + warp * WK;
        const bool full = (kbase >= lo_max) && (kbase + WK - 1 <= hi_min);
        const float cm_a = c_mul * (has_cap ? 1.f : qs_a), cm_b = c_mul * (has_cap ? 1.f : qs_b);
        const float ci_a = cap_in * qs_a, ci_b = cap_in * qs_b;
        float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float y = sacc[nt][e];
            if (e >= 2) y = has_cap ? tanh_fast(y * ci_b) * c_mul : y * cm_b;
            else y = has_cap ? tanh_fast(y * ci_a) * c_mul : y * cm_a;
            if (!full) {
              const int kk = kbase + nt * 8 + 2 * tq + (e & 1);
              const bool okk = e >= 2 ? (kk >= lo_b && kk <= hi_b) : (kk >= lo_a && kk <= hi_a);
              y = okk ? y : -INFINITY;
            }
            sacc[nt][e] = y;
            if (e >= 2) mx_b = fmaxf(mx_b, y); else mx_a = fmaxf(mx_a, y);
          }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
        const float ms_a = mn_a == -INFINITY ? 0.f : mn_a, ms_b = mn_b == -INFINITY ? 0.f : mn_b;
        const float corr_a = ex2(m_a - ms_a), corr_b = ex2(m_b - ms_b);
        m_a = mn_a; m_b = mn_b;
        float ps_a = 0.f, ps_b = 0.f;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          sacc[nt][0] = ex2(sacc[nt][0] - ms_a); sacc[nt][1] = ex2(sacc[nt][1] - ms_a);
          sacc[nt][2] = ex2(sacc[nt][2] - ms_b); sacc[nt][3] = ex2(sacc[nt][3] - ms_b);
          ps_a += sacc[nt][0] + sacc[nt][1];
          ps_b += sacc[nt][2] + sacc[nt][3];
        }
        l_a = l_a * corr_a + ps_a;
        l_b = l_b * corr_b + ps_b;
        if constexpr (KV8) { lr_a = l_a; lr_b = l_b; }   // P is fp16: one sum serves the LSE and the normalisation
        if (__any_sync(0xffffffffu, corr_a != 1.f || corr_b != 1.f)) {
#pragma unroll
          for (int i = 0; i < HDV / 8; ++i) { o[i][0] *= corr_a; o[i][1] *= corr_a; o[i][2] *= corr_b; o[i][3] *= corr_b; }
        }
        // ---- O += P V ----
        if constexpr (!KV8) {
          uint32_t pa[4];
          pa[0] = pack2<TM>(sacc[0][0], sacc[0][1]);
          pa[1] = pack2<TM>(sacc[0][2], sacc[0][3]);
          pa[2] = pack2<TM>(sacc[1][0], sacc[1][1]);
          pa[3] = pack2<TM>(sacc[1][2], sacc[1][3]);
          const uint32_t vrow = vb + (uint32_t)(warp * WK + (mat & 1) * 8 + l7) * 128u;
#pragma unroll
          for (int np = 0; np < HDV / 16; ++np) {
            uint32_t bfr[4];
            const uint32_t chunk = (uint32_t)((np * 2 + (mat >> 1)) & 7);
            ldmatrix_x4_trans(bfr, vrow + (np >> 2) * (TNS * 128) + ((chunk ^ (uint32_t)l7) << 4));
            mma_16816<TM>(o[2 * np], pa, bfr[0], bfr[1]);
            mma_16816<TM>(o[2 * np + 1], pa, bfr[2], bfr[3]);
          }
        } else {
          // P as the fp16 A operand, one k-step of 16 keys at a time.
          // V: the B operand needs pairs of KEYS of one value column per register, i.e. bytes of different rows.
          // ldmatrix.trans on 16-bit units hands lane (g, tq) the byte pairs (columns 2g, 2g+1) of keys 2tq and
          // 2tq+1 of each 8-key group; one byte permute per register pair gathers, for the even and for the odd
          // column, keys {2tq, 2tq+1, 8+2tq, 9+2tq}: widened to fp16 these are b0 and b1 of the k-step.
          // Accumulator tile 2c therefore holds value columns 16c + {0,2,..,14} and tile 2c+1 the odd ones (undone
          // when the result is written out).  One ldmatrix covers the 16 keys of two 16-column chunks.
#pragma unroll
          for (int hf = 0; hf < WK / 16; ++hf) {
            uint32_t pa[4];
            pa[0] = pack2<__half>(sacc[2 * hf][0], sacc[2 * hf][1]);
            pa[1] = pack2<__half>(sacc[2 * hf][2], sacc[2 * hf][3]);
            pa[2] = pack2<__half>(sacc[2 * hf + 1][0], sacc[2 * hf + 1][1]);
            pa[3] = pack2<__half>(sacc[2 * hf + 1][2], sacc[2 * hf + 1][3]);
            const uint32_t vrow = vb + (uint32_t)(warp * WK + hf * 16 + (mat & 1) * 8 + l7) * 128u;
#pragma unroll
            for (int c2 = 0; c2 < HDV / 32; ++c2) {
              uint32_t r4[4];
              ldmatrix_x4_trans(r4, vrow + (((uint32_t)(2 * c2 + (mat >> 1)) ^ (uint32_t)l7) << 4));
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const int c = 2 * c2 + h;
                uint32_t ev, od, be0, be1, bo0, bo1;
                asm("prmt.b32 %0, %1, %2, 0x6420;" : "=r"(ev) : "r"(r4[2 * h]), "r"(r4[2 * h + 1]));
                asm("prmt.b32 %0, %1, %2, 0x7531;" : "=r"(od) : "r"(r4[2 * h]), "r"(r4[2 * h + 1]));
                e4m3x4_to<__half>(ev, be0, be1);
                e4m3x4_to<__half>(od, bo0, bo1);
                mma_16816<__half>(o[2 * c], pa, be0, be1);
                mma_16816<__half>(o[2 * c + 1], pa, bo0, bo1);
              }
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_empty + 8 * s);
      ++cnt;

      if (flags & F_LAST) {
        // ---- merge the four warps' partial results and write the output rows ----
        l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
        l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
        lr_a += __shfl_xor_sync(0xffffffffu, lr_a, 1); lr_a += __shfl_xor_sync(0xffffffffu, lr_a, 2);
        lr_b += __shfl_xor_sync(0xffffffffu, lr_b, 1); lr_b += __shfl_xor_sync(0xffffffffu, lr_b, 2);
        float* so = s_o + warp * 16 * SM::kLdO;
        if (!KV8) {
#pragma unroll
          for (int nt = 0; nt < HDV / 8; ++nt) {
            *reinterpret_cast<float2*>(so + g * SM::kLdO + nt * 8 + 2 * tq) = make_float2(o[nt][0], o[nt][1]);
            *reinterpret_cast<float2*>(so + (g + 8) * SM::kLdO + nt * 8 + 2 * tq) = make_float2(o[nt][2], o[nt][3]);
          }
        } else {
#pragma unroll
          for (int c = 0; c < HDV / 16; ++c) {   // undo the even/odd column split of the fp8 V path
            *reinterpret_cast<float4*>(so + g * SM::kLdO + c * 16 + 4 * tq) =
                make_float4(o[2 * c][0], o[2 * c + 1][0], o[2 * c][1], o[2 * c + 1][1]);
            *reinterpret_cast<float4*>(so + (g + 8) * SM::kLdO + c * 16 + 4 * tq) =
                make_float4(o[2 * c][2], o[2 * c + 1][2], o[2 * c][3], o[2 * c + 1][3]);
          }
        }
        if (tq == 0) {
          s_m[warp * 16 + g] = m_a; s_m[warp * 16 + g + 8] = m_b;
          s_l[warp * 16 + g] = l_a; s_l[warp * 16 + g + 8] = l_b;
          s_lr[warp * 16 + g] = lr_a; s_lr[warp * 16 + g + 8] = lr_b;
        }
        bar_consumers<NC>();
        {
          constexpr int CPT = 16 * HDV / (NC * 32);      // output columns per thread: 16 or 8
          constexpr int GPR = HDV / CPT;                 // threads per row
          const int Rl = tid / GPR, c0 = (tid % GPR) * CPT;   // row within the tile, first column
          const int R = it.mt * 16 + Rl;                     // packed row (token, head)
          const int rows_total = it.seqlen_q * rep;
          float mw[NC], M = -INFINITY;
#pragma unroll
          for (int wi = 0; wi < NC; ++wi) { mw[wi] = s_m[wi * 16 + Rl]; M = fmaxf(M, mw[wi]); }
          float L = 0.f, Lr = 0.f, acc[CPT];
#pragma unroll
          for (int j = 0; j < CPT; ++j) acc[j] = 0.f;
#pragma unroll
          for (int wi = 0; wi < NC; ++wi) {
            const float e = mw[wi] == -INFINITY ? 0.f : ex2(mw[wi] - M);
            L += e * s_l[wi * 16 + Rl];
            Lr += e * s_lr[wi * 16 + Rl];
            const float* src = s_o + (wi * 16 + Rl) * SM::kLdO + c0;
#pragma unroll
            for (int j = 0; j < CPT; j += 4) {
              const float4 v4 = *reinterpret_cast<const float4*>(src + j);
              acc[j] += e * v4.x; acc[j + 1] += e * v4.y; acc[j + 2] += e * v4.z; acc[j + 3] += e * v4.w;
            }
          }
          if (R < rows_total) {
            const int token = R / rep, head = it.hk * rep + R % rep;
            const int64_t qi = it.q0 + token;
            if (p.nsplits > 1) {
              const float Ln = KV8 ? Lr : L;   // e4m3: divide by the sum of the rounded probabilities
              const float inv = Ln > 0.f ? vds / Ln : 0.f;
              float* op = p.o_part + (((int64_t)it.split * p.total_q + qi) * p.hq + head) * p.hdv + c0;
#pragma unroll
              for (int j = 0; j < CPT; j += 4)
                *reinterpret_cast<float4*>(op + j) = make_float4(acc[j] * inv, acc[j + 1] * inv, acc[j + 2] * inv, acc[j + 3] * inv);
              if (tid % GPR == 0)
                p.lse_part[((int64_t)it.split * p.hq + head) * p.total_q + qi] = L > 0.f ? (M + lg2(L)) * kLn2 : -INFINITY;
            } else {
              float osc = 1.f;
              if (p.s_aux) {
                const float ys = p.s_aux[head] * kLog2e;
                const float mn = fmaxf(M, ys);
                osc = M == -INFINITY ? 0.f : ex2(M - mn);
                L = L * osc + ex2(ys - mn);
                Lr = Lr * osc + ex2(ys - mn);
                M = mn;
              }
              const float Ln = KV8 ? Lr : L;
              const float inv = Ln > 0.f ? osc * vds / Ln : 0.f;
              if (p.out_f32) {
                float* of = reinterpret_cast<float*>(p.out) + qi * p.o_row_stride + (int64_t)head * p.o_head_stride + c0;
#pragma unroll
                for (int j = 0; j < CPT; j += 4)
                  *reinterpret_cast<float4*>(of + j) = make_float4(acc[j] * inv, acc[j + 1] * inv, acc[j + 2] * inv, acc[j + 3] * inv);
              } else {
                T* op = reinterpret_cast<T*>(p.out) + qi * p.o_row_stride + (int64_t)head * p.o_head_stride + c0;
#pragma unroll
                for (int j = 0; j < CPT; j += 8) {
                  uint4 v;
                  v.x = pack2<T>(acc[j] * inv, acc[j + 1] * inv);     v.y = pack2<T>(acc[j + 2] * inv, acc[j + 3] * inv);
                  v.z = pack2<T>(acc[j + 4] * inv, acc[j + 5] * inv); v.w = pack2<T>(acc[j + 6] * inv, acc[j + 7] * inv);
                  *reinterpret_cast<uint4*>(op + j) = v;
                }
              }
              if (tid % GPR == 0) p.lse[(int64_t)head * p.total_q + qi] = L > 0.f ? (M + lg2(L)) * kLn2 : -INFINITY;
            }
          }
        }
        bar_consumers<NC>();   // the scratch area is free again
      }
    }
  }
  __syncthreads();
}

// ------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)f;
  });
  return fn;
}

// [rows, cols] row-major, 128-byte wide boxes of box_rows rows, 128-byte swizzle
static bool make_map(CUtensorMap* m, const void* ptr, int dtype, uint64_t rows, uint64_t cols, uint64_t pitch_elems,
                     uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  const uint32_t esz = dtype == FA_DT_FP8_E4M3 ? 1 : 2;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {pitch_elems * esz};
  const cuuint32_t box[2] = {128 / esz, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = dtype == FA_DT_FP8_E4M3 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : dtype == FA_DT_FP16   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                         : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  return fn(m, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename T, bool KV8, int NST, int HD, int HDV, int CPS = ctas_per_sm(KV8 ? 1 : 2), int TNS_ = 64>
static int launch_t(const KParams& kp, const Plan& pl, int num_work_slots, cudaStream_t stream) {
  using SM = Smem<KV8 ? 1 : 2, NST, HD, HDV, TNS_>;
  DecArgs a;
  a.kp = kp;
  a.total_work = num_work_slots * kp.hkv * kp.nsplits;
  constexpr int TNS = SM::TNS;
  const bool paged = kp.page_table != nullptr;
  // (the cp.async producer takes any power-of-two page; measured, pages of 8 and 16 keys are faster as TMA boxes:
  // 0.49 / 0.70 of the HBM peak against 0.48 / 0.60)
  a.gather = paged && (kp.page_size == 1 || kp.page_size == 2 || kp.page_size == 4);
  // rows per TMA box: a whole stage of contiguous K/V, else a page or 64 rows of a larger page.  (Never more than 64
  // of a page: a stage starts at a multiple of 64 keys - split and window boundaries are in 64-key blocks - so a
  // 128-row box of a 128-key stage could start in the middle of a page and run into the physically next one.)
  a.box_rows = a.gather ? 1 : (!paged ? TNS : (kp.page_size < 64 ? kp.page_size : 64));
  const uint64_t rows = paged ? (uint64_t)kp.num_pages * (uint64_t)kp.page_size : (uint64_t)kp.total_k;
  a.kv_total_rows = (int)rows;
  const int kvdt = KV8 ? FA_DT_FP8_E4M3 : (std::is_same<T, __half>::value ? FA_DT_FP16 : FA_DT_BF16);
  CUtensorMap mk, mv;
  if (!make_map(&mk, kp.k, kvdt, rows, (uint64_t)kp.hkv * HD, (uint64_t)kp.k_row_stride, a.box_rows)) return -1;
  if (!make_map(&mv, kp.v, kvdt, rows, (uint64_t)kp.hkv * HDV, (uint64_t)kp.v_row_stride, a.box_rows)) return -1;
  auto kern = fwd_decode_kernel<T, KV8, NST, HD, HDV, CPS, TNS_>;
  const int smem = SM::kBytes + 1024;
  static std::atomic<unsigned long long> attr_done{0};   // one bit per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !((attr_done.load(std::memory_order_acquire) >> dev) & 1ull)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    if (dev >= 0 && dev < 64) attr_done.fetch_or(1ull << dev, std::memory_order_release);
  }
  const int ctas = pl.num_sms * CPS;
  int grid = a.total_work < ctas ? a.total_work : ctas;
  if (grid <= 0) return 0;
  kern<<<grid, (SM::NC + 1) * 32, smem, stream>>>(a, mk, mv);
  return (int)cudaGetLastError();
}

}  // namespace dec

// Shapes the decode route takes: head_dim 64, 128 or 192 (values 128), 16-bit queries, a cache of the same type or
// (head_dim 128) of e4m3 bytes, K/V contiguous or in pages of 1, 2, 4, 8, 16, 32 or a multiple of 64 keys (the small
// pages row by row, as the reference's cp.async producer does for page size 1, kernels/fa4_blackwell.cu:8936-8947).  These are the
// head dims of the reference's paged kernel (kernels/fa4_blackwell.cu:9958-9983).
bool decode_supported(const PlanInput& in) {
  if (in.q_dtype == FA_DT_FP8_E4M3) return false;
  if (in.kv_dtype != in.q_dtype && in.kv_dtype != FA_DT_FP8_E4M3) return false;
  const bool hd_ok = (in.hd == 128 && in.hdv == 128) ||
                     (in.kv_dtype != FA_DT_FP8_E4M3 && ((in.hd == 64 && in.hdv == 64) || (in.hd == 192 && in.hdv == 128)));
  if (!hd_ok) return false;
  const int ps = in.page_size;
  // pages of 8, 16 or 32 keys divide a 64-row stage into whole 1024-byte swizzle atoms; multiples of 64 are whole
  // stages; pages of 1, 2 or 4 keys are fetched row by row with cp.async
  if (!(ps == 0 || ps == 1 || ps == 2 || ps == 4 || ps == 8 || ps == 16 || ps == 32 || ps % 64 == 0)) return false;
  return in.hkv > 0 && in.hq % in.hkv == 0 && in.tc_layout_ok;
}

template <typename T>
static int launch_decode_t(const KParams& kp, const Plan& pl, int slots, cudaStream_t stream) {
  // e4m3 cache: 128-key stages (32 keys = two independent 16-key chains per consumer warp: the chains hide each
  // other's fixed latencies; 0.80 -> 0.92 of the HBM peak against 64-key stages), two stages, two CTAs per SM
  if (kp.kv_fp8) return dec::launch_t<T, true, 2, 128, 128, 2, 128>(kp, pl, slots, stream);
  if (kp.hd == 64) return dec::launch_t<T, false, 5, 64, 64, 2>(kp, pl, slots, stream);   // 16 KB stages: two CTAs per SM
  if (kp.hd == 192) return dec::launch_t<T, false, 4, 192, 128>(kp, pl, slots, stream);
  return dec::launch_t<T, false, 5, 128, 128>(kp, pl, slots, stream);
}

int launch_decode(const KParams& kp, const Plan& pl, int compute_dtype, cudaStream_t stream) {
  // every (batch, m_tile) slot of the metadata may hold a work entry
  const int slots = kp.batch * pl.max_mtiles;
  return compute_dtype != FA_DT_FP16 ? launch_decode_t<__nv_bfloat16>(kp, pl, slots, stream)
                                     : launch_decode_t<__half>(kp, pl, slots, stream);
}

}  // namespace fa
