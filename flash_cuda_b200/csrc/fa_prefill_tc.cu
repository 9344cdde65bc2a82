// fa_prefill_tc.cu — the prefill mainloop on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// One persistent CTA per SM.  A work item is a pair of adjacent 128-row query tiles of one (batch, q head);
// both tiles share every K/V tile that TMA brings in.  Warp roles (384 threads):
//   warps 0-3  softmax of tile 0   (one query row per thread: S row TMEM -> registers -> P row TMEM)
//   warps 4-7  softmax of tile 1
//   warp  8    MMA issuer: S_t = Q_t K^T (operands in shared memory), O_t += P_t V (P in TMEM); the whole
//              warp runs the control flow (warp-uniform values, uniform registers), one elected lane issues
//   warp  9    TMA producer (one lane): Q pair, K ring, V ring (no cluster multicast: each CTA loads its own
//              tiles); also takes work ids from the global counter and decodes them
//   warps 10-11 idle (they complete the third warpgroup so that register tiers can be set per warpgroup)
// Work items (256 query rows of one (batch, head); late = heavy tiles first) are handed out through one global
// atomic counter, so SMs that finish early take more; the TMA lane decodes each item once (sequence bounds,
// key-block ranges) and publishes it, one item ahead, in a two-slot mailbox in shared memory.  The items come
// either from arithmetic on the work id (slots of a ragged batch that own no query row are skipped by the TMA
// lane without a hand-off) or, when the call carries scheduler metadata for this route, from that sorted list.
// Epilogue: a softmax thread pulls its whole O row into registers and releases O at once (the next item's first
// PV may then overwrite it); where a warp's 32 rows all lie inside the sequence the rows go out through a
// swizzled 4 KB staging buffer per warp and one TMA store per 64 columns, else through plain stores.
// TMEM (512 columns): S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P_t overlays the first 64
// columns of S_t once the owning thread has read its S row.
// The tensor pipe runs [PV0(i), QK0(i+1), PV1(i), QK1(i+1)] so that one tile's softmax overlaps the other
// tile's MMAs.  Softmax works in the exp2 domain with a lazy maximum: the running maximum only moves (and
// O is only rescaled) when the new row maximum exceeds it by more than 8.
// Every wait is bounded: on expiry the role records an error in the status word, raises a CTA-wide abort
// flag, and every role drains and leaves.
//
// Plays the role of `fwd_kernel_fa4` / `fwd_kernel_ws2` / `fwd_kernel_fa4dk` of the reference
// (kernels/fa4_blackwell.cu:6935-7407, 6539-6906, 7420-7753) with masks, softcap, sink, leftpad, paged KV
// and head_dim 192/128 in the one kernel.
#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <mutex>

#include "fa_internal.h"
#include "fa_sched.h"
#include "ptx.cuh"

namespace fa {
namespace tc {

constexpr int TM = 128, TN = 128;
constexpr int NTHREADS = 384;   // 12 warps: two softmax warpgroups + one warpgroup holding the MMA and TMA warps
constexpr int WARP_MMA = 8, WARP_TMA = 9;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
#ifndef FA_CAP_EMU_PAIRS
#define FA_CAP_EMU_PAIRS 2
#endif
constexpr int kCapEmuPairs = FA_CAP_EMU_PAIRS;   // of every four pairs in the fused softcap loop
constexpr float kRescaleThreshold = 8.0f;   // log2 units
constexpr float kFastSumLimit = 16384.f;    // 2^14: row sum of a block above which the fast softmax form is redone
enum Role : unsigned { ROLE_TMA = 1, ROLE_MMA = 2, ROLE_SOFTMAX = 3, ROLE_EPILOGUE = 4 };

constexpr int kEndOfWork = 0x7fffffff;
// K/V footprint above which work ids are ordered by kv head: 1.5 x the L2 capacity.  (Below it the order costs:
// the tiles of a head then ask the same L2 lines at the same time; 2 x 16 heads x 4096 keys of head_dim 256, 134 MB,
// ran at 735 TFLOP/s kv-head-major against 827.)
#ifndef FA_HEAD_MAJOR_MB
#define FA_HEAD_MAJOR_MB 192.0
#endif
constexpr double kHeadMajorBytes = FA_HEAD_MAJOR_MB * 1024 * 1024;
constexpr int kTwoTermBlocks = 2;   // e4m3: tiles that see at most this many key blocks keep P as two e4m3 terms

struct TcArgs {
  KParams kp;
  int num_items;     // batch * hq * max_pairs: the work ids of the arithmetic order (an upper bound with a list)
  int max_pairs;     // work items per (batch, head): ceil(max_seqlen_q / rows per item)
  int item_rows;     // query rows per work item: 256 (two tiles) or 128 (one tile: head dims whose O needs > 128 columns)
  int use_list;      // kp.work holds scheduler metadata of this route: items = its valid entries x hq
  int head_major;    // arithmetic order: all tiles of one (batch, kv head) are consecutive ids (K/V larger than L2)
  int stage_out;     // map_o is valid: full 32-row groups leave through shared memory and TMA stores
  int kv_box_rows;   // rows per K/V TMA box: 128 (contiguous KV) or min(page_size, 128)
  int gather;        // pages of 1, 2 or 4 keys: K/V rows are copied with cp.async (the K/V maps are not used)
  int kv_total_rows; // rows of the K/V tensor map (out-of-range y => zero fill)
  int out_cols;      // value columns that exist (head_dim 96 runs as 128 with zero-filled columns 96..127)
};

struct fp8_t { unsigned char x; };   // tag type: Q, K, V and P are e4m3 bytes, the output is bf16

template <typename T> struct Elem {
  static constexpr int kSize = 2;
  static constexpr bool kF8 = false;
  using Out = T;
};
template <> struct Elem<fp8_t> {
  static constexpr int kSize = 1;
  static constexpr bool kF8 = true;
  using Out = __nv_bfloat16;
};

constexpr int kSmemLimit = 232448;   // dynamic shared memory one CTA may ask for on sm_100

template <int ESZ, int HD, int HDV, int KST, int VST, int NTL>
struct Smem {
  static constexpr int kQBytes = NTL * TM * HD * ESZ;
  static constexpr int kKStage = TN * HD * ESZ;
  static constexpr int kVStage = TN * HDV * ESZ;
  static constexpr int kRings = kQBytes + KST * kKStage + VST * kVStage;
  // output staging: 8 softmax warps x (32 rows x 64 16-bit columns), when it fits beside the rings
  static constexpr int kStageBytes = 8 * 4096;
  static constexpr bool kStageOut = kRings + kStageBytes + 3 * 1024 <= kSmemLimit;
  static constexpr int kStageOff = kRings;
  static constexpr int kBarOff = kRings + (kStageOut ? kStageBytes : 0);
  static constexpr int kNumBars = 4 + KST + 2 * VST + 8 + 1 + 4 + 1 + KST + 1;
  static constexpr int kItemOff = kBarOff + ((kNumBars * 8 + 16 + 15) & ~15);   // after abort flags and TMEM base
  static constexpr int kBytes = kItemOff + 2 * 64;             // two mailbox slots of one decoded work item each
};

// One work item, decoded once by the TMA thread and handed to every role through shared memory (64 bytes).
struct alignas(16) Item {
  int b, h, pair, q0;
  int seqlen_q, seqlen_k, k0, leftpad;
  int lo[2], hi[2];   // key-block range per tile
  int ulo, uhi;       // union
  int valid;
  int w;              // work id; kEndOfWork ends the role loops
};
static_assert(sizeof(Item) == 64, "mailbox slot");

template <int NTL>
__device__ __forceinline__ Item decode_item(const TcArgs& a, int w, bool* bad_entry) {
  constexpr int kItemRows = NTL * TM;
  const KParams& p = a.kp;
  Item it;
  it.w = w;
  if (a.use_list) {
    // entry e of the sorted list = (batch, tile of item_rows rows); all q heads of one entry are consecutive work
    // ids, or (K/V larger than L2) the kv head is the slowest index and the list is walked once per kv head
    int e;
    if (a.head_major) {
      const int per_kv = p.work[6] * p.rep;
      const int hk = w / per_kv, rem = w - hk * per_kv;
      e = rem / p.rep;
      it.h = hk * p.rep + (rem - e * p.rep);
    } else {
      e = w / p.hq;
      it.h = w - e * p.hq;
    }
    const int32_t* ent = p.work + kSchedHeader + 4 * e;
    it.b = ent[0];
    it.pair = ent[1];
    if ((unsigned)it.b >= (unsigned)p.batch || (unsigned)it.pair >= (unsigned)a.max_pairs) {
      *bad_entry = true;
      it.b = it.pair = it.h = it.q0 = it.seqlen_q = it.seqlen_k = it.k0 = it.leftpad = 0;
      it.lo[0] = it.lo[1] = it.hi[0] = it.hi[1] = it.ulo = it.uhi = it.valid = 0;
      return it;
    }
  } else if (a.head_major) {
    // K/V that does not fit in L2: the tiles of one (batch, kv head) run at the same time on neighbouring CTAs and
    // walk its keys together, so each key block comes from HBM once instead of once per tile (heavy tiles first
    // within the head)
    const int per_head = a.max_pairs * p.rep;
    const int g = w / per_head, rem = w - g * per_head;
    const int slot = rem / p.rep;
    it.b = g / p.hkv;
    it.h = (g - it.b * p.hkv) * p.rep + (rem - slot * p.rep);
    it.pair = a.max_pairs - 1 - slot;
  } else {
    const int per_slot = p.batch * p.hq;
    const int slot = w / per_slot, rem = w - slot * per_slot;
    it.pair = a.max_pairs - 1 - slot;          // heavy (late) tiles first under causal masking
    it.b = rem / p.hq;
    it.h = rem - it.b * p.hq;
  }
  it.q0 = p.cu_q[it.b];
  it.seqlen_q = p.cu_q[it.b + 1] - it.q0;
  it.k0 = p.page_table ? 0 : p.cu_k[it.b];
  it.seqlen_k = p.seqused_k ? p.seqused_k[it.b] : (p.cu_k[it.b + 1] - p.cu_k[it.b]);
  it.leftpad = p.leftpad_k ? p.leftpad_k[it.b] : 0;
  it.valid = it.pair * kItemRows < it.seqlen_q;
  it.ulo = 0x7fffffff;
  it.uhi = 0;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int row0 = it.pair * kItemRows + t * TM;
    it.lo[t] = it.hi[t] = 0;
    if (it.valid && row0 < it.seqlen_q && t < NTL) {
      const int rmax = min(it.seqlen_q - 1, row0 + TM - 1);
      nblock_range(it.seqlen_k, it.leftpad, it.seqlen_k - it.seqlen_q + row0, it.seqlen_k - it.seqlen_q + rmax,
                   p.is_causal, p.window_left, p.window_right, TN, &it.lo[t], &it.hi[t]);
    }
    if (it.hi[t] > it.lo[t]) { it.ulo = min(it.ulo, it.lo[t]); it.uhi = max(it.uhi, it.hi[t]); }
  }
  if (it.uhi <= it.ulo) { it.ulo = it.uhi = 0; }
  return it;
}

// Position in a ring of N stages: slot index and phase bit, advanced without divisions.
template <int N>
struct Ring {
  uint32_t slot = 0, phase = 0, n = 0;
  __device__ __forceinline__ void advance() {
    ++n;
    if (++slot == (uint32_t)N) { slot = 0; phase ^= 1u; }
  }
};

// Paged K/V tiles.  The TMA boxes of a 128-key tile (one page each, or 128 keys of a larger page) are shared out
// j = j0, j0 + jstride, ..: j0 = lane, jstride = 32 when the whole warp produces (every lane owns one box), 0 and 1
// when lane 0 produces alone (pages of >= 64 keys then: at most two boxes).  With pages of 1, 2 or 4 keys (whole
// warp only) lane g looks up the pool rows of keys g, g + 32, g + 64, g + 96 and the warp copies the tile row by row
// with cp.async (copy_tile_rows).  Either way a lane's share of a tile is at most four pool rows.
struct PageRows { int y[4]; };

// The pool rows of key block nb.  K and V share the page table, so one look-up serves K(nb) and V(nb); it is made a
// block ahead and BEFORE the waits for the free stages, so that the page-table loads fly during the waits (the
// refill of a single V stage is on the critical path: with the look-up after the wait the long-context shape ran
// at 0.73 of its speed over contiguous keys).  Inlined so that the loads' results are awaited at their first use.
__device__ __forceinline__ PageRows page_rows(const TcArgs& a, int nb, int b, int seqlen_k, int lane, int j0, int jstride) {
  const KParams& p = a.kp;
  const int32_t* pt = p.page_table + (int64_t)b * p.page_table_stride;
  PageRows pr;
  if (a.gather) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int kk = nb * TN + lane + 32 * j;
      pr.y[j] = 0;               // beyond the sequence: pool row 0 (finite by contract), masked by the softmax
      if (kk < seqlen_k) {
        const int lp = kk >> p.page_shift;
        pr.y[j] = (pt[lp] << p.page_shift) + (kk - (lp << p.page_shift));
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = (j0 + i * jstride) * a.kv_box_rows, kk = nb * TN + r;
      pr.y[i] = a.kv_total_rows;   // beyond the sequence: out of range => zeros
      if (r < TN && kk < seqlen_k) {
        const int lp = p.page_shift >= 0 ? (kk >> p.page_shift) : (kk / p.page_size);
        pr.y[i] = pt[lp] * p.page_size + (kk - lp * p.page_size);
      }
    }
  }
  return pr;
}

// The copies of one paged K or V tile.  Rolled on purpose: the producer shares its instruction cache with the
// softmax warps, whose loop bodies are large, and the time of this path went with its code size (a fully unrolled
// single-thread form measured 372 TFLOP/s on pages of 16 keys, a rolled one 583).
template <int EPB>
__device__ __forceinline__ void load_tile_paged(const TcArgs& a, const CUtensorMap* map, int width, uint32_t dst, uint32_t bar,
                                             int hk, int r0, int rstride, int y0, int y1, int y2, int y3) {
  const int ncb = width / EPB;
#pragma unroll 1
  for (int i = 0, r = r0; i < 4 && r < TN; ++i, r += rstride) {
    const int y = i == 0 ? y0 : (i == 1 ? y1 : (i == 2 ? y2 : y3));
#pragma unroll 1
    for (int cb = 0; cb < ncb; ++cb) tma_load_3d(dst + cb * (TN * 128) + r * 128, map, cb * EPB, hk, y, bar);
  }
}

// One K or V tile of a cache in pages of 1, 2 or 4 keys, by the whole producer warp with cp.async: the tile's 16-byte
// chunks in row order, CPR consecutive lanes on one row, each written where a 128-byte-swizzled TMA box would have
// put it (column block ch / 8, row r, chunk (ch % 8) ^ (r % 8)).  Row r comes from pool row y[r / 32] of lane
// r % 32.  The TMA unit retires about one copy per 100 cycles whatever its size (128 four-row gathers per key
// block: 401 TFLOP/s); these copies take the load/store path.  Rolled, eight copies per turn with their row
// numbers fetched first (a shuffle followed at once by its copy would cost the shuffle's latency per copy).
template <int CPR>
__device__ __forceinline__ void copy_tile_rows(uint32_t dst0, const unsigned char* src0, uint32_t pitch, const PageRows& pr,
                                               int lane) {
  if constexpr (32 % CPR == 0) {
    // RPI rows per instruction; row r = i * RPI + hb, and (r & 7) = ((i * RPI) & 7) ^ hb because the low bits of
    // i * RPI are clear
    constexpr int RPI = 32 / CPR;
    const int hb = lane / CPR, ch = lane - hb * CPR;
    const uint32_t dl = dst0 + (uint32_t)(ch >> 3) * (TN * 128) + (uint32_t)hb * 128u;
    const uint32_t xs = (uint32_t)(((ch & 7) ^ hb) << 4);
    const unsigned char* sl = src0 + ch * 16;
#pragma unroll 1
    for (int i0 = 0; i0 < TN / RPI; i0 += 8) {
      const int quarter = (i0 * RPI) >> 5;      // the eight copies of a turn take rows of one quarter of the tile
      const int yv = quarter == 0 ? pr.y[0] : (quarter == 1 ? pr.y[1] : (quarter == 2 ? pr.y[2] : pr.y[3]));
      int y[8];
#pragma unroll
      for (int g = 0; g < 8; ++g) y[g] = __shfl_sync(0xffffffffu, yv, (((i0 + g) * RPI) & 31) + hb);
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const int r0 = (i0 + g) * RPI;
        cp_async16(dl + (uint32_t)r0 * 128u + (xs ^ (uint32_t)((r0 & 7) << 4)), sl + (uint64_t)(uint32_t)y[g] * pitch, 16u);
      }
    }
  } else {
    constexpr int N = TN * CPR / 32;
    static_assert(N % 8 == 0, "whole turns");
#pragma unroll 1
    for (int i0 = 0; i0 < N; i0 += 8) {
      int y[8];
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const int r = ((i0 + g) * 32 + lane) / CPR;
        const int quarter = (((i0 + g) * 32) / CPR) >> 5;      // the same for every lane of one instruction
        const int yv = quarter == 0 ? pr.y[0] : (quarter == 1 ? pr.y[1] : (quarter == 2 ? pr.y[2] : pr.y[3]));
        y[g] = __shfl_sync(0xffffffffu, yv, r & 31);
      }
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const int q = (i0 + g) * 32 + lane, r = q / CPR, ch = q - r * CPR;
        cp_async16(dst0 + (uint32_t)(ch >> 3) * (TN * 128) + (uint32_t)r * 128u + (uint32_t)(((ch & 7) ^ (r & 7)) << 4),
                   src0 + (uint64_t)(uint32_t)y[g] * pitch + ch * 16, 16u);
      }
    }
  }
}

// NTL = query tiles per work item: 2, or 1 where one tile's S (128 columns) and O (HDV > 128 columns) leave no room
// in the 512 TMEM columns for a second tile (head_dim 256, head_dim 192 with 192 value columns).  With one tile the
// second softmax warpgroup stays idle and softmax and MMAs of the tile alternate instead of overlapping.
// CAP: the logit soft cap is compiled in (the host picks the instantiation by softcap > 0, so that the common
// kernel carries none of its code: the softmax loop's time follows its instruction count).
// PROD: the form of the TMA producer: 0 = contiguous K/V, lane 0 alone; 1 = paged, lane 0 alone; 2 = paged, the whole
// warp (see the TMA role).  Template arguments rather than run-time flags for the same reason as CAP: code that a
// launch never runs still moved the time of the code it does run by a few per cent.
template <typename T, int HD, int HDV, int KST, int VST, int NTL, bool CAP, int PROD>
__global__ void __launch_bounds__(NTHREADS, 1)
fwd_prefill_tc_kernel(const __grid_constant__ TcArgs a, const __grid_constant__ CUtensorMap map_q,
                      const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                      const __grid_constant__ CUtensorMap map_o) {
  constexpr int ESZ = Elem<T>::kSize;          // bytes per Q/K/V element
  constexpr bool F8 = Elem<T>::kF8;
  constexpr int EPB = 128 / ESZ;               // elements per 128-byte swizzle row
  using TO = typename Elem<T>::Out;
  using SM = Smem<ESZ, HD, HDV, KST, VST, NTL>;
  static_assert(NTL == 2 ? HDV <= 128 : HDV <= 256, "TMEM: NTL x (128 S columns + HDV O columns) <= 512");
  constexpr uint32_t O_BASE = NTL * TN;        // first TMEM column of the O accumulators
  constexpr uint32_t O_STRIDE = NTL == 2 ? 128 : 0;
  const KParams& p = a.kp;
  extern __shared__ unsigned char smem_dyn[];
  // 1024-byte alignment for the 128-byte swizzle atoms, by rounding up inside a request that carries 1 KB of slack.
  // (Declaring the array __align__(1024) instead measured 10 % slower on B200 with identical tile addresses.)
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* sm = smem_dyn + (base - raw);
  const uint32_t sQ = base;
  const uint32_t sK = sQ + SM::kQBytes;
  const uint32_t sV = sK + KST * SM::kKStage;
  const uint32_t bars = base + SM::kBarOff;
  // barrier map
  const uint32_t bar_q_full = bars, bar_q_empty = bars + 16;   // [2] each: one per query tile
  const uint32_t bar_k_empty = bars + 32;                // [KST] (K tiles complete on k0_full / v_full, see the TMA role)
  const uint32_t bar_v_full = bar_k_empty + 8 * KST, bar_v_empty = bar_v_full + 8 * VST;
  const uint32_t bar_s_full = bar_v_empty + 8 * VST;     // [2]
  const uint32_t bar_p_full = bar_s_full + 16;           // [2]
  const uint32_t bar_o_full = bar_p_full + 16;           // [2]
  const uint32_t bar_o_empty = bar_o_full + 16;          // [2]
  const uint32_t bar_drain = bar_o_empty + 16;           // MMA warp's private drain barrier
  const uint32_t bar_w_full = bar_drain + 8;             // [2] work id published by the TMA thread
  const uint32_t bar_w_empty = bar_w_full + 16;          // [2] read by the MMA thread and the 8 softmax warps
  const uint32_t bar_k0_full = bar_w_empty + 16;         // K of an item's first block (later K tiles ride on v_full)
  const uint32_t bar_k_full = bar_k0_full + 8;           // [KST] used instead when the K and V rings differ in depth
  const uint32_t bar_pv_done = bar_k_full + 8 * KST;     // one-tile kernels: the PV of a block has run
  // With rings of equal depth a later K tile completes on the barrier of the V tile before it (one consumer wait per
  // block less).  With a single V stage (head_dim 192) that V tile is the late one, and PV must not wait for the
  // K tile behind it as well: there every K tile has the barrier of its slot.
  constexpr bool MERGE_KV = KST == VST && NTL == 2;
  // One-tile kernels (SDB): the 128 TMEM columns that a second tile's S would take hold a SECOND S buffer of the one
  // tile instead.  QK(i+1) then does not have to wait for PV(i) (P(i) overlays S(i), in the other buffer): it is issued
  // a block ahead, the softmax of block i+1 starts the moment block i is done, and the chain per block shrinks from
  // PV -> QK -> softmax -> PV to max(PV -> load of the single V stage, softmax) -> PV.  Buffers alternate block by
  // block across items; buffer b has s_full / p_full barrier b (the second tile's, unused in these kernels).
  constexpr bool SDB = NTL == 1;
  constexpr uint32_t S1_COL = 384;                       // second S buffer: behind O (128 + up to 256 columns)
  static_assert(!SDB || NTL * TN + HDV <= S1_COL, "O must end before the second S buffer");
  Item* s_item = reinterpret_cast<Item*>(sm + SM::kItemOff);   // [2]
  volatile int* s_abort = reinterpret_cast<volatile int*>(sm + SM::kBarOff + SM::kNumBars * 8);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(sm + SM::kBarOff + SM::kNumBars * 8 + 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int t = 0; t < 2; ++t) { mbar_init(bar_q_full + 8 * t, 1); mbar_init(bar_q_empty + 8 * t, 1); }
    for (int s = 0; s < KST; ++s) mbar_init(bar_k_empty + 8 * s, 1);
    // (rows copied with cp.async: a tile completes on one arrival per producer lane when its copies have landed, plus
    // lane 0's own)
    const int full_cnt = (PROD == 2 && a.gather) ? 33 : 1;
    for (int s = 0; s < VST; ++s) { mbar_init(bar_v_full + 8 * s, full_cnt); mbar_init(bar_v_empty + 8 * s, 1); }
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar_s_full + 8 * t, 1); mbar_init(bar_p_full + 8 * t, 4);     // one elected arrival per softmax warp
      mbar_init(bar_o_full + 8 * t, 1); mbar_init(bar_o_empty + 8 * t, 4);
    }
    mbar_init(bar_drain, 1);
    mbar_init(bar_k0_full, full_cnt);
    for (int s = 0; s < KST; ++s) mbar_init(bar_k_full + 8 * s, full_cnt);
    mbar_init(bar_pv_done, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(bar_w_full + 8 * i, 1); mbar_init(bar_w_empty + 8 * i, 1 + 4 * NTL); }
    s_abort[0] = 0;
    s_abort[1] = 0;   // [1] is never raised: waits that may only end by completion or time limit
    mbar_fence_init();
  }
  if (warp == WARP_MMA) { tmem_alloc(smem_u32(s_tmem), 512); tmem_relinquish(); }
  if (warp == WARP_TMA && lane == 0) { tma_prefetch_desc(&map_q); tma_prefetch_desc(&map_k); tma_prefetch_desc(&map_v); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *s_tmem;

  // register tiers: the launch gives every thread 168; the MMA/TMA warpgroup hands most of its share to the
  // two softmax warpgroups, which hold a full 128-wide fp32 score row per thread
  if (warp >= 8) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 104;");
  if (warp == WARP_TMA) {
    // =========================================== TMA producer ===========================================
    // Two forms, chosen by the host (template argument PROD).  Wide: the whole warp runs the control flow; lane 0 (the
    // leader) waits on the barriers, takes work ids, issues the Q copies and the copies of unpaged K/V tiles; every
    // wait's outcome and every decoded item is broadcast, and for paged tiles all lanes look pages up and issue
    // copies (load_tile_paged): pages of 16 keys 433 -> 817 TFLOP/s.  Narrow: lane 0 does all of it alone and the
    // other lanes leave; the broadcasts' latency is then off the path between a freed V stage and its refill, which
    // is what the kernels with a single V stage (head_dim 192, 256) are bound by: 945 against 868 TFLOP/s wide.
    // (The form is a template argument: with the choice left to a run-time flag the narrow form kept the
    // divergence bookkeeping of the wide one and lost 3-12 %.)
    constexpr bool wide = PROD == 2;
    constexpr bool paged = PROD != 0;
    if (wide || lane == 0) {
      constexpr uint32_t FULLM = 0xffffffffu;
      const bool leader = !wide || lane == 0;
      uint32_t qcnt = 0, k0cnt = 0;
      Ring<KST> kr;
      Ring<VST> vr;
      bool ok = true;
      uint32_t wcnt = 0;
      // number of work ids: from the list's header (checked against this call's geometry before anything is
      // indexed) or the arithmetic count
      int num_items = a.num_items;
      if (a.use_list) {
        if (sched_header_matches(p.work, p.work_expect)) {
          num_items = p.work[6] * p.hq;
        } else {
          if (leader) report_error(p.status, DEV_ERR_BAD_INDEX, ROLE_TMA);
          num_items = 0;
        }
      }
      bool first_ticket = true;
      auto lead_wait = [&](uint32_t bar, uint32_t parity) -> bool {
        int r = 1;
        if (leader) r = wait_or_abort(bar, parity, s_abort) ? 1 : 0;
        if (wide) r = __shfl_sync(FULLM, r, 0);
        return r != 0;
      };
      // work items are handed out heaviest first: a CTA's first id is its block index, later ones come from one
      // global counter; every role of this CTA learns the item from a two-slot mailbox in shared memory
      auto fetch_and_publish = [&]() -> Item {
        Item it{0, 0, 0, 0, 0, 0, 0, 0, {0, 0}, {0, 0}, 0, 0, 0, kEndOfWork};
        const uint32_t slot = wcnt & 1;
        if (!lead_wait(bar_w_empty + 8 * slot, ((wcnt >> 1) & 1) ^ 1)) {
          if (leader) report_error(p.status, DEV_ERR_TIMEOUT, ROLE_TMA);
          ok = false;
          return it;
        }
        if (leader) {
          // ids whose (batch, tile) owns no query row (ragged batches) are dropped here, without a hand-off
          while (true) {
            const int w = first_ticket ? (int)blockIdx.x : (int)gridDim.x + atomicAdd(p.counters, 1);
            first_ticket = false;
            if (w >= num_items) { it.w = kEndOfWork; break; }
            bool bad = false;
            it = decode_item<NTL>(a, w, &bad);   // sequence bounds are read from global memory once per item
            if (bad) { report_error(p.status, DEV_ERR_BAD_INDEX, ROLE_TMA); num_items = 0; it.w = kEndOfWork; break; }
            if (it.valid) break;
          }
          const int4* src = reinterpret_cast<const int4*>(&it);
          int4* dst = reinterpret_cast<int4*>(&s_item[slot]);
#pragma unroll
          for (int i = 0; i < 4; ++i) dst[i] = src[i];
          mbar_arrive(bar_w_full + 8 * slot);   // release: the slot is visible to whoever observes the phase
        }
        if (wide) {
          int* pi = reinterpret_cast<int*>(&it);
#pragma unroll
          for (int i = 0; i < 16; ++i) pi[i] = __shfl_sync(FULLM, pi[i], 0);
        }
        ++wcnt;
        return it;
      };
      Item it_next = fetch_and_publish();
      while (it_next.w != kEndOfWork && ok) {
        const Item it = it_next;
        // the next item is fetched one ahead, but only after this item's first loads are on their way: the
        // counter round trip and the decoding then hide behind them
        if (it.uhi <= it.ulo) { it_next = fetch_and_publish(); continue; }   // rows without keys: only an epilogue
        // Each query tile has its own pair of barriers: tile 0 usually finishes an item one key block before tile 1
        // (causal masking), so its Q slot is free, and refilled, a block earlier; the next item's first loads are
        // then spread over two blocks instead of one.  Order: Q tile 0, K of the first block, Q tile 1.
        auto load_q = [&](int t) -> bool {
          if (!lead_wait(bar_q_empty + 8 * t, (qcnt & 1) ^ 1)) return false;
          if (leader) {
            mbar_expect_tx(bar_q_full + 8 * t, TM * HD * ESZ);
#pragma unroll
            for (int cb = 0; cb < HD / EPB; ++cb)
              tma_load_3d(sQ + t * (TM * HD * ESZ) + cb * (TM * 128), &map_q, cb * EPB, it.h,
                          it.q0 + it.pair * (NTL * TM) + t * TM, bar_q_full + 8 * t);
          }
          return true;
        };
        ok = load_q(0);
        if (!ok) { if (leader) report_error(p.status, DEV_ERR_TIMEOUT, ROLE_TMA); break; }
        const int hk = it.h / p.rep;
        // one K or V tile of key block nb into `dst`, completing on `bar`
        const int pj0 = wide ? lane : 0, pjs = wide ? 32 : 1;
        // first row of this lane's first box and the distance to its next one
        const int pr0 = pj0 * a.kv_box_rows, prs = pjs * a.kv_box_rows;
        const bool cpg = wide && a.gather;      // pages of 1, 2, 4 keys: rows by cp.async, completion by arrivals
        auto open_bar = [&](uint32_t bar, uint32_t bytes) {
          if (leader) { if (cpg) mbar_arrive(bar); else mbar_expect_tx(bar, bytes); }
        };
        auto close_bar = [&](uint32_t bar) { if (cpg) cp_async_arrive_noinc(bar); };
        auto load_tile = [&](const CUtensorMap* map, int width, uint32_t dst, int nb, uint32_t bar, const PageRows& pr) {
          if (cpg) {
            if (map == &map_k)
              copy_tile_rows<HD * ESZ / 16>(dst, reinterpret_cast<const unsigned char*>(p.k) + (int64_t)hk * HD * ESZ,
                                            (uint32_t)(p.k_row_stride * ESZ), pr, lane);
            else
              copy_tile_rows<HDV * ESZ / 16>(dst, reinterpret_cast<const unsigned char*>(p.v) + (int64_t)hk * HDV * ESZ,
                                             (uint32_t)(p.v_row_stride * ESZ), pr, lane);
          } else if (!paged) {
            if (leader) {
              for (int cb = 0; cb < width / EPB; ++cb)
                tma_load_3d(dst + cb * (TN * 128), map, cb * EPB, hk, it.k0 + nb * TN, bar);
            }
          } else {
            load_tile_paged<EPB>(a, map, width, dst, bar, hk, pr0, prs, pr.y[0], pr.y[1], pr.y[2], pr.y[3]);
          }
        };
        // K of the first block has a barrier of its own; every later K tile arrives together with the V tile of
        // the block before it (the MMA warp needs both at the same point), so the consumer waits once per block
        PageRows rows_cur = {{0, 0, 0, 0}};
        if (paged) rows_cur = page_rows(a, it.ulo, it.b, it.seqlen_k, lane, pj0, pjs);
        {
          const uint32_t s = kr.slot;
          ok = lead_wait(bar_k_empty + 8 * s, kr.phase ^ 1u);
          if (!ok) { if (leader) report_error(p.status, DEV_ERR_TIMEOUT, ROLE_TMA); break; }
          const uint32_t kbar = MERGE_KV ? bar_k0_full : bar_k_full + 8 * s;
          open_bar(kbar, SM::kKStage);
          load_tile(&map_k, HD, sK + s * SM::kKStage, it.ulo, kbar, rows_cur);
          close_bar(kbar);
          kr.advance();
          ++k0cnt;
        }
        if constexpr (NTL == 2) {
          ok = load_q(1);
          if (!ok) { if (leader) report_error(p.status, DEV_ERR_TIMEOUT, ROLE_TMA); break; }
        }
        ++qcnt;
        for (int nb = it.ulo; nb < it.uhi; ++nb) {
          const bool nxt = nb + 1 < it.uhi;
          const uint32_t vs = vr.slot, ks = kr.slot;
          PageRows rows_nxt = rows_cur;
          if (paged && nxt) rows_nxt = page_rows(a, nb + 1, it.b, it.seqlen_k, lane, pj0, pjs);
          if constexpr (!MERGE_KV) {
            // separate barriers: K of the next block goes out as soon as its slot is free, without waiting for the
            // (single) V stage, which is released a whole PV later
            if (nxt) {
              ok = lead_wait(bar_k_empty + 8 * ks, kr.phase ^ 1u);
              if (!ok) { if (leader) report_error(p.status, DEV_ERR_TIMEOUT, ROLE_TMA); break; }
              const uint32_t kbar = bar_k_full + 8 * ks;
              open_bar(kbar, SM::kKStage);
              load_tile(&map_k, HD, sK + ks * SM::kKStage, nb + 1, kbar, rows_nxt);
              close_bar(kbar);
              kr.advance();
            }
            ok = lead_wait(bar_v_empty + 8 * vs, vr.phase ^ 1u);
            if (!ok) { if (leader) report_error(p.status, DEV_ERR_TIMEOUT, ROLE_TMA); break; }
            open_bar(bar_v_full + 8 * vs, SM::kVStage);
            load_tile(&map_v, HDV, sV + vs * SM::kVStage, nb, bar_v_full + 8 * vs, rows_cur);
            close_bar(bar_v_full + 8 * vs);
            vr.advance();
          } else {
            ok = lead_wait(bar_v_empty + 8 * vs, vr.phase ^ 1u);
            if (ok && nxt) ok = lead_wait(bar_k_empty + 8 * ks, kr.phase ^ 1u);
            if (!ok) { if (leader) report_error(p.status, DEV_ERR_TIMEOUT, ROLE_TMA); break; }
            open_bar(bar_v_full + 8 * vs, SM::kVStage + (nxt ? SM::kKStage : 0));
            load_tile(&map_v, HDV, sV + vs * SM::kVStage, nb, bar_v_full + 8 * vs, rows_cur);
            vr.advance();
            if (nxt) {
              load_tile(&map_k, HD, sK + ks * SM::kKStage, nb + 1, bar_v_full + 8 * vs, rows_nxt);
              kr.advance();
            }
            close_bar(bar_v_full + 8 * vs);
          }
          rows_cur = rows_nxt;
          if (nb == it.ulo) it_next = fetch_and_publish();
        }
      }
      if (!ok && leader) *s_abort = 1;
      // drain: every copy this warp issued must have landed before the CTA may leave
      if (leader) {
        if (qcnt > 0) {
          wait_or_abort(bar_q_full, (qcnt - 1) & 1, s_abort + 1 /* never set: pure time limit */);
          if constexpr (NTL == 2) wait_or_abort(bar_q_full + 8, (qcnt - 1) & 1, s_abort + 1);
        }
        if constexpr (MERGE_KV) {
          if (k0cnt > 0) wait_or_abort(bar_k0_full, (k0cnt - 1) & 1, s_abort + 1);
        } else {
          for (uint32_t s = 0; s < (uint32_t)KST; ++s) {
            if (kr.n > s) { const uint32_t last = (kr.n - 1 - s) / KST; wait_or_abort(bar_k_full + 8 * s, last & 1, s_abort + 1); }
          }
        }
        for (uint32_t s = 0; s < (uint32_t)VST; ++s) {
          if (vr.n > s) { const uint32_t last = (vr.n - 1 - s) / VST; wait_or_abort(bar_v_full + 8 * s, last & 1, s_abort + 1); }
        }
        counters_release(p.counters);   // this CTA takes no more tickets
      }
    }
  } else if (warp == WARP_MMA) {
    // =========================================== MMA issuer =============================================
    // The WHOLE warp runs this role's control flow, and every value that steers it (work id, block ranges,
    // ring positions, TMEM base) is made warp-uniform by construction (broadcast from lane 0, votes), so the
    // compiler can keep descriptors and addresses in uniform registers, which is where the MMA instruction
    // takes its operands from.  Only the tcgen05 instructions themselves and barrier arrivals sit behind
    // `elect_one()`.  (With the role under `if (lane == 0)` the same code measured ~1900 cycles of thread
    // time per key block beside the 2240 the tensor pipe needs: every MMA paid for moving five operands from
    // per-thread to uniform registers.)
    // operand format code: kind::f16 -> 1 = bf16, 0 = fp16; kind::f8f6f4 -> 0 = e4m3
    constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
    constexpr int KB = 32;                       // bytes of the contraction dimension one MMA consumes
    constexpr int KEL = KB / ESZ;                // ... in elements (16 for 16-bit, 32 for e4m3)
    constexpr uint32_t idesc_qk = umma_idesc(kFmt, TM, TN, false);
    constexpr uint32_t idesc_pv = umma_idesc(kFmt, TM, HDV, true);
    constexpr uint32_t FULL = 0xffffffffu;
    const uint32_t tmem_u = __shfl_sync(FULL, tmem, 0);
    const bool leader = elect_one();   // the same lane every time; decided once
    uint32_t qcnt = 0, k0cnt = 0, pcnt[2] = {0, 0}, oecnt[2] = {0, 0};
    uint32_t qkn = 0, pvn = 0;   // one-tile kernels: QKs / PVs issued so far (buffer = count & 1)
    Ring<KST> kr;
    Ring<VST> vr;
    // A wait that runs out does not branch out of the loops (that would make every loop-carried value
    // lane-dependent): it raises the CTA's abort flag, later waits of this lane return at once, the MMAs of
    // the current item are still issued (on whatever the buffers hold; nothing faults) and the work loop ends
    // at the next item boundary through a vote.
    bool fail = false;
    auto wait = [&](uint32_t bar, uint32_t parity) {
      if (!fail && !wait_or_abort(bar, parity, s_abort)) {
        fail = true;
        report_error(p.status, DEV_ERR_TIMEOUT, ROLE_MMA);
        *s_abort = 1;
      }
    };
    // a K / V tile has landed.  Tiles copied with cp.async were written through the generic proxy; the MMAs read
    // shared memory through the async proxy, so a proxy fence stands between the two.
    auto wait_tile = [&](uint32_t bar, uint32_t parity) {
      wait(bar, parity);
      if constexpr (PROD == 2) { if (a.gather) fence_proxy_async_smem(); }
    };
    const uint64_t qd0 = umma_desc(sQ, 16, 1024), kd0 = umma_desc(sK, 16, 1024), vd0 = umma_desc(sV, TN * 128, 1024);

    // S of tile t into TMEM column `col`, completion on `bar`
    auto issue_qk_to = [&](int t, uint32_t kslot, uint32_t col, uint32_t bar) {
      const uint64_t qd = qd0 + (uint64_t)(t * ((TM * HD * ESZ) >> 4));
      const uint64_t kd = kd0 + (uint64_t)(kslot * (SM::kKStage >> 4));
      if (leader) {
#pragma unroll
        for (int ks = 0; ks < HD / KEL; ++ks) {
          constexpr int kBlk = (TM * 128) >> 4;
          const uint64_t off = (uint64_t)((ks >> 2) * kBlk + (ks & 3) * 2);   // 4 steps of 32 bytes per 128-byte row
          umma_ss<F8>(tmem_u + col, qd + off, kd + off, idesc_qk, ks > 0 ? 1u : 0u);
        }
        umma_commit(bar);
      }
    };
    auto issue_qk = [&](int t, uint32_t kslot) { issue_qk_to(t, kslot, t * TN, bar_s_full + 8 * t); };
    // two_term (e4m3 only): P was written as P_hi (columns 0..31 of S_t) + P_lo (columns 32..63), see the softmax role
    auto issue_pv = [&](int t, uint32_t vslot, bool first, bool two_term, uint32_t pcol = 0xffffffffu) {
      if (pcol == 0xffffffffu) pcol = t * TN;      // P overlays the S it came from
      const uint64_t vd = vd0 + (uint64_t)(vslot * (SM::kVStage >> 4));
      if (leader) {
#pragma unroll
        for (int ks = 0; ks < TN / KEL; ++ks)   // KEL keys per step = KEL rows of 128 bytes; P: 8 TMEM columns per step
          umma_ts<F8>(tmem_u + O_BASE + t * O_STRIDE, tmem_u + pcol + ks * 8, vd + (uint64_t)(ks * ((KEL * 128) >> 4)), idesc_pv,
                      (!first || ks > 0) ? 1u : 0u);
        if constexpr (F8) {
          if (two_term) {
#pragma unroll
            for (int ks = 0; ks < TN / KEL; ++ks)
              umma_ts<F8>(tmem_u + O_BASE + t * O_STRIDE, tmem_u + pcol + 32 + ks * 8, vd + (uint64_t)(ks * ((KEL * 128) >> 4)),
                          idesc_pv, 1u);
          }
        }
      }
    };
    auto commit = [&](uint32_t bar) { if (leader) umma_commit(bar); };

    // One decoded work item as this warp needs it (block ranges, broadcast so that every loop bound is warp-uniform).
    struct MItem { int lo[2], hi[2], ulo, uhi, valid, w; };
    uint32_t wcnt = 0;
    auto read_item = [&]() -> MItem {
      const uint32_t slot = wcnt & 1;
      wait(bar_w_full + 8 * slot, (wcnt >> 1) & 1);
      const int4 ra = reinterpret_cast<const int4*>(&s_item[slot])[2], rb = reinterpret_cast<const int4*>(&s_item[slot])[3];
      MItem m;
      m.lo[0] = __shfl_sync(FULL, ra.x, 0); m.lo[1] = __shfl_sync(FULL, ra.y, 0);
      m.hi[0] = __shfl_sync(FULL, ra.z, 0); m.hi[1] = __shfl_sync(FULL, ra.w, 0);
      m.ulo = __shfl_sync(FULL, rb.x, 0); m.uhi = __shfl_sync(FULL, rb.y, 0);
      m.valid = __shfl_sync(FULL, rb.z, 0); m.w = __shfl_sync(FULL, rb.w, 0);
      if (leader) mbar_arrive(bar_w_empty + 8 * slot);
      ++wcnt;
      return m;
    };
    while (true) {
      const MItem cur = read_item();
      if (__any_sync(FULL, fail) || cur.w == kEndOfWork) break;
      if (!cur.valid || cur.uhi <= cur.ulo) continue;
      const int ulo = cur.ulo, uhi = cur.uhi;
      const int lo[2] = {cur.lo[0], cur.lo[1]}, hi[2] = {cur.hi[0], cur.hi[1]};
      if constexpr (SDB) {
        // one tile, two S buffers: QK runs a block ahead of PV (see SDB above).  Order QK(0) QK(1) | PV(i) QK(i+2).
        wait(bar_q_full, qcnt & 1);
        ++qcnt;
        auto qk_next = [&](int j) {
          const uint32_t ks = kr.slot, b = qkn & 1;
          wait_tile(bar_k_full + 8 * ks, kr.phase);
          issue_qk_to(0, ks, b ? S1_COL : 0u, bar_s_full + 8 * b);
          ++qkn;
          if (j + 1 == uhi) commit(bar_q_empty);     // the item's last QK: its Q slot may be refilled
          commit(bar_k_empty + 8 * ks);
          kr.advance();
        };
        qk_next(ulo);
        if (ulo + 1 < uhi) qk_next(ulo + 1);
        for (int i = ulo; i < uhi; ++i) {
          const uint32_t b = pvn & 1, vs = vr.slot;
          const bool first = i == ulo;
          if (first) {   // O is overwritten: the previous item's epilogue must have read it
            wait(bar_o_empty, (oecnt[0] & 1) ^ 1);
            ++oecnt[0];
          }
          wait_tile(bar_v_full + 8 * vs, vr.phase);
          wait(bar_p_full + 8 * b, (pvn >> 1) & 1);
          tc_fence_after_sync();
          issue_pv(0, vs, first, false, b ? S1_COL : 0u);
          ++pvn;
          commit(bar_pv_done);
          commit(bar_v_empty + 8 * vs);
          vr.advance();
          if (i + 1 == uhi) commit(bar_o_full);
          if (i + 2 < uhi) qk_next(i + 2);
        }
        continue;
      }
      // prologue: QK of the first block
      {
        const uint32_t ks = kr.slot;
        if constexpr (MERGE_KV) wait_tile(bar_k0_full, k0cnt & 1);
        else wait_tile(bar_k_full + 8 * ks, kr.phase);
        ++k0cnt;
#pragma unroll
        for (int t = 0; t < NTL; ++t) {
          wait(bar_q_full + 8 * t, qcnt & 1);
          if (ulo >= lo[t] && ulo < hi[t]) issue_qk(t, ks);
          // tile t's only QK of this item (or it has none): its Q slot may be refilled once that has run
          if (hi[t] <= lo[t] || hi[t] - 1 <= ulo) commit(bar_q_empty + 8 * t);
        }
        ++qcnt;
        commit(bar_k_empty + 8 * ks);
        kr.advance();
      }
      for (int i = ulo; i < uhi; ++i) {
        const bool nxt = i + 1 < uhi;
        const uint32_t vs = vr.slot;
        const uint32_t ks = kr.slot;          // slot of block i+1 (if any)
        wait_tile(bar_v_full + 8 * vs, vr.phase);   // V of this block (and, with merged barriers, K of the next one)
        bool k_ready = MERGE_KV;
#pragma unroll
        for (int t = 0; t < NTL; ++t) {
          if (i >= lo[t] && i < hi[t]) {
            const bool first = i == lo[t];
            if (first) {   // O_t is overwritten: the previous item's epilogue must have read it
              wait(bar_o_empty + 8 * t, (oecnt[t] & 1) ^ 1);
              ++oecnt[t];
            }
            wait(bar_p_full + 8 * t, pcnt[t] & 1);
            tc_fence_after_sync();
            issue_pv(t, vs, first, F8 && hi[t] - lo[t] <= kTwoTermBlocks);
            ++pcnt[t];
            if (i + 1 == hi[t]) commit(bar_o_full + 8 * t);
          }
          if (nxt && i + 1 >= lo[t] && i + 1 < hi[t]) {
            if (!k_ready) { wait_tile(bar_k_full + 8 * ks, kr.phase); k_ready = true; }
            issue_qk(t, ks);
            // tile t's last QK of the item: its Q slot is refilled during the item's remaining blocks
            if (i + 2 == hi[t]) commit(bar_q_empty + 8 * t);
          }
        }
        commit(bar_v_empty + 8 * vs);
        vr.advance();
        if (nxt) {
          if (!k_ready) wait_tile(bar_k_full + 8 * ks, kr.phase);   // block i+1 belongs to neither tile: still consume its K slot
          commit(bar_k_empty + 8 * ks);
          kr.advance();
        }
      }
    }
    // drain: all MMAs this warp issued must have retired before TMEM is released
    if (leader) umma_commit(bar_drain);
    wait_or_abort(bar_drain, 0, s_abort + 1);
  }
  } else if (NTL == 1 && warp >= 4) {
    // one tile per item: warps 4-7 have no rows; they hand their registers to warps 0-3, whose epilogue holds a
    // 256-column O row, and wait at the final barrier
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
  } else {
    if constexpr (NTL == 1) asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    else asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
    // ========================================= softmax + epilogue =======================================
    const int t = warp >> 2;                       // tile of this warpgroup
    const int r = (warp & 3) * 32 + lane;          // row within the tile == TMEM lane
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS0 = tmem + lane_base + t * TN;
    const uint32_t tO = tmem + lane_base + O_BASE + t * O_STRIDE;
    constexpr bool has_cap = CAP;
    uint32_t scnt = 0, ocnt = 0;
    bool ok = true;

    uint32_t wcnt = 0;
    auto next_work = [&]() -> Item {
      Item it;
      it.w = kEndOfWork;
      const uint32_t slot = wcnt & 1;
      if (!wait_or_abort(bar_w_full + 8 * slot, (wcnt >> 1) & 1, s_abort)) { ok = false; return it; }
      const int4* src = reinterpret_cast<const int4*>(&s_item[slot]);
      int4* dst = reinterpret_cast<int4*>(&it);
#pragma unroll
      for (int i = 0; i < 4; ++i) dst[i] = src[i];
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_w_empty + 8 * slot);
      ++wcnt;
      return it;
    };
    for (Item it = next_work(); it.w != kEndOfWork && ok; it = next_work()) {
      if (!it.valid) continue;
      const int row0 = it.pair * (NTL * TM) + t * TM;
      if (row0 >= it.seqlen_q) continue;           // this tile owns no row
      const int row = row0 + r;
      const int hk = it.h / p.rep;
      float sc = p.scale, vds = 1.f;
      {
        const int di = it.b * p.descale_batch_stride + hk * p.descale_head_stride;
        if (p.q_descale) sc *= p.q_descale[di];
        if (p.k_descale) sc *= p.k_descale[di];
        if (p.v_descale) vds = p.v_descale[di];
      }
      const float c_mul = has_cap ? p.softcap * kLog2e : sc * kLog2e;
      const float cap_in = has_cap ? sc / p.softcap : 0.f;
      const int qp = it.seqlen_k - it.seqlen_q + row;
      int lo = it.leftpad, hi = it.seqlen_k - 1;
      if (p.is_causal) hi = min(hi, qp);
      if (p.window_right >= 0) hi = min(hi, qp + p.window_right);
      if (p.window_left >= 0) lo = max(lo, qp - p.window_left);
      // bounds that hold for every row of the tile (warpgroup-uniform): decide "no masking needed"
      const int qp_first = it.seqlen_k - it.seqlen_q + row0, qp_last = qp_first + TM - 1;
      int lo_max = it.leftpad, hi_min = it.seqlen_k - 1;
      if (p.is_causal) hi_min = min(hi_min, qp_first);
      if (p.window_right >= 0) hi_min = min(hi_min, qp_first + p.window_right);
      if (p.window_left >= 0) lo_max = max(lo_max, qp_last - p.window_left);

      const bool two_term = F8 && (it.hi[t] - it.lo[t] <= kTwoTermBlocks);   // tile-uniform; see the P store below
      float m_used = -INFINITY, l = 0.f;
      float lr = 0.f;   // e4m3 only: sum of the ROUNDED probabilities (normalises O); l stays exact for the LSE
      for (int i = it.lo[t]; i < it.hi[t]; ++i) {
        // (one-tile kernels: S buffer and barrier pair alternate block by block, see SDB)
        const uint32_t sb = SDB ? (scnt & 1) : (uint32_t)t;
        const uint32_t tS = SDB ? tS0 + ((scnt & 1) ? S1_COL : 0u) : tS0;
        ok = wait_or_abort(bar_s_full + 8 * sb, SDB ? ((scnt >> 1) & 1) : (scnt & 1), s_abort);
        ++scnt;
        if (!ok) { report_error(p.status, DEV_ERR_TIMEOUT, ROLE_SOFTMAX); break; }
        tc_fence_after_sync();
        const int n0 = i * TN;
        const bool full = (n0 >= lo_max) && (n0 + TN - 1 <= hi_min);
        uint32_t sreg[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(tS + c * 32, sreg[c]);
        tmem_wait_ld();
        // Fast form of a block (16-bit P, no cap, no masked column, a reference point already taken): the
        // exponentials are taken against the reference point as it stands, WITHOUT looking for the row maximum
        // first (64 of the ~400 instructions of a block, and the chain's time follows its instruction count).
        // Whether the reference was too low shows in the block's row sum afterwards: a probability above
        // 2^kFastShift makes the sum exceed it.  Then (rare: the maximum must have grown by more than kFastShift
        // in log2 units since the reference was taken) the block is done again in the general form below, which
        // overwrites P; nothing has been handed to the MMA warp yet.  Both forms leave P within 2^14, far inside
        // the range of bf16 and fp16, and its relative precision does not depend on the magnitude.
        bool fast_done = false;
        if constexpr (!F8 && !CAP) {
          if (__all_sync(0xffffffffu, full && m_used != -INFINITY)) {
            float2 fs[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
            const float2 c2 = make_float2(c_mul, c_mul), nm2 = make_float2(-m_used, -m_used);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t pk[16];
#pragma unroll
              for (int j = 0; j < 32; j += 2) {
                const float2 y = ffma2(make_float2(__uint_as_float(sreg[c][j]), __uint_as_float(sreg[c][j + 1])), c2, nm2);
                const float2 pp = make_float2(ex2(y.x), ex2(y.y));
                fs[(j >> 1) & 3] = fadd2(fs[(j >> 1) & 3], pp);
                pk[j >> 1] = pack2<TO>(pp.x, pp.y);
              }
              tmem_st16(tS + c * 16, pk);
            }
            const float2 s01 = fadd2(fs[0], fs[1]), s23 = fadd2(fs[2], fs[3]);
            const float2 s4 = fadd2(s01, s23);
            const float blk = s4.x + s4.y;
            if (!__any_sync(0xffffffffu, !(blk <= kFastSumLimit))) {   // (a NaN sum takes the general form too)
              l += blk;
              fast_done = true;
            }
          }
        }
        if (!fast_done) {
        float mx = -INFINITY;
        // tanh is monotonic, so on a block without masked columns the row maximum is taken over the raw scores
        // and the cap moves into the exponential pass: one stream of tanh / exp2 pairs instead of two passes
        // over the row with the maximum between them.
        const bool fuse_cap = !F8 && has_cap && full;
        if (has_cap && !fuse_cap) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int j = 0; j < 32; ++j)
              sreg[c][j] = __float_as_uint(tanh_fast(__uint_as_float(sreg[c][j]) * cap_in));
        }
        if (!full) {
          const int rlo = lo - n0, rhi = hi - n0;
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int col = c * 32 + j;
              if (col < rlo || col > rhi) sreg[c][j] = 0xff800000u;   // -inf
            }
        }
        {
          // eight independent chains instead of one 128-deep dependency chain
          float mxa[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) mxa[j] = -INFINITY;
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int j = 0; j < 32; j += 2)
              mxa[(j >> 1) & 7] = fmax3(mxa[(j >> 1) & 7], __uint_as_float(sreg[c][j]), __uint_as_float(sreg[c][j + 1]));
          mx = fmaxf(fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3])),
                     fmaxf(fmaxf(mxa[4], mxa[5]), fmaxf(mxa[6], mxa[7])));
        }
        // c_mul > 0, so the maximum commutes with the scale
        const float y_max = (fuse_cap ? tanh_fast(mx * cap_in) : mx) * c_mul;
        float corr = 1.f;
        bool rescale = false;
        // m_used is the reference point of the exponentials, p = 2^(y - m_used).  For 16-bit P it is the row
        // maximum when it was last taken, so p <= 2^8 between rescales.  e4m3 P has few exponent values below 1
        // (normal down to 2^-6), so there the reference sits 2^5 BELOW the maximum: p runs up to 2^5..2^8 <= 448
        // and probabilities down to 2^-11 of the maximum keep their three mantissa bits.  Numerator and
        // denominator carry the same factor; the LSE is taken from the reference point and the sum as they are.
        constexpr float kRefShift = F8 ? 5.f : 0.f;
        if (m_used == -INFINITY) {
          m_used = y_max - kRefShift;                 // first block with a visible key (may stay -inf)
        } else if (y_max > m_used + kRescaleThreshold) {
          corr = ex2(m_used - (y_max - kRefShift));
          m_used = y_max - kRefShift;
          l *= corr;
          lr *= corr;
          rescale = true;
        }
        const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
        if (__any_sync(0xffffffffu, rescale)) {
          if constexpr (SDB) {
            // QK(i) was issued before PV(i-1): s_full no longer says that O is complete.  PV(i-1) is the PV number
            // scnt - 2 of this CTA (scnt already counts this block); PV(i) cannot have been issued yet.
            if (scnt >= 2 && !wait_or_abort(bar_pv_done, scnt & 1, s_abort)) ok = false;
            tc_fence_after_sync();
          }
          // O_t of the previous blocks is complete: the commit behind s_full also covered PV_t(i-1); PV_t(i)
          // cannot start before this thread's arrival below
#pragma unroll 1
          for (int c = 0; c < HDV / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(tO + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * corr);
            tmem_st32(tO + c * 32, o);
          }
        }
        float2 psum[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
        const float2 c2 = make_float2(c_mul, c_mul), nm2 = make_float2(neg_m, neg_m);
        if constexpr (!F8) {
          if (!fuse_cap) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t pk[16];
#pragma unroll
              for (int j = 0; j < 32; j += 2) {
                const float2 y = ffma2(make_float2(__uint_as_float(sreg[c][j]), __uint_as_float(sreg[c][j + 1])), c2, nm2);
                const float2 pp = make_float2(ex2(y.x), ex2(y.y));
                psum[(j >> 1) & 3] = fadd2(psum[(j >> 1) & 3], pp);
                pk[j >> 1] = pack2<TO>(pp.x, pp.y);
              }
              tmem_st16(tS + c * 16, pk);
            }
          } else {
            const float2 ci2 = make_float2(cap_in, cap_in);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t pk[16];
#pragma unroll
              for (int j = 0; j < 32; j += 2) {
                const float2 x = fmul2(make_float2(__uint_as_float(sreg[c][j]), __uint_as_float(sreg[c][j + 1])), ci2);
                const float2 y = ffma2(make_float2(tanh_fast(x.x), tanh_fast(x.y)), c2, nm2);
                // tanh and exp2 share the special-function unit, which bounds this loop: every fourth pair
                // takes its exponential on the FMA pipe
                const float2 pp = (((j >> 1) & 3) < kCapEmuPairs) ? ex2_poly2(y) : make_float2(ex2(y.x), ex2(y.y));
                psum[(j >> 1) & 3] = fadd2(psum[(j >> 1) & 3], pp);
                pk[j >> 1] = pack2<TO>(pp.x, pp.y);
              }
              tmem_st16(tS + c * 16, pk);
            }
          }
        } else if (!two_term) {
          // four e4m3 probabilities per TMEM column.  The row sum is taken over the ROUNDED probabilities, so that
          // numerator (P V on the tensor cores) and denominator describe the same weights.
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t pk[8];
            __half2 hs[4] = {__half2(), __half2(), __half2(), __half2()};
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const float2 y0 = ffma2(make_float2(__uint_as_float(sreg[c][j]), __uint_as_float(sreg[c][j + 1])), c2, nm2);
              const float2 y1 = ffma2(make_float2(__uint_as_float(sreg[c][j + 2]), __uint_as_float(sreg[c][j + 3])), c2, nm2);
              const float2 p0 = make_float2(ex2(y0.x), ex2(y0.y)), p1 = make_float2(ex2(y1.x), ex2(y1.y));
              psum[(j >> 2) & 3] = fadd2(psum[(j >> 2) & 3], fadd2(p0, p1));
              const uint32_t q4 = pack4_e4m3(p0.x, p0.y, p1.x, p1.y);
              pk[j >> 2] = q4;
              const uint32_t h0 = e4m3x2_to_f16x2((uint16_t)(q4 & 0xffffu)), h1 = e4m3x2_to_f16x2((uint16_t)(q4 >> 16));
              hs[(j >> 2) & 3] = __hadd2(hs[(j >> 2) & 3],
                                         __hadd2(*reinterpret_cast<const __half2*>(&h0), *reinterpret_cast<const __half2*>(&h1)));
            }
            tmem_st8(tS + c * 8, pk);
            const float2 f01 = __half22float2(__hadd2(hs[0], hs[1])), f23 = __half22float2(__hadd2(hs[2], hs[3]));
            lr += (f01.x + f23.x) + (f01.y + f23.y);
          }
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            // A tile whose rows see at most kTwoTermBlocks key blocks in all (256 keys: the first rows of a causal
            // sequence, short sequences) has little averaging over keys to hide the 3-bit mantissa of P: there P
            // is written as two e4m3 terms, P_hi + P_lo with P_lo = round(P - P_hi), and the MMA warp runs PV
            // over both.  Kept apart from the common path above, whose loop body must stay small: the softmax
            // warps run out of the instruction cache (with this code inside the common loop the e4m3 kernel fell
            // from 1160 to 767 TFLOP/s).
            uint32_t pk[8], pl[8];
            float lsum = 0.f;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const float2 y0 = ffma2(make_float2(__uint_as_float(sreg[c][j]), __uint_as_float(sreg[c][j + 1])), c2, nm2);
              const float2 y1 = ffma2(make_float2(__uint_as_float(sreg[c][j + 2]), __uint_as_float(sreg[c][j + 3])), c2, nm2);
              const float2 p0 = make_float2(ex2(y0.x), ex2(y0.y)), p1 = make_float2(ex2(y1.x), ex2(y1.y));
              psum[(j >> 2) & 3] = fadd2(psum[(j >> 2) & 3], fadd2(p0, p1));
              const uint32_t q4 = pack4_e4m3(p0.x, p0.y, p1.x, p1.y);
              pk[j >> 2] = q4;
              const uint32_t h0 = e4m3x2_to_f16x2((uint16_t)(q4 & 0xffffu)), h1 = e4m3x2_to_f16x2((uint16_t)(q4 >> 16));
              const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&h0));
              const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&h1));
              const uint32_t r4 = pack4_e4m3(p0.x - f0.x, p0.y - f0.y, p1.x - f1.x, p1.y - f1.y);
              pl[j >> 2] = r4;
              const uint32_t g0 = e4m3x2_to_f16x2((uint16_t)(r4 & 0xffffu)), g1 = e4m3x2_to_f16x2((uint16_t)(r4 >> 16));
              const float2 e0 = __half22float2(*reinterpret_cast<const __half2*>(&g0));
              const float2 e1 = __half22float2(*reinterpret_cast<const __half2*>(&g1));
              lsum += ((f0.x + e0.x) + (f0.y + e0.y)) + ((f1.x + e1.x) + (f1.y + e1.y));
            }
            tmem_st8(tS + c * 8, pk);
            tmem_st8(tS + 32 + c * 8, pl);
            lr += lsum;
          }
        }
        {
          const float2 s01 = fadd2(psum[0], psum[1]), s23 = fadd2(psum[2], psum[3]);
          const float2 s4 = fadd2(s01, s23);
          l += s4.x + s4.y;
        }
        }   // general form
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_p_full + 8 * sb);
      }
      if (!ok) break;
      if (CAP && kCapEmuPairs > 0 && m_used == -INFINITY) l = 0.f;   // the cubic never returns exactly 0

      // ---- epilogue of this tile ----
      if constexpr (HDV <= 128) {
        // The whole O row goes to registers first and O_t is released at once: the MMA warp may start the next
        // item's first PV while this thread is still normalising and storing.
        const bool had_blocks = it.hi[t] > it.lo[t];
        uint32_t o[HDV / 32][32];
        if (had_blocks) {
          ok = wait_or_abort(bar_o_full + 8 * t, ocnt & 1, s_abort);
          ++ocnt;
          if (!ok) { report_error(p.status, DEV_ERR_TIMEOUT, ROLE_EPILOGUE); break; }
          tc_fence_after_sync();
  #pragma unroll
          for (int c = 0; c < HDV / 32; ++c) tmem_ld32(tO + c * 32, o[c]);
          tmem_wait_ld();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_o_empty + 8 * t);
        } else {
  #pragma unroll
          for (int c = 0; c < HDV / 32; ++c)
  #pragma unroll
            for (int j = 0; j < 32; ++j) o[c][j] = 0u;
        }
        float m_fin = m_used, l_fin = l, osc = 1.f;
        float l_norm = F8 ? lr : l;          // what O is divided by
        if (p.s_aux) {
          const float ys = p.s_aux[it.h] * kLog2e;
          const float mn = fmaxf(m_used, ys);
          osc = (m_used == -INFINITY) ? 0.f : ex2(m_used - mn);
          const float sink = ex2(ys - mn);
          l_fin = l * osc + sink;
          l_norm = l_norm * osc + sink;
          m_fin = mn;
        }
        const float inv = l_norm > 0.f ? osc * vds / l_norm : 0.f;
        const float2 inv2 = make_float2(inv, inv);
        const bool row_ok = row < it.seqlen_q;
        const int wrow0 = row0 + (warp & 3) * 32;            // first row of this warp's 32
        bool staged = false;
        if constexpr (SM::kStageOut) staged = a.stage_out && (wrow0 + 32 <= it.seqlen_q);   // warp-uniform
        if (staged) {
          if constexpr (SM::kStageOut) {
            const uint32_t stg = base + SM::kStageOff + (uint32_t)warp * 4096u;
  #pragma unroll
            for (int hf = 0; hf < HDV / 64; ++hf) {
              uint32_t pk[32];
  #pragma unroll
              for (int j = 0; j < 32; ++j) {
                const float2 v = fmul2(make_float2(__uint_as_float(o[2 * hf + (j >> 4)][(2 * j) & 31]),
                                                   __uint_as_float(o[2 * hf + (j >> 4)][((2 * j) & 31) + 1])), inv2);
                pk[j] = pack2<TO>(v.x, v.y);
              }
              // the store issued for the previous 64 columns (or the previous item) must have read the buffer
              if (lane == 0) bulk_wait_read_all();
              __syncwarp();
  #pragma unroll
              for (int c = 0; c < 8; ++c) {   // 16-byte chunk c of row `lane`, at its 128-byte-swizzle position
                const uint32_t addr = stg + (uint32_t)lane * 128u + ((uint32_t)(c ^ (lane & 7)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk[4 * c]), "r"(pk[4 * c + 1]),
                             "r"(pk[4 * c + 2]), "r"(pk[4 * c + 3]) : "memory");
              }
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_3d(&map_o, stg, hf * 64, it.h, it.q0 + wrow0);
                bulk_commit_group();
              }
            }
          }
        } else if (row_ok) {
          if (p.out_f32) {
            float* op = reinterpret_cast<float*>(p.out) + (int64_t)(it.q0 + row) * p.o_row_stride + (int64_t)it.h * p.o_head_stride;
  #pragma unroll
            for (int c = 0; c < HDV / 32; ++c) {
              if (c * 32 < a.out_cols) {
  #pragma unroll
                for (int j = 0; j < 32; j += 4)
                  *reinterpret_cast<float4*>(op + c * 32 + j) =
                      make_float4(__uint_as_float(o[c][j]) * inv, __uint_as_float(o[c][j + 1]) * inv,
                                  __uint_as_float(o[c][j + 2]) * inv, __uint_as_float(o[c][j + 3]) * inv);
              }
            }
          } else {
            TO* op = reinterpret_cast<TO*>(p.out) + (int64_t)(it.q0 + row) * p.o_row_stride + (int64_t)it.h * p.o_head_stride;
  #pragma unroll
            for (int c = 0; c < HDV / 32; ++c) {
              if (c * 32 < a.out_cols) {
  #pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  uint4 v;
                  v.x = pack2<TO>(__uint_as_float(o[c][j]) * inv, __uint_as_float(o[c][j + 1]) * inv);
                  v.y = pack2<TO>(__uint_as_float(o[c][j + 2]) * inv, __uint_as_float(o[c][j + 3]) * inv);
                  v.z = pack2<TO>(__uint_as_float(o[c][j + 4]) * inv, __uint_as_float(o[c][j + 5]) * inv);
                  v.w = pack2<TO>(__uint_as_float(o[c][j + 6]) * inv, __uint_as_float(o[c][j + 7]) * inv);
                  *reinterpret_cast<uint4*>(op + c * 32 + j) = v;
                }
              }
            }
          }
        }
        if (row_ok)
          p.lse[(int64_t)it.h * p.total_q + it.q0 + row] = l_fin > 0.f ? (m_fin + lg2(l_fin)) * kLn2 : -INFINITY;
      } else {
        // HDV > 128 (one tile per item): the O row is read 64 columns at a time; O_t is released as soon as its last
        // column has been read.  Each 64-column group leaves like a half row of the two-tile form: staged + one TMA
        // store where the warp's 32 rows all lie inside the sequence, direct stores otherwise.
        constexpr int NG = HDV / 64;
        const bool had_blocks = it.hi[t] > it.lo[t];
        if (had_blocks) {
          ok = wait_or_abort(bar_o_full + 8 * t, ocnt & 1, s_abort);
          ++ocnt;
          if (!ok) { report_error(p.status, DEV_ERR_TIMEOUT, ROLE_EPILOGUE); break; }
          tc_fence_after_sync();
        }
        float m_fin = m_used, l_fin = l, osc = 1.f;
        float l_norm = F8 ? lr : l;          // what O is divided by
        if (p.s_aux) {
          const float ys = p.s_aux[it.h] * kLog2e;
          const float mn = fmaxf(m_used, ys);
          osc = (m_used == -INFINITY) ? 0.f : ex2(m_used - mn);
          const float sink = ex2(ys - mn);
          l_fin = l * osc + sink;
          l_norm = l_norm * osc + sink;
          m_fin = mn;
        }
        const float inv = l_norm > 0.f ? osc * vds / l_norm : 0.f;
        const float2 inv2 = make_float2(inv, inv);
        const bool row_ok = row < it.seqlen_q;
        const int wrow0 = row0 + (warp & 3) * 32;            // first row of this warp's 32
        bool staged = false;
        if constexpr (SM::kStageOut) staged = a.stage_out && (wrow0 + 32 <= it.seqlen_q);   // warp-uniform
#pragma unroll 1
        for (int g = 0; g < NG; ++g) {
          uint32_t o[2][32];
          if (had_blocks) {
            tmem_ld32(tO + g * 64, o[0]);
            tmem_ld32(tO + g * 64 + 32, o[1]);
            tmem_wait_ld();
            if (g + 1 == NG) {     // the whole row has been read
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(bar_o_empty + 8 * t);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) { o[0][j] = 0u; o[1][j] = 0u; }
          }
          if (staged) {
            if constexpr (SM::kStageOut) {
              const uint32_t stg = base + SM::kStageOff + (uint32_t)warp * 4096u;
              uint32_t pk[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const float2 v = fmul2(make_float2(__uint_as_float(o[j >> 4][(2 * j) & 31]),
                                                   __uint_as_float(o[j >> 4][((2 * j) & 31) + 1])), inv2);
                pk[j] = pack2<TO>(v.x, v.y);
              }
              if (lane == 0) bulk_wait_read_all();   // the previous store must have read the buffer
              __syncwarp();
#pragma unroll
              for (int c = 0; c < 8; ++c) {   // 16-byte chunk c of row `lane`, at its 128-byte-swizzle position
                const uint32_t addr = stg + (uint32_t)lane * 128u + ((uint32_t)(c ^ (lane & 7)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk[4 * c]), "r"(pk[4 * c + 1]),
                             "r"(pk[4 * c + 2]), "r"(pk[4 * c + 3]) : "memory");
              }
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_3d(&map_o, stg, g * 64, it.h, it.q0 + wrow0);
                bulk_commit_group();
              }
            }
          } else if (row_ok) {
            if (p.out_f32) {
              float* op = reinterpret_cast<float*>(p.out) + (int64_t)(it.q0 + row) * p.o_row_stride + (int64_t)it.h * p.o_head_stride + g * 64;
#pragma unroll
              for (int c = 0; c < 2; ++c)
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                  *reinterpret_cast<float4*>(op + c * 32 + j) =
                      make_float4(__uint_as_float(o[c][j]) * inv, __uint_as_float(o[c][j + 1]) * inv,
                                  __uint_as_float(o[c][j + 2]) * inv, __uint_as_float(o[c][j + 3]) * inv);
            } else {
              TO* op = reinterpret_cast<TO*>(p.out) + (int64_t)(it.q0 + row) * p.o_row_stride + (int64_t)it.h * p.o_head_stride + g * 64;
#pragma unroll
              for (int c = 0; c < 2; ++c)
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  uint4 v;
                  v.x = pack2<TO>(__uint_as_float(o[c][j]) * inv, __uint_as_float(o[c][j + 1]) * inv);
                  v.y = pack2<TO>(__uint_as_float(o[c][j + 2]) * inv, __uint_as_float(o[c][j + 3]) * inv);
                  v.z = pack2<TO>(__uint_as_float(o[c][j + 4]) * inv, __uint_as_float(o[c][j + 5]) * inv);
                  v.w = pack2<TO>(__uint_as_float(o[c][j + 6]) * inv, __uint_as_float(o[c][j + 7]) * inv);
                  *reinterpret_cast<uint4*>(op + c * 32 + j) = v;
                }
            }
          }
        }
        if (row_ok)
          p.lse[(int64_t)it.h * p.total_q + it.q0 + row] = l_fin > 0.f ? (m_fin + lg2(l_fin)) * kLn2 : -INFINITY;
      }
    }
    if constexpr (SM::kStageOut) {
      if (lane == 0) bulk_wait_all();   // this lane's output stores have completed before the CTA leaves
    }
    if (!ok) *s_abort = 1;
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == WARP_MMA) { tc_fence_after_sync(); tmem_dealloc(tmem, 512); }
}

// ------------------------------------------------------------------------------------------------------
// host side: tensor maps + launch
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

// 3-D map over [rows][heads][head_dim] (innermost first: column, head, row); box = 128 bytes of one head x box_rows
// rows.  Columns of a box past head_dim are filled with zeros, which is how head_dim 96 rides on the 128-wide kernel.
// Encoding is pure host arithmetic on its arguments, so the last few results are kept per thread: a serving loop
// that calls with the same tensors again (the KV pool, a reused Q/O buffer) skips the driver call.
struct MapKey {
  const void* ptr;
  uint64_t rows, heads, head_dim, head_stride, row_stride;
  uint32_t box_rows;
  int dtype;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && heads == o.heads && head_dim == o.head_dim && head_stride == o.head_stride &&
           row_stride == o.row_stride && box_rows == o.box_rows && dtype == o.dtype;
  }
};
struct MapCache {
  static constexpr int N = 16;
  MapKey key[N];
  CUtensorMap map[N];
  bool used[N] = {};
  int next = 0;
};

static bool make_map_3d(CUtensorMap* m, const void* ptr, int dtype, uint64_t rows, uint64_t heads, uint64_t head_dim,
                        uint64_t head_stride_elems, uint64_t row_stride_elems, uint32_t box_rows) {
  static thread_local MapCache cache;
  const MapKey k{ptr, rows, heads, head_dim, head_stride_elems, row_stride_elems, box_rows, dtype};
  for (int i = 0; i < MapCache::N; ++i)
    if (cache.used[i] && cache.key[i] == k) { *m = cache.map[i]; return true; }
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  const uint32_t esz = dtype == FA_DT_FP8_E4M3 ? 1 : 2;
  const cuuint64_t dims[3] = {head_dim, heads, rows};
  const cuuint64_t strides[2] = {head_stride_elems * esz, row_stride_elems * esz};
  const cuuint32_t box[3] = {128 / esz, 1, box_rows};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = dtype == FA_DT_FP8_E4M3 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : dtype == FA_DT_FP16   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                         : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const bool good = fn(m, dt, 3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  if (!good) return false;
  const int slot = cache.next;
  cache.next = (cache.next + 1) % MapCache::N;
  cache.key[slot] = k;
  cache.map[slot] = *m;
  cache.used[slot] = true;
  return true;
}

// The whole warp produces where a tile is many boxes or many rows (pages of <= 32 keys) and, on pages of 64 keys,
// where K rides on V's barrier (equal ring depths: measured 1034 -> 1055 TFLOP/s, 1078 -> 1135 on a 1024-row chunk
// over 32768 keys); lane 0 alone otherwise (a tile of a page of >= 128 keys is one box: 1143 against 1117 wide).
template <int KST, int VST>
static bool producer_is_wide(const KParams& kp) {
  if (kp.page_table == nullptr) return false;
  return kp.page_size <= 32 || (KST == VST && kp.page_size <= 64);
}

template <typename T, int HD, int HDV, int KST, int VST, int NTL, bool CAP, int PROD>
static int launch_prod(const KParams& kp, const Plan& pl, int dtype, uint64_t kv_rows, cudaStream_t stream) {
  using SM = Smem<Elem<T>::kSize, HD, HDV, KST, VST, NTL>;
  TcArgs a;
  a.kp = kp;
  a.item_rows = NTL * TM;
  a.max_pairs = (kp.max_seqlen_q + a.item_rows - 1) / a.item_rows;
  a.num_items = kp.batch * kp.hq * a.max_pairs;
  a.use_list = kp.work != nullptr;
  // bytes of K and V the batch can touch, against the L2 capacity the tiles of concurrently running heads share
  {
    const double kv_bytes = (double)kp.batch * kp.hkv * (double)kp.max_seqlen_k * (kp.hd + kp.hdv) * Elem<T>::kSize;
    a.head_major = kv_bytes > kHeadMajorBytes;
  }
  const bool paged = kp.page_table != nullptr;
  a.gather = paged && (kp.page_size == 1 || kp.page_size == 2 || kp.page_size == 4);
  a.kv_box_rows = a.gather ? 1 : (paged ? (kp.page_size < TN ? kp.page_size : TN) : TN);
  if ((PROD != 0) != paged || (PROD == 2) != producer_is_wide<KST, VST>(kp)) return -1;
  a.kv_total_rows = (int)kv_rows;
  a.out_cols = kp.hdv;
  CUtensorMap mq, mk, mv, mo;
  if (!make_map_3d(&mq, kp.q, dtype, (uint64_t)kp.total_q, kp.hq, kp.hd, kp.hd, (uint64_t)kp.q_row_stride, TM)) return -1;
  if (!make_map_3d(&mk, kp.k, dtype, kv_rows, kp.hkv, kp.hd, kp.hd, (uint64_t)kp.k_row_stride, a.kv_box_rows)) return -1;
  if (!make_map_3d(&mv, kp.v, dtype, kv_rows, kp.hkv, kp.hdv, kp.hdv, (uint64_t)kp.v_row_stride, a.kv_box_rows)) return -1;
  // output map (16-bit element type of the output): 64 columns x 32 rows per store.  A layout TMA cannot describe
  // only switches the staged path off.
  a.stage_out = 0;
  mo = mq;
  if (SM::kStageOut && !kp.out_f32) {
    const int odt = dtype == FA_DT_FP16 ? FA_DT_FP16 : FA_DT_BF16;
    if (make_map_3d(&mo, kp.out, odt, (uint64_t)kp.total_q, kp.hq, kp.hdv, (uint64_t)kp.o_head_stride,
                    (uint64_t)kp.o_row_stride, 32))
      a.stage_out = 1;
  }
  auto kern = fwd_prefill_tc_kernel<T, HD, HDV, KST, VST, NTL, CAP, PROD>;
  int smem = SM::kBytes + 1024;
  if (smem < 120 * 1024) smem = 120 * 1024;   // one CTA per SM: the CTA owns all 512 TMEM columns
  static std::atomic<unsigned long long> attr_done{0};   // one bit per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !((attr_done.load(std::memory_order_acquire) >> dev) & 1ull)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    if (dev >= 0 && dev < 64) attr_done.fetch_or(1ull << dev, std::memory_order_release);
  }
  const int grid = a.num_items < pl.num_sms ? a.num_items : pl.num_sms;
  if (grid <= 0) return 0;
  kern<<<grid, NTHREADS, smem, stream>>>(a, mq, mk, mv, mo);
  return (int)cudaGetLastError();
}

template <typename T, int HD, int HDV, int KST, int VST, int NTL, bool CAP>
static int launch_cap(const KParams& kp, const Plan& pl, int dtype, uint64_t kv_rows, cudaStream_t stream) {
  if (kp.page_table == nullptr) return launch_prod<T, HD, HDV, KST, VST, NTL, CAP, 0>(kp, pl, dtype, kv_rows, stream);
  return producer_is_wide<KST, VST>(kp) ? launch_prod<T, HD, HDV, KST, VST, NTL, CAP, 2>(kp, pl, dtype, kv_rows, stream)
                                        : launch_prod<T, HD, HDV, KST, VST, NTL, CAP, 1>(kp, pl, dtype, kv_rows, stream);
}

template <typename T, int HD, int HDV, int KST, int VST, int NTL = 2>
static int launch_impl(const KParams& kp, const Plan& pl, int dtype, uint64_t kv_rows, cudaStream_t stream) {
  return kp.softcap > 0.f ? launch_cap<T, HD, HDV, KST, VST, NTL, true>(kp, pl, dtype, kv_rows, stream)
                          : launch_cap<T, HD, HDV, KST, VST, NTL, false>(kp, pl, dtype, kv_rows, stream);
}

}  // namespace tc

// Shapes the tensor-core prefill route takes. Layout conditions (heads back to back inside a row, pages
// back to back) are checked at launch: fa_b200_fwd re-plans onto the general route when they do not hold.
// Head dims whose O accumulator leaves TMEM room for one query tile only (work items of 128 rows).
bool prefill_tc_single_tile(int hd, int hdv) { return (hd == 256 && hdv == 256) || (hd == 192 && hdv == 192); }

bool prefill_tc_supported(const PlanInput& in) {
  if (in.q_dtype != in.kv_dtype) return false;
  const bool hd_ok = (in.hd == 64 && in.hdv == 64) || (in.hd == 128 && in.hdv == 128) || (in.hd == 192 && in.hdv == 128) ||
                     (in.hd == 96 && in.hdv == 96) ||   // 96 runs as 128: TMA zero-fills columns 96..127
                     prefill_tc_single_tile(in.hd, in.hdv);
  if (!hd_ok) return false;
  if (in.q_dtype == FA_DT_FP8_E4M3 && !(in.hd == 128 && in.hdv == 128)) return false;   // e4m3: head_dim 128 only
  if (in.page_size > 0) {
    const int ps = in.page_size;
    const bool gather = (ps == 1 || ps == 2 || ps == 4) && in.hd != 96;   // rows by cp.async (whole rows: no zero-filled columns)
    if (!gather && (ps % 8 != 0 || !((128 % ps == 0) || (ps % 128 == 0)))) return false;
  }
  return in.hkv > 0 && in.hq % in.hkv == 0;
}

bool prefill_tc_layout_ok(const FaFwdParams* p) {
  if (p->q_head_stride != p->hd || p->k_head_stride != p->hd || p->v_head_stride != p->hdv) return false;
  if (p->q_row_stride < (int64_t)p->hq * p->hd) return false;
  if (p->page_table) {
    if (p->k_page_stride != (int64_t)p->page_size * p->k_row_stride) return false;
    if (p->v_page_stride != (int64_t)p->page_size * p->v_row_stride) return false;
    if (p->num_pages <= 0) return false;
  }
  return true;
}

int launch_prefill_tc(const KParams& kp, const Plan& pl, int dtype, cudaStream_t stream) {
  const uint64_t kv_rows = kp.page_table ? (uint64_t)kp.num_pages * (uint64_t)kp.page_size : (uint64_t)kp.total_k;
  const bool bf = dtype != FA_DT_FP16;
  if (kp.q_fp8 && kp.kv_fp8)
    return kp.hd == 128 && kp.hdv == 128 ? tc::launch_impl<tc::fp8_t, 128, 128, 4, 4>(kp, pl, FA_DT_FP8_E4M3, kv_rows, stream) : -1;
  if ((kp.hd == 128 && kp.hdv == 128) || (kp.hd == 96 && kp.hdv == 96))
    return bf ? tc::launch_impl<__nv_bfloat16, 128, 128, 2, 2>(kp, pl, dtype, kv_rows, stream)
              : tc::launch_impl<__half, 128, 128, 2, 2>(kp, pl, dtype, kv_rows, stream);
  if (kp.hd == 64 && kp.hdv == 64)
    return bf ? tc::launch_impl<__nv_bfloat16, 64, 64, 3, 3>(kp, pl, dtype, kv_rows, stream)
              : tc::launch_impl<__half, 64, 64, 3, 3>(kp, pl, dtype, kv_rows, stream);
  if (kp.hd == 192 && kp.hdv == 128)
    return bf ? tc::launch_impl<__nv_bfloat16, 192, 128, 2, 1>(kp, pl, dtype, kv_rows, stream)
              : tc::launch_impl<__half, 192, 128, 2, 1>(kp, pl, dtype, kv_rows, stream);
  if (kp.hd == 256 && kp.hdv == 256)
    return bf ? tc::launch_impl<__nv_bfloat16, 256, 256, 1, 1, 1>(kp, pl, dtype, kv_rows, stream)
              : tc::launch_impl<__half, 256, 256, 1, 1, 1>(kp, pl, dtype, kv_rows, stream);
  if (kp.hd == 192 && kp.hdv == 192)
    return bf ? tc::launch_impl<__nv_bfloat16, 192, 192, 1, 2, 1>(kp, pl, dtype, kv_rows, stream)
              : tc::launch_impl<__half, 192, 192, 1, 2, 1>(kp, pl, dtype, kv_rows, stream);
  return -1;
}

}  // namespace fa
