// fa_sched.h — layout of the scheduler metadata (int32 words) and the host-side plan that fixes its
// geometry.  The same layout is restated on the CPU in oracle/sched_oracle.py; the two must agree
// bit for bit.
//
// words [0,16): header
//   [0] magic  [1] layout version  [2] batch  [3] nsplits  [4] tile_m  [5] tile_n  [6] num_work
//   [7] max_mtiles  [8] rows_per_token  [9] route  [10] sorted (1 = entries are in LPT order)  [11..15] 0
// words [16 + 4*i, 16 + 4*i + 4): work entry i = {batch, m_tile, n_lo, n_hi}; key blocks in units of
//   tile_n keys, before the split sub-division.  With `sorted` the entries that own at least one query
//   row come first, by descending (n_hi - n_lo), ties by ascending (batch * max_mtiles + m_tile); the
//   remaining slots hold {-1, -1, 0, 0}.  Without it (more than kSchedSortMax slots, or more than
//   kSchedCountMax key blocks in a sequence) slot i describes
//   (batch, m_tile) = (i / max_mtiles, i % max_mtiles), batch = -1 when it owns no row, and num_work is
//   the slot count.
#pragma once
#include <stdint.h>

#include "../../include/fa_b200.h"

namespace fa {

constexpr int32_t kSchedMagic = 0x46413230;
constexpr int32_t kSchedVersion = 1;
constexpr int kSchedHeader = 16;
constexpr int kSchedSortMax = 8192;
// sort key = (kSchedCountMax - block count) << kSchedSlotBits | slot: the list is sorted only while every block
// count fits the 19 bits above the 13 slot bits
constexpr int kSchedSlotBits = 13;
constexpr int kSchedCountMax = (1 << 18) - 1;
inline bool sched_is_sorted(int slots, int max_seqlen_k, int tile_n) {
  return slots <= kSchedSortMax && (max_seqlen_k + tile_n - 1) / tile_n <= kSchedCountMax;
}
// The decode route packs the rep*q_len query rows of one kv head into 16-row tiles; each tile is a work item that
// streams the KV once, so the route is taken while that many passes still beat the other routes.
constexpr int kDecodeMaxRows = 64;

struct Plan {
  int route;            // FA_ROUTE_* actually taken (never AUTO)
  int tile_m, tile_n;   // rows (packed rows when rows_per_token > 1) and keys per tile
  int rows_per_token;   // hq/hkv when the q heads of one kv head are packed into the M tile, else 1
  int max_mtiles;       // ceil(max_seqlen_q * rows_per_token / tile_m)
  int nsplits;          // >= 1
  int num_sms;          // SMs the plan may use (device SM count - sm_margin)
  int err;              // FA_OK or FA_ERR_*
};

// Shape facts the plan depends on; filled from FaFwdParams or FaSchedParams.
struct PlanInput {
  int batch, max_seqlen_q, max_seqlen_k, hq, hkv, hd, hdv;
  int q_dtype, kv_dtype;
  int page_size;   // 0 = not paged
  int is_causal, window_left, window_right, has_softcap;
  int num_splits, sm_margin, route;
  int num_sms_device;
  int tc_layout_ok;   // strides allow the 2-D TMA views the tensor-core prefill route needs
};

Plan make_plan(const PlanInput& in);

// What a kernel expects to find in the header of a scheduler-metadata tensor before it indexes the entries:
// the geometry the plan of THIS call fixed.  Metadata made for another batch size, tile shape, split count or
// route is refused (the kernel records DEV_ERR_BAD_INDEX and produces nothing) instead of being read as ranges.
struct SchedExpect {
  int32_t batch, nsplits, tile_m, tile_n, max_mtiles, rows_per_token, route;
};
#if defined(__CUDACC__)
__host__ __device__
#endif
inline bool sched_header_matches(const int32_t* h, const SchedExpect& e) {
  return h[0] == kSchedMagic && h[1] == kSchedVersion && h[2] == e.batch && h[3] == e.nsplits && h[4] == e.tile_m &&
         h[5] == e.tile_n && h[7] == e.max_mtiles && h[8] == e.rows_per_token && h[9] == e.route && h[6] >= 0 &&
         h[6] <= e.batch * e.max_mtiles;
}

inline int sched_len(const Plan& pl, int batch) { return kSchedHeader + 4 * batch * pl.max_mtiles; }

}  // namespace fa
