"""Integer oracle (TEST INFRASTRUCTURE ONLY): CPU restatement of every index computation on the path.

The reference pins only the *shape* of its scheduler metadata (`zeros({1}, int32)`,
kernels/fa4_blackwell.cu:10175-10183), so the content of ours is "parity unpinned" with respect to the
reference; what is pinned against reference code is the arithmetic the metadata is made of:

  * key-block range of a query tile under causal / window / sequence length
    (kernels/fa4_blackwell.cu:5846-5854), extended by the leftpad prune (kernels/fa3_hopper.cu:326-332);
  * the split sub-range `per = ceil(total / nsplits)` (kernels/fa4_blackwell.cu:5855-5856);
  * the physical row of key `kk` in a paged cache, `page_table[b, kk // page] * page + kk % page`
    (kernels/fa4_blackwell.cu:5868);
  * window normalisation before routing (kernels/fa4_blackwell.cu:10148-10153).

The plan (route, tile geometry, split count) and the metadata layout restate this repository's own host
planner and must match it bit for bit.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

MAGIC, VERSION, HEADER, SORT_MAX = 0x46413230, 1, 16, 8192
COUNT_MAX = (1 << 18) - 1   # block counts above this do not fit the device sort key: the list stays unsorted
ROUTE_AUTO, ROUTE_PREFILL_TC, ROUTE_DECODE, ROUTE_GENERAL = 0, 1, 2, 3
DT_BF16, DT_FP16, DT_FP8 = 0, 1, 2
# which kernel families the library under test ships (the planner only routes to these)
TC_ENABLED, DECODE_ENABLED = True, True


def cdiv(a: int, b: int) -> int:
    return (a + b - 1) // b


def nblock_range(seqlen_k, leftpad, qp_min, qp_max, causal, win_l, win_r, tn):
    n_lo, n_hi = 0, cdiv(seqlen_k, tn)
    if causal:
        n_hi = min(n_hi, qp_max // tn + 1 if qp_max >= 0 else 0)
    if win_r >= 0:
        last = qp_max + win_r
        n_hi = min(n_hi, last // tn + 1 if last >= 0 else 0)
    if win_l >= 0:
        first = qp_min - win_l
        if first > 0:
            n_lo = first // tn
    if leftpad > 0:
        n_lo = max(n_lo, leftpad // tn)
    return min(n_lo, n_hi), n_hi


def split_range(lo, hi, s, nsplits):
    per = cdiv(hi - lo, nsplits)
    return min(hi, lo + s * per), min(hi, lo + (s + 1) * per)


def page_row(page_table_row: Sequence[int], kk: int, page: int) -> int:
    return int(page_table_row[kk // page]) * page + kk % page


def normalize_window(causal, max_seqlen_k, wl, wr):
    if causal and wr >= 0:
        wr = -1
    if wl >= 0 and max_seqlen_k > 0 and wl >= max_seqlen_k - 1:
        wl = -1
    if wr >= 0 and max_seqlen_k > 0 and wr >= max_seqlen_k - 1:
        wr = -1
    return wl, wr


@dataclass
class Plan:
    route: int
    tile_m: int
    tile_n: int
    rows_per_token: int
    max_mtiles: int
    nsplits: int
    num_sms: int


def prefill_tc_supported(*, hq, hkv, hd, hdv, q_dtype, kv_dtype, page_size) -> bool:
    if q_dtype != kv_dtype:
        return False
    if (hd, hdv) not in ((64, 64), (96, 96), (128, 128), (192, 128), (256, 256), (192, 192)):
        return False
    if q_dtype == DT_FP8 and (hd, hdv) != (128, 128):
        return False
    gather = page_size in (1, 2, 4) and hd != 96      # rows copied with cp.async
    if page_size and not gather and not (page_size % 8 == 0 and (128 % page_size == 0 or page_size % 128 == 0)):
        return False
    return hq % hkv == 0


def decode_supported(*, hq, hkv, hd, hdv, q_dtype, kv_dtype, page_size) -> bool:
    if q_dtype == DT_FP8 or (kv_dtype != q_dtype and kv_dtype != DT_FP8):
        return False
    if not ((hd, hdv) == (128, 128) or (kv_dtype != DT_FP8 and (hd, hdv) in ((64, 64), (192, 128)))):
        return False
    if not (page_size in (0, 1, 2, 4, 8, 16, 32) or page_size % 64 == 0):   # contiguous, gathered, atoms of a 64-row stage, whole stages
        return False
    return hq % hkv == 0


DECODE_MAX_ROWS = 64   # rep*q_len rows of one kv head, in 16-row tiles (fa_sched.h: kDecodeMaxRows)


def make_plan(*, batch, max_seqlen_q, max_seqlen_k, hq, hkv, hd, hdv, q_dtype=DT_BF16, kv_dtype=None, page_size=0,
              num_splits=0, sm_margin=0, route=ROUTE_AUTO, num_sms_device=148, tc_enabled=None,
              decode_enabled=None) -> Plan:
    kv_dtype = q_dtype if kv_dtype is None else kv_dtype
    tc_enabled = TC_ENABLED if tc_enabled is None else tc_enabled
    decode_enabled = DECODE_ENABLED if decode_enabled is None else decode_enabled
    num_sms = max(1, num_sms_device - max(sm_margin, 0))
    rep = hq // hkv
    shape = dict(hq=hq, hkv=hkv, hd=hd, hdv=hdv, q_dtype=q_dtype, kv_dtype=kv_dtype, page_size=page_size)
    tc_ok = tc_enabled and prefill_tc_supported(**shape)
    dec_ok = decode_enabled and decode_supported(**shape)
    if route == ROUTE_AUTO:
        if dec_ok and max_seqlen_q * rep <= DECODE_MAX_ROWS:
            route = ROUTE_DECODE
        elif tc_ok:
            route = ROUTE_PREFILL_TC
        else:
            route = ROUTE_GENERAL
    if route == ROUTE_PREFILL_TC:
        # one 128-row tile per work item where the O accumulator (hdv > 128 columns) leaves TMEM no room for two
        tile_m, tile_n, rpt = (128 if (hd, hdv) in ((256, 256), (192, 192)) else 256), 128, 1
    elif route == ROUTE_DECODE:
        tile_m, tile_n, rpt = 16, 64, rep
    else:
        tile_m, tile_n, rpt = 64, 64, rep
    max_mtiles = cdiv(max_seqlen_q * rpt, tile_m)
    max_nb = cdiv(max_seqlen_k, tile_n) if max_seqlen_k > 0 else 1
    heads = hkv if rpt > 1 else hq
    ctas = batch * heads * max_mtiles
    s = 1
    if route == ROUTE_PREFILL_TC or num_splits == 1:
        s = 1
    elif num_splits > 1:
        s = min(num_splits, max_nb)
    elif route != ROUTE_PREFILL_TC and ctas > 0 and ctas * 2 <= num_sms and max_nb >= 8:
        s = min(num_sms // ctas, max_nb // 4, 64)
    return Plan(route, tile_m, tile_n, rpt, max_mtiles, max(s, 1), num_sms)


def scheduler_metadata(plan: Plan, *, batch, max_seqlen_q, max_seqlen_k, q_lens: Optional[Sequence[int]],
                       k_lens: Optional[Sequence[int]], leftpad: Optional[Sequence[int]], causal, window_left,
                       window_right) -> List[int]:
    """The int32 words `get_scheduler_metadata` must produce (layout: flash_cuda_b200/csrc/fa_sched.h)."""
    wl, wr = normalize_window(causal, max_seqlen_k, window_left, window_right)
    E = batch * plan.max_mtiles
    entries = []
    for e in range(E):
        b, mt = divmod(e, plan.max_mtiles)
        sq = max_seqlen_q if q_lens is None else q_lens[b]
        sk = max_seqlen_k if k_lens is None else k_lens[b]
        pad = 0 if leftpad is None else leftpad[b]
        rows_total = sq * plan.rows_per_token
        row0 = mt * plan.tile_m
        if row0 >= rows_total:
            entries.append((False, b, mt, 0, 0))
            continue
        tok_min = row0 // plan.rows_per_token
        tok_max = min(sq - 1, (row0 + plan.tile_m - 1) // plan.rows_per_token)
        lo, hi = nblock_range(sk, pad, sk - sq + tok_min, sk - sq + tok_max, causal, wl, wr, plan.tile_n)
        entries.append((True, b, mt, lo, hi))
    words = [0] * (HEADER + 4 * E)
    is_sorted = E <= SORT_MAX and cdiv(max_seqlen_k, plan.tile_n) <= COUNT_MAX
    if is_sorted:
        valid = [(e, x) for e, x in enumerate(entries) if x[0]]
        valid.sort(key=lambda ex: (-(ex[1][4] - ex[1][3]), ex[0]))
        for i, (_, x) in enumerate(valid):
            words[HEADER + 4 * i:HEADER + 4 * i + 4] = [x[1], x[2], x[3], x[4]]
        for i in range(len(valid), E):
            words[HEADER + 4 * i:HEADER + 4 * i + 4] = [-1, -1, 0, 0]
        num_work = len(valid)
    else:
        for i, x in enumerate(entries):
            words[HEADER + 4 * i:HEADER + 4 * i + 4] = [x[1] if x[0] else -1, x[2] if x[0] else -1, x[3], x[4]]
        num_work = E
    words[0:11] = [MAGIC, VERSION, batch, plan.nsplits, plan.tile_m, plan.tile_n, num_work, plan.max_mtiles,
                   plan.rows_per_token, plan.route, 1 if is_sorted else 0]
    return words
