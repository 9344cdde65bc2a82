"""ctypes binding of the C ABI (include/fa_b200.h) — the thinnest possible caller of libfa_b200.so.

Used by the tests and the bench to reach the library exactly as a foreign-language host would: plain
device pointers and sizes, a caller-owned workspace, an explicit stream.  torch only supplies device
memory and the current stream.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

from . import build as _build

FA_OK, FA_ERR_UNSUPPORTED, FA_ERR_BAD_ARG, FA_ERR_WORKSPACE, FA_ERR_NO_DEVICE, FA_ERR_LAUNCH, FA_ERR_DEVICE_TIMEOUT = range(7)
FA_ERR_STATIC_LIMIT = 7
FA_ERR_BAD_METADATA = 8
STATIC_SCRATCH_BYTES = 8 << 20
FA_DT_BF16, FA_DT_FP16, FA_DT_FP8_E4M3, FA_DT_FP32 = 0, 1, 2, 3
FA_FLAG_WORKSPACE_CLEAN = 1
FA_ROUTE_AUTO, FA_ROUTE_PREFILL_TC, FA_ROUTE_DECODE, FA_ROUTE_GENERAL = 0, 1, 2, 3

EXPORTS = (
    "fa_b200_fwd_workspace_bytes", "fa_b200_fwd", "fa_b200_num_splits", "fa_b200_scheduler_metadata_len",
    "fa_b200_get_scheduler_metadata", "fa_b200_combine", "fa_b200_check_status", "fa_b200_strerror",
    "fa_b200_last_cuda_error", "fa_b200_version", "fa_b200_sizeof_fwd_params", "fa_b200_sizeof_sched_params",
    "fa_b200_decode_fwd_static", "fa_b200_combine_strided", "fa_b200_selftest_timeout", "fa_b200_append_kv",
    "fa_b200_sizeof_append_params",
)

_vp, _i32, _i64, _f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float


class FaFwdParams(C.Structure):
    _fields_ = (
        [(n, _vp) for n in ("q", "k", "v", "out", "lse")]
        + [(n, _i64) for n in ("q_row_stride", "q_head_stride", "k_row_stride", "k_head_stride", "k_page_stride",
                               "v_row_stride", "v_head_stride", "v_page_stride", "o_row_stride", "o_head_stride")]
        + [(n, _vp) for n in ("cu_seqlens_q", "cu_seqlens_k", "seqused_k", "page_table", "leftpad_k", "q_descale",
                              "k_descale", "v_descale", "s_aux", "scheduler_metadata")]
        + [(n, _i32) for n in ("batch", "total_q", "total_k", "hq", "hkv", "hd", "hdv", "max_seqlen_q",
                               "max_seqlen_k", "page_size", "num_pages", "page_table_stride",
                               "descale_batch_stride", "descale_head_stride", "q_dtype", "kv_dtype", "out_dtype")]
        + [("softmax_scale", _f32), ("softcap", _f32)]
        + [(n, _i32) for n in ("is_causal", "window_left", "window_right", "num_splits", "sm_margin", "route",
                               "scheduler_metadata_len", "flags")]
    )


class FaSchedParams(C.Structure):
    _fields_ = (
        [(n, _vp) for n in ("seqused_k", "cu_seqlens_q", "cu_seqlens_k", "leftpad_k")]
        + [(n, _i32) for n in ("batch", "max_seqlen_q", "max_seqlen_k", "hq", "hkv", "hd", "hdv", "qkv_dtype",
                               "page_size", "is_causal", "window_left", "window_right", "has_softcap",
                               "num_splits", "sm_margin")]
    )


class FaAppendParams(C.Structure):
    _fields_ = (
        [(n, _vp) for n in ("k_new", "v_new", "k_cache", "v_cache", "q", "q_out", "rotary_cos", "rotary_sin",
                            "cu_seqlens_k_new", "cu_seqlens_q", "seqused_k", "seqused_k_out", "page_table",
                            "seqlens_rotary")]
        + [(n, _i64) for n in ("kn_row_stride", "kn_head_stride", "vn_row_stride", "vn_head_stride", "k_row_stride",
                               "k_head_stride", "k_page_stride", "v_row_stride", "v_head_stride", "v_page_stride",
                               "q_row_stride", "q_head_stride", "qo_row_stride", "qo_head_stride")]
        + [(n, _i32) for n in ("batch", "total_new", "total_q", "hq", "hkv", "hd", "hdv", "page_size",
                               "page_table_stride", "rotary_dim", "rotary_interleaved", "q_positions_advance",
                               "q_dtype", "kv_dtype")]
    )


_lib = None


def lib_path() -> str:
    return _build.CAPI_SO


def load(build_if_missing: bool = True):
    """Loads libfa_b200.so (building it in-tree when absent).  Raises if it cannot be loaded: there is no
    other implementation to fall back to."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.isfile(_build.CAPI_SO):
        if not build_if_missing:
            raise RuntimeError(f"{_build.CAPI_SO} is missing; run `python -m flash_cuda_b200.build`")
        _build.build_capi()
    lib = C.CDLL(_build.CAPI_SO)
    lib.fa_b200_fwd_workspace_bytes.restype = C.c_size_t
    lib.fa_b200_fwd_workspace_bytes.argtypes = [C.POINTER(FaFwdParams)]
    lib.fa_b200_fwd.restype = C.c_int
    lib.fa_b200_fwd.argtypes = [C.POINTER(FaFwdParams), _vp, C.c_size_t, _vp]
    lib.fa_b200_num_splits.restype = C.c_int
    lib.fa_b200_num_splits.argtypes = [C.POINTER(FaFwdParams)]
    lib.fa_b200_scheduler_metadata_len.restype = C.c_int
    lib.fa_b200_scheduler_metadata_len.argtypes = [C.POINTER(FaSchedParams)]
    lib.fa_b200_get_scheduler_metadata.restype = C.c_int
    lib.fa_b200_get_scheduler_metadata.argtypes = [C.POINTER(FaSchedParams), _vp, _vp]
    lib.fa_b200_combine.restype = C.c_int
    lib.fa_b200_combine.argtypes = [_vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _i64, _i64, _i32, _vp, _vp]
    lib.fa_b200_combine_strided.restype = C.c_int
    lib.fa_b200_combine_strided.argtypes = [_vp, _vp, _i64, _i64, _i32, _i32, _i32, _i32, _vp, _vp, _i64, _i64, _i32,
                                            _vp, _vp]
    lib.fa_b200_selftest_timeout.restype = C.c_int
    lib.fa_b200_selftest_timeout.argtypes = [_vp, _i64, _vp]
    lib.fa_b200_append_kv.restype = C.c_int
    lib.fa_b200_append_kv.argtypes = [C.POINTER(FaAppendParams), _vp]
    lib.fa_b200_sizeof_append_params.restype = C.c_size_t
    lib.fa_b200_check_status.restype = C.c_int
    lib.fa_b200_check_status.argtypes = [_vp, _vp, C.POINTER(C.c_uint32)]
    lib.fa_b200_strerror.restype = C.c_char_p
    lib.fa_b200_strerror.argtypes = [C.c_int]
    lib.fa_b200_last_cuda_error.restype = C.c_char_p
    lib.fa_b200_version.restype = C.c_int
    lib.fa_b200_decode_fwd_static.restype = C.c_int
    lib.fa_b200_decode_fwd_static.argtypes = [C.POINTER(FaFwdParams), _vp]
    lib.fa_b200_sizeof_fwd_params.restype = C.c_size_t
    lib.fa_b200_sizeof_sched_params.restype = C.c_size_t
    if (lib.fa_b200_sizeof_fwd_params() != C.sizeof(FaFwdParams)
            or lib.fa_b200_sizeof_sched_params() != C.sizeof(FaSchedParams)
            or lib.fa_b200_sizeof_append_params() != C.sizeof(FaAppendParams)):
        raise RuntimeError("ctypes struct layout does not match libfa_b200.so; rebuild the library")
    _lib = lib
    return lib


class FaError(RuntimeError):
    def __init__(self, code: int, what: str):
        lib = load()
        msg = lib.fa_b200_strerror(code).decode()
        if code == FA_ERR_LAUNCH:
            msg += " — " + lib.fa_b200_last_cuda_error().decode()
        super().__init__(f"fa_b200 {what}: {msg}")
        self.code = code


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.bfloat16:
        return FA_DT_BF16
    if dt == torch.float16:
        return FA_DT_FP16
    if dt == torch.float8_e4m3fn:
        return FA_DT_FP8_E4M3
    if dt == torch.float32:
        return FA_DT_FP32          # output only
    raise ValueError(f"unsupported dtype {dt}")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def make_params(q, k, v, out, lse, *, cu_seqlens_q, cu_seqlens_k=None, seqused_k=None, page_table=None,
                leftpad_k=None, q_descale=None, k_descale=None, v_descale=None, s_aux=None,
                scheduler_metadata=None, max_seqlen_q, max_seqlen_k, softmax_scale, causal,
                window_left=-1, window_right=-1, softcap=0.0, num_splits=0, sm_margin=0,
                route=FA_ROUTE_AUTO, flags=0):
    """Fills an FaFwdParams from torch tensors.  Returns (params, keepalive list)."""
    keep = []
    paged = page_table is not None
    p = FaFwdParams()
    p.q, p.k, p.v, p.out, p.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr()
    p.q_row_stride, p.q_head_stride = q.stride(0), q.stride(1)
    p.o_row_stride, p.o_head_stride = out.stride(0), out.stride(1)
    p.total_q, p.hq, p.hd = q.shape
    if paged:
        p.k_page_stride, p.k_row_stride, p.k_head_stride = k.stride(0), k.stride(1), k.stride(2)
        p.v_page_stride, p.v_row_stride, p.v_head_stride = v.stride(0), v.stride(1), v.stride(2)
        p.num_pages, p.page_size, p.hkv = k.shape[0], k.shape[1], k.shape[2]
        p.hdv = v.shape[3]
        p.page_table_stride = page_table.stride(0)
    else:
        p.k_row_stride, p.k_head_stride = k.stride(0), k.stride(1)
        p.v_row_stride, p.v_head_stride = v.stride(0), v.stride(1)
        p.total_k, p.hkv = k.shape[0], k.shape[1]
        p.hdv = v.shape[2]
    p.batch = cu_seqlens_q.numel() - 1
    p.cu_seqlens_q, p.cu_seqlens_k, p.seqused_k = _ptr(cu_seqlens_q), _ptr(cu_seqlens_k), _ptr(seqused_k)
    p.page_table, p.leftpad_k = _ptr(page_table), _ptr(leftpad_k)

    def descale(d):
        if d is None:
            return None
        f = d.to(torch.float32)
        if f.numel() == 1:
            f = f.reshape(1, 1)
        f = f.expand(p.batch, p.hkv).contiguous()
        keep.append(f)
        return f.data_ptr()

    p.q_descale, p.k_descale, p.v_descale = descale(q_descale), descale(k_descale), descale(v_descale)
    p.descale_batch_stride, p.descale_head_stride = p.hkv, 1
    if s_aux is not None:
        sf = s_aux.to(torch.float32).contiguous()
        keep.append(sf)
        p.s_aux = sf.data_ptr()
    p.scheduler_metadata = _ptr(scheduler_metadata)
    p.scheduler_metadata_len = 0 if scheduler_metadata is None else scheduler_metadata.numel()
    p.flags = int(flags)
    p.max_seqlen_q, p.max_seqlen_k = int(max_seqlen_q), int(max_seqlen_k)
    p.q_dtype, p.kv_dtype, p.out_dtype = dtype_code(q.dtype), dtype_code(k.dtype), dtype_code(out.dtype)
    p.softmax_scale, p.softcap = float(softmax_scale), float(softcap)
    p.is_causal, p.window_left, p.window_right = int(bool(causal)), int(window_left), int(window_right)
    p.num_splits, p.sm_margin, p.route = int(num_splits), int(sm_margin), int(route)
    return p, keep


def fwd(q, k, v, *, out=None, lse=None, workspace=None, check=False, **kw):
    """Attention forward through `fa_b200_fwd`.  Returns (out, lse, workspace).

    `kw` are the keyword arguments of make_params.  With check=True the stream is synchronised and the
    device status word is read (raises FaError on a device-side timeout or refused metadata).  `out` may be a
    float32 tensor (the normalised result in fp32: the form of a partial result before a merge); `out` and `lse`
    may be views into a larger buffer."""
    lib = load()
    total_q, hq, _ = q.shape
    hdv = v.shape[-1]
    out_dtype = torch.bfloat16 if q.dtype == torch.float8_e4m3fn else q.dtype
    if out is None:
        out = torch.empty(total_q, hq, hdv, device=q.device, dtype=out_dtype)
    if lse is None:
        lse = torch.empty(hq, total_q, device=q.device, dtype=torch.float32)
    p, keep = make_params(q, k, v, out, lse, **kw)
    need = lib.fa_b200_fwd_workspace_bytes(C.byref(p))
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(max(need, 256), device=q.device, dtype=torch.uint8)
    rc = lib.fa_b200_fwd(C.byref(p), workspace.data_ptr(), workspace.numel(), _stream())
    if rc != FA_OK:
        raise FaError(rc, "fwd")
    if check:
        check_status(workspace)
    del keep
    return out, lse, workspace


def decode_fwd_static(q, k, v, *, out=None, **kw):
    """Paged decode through `fa_b200_decode_fwd_static`: no workspace is passed and nothing is allocated by the
    library (the output tensors here are the caller's).  Returns (out, lse)."""
    lib = load()
    total_q, hq, _ = q.shape
    if out is None:
        out = torch.empty(total_q, hq, v.shape[-1], device=q.device, dtype=q.dtype)
    lse = torch.empty(hq, total_q, device=q.device, dtype=torch.float32)
    p, keep = make_params(q, k, v, out, lse, **kw)
    rc = lib.fa_b200_decode_fwd_static(C.byref(p), _stream())
    if rc != FA_OK:
        raise FaError(rc, "decode_fwd_static")
    del keep
    return out, lse


def num_splits(q, k, v, **kw) -> int:
    lib = load()
    out = torch.empty(q.shape[0], q.shape[1], v.shape[-1], device=q.device,
                      dtype=torch.bfloat16 if q.dtype == torch.float8_e4m3fn else q.dtype)
    lse = torch.empty(q.shape[1], q.shape[0], device=q.device, dtype=torch.float32)
    p, _ = make_params(q, k, v, out, lse, **kw)
    return lib.fa_b200_num_splits(C.byref(p))


def check_status(workspace: torch.Tensor) -> None:
    lib = load()
    detail = C.c_uint32(0)
    rc = lib.fa_b200_check_status(workspace.data_ptr(), _stream(), C.byref(detail))
    if rc != FA_OK:
        e = FaError(rc, "status")
        e.detail = detail.value
        raise e


def sched_params(*, batch, max_seqlen_q, max_seqlen_k, hq, hkv, hd, hdv, dtype, seqused_k=None, cu_seqlens_q=None,
                 cu_seqlens_k=None, leftpad_k=None, page_size=0, causal=True, window_left=-1, window_right=-1,
                 has_softcap=False, num_splits=0, sm_margin=0) -> FaSchedParams:
    sp = FaSchedParams()
    sp.seqused_k, sp.cu_seqlens_q, sp.cu_seqlens_k, sp.leftpad_k = (_ptr(seqused_k), _ptr(cu_seqlens_q),
                                                                     _ptr(cu_seqlens_k), _ptr(leftpad_k))
    sp.batch, sp.max_seqlen_q, sp.max_seqlen_k = batch, max_seqlen_q, max_seqlen_k
    sp.hq, sp.hkv, sp.hd, sp.hdv = hq, hkv, hd, hdv
    sp.qkv_dtype = dtype_code(dtype)
    sp.page_size = page_size
    sp.is_causal, sp.window_left, sp.window_right = int(bool(causal)), window_left, window_right
    sp.has_softcap, sp.num_splits, sp.sm_margin = int(bool(has_softcap)), num_splits, sm_margin
    return sp


def get_scheduler_metadata(device, **kw) -> torch.Tensor:
    lib = load()
    sp = sched_params(**kw)
    n = lib.fa_b200_scheduler_metadata_len(C.byref(sp))
    md = torch.empty(n, device=device, dtype=torch.int32)
    rc = lib.fa_b200_get_scheduler_metadata(C.byref(sp), md.data_ptr(), _stream())
    if rc != FA_OK:
        raise FaError(rc, "get_scheduler_metadata")
    return md


def combine(o_part: torch.Tensor, lse_part: torch.Tensor, s_aux: Optional[torch.Tensor] = None,
            out_dtype: torch.dtype = torch.bfloat16):
    """LSE-weighted merge of partials: o_part (S, total_q, hq, hdv) fp32, lse_part (S, hq, total_q) fp32.
    Each split must be contiguous inside; the distance between splits is free (views into a gathered buffer of
    packed [O | LSE] partials are merged where they lie, through `fa_b200_combine_strided`)."""
    lib = load()
    S, total_q, hq, hdv = o_part.shape
    assert o_part.dtype == torch.float32 and lse_part.dtype == torch.float32
    assert o_part[0].is_contiguous() and lse_part[0].is_contiguous() and lse_part.shape == (S, hq, total_q)
    o_ss = o_part.stride(0) if S > 1 else total_q * hq * hdv
    l_ss = lse_part.stride(0) if S > 1 else hq * total_q
    out = torch.empty(total_q, hq, hdv, device=o_part.device, dtype=out_dtype)
    lse = torch.empty(hq, total_q, device=o_part.device, dtype=torch.float32)
    sf = None if s_aux is None else s_aux.to(torch.float32).contiguous()
    rc = lib.fa_b200_combine_strided(o_part.data_ptr(), lse_part.data_ptr(), o_ss, l_ss, S, total_q, hq, hdv,
                                     _ptr(sf), out.data_ptr(), out.stride(0), out.stride(1), dtype_code(out_dtype),
                                     lse.data_ptr(), _stream())
    if rc != FA_OK:
        raise FaError(rc, "combine")
    return out, lse


def partial_layout(total_q: int, hq: int, hdv: int):
    """(floats of O, floats of one packed partial): [O (total_q, hq, hdv) | LSE (hq, total_q) | pad to 4 floats]."""
    n_o = total_q * hq * hdv
    return n_o, n_o + (hq * total_q + 3) // 4 * 4


def partial_buffer(total_q: int, hq: int, hdv: int, device):
    """One packed fp32 buffer [O | LSE] and the two views `fwd(..., out=o_view, lse=lse_view)` writes into."""
    n_o, per = partial_layout(total_q, hq, hdv)
    buf = torch.empty(per, device=device, dtype=torch.float32)
    return buf, buf[:n_o].view(total_q, hq, hdv), buf[n_o:n_o + hq * total_q].view(hq, total_q)


def append_kv(k_new, v_new, k_cache, v_cache, *, page_table, seqused_k, cu_seqlens_k_new, q=None, cu_seqlens_q=None,
              rotary_cos=None, rotary_sin=None, seqlens_rotary=None, rotary_interleaved=True,
              q_positions_advance=True):
    """Appends k_new / v_new (total_new, hkv, d) to the paged cache IN PLACE through `fa_b200_append_kv` and, with a
    rotary table, rotates them and returns a rotated copy of q.  Returns (q_rotated or q, seqused_k after the append)."""
    lib = load()
    p = FaAppendParams()
    p.k_new, p.v_new, p.k_cache, p.v_cache = k_new.data_ptr(), v_new.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr()
    p.kn_row_stride, p.kn_head_stride = k_new.stride(0), k_new.stride(1)
    p.vn_row_stride, p.vn_head_stride = v_new.stride(0), v_new.stride(1)
    p.k_page_stride, p.k_row_stride, p.k_head_stride = k_cache.stride(0), k_cache.stride(1), k_cache.stride(2)
    p.v_page_stride, p.v_row_stride, p.v_head_stride = v_cache.stride(0), v_cache.stride(1), v_cache.stride(2)
    p.total_new, p.hkv, p.hd = k_new.shape
    p.hdv = v_new.shape[2]
    p.page_size = k_cache.shape[1]
    p.page_table, p.page_table_stride = page_table.data_ptr(), page_table.stride(0)
    p.batch = seqused_k.numel()
    seq_out = torch.empty_like(seqused_k)
    p.seqused_k, p.seqused_k_out, p.cu_seqlens_k_new = seqused_k.data_ptr(), seq_out.data_ptr(), cu_seqlens_k_new.data_ptr()
    p.kv_dtype = dtype_code(k_cache.dtype)
    q_out = q
    if rotary_cos is not None:
        q_out = torch.empty(q.shape, device=q.device, dtype=q.dtype)
        p.q, p.q_out, p.cu_seqlens_q = q.data_ptr(), q_out.data_ptr(), cu_seqlens_q.data_ptr()
        p.total_q, p.hq, _ = q.shape
        p.q_row_stride, p.q_head_stride = q.stride(0), q.stride(1)
        p.qo_row_stride, p.qo_head_stride = q_out.stride(0), q_out.stride(1)
        p.rotary_cos, p.rotary_sin = rotary_cos.data_ptr(), rotary_sin.data_ptr()
        p.rotary_dim = 2 * rotary_cos.shape[1]
        p.seqlens_rotary = _ptr(seqlens_rotary)
        p.rotary_interleaved, p.q_positions_advance = int(bool(rotary_interleaved)), int(bool(q_positions_advance))
        p.q_dtype = dtype_code(q.dtype)
    else:
        p.q_dtype = FA_DT_BF16 if k_cache.dtype == torch.float8_e4m3fn else dtype_code(k_new.dtype)
    rc = lib.fa_b200_append_kv(C.byref(p), _stream())
    if rc != FA_OK:
        raise FaError(rc, "append_kv")
    return q_out, seq_out


def selftest_timeout(device, max_cycles: int = 200_000) -> torch.Tensor:
    """Launches the bounded-wait self-test (a wait that must give up by itself); returns the workspace whose status
    word `check_status` then reads."""
    lib = load()
    ws = torch.empty(256, device=device, dtype=torch.uint8)
    rc = lib.fa_b200_selftest_timeout(ws.data_ptr(), int(max_cycles), _stream())
    if rc != FA_OK:
        raise FaError(rc, "selftest_timeout")
    return ws
