"""ctypes binding of libpope_b200.so (the C ABI in include/pope_b200.h) and the autograd
functions built on it.

This is the seam where the reference re-points its two Triton imports
(PoPE_pytorch/attention.py:21-26): ``similarity`` stands in for
``triton_compute_qk_similarity`` (PoPE_pytorch/triton_pope.py:364-372) and ``flash_attn`` for
``flash_attn`` (PoPE_pytorch/triton_pope_flash_attn.py:364-373).  PyTorch is used for device
memory, streams and autograd bookkeeping only; all arithmetic happens in the library.
There is no fallback: if the library cannot be loaded every call raises.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libpope_b200.so")

OP_SIM_FWD, OP_SIM_BWD, OP_ATTN_FWD, OP_ATTN_BWD, OP_DECODE_PAGED = 0, 1, 2, 3, 4
_DTYPES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


class Stride3(C.Structure):
    _fields_ = [("b", C.c_int64), ("h", C.c_int64), ("n", C.c_int64)]


class Shape(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("B", "H", "Hk", "Nq", "Nk", "d", "r", "dtype")]


class Embed(C.Structure):
    _fields_ = [("freqs", C.c_void_p), ("sf", Stride3), ("bias", C.c_void_p), ("bias_stride_h", C.c_int64),
                ("positions", C.c_void_p), ("pos_stride_n", C.c_int64), ("inv_freqs", C.c_void_p), ("axis_of", C.c_void_p)]


class SimArgs(C.Structure):
    _fields_ = [("struct_bytes", C.c_uint32), ("allow_tf32", C.c_int32), ("shape", Shape), ("embed", Embed),
                ("q", C.c_void_p), ("sq", Stride3), ("k", C.c_void_p), ("sk", Stride3),
                ("sim", C.c_void_p), ("ss", Stride3), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


class SimBwdArgs(C.Structure):
    _fields_ = [("struct_bytes", C.c_uint32), ("allow_tf32", C.c_int32), ("shape", Shape), ("embed", Embed),
                ("q", C.c_void_p), ("sq", Stride3), ("k", C.c_void_p), ("sk", Stride3),
                ("dsim", C.c_void_p), ("sds", Stride3), ("dq", C.c_void_p), ("sdq", Stride3),
                ("dk", C.c_void_p), ("sdk", Stride3), ("dfreqs", C.c_void_p), ("sdf", Stride3),
                ("dbias", C.c_void_p), ("dbias_stride_h", C.c_int64),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


class AttnArgs(C.Structure):
    _fields_ = [("struct_bytes", C.c_uint32), ("causal", C.c_int32), ("softmax_scale", C.c_float),
                ("reserved0", C.c_int32), ("shape", Shape), ("embed", Embed),
                ("q", C.c_void_p), ("sq", Stride3), ("k", C.c_void_p), ("sk", Stride3),
                ("v", C.c_void_p), ("sv", Stride3), ("out", C.c_void_p), ("so", Stride3),
                ("lse", C.c_void_p), ("mask", C.c_void_p), ("mask_stride_b", C.c_int64),
                ("mask_stride_n", C.c_int64), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


class AttnBwdArgs(C.Structure):
    _fields_ = [("struct_bytes", C.c_uint32), ("causal", C.c_int32), ("softmax_scale", C.c_float),
                ("reserved0", C.c_int32), ("shape", Shape), ("embed", Embed),
                ("q", C.c_void_p), ("sq", Stride3), ("k", C.c_void_p), ("sk", Stride3),
                ("v", C.c_void_p), ("sv", Stride3), ("out", C.c_void_p), ("so", Stride3),
                ("dout", C.c_void_p), ("sdo", Stride3), ("lse", C.c_void_p),
                ("mask", C.c_void_p), ("mask_stride_b", C.c_int64), ("mask_stride_n", C.c_int64),
                ("dq", C.c_void_p), ("sdq", Stride3), ("dk", C.c_void_p), ("sdk", Stride3),
                ("dv", C.c_void_p), ("sdv", Stride3), ("dfreqs", C.c_void_p), ("sdf", Stride3),
                ("dbias", C.c_void_p), ("dbias_stride_h", C.c_int64),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


ABI_VERSION = 3


class ApplyArgs(C.Structure):
    _fields_ = [("struct_bytes", C.c_uint32), ("reserved0", C.c_int32), ("shape", Shape), ("embed", Embed),
                ("q", C.c_void_p), ("sq", Stride3), ("k", C.c_void_p), ("sk", Stride3),
                ("q_out", C.c_void_p), ("sqo", Stride3), ("k_out", C.c_void_p), ("sko", Stride3)]


class ApplyBwdArgs(C.Structure):
    _fields_ = [("struct_bytes", C.c_uint32), ("reserved0", C.c_int32), ("shape", Shape), ("embed", Embed),
                ("q", C.c_void_p), ("sq", Stride3), ("k", C.c_void_p), ("sk", Stride3),
                ("dq_out", C.c_void_p), ("sdqo", Stride3), ("dk_out", C.c_void_p), ("sdko", Stride3),
                ("dq", C.c_void_p), ("sdq", Stride3), ("dk", C.c_void_p), ("sdk", Stride3),
                ("dfreqs", C.c_void_p), ("sdf", Stride3), ("dbias", C.c_void_p), ("dbias_stride_h", C.c_int64)]


class PagedKV(C.Structure):
    _fields_ = [("k_pages", C.c_void_p), ("v_pages", C.c_void_p), ("page_table", C.c_void_p), ("seq_lens", C.c_void_p),
                ("num_pages", C.c_int32), ("page_size", C.c_int32), ("max_pages_per_seq", C.c_int32), ("reserved0", C.c_int32)]


class KvAppendArgs(C.Structure):
    _fields_ = [("struct_bytes", C.c_uint32), ("dtype", C.c_int32), ("B", C.c_int32), ("Hk", C.c_int32), ("d", C.c_int32),
                ("n_new", C.c_int32), ("advance", C.c_int32), ("reserved0", C.c_int32), ("kv", PagedKV),
                ("k", C.c_void_p), ("sk", Stride3), ("v", C.c_void_p), ("sv", Stride3)]


class PagedDecodeArgs(C.Structure):
    _fields_ = [("struct_bytes", C.c_uint32), ("softmax_scale", C.c_float), ("shape", Shape), ("embed", Embed), ("kv", PagedKV),
                ("q", C.c_void_p), ("sq", Stride3), ("out", C.c_void_p), ("so", Stride3), ("lse", C.c_void_p),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


EXPORTS = ("pope_b200_abi_version", "pope_b200_apply_qk_fwd", "pope_b200_apply_qk_bwd", "pope_b200_status_str", "pope_b200_last_path", "pope_b200_device_status",
           "pope_b200_clear_device_status", "pope_b200_selftest_bounded_wait",
           "pope_b200_workspace_bytes", "pope_b200_attn_fwd_noalloc", "pope_b200_kv_append", "pope_b200_attn_decode_paged",
           "pope_b200_sim_fwd", "pope_b200_sim_bwd", "pope_b200_attn_fwd", "pope_b200_attn_bwd")

_lib = None
_load_error: Optional[str] = None


def _bind(lib):
    lib.pope_b200_abi_version.restype = C.c_int
    lib.pope_b200_status_str.restype = C.c_char_p
    lib.pope_b200_status_str.argtypes = [C.c_int]
    lib.pope_b200_last_path.restype = C.c_char_p
    lib.pope_b200_workspace_bytes.restype = C.c_size_t
    lib.pope_b200_workspace_bytes.argtypes = [C.c_int, C.c_void_p]
    for name in ("pope_b200_sim_fwd", "pope_b200_sim_bwd", "pope_b200_attn_fwd", "pope_b200_attn_bwd",
                 "pope_b200_apply_qk_fwd", "pope_b200_apply_qk_bwd", "pope_b200_kv_append", "pope_b200_attn_decode_paged"):
        fn = getattr(lib, name)
        fn.restype = C.c_int
        fn.argtypes = [C.c_void_p, C.c_void_p]
    lib.pope_b200_device_status.restype = C.c_int
    lib.pope_b200_clear_device_status.restype = C.c_int
    lib.pope_b200_selftest_bounded_wait.restype = C.c_int
    lib.pope_b200_selftest_bounded_wait.argtypes = [C.c_void_p]
    lib.pope_b200_attn_fwd_noalloc.restype = C.c_int
    lib.pope_b200_attn_fwd_noalloc.argtypes = [C.c_void_p, C.c_void_p]
    if lib.pope_b200_abi_version() != ABI_VERSION:
        raise RuntimeError("libpope_b200.so has an unexpected ABI version; rebuild it")
    return lib


def load_library():
    """dlopen the in-tree library once; raises RuntimeError when it is missing or stale."""
    global _lib, _load_error
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        _load_error = f"{LIB_PATH} is missing: build it with `python -m pope_pytorch_b200.build`"
        raise RuntimeError(_load_error)
    try:
        lib = _bind(C.CDLL(LIB_PATH))
    except AttributeError as exc:     # a symbol of the current header is missing: the build is stale
        raise RuntimeError(f"{LIB_PATH} is stale ({exc}); rebuild it with `python -m pope_pytorch_b200.build`") from exc
    _lib = lib
    return lib


def is_available() -> bool:
    try:
        load_library()
        return True
    except (RuntimeError, OSError):
        return False


def last_path() -> str:
    return load_library().pope_b200_last_path().decode()


def device_status() -> int:
    """Sticky health word of the tensor-core kernels on the current device (synchronises)."""
    return load_library().pope_b200_device_status()


def clear_device_status() -> None:
    """Reset the sticky health word of the current device (synchronises)."""
    _check(load_library().pope_b200_clear_device_status(), "pope_b200_clear_device_status")


def selftest_bounded_wait(device=None) -> None:
    """Launch the diagnostic kernel whose only barrier never completes: it gives up after a few
    microseconds and sets bit 0 of the status word (see include/pope_b200.h)."""
    dev = torch.device("cuda" if device is None else device)
    with torch.cuda.device(dev):
        _check(load_library().pope_b200_selftest_bounded_wait(torch.cuda.current_stream(dev).cuda_stream),
               "pope_b200_selftest_bounded_wait")


def _check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load_library().pope_b200_status_str(rc).decode()
        raise RuntimeError(f"{what} failed: {msg} (status {rc})")


# What a call costs on the host matters for the small shapes (a (2, 8, 1024, 64) forward is 29 us of GPU time): the
# raw stream handle and the current device come from torch's C bindings directly, and the device guard is entered only
# when the tensors live on another device than the current one.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_get_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream_ptr(t: torch.Tensor) -> int:
    if _raw_stream is not None:
        return _raw_stream(t.device.index if t.device.index is not None else torch.cuda.current_device())
    return torch.cuda.current_stream(t.device).cuda_stream


class _NoGuard:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def _on_device(dev: torch.device):
    """Context that makes ``dev`` the current CUDA device for the library call (a no-op when it already is)."""
    if _get_device is not None and dev.index is not None and _get_device() == dev.index:
        return _NO_GUARD
    return torch.cuda.device(dev)


def _s3(t: torch.Tensor) -> Stride3:
    """Strides of a head-first (b, h, n, x) view; the innermost stride must be 1."""
    s = t.stride()
    return Stride3(s[0], s[1], s[2])


def _inner_contig(t: torch.Tensor) -> torch.Tensor:
    return t if t.shape[-1] <= 1 or t.stride(-1) == 1 else t.contiguous()


def _freq_strides(freqs: torch.Tensor) -> Stride3:
    """(batch, head, row) strides with 0 = broadcast.  A 4-D table is (b, h, n, r), the layout
    apply_pope_to_qk and the similarity kernel of the reference use
    (PoPE_pytorch/pope.py:53-56, triton_pope.py:267-272)."""
    if freqs.ndim == 2:
        return Stride3(0, 0, freqs.stride(0))
    if freqs.ndim == 3:
        return Stride3(freqs.stride(0) if freqs.shape[0] > 1 else 0, 0, freqs.stride(1))
    if freqs.ndim == 4:
        return Stride3(freqs.stride(0) if freqs.shape[0] > 1 else 0,
                       freqs.stride(1) if freqs.shape[1] > 1 else 0, freqs.stride(2))
    raise ValueError("freqs must have 2, 3 or 4 dimensions")


def _prep_embed(freqs: torch.Tensor, bias: torch.Tensor, nk: int, r: int):
    freqs = _inner_contig(freqs.float()) if freqs.dtype != torch.float32 else _inner_contig(freqs)
    bias = _inner_contig(bias.float()) if bias.dtype != torch.float32 else _inner_contig(bias)
    assert freqs.shape[-2] == nk or r == 0, "freqs must have one row per key position"
    return freqs, bias


def _factors_of(freqs):
    """(positions, inv_freqs, axis_of) riding on a table built by PoPE / AxialPoPE, when usable as is."""
    f = getattr(freqs, "_pope_factored", None)
    if f is None or freqs.ndim != 2:
        return None
    pos, inv, axis = f
    ok = (pos.device == freqs.device and inv.device == freqs.device and pos.dtype == torch.float32 and inv.dtype == torch.float32
          and pos.shape[0] == freqs.shape[0] and inv.numel() == freqs.shape[1] and pos.stride(-1) == 1 and inv.is_contiguous()
          and (axis is None or (axis.device == freqs.device and axis.dtype == torch.int32 and axis.is_contiguous())))
    return f if ok else None


def _embed_struct(freqs, bias, r, factors=None) -> Embed:
    if r == 0:
        return Embed(None, Stride3(0, 0, 0), None, 0, None, 0, None, None)
    if factors is None:
        return Embed(freqs.data_ptr(), _freq_strides(freqs), bias.data_ptr(), bias.stride(0), None, 0, None, None)
    pos, inv, axis = factors
    return Embed(freqs.data_ptr(), _freq_strides(freqs), bias.data_ptr(), bias.stride(0), pos.data_ptr(),
                 pos.stride(0) if pos.ndim == 2 else 1, inv.data_ptr(), None if axis is None else axis.data_ptr())


def _shape(q, k, r) -> Shape:
    b, h, nq, d = q.shape
    hk, nk = k.shape[1], k.shape[2]
    return Shape(b, h, hk, nq, nk, d, r, _DTYPES[q.dtype])


def _workspace(op: int, args, device) -> Optional[torch.Tensor]:
    need = load_library().pope_b200_workspace_bytes(op, C.addressof(args))
    if need == 0:
        return None
    ws = torch.empty(need, dtype=torch.uint8, device=device)
    args.workspace, args.workspace_bytes = ws.data_ptr(), need
    return ws


def _validate(q, k, freqs, bias):
    if not (q.is_cuda and k.is_cuda):
        raise RuntimeError("the native PoPE kernels need CUDA tensors")
    if q.dtype not in _DTYPES or k.dtype != q.dtype:
        raise TypeError(f"q and k must share a dtype among fp32/bf16/fp16, got {q.dtype}, {k.dtype}")
    assert q.shape[1] % k.shape[1] == 0, "query heads must be a multiple of key heads"
    assert q.shape[2] <= k.shape[2] and freqs.shape[-1] <= q.shape[-1]


# ----------------------------------------------------------------------------------------------
# the stand-alone transform
# ----------------------------------------------------------------------------------------------

def apply_qk_supported(q, k, freqs, bias) -> bool:
    """CUDA 4-D head-first q / k of one supported dtype, fp32 table, even expanded width."""
    if not (q.is_cuda and k.is_cuda and freqs.is_cuda and bias.is_cuda and q.ndim == 4 and k.ndim == 4):
        return False
    d, r = q.shape[-1], freqs.shape[-1]
    return (q.dtype in _DTYPES and k.dtype == q.dtype and d <= 256 and (d + r) % 2 == 0 and q.shape[1] % k.shape[1] == 0
            and freqs.ndim in (2, 3, 4) and bias.ndim == 2 and is_available())


class _ApplyQK(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, freqs, bias):
        lib = load_library()
        r = freqs.shape[-1]
        qc, kc = _inner_contig(q), _inner_contig(k)
        fr, bi = _prep_embed(freqs, bias, k.shape[2], r)
        q_out = torch.empty(*q.shape[:-1], q.shape[-1] + r, dtype=torch.float32, device=q.device)
        k_out = torch.empty(*k.shape[:-1], k.shape[-1] + r, dtype=torch.float32, device=q.device)
        a = ApplyArgs(C.sizeof(ApplyArgs), 0, _shape(qc, kc, r), _embed_struct(fr, bi, r),
                      qc.data_ptr(), _s3(qc), kc.data_ptr(), _s3(kc), q_out.data_ptr(), _s3(q_out), k_out.data_ptr(), _s3(k_out))
        with _on_device(q.device):
            _check(lib.pope_b200_apply_qk_fwd(C.addressof(a), _stream_ptr(q)), "pope_b200_apply_qk_fwd")
        ctx.save_for_backward(qc, kc, fr, bi)
        ctx.shapes = (freqs.shape, bias.shape, freqs.dtype, bias.dtype)
        return q_out, k_out

    @staticmethod
    def backward(ctx, dq_out, dk_out):
        lib = load_library()
        q, k, freqs, bias = ctx.saved_tensors
        r = freqs.shape[-1]
        dq_out, dk_out = dq_out.contiguous().float(), dk_out.contiguous().float()
        dq, dk = torch.empty_like(q), torch.empty_like(k)
        need_df, need_db = ctx.needs_input_grad[2] and r > 0, ctx.needs_input_grad[3] and r > 0
        dfreqs = torch.zeros(freqs.shape, dtype=torch.float32, device=q.device) if need_df else None
        dbias = torch.zeros(bias.shape, dtype=torch.float32, device=q.device) if need_db else None
        a = ApplyBwdArgs(C.sizeof(ApplyBwdArgs), 0, _shape(q, k, r), _embed_struct(freqs, bias, r),
                         q.data_ptr(), _s3(q), k.data_ptr(), _s3(k), dq_out.data_ptr(), _s3(dq_out), dk_out.data_ptr(), _s3(dk_out),
                         dq.data_ptr(), _s3(dq), dk.data_ptr(), _s3(dk),
                         dfreqs.data_ptr() if dfreqs is not None else None,
                         _freq_strides(dfreqs) if dfreqs is not None else Stride3(0, 0, 0),
                         dbias.data_ptr() if dbias is not None else None, dbias.stride(0) if dbias is not None else 0)
        with _on_device(q.device):
            _check(lib.pope_b200_apply_qk_bwd(C.addressof(a), _stream_ptr(q)), "pope_b200_apply_qk_bwd")
        fshape, bshape, fdt, bdt = ctx.shapes
        if ctx.needs_input_grad[2] and dfreqs is None:
            dfreqs = torch.zeros(fshape, dtype=fdt, device=q.device)
        if ctx.needs_input_grad[3] and dbias is None:
            dbias = torch.zeros(bshape, dtype=bdt, device=q.device)
        return dq, dk, None if dfreqs is None else dfreqs.to(fdt), None if dbias is None else dbias.to(bdt)


def apply_qk(q, k, freqs, bias):
    """Differentiable fused transform on head-first (b,h,n,d) tensors -> fp32 (q', k') in the
    reference's interleaved layout."""
    return _ApplyQK.apply(q, k, freqs, bias)


# ----------------------------------------------------------------------------------------------
# similarity
# ----------------------------------------------------------------------------------------------

def sim_forward(q, k, freqs, bias, allow_tf32=True, factors=None) -> torch.Tensor:
    """q (b,h,nq,d), k (b,hk,nk,d) head-first views -> sim (b,h,nq,nk) in q's dtype."""
    lib = load_library()
    r = freqs.shape[-1]
    _validate(q, k, freqs, bias)
    q, k = _inner_contig(q), _inner_contig(k)
    factors = factors or _factors_of(freqs)
    freqs, bias = _prep_embed(freqs, bias, k.shape[2], r)
    sim = torch.empty(q.shape[0], q.shape[1], q.shape[2], k.shape[2], dtype=q.dtype, device=q.device)
    a = SimArgs(C.sizeof(SimArgs), int(allow_tf32), _shape(q, k, r), _embed_struct(freqs, bias, r, factors),
                q.data_ptr(), _s3(q), k.data_ptr(), _s3(k), sim.data_ptr(), _s3(sim), None, 0)
    ws = _workspace(OP_SIM_FWD, a, q.device)
    with _on_device(q.device):
        _check(lib.pope_b200_sim_fwd(C.addressof(a), _stream_ptr(q)), "pope_b200_sim_fwd")
    del ws
    return sim


def sim_backward(dsim, q, k, freqs, bias, need_dfreqs, need_dbias, allow_tf32=True):
    lib = load_library()
    r = freqs.shape[-1]
    q, k, dsim = _inner_contig(q), _inner_contig(k), _inner_contig(dsim)
    freqs, bias = _prep_embed(freqs, bias, k.shape[2], r)
    dq, dk = torch.empty_like(q), torch.empty_like(k)
    dfreqs = torch.zeros(freqs.shape, dtype=torch.float32, device=q.device) if (need_dfreqs and r > 0) else None
    dbias = torch.zeros(bias.shape, dtype=torch.float32, device=q.device) if (need_dbias and r > 0) else None
    a = SimBwdArgs(C.sizeof(SimBwdArgs), int(allow_tf32), _shape(q, k, r), _embed_struct(freqs, bias, r),
                   q.data_ptr(), _s3(q), k.data_ptr(), _s3(k), dsim.data_ptr(), _s3(dsim),
                   dq.data_ptr(), _s3(dq), dk.data_ptr(), _s3(dk),
                   dfreqs.data_ptr() if dfreqs is not None else None,
                   _freq_strides(dfreqs) if dfreqs is not None else Stride3(0, 0, 0),
                   dbias.data_ptr() if dbias is not None else None,
                   dbias.stride(0) if dbias is not None else 0, None, 0)
    ws = _workspace(OP_SIM_BWD, a, q.device)
    with _on_device(q.device):
        _check(lib.pope_b200_sim_bwd(C.addressof(a), _stream_ptr(q)), "pope_b200_sim_bwd")
    del ws
    if need_dfreqs and dfreqs is None:
        dfreqs = torch.zeros_like(freqs)
    if need_dbias and dbias is None:
        dbias = torch.zeros_like(bias)
    return dq, dk, dfreqs, dbias


class _Similarity(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, freqs, bias, allow_tf32):
        ctx.save_for_backward(q, k, freqs, bias)
        ctx.allow_tf32 = allow_tf32
        return sim_forward(q, k, freqs, bias, allow_tf32)

    @staticmethod
    def backward(ctx, dsim):
        q, k, freqs, bias = ctx.saved_tensors
        dq, dk, dfreqs, dbias = sim_backward(dsim.to(q.dtype), q, k, freqs, bias,
                                             ctx.needs_input_grad[2], ctx.needs_input_grad[3], ctx.allow_tf32)
        if dfreqs is not None:
            dfreqs = dfreqs.to(freqs.dtype)
        if dbias is not None:
            dbias = dbias.to(bias.dtype)
        return dq, dk, dfreqs, dbias, None


def similarity(q, k, freqs, bias, allow_tf32=True):
    """Differentiable fused similarity on head-first tensors."""
    return _Similarity.apply(q, k, freqs, bias, allow_tf32)


# ----------------------------------------------------------------------------------------------
# attention
# ----------------------------------------------------------------------------------------------

def _mask_u8(mask: Optional[torch.Tensor]):
    if mask is None:
        return None
    m = mask if mask.dtype in (torch.bool, torch.uint8) else (mask != 0)
    return m.view(torch.uint8) if m.dtype == torch.bool else m


def attn_forward(q, k, v, freqs, bias, mask, causal, scale, factors=None):
    """Head-first VIEWS (b,h,n,d) of any stride with contiguous features -> (out, lse)."""
    lib = load_library()
    r = freqs.shape[-1]
    _validate(q, k, freqs, bias)
    q, k, v = _inner_contig(q), _inner_contig(k), _inner_contig(v)
    factors = factors or _factors_of(freqs)
    freqs, bias = _prep_embed(freqs, bias, k.shape[2], r)
    # the output takes the memory layout of q, so a (b,n,h,d) caller gets a (b,n,h,d)-contiguous result
    out = torch.empty_like(q)
    lse = torch.empty(q.shape[0], q.shape[1], q.shape[2], dtype=torch.float32, device=q.device)
    m8 = _mask_u8(mask)
    a = AttnArgs(C.sizeof(AttnArgs), int(causal), float(scale), 0, _shape(q, k, r), _embed_struct(freqs, bias, r, factors),
                 q.data_ptr(), _s3(q), k.data_ptr(), _s3(k), v.data_ptr(), _s3(v), out.data_ptr(), _s3(out),
                 lse.data_ptr(), m8.data_ptr() if m8 is not None else None,
                 m8.stride(0) if m8 is not None else 0, m8.stride(1) if m8 is not None else 0, None, 0)
    ws = _workspace(OP_ATTN_FWD, a, q.device)
    with _on_device(q.device):
        _check(lib.pope_b200_attn_fwd(C.addressof(a), _stream_ptr(q)), "pope_b200_attn_fwd")
    del ws
    return out, lse


def attn_backward(dout, q, k, v, out, lse, freqs, bias, mask, causal, scale, need_dfreqs, need_dbias, factors=None):
    lib = load_library()
    r = freqs.shape[-1]
    q, k, v, out, dout = (_inner_contig(t) for t in (q, k, v, out, dout))
    factors = factors or _factors_of(freqs)
    freqs, bias = _prep_embed(freqs, bias, k.shape[2], r)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    dfreqs = torch.zeros(freqs.shape, dtype=torch.float32, device=q.device) if (need_dfreqs and r > 0) else None
    dbias = torch.zeros(bias.shape, dtype=torch.float32, device=q.device) if (need_dbias and r > 0) else None
    m8 = _mask_u8(mask)
    a = AttnBwdArgs(C.sizeof(AttnBwdArgs), int(causal), float(scale), 0, _shape(q, k, r),
                    _embed_struct(freqs, bias, r, factors),
                    q.data_ptr(), _s3(q), k.data_ptr(), _s3(k), v.data_ptr(), _s3(v), out.data_ptr(), _s3(out),
                    dout.data_ptr(), _s3(dout), lse.data_ptr(),
                    m8.data_ptr() if m8 is not None else None,
                    m8.stride(0) if m8 is not None else 0, m8.stride(1) if m8 is not None else 0,
                    dq.data_ptr(), _s3(dq), dk.data_ptr(), _s3(dk), dv.data_ptr(), _s3(dv),
                    dfreqs.data_ptr() if dfreqs is not None else None,
                    _freq_strides(dfreqs) if dfreqs is not None else Stride3(0, 0, 0),
                    dbias.data_ptr() if dbias is not None else None,
                    dbias.stride(0) if dbias is not None else 0, None, 0)
    ws = _workspace(OP_ATTN_BWD, a, q.device)
    with _on_device(q.device):
        _check(lib.pope_b200_attn_bwd(C.addressof(a), _stream_ptr(q)), "pope_b200_attn_bwd")
    del ws
    if need_dfreqs and dfreqs is None:
        dfreqs = torch.zeros_like(freqs)
    if need_dbias and dbias is None:
        dbias = torch.zeros_like(bias)
    return dq, dk, dv, dfreqs, dbias


NOALLOC_MAX_SCRATCH = 16 << 20


def attn_forward_noalloc(q, k, v, freqs, bias, mask, causal, scale, out, lse):
    """Forward attention through ``pope_b200_attn_fwd_noalloc``: for hosts that must not allocate
    device memory at call time.  Every tensor, including ``out`` (like q) and ``lse``
    (b, h, nq) fp32, is supplied by the caller; the library keeps its scratch in a fixed internal
    array, so this wrapper creates no tensor either.  Inputs must already be in the form the
    kernel reads (CUDA, fp32 contiguous freqs/bias, feature-contiguous q/k/v, uint8/bool mask).
    Raises RuntimeError when the shape is not served or needs more than NOALLOC_MAX_SCRATCH.
    Calls that overlap on the GPU share the scratch and race; keep them on one stream."""
    lib = load_library()
    r = freqs.shape[-1]
    m8 = _mask_u8(mask)
    a = AttnArgs(C.sizeof(AttnArgs), int(causal), float(scale), 0, _shape(q, k, r), _embed_struct(freqs, bias, r),
                 q.data_ptr(), _s3(q), k.data_ptr(), _s3(k), v.data_ptr(), _s3(v), out.data_ptr(), _s3(out),
                 lse.data_ptr(), m8.data_ptr() if m8 is not None else None,
                 m8.stride(0) if m8 is not None else 0, m8.stride(1) if m8 is not None else 0, None, 0)
    with _on_device(q.device):
        _check(lib.pope_b200_attn_fwd_noalloc(C.addressof(a), _stream_ptr(q)), "pope_b200_attn_fwd_noalloc")
    return out, lse


class _FlashAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, freqs, bias, mask, causal, scale):
        ctx.factors = _factors_of(freqs)        # saved tensors come back as new objects: keep the factors here
        out, lse = attn_forward(q, k, v, freqs, bias, mask, causal, scale, ctx.factors)
        ctx.save_for_backward(q, k, v, freqs, bias, out, lse)
        ctx.mask, ctx.causal, ctx.scale = mask, causal, scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, freqs, bias, out, lse = ctx.saved_tensors
        dq, dk, dv, dfreqs, dbias = attn_backward(dout.to(q.dtype), q, k, v, out, lse, freqs, bias, ctx.mask,
                                                  ctx.causal, ctx.scale,
                                                  ctx.needs_input_grad[3], ctx.needs_input_grad[4], ctx.factors)
        if dfreqs is not None:
            dfreqs = dfreqs.to(freqs.dtype)
        if dbias is not None:
            dbias = dbias.to(bias.dtype)
        return dq, dk, dv, dfreqs, dbias, None, None, None


def flash_attn(q, k, v, freqs=None, bias=None, mask=None, causal=False, softmax_scale=None):
    """Differentiable fused PoPE attention on head-first (b,h,n,d) views.  Without ``freqs`` /
    ``bias`` this is plain softmax attention, as the seam it replaces behaves with ``HAS_POPE``
    off (PoPE_pytorch/triton_pope_flash_attn.py:364-373): the kernels run with zero rotated dims."""
    scale = q.shape[-1] ** -0.5 if softmax_scale is None else softmax_scale
    if freqs is None or bias is None:
        freqs = torch.empty(k.shape[2], 0, dtype=torch.float32, device=q.device)
        bias = torch.empty(k.shape[1], 0, dtype=torch.float32, device=q.device)
    return _FlashAttn.apply(q, k, v, freqs, bias, mask, causal, scale)
