"""ctypes bindings of the native libraries (C ABI declared in csrc/include/hipress/capi.h).

``cpu()`` and ``cuda()`` load ``libhipress_cpu.so`` / ``libhipress_cuda.so`` from this
directory, building them first when they are missing and a compiler is present.
``cuda()`` raises :class:`NativeLibraryError` rather than falling back to anything
else: on a GPU box the CUDA path is the only path.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

HERE = Path(__file__).resolve().parent

MAX_RANKS = 8
MAX_SEGS = 40
TOPO_RING = 0
TOPO_PS = 1
STATUS_TIMEOUT = 0x80000000

ERR_NAMES = {-1: "bad argument", -2: "bucket too large", -3: "emulated ranks would not be co-resident"}


class NativeLibraryError(RuntimeError):
    pass


class HpSeg(C.Structure):
    _fields_ = [("g", C.c_void_p), ("r", C.c_void_p), ("out", C.c_void_p), ("sr", C.c_void_p),
                ("n", C.c_uint64), ("id", C.c_uint32), ("pad", C.c_uint32)]


class HpComm(C.Structure):
    _fields_ = [("nranks", C.c_int32), ("rank", C.c_int32), ("emulate", C.c_int32),
                ("epoch", C.c_uint32), ("timeout_ns", C.c_uint64),
                ("inbox", C.c_void_p * MAX_RANKS), ("flags", C.c_void_p * MAX_RANKS),
                ("status", C.c_void_p),
                ("emu_stride_g", C.c_int64), ("emu_stride_r", C.c_int64),
                ("emu_stride_out", C.c_int64), ("emu_stride_sr", C.c_int64),
                ("trace", C.c_void_p)]


_cpu = None
_cuda = None


def _ensure_built():
    from . import build as _b
    try:
        _b.build()
    except Exception as e:  # compiler missing or failing: report at load time
        return e
    return None


def _sig(fn, restype, *argtypes):
    fn.restype = restype
    fn.argtypes = list(argtypes)


def cpu():
    """The CPU library (oracle + host runtime)."""
    global _cpu
    if _cpu is not None:
        return _cpu
    path = HERE / "libhipress_cpu.so"
    err = None
    if not path.exists() or os.environ.get("HIPRESS_REBUILD"):
        err = _ensure_built()
    if not path.exists():
        raise NativeLibraryError(f"{path} missing and could not be built: {err}")
    L = C.CDLL(str(path))
    u8p, f32p, vp = C.c_void_p, C.c_void_p, C.c_void_p
    _sig(L.hp_dense_payload_bytes, C.c_uint64, C.c_int, C.c_int, C.c_uint64)
    _sig(L.hp_sparse_payload_bytes, C.c_uint64, C.c_uint64)
    _sig(L.hp_sparse_k, C.c_uint64, C.c_uint64, C.c_float)
    _sig(L.hp_tile_elems, C.c_int)
    _sig(L.hp_cpu_dense_encode, C.c_int, C.c_int, C.c_int, f32p, f32p, u8p, u8p, C.c_uint64,
         C.c_float, C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint64)
    _sig(L.hp_cpu_dense_decode, C.c_int, C.c_int, C.c_int, u8p, f32p, C.c_uint64, C.c_float,
         C.c_float, C.c_int)
    _sig(L.hp_cpu_dgc_update, C.c_int, f32p, f32p, f32p, C.c_uint64, C.c_float)
    _sig(L.hp_cpu_acc_update, C.c_int, f32p, f32p, C.c_uint64)
    _sig(L.hp_cpu_sparse_select, C.c_int, C.c_int, f32p, f32p, C.c_uint64, C.c_uint64, u8p,
         C.c_uint64)
    _sig(L.hp_cpu_sparse_decode, C.c_int, u8p, f32p, C.c_uint64, C.c_uint64, C.c_float, C.c_int)
    for name, sig in _CPU_OPTIONAL.items():
        if hasattr(L, name):
            _sig(getattr(L, name), *sig)
    _cpu = L
    return L


# symbols added by later translation units of the CPU library (planner, scheduler)
_CPU_OPTIONAL: dict = {
    "hp_payload_check": (C.c_int, C.c_void_p, C.c_uint64, C.c_int, C.c_int, C.c_uint64, C.c_uint64),
    "hp_plan_buckets": (C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64,
                        C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                        C.c_void_p, C.c_void_p, C.c_void_p),
}


def cuda():
    """The CUDA library.  Raises if it is missing: there is no silent fallback."""
    global _cuda
    if _cuda is not None:
        return _cuda
    path = HERE / "libhipress_cuda.so"
    err = None
    if os.environ.get("HIPRESS_DEBUG", "0") not in ("", "0"):
        # the build with per-access bounds checks in the kernels (-DHIPRESS_DEBUG)
        from . import build as _b
        path = HERE / "libhipress_cuda_debug.so"
        try:
            _b.build_debug()
        except Exception as e:  # noqa: BLE001
            err = e
    elif not path.exists() or os.environ.get("HIPRESS_REBUILD"):
        err = _ensure_built()
    if not path.exists():
        raise NativeLibraryError(
            f"{path} missing and could not be built ({err}); run python -m hipress_b200._native.build")
    L = C.CDLL(str(path))
    vp = C.c_void_p
    _sig(L.hp_cuda_device_count, C.c_int)
    _sig(L.hp_cuda_error_string, C.c_char_p, C.c_int)
    _sig(L.hp_cuda_dense_encode, C.c_int, C.c_int, C.c_int, vp, vp, vp, vp, C.c_uint64, C.c_float,
         C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint64, C.c_int, vp)
    _sig(L.hp_cuda_dense_decode, C.c_int, C.c_int, C.c_int, vp, vp, C.c_uint64, C.c_float,
         C.c_float, C.c_int, C.c_int, vp)
    _sig(L.hp_fused_dense_layout, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_uint64),
         C.c_int, C.c_int, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.POINTER(C.c_uint32))
    _sig(L.hp_fused_chunk_elems, C.c_uint64, C.c_uint64, C.c_int)
    _sig(L.hp_cuda_debug_build, C.c_int)
    _sig(L.hp_cuda_debug_set_inbox_limit, C.c_int, C.c_uint64)
    _sig(L.hp_cuda_fused_dense, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(HpSeg), C.c_int,
         C.POINTER(HpComm), C.c_float, C.c_uint64, C.c_uint32, C.c_uint32, C.c_int, vp)
    _sig(L.hp_sparse_workspace_bytes, C.c_uint64)
    _sig(L.hp_cuda_sparse_encode, C.c_int, C.c_int, vp, vp, vp, C.c_uint64, C.c_uint64,
         C.c_uint64, C.c_float, C.c_int, vp, vp, C.c_uint64, C.c_int, vp)
    _sig(L.hp_sparse_workspace_bytes_for, C.c_uint64, C.c_uint64)
    _sig(L.hp_cuda_sparse_decode, C.c_int, vp, vp, C.c_uint64, C.c_uint64, C.c_float, C.c_int, vp)
    _sig(L.hp_cuda_arena_alloc, C.c_int, C.c_uint64, C.POINTER(C.c_void_p))
    _sig(L.hp_cuda_arena_free, C.c_int, vp)
    _sig(L.hp_cuda_ipc_handle_bytes, C.c_int)
    _sig(L.hp_cuda_ipc_export, C.c_int, vp, vp)
    _sig(L.hp_cuda_ipc_open, C.c_int, vp, C.POINTER(C.c_void_p))
    _sig(L.hp_cuda_ipc_close, C.c_int, vp)
    _sig(L.hp_cuda_enable_peer, C.c_int, C.c_int, C.c_int)
    _sig(L.hp_cuda_peer_store, C.c_int, vp, vp, C.c_uint64, C.c_int, vp)
    _sig(L.hp_cuda_wait_probe, C.c_int, vp, C.c_uint32, C.c_uint64, vp, vp)
    _sig(L.hp_cuda_set_flag, C.c_int, vp, C.c_uint32, vp)
    _sig(L.hp_cuda_partition_stream_create, C.c_int, C.c_int, C.c_int, C.c_int,
         C.POINTER(C.c_void_p), C.POINTER(C.c_int), C.POINTER(C.c_void_p))
    _sig(L.hp_cuda_partition_stream_destroy, C.c_int, vp, vp)
    for name, sig in _CUDA_OPTIONAL.items():
        if hasattr(L, name):
            _sig(getattr(L, name), *sig)
    _cuda = L
    return L


_CUDA_OPTIONAL: dict = {}


def check(code: int, what: str = "native call", device_call: bool = True):
    """Raise on a non-zero return code of an ``hp_*`` function (``device_call``:
    positive codes are CUDA runtime errors; otherwise the CPU library's own)."""
    if code == 0:
        return
    if code < 0:
        raise NativeLibraryError(f"{what}: {ERR_NAMES.get(code, code)}")
    if not device_call:
        raise NativeLibraryError(f"{what}: invalid argument or payload (code {code})")
    msg = cuda().hp_cuda_error_string(code).decode() if _cuda is not None else str(code)
    raise NativeLibraryError(f"{what}: CUDA error {code}: {msg}")


def ptr(t):
    """Device or host address of a tensor (``None`` -> NULL)."""
    return None if t is None else t.data_ptr()


def stream_ptr(stream=None):
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream
