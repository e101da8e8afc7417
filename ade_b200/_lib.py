"""ctypes binding of libade_b200.so (the C ABI declared in include/ade_b200.h).

There is no fallback: if the shared object has not been built (``python -m ade_b200.build``)
loading raises, and every kernel entry raises on a non-zero status.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libade_b200.so")
SHIM_PATH = os.path.join(_HERE, "libade_b200_torch.so")

ADE_OK = 0
ERRORS = {
    -1: "ADE_ERR_NULL: a required pointer is NULL",
    -2: "ADE_ERR_SHAPE: a dimension is outside the supported set",
    -3: "ADE_ERR_ALIGN: a pointer is not 16-byte aligned",
    -4: "ADE_ERR_SCRATCH: scratch buffer too small",
    -5: "ADE_ERR_CUDA: a CUDA runtime call failed",
    -6: "ADE_ERR_DEVICE: the current device is not compute capability 10.x",
}
# ADE_DEV_* of include/ade_b200.h: what the reconstruction kernels write to *status_dev when a wait expires
DEVICE_STATUS = {
    1: "ADE_DEV_TIMEOUT_FULL: MMA warp gave up waiting for an operand stage",
    2: "ADE_DEV_TIMEOUT_EMPTY: unpack warps gave up waiting for a free operand stage",
    3: "ADE_DEV_TIMEOUT_TMEM_FULL: epilogue gave up waiting for an accumulator",
    4: "ADE_DEV_TIMEOUT_TMEM_EMPTY: MMA warp gave up waiting for a free accumulator",
    5: "ADE_DEV_TIMEOUT_SCALES: epilogue gave up waiting for the scale tables of a tile",
    6: "ADE_DEV_TIMEOUT_BASE: epilogue gave up waiting for its box of w_b",
    7: "ADE_DEV_TIMEOUT_STRIP_FREE: unpack warps gave up waiting for the resident U strip to retire",
    8: "ADE_DEV_TIMEOUT_RAW_FULL: unpack warps gave up waiting for packed codes",
    9: "ADE_DEV_TIMEOUT_STRIP_FULL: MMA warp gave up waiting for the resident U strip",
    10: "ADE_DEV_TIMEOUT_RAW_EMPTY: load thread gave up waiting for a free raw slot",
    11: "ADE_DEV_TIMEOUT_SCALES_FREE: scale warp gave up waiting for a free table buffer",
}
# ade_b200_set_option
OPT_WAIT_LIMIT_CYCLES, OPT_COOPERATIVE_LAUNCH, OPT_DROP_SIGNALS, OPT_ATTN_SINGLE_PASS = 1, 2, 3, 4

# every symbol include/ade_b200.h declares
EXPORTS = (
    "ade_b200_device_status", "ade_b200_version", "ade_b200_last_cuda_error",
    "ade_b200_pack_codes", "ade_b200_pack_zeros", "ade_b200_compress_rows",
    "ade_b200_factored_scratch_bytes", "ade_b200_factored_sync_offset", "ade_b200_factored",
    "ade_b200_factored_static", "ade_b200_factored_static_status", "ade_b200_recon", "ade_b200_expand_codes",
    "ade_b200_recon_expanded", "ade_b200_set_option",
    "ade_b200_rmsnorm", "ade_b200_add_rmsnorm", "ade_b200_rope", "ade_b200_silu_mul", "ade_b200_attn_decode",
)


MAX_BLOCKS = 4   # ADE_B200_MAX_BLOCKS


class AdeDelta(ctypes.Structure):
    """struct ade_delta of include/ade_b200.h."""
    _fields_ = [
        ("uq", ctypes.c_void_p), ("vq", ctypes.c_void_p), ("vt", ctypes.c_void_p),
        ("us", ctypes.c_void_p), ("uz", ctypes.c_void_p), ("vs", ctypes.c_void_p), ("vz", ctypes.c_void_p),
        ("M", ctypes.c_int), ("N", ctypes.c_int), ("r", ctypes.c_int),
        ("n_blocks", ctypes.c_int), ("block_rows", ctypes.c_int * (MAX_BLOCKS + 1)), ("block_groups", ctypes.c_int * (MAX_BLOCKS + 1)),
    ]


class AdeKernelError(RuntimeError):
    pass


_lib = None


def load() -> ctypes.CDLL:
    """Load the kernel library; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise AdeKernelError(
            f"{LIB_PATH} is missing: build the CUDA kernels with `python -m ade_b200.build` "
            "(there is no CPU or PyTorch fallback)")
    lib = ctypes.CDLL(LIB_PATH)
    vp, ci, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
    lib.ade_b200_device_status.restype = ci
    lib.ade_b200_version.restype = ci
    lib.ade_b200_last_cuda_error.restype = ci
    lib.ade_b200_pack_codes.argtypes = [vp, vp, ci, ci, ci, vp]
    lib.ade_b200_pack_zeros.argtypes = [vp, vp, sz, vp]
    lib.ade_b200_compress_rows.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, vp]
    lib.ade_b200_compress_rows.restype = ci
    lib.ade_b200_factored_scratch_bytes.argtypes = [ci, ci]
    lib.ade_b200_factored_scratch_bytes.restype = sz
    lib.ade_b200_factored_sync_offset.argtypes = [ci, ci]
    lib.ade_b200_factored_sync_offset.restype = sz
    lib.ade_b200_factored.argtypes = [ctypes.POINTER(AdeDelta), vp, vp, vp, vp, vp, sz, ci, vp]
    lib.ade_b200_factored_static.argtypes = [ctypes.POINTER(AdeDelta), vp, vp, vp, vp, ci, vp]
    lib.ade_b200_factored_static.restype = ci
    lib.ade_b200_recon.argtypes = [ctypes.POINTER(AdeDelta), vp, vp, vp, vp, vp]
    lib.ade_b200_expand_codes.argtypes = [ctypes.POINTER(AdeDelta), vp, vp, vp]
    lib.ade_b200_recon_expanded.argtypes = [ctypes.POINTER(AdeDelta), vp, vp, vp, vp, vp, vp, vp]
    lib.ade_b200_factored_static_status.argtypes = [vp, ci, vp]
    lib.ade_b200_factored_static_status.restype = ci
    ll = ctypes.c_longlong
    lib.ade_b200_rmsnorm.argtypes = [vp, vp, vp, ci, ci, ll, ctypes.c_float, vp]
    lib.ade_b200_rope.argtypes = [vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ll, ll, ll, vp]
    lib.ade_b200_silu_mul.argtypes = [vp, vp, vp, ci, ci, ll, ll, vp]
    lib.ade_b200_add_rmsnorm.argtypes = [vp, vp, vp, vp, vp, ci, ci, ll, ll, ctypes.c_float, vp]
    lib.ade_b200_attn_decode.argtypes = [vp] * 11 + [ci] * 5 + [ll] * 5 + [ctypes.c_float, vp]
    for name in ("ade_b200_rmsnorm", "ade_b200_add_rmsnorm", "ade_b200_rope", "ade_b200_silu_mul", "ade_b200_attn_decode"):
        getattr(lib, name).restype = ci
    lib.ade_b200_set_option.argtypes = [ci, ctypes.c_longlong]
    lib.ade_b200_set_option.restype = ci
    for name in ("ade_b200_pack_codes", "ade_b200_pack_zeros", "ade_b200_factored", "ade_b200_recon", "ade_b200_expand_codes",
                 "ade_b200_recon_expanded"):
        getattr(lib, name).restype = ci
    _lib = lib
    return lib


_ops = None


def ops():
    """``torch.ops.ade_b200``: the thin torch binding of the two hot entry points (csrc/torch_shim.cpp).  Raises if it
    has not been built; there is nothing to fall back to."""
    global _ops
    if _ops is None:
        import torch

        load()                                  # the binding links against the kernel library
        if not os.path.exists(SHIM_PATH):
            raise AdeKernelError(f"{SHIM_PATH} is missing: build it with `python -m ade_b200.build`")
        torch.ops.load_library(SHIM_PATH)
        _ops = torch.ops.ade_b200
    return _ops


def set_option(option: int, value: int) -> None:
    """ade_b200_set_option: wait limit in clock cycles, cooperative launch on / off, diagnostic signal drop."""
    check(load().ade_b200_set_option(option, value), "ade_b200_set_option")


def check(rc: int, what: str) -> None:
    if rc != ADE_OK:
        extra = ""
        if rc == -5:
            extra = f" (cudaError {load().ade_b200_last_cuda_error()})"
        raise AdeKernelError(f"{what}: {ERRORS.get(rc, rc)}{extra}")
