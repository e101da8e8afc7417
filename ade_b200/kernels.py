"""Host side of the B200 delta-application kernels.

Mirrors the public surface of the reference's ``src/kernels.py`` -- ``pack_int4``,
``decode_forward_packed``, ``recon_int4``, ``decode_kernel_status``, ``recon_kernel_status``
(the five names ``src/serving.py:35`` imports) -- on top of the C ABI of include/ade_b200.h.
Differences a caller sees: 16-bit tensors are bfloat16 (the reference kernels are float16),
the stored form has its own layout (see ``pack_int4``), nothing is compiled at run time and
there is no autotuning pass or PyTorch fallback: a missing library or an unsupported shape
raises.
"""
from __future__ import annotations

import contextlib
import ctypes

import torch

from . import _lib

GROUP = 128
_NIBBLE_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)      # nibble i of a 32-bit word holds code _NIBBLE_ORDER[i]
STORED_KEYS = ("uq", "vq", "vt", "us", "uz", "vs", "vz")


# ---------------------------------------------------------------------------- status
def _status(device) -> tuple[bool, str]:
    dev = torch.device(device)
    if dev.type != "cuda" or not torch.cuda.is_available():
        return False, "no CUDA device"
    major, minor = torch.cuda.get_device_capability(dev)
    if major != 10:
        return False, f"compute capability {major}.{minor} is not 10.x (the kernels are built for sm_100a only)"
    try:
        lib = _lib.load()
    except _lib.AdeKernelError as e:
        return False, str(e)
    with torch.cuda.device(dev):
        rc = lib.ade_b200_device_status()
    if rc != 0:
        return False, _lib.ERRORS.get(rc, str(rc))
    return True, f"sm_{major}{minor}a"


def recon_kernel_status(device="cuda"):
    """Whether the tcgen05 reconstruction kernel can run on `device` (src/kernels.py:86-104)."""
    return _status(device)


def decode_kernel_status(device="cuda"):
    """Whether the factored-application kernels can run on `device` (src/kernels.py:107-124)."""
    return _status(device)


# ---------------------------------------------------------------------------- stored form
def pack_nibbles(codes: torch.Tensor) -> torch.Tensor:
    """(..., K) uint8 codes in 0..15 -> (..., K/2) uint8, eight codes per 32-bit word.

    Replaces ``_pack_nibbles`` (src/kernels.py:145-161).  Nibble i of each little-endian word
    holds code (0, 2, 4, 6, 1, 3, 5, 7)[i] of its 8 codes, so ``(w >> 4j) & 0x000F000F`` is the
    adjacent pair (c_2j, c_2j+1) in the two halves of a register.
    """
    K = codes.shape[-1]
    if K % 8:
        raise ValueError(f"pack_nibbles: last dimension {K} is not a multiple of 8")
    c = codes.to(torch.uint8).reshape(*codes.shape[:-1], K // 8, 8)[..., list(_NIBBLE_ORDER)]
    return (c[..., 0::2] | (c[..., 1::2] << 4)).reshape(*codes.shape[:-1], K // 2).contiguous()


def unpack_nibbles(packed: torch.Tensor) -> torch.Tensor:
    """Inverse of ``pack_nibbles`` (used by tests and tools, not by the kernels)."""
    K2 = packed.shape[-1]
    b = packed.reshape(*packed.shape[:-1], K2 // 4, 4)
    nib = torch.stack([b & 15, b >> 4], -1).reshape(*packed.shape[:-1], K2 // 4, 8)   # nibble order
    out = torch.empty_like(nib)
    out[..., list(_NIBBLE_ORDER)] = nib
    return out.reshape(*packed.shape[:-1], K2 * 2)


def pack_int4(packed: dict, group_size: int = GROUP, device=None) -> dict:
    """Stored form of one compressed module, read by both kernels (replaces src/kernels.py:164-188).

    Parameters:
        packed: dict with U_codes, U_scale, U_zero, Vt_codes, Vt_scale, Vt_zero as
            ``quantization.compress_module`` writes them (src/quantization.py:276-285).
        group_size: G; only 128 is supported.
        device: where to build the stored form (default: where the packed tensors are).

    Returns:
        dict with ``uq`` (M, r/2), ``vq`` (N, r/2), ``vt`` (r, N/2) uint8 nibble-packed codes,
        ``us`` (M, ng) / ``vs`` (ng, N) bfloat16 scales, ``uz`` (M, ng) / ``vz`` (ng, N) uint8
        zero-points, and the ints ``M``, ``N``, ``r``.  Unlike the reference there are no FP32
        side tables: the kernels subtract the zero-points from the codes before contracting.
    """
    if group_size != GROUP:
        raise ValueError("the kernels are specialised for group size 128")
    dev = torch.device(device) if device is not None else packed["U_codes"].device
    M, r = packed["U_codes"].shape
    r2, N = packed["Vt_codes"].shape
    if r != r2 or r % GROUP:
        raise ValueError(f"pack_int4: rank {r} / {r2} must match and be a multiple of {GROUP}")
    if N % 8:
        raise ValueError(f"pack_int4: d_i = {N} must be a multiple of 8")
    if dev.type == "cuda":
        return _pack_int4_cuda(packed, dev)
    uc = packed["U_codes"].to(dev, torch.uint8)
    vc = packed["Vt_codes"].to(dev, torch.uint8)
    out = {
        "uq": pack_nibbles(uc),
        "vq": pack_nibbles(vc.t().contiguous()),
        "vt": pack_nibbles(vc),
        "us": packed["U_scale"].to(dev, torch.bfloat16).contiguous(),
        "uz": packed["U_zero"].to(dev).to(torch.float32).to(torch.uint8).contiguous(),
        "vs": packed["Vt_scale"].to(dev, torch.bfloat16).contiguous(),
        "vz": packed["Vt_zero"].to(dev).to(torch.float32).to(torch.uint8).contiguous(),
        "M": M, "N": N, "r": r,
    }
    return out


_loaders: dict = {}


def _pack_int4_cuda(packed: dict, dev: torch.device) -> dict:
    """Stored form built by the packing kernels of the C ABI.  Fields that live on the CPU go through the pinned
    staging path of ``packed_io.DeviceDeltaLoader`` (one copy, then kernels); fields already on the device are
    packed where they are, on the current stream."""
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    if all(packed[k].device.type == "cpu" for k in ("U_codes", "Vt_codes", "U_scale", "U_zero", "Vt_scale", "Vt_zero")):
        from .packed_io import DeviceDeltaLoader

        loader = _loaders.get(dev.index)
        if loader is None:
            loader = _loaders[dev.index] = DeviceDeltaLoader(dev)
        out = loader.load(packed)
        loader.finish()
        return out
    lib = _lib.load()
    uc = packed["U_codes"].to(dev, torch.uint8).contiguous()
    vc = packed["Vt_codes"].to(dev, torch.uint8).contiguous()
    uzb = packed["U_zero"].to(dev, torch.bfloat16).contiguous()
    vzb = packed["Vt_zero"].to(dev, torch.bfloat16).contiguous()
    M, r = uc.shape
    N = vc.shape[1]
    ng = r // GROUP
    out = {
        "uq": torch.empty(M, r // 2, dtype=torch.uint8, device=dev),
        "vq": torch.empty(N, r // 2, dtype=torch.uint8, device=dev),
        "vt": torch.empty(r, N // 2, dtype=torch.uint8, device=dev),
        "us": packed["U_scale"].to(dev, torch.bfloat16).contiguous(),
        "uz": torch.empty(M, ng, dtype=torch.uint8, device=dev),
        "vs": packed["Vt_scale"].to(dev, torch.bfloat16).contiguous(),
        "vz": torch.empty(ng, N, dtype=torch.uint8, device=dev),
        "M": M, "N": N, "r": r,
    }
    with _on_device(dev):
        sp = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.ade_b200_pack_codes(uc.data_ptr(), out["uq"].data_ptr(), M, r, 0, sp), "ade_b200_pack_codes(U)")
        _lib.check(lib.ade_b200_pack_codes(vc.data_ptr(), out["vt"].data_ptr(), r, N, 0, sp), "ade_b200_pack_codes(Vt)")
        _lib.check(lib.ade_b200_pack_codes(vc.data_ptr(), out["vq"].data_ptr(), N, r, 1, sp), "ade_b200_pack_codes(V)")
        _lib.check(lib.ade_b200_pack_zeros(uzb.data_ptr(), out["uz"].data_ptr(), M * ng, sp), "ade_b200_pack_zeros(U)")
        _lib.check(lib.ade_b200_pack_zeros(vzb.data_ptr(), out["vz"].data_ptr(), ng * N, sp), "ade_b200_pack_zeros(Vt)")
    return out


def _cdelta(p4: dict):
    """ctypes view of a stored form, cached in the dict (rebuilt if the tensors moved)."""
    key = tuple(p4[k].data_ptr() for k in STORED_KEYS)
    c = p4.get("_cdelta")
    if c is None or c[0] != key:
        for k in STORED_KEYS:
            t = p4[k]
            if not (t.is_cuda and t.is_contiguous()):
                raise ValueError(f"stored form tensor {k} must be a contiguous CUDA tensor")
        d = _lib.AdeDelta(*key, int(p4["M"]), int(p4["N"]), int(p4["r"]))
        blocks = p4.get("blocks")              # [(row_begin, group_begin), ..., (M, ng)] of a block-diagonal U^
        if blocks:
            if not 2 <= len(blocks) <= _lib.MAX_BLOCKS + 1:
                raise ValueError("stored form: at most %d blocks" % _lib.MAX_BLOCKS)
            d.n_blocks = len(blocks) - 1
            for i, (row, grp) in enumerate(blocks):
                d.block_rows[i], d.block_groups[i] = int(row), int(grp)
        c = p4["_cdelta"] = (key, d)
    return c[1]


# ---------------------------------------------------------------------------- launches
_NULL = contextlib.nullcontext()


def _on_device(dev: torch.device):
    """Device guard for a launch; free when `dev` is already current (the guard costs ~10 us of host time)."""
    return _NULL if dev.index is None or dev.index == torch.cuda.current_device() else torch.cuda.device(dev)


_scratch: dict = {}


def _scratch_for(dev: torch.device, stream_ptr: int, T: int, r: int, nbytes: int) -> torch.Tensor:
    """Scratch per (device, stream, T, r): h = V^T x and the kernel's three sync words, which must
    start at zero and are left at zero by every completed call (so one zero-fill at allocation)."""
    key = (dev.index, stream_ptr, T, r)
    buf = _scratch.get(key)
    if buf is None:
        buf = _scratch[key] = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    return buf


def check_factored_status(dev=None) -> None:
    """Raise if any factored launch on `dev` (default: every device) recorded an expired wait for h in its
    scratch buffer: the output of that launch was undefined.  Synchronises the devices it looks at, so it belongs
    at the end of a generation or a benchmark, not between launches."""
    lib = _lib.load()
    index = None if dev is None else (torch.device(dev).index if torch.device(dev).index is not None else torch.cuda.current_device())
    for (di, stream_ptr, T, r), buf in list(_scratch.items()):
        if index is not None and di != index:
            continue
        off = lib.ade_b200_factored_sync_offset(T, r)
        if int(buf[off:off + 12].view(torch.int32)[2].item()) != 0:
            raise _lib.AdeKernelError(
                f"factored kernel on cuda:{di} (T={T}, r={r}): the grid-wide wait for h = V^T x expired; the output of "
                "that launch is undefined (zero the scratch buffer's sync words before reusing it)")


def reset_factored_scratch(dev=None) -> None:
    """Zero the sync words of the cached scratch buffers (after a launch whose wait expired)."""
    index = None if dev is None else (torch.device(dev).index if torch.device(dev).index is not None else torch.cuda.current_device())
    for (di, _, _, _), buf in _scratch.items():
        if index is None or di == index:
            buf.zero_()


def factored_status(dev, T: int, r: int, stream_ptr: int | None = None) -> int:
    """Status word of the scratch buffer used for (T, r) on `dev` (0 = every wait completed).
    Synchronises the device."""
    dev = torch.device(dev)
    if stream_ptr is None:
        with torch.cuda.device(dev):
            stream_ptr = torch.cuda.current_stream().cuda_stream
    buf = _scratch.get((dev.index if dev.index is not None else torch.cuda.current_device(), stream_ptr, T, r))
    if buf is None:
        return 0
    off = _lib.load().ade_b200_factored_sync_offset(T, r)
    return int(buf[off:off + 12].view(torch.int32)[2].item())


def _check_x(x: torch.Tensor, N: int, what: str):
    if x.dtype != torch.bfloat16 or not x.is_cuda or not x.is_contiguous() or x.dim() != 2 or x.shape[1] != N:
        raise ValueError(f"{what} must be a contiguous CUDA bfloat16 tensor of shape (T, {N}); got "
                         f"{tuple(x.shape)} {x.dtype} on {x.device}")


def factored_forward(x: torch.Tensor, p4: dict, weight: torch.Tensor | None = None,
                     y_dense: torch.Tensor | None = None) -> torch.Tensor:
    """out = base + U^(V^T x) for T <= 128 tokens; base = x W_b^T computed in-kernel when `weight`
    is given, else the supplied `y_dense`.  One call of ``ade_b200_factored``."""
    lib = _lib.load()
    M, N, r = int(p4["M"]), int(p4["N"]), int(p4["r"])
    _check_x(x, N, "x")
    T = x.shape[0]
    if (weight is None) == (y_dense is None):
        raise ValueError("give exactly one of weight (fused base GEMM) or y_dense")
    if weight is not None and not (weight.dtype == torch.bfloat16 and weight.is_contiguous()
                                   and tuple(weight.shape) == (M, N) and weight.device == x.device):
        raise ValueError("weight must be a contiguous bfloat16 (d_o, d_i) tensor on x's device")
    if y_dense is not None:
        _check_x(y_dense, M, "y_dense")
        if y_dense.shape[0] != T:
            raise ValueError("y_dense and x disagree on T")
    with _on_device(x.device):
        stream = torch.cuda.current_stream().cuda_stream
        scratch = _scratch_for(x.device, stream, T, r, lib.ade_b200_factored_scratch_bytes(T, r))
        # through the torch binding: it allocates the output, takes torch's current stream and calls ade_b200_factored
        try:
            return _lib.ops().factored(x, weight, y_dense, p4["uq"], p4["vq"], p4["vt"], p4["us"], p4["uz"], p4["vs"], p4["vz"],
                                       M, N, r, _flat_blocks(p4), scratch)
        except RuntimeError as e:
            raise _kernel_error(e) from None


def _kernel_error(e: RuntimeError) -> Exception:
    """A status the C ABI returned comes back from the binding as a RuntimeError; give it the library's own type."""
    msg = str(e).split("\n")[0]
    return _lib.AdeKernelError(msg) if msg.startswith("ade_b200_") else e


def _flat_blocks(p4: dict):
    """Block structure of a fused group's U^ as the flat (row, group, row, group, ...) list the binding takes."""
    fb = p4.get("_flat_blocks")
    if fb is None:
        blocks = p4.get("blocks")
        if blocks and not 2 <= len(blocks) <= _lib.MAX_BLOCKS + 1:
            raise ValueError("stored form: at most %d blocks" % _lib.MAX_BLOCKS)
        fb = p4["_flat_blocks"] = [int(v) for pair in (blocks or []) for v in pair]
    return fb


def decode_forward_packed(x, y_dense, p4, group_size=GROUP, split_k=False):
    """Factored application y_dense + U^ (V^^T x) (same signature as src/kernels.py:1182-1200).

    x (T, d_i) and y_dense (T, d_o) are contiguous bfloat16 CUDA tensors; returns a fresh (T, d_o)
    bfloat16 tensor.  `split_k` is accepted for compatibility and ignored: the contraction is
    split inside a CTA and reduced in a fixed order, so there is no atomic variant to choose.
    """
    if group_size != GROUP:
        raise ValueError("the kernels are specialised for group size 128")
    return factored_forward(x, p4, y_dense=y_dense)


def expand_codes(p4):
    """(u8, v8): the int8 operands of the reconstruction, code minus zero-point, (d_o, r) and (d_i, r).

    The reference's kernel unpacks nibbles and subtracts zero-points in its main loop on every call
    (src/kernels.py:296-331).  A module that reconstructs often does it once: `recon_int4(..., expanded=(u8, v8))`
    reads these arrays by TMA straight into the operand tiles and has no unpack role.  Costs (d_o + d_i) * r bytes
    (twice the packed codes)."""
    M, N, r = int(p4["M"]), int(p4["N"]), int(p4["r"])
    with _on_device(p4["uq"].device):
        try:
            return _lib.ops().expand(p4["uq"], p4["vq"], p4["vt"], p4["us"], p4["uz"], p4["vs"], p4["vz"], M, N, r)
        except RuntimeError as e:
            raise _kernel_error(e) from None


def recon_int4(p4, base, group_size=GROUP, dbg_acc=None, status=None, expanded=None):
    """W_b + U^ V^^T of one module in bfloat16 (same role as src/kernels.py:431-444).

    `dbg_acc`: optional int32 (ng, d_o, d_i) CUDA tensor that receives every group's INT32
    accumulator; `status`: optional int32 CUDA scalar tensor for the kernel's timeout code;
    `expanded`: optional (u8, v8) from `expand_codes(p4)`: same result, bit for bit, from the faster kernel.
    """
    if group_size != GROUP:
        raise ValueError("the kernels are specialised for group size 128")
    M, N, r = int(p4["M"]), int(p4["N"]), int(p4["r"])
    if not (base.dtype == torch.bfloat16 and base.is_cuda and tuple(base.shape) == (M, N)):
        raise ValueError(f"base must be a CUDA bfloat16 ({M}, {N}) tensor")
    if dbg_acc is not None and not (dbg_acc.dtype == torch.int32 and dbg_acc.is_contiguous()
                                    and tuple(dbg_acc.shape) == (r // GROUP, M, N)):
        raise ValueError("dbg_acc must be a contiguous int32 (ng, d_o, d_i) tensor")
    with _on_device(base.device):
        try:
            u8, v8 = expanded if expanded is not None else (None, None)
            return _lib.ops().recon(base, p4["uq"], p4["vq"], p4["vt"], p4["us"], p4["uz"], p4["vs"], p4["vz"], M, N, r, dbg_acc, status,
                                    u8, v8)
        except RuntimeError as e:
            raise _kernel_error(e) from None
