"""Compressed-delta files (``ade_packed_v1``) and their one-pass route to the device stored form.

The file format is the reference's (``save_packed`` / ``load_packed``, src/utils.py:146-186): a ``.pt`` file
holding one flat dict, ``"<module prefix>.<field>"`` -> tensor for the six packed fields of every module plus
``"__meta__"`` with ``format == "ade_packed_v1"``; files written by either implementation load in the other.

What differs is how a file becomes something the kernels can read.  The reference loads every tensor to the
CPU, and each module constructor then packs nibbles and builds side tables with int64 torch ops on the CPU
(src/kernels.py:145-188 called from src/serving.py:174-190): O(d r) host work per module, 224-280 modules per
model.  Here ``PackedDeltaFile`` memory-maps the file, and ``DeviceDeltaLoader`` streams it module by module
through a pinned staging buffer to the GPU, where the packing kernels of the C ABI (``ade_b200_pack_codes`` /
``ade_b200_pack_zeros``) write ``uq / vq / vt / uz / vz`` straight into their final buffers on a side stream:
the host only copies bytes, and the copy of module i+1 overlaps the packing of module i.
"""
from __future__ import annotations

import os
import tempfile

import torch

from . import _lib

PACKED_FORMAT = "ade_packed_v1"
PACKED_FIELDS = ("U_codes", "U_scale", "U_zero", "Vt_codes", "Vt_scale", "Vt_zero")
GROUP = 128


def _check_module(prefix: str, packed: dict) -> tuple[int, int, int]:
    """Shapes of one module's fields must agree with each other; returns (d_o, d_i, rank)."""
    absent = [f for f in PACKED_FIELDS if f not in packed]
    if absent:
        raise ValueError(f"{prefix} misses {absent}")
    M, r = packed["U_codes"].shape
    r2, N = packed["Vt_codes"].shape
    ng = r // GROUP
    want = {"U_scale": (M, ng), "U_zero": (M, ng), "Vt_scale": (ng, N), "Vt_zero": (ng, N)}
    if r != r2 or r % GROUP or any(tuple(packed[k].shape) != v for k, v in want.items()):
        raise ValueError(f"{prefix}: inconsistent packed shapes " + str({k: tuple(packed[k].shape) for k in PACKED_FIELDS}))
    return M, N, r


def save_packed(path: str, per_module: dict, meta: dict) -> None:
    """Write {module prefix: packed dict} as an ``ade_packed_v1`` file.  Every module is validated first; the
    file appears under its final name only when it is complete (written next to it, then renamed)."""
    entries = {"__meta__": {**meta, "format": PACKED_FORMAT}}
    for prefix, packed in per_module.items():
        _check_module(prefix, packed)
        entries.update((f"{prefix}.{field}", packed[field]) for field in PACKED_FIELDS)
    folder = os.path.dirname(os.path.abspath(path))
    os.makedirs(folder, exist_ok=True)
    fd, tmp = tempfile.mkstemp(dir=folder, prefix=os.path.basename(path) + ".", suffix=".part")
    os.close(fd)
    try:
        torch.save(entries, tmp)
        os.replace(tmp, path)
    except BaseException:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise


class PackedDeltaFile:
    """An ``ade_packed_v1`` file opened for reading.  Tensors are memory-mapped where torch can (files written by
    ``torch.save`` in its zip format), so opening costs no copy and a module's bytes are read when it is used."""

    def __init__(self, path: str):
        self.path = path
        try:
            flat = torch.load(path, map_location="cpu", mmap=True)
        except (RuntimeError, ValueError):            # legacy (non-zip) serialisation cannot be mapped
            flat = torch.load(path, map_location="cpu")
        meta = flat.pop("__meta__", None) if isinstance(flat, dict) else None
        if not isinstance(meta, dict) or meta.get("format") != PACKED_FORMAT:
            raise ValueError(f"{path} is not an ADE compressed delta (meta={meta!r})")
        self.meta = meta
        self._modules: dict = {}
        for key, tensor in flat.items():
            prefix, _, field = key.rpartition(".")
            self._modules.setdefault(prefix, {})[field] = tensor
        self.dims = {}
        for prefix, packed in self._modules.items():
            try:
                self.dims[prefix] = _check_module(prefix, packed)
            except ValueError as e:
                raise ValueError(f"{e} in {path}") from None

    def __len__(self):
        return len(self._modules)

    def __iter__(self):
        return iter(self._modules)

    def __contains__(self, prefix):
        return prefix in self._modules

    def module(self, prefix: str) -> dict:
        return self._modules[prefix]

    def as_dict(self) -> dict:
        return dict(self._modules)


def load_packed(path: str):
    """(per_module, meta) of a compressed delta, the reference's return convention (src/utils.py:162-186)."""
    f = PackedDeltaFile(path)
    return f.as_dict(), f.meta


class DeviceDeltaLoader:
    """Builds device stored forms (the dict ``kernels.pack_int4`` returns) from packed modules in one pass.

    Per module: the six fields are copied into one pinned staging block (two blocks alternate), sent to the GPU
    with one asynchronous copy on a side stream, and packed there by ``ade_b200_pack_codes`` (uq, vt, and vq
    with the transposing read) and ``ade_b200_pack_zeros``; scales are already in their final form.  The staging
    blocks are sized for the largest module seen and reused.  ``finish()`` joins the side stream.
    """

    def __init__(self, device="cuda"):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ValueError("DeviceDeltaLoader needs a CUDA device")
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.lib = _lib.load()
        self.stream = torch.cuda.Stream(device=self.device)
        self._pinned = [None, None]
        self._staged = [None, None]
        self._free = [None, None]                 # event: the packing kernels that read this block are done
        self._turn = 0

    @staticmethod
    def _layout(M, N, r):
        """Byte offsets of the fields inside a staging block (256-byte aligned) and its total size."""
        ng = r // GROUP
        sizes = {"U_codes": M * r, "Vt_codes": r * N, "U_scale": 2 * M * ng, "Vt_scale": 2 * ng * N,
                 "U_zero": 2 * M * ng, "Vt_zero": 2 * ng * N}
        off, pos = {}, 0
        for k in ("U_codes", "Vt_codes", "U_scale", "Vt_scale", "U_zero", "Vt_zero"):
            off[k] = (pos, sizes[k])
            pos += (sizes[k] + 255) & ~255
        return off, pos

    def _blocks(self, nbytes):
        t = self._turn
        if self._pinned[t] is None or self._pinned[t].numel() < nbytes:
            if self._free[t] is not None:
                self._free[t].synchronize()
            self._pinned[t] = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
            self._staged[t] = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        return self._pinned[t], self._staged[t]

    def load(self, packed: dict) -> dict:
        """Stored form of one module on the device.  `packed` holds CPU (or memory-mapped) tensors in the layout
        of src/quantization.py:276-285: uint8 codes, bfloat16 scales and zero-points."""
        M, N, r = _check_module("module", packed)
        if N % 8:
            raise ValueError(f"d_i = {N} must be a multiple of 8")
        ng = r // GROUP
        off, total = self._layout(M, N, r)
        pinned, staged = self._blocks(total)
        t = self._turn
        if self._free[t] is not None:
            self._free[t].synchronize()            # the block's previous contents have been consumed
        for k, (o, n) in off.items():
            src = packed[k]
            src = src.to(torch.uint8) if k.endswith("codes") else src.to(torch.bfloat16)
            pinned[o:o + n].copy_(src.contiguous().reshape(-1).view(torch.uint8))
        dev = self.device
        out = {
            "uq": torch.empty(M, r // 2, dtype=torch.uint8, device=dev),
            "vq": torch.empty(N, r // 2, dtype=torch.uint8, device=dev),
            "vt": torch.empty(r, N // 2, dtype=torch.uint8, device=dev),
            "us": torch.empty(M, ng, dtype=torch.bfloat16, device=dev),
            "uz": torch.empty(M, ng, dtype=torch.uint8, device=dev),
            "vs": torch.empty(ng, N, dtype=torch.bfloat16, device=dev),
            "vz": torch.empty(ng, N, dtype=torch.uint8, device=dev),
            "M": M, "N": N, "r": r,
        }
        lib, check = self.lib, _lib.check
        with torch.cuda.device(dev), torch.cuda.stream(self.stream):
            sp = self.stream.cuda_stream
            staged[:total].copy_(pinned[:total], non_blocking=True)
            base = staged.data_ptr()
            at = lambda k: base + off[k][0]
            check(lib.ade_b200_pack_codes(at("U_codes"), out["uq"].data_ptr(), M, r, 0, sp), "ade_b200_pack_codes(U)")
            check(lib.ade_b200_pack_codes(at("Vt_codes"), out["vt"].data_ptr(), r, N, 0, sp), "ade_b200_pack_codes(Vt)")
            check(lib.ade_b200_pack_codes(at("Vt_codes"), out["vq"].data_ptr(), N, r, 1, sp), "ade_b200_pack_codes(V)")
            check(lib.ade_b200_pack_zeros(at("U_zero"), out["uz"].data_ptr(), M * ng, sp), "ade_b200_pack_zeros(U)")
            check(lib.ade_b200_pack_zeros(at("Vt_zero"), out["vz"].data_ptr(), ng * N, sp), "ade_b200_pack_zeros(Vt)")
            out["us"].view(torch.uint8).reshape(-1).copy_(staged[off["U_scale"][0]:off["U_scale"][0] + off["U_scale"][1]])
            out["vs"].view(torch.uint8).reshape(-1).copy_(staged[off["Vt_scale"][0]:off["Vt_scale"][0] + off["Vt_scale"][1]])
            ev = torch.cuda.Event()
            ev.record(self.stream)
        for v in out.values():
            if torch.is_tensor(v):
                v.record_stream(self.stream)
        self._free[t] = ev
        self._turn ^= 1
        return out

    def finish(self):
        """Make the current stream wait for every packing kernel issued so far."""
        torch.cuda.current_stream(self.device).wait_stream(self.stream)
