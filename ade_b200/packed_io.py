"""On-disk format of a compressed delta: the ``ade_packed_v1`` flat dict in a ``.pt`` file.

Same format as the reference's ``save_packed`` / ``load_packed`` (src/utils.py:146-186): one entry
``"<module prefix>.<field>"`` per packed field plus ``"__meta__"`` with ``format = "ade_packed_v1"``.
Files written by either implementation load in the other.
"""
from __future__ import annotations

import os

import torch

PACKED_FORMAT = "ade_packed_v1"
PACKED_FIELDS = ("U_codes", "U_scale", "U_zero", "Vt_codes", "Vt_scale", "Vt_zero")


def save_packed(path: str, per_module: dict, meta: dict) -> None:
    """Write `per_module` (prefix -> packed dict) atomically: temp file, then rename."""
    os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
    flat = {"__meta__": dict(meta, format=PACKED_FORMAT)}
    for prefix, packed in per_module.items():
        for field in PACKED_FIELDS:
            flat[f"{prefix}.{field}"] = packed[field]
    torch.save(flat, path + ".tmp")
    os.replace(path + ".tmp", path)


def load_packed(path: str):
    """Read a compressed delta; returns (per_module, meta).  Rejects files of another format
    and modules with missing fields."""
    flat = torch.load(path, map_location="cpu")
    meta = flat.pop("__meta__", None)
    if not isinstance(meta, dict) or meta.get("format") != PACKED_FORMAT:
        raise ValueError(f"{path} is not an ADE compressed delta (meta={meta!r})")
    per_module: dict = {}
    for k, v in flat.items():
        prefix, field = k.rsplit(".", 1)
        per_module.setdefault(prefix, {})[field] = v
    for prefix, packed in per_module.items():
        missing = [f for f in PACKED_FIELDS if f not in packed]
        if missing:
            raise ValueError(f"{prefix} misses {missing} in {path}")
    return per_module, meta
