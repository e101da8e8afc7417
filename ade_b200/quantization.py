"""Producer of the packed-delta format (4-bit codes, bfloat16 scales, 4-bit zero-points).

Restates what the reference's ``src/quantization.py`` writes so that synthetic deltas of the
benchmark shapes can be produced where the reference is not installed (and on the GPU: every
function runs on the device of its inputs).  The serving kernels only *read* this format;
tests pin these functions against tensors produced by the reference itself.

    compress_module(U, S, V)  ->  Q_r(U S^1/2 H),  Q_c(H^T S^1/2 V^T)        (eqs. 5 and 8)
"""
from __future__ import annotations

import math

import torch

PACKED_FIELDS = ("U_codes", "U_scale", "U_zero", "Vt_codes", "Vt_scale", "Vt_zero")


def hadamard(k: int, dtype=torch.float32, device=None) -> torch.Tensor:
    """Orthonormal Sylvester Hadamard matrix of order k = 2^p (src/quantization.py:56-70)."""
    if k < 1 or k & (k - 1):
        raise ValueError(f"hadamard: order {k} is not a power of two")
    H = torch.ones(1, 1, dtype=dtype, device=device)
    while H.shape[0] < k:
        H = torch.cat([torch.cat([H, H], 1), torch.cat([H, -H], 1)], 0)
    return H / math.sqrt(k)


def rotation_matrix(rank: int, generator=None) -> torch.Tensor:
    """Shared rotation H: Hadamard for a power-of-two rank, otherwise Q of the QR decomposition of a
    seeded Gaussian with the signs of diag(R) folded in (src/quantization.py:73-106).  CPU float32."""
    if rank & (rank - 1) == 0:
        return hadamard(rank)
    A = torch.randn(rank, rank, dtype=torch.float32, generator=generator)
    Q, R = torch.linalg.qr(A)
    return Q * torch.sign(torch.diagonal(R)).unsqueeze(0)


def quantize_groups(Xg: torch.Tensor, dim: int, bits: int = 4):
    """Asymmetric uniform quantization (eq. 2) of every slice of `Xg` along `dim` (the in-group axis).

    Follows src/quantization.py:149-165 / 183-199: scale = (max - min) / (2^b - 1) floored at
    1e-5 / (2^b - 1); zero = round(-min / scale); all-zero groups quantize as [-1, 1]; one-signed
    groups are widened to contain 0 so that the zero-point stays in [0, 2^b - 1]
    (src/quantization.py:109-131).  Returns (codes uint8, scale float32, zero float32) with `dim`
    kept (size 1) in scale and zero.
    """
    maxq = float(2 ** bits - 1)
    lo = Xg.amin(dim=dim, keepdim=True)
    hi = Xg.amax(dim=dim, keepdim=True)
    flat = (lo == 0) & (hi == 0)
    lo = torch.where(flat, torch.full_like(lo, -1.0), lo)
    hi = torch.where(flat, torch.full_like(hi, 1.0), hi)
    scale = (hi - lo).clamp(min=1e-5) / maxq
    zero = torch.round(-lo / scale)
    below, above = zero < 0, zero > maxq
    if bool((below | above).any()):
        widened = torch.where(below, hi.clamp(min=1e-5) / maxq, (-lo).clamp(min=1e-5) / maxq)
        scale = torch.where(below | above, widened, scale)
        zero = torch.where(below, torch.zeros_like(zero), torch.where(above, torch.full_like(zero, maxq), zero))
    codes = torch.clamp(torch.round(Xg / scale) + zero, 0, maxq).to(torch.uint8)
    return codes, scale, zero


def quantize_rowwise(X: torch.Tensor, bits: int = 4, group_size: int = 128):
    """Q_r: groups of G consecutive entries of each row of X (d_o, r).  Returns codes (d_o, r) uint8,
    scale and zero (d_o, r/G) bfloat16 (src/quantization.py:134-165)."""
    d_o, rank = X.shape
    if rank % group_size:
        raise ValueError(f"rank={rank} is not a multiple of group_size={group_size}")
    c, s, z = quantize_groups(X.reshape(d_o, rank // group_size, group_size), 2, bits)
    return c.reshape(d_o, rank), s.squeeze(2).to(torch.bfloat16), z.squeeze(2).to(torch.bfloat16)


def quantize_colwise(X: torch.Tensor, bits: int = 4, group_size: int = 128):
    """Q_c: groups of G consecutive entries of each column of X (r, d_i).  Returns codes (r, d_i)
    uint8, scale and zero (r/G, d_i) bfloat16 (src/quantization.py:168-199)."""
    rank, d_i = X.shape
    if rank % group_size:
        raise ValueError(f"rank={rank} is not a multiple of group_size={group_size}")
    c, s, z = quantize_groups(X.reshape(rank // group_size, group_size, d_i), 1, bits)
    return c.reshape(rank, d_i), s.squeeze(1).to(torch.bfloat16), z.squeeze(1).to(torch.bfloat16)


def compress_module(U, S, V, bits: int = 4, group_size: int = 128, generator=None, keep_device: bool = False):
    """Inference-aligned quantization of one module's truncated SVD (src/quantization.py:244-285).

    U (d_o, r), S (r,), V (d_i, r) on any device.  Returns the packed dict (CPU tensors unless
    `keep_device`).  `generator` (CPU) is consumed only for non-power-of-two ranks.
    """
    if U.is_cuda and bits == 4 and group_size == 128 and S.shape[0] % 128 == 0 and S.shape[0] <= 2048:
        out = compress_module_cuda(U, S, V, generator)
        return out if keep_device else {k: v.cpu() for k, v in out.items()}
    U = U.float()
    S = S.float().clamp(min=1e-8)
    Vt = V.transpose(-1, -2).contiguous().float()
    rank = S.shape[0]
    if rank % group_size:
        raise ValueError(f"compress_module: rank={rank} is not a multiple of group_size={group_size}")
    root = torch.sqrt(S)
    H = rotation_matrix(rank, generator=generator).to(U.device)
    Uc, Us, Uz = quantize_rowwise((U * root.unsqueeze(0)) @ H, bits, group_size)
    Vc, Vs, Vz = quantize_colwise(H.T @ (root.unsqueeze(1) * Vt), bits, group_size)
    out = {"U_codes": Uc, "U_scale": Us, "U_zero": Uz, "Vt_codes": Vc, "Vt_scale": Vs, "Vt_zero": Vz}
    return out if keep_device else {k: v.cpu() for k, v in out.items()}


def compress_module_cuda(U, S, V, generator=None) -> dict:
    """compress_module on the GPU through ``ade_b200_compress_rows``: per factor one kernel that scales by sqrt(S),
    rotates (fast Walsh-Hadamard transform for a power-of-two rank; for other ranks the seeded random orthogonal H is
    applied here with one dense matmul, as the reference does) and quantises the groups in shared memory.  4 bits,
    groups of 128.  Returns the packed dict on the device of U."""
    from . import _lib

    lib = _lib.load()
    dev = U.device
    rank = int(S.shape[0])
    root = torch.sqrt(S.to(dev, torch.float32).clamp(min=1e-8)).contiguous()
    Uf = U.to(torch.float32).contiguous()
    Vf = V.to(dev, torch.float32).contiguous()                         # (d_i, r): the V side is quantised row by row too
    pow2 = rank & (rank - 1) == 0
    if not pow2:
        H = rotation_matrix(rank, generator=generator).to(dev)
        Uf = (Uf * root.unsqueeze(0)) @ H
        Vf = (Vf * root.unsqueeze(0)) @ H                              # ((V sqrt(S)) H)^T = H^T (sqrt(S) V^T)
    d_o, d_i, ng = Uf.shape[0], Vf.shape[0], rank // 128
    out = {"U_codes": torch.empty(d_o, rank, dtype=torch.uint8, device=dev),
           "U_scale": torch.empty(d_o, ng, dtype=torch.bfloat16, device=dev),
           "U_zero": torch.empty(d_o, ng, dtype=torch.bfloat16, device=dev),
           "Vt_codes": torch.empty(rank, d_i, dtype=torch.uint8, device=dev),
           "Vt_scale": torch.empty(ng, d_i, dtype=torch.bfloat16, device=dev),
           "Vt_zero": torch.empty(ng, d_i, dtype=torch.bfloat16, device=dev)}
    with torch.cuda.device(dev):
        st = torch.cuda.current_stream().cuda_stream
        sp = root.data_ptr() if pow2 else None
        _lib.check(lib.ade_b200_compress_rows(Uf.data_ptr(), sp, out["U_codes"].data_ptr(), out["U_scale"].data_ptr(),
                                              out["U_zero"].data_ptr(), d_o, rank, int(pow2), 0, st), "ade_b200_compress_rows(U)")
        _lib.check(lib.ade_b200_compress_rows(Vf.data_ptr(), sp, out["Vt_codes"].data_ptr(), out["Vt_scale"].data_ptr(),
                                              out["Vt_zero"].data_ptr(), d_i, rank, int(pow2), 1, st), "ade_b200_compress_rows(V)")
    return out


def fold_scales(packed: dict, gamma: torch.Tensor, rho: torch.Tensor) -> dict:
    """Fold the tuning vectors of the reference's fold-in stage into the per-group scales, u <- gamma u (per output
    row), v <- rho v (per input column): what ``FoldInLinear.export_folded`` writes (src/adaptation.py:244-263).  The
    codes and zero-points are shared with `packed`; the scales are new bfloat16 tensors."""
    us, vs = packed["U_scale"], packed["Vt_scale"]
    out = dict(packed)
    out["U_scale"] = (us.float() * gamma.to(us.device).float().unsqueeze(1)).to(us.dtype)
    out["Vt_scale"] = (vs.float() * rho.to(vs.device).float().unsqueeze(0)).to(vs.dtype)
    return out


def group_cost_bits(d_o: int, d_i: int, b_quant: int = 4, b_s: int = 16, b_z: int | None = None,
                    group_size: int = 128) -> int:
    """Storage cost in bits of G ranks of a module, (G b + b_s + b_z)(d_o + d_i)
    (src/allocation.py:168-187)."""
    bz = b_quant if b_z is None else b_z
    return (group_size * b_quant + b_s + bz) * (d_o + d_i)
