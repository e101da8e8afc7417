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


def group_cost_bits(d_o: int, d_i: int, b_quant: int = 4, b_s: int = 16, b_z: int | None = None,
                    group_size: int = 128) -> int:
    """Storage cost in bits of G ranks of a module, (G b + b_s + b_z)(d_o + d_i)
    (src/allocation.py:168-187)."""
    bz = b_quant if b_z is None else b_z
    return (group_size * b_quant + b_s + bz) * (d_o + d_i)
