"""CPU oracle of ADE's delta-application path -- TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this module.  It exists so that tests, the smoke
check and the benchmark's CPU leg have an independent statement of what the CUDA kernels
must compute.  Two layers:

* pure-numpy functions (suffix ``_np``) that follow the reference's PyTorch code line by
  line and are only meant for small cases;
* ctypes wrappers over oracle/ade_oracle.c (OpenMP) for full-size modules.

Parity status: the reference has no test suite for this path, so the oracle is pinned
against outputs of the reference's own Python functions (tests/golden/*.npz, produced by
tests/golden/make_golden.py); tests/test_oracle_golden.py checks every one of them.

Conventions: a *packed delta* is a dict of numpy arrays with the six fields that
src/quantization.py:276-285 returns -- ``U_codes`` (M, r) uint8, ``U_scale`` / ``U_zero``
(M, r/G), ``Vt_codes`` (r, N) uint8, ``Vt_scale`` / ``Vt_zero`` (r/G, N) -- where the 16-bit
fields are bfloat16 bit patterns stored as uint16.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

PACKED_FIELDS = ("U_codes", "U_scale", "U_zero", "Vt_codes", "Vt_scale", "Vt_zero")
_HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None


# ----------------------------------------------------------------------------- bfloat16
def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    """bfloat16 bit patterns (uint16) -> float32 (exact)."""
    return (np.ascontiguousarray(bits).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns, round to nearest even (torch's .to(bfloat16))."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return np.where(nan, ((u >> 16) | 0x40).astype(np.uint16), r)


def packed_from_torch(packed: dict) -> dict:
    """Packed dict of torch CPU tensors (as the reference writes it) -> numpy oracle form."""
    import torch

    out = {}
    for k in PACKED_FIELDS:
        t = packed[k].detach().cpu().contiguous()
        if t.dtype == torch.bfloat16:
            out[k] = t.view(torch.uint16).numpy().copy()
        elif t.dtype == torch.uint8:
            out[k] = t.numpy().copy()
        else:
            raise TypeError(f"{k}: unexpected dtype {t.dtype}")
    return out


def _dims(p: dict, G: int):
    M, r = p["U_codes"].shape
    r2, N = p["Vt_codes"].shape
    assert r == r2 and r % G == 0, (r, r2, G)
    return M, N, r, r // G


# ----------------------------------------------------------------- pure numpy (small cases)
def zero_points(p: dict):
    """Integer zero-points mu (M, ng), nu (ng, N): .to(int16) of src/quantization.py:306,308."""
    return (bf16_to_f32(p["U_zero"]).astype(np.int32), bf16_to_f32(p["Vt_zero"]).astype(np.int32))


def group_products_np(p: dict, G: int = 128) -> np.ndarray:
    """INT32 ``prod`` of every group, (ng, M, N): src/quantization.py:303-312."""
    M, N, r, ng = _dims(p, G)
    mu, nu = zero_points(p)
    out = np.empty((ng, M, N), dtype=np.int32)
    for g in range(ng):
        u_i = p["U_codes"][:, g * G:(g + 1) * G].astype(np.int32) - mu[:, g:g + 1]
        v_i = p["Vt_codes"][g * G:(g + 1) * G, :].astype(np.int32) - nu[g:g + 1, :]
        out[g] = u_i @ v_i
    return out


def reconstruct_delta_np(p: dict, G: int = 128) -> np.ndarray:
    """float32 delta of eq. (7), bit for bit as src/quantization.py:288-317 computes it."""
    M, N, r, ng = _dims(p, G)
    prod = group_products_np(p, G)
    us, vs = bf16_to_f32(p["U_scale"]), bf16_to_f32(p["Vt_scale"])
    acc = np.zeros((M, N), dtype=np.float32)
    for g in range(ng):
        s = us[:, g:g + 1] * vs[g:g + 1, :]                 # float32, exact
        acc = acc + prod[g].astype(np.float32) * s          # one multiply, one add
    return acc


def merged_weight_np(p: dict, base_bits: np.ndarray, G: int = 128) -> np.ndarray:
    """bf16(W_b + delta): the merged weight of src/serving.py:84-92, kept in bfloat16."""
    return f32_to_bf16(bf16_to_f32(base_bits) + reconstruct_delta_np(p, G))


def dequantize_np(p: dict, G: int = 128):
    """Dequantized factors (eq. 6), float32: src/quantization.py:202-241."""
    M, N, r, ng = _dims(p, G)
    mu, nu = zero_points(p)
    Uh = (p["U_codes"].reshape(M, ng, G).astype(np.float32) - mu[:, :, None].astype(np.float32)) \
        * bf16_to_f32(p["U_scale"])[:, :, None]
    Vh = (p["Vt_codes"].reshape(ng, G, N).astype(np.float32) - nu[:, None, :].astype(np.float32)) \
        * bf16_to_f32(p["Vt_scale"])[:, None, :]
    return Uh.reshape(M, r), Vh.reshape(r, N)


def factored_apply_np(x_bits, base_bits, p: dict, G: int = 128) -> np.ndarray:
    """float64 y = x W_b^T + (x V^)(U^)^T: src/adaptation.py:201-242 with gamma = rho = 1."""
    Uh, Vh = dequantize_np(p, G)
    x = bf16_to_f32(x_bits).astype(np.float64)
    y = (x @ Vh.astype(np.float64).T) @ Uh.astype(np.float64).T
    if base_bits is not None:
        y = y + x @ bf16_to_f32(base_bits).astype(np.float64).T
    return y


def recon_apply_np(x_bits, base_bits, p: dict, G: int = 128) -> np.ndarray:
    """float64 y = x (bf16(W_b + delta))^T: src/serving.py:109-111 (merged weight, then F.linear)."""
    W = bf16_to_f32(merged_weight_np(p, base_bits, G)).astype(np.float64)
    return bf16_to_f32(x_bits).astype(np.float64) @ W.T


def pack_nibbles_ref_np(codes: np.ndarray) -> np.ndarray:
    """Reference stored form of the codes (src/kernels.py:145-161): 8 codes per int32 word."""
    K = codes.shape[-1]
    assert K % 8 == 0
    c = codes.astype(np.uint32).reshape(*codes.shape[:-1], K // 8, 8)
    w = np.zeros(c.shape[:-1], dtype=np.uint32)
    for j in range(8):
        w |= (c[..., j] & 15) << np.uint32(4 * j)
    return w.view(np.int32)


def ref_tables_np(p: dict, G: int = 128):
    """FP32 tables R (M, ng, 4) and C (N, ng, 4) of the reference stored form (src/kernels.py:180-187)."""
    M, N, r, ng = _dims(p, G)
    us, vs = bf16_to_f32(p["U_scale"]), bf16_to_f32(p["Vt_scale"])
    mu = np.round(bf16_to_f32(p["U_zero"]))
    nu = np.round(bf16_to_f32(p["Vt_zero"]))
    rowsum = p["U_codes"].reshape(M, ng, G).astype(np.float32).sum(-1)
    colsum = p["Vt_codes"].reshape(ng, G, N).astype(np.float32).sum(1)
    R = np.stack([us, us * mu, us * rowsum, us * mu * np.float32(G)], -1).astype(np.float32)
    C = np.stack([vs, vs * colsum, vs * nu, np.zeros_like(vs)], -1).transpose(1, 0, 2).astype(np.float32)
    return np.ascontiguousarray(R), np.ascontiguousarray(C)


# ------------------------------------------------------------------------- C oracle (ctypes)
def lib():
    """Load oracle/libade_oracle.so, building it with gcc on first use."""
    global _lib
    if _lib is None:
        import importlib.util

        spec = importlib.util.spec_from_file_location("_ade_oracle_build", os.path.join(_HERE, "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _lib = ctypes.CDLL(mod.build())
    return _lib


def _p(a, ct=ctypes.c_void_p):
    return None if a is None else a.ctypes.data_as(ct)


def _fields(p: dict):
    arrs = [np.ascontiguousarray(p[k]) for k in PACKED_FIELDS]
    assert arrs[0].dtype == np.uint8 and arrs[3].dtype == np.uint8
    assert all(a.dtype == np.uint16 for a in (arrs[1], arrs[2], arrs[4], arrs[5]))
    return arrs


def threads() -> int:
    return int(lib().ade_oracle_threads())


def use_all_cores() -> int:
    """Let the C oracle and numpy's BLAS use every host core, whatever OMP_NUM_THREADS the launcher
    exported; returns the thread count of the C oracle."""
    n = os.cpu_count() or 1
    lib().ade_oracle_set_threads(n)
    try:
        from threadpoolctl import threadpool_limits

        threadpool_limits(limits=n)
    except Exception:
        pass
    return threads()


def group_product(p: dict, g: int, G: int = 128, rows=None) -> np.ndarray:
    """INT32 ``prod`` of group g for rows [m0, m1) (default all): src/quantization.py:309-312."""
    M, N, r, ng = _dims(p, G)
    m0, m1 = rows if rows is not None else (0, M)
    Uc, Us, Uz, Vc, Vs, Vz = _fields(p)
    out = np.empty((m1 - m0, N), dtype=np.int32)
    rc = lib().ade_oracle_group_product(_p(Uc), _p(Uz), _p(Vc), _p(Vz), M, N, r, G, g, m0, m1, _p(out))
    if rc:
        raise RuntimeError(f"ade_oracle_group_product rc={rc}")
    return out


def reconstruct(p: dict, G: int = 128, rows=None, base_bits=None):
    """(delta float32, merged bf16 bits or None) for rows [m0, m1): src/quantization.py:288-317."""
    M, N, r, ng = _dims(p, G)
    m0, m1 = rows if rows is not None else (0, M)
    Uc, Us, Uz, Vc, Vs, Vz = _fields(p)
    delta = np.empty((m1 - m0, N), dtype=np.float32)
    merged = None
    base = None
    if base_bits is not None:
        base = np.ascontiguousarray(base_bits, dtype=np.uint16)
        assert base.shape == (M, N)
        merged = np.empty((m1 - m0, N), dtype=np.uint16)
    rc = lib().ade_oracle_reconstruct(_p(Uc), _p(Us), _p(Uz), _p(Vc), _p(Vs), _p(Vz), M, N, r, G, m0, m1,
                                      _p(delta), _p(base), _p(merged))
    if rc:
        raise RuntimeError(f"ade_oracle_reconstruct rc={rc}")
    return delta, merged


def dequantize(p: dict, G: int = 128):
    M, N, r, ng = _dims(p, G)
    Uc, Us, Uz, Vc, Vs, Vz = _fields(p)
    Uh = np.empty((M, r), dtype=np.float32)
    Vh = np.empty((r, N), dtype=np.float32)
    rc = lib().ade_oracle_dequantize(_p(Uc), _p(Us), _p(Uz), _p(Vc), _p(Vs), _p(Vz), M, N, r, G, _p(Uh), _p(Vh))
    if rc:
        raise RuntimeError(f"ade_oracle_dequantize rc={rc}")
    return Uh, Vh


def factored_apply(x_bits, base_bits, p: dict, G: int = 128) -> np.ndarray:
    """float64 y (T, M) = x W_b^T + U^(V^^T x); base_bits None -> delta term only."""
    M, N, r, ng = _dims(p, G)
    x = np.ascontiguousarray(x_bits, dtype=np.uint16)
    T = x.shape[0]
    assert x.shape == (T, N)
    base = None if base_bits is None else np.ascontiguousarray(base_bits, dtype=np.uint16)
    Uc, Us, Uz, Vc, Vs, Vz = _fields(p)
    y = np.empty((T, M), dtype=np.float64)
    rc = lib().ade_oracle_factored(_p(x), _p(base), _p(Uc), _p(Us), _p(Uz), _p(Vc), _p(Vs), _p(Vz),
                                   T, M, N, r, G, _p(y))
    if rc:
        raise RuntimeError(f"ade_oracle_factored rc={rc}")
    return y


def pack_nibbles_ref(codes: np.ndarray) -> np.ndarray:
    c = np.ascontiguousarray(codes, dtype=np.uint8)
    rows, K = c.reshape(-1, c.shape[-1]).shape
    out = np.empty((rows, K // 8), dtype=np.uint32)
    rc = lib().ade_oracle_pack_nibbles_ref(_p(c), rows, K, _p(out))
    if rc:
        raise RuntimeError(f"ade_oracle_pack_nibbles_ref rc={rc}")
    return out.view(np.int32).reshape(*c.shape[:-1], K // 8)


# ------------------------------------------------------------------------ parity metrics
def parity(y, ref):
    """(max|y - ref| / max|ref|, cosine) on the flattened arrays, in float64."""
    a = np.asarray(y, dtype=np.float64).ravel()
    b = np.asarray(ref, dtype=np.float64).ravel()
    err = float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))
    cos = float(a @ b / max(np.linalg.norm(a) * np.linalg.norm(b), 1e-30))
    return err, cos
