"""GPU parity tests: the CUDA kernels, called through the C ABI, against the CPU oracle.

Integer work (packing, per-group INT32 accumulators) must match bit for bit.  The merged weight of
the reconstruction kernel is also compared bit for bit: it performs the reference's float32
operations in the reference's order.  The factored path is compared within the stated tolerance
(max normalised error <= 1e-2, cosine >= 0.9999).
"""
from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from ade_b200 import _lib, kernels, synth
from ade_b200.serving import ADEKernelLinear
from conftest import golden_cases, load_case
from oracle import oracle as O

pytestmark = pytest.mark.gpu
TOL_ERR, TOL_COS = 1e-2, 0.9999
DEV = "cuda"


def _bf16(bits):
    return torch.from_numpy(np.ascontiguousarray(bits)).view(torch.bfloat16)


def _bits(t):
    return t.detach().cpu().contiguous().view(torch.uint16).numpy()


def _torch_packed(p):
    out = {}
    for k, v in p.items():
        t = torch.from_numpy(np.ascontiguousarray(v))
        out[k] = t.view(torch.bfloat16) if v.dtype == np.uint16 else t
    return out


def _random_case(M, N, r, T, seed):
    tp = synth.random_packed(M, N, r, seed)
    return {
        "M": M, "N": N, "r": r, "T": T, "G": 128,
        "packed": O.packed_from_torch(tp), "tpacked": tp,
        "W_b": _bits(synth.base_weight(M, N, seed + 1)), "x": _bits(synth.activations(T, N, seed + 2)),
    }


def _run_recon(case, dbg=True, expanded=False):
    tp = case.get("tpacked") or _torch_packed(case["packed"])
    p4 = kernels.pack_int4(tp, device=DEV)
    x8 = kernels.expand_codes(p4) if expanded else None
    base = _bf16(case["W_b"]).to(DEV)
    ng = case["r"] // 128
    acc = torch.full((ng, case["M"], case["N"]), -7, dtype=torch.int32, device=DEV) if dbg else None
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = kernels.recon_int4(p4, base, dbg_acc=acc, status=status, expanded=x8)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, _lib.DEVICE_STATUS.get(int(status.item()))
    return out, acc


def test_device_status():
    assert kernels.recon_kernel_status(DEV)[0] and kernels.decode_kernel_status(DEV)[0]


def test_pack_kernels_match_host_packing():
    lib = _lib.load()
    g = torch.Generator().manual_seed(1)
    codes = torch.randint(0, 16, (384, 256), generator=g, dtype=torch.uint8)
    dc = codes.to(DEV)
    out = torch.empty(384, 128, dtype=torch.uint8, device=DEV)
    _lib.check(lib.ade_b200_pack_codes(dc.data_ptr(), out.data_ptr(), 384, 256, 0, None), "pack_codes")
    assert torch.equal(out.cpu(), kernels.pack_nibbles(codes))
    outT = torch.empty(256, 192, dtype=torch.uint8, device=DEV)       # [K=384][rows=256] read transposed
    _lib.check(lib.ade_b200_pack_codes(dc.data_ptr(), outT.data_ptr(), 256, 384, 1, None), "pack_codes T")
    assert torch.equal(outT.cpu(), kernels.pack_nibbles(codes.t().contiguous()))
    z = torch.randint(0, 16, (1000,), generator=g).to(torch.bfloat16).to(DEV)
    oz = torch.empty(1000, dtype=torch.uint8, device=DEV)
    _lib.check(lib.ade_b200_pack_zeros(z.data_ptr(), oz.data_ptr(), 1000, None), "pack_zeros")
    assert torch.equal(oz.cpu().float(), z.cpu().float())


@pytest.mark.parametrize("path", golden_cases(), ids=lambda p: p.split("case_")[1][:-4])
def test_recon_golden_bit_exact(path):
    case = load_case(path)
    out, acc = _run_recon(case)
    assert np.array_equal(acc.cpu().numpy(), case["ref_prod"]), "per-group INT32 accumulators differ"
    merged = O.f32_to_bf16(O.bf16_to_f32(case["W_b"]) + case["ref_delta"])
    assert np.array_equal(_bits(out), merged), "merged weight differs from the reference arithmetic"
    out2, _ = _run_recon(case, dbg=False)                  # the production instantiation
    assert torch.equal(out, out2)
    out3, acc3 = _run_recon(case, expanded=True)           # the same from expanded int8 operands
    assert torch.equal(out, out3) and torch.equal(acc, acc3)


@pytest.mark.parametrize("M,N,r", [(128, 128, 128), (256, 384, 256), (192, 128, 384), (100, 256, 512),
                                   (384, 128, 1024), (1024, 1152, 640), (2048, 2304, 768), (2100, 1920, 384),
                                   (256, 256, 1152), (200, 384, 2048), (1, 128, 128), (129, 128, 256)])
def test_recon_shapes_bit_exact(M, N, r):
    """Ranks up to 512 and 640-1024 take the two configurations of the strip-resident kernel (several tiles and
    strips per CTA in the larger cases), ranks above 1024 the general kernel."""
    case = _random_case(M, N, r, 1, seed=31 * M + N + r)
    out, acc = _run_recon(case)
    for g in range(r // 128):
        assert np.array_equal(acc[g].cpu().numpy(), O.group_product(case["packed"], g)), f"group {g}"
    _, merged = O.reconstruct(case["packed"], base_bits=case["W_b"])
    assert np.array_equal(_bits(out), merged)
    out2, _ = _run_recon(case, dbg=False)
    assert torch.equal(out, out2)
    # expanded int8 operands (TMA-fed kernel without an unpack role; ranks above 1024 ignore them): identical bits
    out3, acc3 = _run_recon(case, expanded=True)
    assert torch.equal(out, out3) and torch.equal(acc, acc3)
    out4, _ = _run_recon(case, dbg=False, expanded=True)
    assert torch.equal(out, out4)


def test_expand_codes_layout():
    """u8 / v8 hold code minus zero-point; inside every 8 consecutive ranks the order is that of the stored nibbles
    (low nibbles of the word's four bytes, then the high ones): position j holds code (0, 4, 1, 5, 2, 6, 3, 7)[j]."""
    M, N, r = 200, 256, 384
    tp = synth.random_packed(M, N, r, 5)
    p4 = kernels.pack_int4(tp, device=DEV)
    u8, v8 = kernels.expand_codes(p4)
    torch.cuda.synchronize()
    assert u8.dtype == torch.int8 and tuple(u8.shape) == (M, r) and tuple(v8.shape) == (N, r)
    perm = torch.tensor([0, 4, 1, 5, 2, 6, 3, 7])
    uc = tp["U_codes"].to(torch.int16) - tp["U_zero"].to(torch.float32).to(torch.int16).repeat_interleave(128, dim=1)
    vc = (tp["Vt_codes"].to(torch.int16) - tp["Vt_zero"].to(torch.float32).to(torch.int16).repeat_interleave(128, dim=0)).t()
    for got, want in ((u8, uc), (v8, vc)):
        want = want.reshape(want.shape[0], r // 8, 8)[..., perm].reshape(want.shape[0], r)
        assert torch.equal(got.cpu().to(torch.int16), want)


def _check_factored(case, fused):
    tp = case.get("tpacked") or _torch_packed(case["packed"])
    p4 = kernels.pack_int4(tp, device=DEV)
    x = _bf16(case["x"]).to(DEV)
    W = _bf16(case["W_b"]).to(DEV)
    ref = O.factored_apply(case["x"], case["W_b"], case["packed"])
    if fused:
        y = kernels.factored_forward(x, p4, weight=W)
    else:
        # the reference's calling convention: y_dense = x W_b^T computed by the caller, in 16-bit
        y_dense = torch.nn.functional.linear(x, W)
        y = kernels.decode_forward_packed(x, y_dense, p4)
    torch.cuda.synchronize()
    kernels.check_factored_status(DEV)                     # no grid-wide wait expired in any launch so far
    err, cos = O.parity(y.float().cpu().numpy(), ref)
    assert err <= TOL_ERR and cos >= TOL_COS, (err, cos)
    return y


@pytest.mark.parametrize("path", golden_cases(), ids=lambda p: p.split("case_")[1][:-4])
@pytest.mark.parametrize("fused", [True, False])
def test_factored_golden(path, fused):
    case = load_case(path)
    y = _check_factored(case, fused)
    if fused:   # also against what the reference's own PyTorch factored module produced
        err, cos = O.parity(y.float().cpu().numpy(), case["ref_y_factored_fp32"])
        assert err <= TOL_ERR and cos >= TOL_COS, (err, cos)


@pytest.mark.parametrize("T", [1, 2, 7, 8, 9, 16, 17, 31, 33, 64, 65, 100, 128])
def test_factored_token_counts(T):
    case = _random_case(256, 384, 256, T, seed=500 + T)
    _check_factored(case, True)
    _check_factored(case, False)


@pytest.mark.parametrize("M,N,r", [(32, 128, 128), (160, 256, 384), (512, 1152, 1024), (1024, 2048, 1152), (1, 128, 128),
                                   (7, 256, 2048), (333, 384, 256)])
def test_factored_shapes(M, N, r):
    """Ragged row counts (fewer rows than CTAs, a single row), the smallest d_i and the largest rank."""
    _check_factored(_random_case(M, N, r, 5, seed=M + N + r), True)
    _check_factored(_random_case(M, N, r, 19, seed=M + N + r + 1), True)


def test_delta_term_alone_is_tight():
    """With a zero base the output is the delta term only: the 16-bit roundings of the two factors
    are the whole error budget, so the comparison is much tighter than the stated tolerance."""
    case = _random_case(256, 256, 256, 16, seed=77)
    tp = case["tpacked"]
    p4 = kernels.pack_int4(tp, device=DEV)
    x = _bf16(case["x"]).to(DEV)
    y = kernels.decode_forward_packed(x, torch.zeros(16, 256, dtype=torch.bfloat16, device=DEV), p4)
    ref = O.factored_apply(case["x"], None, case["packed"])
    err, cos = O.parity(y.float().cpu().numpy(), ref)
    assert err <= 8e-3 and cos >= 0.99995, (err, cos)


def test_runs_are_deterministic():
    case = _random_case(256, 256, 512, 24, seed=9)
    p4 = kernels.pack_int4(case["tpacked"], device=DEV)
    x, W = _bf16(case["x"]).to(DEV), _bf16(case["W_b"]).to(DEV)
    a = kernels.factored_forward(x, p4, weight=W)
    b = kernels.factored_forward(x, p4, weight=W)
    c = kernels.recon_int4(p4, W)
    d = kernels.recon_int4(p4, W)
    assert torch.equal(a, b) and torch.equal(c, d)


def test_entry_points_reject_bad_arguments():
    case = _random_case(128, 128, 128, 4, seed=3)
    p4 = kernels.pack_int4(case["tpacked"], device=DEV)
    x, W = _bf16(case["x"]).to(DEV), _bf16(case["W_b"]).to(DEV)
    with pytest.raises(ValueError):
        kernels.factored_forward(x.float(), p4, weight=W)
    with pytest.raises(ValueError):
        kernels.factored_forward(x, p4)
    with pytest.raises(ValueError):
        kernels.recon_int4(p4, W.float())
    big = torch.zeros(129, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(_lib.AdeKernelError):
        kernels.factored_forward(big, p4, weight=W)
    lib = _lib.load()
    d = kernels._cdelta(p4)
    assert lib.ade_b200_recon(ctypes.byref(d), W.data_ptr(), W.data_ptr(), None, None, None) == -1   # aliasing
    torch.cuda.synchronize()


def test_module_dispatch_matches_oracle():
    """ADEKernelLinear: factored for T <= decode_max_tokens, reconstructed above (src/serving.py:94-112)."""
    W_b, packed = synth.synthetic_module(256, 256, 256, config=8, module=0)
    p = O.packed_from_torch(packed)
    lin = ADEKernelLinear(W_b, packed).to(DEV)
    for shape in [(1, 1, 256), (2, 5, 256), (3, 50, 256)]:          # T = 1, 10, 150
        x = synth.activations(shape[0] * shape[1], 256, 99).reshape(shape).to(DEV)
        y = lin(x)
        assert y.shape == (*shape[:-1], 256) and y.dtype == torch.bfloat16
        xb = _bits(x.reshape(-1, 256))
        T = xb.shape[0]
        ref = O.factored_apply(xb, _bits(W_b), p) if T <= 128 else O.recon_apply_np(xb, _bits(W_b), p)
        err, cos = O.parity(y.float().cpu().numpy().reshape(T, 256), ref)
        assert err <= TOL_ERR and cos >= TOL_COS, (shape, err, cos)
    assert lin(torch.zeros(0, 256, device=DEV)).shape == (0, 256)
