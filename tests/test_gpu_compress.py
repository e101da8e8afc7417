"""Producer side on the GPU (`ade_b200_compress_rows`): the fused scale / rotate / quantise kernel against the restated
quantizer of ade_b200.quantization, which tests/test_host_cpu.py pins bit for bit against the reference's outputs."""
from __future__ import annotations

import pytest
import torch

from ade_b200 import _lib, quantization as Q

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _kernel(X, root, rotate, transposed):
    lib = _lib.load()
    rows, r = X.shape
    ng = r // 128
    shape_c, shape_s = ((r, rows), (ng, rows)) if transposed else ((rows, r), (rows, ng))
    codes = torch.full(shape_c, 255, dtype=torch.uint8, device=DEV)
    scale = torch.zeros(shape_s, dtype=torch.bfloat16, device=DEV)
    zero = torch.full(shape_s, -1.0, dtype=torch.bfloat16, device=DEV)
    rc = lib.ade_b200_compress_rows(X.data_ptr(), None if root is None else root.data_ptr(), codes.data_ptr(), scale.data_ptr(),
                                    zero.data_ptr(), rows, r, int(rotate), int(transposed), torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "ade_b200_compress_rows")
    torch.cuda.synchronize()
    return codes, scale, zero


@pytest.mark.parametrize("rows,r", [(1, 128), (33, 256), (1000, 384), (4096, 512), (130, 2048)])
def test_quantise_groups_bit_exact(rows, r):
    """Without a rotation the kernel is the reference's quantizer, bit for bit: row-wise (the U side) and with the
    outputs transposed (the V side, against quantize_colwise of the transposed input).  The input holds the cases
    the reference treats apart: all-zero groups, all-positive and all-negative groups, tiny ranges."""
    g = torch.Generator().manual_seed(rows + r)
    X = torch.randn(rows, r, generator=g) * 0.01
    X[0, :128] = 0.0
    if rows > 2:
        X[1, :128] = X[1, :128].abs() + 0.5
        X[2, :128] = -X[2, :128].abs() - 0.5
        X[2, 128:256 if r >= 256 else 128] = 1e-9
    Xd = X.to(DEV)
    c, s, z = _kernel(Xd, None, False, False)
    rc, rs, rz = Q.quantize_rowwise(X, 4, 128)
    assert torch.equal(c.cpu(), rc) and torch.equal(s.cpu(), rs) and torch.equal(z.cpu(), rz)
    c, s, z = _kernel(Xd, None, False, True)
    cc, cs, cz = Q.quantize_colwise(X.t().contiguous(), 4, 128)
    assert torch.equal(c.cpu(), cc) and torch.equal(s.cpu(), cs) and torch.equal(z.cpu(), cz)


@pytest.mark.parametrize("d_o,d_i,r", [(512, 384, 256), (1024, 1024, 512), (300, 4096, 1024), (256, 256, 384)])
def test_compress_module_on_the_gpu(d_o, d_i, r):
    """Whole compress_module: power-of-two ranks take the in-kernel Walsh-Hadamard transform, rank 384 the dense seeded
    rotation.  Against the CPU chain on the same factors: the transform sums in another order than the dense
    matmul, so a code may move by one step where a value sits on a rounding boundary; scales agree to bf16 rounding and
    the dequantised product agrees closely."""
    g = torch.Generator().manual_seed(d_o + r)
    U = torch.linalg.qr(torch.randn(d_o, min(r, d_o), generator=g))[0]
    V = torch.linalg.qr(torch.randn(d_i, min(r, d_i), generator=g))[0]
    if U.shape[1] < r:
        U = torch.cat([U, torch.randn(d_o, r - U.shape[1], generator=g) * 0.05], 1)
    if V.shape[1] < r:
        V = torch.cat([V, torch.randn(d_i, r - V.shape[1], generator=g) * 0.05], 1)
    S = torch.logspace(0, -2, r)
    cpu = Q.compress_module(U, S, V, 4, 128, torch.Generator().manual_seed(0))
    gpu = Q.compress_module(U.to(DEV), S.to(DEV), V.to(DEV), 4, 128, torch.Generator().manual_seed(0))
    for k in Q.PACKED_FIELDS:
        assert gpu[k].shape == cpu[k].shape and gpu[k].dtype == cpu[k].dtype, k
    for k in ("U_codes", "Vt_codes"):
        d = (gpu[k].int() - cpu[k].int()).abs()
        assert int(d.max()) <= 1 and float((d != 0).float().mean()) < 5e-3, (k, int(d.max()), float((d != 0).float().mean()))
    for k in ("U_scale", "Vt_scale"):
        assert torch.allclose(gpu[k].float(), cpu[k].float(), rtol=1e-2, atol=0)
    for k in ("U_zero", "Vt_zero"):
        assert float((gpu[k].float() - cpu[k].float()).abs().max()) <= 1
    deq = lambda p: ((p["U_codes"].float().reshape(d_o, -1, 128) - p["U_zero"].float().unsqueeze(-1)) * p["U_scale"].float().unsqueeze(-1)
                     ).reshape(d_o, r) @ ((p["Vt_codes"].float().reshape(-1, 128, d_i) - p["Vt_zero"].float().unsqueeze(1))
                                          * p["Vt_scale"].float().unsqueeze(1)).reshape(r, d_i)
    a, b = deq(gpu), deq(cpu)
    assert float((a - b).norm() / b.norm()) < 2e-2
    # folding tuning vectors into the scales (the export of the reference's fold-in stage)
    gamma, rho = torch.rand(d_o, generator=g) + 0.5, torch.rand(d_i, generator=g) + 0.5
    folded = Q.fold_scales(cpu, gamma, rho)
    assert torch.equal(folded["U_scale"], (cpu["U_scale"].float() * gamma.unsqueeze(1)).to(torch.bfloat16))
    assert torch.equal(folded["Vt_scale"], (cpu["Vt_scale"].float() * rho.unsqueeze(0)).to(torch.bfloat16))
    assert folded["U_codes"] is cpu["U_codes"]
