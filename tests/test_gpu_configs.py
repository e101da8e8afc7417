"""GPU parity at the benchmark configurations' full sizes (configs 0 and 1)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from ade_b200 import kernels, synth
from ade_b200.serving import ADEKernelLinear
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _bits(t):
    return t.detach().cpu().contiguous().view(torch.uint16).numpy()


def _torch_reconstruct(packed, W_b, dev):
    """The reference's fallback arithmetic (src/quantization.py:303-315, src/serving.py:92) restated
    with torch ops on the GPU: an independent second check at sizes the CPU oracle only samples."""
    Uc, Vc = packed["U_codes"].to(dev), packed["Vt_codes"].to(dev)
    ng = Uc.shape[1] // 128
    acc = torch.zeros(Uc.shape[0], Vc.shape[1], device=dev, dtype=torch.float32)
    prods = []
    for g in range(ng):
        cs = slice(g * 128, (g + 1) * 128)
        u_i = (Uc[:, cs].to(torch.int16) - packed["U_zero"][:, g].to(dev).to(torch.int16).unsqueeze(1)).to(torch.int8)
        v_i = (Vc[cs, :].to(torch.int16) - packed["Vt_zero"][g, :].to(dev).to(torch.int16).unsqueeze(0)).to(torch.int8)
        prod = torch._int_mm(u_i.contiguous(), v_i.contiguous())
        s = packed["U_scale"][:, g].to(dev).float().unsqueeze(1) * packed["Vt_scale"][g, :].to(dev).float().unsqueeze(0)
        t = prod.to(torch.float32) * s
        acc += t
        prods.append(prod)
    return (W_b.to(dev).float() + acc).to(torch.bfloat16), prods


def test_config0_factored_q_proj():
    """Config 0: 4096 x 4096 q_proj delta, r = 256 (Hadamard rotation), T = 16, factored path."""
    W_b, packed = synth.synthetic_module(4096, 4096, 256, config=0, module=0, device=DEV)
    x = synth.activations(16, 4096, synth.seed_for(0, 0, 2))
    lin = ADEKernelLinear(W_b, packed).to(DEV)
    y = lin(x.to(DEV))
    p = O.packed_from_torch(packed)
    ref = O.factored_apply(_bits(x), _bits(W_b), p)
    err, cos = O.parity(y.float().cpu().numpy(), ref)
    assert err <= 1e-2 and cos >= 0.9999, (err, cos)
    # the delta must actually be in the output: without it the error is far above the tolerance
    err0, _ = O.parity(torch.nn.functional.linear(x.to(DEV), W_b.to(DEV)).float().cpu().numpy(), ref)
    assert err0 > 2 * err


@pytest.mark.parametrize("M,N,r,T", [(11008, 4096, 512, 1), (11008, 4096, 512, 2), (11008, 4096, 512, 8), (4096, 11008, 512, 8),
                                     (4096, 11008, 256, 16), (11008, 4096, 1024, 3)])
def test_factored_mlp_modules_long_streams(M, N, r, T):
    """Decode sizes on the MLP shapes of configs 2-4: every CTA streams more than 400 KB of W_b, which for
    2 <= T <= 16 selects the shared-memory FIFO variant of the factored kernel (d_i = 11008 also needs several
    staging waves); T = 1 stays on the register-prefetch variant."""
    tp = synth.random_packed(M, N, r, 31 * T + r)
    W_b = synth.base_weight(M, N, 7)
    x = synth.activations(T, N, 8)
    p4 = kernels.pack_int4(tp, device=DEV)
    y = kernels.factored_forward(x.to(DEV), p4, weight=W_b.to(DEV))
    y2 = kernels.factored_forward(x.to(DEV), p4, weight=W_b.to(DEV))
    torch.cuda.synchronize()
    assert kernels.factored_status(DEV, T, r) == 0
    assert torch.equal(y, y2)                      # deterministic, and the sync words re-armed themselves
    ref = O.factored_apply(_bits(x), _bits(W_b), O.packed_from_torch(tp))
    err, cos = O.parity(y.float().cpu().numpy(), ref)
    assert err <= 1e-2 and cos >= 0.9999, (err, cos)


@pytest.mark.parametrize("M,N,r,T", [(4096, 4096, 256, 64), (4096, 4096, 128, 17), (11008, 4096, 512, 128), (4096, 11008, 512, 33),
                                     (1000, 2048, 1024, 40)])
def test_delta_only_launch_above_16_tokens(M, N, r, T):
    """The reference's split (cuBLAS base term + delta kernel) at 17-128 tokens on full-size modules: the launch that
    slices every phase-A unit over d_i (2048 / r slices, float32 partial sums, second grid-wide step) and stages h
    and the base term in shared memory.  Also through the module, which takes this route above 16 tokens."""
    tp = synth.random_packed(M, N, r, 17 * T + r)
    W_b = synth.base_weight(M, N, 9)
    x = synth.activations(T, N, 10)
    p4 = kernels.pack_int4(tp, device=DEV)
    xd, Wd = x.to(DEV), W_b.to(DEV)
    y_dense = torch.nn.functional.linear(xd, Wd)
    y = kernels.decode_forward_packed(xd, y_dense, p4)
    y2 = kernels.decode_forward_packed(xd, y_dense, p4)
    torch.cuda.synchronize()
    assert kernels.factored_status(DEV, T, r) == 0
    assert torch.equal(y, y2)
    ref = O.factored_apply(_bits(x), _bits(W_b), O.packed_from_torch(tp))
    err, cos = O.parity(y.float().cpu().numpy(), ref)
    assert err <= 1e-2 and cos >= 0.9999, (err, cos)
    lin = ADEKernelLinear(W_b, tp).to(DEV)
    assert torch.equal(lin(xd), y)


@pytest.mark.parametrize("name,M,N", [("gate", 11008, 4096), ("down", 4096, 11008)])
def test_config1_reconstructed_mlp(name, M, N):
    """Config 1: Llama-2-7B MLP deltas, r = 512, X 2048 x d_i, reconstructed path."""
    mi = {"gate": 0, "down": 2}[name]
    W_b, packed = synth.synthetic_module(M, N, 512, config=1, module=mi, device=DEV, exact_svd=False)
    p4 = kernels.pack_int4(packed, device=DEV)
    Wd = W_b.to(DEV)
    acc = torch.empty(4, M, N, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = kernels.recon_int4(p4, Wd, dbg_acc=acc, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    # every INT32 accumulator of the module, against cuBLASLt's integer GEMM
    merged_t, prods = _torch_reconstruct(packed, W_b, DEV)
    for g in range(4):
        assert torch.equal(acc[g], prods[g]), f"group {g}"
    assert torch.equal(out, merged_t)
    del acc, prods
    # and against the CPU oracle on two row windows (first tile rows, last ragged rows)
    p = O.packed_from_torch(packed)
    wb = _bits(W_b)
    for rows in [(0, 160), (M - 96, M)]:
        _, merged = O.reconstruct(p, rows=rows, base_bits=wb)
        assert np.array_equal(_bits(out[rows[0]:rows[1]]), merged)
    # the application itself: y = x W'^T, against the float64 oracle on a sample of tokens
    x = synth.activations(2048, N, synth.seed_for(1, mi, 2)).to(DEV)
    lin = ADEKernelLinear(W_b, packed).to(DEV)
    y = lin(x)
    assert y.shape == (2048, M)
    Wm = O.bf16_to_f32(_bits(out)).astype(np.float64)
    ref = O.bf16_to_f32(_bits(x[:64])).astype(np.float64) @ Wm.T
    err, cos = O.parity(y[:64].float().cpu().numpy(), ref)
    assert err <= 1e-2 and cos >= 0.9999, (err, cos)
    # size-independent property: reconstruction is additive in the base, W'(W_b) - W'(0) == W_b up to
    # one bf16 rounding of each side
    out0 = kernels.recon_int4(p4, torch.zeros_like(Wd))
    diff = (out.float() - out0.float() - Wd.float()).abs().max().item()
    assert diff <= 2.0 ** -8 * float(out.float().abs().max())
