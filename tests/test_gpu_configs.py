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
    # the module's own route: int8 operands expanded once and kept, kernel fed by TMA; same bits
    assert torch.equal(lin.merged_weight(), out) and lin._x8 is not None
    kept = lin._x8[1][0].data_ptr()
    assert torch.equal(lin.merged_weight(), out) and lin._x8[1][0].data_ptr() == kept


# ---------------------------------------------------------------------------------------------------------------
# Configs 2-4: 13B-architecture shapes, non-power-of-two ranks on full-size modules, one full-size 7B decoder layer
# ---------------------------------------------------------------------------------------------------------------
_cache = {}


def _base(M, N, seed):
    key = (M, N, seed)
    if key not in _cache:
        _cache.clear()                                     # one full-size base weight at a time
        _cache[key] = synth.base_weight(M, N, seed)
    return _cache[key]


@pytest.mark.parametrize("M,N", [(5120, 5120), (13824, 5120), (5120, 13824)])
@pytest.mark.parametrize("T,r", [(1, 384), (4, 640), (8, 896), (64, 1024), (1, 1024), (64, 384)])
def test_factored_13b_shapes(M, N, T, r):
    """Config 3 / 4 module shapes (hidden 5120, MLP 13824) on the factored path, at decode sizes and at a 64-token
    prompt, with the non-power-of-two ranks an alpha = 1/16 allocation produces, through the module (fused base
    GEMM up to 16 tokens, cuBLAS base + delta launch above)."""
    tp = synth.random_packed(M, N, r, 13 * T + r + M)
    W_b = _base(M, N, 21)
    x = synth.activations(T, N, 22 + T)
    lin = ADEKernelLinear(W_b, tp).to(DEV)
    y = lin(x.to(DEV))
    torch.cuda.synchronize()
    kernels.check_factored_status(DEV)
    ref = O.factored_apply(_bits(x), _bits(W_b), O.packed_from_torch(tp))
    err, cos = O.parity(y.float().cpu().numpy(), ref)
    assert err <= 1e-2 and cos >= 0.9999, (err, cos)


@pytest.mark.parametrize("M,N,r", [(4096, 4096, 384), (4096, 4096, 640), (4096, 4096, 896), (11008, 4096, 640)])
@pytest.mark.parametrize("T", [1, 8, 64])
def test_factored_7b_shapes_odd_ranks(M, N, r, T):
    """Ranks 384 / 640 / 896 (seeded random-orthogonal rotation in the reference's compressor, no Hadamard) on the
    4096-wide modules of configs 2 and 4."""
    tp = synth.random_packed(M, N, r, 7 * T + r)
    W_b = _base(M, N, 23)
    x = synth.activations(T, N, 24 + T)
    lin = ADEKernelLinear(W_b, tp).to(DEV)
    y = lin(x.to(DEV))
    torch.cuda.synchronize()
    kernels.check_factored_status(DEV)
    ref = O.factored_apply(_bits(x), _bits(W_b), O.packed_from_torch(tp))
    err, cos = O.parity(y.float().cpu().numpy(), ref)
    assert err <= 1e-2 and cos >= 0.9999, (err, cos)


@pytest.mark.parametrize("members,T", [([(5120, 640), (5120, 384), (5120, 896)], 1), ([(5120, 640), (5120, 384), (5120, 896)], 8),
                                       ([(13824, 896), (13824, 1024)], 1), ([(13824, 896), (13824, 1024)], 8)])
def test_fused_groups_13b_layer(members, T):
    """q/k/v (15360 rows, rank 1920) and gate/up (27648 rows, rank 1920) of a 13B decoder layer served by one launch
    each: every member's slice against the oracle for that member alone."""
    from ade_b200.serving import FusedADEGroup

    N = 5120
    mods, refs = [], []
    x = synth.activations(T, N, 30 + T)
    for i, (M, r) in enumerate(members):
        tp = synth.random_packed(M, N, r, 40 + i + r)
        W_b = synth.base_weight(M, N, 50 + i)
        mods.append(ADEKernelLinear(W_b, tp).to(DEV))
        refs.append(O.factored_apply(_bits(x), _bits(W_b), O.packed_from_torch(tp)))
    g = FusedADEGroup(mods)
    assert g.p4["M"] == sum(m for m, _ in members) and g.p4["r"] == sum(r for _, r in members)
    xd = x.to(DEV)
    ys = [m(xd) for m in mods]
    torch.cuda.synchronize()
    assert g._y is None                                    # one launch served all members
    kernels.check_factored_status(DEV)
    for y, ref in zip(ys, refs):
        err, cos = O.parity(y.float().cpu().numpy(), ref)
        assert err <= 1e-2 and cos >= 0.9999, (err, cos)


@pytest.mark.parametrize("M,N,r", [(13824, 5120, 640), (5120, 13824, 384), (5120, 5120, 1024)])
def test_reconstruction_13b_shapes_bit_exact(M, N, r):
    """Config 3 / 4b module shapes on the reconstructed path: every INT32 accumulator and the merged bf16 weight
    against the integer GEMM + float sequence restated in torch (whole matrix) and the C oracle (row windows)."""
    tp = synth.random_packed(M, N, r, 3 * r + M)
    W_b = synth.base_weight(M, N, 61)
    p4 = kernels.pack_int4(tp, device=DEV)
    Wd = W_b.to(DEV)
    ng = r // 128
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    merged_t, prods = _torch_reconstruct(tp, W_b, DEV)
    out = kernels.recon_int4(p4, Wd, status=status)         # production instantiation first
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(out, merged_t)
    out_x = kernels.recon_int4(p4, Wd, status=status, expanded=kernels.expand_codes(p4))   # and from int8 operands
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(out_x, merged_t)
    del out_x
    for g0 in range(0, ng, 2):                              # accumulators two groups at a time (memory)
        g1 = min(g0 + 2, ng)
        sub = {k: (v[:, g0 * 128:g1 * 128] if k == "U_codes" else v[g0 * 128:g1 * 128] if k == "Vt_codes"
                   else v[:, g0:g1] if k.startswith("U_") else v[g0:g1]) for k, v in tp.items()}
        acc = torch.empty(g1 - g0, M, N, dtype=torch.int32, device=DEV)
        kernels.recon_int4(kernels.pack_int4(sub, device=DEV), Wd, dbg_acc=acc, status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        for g in range(g0, g1):
            assert torch.equal(acc[g - g0], prods[g]), f"group {g}"
        del acc
    del prods
    p = O.packed_from_torch(tp)
    wb = _bits(W_b)
    for rows in [(0, 130), (M - 70, M)]:
        _, merged = O.reconstruct(p, rows=rows, base_bits=wb)
        assert np.array_equal(_bits(out[rows[0]:rows[1]]), merged)


def test_full_size_7b_decoder_layer_against_merged_weights():
    """Config 2 at full module size: one Llama-2-7B-shaped decoder layer (hidden 4096, MLP 11008, 32 heads) whose seven
    linear modules carry deltas with ranks drawn for the alpha = 1/16 budget, against the same layer with the oracle's
    merged weights bf16(W_b + U^V^^T) in plain nn.Linear modules.  Every module's output on the input it actually
    receives must meet the stated tolerance (T = 1: fused decode launches, T = 64: base GEMM + delta launch), with
    q/k/v and gate/up served by fused groups; the logits of the whole model are compared as well."""
    import copy

    from transformers import LlamaConfig, LlamaForCausalLM

    from ade_b200.serving import LINEAR_MODULE_NAMES, attach_kernel_linears, fuse_kernel_linears

    cfg = LlamaConfig(hidden_size=4096, intermediate_size=11008, num_hidden_layers=1, num_attention_heads=32,
                      num_key_value_heads=32, vocab_size=4096, max_position_embeddings=512)
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg).to(torch.bfloat16).eval()
    sd = {k: v.clone() for k, v in model.state_dict().items()}
    shapes = [tuple(sd[f"model.layers.0.{n}.weight"].shape) for n in LINEAR_MODULE_NAMES]
    ranks = synth.draw_ranks(shapes * 32, alpha=1.0 / 16, seed=0)[:7]          # the first layer of the 224-module draw
    assert all(128 <= r <= 1024 and r % 128 == 0 for r in ranks)
    per_module = {f"model.layers.0.{n}": synth.random_packed(*shp, r, seed=70 + i)
                  for i, (n, shp, r) in enumerate(zip(LINEAR_MODULE_NAMES, shapes, ranks))}
    ref = copy.deepcopy(model)
    with torch.no_grad():
        for prefix, packed in per_module.items():
            merged = O.merged_weight_np(O.packed_from_torch(packed), sd[prefix + ".weight"].view(torch.uint16).numpy())
            ref.get_submodule(prefix).weight.copy_(torch.from_numpy(merged.copy()).view(torch.bfloat16))
    assert attach_kernel_linears(model, sd, per_module, device=DEV) == 7      # stored forms built by the device loader
    model, ref = model.to(DEV), ref.to(DEV)
    assert fuse_kernel_linears(model) == 2                  # q/k/v (or q/k when the three ranks exceed 2048) and gate/up
    g = torch.Generator().manual_seed(9)
    for T in (1, 64):
        ids = torch.randint(0, 4096, (1, T), generator=g).to(DEV)
        seen = {}
        hooks = [model.get_submodule(p).register_forward_hook(lambda m, a, o, p=p: seen.__setitem__(p, (a[0].detach(), o.detach())))
                 for p in per_module]
        with torch.no_grad():
            logits = model(ids).logits.float().cpu().numpy()
            logits_ref = ref(ids).logits.float().cpu().numpy()
        for h in hooks:
            h.remove()
        torch.cuda.synchronize()
        kernels.check_factored_status(DEV)
        for prefix, (xin, yout) in seen.items():
            W = ref.get_submodule(prefix).weight.detach().float()
            want = (xin.reshape(-1, xin.shape[-1]).float() @ W.t()).cpu().numpy()
            err, cos = O.parity(yout.reshape(want.shape).float().cpu().numpy(), want)
            assert err <= 1e-2 and cos >= 0.9999, (T, prefix, err, cos)
        err, cos = O.parity(logits, logits_ref)
        assert err <= 2e-2 and cos >= 0.9995, (T, err, cos)     # seven bf16 modules, a softmax and two norms deep
