"""Whole-model wiring: a random-init LLaMA-architecture model whose linear modules are replaced by
ADEKernelLinear (the loop of the reference's build_kernel_model), small enough for a test.

CPU part: the module swap itself.  GPU part: prompt forward on the factored path (T <= 128), on the
reconstructed path (T > 128) and a short greedy decode, against the same model with every linear
weight replaced by the oracle's merged weight bf16(W_b + U^V^^T).
"""
from __future__ import annotations

import copy

import numpy as np
import pytest
import torch

from ade_b200 import synth
from ade_b200.serving import ADEKernelLinear, LINEAR_MODULE_NAMES, attach_kernel_linears
from oracle import oracle as O


def _tiny_model(layers=2):
    from transformers import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=layers, num_attention_heads=4,
                      num_key_value_heads=4, vocab_size=512, max_position_embeddings=512)
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg).to(torch.bfloat16).eval()


def _deltas(model, seed=0):
    """One packed delta per linear module, ranks 128 / 256 alternating, modest magnitude."""
    per_module, sd = {}, model.state_dict()
    i = 0
    for li in range(model.config.num_hidden_layers):
        for name in LINEAR_MODULE_NAMES:
            prefix = f"model.layers.{li}.{name}"
            d_o, d_i = sd[prefix + ".weight"].shape
            per_module[prefix] = synth.random_packed(d_o, d_i, 128 if i % 2 else 256, seed=seed + i)
            i += 1
    return per_module


def test_attach_replaces_every_linear_module():
    model = _tiny_model()
    per_module = _deltas(model)
    base_sd = {k: v.clone() for k, v in model.state_dict().items()}
    n = attach_kernel_linears(model, base_sd, per_module)
    assert n == 14
    for layer in model.model.layers:
        for name in LINEAR_MODULE_NAMES:
            m = layer.get_submodule(name)
            assert isinstance(m, ADEKernelLinear) and m.weight.dtype == torch.bfloat16
    # modules without a packed delta stay untouched
    model2 = _tiny_model()
    part = {k: v for k, v in per_module.items() if "layers.0." in k}
    assert attach_kernel_linears(model2, base_sd, part) == 7
    assert isinstance(model2.model.layers[1].mlp.up_proj, torch.nn.Linear)


@pytest.mark.gpu
def test_model_forward_and_greedy_decode_match_merged_weights():
    dev = "cuda"
    model = _tiny_model()
    per_module = _deltas(model)
    base_sd = {k: v.clone() for k, v in model.state_dict().items()}
    ref = copy.deepcopy(model)
    with torch.no_grad():                                  # reference: dense model with the oracle's merged weights
        for prefix, packed in per_module.items():
            p = O.packed_from_torch(packed)
            wb = base_sd[prefix + ".weight"].view(torch.uint16).numpy()
            merged = O.merged_weight_np(p, wb)
            ref.get_submodule(prefix).weight.copy_(torch.from_numpy(merged.copy()).view(torch.bfloat16))
    attach_kernel_linears(model, base_sd, per_module)
    model, ref = model.to(dev), ref.to(dev)
    g = torch.Generator().manual_seed(3)
    for T in (16, 160):                                    # factored path, then reconstructed path
        ids = torch.randint(0, 512, (1, T), generator=g).to(dev)
        with torch.no_grad():
            a = model(ids).logits.float().cpu().numpy()
            b = ref(ids).logits.float().cpu().numpy()
        err, cos = O.parity(a, b)
        assert err <= 3e-2 and cos >= 0.999, (T, err, cos)   # 14 bf16 linears deep: looser than one module
    ids = torch.randint(0, 512, (2, 12), generator=g).to(dev)
    with torch.no_grad():
        out = model.generate(ids, max_new_tokens=8, do_sample=False)
        out_ref = ref.generate(ids, max_new_tokens=8, do_sample=False)
    assert out.shape == (2, 20)
    assert (out[:, :12] == ids).all()
    # greedy tokens agree except where two logits are within rounding of each other
    assert (out == out_ref).float().mean().item() >= 0.8


def test_fused_group_is_a_block_diagonal_module():
    """q/k/v (or gate/up) as one ADE module: V^T stacked along the rank axis, U block diagonal with code 0,
    zero-point 0 and scale 0 outside the blocks, base weights shared as views of one buffer."""
    from ade_b200 import kernels
    from ade_b200.serving import FusedADEGroup, fuse_kernel_linears

    mods = []
    for i, (M, r) in enumerate([(256, 128), (128, 256), (384, 128)]):
        mods.append(ADEKernelLinear(synth.base_weight(M, 256, 20 + i), synth.random_packed(M, 256, r, 10 + i)))
    singles = [{k: v.clone() if torch.is_tensor(v) else v for k, v in m._stored_form().items()} for m in mods]
    weights = [m.weight.clone() for m in mods]
    g = FusedADEGroup(mods)
    assert (g.p4["M"], g.p4["N"], g.p4["r"]) == (768, 256, 512) and g.offsets == [0, 256, 384, 768]
    U = kernels.unpack_nibbles(g.p4["uq"])
    k0 = 0
    for m, f, w, lo, hi in zip(mods, singles, weights, g.offsets[:-1], g.offsets[1:]):
        r = f["r"]
        assert torch.equal(U[lo:hi, k0:k0 + r], kernels.unpack_nibbles(f["uq"]))
        assert int(U[lo:hi, :k0].sum()) == 0 and int(U[lo:hi, k0 + r:].sum()) == 0
        assert torch.equal(g.p4["us"][lo:hi, k0 // 128:(k0 + r) // 128], f["us"])
        assert float(g.p4["us"][lo:hi, :k0 // 128].float().abs().sum()) == 0.0
        assert torch.equal(g.p4["vt"][k0:k0 + r], f["vt"]) and torch.equal(g.p4["vs"][k0 // 128:(k0 + r) // 128], f["vs"])
        assert m.weight.data_ptr() == g.weight[lo:hi].data_ptr() and torch.equal(m.weight, w)
        k0 += r
    # model level: q/k/v and gate/up of every layer, unless the ranks do not fit
    model = _tiny_model()
    attach_kernel_linears(model, {k: v.clone() for k, v in model.state_dict().items()}, _deltas(model))
    assert fuse_kernel_linears(model) == 4
    assert model.model.layers[0].self_attn.o_proj._group is None
    assert model.model.layers[1].mlp.up_proj._group[1] == 1
    model2 = _tiny_model()
    attach_kernel_linears(model2, {k: v.clone() for k, v in model2.state_dict().items()}, _deltas(model2))
    assert fuse_kernel_linears(model2, max_rank=400) == 4          # q/k fit (256 + 128), v is left alone
    assert model2.model.layers[0].self_attn.v_proj._group is None


@pytest.mark.gpu
def test_fused_groups_match_separate_launches():
    """One launch for q/k/v and one for gate/up give what the per-module launches give (the base term bit for
    bit per row; the delta term may be summed in another order over the warps)."""
    from ade_b200.serving import FusedADEGroup, fuse_kernel_linears

    dev = "cuda"
    mods = []
    for i, (M, r) in enumerate([(512, 256), (512, 128), (1024, 384)]):
        mods.append(ADEKernelLinear(synth.base_weight(M, 768, 40 + i), synth.random_packed(M, 768, r, 50 + i)).to(dev))
    for T in (1, 5, 16, 40):
        x = synth.activations(T, 768, 60 + T).to(dev)
        sep = [m(x) for m in mods]
        g = FusedADEGroup(mods)
        fused = [m(x) for m in mods]
        assert g._y is None                                 # all three slices served from one launch
        for a, b in zip(sep, fused):
            err, cos = O.parity(b.float().cpu().numpy(), a.float().cpu().numpy())
            assert err <= 2e-3 and cos >= 0.99999, (T, err, cos)
        for m in mods:                                      # ungroup for the next round
            m._group = None
    # the block hint is validated before any launch: it must tile [0, M) x [0, ng) in ascending order
    import ctypes
    from ade_b200 import _lib, kernels
    g = FusedADEGroup(mods)
    d = kernels._cdelta(g.p4)
    assert d.n_blocks == 3 and list(d.block_rows)[:4] == [0, 512, 1024, 2048] and list(d.block_groups)[:4] == [0, 2, 3, 6]
    x = synth.activations(4, 768, 61).to(dev)
    out = torch.empty(4, 2048, dtype=torch.bfloat16, device=dev)
    scratch = torch.zeros(1 << 20, dtype=torch.uint8, device=dev)
    lib = _lib.load()
    call = lambda: lib.ade_b200_factored(ctypes.byref(d), x.data_ptr(), None, g.weight.data_ptr(), out.data_ptr(),
                                         scratch.data_ptr(), scratch.numel(), 4, None)
    assert call() == 0
    d.block_rows[1] = 1024                              # not ascending
    assert call() == -2
    d.block_rows[1] = 512
    d.block_groups[3] = 5                               # does not end at ng
    assert call() == -2
    g.p4.pop("_cdelta")
    for m in mods:
        m._group = None
    # whole model: same greedy tokens with and without fusion, graph of calls unchanged
    model = _tiny_model()
    per_module = _deltas(model)
    base_sd = {k: v.clone() for k, v in model.state_dict().items()}
    attach_kernel_linears(model, base_sd, per_module)
    model = model.to(dev)
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 512, (2, 12), generator=g).to(dev)
    with torch.no_grad():
        plain = model(ids).logits.float().cpu().numpy()
        out_plain = model.generate(ids, max_new_tokens=8, do_sample=False)
        assert fuse_kernel_linears(model) == 4
        fused = model(ids).logits.float().cpu().numpy()
        out_fused = model.generate(ids, max_new_tokens=8, do_sample=False)
        long_ids = torch.randint(0, 512, (1, 160), generator=g).to(dev)     # T > 128: the members' own reconstructed path
        assert model(long_ids).logits.shape == (1, 160, 512)
    err, cos = O.parity(fused, plain)
    assert err <= 1e-2 and cos >= 0.9999, (err, cos)
    assert (out_plain == out_fused).float().mean().item() >= 0.8
