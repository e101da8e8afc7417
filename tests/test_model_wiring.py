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
