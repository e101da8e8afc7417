"""One-pass packed-file loader (device stored form identical to the host packing) and the graph-captured greedy
decoder (same tokens as the eager loop)."""
from __future__ import annotations

import pytest
import torch

from ade_b200 import kernels, packed_io, synth
from ade_b200.serving import ADEKernelLinear, GreedyGraphDecoder, attach_kernel_linears, fuse_kernel_linears, greedy_generate

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_device_loader_builds_the_host_stored_form(tmp_path):
    mods = {f"model.layers.0.{n}": synth.random_packed(M, N, r, seed=i)
            for i, (n, M, N, r) in enumerate([("self_attn.q_proj", 384, 256, 256), ("mlp.gate_proj", 1000, 384, 640),
                                              ("mlp.down_proj", 256, 1152, 128), ("self_attn.o_proj", 8, 128, 1024)])}
    path = str(tmp_path / "delta.pt")
    packed_io.save_packed(path, mods, {"bits": 4, "group_size": 128})
    f = packed_io.PackedDeltaFile(path)
    loader = packed_io.DeviceDeltaLoader(DEV)
    built = {p: loader.load(f.module(p)) for p in f}       # back to back: the two staging blocks alternate
    loader.finish()
    torch.cuda.synchronize()
    for prefix, packed in mods.items():
        host = kernels.pack_int4(packed)                   # torch ops on the CPU
        for k in kernels.STORED_KEYS:
            assert torch.equal(built[prefix][k].cpu(), host[k]), (prefix, k)
        assert (built[prefix]["M"], built[prefix]["N"], built[prefix]["r"]) == (host["M"], host["N"], host["r"])
        # and the other two routes of pack_int4: CPU fields to a CUDA device, fields already on the device
        for src in (packed, {k: v.to(DEV) for k, v in packed.items()}):
            p4 = kernels.pack_int4(src, device=DEV)
            torch.cuda.synchronize()
            for k in kernels.STORED_KEYS:
                assert torch.equal(p4[k].cpu(), host[k]), (prefix, k)
    # a module built from a loaded stored form computes what a module built from the packed fields computes
    prefix = "model.layers.0.mlp.gate_proj"
    W = synth.base_weight(1000, 384, 3)
    a = ADEKernelLinear(W, mods[prefix]).to(DEV)
    b = ADEKernelLinear(W, None, stored=built[prefix])
    assert b.weight.is_cuda
    x = synth.activations(5, 384, 4).to(DEV)
    assert torch.equal(a(x), b(x))


def _tiny(layers=2):
    from transformers import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=layers, num_attention_heads=4,
                      num_key_value_heads=4, vocab_size=512, max_position_embeddings=512)
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg).to(torch.bfloat16).eval()


def test_graph_decoder_reproduces_the_eager_loop():
    from ade_b200.serving import LINEAR_MODULE_NAMES

    model = _tiny()
    sd = {k: v.clone() for k, v in model.state_dict().items()}
    per_module = {}
    for li in range(2):
        for i, n in enumerate(LINEAR_MODULE_NAMES):
            d_o, d_i = sd[f"model.layers.{li}.{n}.weight"].shape
            per_module[f"model.layers.{li}.{n}"] = synth.random_packed(d_o, d_i, 128 if i % 2 else 256, seed=10 * li + i)
    attach_kernel_linears(model, sd, per_module, device=DEV)
    model = model.to(DEV)
    assert fuse_kernel_linears(model) == 4
    g = torch.Generator().manual_seed(1)
    dec = GreedyGraphDecoder(model)
    for batch, prompt, new in [(1, 12, 10), (3, 7, 6), (1, 150, 5)]:      # the last prompt takes the reconstructed path
        ids = torch.randint(0, 512, (batch, prompt), generator=g).to(DEV)
        eager = dec.generate(ids, new, use_graph=False)
        graphed = dec.generate(ids, new)
        again = dec.generate(ids, new)                     # the captured graph and its cache are reused
        assert graphed.shape == (batch, prompt + new) and torch.equal(graphed[:, :prompt], ids)
        assert torch.equal(graphed, eager) and torch.equal(graphed, again)
    ids = torch.randint(0, 512, (2, 12), generator=g).to(DEV)
    mine = greedy_generate(model, ids, 8)
    with torch.no_grad():
        hf = model.generate(ids, max_new_tokens=8, do_sample=False, eos_token_id=None, pad_token_id=0)
    # the same kernels, but Hugging Face's dynamic cache attends over another padded length: tokens may part ways
    # where two logits are within rounding of each other
    assert (mine == hf).float().mean().item() >= 0.8
    # rows that hit the end-of-sequence token are padded from then on
    eos = int(mine[0, 14])
    stopped = greedy_generate(model, ids, 8, eos_token_id=eos, pad_token_id=0)
    assert int(stopped[0, 14]) == eos and bool((stopped[0, 15:] == 0).all())
