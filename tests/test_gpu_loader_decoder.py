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
    first = 12 + int((mine[0, 12:] == eos).nonzero()[0])                   # the token may occur before position 14 too
    stopped = greedy_generate(model, ids, 8, eos_token_id=eos, pad_token_id=0)
    assert torch.equal(stopped[0, :first + 1], mine[0, :first + 1]) and bool((stopped[0, first + 1:] == 0).all())


def test_fused_decode_ops_keep_the_torch_arithmetic():
    """RMSNorm, rotary embedding and SiLU * up as single launches against the transformers / torch operations they stand
    in for: rotary embedding and SiLU product bit for bit (same roundings); RMSNorm to within one bfloat16 step on a
    vanishing share of elements (its float32 mean is summed in another order)."""
    from transformers.models.llama import modeling_llama as ml

    from ade_b200 import decode_ops

    g = torch.Generator().manual_seed(5)
    for rows, H in [(1, 4096), (4, 5120), (64, 4096)]:
        x = (torch.randn(rows, H, generator=g) * 3).to(torch.bfloat16).to(DEV)
        norm = ml.LlamaRMSNorm(H, eps=1e-5).to(DEV).to(torch.bfloat16)
        with torch.no_grad():
            norm.weight.copy_((torch.rand(H, generator=g) + 0.5).to(torch.bfloat16))
            want = norm(x)
        got = decode_ops.rmsnorm(x, norm.weight, norm.variance_epsilon)
        diff = (got.float() - want.float()).abs()
        assert float((diff > 0).float().mean()) < 1e-3 and float((diff / want.float().abs().clamp(min=1e-3)).max()) < 1e-2
    for B, T, hq, hk, hd, fused in [(1, 1, 32, 32, 128, True), (4, 1, 40, 40, 128, True), (2, 7, 8, 2, 64, False)]:
        width = (hq + 2 * hk) * hd if fused else None
        if fused:                                           # q and k as column slices of one fused q/k/v output
            y = torch.randn(B * T, width, generator=g).to(torch.bfloat16).to(DEV)
            q2, k2 = y[:, :hq * hd].reshape(B, T, hq * hd), y[:, hq * hd:(hq + hk) * hd].reshape(B, T, hk * hd)
        else:
            q2 = torch.randn(B, T, hq * hd, generator=g).to(torch.bfloat16).to(DEV)
            k2 = torch.randn(B, T, hk * hd, generator=g).to(torch.bfloat16).to(DEV)
        q = q2.view(B, T, hq, hd).transpose(1, 2)
        k = k2.view(B, T, hk, hd).transpose(1, 2)
        ang = torch.rand(B, T, hd, generator=g) * 6.28
        cos, sin = ang.cos().to(torch.bfloat16).to(DEV), ang.sin().to(torch.bfloat16).to(DEV)
        c1 = lambda t: t.unsqueeze(1)
        rot = lambda t: torch.cat((-t[..., hd // 2:], t[..., :hd // 2]), dim=-1)
        want_q, want_k = (q * c1(cos)) + (rot(q) * c1(sin)), (k * c1(cos)) + (rot(k) * c1(sin))
        got_q, got_k = decode_ops.rope(q, k, cos, sin)
        assert torch.equal(got_q, want_q) and torch.equal(got_k, want_k)
    for rows, H in [(1, 4096), (8, 5120), (3, 1000)]:       # residual add + norm in one launch (1000: the element-wise path)
        a = torch.randn(rows, H, generator=g).to(torch.bfloat16).to(DEV)
        r = (torch.randn(rows, H, generator=g) * 4).to(torch.bfloat16).to(DEV)
        norm = ml.LlamaRMSNorm(H, eps=1e-5).to(DEV).to(torch.bfloat16)
        with torch.no_grad():
            want_sum = r + a
            want = norm(want_sum)
        got_sum, got = decode_ops.add_rmsnorm(a, r, norm.weight, norm.variance_epsilon)
        assert torch.equal(got_sum, want_sum)
        diff = (got.float() - want.float()).abs()
        assert float((diff > 0).float().mean()) < 1e-3 and float((diff / want.float().abs().clamp(min=1e-3)).max()) < 1e-2
    for rows, cols in [(1, 11008), (8, 13824)]:
        y = (torch.randn(rows, 2 * cols, generator=g) * 2).to(torch.bfloat16).to(DEV)
        gate, up = y[:, :cols], y[:, cols:]
        want = torch.nn.functional.silu(gate) * up
        assert torch.equal(decode_ops.silu_mul(gate, up), want)


def test_fused_decode_ops_in_the_model():
    """A patched model produces the logits of the unpatched one (to the RMSNorm's last bit) and the same greedy tokens
    through the graph decoder; long prompts and float32 inputs still take the original code."""
    from ade_b200 import decode_ops
    from ade_b200.serving import LINEAR_MODULE_NAMES

    model = _tiny()
    sd = {k: v.clone() for k, v in model.state_dict().items()}
    per_module = {}
    for li in range(2):
        for i, n in enumerate(LINEAR_MODULE_NAMES):
            d_o, d_i = sd[f"model.layers.{li}.{n}.weight"].shape
            per_module[f"model.layers.{li}.{n}"] = synth.random_packed(d_o, d_i, 128, seed=20 * li + i)
    attach_kernel_linears(model, sd, per_module, device=DEV)
    model = model.to(DEV)
    fuse_kernel_linears(model)
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, 512, (2, 9), generator=g).to(DEV)
    with torch.no_grad():
        before = model(ids).logits.float()
        tokens_before = GreedyGraphDecoder(model).generate(ids, 12)
    # two norms per layer, the final norm, two MLPs, two attentions, two decoder layers (residual add + norm)
    assert decode_ops.enable_fused_decode_ops(model) == 2 * 2 + 1 + 2 + 2 + 2
    assert decode_ops.enable_fused_decode_ops(model) == 0                      # idempotent
    with torch.no_grad():
        after = model(ids).logits.float()
        tokens_after = GreedyGraphDecoder(model).generate(ids, 12)
        long_ids = torch.randint(0, 512, (1, 600), generator=g).to(DEV)        # more than MAX_ROWS token rows: original code
        assert model(long_ids).logits.shape == (1, 600, 512)
    assert float((after - before).abs().max()) <= 2e-2 * float(before.abs().max())
    assert (tokens_after == tokens_before).float().mean().item() >= 0.9


def test_attention_decode_step_against_torch():
    """The fused single-token attention step (rotary embedding, cache write, attention) against the same step done with
    torch operations on a static cache: grouped-query heads, a padded batch (masked positions), several steps in a
    row so that the cache written by one step is read by the next."""
    from types import SimpleNamespace

    from ade_b200 import decode_ops

    from ade_b200 import _lib

    g = torch.Generator().manual_seed(7)
    # head dimensions 64 / 128 / 32 take the single-pass kernel (and, with the option off, the two-pass one); 96 only has
    # the two-pass kernel; the long cache makes every row group walk several batches of rows
    cases = [(1, 32, 32, 128, 193, 64), (3, 8, 2, 64, 40, 5), (2, 40, 40, 128, 64, 0), (2, 8, 4, 128, 700, 640), (2, 4, 4, 96, 50, 10),
             (1, 4, 2, 32, 300, 200)]
    for single_pass, (B, hq, hk, hd, L, start) in [(sp, c) for sp in (1, 0) for c in cases]:
        _lib.set_option(_lib.OPT_ATTN_SINGLE_PASS, single_pass)
        keys = torch.zeros(B, hk, L, hd, dtype=torch.bfloat16, device=DEV)
        vals = torch.zeros_like(keys)
        if start:
            keys[:, :, :start] = torch.randn(B, hk, start, hd, generator=g).to(torch.bfloat16).to(DEV)
            vals[:, :, :start] = torch.randn(B, hk, start, hd, generator=g).to(torch.bfloat16).to(DEV)
        rk, rv = keys.clone(), vals.clone()
        layer = SimpleNamespace(keys=keys, values=vals, cumulative_length=torch.tensor([start], device=DEV), is_initialized=True)
        scale = hd ** -0.5
        for step in range(3):
            pos = start + step
            y = torch.randn(B, (hq + 2 * hk) * hd, generator=g).to(torch.bfloat16).to(DEV)         # fused q/k/v output
            q, k, v = (t.unsqueeze(1) for t in (y[:, :hq * hd], y[:, hq * hd:(hq + hk) * hd], y[:, (hq + hk) * hd:]))
            ang = torch.rand(1, 1, hd, generator=g) * 6.28
            cos, sin = ang.cos().to(torch.bfloat16).to(DEV), ang.sin().to(torch.bfloat16).to(DEV)
            mask = torch.zeros(B, 1, 1, L, dtype=torch.bool, device=DEV)
            mask[..., :pos + 1] = True
            if B > 1:
                mask[1, ..., :min(2, pos)] = False                                                  # left padding of one row
            got = decode_ops.attn_decode(q, k, v, cos, sin, mask if step != 1 or B > 1 else None, layer, scale)
            # the same step with torch operations
            q4, k4, v4 = q.view(B, 1, hq, hd).transpose(1, 2), k.view(B, 1, hk, hd).transpose(1, 2), v.view(B, 1, hk, hd).transpose(1, 2)
            rot = lambda t: torch.cat((-t[..., hd // 2:], t[..., :hd // 2]), dim=-1)
            qe, ke = (q4 * cos.unsqueeze(1)) + (rot(q4) * sin.unsqueeze(1)), (k4 * cos.unsqueeze(1)) + (rot(k4) * sin.unsqueeze(1))
            rk[:, :, pos], rv[:, :, pos] = ke[:, :, 0], v4[:, :, 0]
            kk, vv = rk.repeat_interleave(hq // hk, dim=1).float(), rv.repeat_interleave(hq // hk, dim=1).float()
            s = (qe.float() @ kk.transpose(-1, -2)) * scale
            s = s.masked_fill(~mask, float("-inf"))
            want = (torch.softmax(s, -1) @ vv).transpose(1, 2).reshape(B, 1, hq * hd)
            assert int(layer.cumulative_length) == pos + 1 and int(layer._ade_ticket) == 0     # advanced by the launch itself
            assert torch.equal(keys, rk) and torch.equal(vals, rv)                                  # cache written exactly
            assert float((got.float() - want).abs().max()) <= 1e-2 * float(want.abs().max()) + 1e-3
    _lib.set_option(_lib.OPT_ATTN_SINGLE_PASS, 1)
