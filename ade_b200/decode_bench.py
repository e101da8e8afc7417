"""Greedy decoding of a random-init LLaMA-architecture model with a synthetic delta on every linear module.

    python -m ade_b200.decode_bench [--arch 7b|13b|tiny] [--layers L] [--batch B] [--prompt P] [--new N] [--seed S] [--no-fuse]

Stands in for the whole-model configurations of the benchmark (no checkpoints or datasets are needed):
the base model is random-init bfloat16 of the named architecture, every q/k/v/o/gate/up/down projection
carries a delta whose rank is drawn from a seed so that the total fits the alpha = 1/16 bit budget
(`synth.draw_ranks`), packed fields are drawn directly (`random_packed` value ranges).  The prompt is run in
one forward (factored path if batch * prompt <= 128 tokens, reconstructed path above), then N greedy steps
on the factored path; the decode step is captured in a CUDA graph (static KV cache), and also timed
eagerly.  q/k/v and gate/up of every layer are served by one launch each (`fuse_kernel_linears`) unless
--no-fuse is given.  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import time

import torch

from . import synth
from .serving import LINEAR_MODULE_NAMES, ADEKernelLinear, fuse_kernel_linears

ARCH = {
    "7b": dict(hidden_size=4096, intermediate_size=11008, num_hidden_layers=32, num_attention_heads=32),
    "13b": dict(hidden_size=5120, intermediate_size=13824, num_hidden_layers=40, num_attention_heads=40),
    "tiny": dict(hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=8),
}


def random_packed_cuda(d_o, d_i, rank, seed, device):
    """`synth.random_packed` drawn on the device (same shapes, dtypes and value ranges)."""
    g = torch.Generator(device=device).manual_seed(seed)
    ng = rank // 128
    r = lambda *shape: torch.randint(0, 16, shape, generator=g, device=device)
    s = lambda *shape: (torch.exp(torch.randn(*shape, generator=g, device=device) * 0.3) * 2e-4).to(torch.bfloat16)
    return {"U_codes": r(d_o, rank).to(torch.uint8), "U_scale": s(d_o, ng), "U_zero": r(d_o, ng).to(torch.bfloat16),
            "Vt_codes": r(rank, d_i).to(torch.uint8), "Vt_scale": s(ng, d_i), "Vt_zero": r(ng, d_i).to(torch.bfloat16)}


def build_model(arch="7b", layers=None, seed=0, device="cuda", vocab=32000, fuse=True):
    from transformers import LlamaConfig, LlamaForCausalLM

    kw = dict(ARCH[arch])
    if layers is not None:
        kw["num_hidden_layers"] = layers
    cfg = LlamaConfig(vocab_size=vocab, num_key_value_heads=kw["num_attention_heads"], max_position_embeddings=4096, **kw)
    torch.manual_seed(seed)
    with torch.device(device):
        model = LlamaForCausalLM(cfg).to(torch.bfloat16).eval()
    shapes = []
    for li in range(cfg.num_hidden_layers):
        for name in LINEAR_MODULE_NAMES:
            shapes.append(tuple(model.model.layers[li].get_submodule(name).weight.shape))
    ranks = synth.draw_ranks(shapes, alpha=1.0 / 16, seed=seed)
    i = 0
    for li in range(cfg.num_hidden_layers):
        layer = model.model.layers[li]
        for name in LINEAR_MODULE_NAMES:
            parts = name.split(".")
            parent = layer.get_submodule(parts[0])
            lin = getattr(parent, parts[1])
            d_o, d_i = lin.weight.shape
            packed = random_packed_cuda(d_o, d_i, ranks[i], 1000 * seed + i, device)
            setattr(parent, parts[1], ADEKernelLinear(lin.weight.data, packed))
            i += 1
    groups = fuse_kernel_linears(model) if fuse else 0
    return model, ranks, groups


@torch.no_grad()
def run(arch="7b", layers=None, batch=1, prompt=64, new=128, seed=0, device="cuda", fuse=True):
    from transformers import StaticCache

    model, ranks, groups = build_model(arch, layers, seed, device, fuse=fuse)
    cfg = model.config
    g = torch.Generator().manual_seed(seed + 1)
    ids = torch.randint(0, cfg.vocab_size, (batch, prompt), generator=g).to(device)
    max_len = prompt + new + 1

    def fresh_cache():
        return StaticCache(config=cfg, max_cache_len=max_len)

    def prefill(cache):
        pos = torch.arange(prompt, device=device)
        out = model(input_ids=ids, past_key_values=cache, cache_position=pos, use_cache=True)
        return out.logits[:, -1].argmax(-1, keepdim=True)

    def step(cache, tok, pos):
        out = model(input_ids=tok, past_key_values=cache, cache_position=pos, use_cache=True)
        return out.logits[:, -1].argmax(-1, keepdim=True)

    # eager
    cache = fresh_cache()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    tok = prefill(cache)
    torch.cuda.synchronize()
    t_prefill = time.perf_counter() - t0
    pos = torch.tensor([prompt], device=device)
    eager_tokens = [tok]
    n_eager = min(new, 16)
    t0 = time.perf_counter()
    for _ in range(n_eager):
        tok = step(cache, tok, pos)
        pos = pos + 1
        eager_tokens.append(tok)
    torch.cuda.synchronize()
    t_eager = (time.perf_counter() - t0) / n_eager

    # CUDA graph of one decode step.  The static cache advances a write position of its own on every
    # step, so the warm-up (lazy initialisation, scratch buffers) runs on a throw-away cache.
    spare = fresh_cache()
    s_tok = prefill(spare).clone()
    s_pos = torch.tensor([prompt], device=device)
    side = torch.cuda.Stream(device=device)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step(spare, s_tok, s_pos)
    torch.cuda.current_stream().wait_stream(side)
    cache = fresh_cache()
    tok0 = prefill(cache)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        s_next = step(cache, s_tok, s_pos)
    s_tok.copy_(tok0)
    s_pos.fill_(prompt)
    out_tokens = [tok0.clone()]
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(new):
        graph.replay()
        s_tok.copy_(s_next)
        s_pos.add_(1)
        out_tokens.append(s_next.clone())
    e1.record()
    torch.cuda.synchronize()
    t_graph = e0.elapsed_time(e1) / 1e3 / new
    same = all(bool((a == b).all()) for a, b in zip(eager_tokens, out_tokens[:len(eager_tokens)]))
    n_mod = len(ranks)
    return {
        "metric": "decode_tokens_per_s", "arch": arch, "layers": cfg.num_hidden_layers, "modules": n_mod,
        "batch": batch, "prompt": prompt, "new_tokens": new,
        "value": batch / t_graph, "unit": "tokens/s", "ms_per_step_graph": t_graph * 1e3,
        "eager_tokens_per_s": batch / t_eager, "prefill_s": t_prefill,
        "rank_mean": sum(ranks) / n_mod, "fused_groups": groups, "graph_matches_eager_prefix": same, "data": "synthetic, random-init",
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--arch", default="7b", choices=sorted(ARCH))
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=64)
    ap.add_argument("--new", type=int, default=128)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-fuse", action="store_true")
    a = ap.parse_args()
    print(json.dumps(run(a.arch, a.layers, a.batch, a.prompt, a.new, a.seed, fuse=not a.no_fuse)))


if __name__ == "__main__":
    main()
