"""Seeded synthetic inputs of the benchmark configurations (no real checkpoints or datasets).

A module's delta is low rank plus noise, dW = A B + E with A (d_o, 64), B (64, d_i) ~ N(0,1) * 0.004
and E ~ N(0, 1e-4^2); it is compressed with ``quantization.compress_module`` at the configured
rank.  For whole-model configurations (hundreds of modules) the exact SVD is replaced by a
randomised range finder of the same rank, which is what makes generation fit in a test run;
the kernels' inputs (codes, scales, zero-points) keep the same shapes, dtypes and value ranges.
"""
from __future__ import annotations

import torch

from . import quantization as Q


def seed_for(config: int, module: int, what: int) -> int:
    """what: 0 = W_b, 1 = delta (A, B, E), 2 = activations."""
    return 10_000 * config + 10 * module + what


def base_weight(d_o, d_i, seed, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(d_o, d_i, generator=g) * 0.02).to(torch.bfloat16).to(device)


def activations(T, d_i, seed, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(T, d_i, generator=g).to(torch.bfloat16).to(device)


def delta_weight(d_o, d_i, seed, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    A = (torch.randn(d_o, 64, generator=g) * 0.004).to(device)
    B = (torch.randn(64, d_i, generator=g) * 0.004).to(device)
    if torch.device(device).type == "cuda":
        gd = torch.Generator(device=device).manual_seed(seed + 7)
        E = torch.randn(d_o, d_i, generator=gd, device=device) * 1e-4
    else:
        E = torch.randn(d_o, d_i, generator=g) * 1e-4
    return A @ B + E


def truncated_svd(dW, rank, exact=True, seed=0):
    """(U, S, V) with V as columns.  exact: torch.linalg.svd; otherwise a randomised range finder
    with two power iterations."""
    if exact:
        U, S, Vh = torch.linalg.svd(dW.float(), full_matrices=False)
        return U[:, :rank].contiguous(), S[:rank].contiguous(), Vh[:rank].t().contiguous()
    g = torch.Generator(device=dW.device).manual_seed(seed)
    k = min(rank + 32, min(dW.shape))
    Y = dW @ torch.randn(dW.shape[1], k, generator=g, device=dW.device)
    for _ in range(2):
        Y, _ = torch.linalg.qr(Y)
        Y = dW @ (dW.t() @ Y)
    Qm, _ = torch.linalg.qr(Y)
    Ub, S, Vh = torch.linalg.svd(Qm.t() @ dW, full_matrices=False)
    U = Qm @ Ub
    return U[:, :rank].contiguous(), S[:rank].contiguous(), Vh[:rank].t().contiguous()


def synthetic_module(d_o, d_i, rank, config=0, module=0, device="cpu", exact_svd=True, generator=None):
    """(W_b bfloat16 on `device`, packed dict on CPU) of one module."""
    W_b = base_weight(d_o, d_i, seed_for(config, module, 0), device)
    dW = delta_weight(d_o, d_i, seed_for(config, module, 1), device)
    r_eff = min(rank, min(d_o, d_i))
    U, S, V = truncated_svd(dW, r_eff, exact=exact_svd, seed=seed_for(config, module, 1))
    if r_eff < rank:        # rank above the matrix size (tiny test shapes only)
        pad = rank - r_eff
        g = torch.Generator().manual_seed(seed_for(config, module, 1) + 3)
        U = torch.cat([U, (torch.randn(d_o, pad, generator=g) * 1e-3).to(U.device)], 1)
        V = torch.cat([V, (torch.randn(d_i, pad, generator=g) * 1e-3).to(V.device)], 1)
        S = torch.cat([S, torch.full((pad,), 1e-6, device=S.device)])
    gen = generator if generator is not None else torch.Generator().manual_seed(0)
    packed = Q.compress_module(U, S, V, 4, 128, gen)
    return W_b, packed


def random_packed(d_o, d_i, rank, seed, device="cpu", on_device=False):
    """Packed fields drawn directly (uniform codes, log-normal scales, uniform zero-points): same
    shapes, dtypes and value ranges as a compressed module, no SVD.  For size sweeps and
    multi-hundred-module models.  on_device=True draws with the device's own generator (another
    stream of numbers, same distributions), which is what makes a 224-module model a matter of seconds."""
    ng = rank // 128
    if on_device:
        g = torch.Generator(device=device).manual_seed(seed)
        ri = lambda *shape: torch.randint(0, 16, shape, generator=g, device=device)
        sc = lambda *shape: (torch.exp(torch.randn(*shape, generator=g, device=device) * 0.3) * 2e-4).to(torch.bfloat16)
        return {"U_codes": ri(d_o, rank).to(torch.uint8), "U_scale": sc(d_o, ng), "U_zero": ri(d_o, ng).to(torch.bfloat16),
                "Vt_codes": ri(rank, d_i).to(torch.uint8), "Vt_scale": sc(ng, d_i), "Vt_zero": ri(ng, d_i).to(torch.bfloat16)}
    g = torch.Generator().manual_seed(seed)
    return {
        "U_codes": torch.randint(0, 16, (d_o, rank), generator=g, dtype=torch.uint8).to(device),
        "U_scale": (torch.exp(torch.randn(d_o, ng, generator=g) * 0.3) * 2e-4).to(torch.bfloat16).to(device),
        "U_zero": torch.randint(0, 16, (d_o, ng), generator=g).to(torch.bfloat16).to(device),
        "Vt_codes": torch.randint(0, 16, (rank, d_i), generator=g, dtype=torch.uint8).to(device),
        "Vt_scale": (torch.exp(torch.randn(ng, d_i, generator=g) * 0.3) * 2e-4).to(torch.bfloat16).to(device),
        "Vt_zero": torch.randint(0, 16, (ng, d_i), generator=g).to(torch.bfloat16).to(device),
    }


def draw_ranks(shapes, alpha=1.0 / 16, seed=0, lo=128, hi=1024):
    """Per-module ranks (multiples of 128 in [lo, hi]) drawn from a seed and trimmed, largest first,
    until sum of group_cost_bits * r/128 fits the budget alpha * 16 * sum(d_o d_i) bits
    (src/allocation.py:168-187, 275-288)."""
    g = torch.Generator().manual_seed(seed)
    ranks = [int(torch.randint(lo // 128, hi // 128 + 1, (1,), generator=g)) * 128 for _ in shapes]
    budget = int(alpha * 16 * sum(a * b for a, b in shapes))
    cost = lambda: sum(Q.group_cost_bits(a, b) * (r // 128) for (a, b), r in zip(shapes, ranks))
    while cost() > budget:
        i = max(range(len(ranks)), key=lambda j: (ranks[j], -j))
        if ranks[i] <= lo:
            break
        ranks[i] -= 128
    return ranks


LLAMA_ARCH = {
    "7b": dict(hidden_size=4096, intermediate_size=11008, num_hidden_layers=32, num_attention_heads=32),
    "13b": dict(hidden_size=5120, intermediate_size=13824, num_hidden_layers=40, num_attention_heads=40),
    "tiny": dict(hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=8),
}


def synthetic_llama(arch="7b", layers=None, seed=0, device="cuda", vocab=32000, fuse=True, alpha=1.0 / 16, fused_ops=True):
    """Random-init bfloat16 LLaMA-architecture model with a synthetic delta on every linear module, each an
    ``ADEKernelLinear`` (configs 2-4 of the benchmark; no checkpoint or dataset is involved).  Ranks are drawn for
    the alpha bit budget (``draw_ranks``), packed fields directly on the device (``random_packed``).  q/k/v and gate/up
    of every layer are served by one launch each (`fuse`), RMSNorm / rotary embedding / SiLU product by one launch each
    (`fused_ops`).  Returns (model, ranks, number of fused q/k/v and gate/up groups)."""
    from transformers import LlamaConfig, LlamaForCausalLM

    from .serving import LINEAR_MODULE_NAMES, ADEKernelLinear, fuse_kernel_linears

    kw = dict(LLAMA_ARCH[arch])
    if layers is not None:
        kw["num_hidden_layers"] = layers
    cfg = LlamaConfig(vocab_size=vocab, num_key_value_heads=kw["num_attention_heads"], max_position_embeddings=4096, **kw)
    torch.manual_seed(seed)
    with torch.device(device):
        model = LlamaForCausalLM(cfg).to(torch.bfloat16).eval()
    shapes = [tuple(model.model.layers[li].get_submodule(n).weight.shape)
              for li in range(cfg.num_hidden_layers) for n in LINEAR_MODULE_NAMES]
    ranks = draw_ranks(shapes, alpha=alpha, seed=seed)
    i = 0
    for li in range(cfg.num_hidden_layers):
        layer = model.model.layers[li]
        for name in LINEAR_MODULE_NAMES:
            owner, _, leaf = name.rpartition(".")
            parent = layer.get_submodule(owner)
            lin = getattr(parent, leaf)
            d_o, d_i = lin.weight.shape
            packed = random_packed(d_o, d_i, ranks[i], 1000 * seed + i, device, on_device=True)
            setattr(parent, leaf, ADEKernelLinear(lin.weight.data, packed))
            i += 1
    groups = fuse_kernel_linears(model) if fuse else 0
    if fused_ops:
        from .decode_ops import enable_fused_decode_ops

        enable_fused_decode_ops(model)
    return model, ranks, groups
