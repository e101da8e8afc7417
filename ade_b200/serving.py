"""Serving boundary: the delta-linear module the Hugging Face forward calls.

Keeps the API of the reference's ``src/serving.py`` -- ``ADEKernelLinear(W_b, packed, group_size,
decode_max_tokens, use_decode, use_recon, split_k)`` with ``forward(x)`` and the attributes
``out_features / in_features / weight``, and ``build_kernel_model`` -- on top of the B200 kernels.
Differences: tensors are bfloat16 (the reference module is float16), there is no float
fallback (``use_decode`` / ``use_recon`` = False raise), and for T <= decode_max_tokens the base
GEMM x W_b^T runs inside the factored kernel instead of a separate ``F.linear`` up to 16 tokens.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .kernels import (GROUP, STORED_KEYS, decode_forward_packed, decode_kernel_status, expand_codes, factored_forward,
                      pack_int4, recon_int4, recon_kernel_status)

# Up to this many tokens the base GEMM x W_b^T runs inside the factored kernel (one launch, W_b streamed once by
# a kernel built for skinny operands, h computed by side warps under the stream).  Above it cuBLAS is faster at the
# base term, so the module falls back to the reference's split: F.linear for the base, the kernel for the delta
# only (measured on B200 per call, fused / split: 4096 x 4096 T = 16 14.5 / 21.0 us, T = 32 22.4 / 23.7, T = 64
# 46.3 / 29.2; 11008 x 4096 T = 16 30.1 / 34.0, T = 24 40.6 / 39.2, T = 64 117.6 / 55.9).
FUSED_BASE_MAX_TOKENS = 16
# Modules keep int8 operands for the reconstructed path once they have served a long input (see ADEKernelLinear._expanded).
EXPAND_FOR_RECON = True

# the seven linear modules of a LLaMA decoder layer (same list as src/adaptation.py:39-42)
LINEAR_MODULE_NAMES = (
    "self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
    "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj",
)


class ADEKernelLinear(nn.Module):
    """Linear module W_b + U^ V^^T applied with the B200 kernels (bfloat16): factored application
    for T <= decode_max_tokens tokens, reconstructed application otherwise (src/serving.py:40-112)."""

    def __init__(self, W_b: torch.Tensor, packed: dict, group_size: int = GROUP,
                 decode_max_tokens: int = 128, use_decode: bool = True, use_recon: bool = True,
                 split_k: bool = False, stored: dict | None = None):
        """
        Parameters:
            W_b: Base weight (d_o, d_i).
            packed: Packed factors of the module (src/quantization.py:276-285 layout); may be None when
                `stored` is given.
            group_size: Group size G (128).
            decode_max_tokens: Largest T handled by factored application (at most 128).
            use_decode / use_recon: must stay True; there is no float reconstruction fallback.
            split_k: accepted for compatibility, ignored (the kernels are deterministic).
            stored: the module's stored form if it has been built already (``pack_int4`` or
                ``packed_io.DeviceDeltaLoader.load``); the module then packs nothing itself and its buffers live
                where the stored form lives.  No counterpart in the reference.
        """
        super().__init__()
        if not (use_decode and use_recon):
            raise ValueError("ADEKernelLinear: the B200 build has no float-reconstruction fallback; "
                             "use_decode and use_recon must be True")
        if not 1 <= int(decode_max_tokens) <= 128:
            raise ValueError("decode_max_tokens must be in 1..128")
        self.group_size = group_size
        self.decode_max_tokens = int(decode_max_tokens)
        self.use_decode, self.use_recon, self.split_k = use_decode, use_recon, split_k
        self.out_features, self.in_features = W_b.shape
        p4 = stored if stored is not None else pack_int4(packed, group_size)
        if (p4["M"], p4["N"]) != tuple(W_b.shape):
            raise ValueError(f"delta is {p4['M']} x {p4['N']}, base weight {tuple(W_b.shape)}")
        W_b = W_b.detach().to(device=p4["uq"].device, dtype=torch.bfloat16) if stored is not None else W_b.detach().to(torch.bfloat16)
        self.register_buffer("weight", W_b.contiguous())
        self._dims = (p4["M"], p4["N"], p4["r"])
        for k in STORED_KEYS:
            self.register_buffer(f"p4_{k}", p4[k])
        self._p4 = None
        self._x8 = None               # (uq pointer, (u8, v8)): expanded operands of the reconstruction, built on demand
        self._group = None            # (FusedADEGroup, index) once fuse_kernel_linears has grouped this module

    def _stored_form(self) -> dict:
        """Stored form on the module's device (rebuilt after .to(device))."""
        if self._p4 is None or self._p4["uq"].data_ptr() != self.p4_uq.data_ptr():
            self._p4 = {k: getattr(self, f"p4_{k}") for k in STORED_KEYS}
            self._p4["M"], self._p4["N"], self._p4["r"] = self._dims
        return self._p4

    def _expanded(self):
        """int8 operands of the reconstruction kernel, built on the first long input and kept ((d_o + d_i) * r bytes;
        EXPAND_FOR_RECON = False keeps the packed codes only and unpacks inside the kernel on every call)."""
        p4 = self._stored_form()
        if self._x8 is None or self._x8[0] != p4["uq"].data_ptr():
            self._x8 = (p4["uq"].data_ptr(), expand_codes(p4))
        return self._x8[1]

    def merged_weight(self) -> torch.Tensor:
        """bf16(W_b + U^ V^^T), one launch of the reconstruction kernel."""
        p4 = self._stored_form()
        expanded = self._expanded() if EXPAND_FOR_RECON and p4["r"] <= 1024 else None
        return recon_int4(p4, self.weight, self.group_size, expanded=expanded)

    def forward(self, x):
        """x (..., d_i) -> (..., d_o) in bfloat16."""
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).to(torch.bfloat16).contiguous()
        T = x2.shape[0]
        if T == 0:
            return x2.new_empty(*shape[:-1], self.out_features)
        if T <= FUSED_BASE_MAX_TOKENS and T <= self.decode_max_tokens:
            y = self._group[0].apply(self._group[1], x, x2) if self._group is not None else None
            if y is None:
                y = factored_forward(x2, self._stored_form(), weight=self.weight)
        elif T <= self.decode_max_tokens:
            # the reference's own split (src/serving.py:106-111): library GEMM for the base term, kernel for the delta
            y = decode_forward_packed(x2, F.linear(x2, self.weight), self._stored_form())
        else:
            y = F.linear(x2, self.merged_weight())
        return y.reshape(*shape[:-1], self.out_features)


class FusedADEGroup:
    """Several ADEKernelLinear modules that are always applied to the same input (q/k/v of an attention block,
    gate/up of an MLP), served by ONE launch of the factored kernel per decode step.

    The group is an ordinary ADE module in disguise: d_o = sum of the members' d_o, rank = sum of their ranks,
    V^T = the members' V^T stacked along the rank axis, U = block diagonal.  Outside its own block a row of U
    holds code 0 with zero-point 0 and scale 0, so the extra rank groups contribute exactly 0.0 and the kernel
    needs no change; the price is the extra zero codes of U ((k - 1) * d_o * r / 2 bytes, ~1 % of the base weight)
    against k - 1 launches, pipeline fills and grid-wide hand-overs saved.  The members' base weights become views
    of one concatenated buffer (no copy is kept).  Only the factored path (T <= decode_max_tokens) is fused;
    longer inputs go through the members' own reconstructed path.

    This has no counterpart in the reference, which launches its kernels per module (src/serving.py:94-112).
    """

    def __init__(self, members):
        self.members = list(members)
        m0 = self.members[0]
        dev = m0.weight.device
        if any(m.in_features != m0.in_features or m.weight.device != dev or m.decode_max_tokens != m0.decode_max_tokens
               for m in self.members):
            raise ValueError("FusedADEGroup: members must share d_i, device and decode_max_tokens")
        forms = [m._stored_form() for m in self.members]
        Ms = [f["M"] for f in forms]
        rs = [f["r"] for f in forms]
        N, M, r = m0.in_features, sum(Ms), sum(rs)
        ng = r // GROUP
        self.offsets = [sum(Ms[:i]) for i in range(len(Ms) + 1)]
        # base weights: one buffer, the members keep views of it
        W = torch.cat([m.weight for m in self.members], dim=0)
        for m, lo, hi in zip(self.members, self.offsets[:-1], self.offsets[1:]):
            m._buffers["weight"] = W[lo:hi]
        self.weight = W
        uq = torch.zeros(M, r // 2, dtype=torch.uint8, device=dev)
        us = torch.zeros(M, ng, dtype=forms[0]["us"].dtype, device=dev)
        uz = torch.zeros(M, ng, dtype=torch.uint8, device=dev)
        k0 = 0
        for f, lo, hi in zip(forms, self.offsets[:-1], self.offsets[1:]):
            uq[lo:hi, k0 // 2:(k0 + f["r"]) // 2] = f["uq"]
            us[lo:hi, k0 // GROUP:(k0 + f["r"]) // GROUP] = f["us"]
            uz[lo:hi, k0 // GROUP:(k0 + f["r"]) // GROUP] = f["uz"]
            k0 += f["r"]
        self.p4 = {
            "uq": uq, "us": us, "uz": uz,
            "vq": torch.cat([f["vq"] for f in forms], dim=1).contiguous(),
            "vt": torch.cat([f["vt"] for f in forms], dim=0).contiguous(),
            "vs": torch.cat([f["vs"] for f in forms], dim=0).contiguous(),
            "vz": torch.cat([f["vz"] for f in forms], dim=0).contiguous(),
            "M": M, "N": N, "r": r,
            # rows of member i use only its own rank groups: the kernel skips the zero blocks of U
            "blocks": [(self.offsets[i], sum(rs[:i]) // GROUP) for i in range(len(Ms) + 1)] if len(Ms) <= 4 else None,
        }
        self._x = None                # the input tensor the cached result belongs to (kept alive while cached)
        self._ver = -1
        self._y = None
        self._used = set()
        for i, m in enumerate(self.members):
            m._group = (self, i)

    def release(self):
        """Dissolve the group: the members go back to their own launches and the fused buffers are dropped."""
        for m in self.members:
            if m._group is not None and m._group[0] is self:
                m._group = None
        self.weight = self.p4 = self._x = self._y = None

    def apply(self, index: int, x, x2):
        """Output of member `index` for the input x (x2 = x as a contiguous (T, d_i) bfloat16 matrix), or None when
        the group cannot serve it (the members moved to another device since the group was built; the group then
        dissolves).  The first member asked about a given tensor launches for all; the others get their slices of
        that result as long as they present the very same tensor object, unmodified: the group holds a reference to
        it while a result is cached, so no other tensor can take its place in memory, and an in-place write bumps
        its version."""
        if self.weight is None or self.members[0].weight.data_ptr() != self.weight.data_ptr():
            self.release()
            return None
        if self._y is None or x is not self._x or x._version != self._ver or index in self._used:
            self._y = factored_forward(x2, self.p4, weight=self.weight)
            self._x, self._ver = x, x._version
            self._used = set()
        self._used.add(index)
        y = self._y[:, self.offsets[index]:self.offsets[index + 1]]
        if len(self._used) == len(self.members):
            self._x = self._y = None           # every member has taken its slice: nothing is served twice
        return y


# modules of a decoder layer that read the same activations
FUSABLE_GROUPS = (("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"), ("mlp.gate_proj", "mlp.up_proj"))


def fuse_kernel_linears(model, max_rank: int = 2048) -> int:
    """Group q/k/v and gate/up of every decoder layer into FusedADEGroups (after the model is on its device).
    A group is formed when all its modules are ADEKernelLinear and their ranks add up to at most `max_rank`
    (the kernels' limit); q/k alone are tried when q/k/v does not fit.  Returns the number of groups."""
    n = 0
    for layer in _decoder_layers(model):
        for names in FUSABLE_GROUPS:
            mods = []
            for sn in names:
                try:
                    m = layer.get_submodule(sn)
                except AttributeError:
                    m = None
                mods.append(m)
            if not all(isinstance(m, ADEKernelLinear) and m._group is None for m in mods):
                continue
            while len(mods) >= 2 and sum(m._dims[2] for m in mods) > max_rank:
                mods = mods[:-1]
            if len(mods) >= 2:
                FusedADEGroup(mods)
                n += 1
    return n


def _decoder_layers(model):
    """The ``nn.ModuleList`` of decoder layers, wherever the architecture keeps it: a LLaMA-family causal LM
    (``model.model.layers``) or a llava-hf LLaVA model, whose language model sits under ``model.language_model``
    or, in newer transformers, ``model.model.language_model`` (what src/serving.py:115-130 resolves)."""
    for path in ("model.language_model.model", "model.language_model", "language_model.model", "language_model", "model"):
        node = model
        for name in path.split("."):
            node = getattr(node, name, None)
            if node is None:
                break
        if node is not None and isinstance(getattr(node, "layers", None), nn.ModuleList):
            return node.layers
    raise AttributeError(f"{type(model).__name__} has no decoder layer list this build knows how to find")


def attach_kernel_linears(model, base_state_dict: dict, per_module, group_size: int = GROUP,
                          decode_max_tokens: int = 128, split_k: bool = False, device=None) -> int:
    """Give every linear module that has a packed delta an ADEKernelLinear in its place.

    Does for a model that is already in memory what the module-swap loop of src/serving.py:178-190 does after
    loading one: `base_state_dict` maps ``model.layers.<i>.<name>.weight`` to the base weight, `per_module` (a
    dict or a ``packed_io.PackedDeltaFile``) maps ``model.layers.<i>.<name>`` to the packed fields.  With a CUDA
    `device` the stored forms are built there in one pass (pinned staging + the packing kernels, see
    ``packed_io.DeviceDeltaLoader``) and the new modules are born on that device; otherwise they are packed on
    the CPU and move with ``model.to``.  Returns the number of modules replaced.
    """
    loader = None
    if device is not None and torch.device(device).type == "cuda":
        from .packed_io import DeviceDeltaLoader

        loader = DeviceDeltaLoader(device)
    fetch = per_module.module if hasattr(per_module, "module") else per_module.__getitem__
    swapped = 0
    for li, layer in enumerate(_decoder_layers(model)):
        for sub in LINEAR_MODULE_NAMES:
            prefix = f"model.layers.{li}.{sub}"
            if prefix not in per_module:
                continue
            owner_path, _, leaf = sub.rpartition(".")
            stored = loader.load(fetch(prefix)) if loader is not None else None
            new = ADEKernelLinear(base_state_dict[prefix + ".weight"], None if loader is not None else fetch(prefix),
                                  group_size, decode_max_tokens, split_k=split_k, stored=stored)
            setattr(layer.get_submodule(owner_path), leaf, new)
            swapped += 1
    if loader is not None:
        loader.finish()
    return swapped


def build_kernel_model(task: str, aligned_path: str, base_path: str, packed_path: str,
                       llava_hf_path: str | None = None, device: str = "cuda",
                       decode_max_tokens: int = 128, split_k: bool = False):
    """bfloat16 evaluation model: the aligned model with every compressed linear module replaced
    by an ADEKernelLinear (same signature as src/serving.py:133-194).

    Raises when the kernels cannot run on `device`: the reference degrades to a PyTorch
    reconstruction there (src/serving.py:155-165), this build does not.
    """
    from transformers import AutoModelForCausalLM, AutoProcessor, AutoTokenizer

    from .packed_io import PackedDeltaFile

    for ok, reason in (decode_kernel_status(device), recon_kernel_status(device)):
        if not ok:
            raise RuntimeError(f"[kernels] B200 delta kernels unavailable on {device}: {reason}")
    if task == "multimodal":
        from transformers import LlavaForConditionalGeneration
        model = LlavaForConditionalGeneration.from_pretrained(llava_hf_path, dtype=torch.bfloat16)
        processor = AutoProcessor.from_pretrained(llava_hf_path)
    else:
        model = AutoModelForCausalLM.from_pretrained(aligned_path, dtype=torch.bfloat16)
        processor = AutoTokenizer.from_pretrained(aligned_path)
    base_sd = AutoModelForCausalLM.from_pretrained(base_path, dtype=torch.bfloat16).state_dict()
    delta = PackedDeltaFile(packed_path)                       # memory-mapped; streamed to the device module by module
    n = attach_kernel_linears(model, base_sd, delta, int(delta.meta["group_size"]), decode_max_tokens, split_k, device=device)
    del base_sd, delta
    model = model.to(device).eval()
    print(f"[kernels] {n} linear modules apply the compressed delta at every forward")
    return model, processor


class GreedyGraphDecoder:
    """Greedy generation whose per-token step is one CUDA-graph replay.

    The reference generates with Hugging Face ``model.generate(..., do_sample=False)`` (src/evaluate.py:241): one
    Python pass over every module per token, three launches per delta module.  At decode sizes that host work is
    several times the GPU time, so here the single-token forward (static KV cache, fixed shapes) is captured once
    per (batch, cache length) and replayed; the prompt runs as one ordinary forward (factored path up to 128
    tokens, reconstructed path above).  Output format is ``generate``'s: (batch, prompt + new) token ids.  Stopping
    criteria are the caller's business: all `max_new_tokens` tokens are produced, unless `eos_token_id` is given, in
    which case rows that have emitted it are padded with `pad_token_id` from then on (as ``generate`` pads them).

    ``check_status=True`` (default) reads the factored kernel's status words once at the end of every call and
    raises if a grid-wide wait expired during it.
    """

    def __init__(self, model, check_status: bool = True):
        self.model = model
        self.check_status = check_status
        self._graphs = {}          # (batch, max_len) -> (graph, cache, tok, pos, next)

    def _step(self, cache, tok, pos):
        out = self.model(input_ids=tok, past_key_values=cache, cache_position=pos, use_cache=True)
        return out.logits[:, -1].argmax(-1, keepdim=True)

    def _prefill(self, cache, ids):
        pos = torch.arange(ids.shape[1], device=ids.device)
        out = self.model(input_ids=ids, past_key_values=cache, cache_position=pos, use_cache=True)
        return out.logits[:, -1].argmax(-1, keepdim=True)

    def _captured(self, batch, max_len, device):
        from transformers import StaticCache

        for (b, ml), entry in self._graphs.items():            # a graph with a longer cache serves shorter requests too
            if b == batch and ml >= max_len:
                return entry
        key = (batch, max_len)
        if key not in self._graphs:
            cfg = self.model.config
            tok = torch.zeros(batch, 1, dtype=torch.long, device=device)
            pos = torch.zeros(1, dtype=torch.long, device=device)
            # warm-up on a throw-away cache (lazy initialisation, scratch buffers of the kernels) on a side stream
            spare = StaticCache(config=cfg, max_cache_len=max_len)
            side = torch.cuda.Stream(device=device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._step(spare, tok, pos)
            torch.cuda.current_stream().wait_stream(side)
            del spare
            cache = StaticCache(config=cfg, max_cache_len=max_len)
            # two steps outside the capture: the first allocates the cache's tensors (lazily, inside transformers), the
            # second lets code that only engages on an initialised cache (the fused attention step) allocate its own
            for _ in range(2):
                self._step(cache, tok, pos)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                nxt = self._step(cache, tok, pos)
            self._graphs[key] = (graph, cache, tok, pos, nxt)
        return self._graphs[key]

    @torch.no_grad()
    def generate(self, input_ids, max_new_tokens: int, eos_token_id=None, pad_token_id=0, use_graph: bool = True,
                 timings: dict | None = None):
        """(batch, prompt) token ids -> (batch, prompt + max_new_tokens).  use_graph=False runs the same loop eagerly
        (the two produce the same tokens; the eager loop is what a plain ``model.generate`` costs).  When `timings`
        is a dict it receives ``prefill_ms`` and ``decode_ms`` (CUDA events around the prompt forward and around the
        max_new_tokens - 1 decode steps; the call then synchronises)."""
        from transformers import StaticCache

        batch, prompt = input_ids.shape
        device = input_ids.device
        max_len = prompt + max_new_tokens + 1
        if use_graph:
            graph, cache, tok, pos, nxt = self._captured(batch, max_len, device)
        else:
            cache = StaticCache(config=self.model.config, max_cache_len=max_len)
            tok = torch.zeros(batch, 1, dtype=torch.long, device=device)
            pos = torch.zeros(1, dtype=torch.long, device=device)
        cache.reset()
        out = torch.empty(batch, prompt + max_new_tokens, dtype=torch.long, device=device)
        out[:, :prompt] = input_ids
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)] if timings is not None else None
        if ev:
            ev[0].record()
        first = self._prefill(cache, input_ids)
        if ev:
            ev[1].record()
        tok.copy_(first)
        pos.fill_(prompt)
        alive = torch.ones(batch, 1, dtype=torch.bool, device=device)
        for i in range(max_new_tokens):
            cur = tok.clone()
            if eos_token_id is not None:
                cur = torch.where(alive, cur, torch.full_like(cur, pad_token_id))
                alive = alive & (cur != eos_token_id)
            out[:, prompt + i] = cur[:, 0]
            if i + 1 == max_new_tokens:
                break
            if use_graph:
                graph.replay()
                tok.copy_(nxt)
            else:
                tok.copy_(self._step(cache, tok, pos))
            pos.add_(1)
        if ev:
            ev[2].record()
            torch.cuda.synchronize(device)
            timings["prefill_ms"], timings["decode_ms"] = ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2])
        if self.check_status:
            from .kernels import check_factored_status

            check_factored_status(device)
        return out


def greedy_generate(model, input_ids, max_new_tokens: int, **kw):
    """``model.generate(input_ids, do_sample=False, max_new_tokens=...)`` with the decode step replayed from a CUDA
    graph; the decoder (and its captured graphs) is cached on the model."""
    dec = getattr(model, "_ade_graph_decoder", None)
    if dec is None:
        dec = model._ade_graph_decoder = GreedyGraphDecoder(model)
    return dec.generate(input_ids, max_new_tokens, **kw)
