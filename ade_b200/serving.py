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

from .kernels import (GROUP, STORED_KEYS, decode_forward_packed, decode_kernel_status, factored_forward, pack_int4,
                      recon_int4, recon_kernel_status)

# Up to this many tokens the base GEMM x W_b^T runs inside the factored kernel (one launch, W_b streamed once by
# a kernel built for skinny operands, h computed by side warps under the stream).  Above it cuBLAS is faster at the
# base term, so the module falls back to the reference's split: F.linear for the base, the kernel for the delta
# only (measured on B200 per call, fused / split: 4096 x 4096 T = 16 14.5 / 21.0 us, T = 32 22.4 / 23.7, T = 64
# 46.3 / 29.2; 11008 x 4096 T = 16 30.1 / 34.0, T = 24 40.6 / 39.2, T = 64 117.6 / 55.9).
FUSED_BASE_MAX_TOKENS = 16

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
                 split_k: bool = False):
        """
        Parameters:
            W_b: Base weight (d_o, d_i).
            packed: Packed factors of the module (src/quantization.py:276-285 layout).
            group_size: Group size G (128).
            decode_max_tokens: Largest T handled by factored application (at most 128).
            use_decode / use_recon: must stay True; there is no float reconstruction fallback.
            split_k: accepted for compatibility, ignored (the kernels are deterministic).
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
        self.register_buffer("weight", W_b.detach().to(torch.bfloat16).contiguous())
        p4 = pack_int4(packed, group_size)
        self._dims = (p4["M"], p4["N"], p4["r"])
        for k in STORED_KEYS:
            self.register_buffer(f"p4_{k}", p4[k])
        self._p4 = None
        self._group = None            # (FusedADEGroup, index) once fuse_kernel_linears has grouped this module

    def _stored_form(self) -> dict:
        """Stored form on the module's device (rebuilt after .to(device))."""
        if self._p4 is None or self._p4["uq"].data_ptr() != self.p4_uq.data_ptr():
            self._p4 = {k: getattr(self, f"p4_{k}") for k in STORED_KEYS}
            self._p4["M"], self._p4["N"], self._p4["r"] = self._dims
        return self._p4

    def merged_weight(self) -> torch.Tensor:
        """bf16(W_b + U^ V^^T), one launch of the reconstruction kernel."""
        return recon_int4(self._stored_form(), self.weight, self.group_size)

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
        self._key = None
        self._y = None
        self._used = set()
        for i, m in enumerate(self.members):
            m._group = (self, i)

    def apply(self, index: int, x, x2):
        """Output of member `index` for the input x (x2 = x as a contiguous (T, d_i) bfloat16 matrix), or None when
        the group cannot serve it (the members moved to another device since the group was built)."""
        if self.members[0].weight.data_ptr() != self.weight.data_ptr():
            return None
        key = (x.data_ptr(), tuple(x.shape), x._version, x.dtype)
        if self._y is None or key != self._key or index in self._used:
            self._y = factored_forward(x2, self.p4, weight=self.weight)
            self._key = key
            self._used = set()
        self._used.add(index)
        y = self._y[:, self.offsets[index]:self.offsets[index + 1]]
        if len(self._used) == len(self.members):
            self._y = None                     # every member has taken its slice: nothing is served twice
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
    """Decoder layers of a LLaMA-family causal LM or of a llava-hf LLaVA model (src/serving.py:115-130)."""
    lm = getattr(getattr(model, "model", None), "language_model", None)
    if lm is None:
        lm = getattr(model, "language_model", None)
    if lm is not None:
        return getattr(lm, "model", lm).layers
    return model.model.layers


def attach_kernel_linears(model, base_state_dict: dict, per_module: dict, group_size: int = GROUP,
                          decode_max_tokens: int = 128, split_k: bool = False) -> int:
    """Replace every linear module that has a packed delta by an ADEKernelLinear, in place.

    The loop of src/serving.py:178-190 for a model that is already in memory: `base_state_dict`
    maps ``model.layers.<i>.<name>.weight`` to the base weight, `per_module` maps
    ``model.layers.<i>.<name>`` to its packed dict.  Returns the number of modules replaced.
    """
    layers = _decoder_layers(model)
    n = 0
    for li in range(len(layers)):
        for sn in LINEAR_MODULE_NAMES:
            prefix = f"model.layers.{li}.{sn}"
            if prefix not in per_module:
                continue
            parts = sn.split(".")
            parent = layers[li].get_submodule(".".join(parts[:-1]))
            setattr(parent, parts[-1], ADEKernelLinear(base_state_dict[prefix + ".weight"], per_module[prefix],
                                                       group_size, decode_max_tokens, split_k=split_k))
            n += 1
    return n


def build_kernel_model(task: str, aligned_path: str, base_path: str, packed_path: str,
                       llava_hf_path: str | None = None, device: str = "cuda",
                       decode_max_tokens: int = 128, split_k: bool = False):
    """bfloat16 evaluation model: the aligned model with every compressed linear module replaced
    by an ADEKernelLinear (same signature as src/serving.py:133-194).

    Raises when the kernels cannot run on `device`: the reference degrades to a PyTorch
    reconstruction there (src/serving.py:155-165), this build does not.
    """
    from transformers import AutoModelForCausalLM, AutoProcessor, AutoTokenizer

    from .packed_io import load_packed

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
    per_module, meta = load_packed(packed_path)
    n = attach_kernel_linears(model, base_sd, per_module, int(meta["group_size"]), decode_max_tokens, split_k)
    del base_sd, per_module
    model = model.to(device).eval()
    print(f"[kernels] {n} linear modules apply the compressed delta at every forward")
    return model, processor
