"""Serving boundary: the delta-linear module the Hugging Face forward calls.

Keeps the API of the reference's ``src/serving.py`` -- ``ADEKernelLinear(W_b, packed, group_size,
decode_max_tokens, use_decode, use_recon, split_k)`` with ``forward(x)`` and the attributes
``out_features / in_features / weight``, and ``build_kernel_model`` -- on top of the B200 kernels.
Differences: tensors are bfloat16 (the reference module is float16), there is no float
fallback (``use_decode`` / ``use_recon`` = False raise), and for T <= decode_max_tokens the base
GEMM x W_b^T runs inside the factored kernel instead of a separate ``F.linear``.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .kernels import (GROUP, STORED_KEYS, decode_kernel_status, factored_forward, pack_int4, recon_int4,
                      recon_kernel_status)

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
        if T <= self.decode_max_tokens:
            y = factored_forward(x2, self._stored_form(), weight=self.weight)
        else:
            y = F.linear(x2, self.merged_weight())
        return y.reshape(*shape[:-1], self.out_features)


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
