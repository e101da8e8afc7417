"""Fused elementwise operations of a LLaMA decoder layer for the token-by-token decode step.

``enable_fused_decode_ops(model)`` swaps pieces of a transformers LLaMA model for single CUDA launches of the C
ABI: RMSNorm (``ade_b200_rmsnorm``), the rotary position embedding of q and k (``ade_b200_rope``), SiLU(gate) * up
(``ade_b200_silu_mul``) and, for single-token steps on a static KV cache, the whole attention step: rotary embedding,
cache write and attention (``ade_b200_attn_decode``).  The arithmetic and the bfloat16 roundings of the first three
are those of the torch operations they replace, so the logits do not move; the attention step keeps scores and
sums in float32 where torch's fused attention rounds the probabilities to bfloat16, a difference below the
tolerance of the path.  What changes is the number of kernels per token (about sixty per layer fewer), which at
decode sizes is what the time outside the delta application consists of.  They apply to small inputs only (at most
``MAX_ROWS`` token rows); longer inputs, other dtypes and CPU tensors take the original code.

The reference has no counterpart: it generates with ``model.generate`` of transformers (src/evaluate.py:241).
"""
from __future__ import annotations

import torch

from . import _lib

MAX_ROWS = 512          # token rows (batch * sequence) up to which the fused kernels are used


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _rows_ok(t: torch.Tensor, rows: int) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16 and 0 < rows <= MAX_ROWS


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """LlamaRMSNorm.forward for a bfloat16 CUDA tensor whose last dimension is contiguous."""
    H = x.shape[-1]
    x2 = x.reshape(-1, H)
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    out = torch.empty((x2.shape[0], H), dtype=torch.bfloat16, device=x.device)
    _lib.check(_lib.load().ade_b200_rmsnorm(x2.data_ptr(), weight.data_ptr(), out.data_ptr(), x2.shape[0], H, x2.stride(0), float(eps),
                                            _stream()), "ade_b200_rmsnorm")
    return out.view(x.shape)


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float):
    """(residual + x, LlamaRMSNorm(residual + x)) in one launch: the residual connection of a decoder layer and the
    normalisation that follows it.  Both inputs bfloat16 CUDA with a contiguous last dimension."""
    H = x.shape[-1]
    x2, r2 = x.reshape(-1, H), residual.reshape(-1, H)
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    if r2.stride(1) != 1:
        r2 = r2.contiguous()
    total = torch.empty((x2.shape[0], H), dtype=torch.bfloat16, device=x.device)
    out = torch.empty_like(total)
    _lib.check(_lib.load().ade_b200_add_rmsnorm(x2.data_ptr(), r2.data_ptr(), weight.data_ptr(), total.data_ptr(), out.data_ptr(), x2.shape[0], H,
                                                x2.stride(0), r2.stride(0), float(eps), _stream()), "ade_b200_add_rmsnorm")
    return total.view(x.shape), out.view(x.shape)


def rope(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
    """apply_rotary_pos_emb for q (B, heads, T, hd) and k given as transposed views of (B, T, heads, hd) projections;
    returns contiguous (B, heads, T, hd) tensors."""
    B, hq, T, hd = q.shape
    hk = k.shape[1]
    qo = torch.empty((B, hq, T, hd), dtype=torch.bfloat16, device=q.device)
    ko = torch.empty((B, hk, T, hd), dtype=torch.bfloat16, device=q.device)
    cs_stride = 0 if cos.shape[0] == 1 else T * hd
    # distance between consecutive (batch, token) rows of the projection; a dimension of size 1 reports an arbitrary stride
    rq = q.stride(2) if T > 1 else q.stride(0)
    rk = k.stride(2) if T > 1 else k.stride(0)
    _lib.check(_lib.load().ade_b200_rope(q.data_ptr(), k.data_ptr(), cos.data_ptr(), sin.data_ptr(), qo.data_ptr(), ko.data_ptr(), B, T, hq, hk,
                                         hd, rq, rk, cs_stride, _stream()), "ade_b200_rope")
    return qo, ko


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """act_fn(gate) * up for SiLU, bfloat16, last dimension contiguous (row strides free)."""
    cols = gate.shape[-1]
    g2, u2 = gate.reshape(-1, cols), up.reshape(-1, cols)
    out = torch.empty((g2.shape[0], cols), dtype=torch.bfloat16, device=gate.device)
    _lib.check(_lib.load().ade_b200_silu_mul(g2.data_ptr(), u2.data_ptr(), out.data_ptr(), g2.shape[0], cols, g2.stride(0), u2.stride(0),
                                             _stream()), "ade_b200_silu_mul")
    return out.view(*gate.shape[:-1], cols)


def attn_decode(q, k, v, cos, sin, mask, layer, scale: float) -> torch.Tensor:
    """Single-token attention step on a static cache layer: q (B, 1, hq*hd), k / v (B, 1, hk*hd) straight from the
    projections, cos / sin (B or 1, 1, hd), mask None or bool (B, 1, 1, L).  Writes k, v into the layer's cache at its
    running position, advances that position (inside the same launch), returns (B, 1, hq*hd)."""
    B = q.shape[0]
    hk, L, hd = layer.keys.shape[1], layer.keys.shape[2], layer.keys.shape[3]
    hq = q.shape[-1] // hd
    out = torch.empty((B, 1, hq * hd), dtype=torch.bfloat16, device=q.device)
    row = lambda t: t.stride(0) if B > 1 else t.shape[-1]
    ticket = getattr(layer, "_ade_ticket", None)           # counter through which the launch advances the position itself
    if ticket is None or ticket.device != q.device:
        ticket = layer._ade_ticket = torch.zeros(1, dtype=torch.int32, device=q.device)
    _lib.check(_lib.load().ade_b200_attn_decode(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), cos.data_ptr(), sin.data_ptr(), None if mask is None else mask.data_ptr(),
        layer.keys.data_ptr(), layer.values.data_ptr(), layer.cumulative_length.data_ptr(), ticket.data_ptr(), out.data_ptr(), B, hq, hk, hd, L,
        row(q), row(k), row(v), 0 if cos.shape[0] == 1 else hd, 0 if mask is None else mask.stride(0), float(scale), _stream()),
        "ade_b200_attn_decode")
    return out


def _attn_decode_ok(mod, x, cos, mask, layer) -> bool:
    if not (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 3 and x.shape[1] == 1 and not mod.training):
        return False
    if type(layer).__name__ != "StaticLayer" or not getattr(layer, "is_initialized", False):
        return False
    kc = layer.keys
    if not (kc.dtype == torch.bfloat16 and kc.is_contiguous() and layer.values.is_contiguous() and kc.shape[0] == x.shape[0]):
        return False
    hd = kc.shape[3]
    if hd % 32 or hd > 256 or (7 * hd + kc.shape[2]) * 4 > 48 * 1024 or layer.cumulative_length.dtype != torch.int64:
        return False
    if not (cos.dtype == torch.bfloat16 and cos.dim() == 3 and cos.shape[1] == 1 and cos.is_contiguous() and cos.shape[0] in (1, x.shape[0])):
        return False
    if mask is not None and not (mask.dtype == torch.bool and mask.dim() == 4 and mask.shape[1] == 1 and mask.shape[2] == 1
                                 and mask.shape[3] == kc.shape[2] and mask.stride(3) == 1 and mask.shape[0] == x.shape[0]):
        return False
    return True


def _rope_layout_ok(x: torch.Tensor) -> bool:
    """(B, heads, T, hd) view of a (B, T, heads, hd) projection: head_dim contiguous, heads hd apart, batch rows T apart."""
    B, h, T, hd = x.shape
    return x.stride(3) == 1 and (h == 1 or x.stride(1) == hd) and (B == 1 or T == 1 or x.stride(0) == T * x.stride(2))


def enable_fused_decode_ops(model) -> int:
    """Patch `model` (a transformers LLaMA-architecture causal LM) in place; returns the number of modules patched.
    The rotary embedding is a module-level function of transformers' LLaMA implementation, so that patch is
    process-wide (it falls back to the original for anything but small bfloat16 CUDA inputs)."""
    from transformers.models.llama import modeling_llama as ml

    if not getattr(ml, "_ade_rope_patched", False):
        original = ml.apply_rotary_pos_emb

        def apply_rotary_pos_emb(q, k, cos, sin, unsqueeze_dim=1):
            if (unsqueeze_dim == 1 and q.dim() == 4 and _rows_ok(q, q.shape[0] * q.shape[2]) and k.dtype == torch.bfloat16
                    and cos.dtype == torch.bfloat16 and cos.dim() == 3 and cos.is_contiguous() and sin.is_contiguous()
                    and cos.shape[0] in (1, q.shape[0]) and _rope_layout_ok(q) and _rope_layout_ok(k)):
                return rope(q, k, cos, sin)
            return original(q, k, cos, sin, unsqueeze_dim)

        ml.apply_rotary_pos_emb = apply_rotary_pos_emb
        ml._ade_rope_patched = True
    n = 0
    for mod in model.modules():
        if isinstance(mod, ml.LlamaAttention) and not hasattr(mod, "_ade_orig_forward"):
            mod._ade_orig_forward = mod.forward

            def attn_forward(hidden_states, position_embeddings=None, attention_mask=None, past_key_values=None, mod=mod, **kw):
                layers = getattr(past_key_values, "layers", None)
                layer = layers[mod.layer_idx] if layers is not None and mod.layer_idx < len(layers) else None
                if (position_embeddings is not None and layer is not None
                        and _attn_decode_ok(mod, hidden_states, position_embeddings[0], attention_mask, layer)):
                    q, k, v = mod.q_proj(hidden_states), mod.k_proj(hidden_states), mod.v_proj(hidden_states)
                    if all(t.dtype == torch.bfloat16 and t.stride(-1) == 1 for t in (q, k, v)) and position_embeddings[1].is_contiguous():
                        ctx = attn_decode(q, k, v, position_embeddings[0], position_embeddings[1], attention_mask, layer, mod.scaling)
                        return mod.o_proj(ctx), None
                return mod._ade_orig_forward(hidden_states, position_embeddings=position_embeddings, attention_mask=attention_mask,
                                             past_key_values=past_key_values, **kw)

            mod.forward = attn_forward
            n += 1
        elif isinstance(mod, ml.LlamaRMSNorm) and not hasattr(mod, "_ade_orig_forward"):
            mod._ade_orig_forward = mod.forward

            mod._ade_pre = None                   # (input tensor, its normalisation) left by the layer in front, see below

            def norm_forward(x, mod=mod):
                pre = mod._ade_pre
                if pre is not None:
                    mod._ade_pre = None
                    if x is pre[0]:
                        return pre[1]
                if _rows_ok(x, x.numel() // x.shape[-1]) and x.stride(-1) == 1 and mod.weight.dtype == torch.bfloat16:
                    return rmsnorm(x, mod.weight, mod.variance_epsilon)
                return mod._ade_orig_forward(x)

            mod.forward = norm_forward
            n += 1
        elif (isinstance(mod, ml.LlamaMLP) and not hasattr(mod, "_ade_orig_forward")
              and type(mod.act_fn).__name__ in ("SiLU", "SiLUActivation")):
            mod._ade_orig_forward = mod.forward

            def mlp_forward(x, mod=mod):
                if _rows_ok(x, x.numel() // x.shape[-1]):
                    g, u = mod.gate_proj(x), mod.up_proj(x)
                    if g.dtype == torch.bfloat16 and g.stride(-1) == 1 and u.stride(-1) == 1:
                        return mod.down_proj(silu_mul(g, u))
                    return mod.down_proj(mod.act_fn(g) * u)
                return mod._ade_orig_forward(x)

            mod.forward = mlp_forward
            n += 1
    # Residual connections: a decoder layer adds the attention output and the MLP output to its input, each time right in
    # front of an RMSNorm (its own post-attention norm; the next layer's input norm, or the model's final norm).  A
    # patched layer does add + norm in one launch each and leaves the second normalisation with the norm module that is
    # about to be asked for it, which recognises the tensor by identity.
    for lm in model.modules():
        if not isinstance(lm, ml.LlamaModel):
            continue
        layers = list(lm.layers[: lm.config.num_hidden_layers])
        for i, layer in enumerate(layers):
            if hasattr(layer, "_ade_orig_forward") or not isinstance(layer, ml.LlamaDecoderLayer):
                continue
            nxt = layers[i + 1].input_layernorm if i + 1 < len(layers) else lm.norm
            if not all(hasattr(nm, "_ade_pre") for nm in (layer.input_layernorm, layer.post_attention_layernorm, nxt)):
                continue
            layer._ade_orig_forward = layer.forward

            def layer_forward(hidden_states, attention_mask=None, position_ids=None, past_key_values=None, use_cache=False,
                              position_embeddings=None, layer=layer, nxt=nxt, **kw):
                post = layer.post_attention_layernorm
                if not (_rows_ok(hidden_states, hidden_states.numel() // hidden_states.shape[-1]) and hidden_states.is_contiguous()
                        and post.weight.dtype == torch.bfloat16 and nxt.weight.dtype == torch.bfloat16 and not layer.training):
                    return layer._ade_orig_forward(hidden_states, attention_mask=attention_mask, position_ids=position_ids,
                                                   past_key_values=past_key_values, use_cache=use_cache,
                                                   position_embeddings=position_embeddings, **kw)
                h = layer.input_layernorm(hidden_states)
                a, _ = layer.self_attn(hidden_states=h, attention_mask=attention_mask, position_ids=position_ids,
                                       past_key_values=past_key_values, use_cache=use_cache, position_embeddings=position_embeddings, **kw)
                s1, h2 = add_rmsnorm(a, hidden_states, post.weight, post.variance_epsilon)
                m = layer.mlp(h2)
                s2, h3 = add_rmsnorm(m, s1, nxt.weight, nxt.variance_epsilon)
                nxt._ade_pre = (s2, h3)
                return s2

            layer.forward = layer_forward
            n += 1
    return n
