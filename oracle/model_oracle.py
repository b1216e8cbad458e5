"""Model-level checker (TEST INFRASTRUCTURE, CPU only): an HF model whose attention modules are replaced by
modules that keep the original projections and evaluate the attention core with `tq_oracle.attention_core`,
i.e. with the reference's arithmetic (src/transformers_turboquant/families/llama.py:79-122, gpt2.py:78-119),
layer by layer with the reference's seeds (patch.py:62-75: layer i compresses keys with seed+i and values with
seed+i+10000).

It fixes, on the checker's side only, what stops the reference's own adapters from running under
transformers 5: head counts are taken from the module's config, the 2-tuple the decoder layers unpack is
returned, and attention is causal whether or not HF hands over a mask.

Only tests/, __graft_entry__.smoke() and bench.py's CPU legs may import this module.
"""

from __future__ import annotations

import copy

import torch
import torch.nn as nn

from . import tq_oracle as orc


def additive_mask(attention_mask, T: int, Sk: int) -> torch.Tensor:
    """The mask an adapter receives from HF as an additive fp32 mask that always includes the causal rule.
    HF's eager path hands over an additive float mask (causal and padding already in it), its sdpa path a
    boolean one (True = visible) or nothing at all for a plain causal prefill."""
    causal = orc.causal_mask(T, Sk)
    if attention_mask is None:
        return causal
    m = attention_mask
    if m.dtype == torch.bool:
        m = torch.zeros(m.shape, dtype=torch.float32).masked_fill_(~m, torch.finfo(torch.float32).min)
    # finite large negatives plus -inf stay -inf; clamp so that two finite minima cannot overflow
    return torch.clamp(m.float() + causal, min=torch.finfo(torch.float32).min)


class OracleCore(nn.Module):
    """Stands in for one HF attention module on the CPU.  `kind` is "gpt2" (fused c_attn, no rotary) or
    "rope" (separate projections, rotary embeddings handed in as (cos, sin))."""

    def __init__(self, original: nn.Module, kind: str, layer: int, bits: int, seed: int, literal: bool = True):
        super().__init__()
        self.o, self.kind, self.literal = original, kind, literal
        ks, vs = orc.layer_seeds(seed, layer)
        d = original.head_dim
        self.kp, self.vp = orc.make_key_params(d, bits, ks), orc.make_value_params(d, bits, vs)
        self.record = None  # set to a dict to keep q, k, raw scores and the core's output of the last call

    def forward(self, hidden_states, position_embeddings=None, attention_mask=None, **kw):
        o = self.o
        B, T, _ = hidden_states.shape
        shp = (B, T, -1, o.head_dim)
        if self.kind == "gpt2":
            q, k, v = o.c_attn(hidden_states).split(o.embed_dim, dim=2)
            q, k, v = (t.view(shp).transpose(1, 2) for t in (q, k, v))
        else:
            from transformers.models.llama.modeling_llama import apply_rotary_pos_emb
            q = o.q_proj(hidden_states).view(shp).transpose(1, 2)
            k = o.k_proj(hidden_states).view(shp).transpose(1, 2)
            v = o.v_proj(hidden_states).view(shp).transpose(1, 2)
            q, k = apply_rotary_pos_emb(q, k, *position_embeddings)
        mask = additive_mask(attention_mask, T, T)
        out, raw = orc.attention_core(q, k, v, self.kp, self.vp, mask=mask, literal=self.literal)
        if self.record is not None:
            self.record.update(q=q.detach(), k=k.detach(), v=v.detach(), scores=raw.detach(), out=out.detach())
        out = out.transpose(1, 2).reshape(B, T, -1)
        return (o.c_proj(out) if self.kind == "gpt2" else o.o_proj(out)), None


def oracle_model(model: nn.Module, cls_name: str, kind: str, bits: int, seed: int, literal: bool = True):
    """A deep copy of `model` (on the CPU) with every module whose class is named `cls_name` replaced by an
    OracleCore, numbered in traversal order as apply_turboquant numbers its layers."""
    ref = copy.deepcopy(model)
    layer = 0
    for _, parent in list(ref.named_modules()):
        for name, child in list(parent.named_children()):
            if type(child).__name__ == cls_name:
                setattr(parent, name, OracleCore(child, kind, layer, bits, seed, literal))
                layer += 1
    if layer == 0:
        raise ValueError(f"no module of class {cls_name} found")
    return ref


def causal_score_cosine(estimate: torch.Tensor, exact: torch.Tensor) -> torch.Tensor:
    """Cosine similarity between estimated and exact raw scores over the causally visible entries (key <= query)
    of every head: [B, H, T, T] -> [B, H].  The reference's quality figure for the estimator is this value
    averaged over heads, per layer."""
    T = estimate.shape[-1]
    keep = torch.ones(T, T, dtype=torch.bool, device=estimate.device).tril()
    a = estimate.float().masked_fill(~keep, 0.0).flatten(-2)
    b = exact.float().masked_fill(~keep, 0.0).flatten(-2)
    return torch.nn.functional.cosine_similarity(a, b, dim=-1)


def logits_agreement(a: torch.Tensor, b: torch.Tensor) -> dict:
    """Norm-wise relative error of `a` against `b`, mean cosine per position and top-1 agreement."""
    a, b = a.double().cpu(), b.double().cpu()
    return {"rel_err": float((a - b).norm() / b.norm()),
            "cosine": float(torch.nn.functional.cosine_similarity(a, b, dim=-1).mean()),
            "top1": float((a.argmax(-1) == b.argmax(-1)).double().mean())}
