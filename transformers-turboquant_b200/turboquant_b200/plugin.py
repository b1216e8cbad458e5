"""Plugin API: family registry, adapter base class and `apply_turboquant`.

Same surface as the reference's `transformers_turboquant` package
(registry.py:5-38, base.py:14-39, patch.py:13-82): adapters register themselves for
`config.model_type` strings, declare which HF attention class names they replace, and
`apply_turboquant` swaps every matching module for an adapter that owns one key and one
value compressor seeded from (seed, layer index).
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Callable, ClassVar

import torch
import torch.nn as nn

from .compressors import TurboQuantCompressorMSE, TurboQuantCompressorV2

_REGISTRY: dict[str, type["TurboQuantAttentionBase"]] = {}


class UnsupportedModelError(ValueError):
    """`apply_turboquant` met a `model_type` no adapter is registered for."""


class TurboQuantAttentionBase(ABC, nn.Module):
    """Base of the attention replacements.  Subclasses list the HF class names they
    replace in ATTENTION_CLASS_NAMES, build themselves from the original module in
    `from_original` and run compressed attention in `forward`."""

    ATTENTION_CLASS_NAMES: ClassVar[tuple[str, ...]]

    key_compressor: TurboQuantCompressorV2
    val_compressor: TurboQuantCompressorMSE

    @classmethod
    @abstractmethod
    def from_original(cls, original: nn.Module, key_compressor: TurboQuantCompressorV2,
                      val_compressor: TurboQuantCompressorMSE) -> "TurboQuantAttentionBase":
        ...

    @abstractmethod
    def forward(self, hidden_states, **kwargs):
        ...

    def _apply(self, fn, recurse=True):
        """`.to()/.cuda()` also moves the compressors' constants.  They stay fp32
        whatever dtype the model is cast to: only the device of `fn` is honoured."""
        super()._apply(fn, recurse=recurse)
        for comp in (getattr(self, "key_compressor", None), getattr(self, "val_compressor", None)):
            if comp is not None:
                comp.to(fn(torch.empty(0, device=comp.Pi.device)).device)
        return self


def register_family(*model_types: str) -> Callable[[type], type]:
    """Class decorator: `@register_family("llama", "mistral")`."""

    def bind(cls):
        _REGISTRY.update({mt: cls for mt in model_types})
        return cls

    return bind


def get_attention_class(model_type: str) -> type[TurboQuantAttentionBase]:
    try:
        return _REGISTRY[model_type]
    except KeyError:
        raise UnsupportedModelError(
            f"model_type={model_type!r} is not supported. Supported: {sorted(_REGISTRY)}. "
            f"Add an adapter deriving from TurboQuantAttentionBase and decorate it with "
            f"@register_family({model_type!r}).") from None


def _head_dim_of(module: nn.Module, config) -> int:
    hd = getattr(module, "head_dim", None)
    if hd is None:
        hidden = getattr(config, "hidden_size", getattr(config, "n_embd", None))
        heads = getattr(config, "num_attention_heads", getattr(config, "n_head", None))
        hd = hidden // heads
    return int(hd)


def apply_turboquant(model, bits: int = 3, seed: int = 42, use_triton: bool = True,
                     kv_cache_capacity: int | None = None):
    """Replace every attention layer of a HF `PreTrainedModel` by its TurboQuant adapter,
    in place, and return the model.  Layer i (module traversal order) compresses keys with
    seed `seed + i` and values with `seed + i + 10000`; `config.use_cache` is switched off
    because the adapters recompute full-sequence attention (patch.py:13-82).
    `use_triton` is accepted for call compatibility and ignored.

    `kv_cache_capacity` (an extension; the reference has no such mode) keeps `use_cache` on
    instead: adapters that support it hold a `CompressedKVCache` of that many tokens per
    sequence, so that `generate()` compresses every token once and a decode step reads the
    packed cache in place."""
    adapter = get_attention_class(model.config.model_type)
    device = str(next(model.parameters()).device)
    layer = 0
    for _, parent in list(model.named_modules()):
        for name, child in list(parent.named_children()):
            if type(child).__name__ not in adapter.ATTENTION_CLASS_NAMES:
                continue
            hd = _head_dim_of(child, model.config)
            kc = TurboQuantCompressorV2(hd, bits, seed=seed + layer, device=device, use_triton=use_triton)
            vc = TurboQuantCompressorMSE(hd, bits, seed=seed + layer + 10000, device=device, use_triton=use_triton)
            new = adapter.from_original(child, kc, vc)
            if kv_cache_capacity is not None:
                if not getattr(new, "SUPPORTS_KV_CACHE", False):
                    raise UnsupportedModelError(f"{type(new).__name__} has no compressed-cache mode")
                new.kv_cache_capacity = int(kv_cache_capacity)
            setattr(parent, name, new)
            layer += 1
    model.config.use_cache = kv_cache_capacity is not None
    # generate() reads its own copy of the flag: left on, it would feed the cache-less adapters one token
    # at a time and every step would attend over that token alone
    gen_cfg = getattr(model, "generation_config", None)
    if gen_cfg is not None:
        gen_cfg.use_cache = model.config.use_cache
    return model
