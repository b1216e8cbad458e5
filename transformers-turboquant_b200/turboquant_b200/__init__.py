"""turboquant_b200: TurboQuant KV compression + compressed attention on B200 (sm_100a).

    from turboquant_b200 import apply_turboquant
    model = apply_turboquant(model.cuda(), bits=3, seed=42)
"""
from . import _lib  # noqa: F401  (fails loudly when the CUDA library is missing)
from .compressors import (TurboQuantCompressorMSE, TurboQuantCompressorV2, device_fault_count,
                          fused_attention)
from .plugin import (TurboQuantAttentionBase, UnsupportedModelError, apply_turboquant,
                     get_attention_class, register_family)
from . import families  # noqa: F401,E402  (registers the adapters)

__version__ = "0.1.0"
__all__ = ["apply_turboquant", "register_family", "get_attention_class", "UnsupportedModelError",
           "TurboQuantAttentionBase", "TurboQuantCompressorV2", "TurboQuantCompressorMSE",
           "fused_attention", "device_fault_count"]
