"""turboquant_b200: TurboQuant KV compression + compressed attention on B200 (sm_100a).

    from turboquant_b200 import apply_turboquant
    model = apply_turboquant(model.cuda(), bits=3, seed=42)
"""
from . import _lib  # noqa: F401  (fails loudly when the CUDA library is missing)
from .compressors import (TurboQuantCompressorMSE, TurboQuantCompressorV2, compress_kv, device_fault_count,
                          fused_attention, prepared_constants)
from .plugin import (TurboQuantAttentionBase, UnsupportedModelError, apply_turboquant,
                     get_attention_class, register_family)
from . import families  # noqa: F401,E402  (registers the adapters)
from .kernels import (asymmetric_attention_scores, lloyd_max_dequantize, lloyd_max_quantize,  # noqa: E402
                      pack_bits, unpack_bits)
from .scalar_codebook import LloydMaxCodebook, solve_lloyd_max  # noqa: E402
from .quantizers import TurboQuantKVCache, TurboQuantMSE, TurboQuantProd  # noqa: E402
from .kv_cache import CompressedKVCache  # noqa: E402
from .rotary import rope  # noqa: E402

__version__ = "0.1.0"
__all__ = ["apply_turboquant", "register_family", "get_attention_class", "UnsupportedModelError",
           "TurboQuantAttentionBase", "TurboQuantCompressorV2", "TurboQuantCompressorMSE",
           "fused_attention", "compress_kv", "prepared_constants", "rope", "device_fault_count", "pack_bits",
           "unpack_bits", "lloyd_max_quantize", "lloyd_max_dequantize", "asymmetric_attention_scores", "LloydMaxCodebook", "solve_lloyd_max",
           "TurboQuantMSE", "TurboQuantProd", "TurboQuantKVCache", "CompressedKVCache"]
