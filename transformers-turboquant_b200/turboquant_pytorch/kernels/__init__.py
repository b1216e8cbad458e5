"""Import-name compatibility for `turboquant_pytorch.kernels`."""
from turboquant_b200.kernels import (asymmetric_attention_scores, lloyd_max_dequantize, lloyd_max_quantize,  # noqa: F401
                                     pack_bits, unpack_bits)

__all__ = ["pack_bits", "unpack_bits", "lloyd_max_quantize", "lloyd_max_dequantize", "asymmetric_attention_scores"]
