"""Import-name compatibility for `turboquant_pytorch` (same public names as the reference package)."""
from turboquant_b200.compressors import TurboQuantCompressorMSE, TurboQuantCompressorV2  # noqa: F401
from turboquant_b200.scalar_codebook import LloydMaxCodebook, solve_lloyd_max  # noqa: F401
from turboquant_b200.quantizers import TurboQuantKVCache, TurboQuantMSE, TurboQuantProd  # noqa: F401
