"""Import-name compatibility for `turboquant_pytorch.turboquant`."""
from turboquant_b200.quantizers import (TurboQuantKVCache, TurboQuantMSE, TurboQuantProd,  # noqa: F401
                                        generate_qjl_matrix, generate_rotation_matrix)
