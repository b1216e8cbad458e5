"""Import-name compatibility for `turboquant_pytorch.lloyd_max`."""
from turboquant_b200.scalar_codebook import (LloydMaxCodebook, beta_pdf, compute_expected_distortion,  # noqa: F401
                                       gaussian_approx_pdf, solve_lloyd_max)
