"""Lloyd-Max codebook for N(0, 1/d), the coordinate law of a randomly rotated unit vector.

Host-side, one-off per compressor.  The fixed-point iteration, its start, its cell edges
and its stopping rule are those of the reference (src/turboquant_pytorch/compressors.py:72-96):
uniform start in +-3.5 sigma, outer edges at +-10.5 sigma, stop when no centroid moves by
1e-10, keep the iterate *before* the final update, at most 200 sweeps.  The conditional
means are evaluated with the same adaptive quadrature so that the fp32 values agree to the
bit with the reference's.
"""

from __future__ import annotations

import functools
import math

import torch


@functools.lru_cache(maxsize=None)
def _centroids(d: int, bits: int) -> tuple[float, ...]:
    from scipy.integrate import quad

    levels = 1 << bits
    sigma = 1.0 / math.sqrt(d)
    scale = 1.0 / math.sqrt(2 * math.pi * sigma ** 2)
    two_var = 2 * sigma ** 2

    def pdf(x: float) -> float:
        return scale * math.exp(-x * x / two_var)

    def xpdf(x: float) -> float:
        return x * pdf(x)

    lo, hi = -3.5 * sigma, 3.5 * sigma
    width = hi - lo
    current = [lo + width * (k + 0.5) / levels for k in range(levels)]
    for _sweep in range(200):
        edges = [3 * lo, *((a + b) / 2.0 for a, b in zip(current, current[1:])), 3 * hi]
        proposal = []
        for k, (a, b) in enumerate(zip(edges, edges[1:])):
            mean_num = quad(xpdf, a, b)[0]
            mass = quad(pdf, a, b)[0]
            proposal.append(mean_num / mass if mass > 1e-15 else current[k])
        if max(abs(p - c) for p, c in zip(proposal, current)) < 1e-10:
            break
        current = proposal
    return tuple(current)


def lloyd_max_centroids(d: int, bits: int) -> torch.Tensor:
    """fp32 tensor of 2**bits ascending centroids."""
    return torch.tensor(_centroids(d, bits), dtype=torch.float32)


def midpoints(centroids: torch.Tensor) -> torch.Tensor:
    """Decision boundaries: fp32 midpoints of neighbouring centroids (compressors.py:62)."""
    return (centroids[:-1] + centroids[1:]) / 2
