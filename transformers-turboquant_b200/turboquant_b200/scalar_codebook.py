"""Standalone Lloyd-Max codebook API of the reference (src/turboquant_pytorch/lloyd_max.py:18-171) on the
GPU wire-format kernels: `solve_lloyd_max`, `compute_expected_distortion`, `LloydMaxCodebook`.

The solver differs from the compressors' one (codebook.py) in three details that the reference's two files
also differ in, and that are kept so that values agree to the bit: the variance enters as 1/d, the iterate
kept is the one AFTER the last update, and the boundaries are fp64 midpoints rounded to fp32 once.
"""

from __future__ import annotations

import math

import torch


def beta_pdf(x: float, d: int) -> float:
    """Exact density of one coordinate of a uniformly random unit vector in R^d (lloyd_max.py:18-23)."""
    if abs(x) >= 1.0:
        return 0.0
    norm = math.gamma(d / 2) / (math.sqrt(math.pi) * math.gamma((d - 1) / 2))
    return norm * (1 - x * x) ** ((d - 3) / 2)


def gaussian_approx_pdf(x: float, d: int) -> float:
    """N(0, 1/d), the large-d limit of beta_pdf (lloyd_max.py:26-29)."""
    var = 1.0 / d
    return (1.0 / math.sqrt(2 * math.pi * var)) * math.exp(-x * x / (2 * var))


def _pdf(d: int, use_exact: bool):
    return (lambda x: beta_pdf(x, d)) if use_exact else (lambda x: gaussian_approx_pdf(x, d))


def solve_lloyd_max(d: int, bits: int, use_exact: bool = False, max_iter: int = 200, tol: float = 1e-10):
    """(centroids fp32 [2^bits], boundaries fp32 [2^bits - 1]) of the MSE-optimal scalar quantiser for the
    coordinate law; fixed-point iteration of lloyd_max.py:32-86."""
    from scipy.integrate import quad

    pdf = _pdf(d, use_exact)
    levels = 1 << bits
    sigma = 1.0 / math.sqrt(d)
    lo, hi = -3.5 * sigma, 3.5 * sigma
    cur = [lo + (hi - lo) * (k + 0.5) / levels for k in range(levels)]
    for _ in range(max_iter):
        cuts = [3 * lo, *((a + b) / 2.0 for a, b in zip(cur, cur[1:])), 3 * hi]
        nxt = []
        for k in range(levels):
            mass = quad(pdf, cuts[k], cuts[k + 1])[0]
            moment = quad(lambda x: x * pdf(x), cuts[k], cuts[k + 1])[0]
            nxt.append(moment / mass if mass > 1e-15 else cur[k])
        moved = max(abs(n - c) for n, c in zip(nxt, cur))
        cur = nxt
        if moved < tol:
            break
    mids = [(a + b) / 2.0 for a, b in zip(cur, cur[1:])]
    return torch.tensor(cur, dtype=torch.float32), torch.tensor(mids, dtype=torch.float32)


def compute_expected_distortion(d: int, bits: int, centroids: torch.Tensor, boundaries: torch.Tensor,
                                use_exact: bool = False) -> float:
    """Expected squared error per coordinate of the quantiser (lloyd_max.py:89-104)."""
    from scipy.integrate import quad

    pdf = _pdf(d, use_exact)
    sigma = 1.0 / math.sqrt(d)
    cuts = [-3.5 * sigma * 3, *boundaries.tolist(), 3.5 * sigma * 3]
    total = 0.0
    for k in range(1 << bits):
        c = centroids[k].item()
        total += quad(lambda x: (x - c) ** 2 * pdf(x), cuts[k], cuts[k + 1])[0]
    return total


class LloydMaxCodebook:
    """Codebook for (d, bits) with `quantize` / `dequantize` (lloyd_max.py:107-171).

    CUDA inputs go through the packed wire format, as the reference's kernel path does: `quantize` returns
    uint8 [N, d*bits/8] and `dequantize` takes it back to fp16 centroid values [N, d].  CPU tensors keep the
    reference's fallback semantics (integer indices in, centroid values out) — a host-side convenience of a
    few tensor ops, not a compute path.
    """

    def __init__(self, d: int, bits: int, use_exact: bool = False, use_triton: bool = True):
        self.d, self.bits, self.n_levels = d, bits, 1 << bits
        self.use_triton = use_triton  # kept for signature compatibility: CUDA tensors always use the kernels
        self.centroids, self.boundaries = solve_lloyd_max(d, bits, use_exact)
        self.distortion = compute_expected_distortion(d, bits, self.centroids, self.boundaries, use_exact)

    def quantize(self, x: torch.Tensor) -> torch.Tensor:
        if x.is_cuda:
            from .kernels import lloyd_max_quantize
            return lloyd_max_quantize(x.reshape(-1, self.d).float(), self.boundaries.to(x.device), self.bits)
        return (x.unsqueeze(-1) - self.centroids).abs().argmin(dim=-1)

    def dequantize(self, indices: torch.Tensor) -> torch.Tensor:
        if indices.is_cuda:
            from .kernels import lloyd_max_dequantize
            return lloyd_max_dequantize(indices, self.centroids.half().to(indices.device), self.bits, self.d)
        return self.centroids[indices]

    def __repr__(self) -> str:
        return (f"LloydMaxCodebook(d={self.d}, bits={self.bits}, levels={self.n_levels}, "
                f"distortion_per_coord={self.distortion:.6f}, use_triton={self.use_triton})")
