"""Standalone quantisers of the reference (src/turboquant_pytorch/turboquant.py:18-286) on the GPU
wire-format kernels: `TurboQuantMSE` (rotate + Lloyd-Max), `TurboQuantProd` (MSE with bits-1 bits plus the
1-bit QJL sketch of the residual, unbiased inner products) and `TurboQuantKVCache`.

These classes quantise vectors AS GIVEN (no per-vector norm, QJL matrix from seed+1, residual in the
original coordinates), unlike the attention compressors.  The per-coordinate work (boundary search, bit
packing, centroid look-up) runs in the library's kernels; the d x d rotations and sketches are torch
matmuls on the same device.  CUDA only.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
from torch import nn

from .kernels import lloyd_max_dequantize, lloyd_max_quantize, unpack_bits
from .lloyd_max import LloydMaxCodebook


def generate_rotation_matrix(d: int, seed: Optional[int] = None, device: str = "cuda") -> torch.Tensor:
    """Haar rotation: Q of a seeded Gaussian matrix with the signs of diag(R) folded in (turboquant.py:18-33).
    Drawn on the CPU generator so that a seed means the same matrix everywhere."""
    g = torch.Generator(device="cpu")
    if seed is not None:
        g.manual_seed(seed)
    q, r = torch.linalg.qr(torch.randn(d, d, generator=g))
    s = torch.sign(torch.diag(r))
    s[s == 0] = 1.0
    return (q * s.unsqueeze(0)).contiguous().to(device)


def generate_qjl_matrix(d: int, m: Optional[int] = None, seed: Optional[int] = None, device: str = "cuda") -> torch.Tensor:
    """i.i.d. N(0, 1) sketch matrix [m, d], m = d by default (turboquant.py:36-48)."""
    g = torch.Generator(device="cpu")
    if seed is not None:
        g.manual_seed(seed)
    return torch.randn(m or d, d, generator=g).to(device)


def _need_cuda(t: torch.Tensor) -> None:
    if not t.is_cuda:
        raise RuntimeError("turboquant_b200 quantisers run on CUDA tensors only (there is no CPU path)")


class TurboQuantMSE(nn.Module):
    """y = x Pi^T, nearest Lloyd-Max centroid per coordinate (turboquant.py:51-100)."""

    def __init__(self, d: int, bits: int, seed: int = 42, device: str = "cuda"):
        super().__init__()
        self.d, self.bits, self.device = d, bits, device
        self.register_buffer("Pi", generate_rotation_matrix(d, seed=seed, device=device))
        self.codebook = LloydMaxCodebook(d, bits)
        self.register_buffer("centroids", self.codebook.centroids.to(device))
        self.register_buffer("boundaries", self.codebook.boundaries.to(device))

    def rotate(self, x: torch.Tensor) -> torch.Tensor:
        return x @ self.Pi.T

    def unrotate(self, y: torch.Tensor) -> torch.Tensor:
        return y @ self.Pi

    def quantize(self, x: torch.Tensor) -> torch.Tensor:
        """Integer indices, shape of x (the reference's contract); the packed form is `quantize_packed`."""
        packed = self.quantize_packed(x)
        return unpack_bits(packed, self.bits, self.d).to(torch.int64).reshape(x.shape)

    def quantize_packed(self, x: torch.Tensor) -> torch.Tensor:
        """uint8 [N, d*bits/8] in the library's wire format."""
        _need_cuda(x)
        y = self.rotate(x.float()).reshape(-1, self.d)
        return lloyd_max_quantize(y, self.boundaries, self.bits)

    def dequantize(self, indices: torch.Tensor) -> torch.Tensor:
        """Indices (integer, shape [..., d]) or packed bytes (uint8 [N, d*bits/8]) -> vectors."""
        _need_cuda(indices)
        if indices.dtype == torch.uint8 and indices.shape[-1] == self.d * self.bits // 8 and self.bits != 8:
            y_hat = lloyd_max_dequantize(indices.reshape(-1, indices.shape[-1]), self.centroids, self.bits, self.d)
        else:
            y_hat = self.centroids[indices]
        return self.unrotate(y_hat)

    def forward(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        idx = self.quantize(x)
        return self.dequantize(idx), idx


class TurboQuantProd(nn.Module):
    """(bits-1)-bit MSE quantiser + 1-bit QJL sketch of the residual; `inner_product` is unbiased
    (turboquant.py:103-196)."""

    def __init__(self, d: int, bits: int, qjl_dim: Optional[int] = None, seed: int = 42, device: str = "cuda"):
        super().__init__()
        self.d, self.bits, self.device = d, bits, device
        self.mse_bits = max(bits - 1, 1)
        self.qjl_dim = qjl_dim or d
        self.mse = TurboQuantMSE(d, self.mse_bits, seed=seed, device=device)
        self.register_buffer("S", generate_qjl_matrix(d, m=self.qjl_dim, seed=seed + 1, device=device))

    def quantize(self, x: torch.Tensor) -> dict:
        x_hat, idx = self.mse(x)
        r = x - x_hat
        signs = torch.sign(r @ self.S.T)
        signs[signs == 0] = 1.0
        return {"mse_indices": idx, "qjl_signs": signs, "residual_norm": torch.norm(r, dim=-1)}

    def dequantize(self, compressed: dict) -> torch.Tensor:
        return self.mse.dequantize(compressed["mse_indices"])

    def inner_product(self, y: torch.Tensor, compressed: dict) -> torch.Tensor:
        """<y, x_mse> + ||r|| sqrt(pi/2)/m <S y, signs>."""
        first = (y * self.mse.dequantize(compressed["mse_indices"])).sum(dim=-1)
        sketch = ((y @ self.S.T) * compressed["qjl_signs"]).sum(dim=-1)
        return first + compressed["residual_norm"] * (math.sqrt(math.pi / 2) / self.qjl_dim) * sketch

    def forward(self, x: torch.Tensor) -> dict:
        return self.quantize(x)


class TurboQuantKVCache:
    """Append-only compressed key / value store with estimator scores (turboquant.py:199-286)."""

    def __init__(self, d_key: int, d_value: int, bits: int = 3, seed: int = 42, device: str = "cuda"):
        self.d_key, self.d_value, self.bits, self.device = d_key, d_value, bits, device
        self.key_quantizer = TurboQuantProd(d_key, bits, seed=seed, device=device)
        self.value_quantizer = TurboQuantMSE(d_value, bits, seed=seed + 100, device=device)
        self.key_cache: list = []
        self.value_cache: list = []

    def append(self, keys: torch.Tensor, values: torch.Tensor) -> None:
        ck = self.key_quantizer.quantize(keys.reshape(-1, self.d_key))
        self.key_cache.append({**ck, "shape": keys.shape})
        self.value_cache.append({"indices": self.value_quantizer.quantize(values.reshape(-1, self.d_value)),
                                 "shape": values.shape})

    def attention_scores(self, queries: torch.Tensor) -> torch.Tensor:
        parts = [self.key_quantizer.inner_product(queries, c) for c in self.key_cache]
        return torch.cat(parts, dim=-1) if parts else torch.tensor([])

    def get_values(self) -> torch.Tensor:
        parts = [self.value_quantizer.dequantize(c["indices"]) for c in self.value_cache]
        return torch.cat(parts, dim=0) if parts else torch.tensor([])

    def memory_usage_bits(self) -> dict:
        n_idx = sum(c["mse_indices"].numel() for c in self.key_cache)
        n_sgn = sum(c["qjl_signs"].numel() for c in self.key_cache)
        n_nrm = sum(c["residual_norm"].numel() for c in self.key_cache)
        n_val = sum(c["indices"].numel() for c in self.value_cache)
        key_bits = n_idx * self.key_quantizer.mse_bits + n_sgn + 16 * n_nrm
        val_bits = n_val * self.bits
        fp16 = 16 * (n_idx + n_val)
        total = key_bits + val_bits
        return {"key_bits": key_bits, "value_bits": val_bits, "total_bits": total, "fp16_bits": fp16,
                "compression_ratio": fp16 / total if total else 0}

    def __len__(self) -> int:
        return sum(c["mse_indices"].shape[0] for c in self.key_cache)
