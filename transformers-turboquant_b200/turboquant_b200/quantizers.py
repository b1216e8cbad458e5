"""Standalone vector quantisers with the reference's class names and call signatures
(src/turboquant_pytorch/turboquant.py:18-286): `TurboQuantMSE`, `TurboQuantProd`, `TurboQuantKVCache`.

Unlike the attention compressors these quantise a vector AS GIVEN: no per-vector norm is taken out, the
sketch matrix comes from seed + 1 and the residual lives in the original coordinates.  Per-coordinate work
(boundary search, bit packing, centroid look-up) runs in the library's wire-format kernels; the d x d
rotation and sketch products are torch matmuls on the same device.  CUDA tensors only.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
from torch import nn

from . import kernels as _k
from .scalar_codebook import LloydMaxCodebook

_SKETCH_GAIN = math.sqrt(math.pi / 2)


def _seeded(seed: Optional[int]) -> torch.Generator:
    g = torch.Generator(device="cpu")  # CPU generator: a seed means the same matrix on every machine
    return g.manual_seed(seed) if seed is not None else g


def generate_rotation_matrix(d: int, seed: Optional[int] = None, device: str = "cuda") -> torch.Tensor:
    """Haar-distributed rotation: the Q factor of a Gaussian matrix, columns flipped so that diag(R) > 0
    (turboquant.py:18-33)."""
    q, r = torch.linalg.qr(torch.randn(d, d, generator=_seeded(seed)))
    flip = torch.where(torch.diag(r) < 0, -1.0, 1.0)
    return (q * flip).contiguous().to(device)


def generate_qjl_matrix(d: int, m: Optional[int] = None, seed: Optional[int] = None, device: str = "cuda") -> torch.Tensor:
    """[m, d] sketch matrix of independent standard normals; m defaults to d (turboquant.py:36-48)."""
    return torch.randn(d if m is None else m, d, generator=_seeded(seed)).to(device)


def _on_gpu(t: torch.Tensor) -> torch.Tensor:
    if not t.is_cuda:
        raise RuntimeError("turboquant_b200 quantisers take CUDA tensors only (there is no CPU path)")
    return t


class TurboQuantMSE(nn.Module):
    """Rotate, then snap every coordinate to its Lloyd-Max centroid (turboquant.py:51-100)."""

    def __init__(self, d: int, bits: int, seed: int = 42, device: str = "cuda"):
        super().__init__()
        self.d, self.bits, self.device = d, bits, device
        self.codebook = LloydMaxCodebook(d, bits)
        for name, value in (("Pi", generate_rotation_matrix(d, seed, device)),
                            ("centroids", self.codebook.centroids.to(device)),
                            ("boundaries", self.codebook.boundaries.to(device))):
            self.register_buffer(name, value)

    # --- rotations (y = x Pi^T, x = y Pi) ---
    def rotate(self, x: torch.Tensor) -> torch.Tensor:
        return torch.matmul(x, self.Pi.transpose(0, 1))

    def unrotate(self, y: torch.Tensor) -> torch.Tensor:
        return torch.matmul(y, self.Pi)

    # --- quantise ---
    def quantize_packed(self, x: torch.Tensor) -> torch.Tensor:
        """Wire format: uint8 [N, d * bits / 8], LSB-first bit stream per vector."""
        rows = self.rotate(_on_gpu(x).float()).reshape(-1, self.d)
        return _k.lloyd_max_quantize(rows, self.boundaries, self.bits)

    def quantize(self, x: torch.Tensor) -> torch.Tensor:
        """Integer indices shaped like x, the reference's contract."""
        flat = _k.unpack_bits(self.quantize_packed(x), self.bits, self.d)
        return flat.long().reshape(x.shape)

    # --- reconstruct ---
    def dequantize(self, indices: torch.Tensor) -> torch.Tensor:
        """Accepts integer indices [..., d] or the packed bytes of `quantize_packed`."""
        _on_gpu(indices)
        packed_width = self.d * self.bits // 8
        if indices.dtype == torch.uint8 and self.bits < 8 and indices.shape[-1] == packed_width:
            levels = _k.lloyd_max_dequantize(indices.reshape(-1, packed_width), self.centroids, self.bits, self.d)
        else:
            levels = self.centroids[indices]
        return self.unrotate(levels)

    def forward(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        idx = self.quantize(x)
        return self.dequantize(idx), idx


class TurboQuantProd(nn.Module):
    """MSE quantiser with bits - 1 bits plus one sign bit per sketch coordinate of the residual; its
    `inner_product` estimate is unbiased (turboquant.py:103-196)."""

    def __init__(self, d: int, bits: int, qjl_dim: Optional[int] = None, seed: int = 42, device: str = "cuda"):
        super().__init__()
        self.d, self.bits, self.device = d, bits, device
        self.mse_bits = bits - 1 if bits > 1 else 1
        self.qjl_dim = d if not qjl_dim else qjl_dim
        self.mse = TurboQuantMSE(d, self.mse_bits, seed=seed, device=device)
        self.register_buffer("S", generate_qjl_matrix(d, self.qjl_dim, seed + 1, device))

    def _sketch(self, v: torch.Tensor) -> torch.Tensor:
        return torch.matmul(v, self.S.transpose(0, 1))

    def quantize(self, x: torch.Tensor) -> dict:
        approx, idx = self.mse(x)
        rest = x - approx
        bits = torch.where(self._sketch(rest) < 0, -1.0, 1.0)  # zero counts as +1
        return dict(mse_indices=idx, qjl_signs=bits, residual_norm=rest.norm(dim=-1))

    forward = quantize

    def dequantize(self, compressed: dict) -> torch.Tensor:
        return self.mse.dequantize(compressed["mse_indices"])

    def inner_product(self, y: torch.Tensor, compressed: dict) -> torch.Tensor:
        """<y, x_mse> + |r| * sqrt(pi/2) / m * <S y, signs>."""
        coarse = torch.sum(y * self.dequantize(compressed), dim=-1)
        fine = torch.sum(self._sketch(y) * compressed["qjl_signs"], dim=-1)
        return coarse + (_SKETCH_GAIN / self.qjl_dim) * compressed["residual_norm"] * fine


class TurboQuantKVCache:
    """Append-only store of compressed keys (TurboQuantProd) and values (TurboQuantMSE, seed + 100) with
    estimator scores over everything cached (turboquant.py:199-286)."""

    def __init__(self, d_key: int, d_value: int, bits: int = 3, seed: int = 42, device: str = "cuda"):
        self.d_key, self.d_value, self.bits, self.device = d_key, d_value, bits, device
        self.key_quantizer = TurboQuantProd(d_key, bits, seed=seed, device=device)
        self.value_quantizer = TurboQuantMSE(d_value, bits, seed=seed + 100, device=device)
        self.key_cache: list[dict] = []
        self.value_cache: list[dict] = []

    def append(self, keys: torch.Tensor, values: torch.Tensor) -> None:
        entry = self.key_quantizer.quantize(keys.reshape(-1, self.d_key))
        entry["shape"] = keys.shape
        self.key_cache.append(entry)
        self.value_cache.append(dict(indices=self.value_quantizer.quantize(values.reshape(-1, self.d_value)),
                                     shape=values.shape))

    def attention_scores(self, queries: torch.Tensor) -> torch.Tensor:
        if not self.key_cache:
            return torch.tensor([])
        return torch.cat([self.key_quantizer.inner_product(queries, e) for e in self.key_cache], dim=-1)

    def get_values(self) -> torch.Tensor:
        if not self.value_cache:
            return torch.tensor([])
        return torch.cat([self.value_quantizer.dequantize(e["indices"]) for e in self.value_cache], dim=0)

    def __len__(self) -> int:
        return sum(e["mse_indices"].shape[0] for e in self.key_cache)

    def memory_usage_bits(self) -> dict:
        count = lambda entries, field: sum(e[field].numel() for e in entries)  # noqa: E731
        idx, sgn, nrm = (count(self.key_cache, f) for f in ("mse_indices", "qjl_signs", "residual_norm"))
        val = count(self.value_cache, "indices")
        report = {"key_bits": idx * self.key_quantizer.mse_bits + sgn + 16 * nrm, "value_bits": val * self.bits,
                  "fp16_bits": 16 * (idx + val)}
        report["total_bits"] = report["key_bits"] + report["value_bits"]
        report["compression_ratio"] = report["fp16_bits"] / report["total_bits"] if report["total_bits"] else 0
        return report
