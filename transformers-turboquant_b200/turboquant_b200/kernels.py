"""Wire-format operators on the GPU under the reference's function names
(src/turboquant_pytorch/kernels/__init__.py:1-11): pack_bits / unpack_bits (bit_ops.py:65-155),
lloyd_max_quantize / lloyd_max_dequantize (quantize.py:201-290) and asymmetric_attention_scores
(attention.py:274-372).  Each is a thin call into the C ABI (include/tq_b200.h); inputs must live on
a CUDA device, there is no CPU path.
"""

from __future__ import annotations

import math

import torch

from . import _lib
from .compressors import _require_cuda, _stream_ptr

__all__ = ["pack_bits", "unpack_bits", "lloyd_max_quantize", "lloyd_max_dequantize",
           "asymmetric_attention_scores"]


def _rows(t: torch.Tensor, what: str) -> torch.Tensor:
    _require_cuda(t, what)
    if t.dim() != 2:
        raise ValueError(f"{what} must be 2-D [N, d], got shape {tuple(t.shape)}")
    return t.contiguous()


def _check_bits(d: int, b: int) -> None:
    if not 1 <= b <= 8:
        raise ValueError(f"bits per index must be between 1 and 8, got {b}")
    if (d * b) % 8 != 0:
        raise ValueError(f"a row of {d} indices of {b} bits does not fill whole bytes")


def pack_bits(indices: torch.Tensor, b: int) -> torch.Tensor:
    """int32 [N, d] indices -> uint8 [N, d*b/8], LSB-first bit stream (index i at bits [i*b, i*b+b))."""
    x = _rows(indices, "indices").to(torch.int32)
    n, d = x.shape
    _check_bits(d, b)
    out = torch.empty((n, d * b // 8), dtype=torch.uint8, device=x.device)
    _lib.check(_lib.lib.tq_pack_bits(x.data_ptr(), n, d, b, out.data_ptr(), _stream_ptr(x.device)))
    return out


def unpack_bits(packed: torch.Tensor, b: int, d: int) -> torch.Tensor:
    """Inverse of pack_bits: uint8 [N, d*b/8] -> int32 [N, d]."""
    p = _rows(packed, "packed")
    _check_bits(d, b)
    if p.dtype != torch.uint8 or p.shape[1] != d * b // 8:
        raise ValueError(f"packed must be uint8 [N, {d * b // 8}], got {p.dtype} {tuple(p.shape)}")
    out = torch.empty((p.shape[0], d), dtype=torch.int32, device=p.device)
    _lib.check(_lib.lib.tq_unpack_bits(p.data_ptr(), p.shape[0], d, b, out.data_ptr(), _stream_ptr(p.device)))
    return out


def lloyd_max_quantize(rotated: torch.Tensor, boundaries: torch.Tensor, b_eff: int) -> torch.Tensor:
    """fp32 [N, d] rotated coordinates -> packed indices uint8 [N, d*b_eff/8]; index = number of boundaries
    strictly below the coordinate (the first-minimum argmin of the reference's PyTorch path)."""
    x = _rows(rotated, "rotated").float()
    n, d = x.shape
    _check_bits(d, b_eff)
    if boundaries.numel() != (1 << b_eff) - 1:
        raise ValueError(f"expected {(1 << b_eff) - 1} boundaries for b_eff={b_eff}, got {boundaries.numel()}")
    bnd = boundaries.to(device=x.device, dtype=torch.float32).contiguous()
    out = torch.empty((n, d * b_eff // 8), dtype=torch.uint8, device=x.device)
    _lib.check(_lib.lib.tq_quantize_rotated(x.data_ptr(), n, d, bnd.data_ptr(), b_eff, out.data_ptr(),
                                            _stream_ptr(x.device)))
    return out


def lloyd_max_dequantize(packed: torch.Tensor, centroids: torch.Tensor, b: int, d: int) -> torch.Tensor:
    """Packed indices -> centroid values [N, d] in the dtype of `centroids` (fp16 in the reference)."""
    p = _rows(packed, "packed")
    _check_bits(d, b)
    if centroids.numel() != 1 << b:
        raise ValueError(f"expected {1 << b} centroids for b={b}, got {centroids.numel()}")
    cen = centroids.to(device=p.device, dtype=torch.float32).contiguous()
    out = torch.empty((p.shape[0], d), dtype=torch.float32, device=p.device)
    _lib.check(_lib.lib.tq_dequantize(p.data_ptr(), p.shape[0], d, cen.data_ptr(), b, out.data_ptr(),
                                      _stream_ptr(p.device)))
    return out.to(centroids.dtype) if centroids.dtype.is_floating_point else out


def asymmetric_attention_scores(query: torch.Tensor, packed_key_indices: torch.Tensor,
                                packed_qjl_signs: torch.Tensor, residual_norms: torch.Tensor,
                                centroids: torch.Tensor, qjl_matrix: torch.Tensor, vec_norms: torch.Tensor,
                                b: int, coeff: float) -> torch.Tensor:
    """fp32 [B, H, Sq, Sk] estimator scores from PRE-ROTATED queries (q @ Pi^T) and packed keys:
    n_k <q_rot, C[idx_k]> + coeff rn_k <q_rot S_eff^T, sign_k>, `qjl_matrix` = S_eff = S Pi^T [d, d].
    `centroids` is [2^(b-1)] or [H, 2^(b-1)] (one codebook per head)."""
    _require_cuda(query, "query")
    B, H, Sq, d = query.shape
    Sk = packed_key_indices.shape[2]
    if qjl_matrix.shape != (d, d):
        raise ValueError("the QJL sketch must have as many rows as head_dim")
    dev = query.device
    q = query.contiguous()
    if q.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        q = q.float()
    eye = torch.eye(d, device=dev, dtype=torch.float32)              # the queries are rotated already
    # the kernel's correction factor is sqrt(pi/2)/d; any other `coeff` is folded into the sketch matrix
    s_eff = (qjl_matrix.to(device=dev, dtype=torch.float32) * (coeff / (math.sqrt(math.pi / 2) / d))).contiguous()
    idx = packed_key_indices.contiguous()
    sgn = packed_qjl_signs.contiguous()
    rn = residual_norms.to(torch.float16).contiguous()
    vn = vec_norms.to(torch.float16).contiguous()
    cen = centroids.to(device=dev, dtype=torch.float32)
    per_head = cen.dim() == 2 and H > 1 and not bool((cen == cen[:1]).all())
    out = torch.empty((B, H, Sq, Sk), dtype=torch.float32, device=dev)
    if B * H * Sq * Sk == 0:
        return out
    from .compressors import _DTYPES

    def run(qh, idxh, sgnh, vnh, rnh, cenh, outh):
        Bh, Hh = qh.shape[:2]
        ws_bytes = _lib.lib.tq_attention_workspace_bytes(Bh, Hh, Sq, d, _lib.TQ_MODE_FP32)
        ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
        _lib.check(_lib.lib.tq_attention_scores(
            qh.data_ptr(), _DTYPES[qh.dtype], Bh, Hh, Sq, d, qh.stride(0), qh.stride(1), qh.stride(2), Hh, Sk,
            idxh.data_ptr(), sgnh.data_ptr(), vnh.data_ptr(), rnh.data_ptr(), eye.data_ptr(), s_eff.data_ptr(),
            cenh.contiguous().data_ptr(), b, outh.data_ptr(), ws.data_ptr(), ws.numel(), _lib.TQ_MODE_FP32,
            _stream_ptr(dev)))

    if not per_head:
        run(q, idx, sgn, vn, rn, cen.reshape(-1, cen.shape[-1])[0], out)
    else:
        for h in range(H):
            oh = torch.empty((B, 1, Sq, Sk), dtype=torch.float32, device=dev)
            run(q[:, h:h + 1].contiguous(), idx[:, h:h + 1].contiguous(), sgn[:, h:h + 1].contiguous(),
                vn[:, h:h + 1].contiguous(), rn[:, h:h + 1].contiguous(), cen[h], oh)
            out[:, h:h + 1] = oh
    return out
