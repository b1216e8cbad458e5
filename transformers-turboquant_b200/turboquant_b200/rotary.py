"""Rotary position embedding of a layer's query and key heads in one CUDA launch.

The reference's adapters call HF's `apply_rotary_pos_emb(q, k, cos, sin)` right before they compress the keys
(src/transformers_turboquant/families/llama.py:98): four elementwise torch kernels and a concatenation per
tensor.  `rope` does the same arithmetic, to the bit, reading and writing every element once."""

from __future__ import annotations

import torch

from . import _lib
from .compressors import _DTYPES, _require_cuda, _stream_ptr


def rope_applies(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> bool:
    """Whether `rope` covers these tensors: CUDA, one dtype the kernels know, rotary width = head_dim (a multiple
    of 32), cos/sin shaped [B or 1, S, d] with contiguous rows."""
    d = q.shape[-1]
    return (q.is_cuda and q.dtype in _DTYPES and k.dtype == q.dtype and cos.dtype == q.dtype and sin.dtype == q.dtype
            and q.dim() == 4 and k.dim() == 4 and cos.dim() == 3 and cos.shape == sin.shape and cos.shape[-1] == d
            and d % 32 == 0 and cos.shape[0] in (1, q.shape[0]) and cos.shape[1] == q.shape[2]
            and k.shape[-1] == d and k.shape[2] == q.shape[2] and q.stride(-1) == 1 and k.stride(-1) == 1)


@torch.no_grad()
def rope(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
    """(q * cos + rotate_half(q) * sin, k * cos + rotate_half(k) * sin) for q [B, Hq, S, d], k [B, Hkv, S, d] (any
    strides with contiguous rows) and cos, sin [B or 1, S, d]; returns new contiguous tensors."""
    _require_cuda(q, "q")
    if not rope_applies(q, k, cos, sin):
        raise ValueError(f"rope: unsupported arguments q {tuple(q.shape)} {q.dtype}, k {tuple(k.shape)} {k.dtype}, "
                         f"cos {tuple(cos.shape)} {cos.dtype}")
    B, Hq, S, d = q.shape
    Hkv = k.shape[1]
    if cos.stride(-1) != 1 or sin.stride() != cos.stride():
        cos, sin = cos.contiguous(), sin.contiguous()
    q_out = torch.empty((B, Hq, S, d), dtype=q.dtype, device=q.device)
    k_out = torch.empty((B, Hkv, S, d), dtype=k.dtype, device=k.device)
    _lib.check(_lib.lib.tq_rope(
        q.data_ptr(), k.data_ptr(), _DTYPES[q.dtype], B, Hq, Hkv, S, d, q.stride(0), q.stride(1), q.stride(2),
        k.stride(0), k.stride(1), k.stride(2), cos.data_ptr(), sin.data_ptr(),
        0 if cos.shape[0] == 1 else cos.stride(0), cos.stride(1), q_out.data_ptr(), k_out.data_ptr(),
        _stream_ptr(q.device)))
    return q_out, k_out
