"""A persistent compressed KV cache on the device, in the library's wire format.

The reference patches models with `use_cache = False` and recompresses the whole prefix for every
generated token (src/transformers_turboquant/patch.py:80-81); its cache exists as a concept only
(src/turboquant_pytorch/turboquant.py:199-286: append compressed entries, score queries against
them).  `CompressedKVCache` is that concept on the CUDA kernels: packed buffers with room for
`capacity` tokens per (batch, KV head), `append` compresses new tokens behind the ones in use, and
`attend` runs compressed attention of new queries over everything stored -- the split-KV kernel reads
the buffers in place, so a decode step touches each packed byte once and copies nothing.
"""

from __future__ import annotations

import math

import torch

from . import _lib
from .compressors import (_DTYPES, _mask_args, _require_cuda, _rows_view, _stream_ptr, _workspace,
                          TurboQuantCompressorMSE, TurboQuantCompressorV2, fused_attention, prepared_constants,
                          resolve_mode)


class CompressedKVCache:
    """Packed keys and values of `batch` sequences and `kv_heads` KV heads, up to `capacity` tokens each.

    Buffers (row (b, h, t)): key indices u8 [.., d*(bits-1)/8], key sign bits u8 [.., d/8], key vector and
    residual norms fp16, value indices u8 [.., d*bits/8], value vector norms fp16 -- the layout
    `compress()` returns, with a token stride of `capacity` instead of the current length.
    """

    def __init__(self, key_compressor: TurboQuantCompressorV2, val_compressor: TurboQuantCompressorMSE,
                 batch: int, kv_heads: int, capacity: int, device="cuda"):
        if key_compressor.bits != val_compressor.bits or key_compressor.head_dim != val_compressor.head_dim:
            raise ValueError("key and value compressors must share bit width and head_dim")
        if capacity < 1:
            raise ValueError("capacity must be positive")
        self.key_compressor, self.val_compressor = key_compressor, val_compressor
        self.batch, self.kv_heads, self.capacity = int(batch), int(kv_heads), int(capacity)
        self.head_dim, self.bits = key_compressor.head_dim, key_compressor.bits
        d, kb, vb = self.head_dim, key_compressor.mse_bits, val_compressor.bits
        dev = torch.device(device)
        shape = (self.batch, self.kv_heads, self.capacity)
        self.key_indices = torch.zeros(shape + (d * kb // 8,), dtype=torch.uint8, device=dev)
        self.key_signs = torch.zeros(shape + (d // 8,), dtype=torch.uint8, device=dev)
        self.key_norms = torch.zeros(shape, dtype=torch.float16, device=dev)
        self.key_residual_norms = torch.zeros(shape, dtype=torch.float16, device=dev)
        self.value_indices = torch.zeros(shape + (d * vb // 8,), dtype=torch.uint8, device=dev)
        self.value_norms = torch.zeros(shape, dtype=torch.float16, device=dev)
        self.length = 0

    def __len__(self) -> int:
        return self.length

    def nbytes(self) -> int:
        """Bytes the tokens in use occupy (what a decode step reads)."""
        d, kb, vb = self.head_dim, self.key_compressor.mse_bits, self.val_compressor.bits
        per_token = d * kb // 8 + d // 8 + 4 + d * vb // 8 + 2
        return self.batch * self.kv_heads * self.length * per_token

    def reset(self) -> None:
        self.length = 0

    @torch.no_grad()
    def append(self, keys: torch.Tensor, values: torch.Tensor) -> None:
        """Compress [B, Hkv, S_new, D] keys and values and store them behind the tokens in use."""
        B, H, S, D = keys.shape
        if values.shape != keys.shape or (B, H, D) != (self.batch, self.kv_heads, self.head_dim):
            raise ValueError(f"expected [{self.batch}, {self.kv_heads}, S, {self.head_dim}] keys and values, got "
                             f"{tuple(keys.shape)} and {tuple(values.shape)}")
        if self.length + S > self.capacity:
            raise ValueError(f"cache holds {self.length} of {self.capacity} tokens; cannot append {S}")
        _require_cuda(keys, "keys")
        kc, vc = self.key_compressor, self.val_compressor
        kc._check_device(keys)
        vc._check_device(keys)
        k, v = _rows_view(keys), _rows_view(values)
        if v.dtype != k.dtype:
            v = v.to(k.dtype)
        # one launch compresses both sides straight behind the tokens in use: no scratch, no copies
        _lib.check(_lib.lib.tq_compress_kv(
            k.data_ptr(), v.data_ptr(), _DTYPES[k.dtype], B, H, S, D, k.stride(0), k.stride(1), k.stride(2),
            v.stride(0), v.stride(1), v.stride(2), prepared_constants(kc, vc).data_ptr(), kc.bits,
            self.key_indices.data_ptr(), self.key_signs.data_ptr(), self.key_norms.data_ptr(),
            self.key_residual_norms.data_ptr(), self.value_indices.data_ptr(), self.value_norms.data_ptr(),
            self.capacity, self.length, resolve_mode(k.dtype, kc.mode), _stream_ptr(k.device)))
        self.length += S

    def _contiguous_prefix(self) -> tuple[dict, dict]:
        """The tokens in use as the contiguous dictionaries `compress()` returns (copies: the cache rows are
        `capacity` apart).  `reshape` alone is not enough: for a single token per head it returns a strided view."""
        n, shape = self.length, (self.batch, self.kv_heads, self.length, self.head_dim)

        def rows(t):
            return t[:, :, :n].reshape(-1, t.shape[-1]).contiguous()

        ck = {"packed_key_indices": rows(self.key_indices), "packed_qjl_signs": rows(self.key_signs),
              "vec_norms": self.key_norms[:, :, :n].contiguous(),
              "residual_norm": self.key_residual_norms[:, :, :n].contiguous(), "shape": shape}
        cv = {"packed_indices": rows(self.value_indices),
              "vec_norms": self.value_norms[:, :, :n].reshape(-1).contiguous(), "shape": shape}
        return ck, cv

    @torch.no_grad()
    def attend(self, q: torch.Tensor, causal: bool = True, sm_scale: float | None = None,
               attention_mask: torch.Tensor | None = None) -> torch.Tensor:
        """softmax(scores * sm_scale) @ V_hat of q [B, Hq, Sq, D] over the tokens in use; with `causal` the
        queries are the last Sq positions (append their keys first).  Returns [B, Hq, Sq, D] in q.dtype.

        `attention_mask` is an optional additive mask broadcastable to [B, 1, Sq, tokens in use] (padding).
        Decode-sized calls (head_dim 128, (Hq / Hkv) * Sq <= 16, 16-bit queries) read the cache in place;
        anything else gathers the prefix once and takes the prefill kernels."""
        _require_cuda(q, "q")
        B, Hq, Sq, D = q.shape
        if (B, D) != (self.batch, self.head_dim) or Hq % self.kv_heads != 0:
            raise ValueError(f"queries {tuple(q.shape)} do not match the cache")
        if self.length == 0:
            raise ValueError("attention over an empty cache is undefined")
        in_place = (D == 128 and (Hq // self.kv_heads) * Sq <= 16 and q.dtype in (torch.bfloat16, torch.float16)
                    and self.key_compressor.mode in (None, "bf16"))
        if not in_place:
            ck, cv = self._contiguous_prefix()
            return fused_attention(q, ck, cv, self.key_compressor, self.val_compressor, causal=causal,
                                   attention_mask=attention_mask, sm_scale=sm_scale)
        kc, vc = self.key_compressor, self.val_compressor
        kc._check_device(q)
        vc._check_device(q)
        qv = _rows_view(q)
        dev = qv.device
        out = torch.empty((B, Sq, Hq, D), dtype=qv.dtype, device=dev).transpose(1, 2)  # position-major, as fused_attention
        ws = _workspace(dev, _lib.lib.tq_attention_prepared_workspace_bytes(B, Hq, Sq, self.kv_heads, self.length,
                                                                            self.capacity, D, _lib.TQ_MODE_BF16))
        scale = float(sm_scale) if sm_scale is not None else 1.0 / math.sqrt(D)
        mk, mask_ptr, msb, msq = _mask_args(attention_mask, B, Sq, self.length, dev)  # mk keeps the mask alive
        _lib.check(_lib.lib.tq_attention_fwd_prepared(
            qv.data_ptr(), _DTYPES[qv.dtype], B, Hq, Sq, D, qv.stride(0), qv.stride(1), qv.stride(2),
            self.kv_heads, self.length, self.capacity,
            self.key_indices.data_ptr(), self.key_signs.data_ptr(), self.key_norms.data_ptr(),
            self.key_residual_norms.data_ptr(), self.value_indices.data_ptr(), self.value_norms.data_ptr(),
            prepared_constants(kc, vc).data_ptr(), kc.bits, scale, 1 if causal else 0, mask_ptr, msb, msq,
            out.data_ptr(), out.stride(0), out.stride(1), out.stride(2),
            ws.data_ptr(), ws.numel(), _lib.TQ_MODE_BF16, _stream_ptr(dev)))
        return out
