"""Key / value compressors backed by the sm_100a CUDA library.

`TurboQuantCompressorV2` and `TurboQuantCompressorMSE` keep the constructor signature,
attribute names (`Pi, PiT, S, centroids, boundaries, bits, mse_bits, head_dim, device`)
and methods (`compress`, `asymmetric_attention_scores`, `decompress`) of the reference
classes (src/turboquant_pytorch/compressors.py:36-317) and always produce its bit-packed
result layout (compressors.py:132-138, :281-285).  Inputs must live on a CUDA device; there
is no CPU path.  `fused_attention` is the entry the family adapters call: compressed causal
attention without the score matrix or decompressed K/V.
"""

from __future__ import annotations

import math
import os

import torch

from . import _lib
from .codebook import lloyd_max_centroids, midpoints

_DTYPES = {torch.float32: _lib.TQ_F32, torch.bfloat16: _lib.TQ_BF16, torch.float16: _lib.TQ_F16}
_MODES = {"fp32": _lib.TQ_MODE_FP32, "bf16": _lib.TQ_MODE_BF16}


def resolve_mode(dtype: torch.dtype, mode: str | None = None) -> int:
    """Arithmetic mode of a call.  Explicit `mode`, else the TQ_B200_MODE environment
    variable ("fp32" | "bf16"), else by input type: fp32 inputs run the fp32 parity
    kernels, 16-bit inputs the tensor-core kernels."""
    mode = mode or os.environ.get("TQ_B200_MODE") or "auto"
    if mode == "auto":
        return _lib.TQ_MODE_FP32 if dtype == torch.float32 else _lib.TQ_MODE_BF16
    if mode not in _MODES:
        raise ValueError(f"mode must be 'fp32', 'bf16' or 'auto', got {mode!r}")
    return _MODES[mode]


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what} must be a CUDA tensor: turboquant_b200 has no CPU path")


_KEY_ARRAYS = ("packed_key_indices", "packed_qjl_signs", "vec_norms", "residual_norm")
_VALUE_ARRAYS = ("packed_indices", "vec_norms")


def _dense_packed(compressed: dict, keys: tuple) -> dict:
    """The packed arrays of a compressed dictionary as the kernels read them: dense rows, one per (b, h, s) in that
    order.  A strided view (a slice of a larger buffer) is copied; a wrong row count is refused, not read past."""
    B, H, S, _ = compressed["shape"]
    out = dict(compressed)
    for name in keys:
        t = compressed[name]
        rows = t.numel() // max(t.shape[-1], 1) if name.startswith("packed") else t.numel()  # packed: [..., bytes]
        if rows != B * H * S:
            raise ValueError(f"{name} holds {tuple(t.shape)} entries for a compressed shape {compressed['shape']}")
        out[name] = t if t.is_contiguous() else t.contiguous()
    return out


def _rows_view(t: torch.Tensor) -> torch.Tensor:
    """[B, H, S, D] tensor whose rows the kernels can read in place: supported dtype, unit
    inner stride, 16-byte aligned rows.  Anything else is copied once."""
    if t.dtype not in _DTYPES:
        t = t.float()
    esz = t.element_size()
    ok = t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and all((s * esz) % 16 == 0 for s in t.stride()[:-1])
    return t if ok else t.contiguous()


def _haar_rotation(d: int, seed: int) -> torch.Tensor:
    """Seeded random rotation: Q factor of a Gaussian matrix with the sign convention
    diag(R) > 0 (compressors.py:50-56).  Generated on the CPU generator so that a seed
    means the same matrix everywhere."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    q, r = torch.linalg.qr(torch.randn(d, d, generator=g))
    s = torch.sign(torch.diagonal(r))
    s[s == 0] = 1.0
    return q * s


class _Constants:
    """Device-resident fp32 constants of a compressor and their movement between devices."""

    _tensor_attrs: tuple[str, ...] = ()

    def __setattr__(self, name, value):
        # Replacing a constant (tests overwrite them with the oracle's) invalidates the operand images prepared
        # from it.  In-place edits of a constant tensor are not seen: assign a new tensor instead.
        if name in self._tensor_attrs:
            self.__dict__["_version"] = self.__dict__.get("_version", 0) + 1
        object.__setattr__(self, name, value)

    def to(self, device):
        device = torch.device(device)
        for name in self._tensor_attrs:
            setattr(self, name, getattr(self, name).to(device=device, dtype=torch.float32).contiguous())
        self.device = str(device)
        return self

    def _check_device(self, t: torch.Tensor) -> None:
        if self.Pi.device != t.device:
            self.to(t.device)


_PAD = {}


def _zeros16(dev) -> torch.Tensor:
    """Stand-in for the codebook of a side that a one-sided constants buffer does not have."""
    key = str(dev)
    if key not in _PAD:
        _PAD[key] = torch.zeros(16, dtype=torch.float32, device=dev)
    return _PAD[key]


def _prepare(kc, vc, bits: int, d: int, dev) -> torch.Tensor:
    """One constants buffer (tq_prepare_constants) for a key compressor, a value compressor or both; the missing
    side is filled with stand-ins that no call reads."""
    pad = _zeros16(dev)
    any_pi = (kc or vc).Pi
    args = [kc.Pi if kc else any_pi, kc.S_eff if kc else any_pi, kc.centroids if kc else pad,
            kc.boundaries if kc else pad, vc.Pi if vc else any_pi, vc.centroids if vc else pad,
            vc.boundaries if vc else pad]
    nbytes = _lib.lib.tq_constants_bytes(d, bits)
    buf = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    _lib.check(_lib.lib.tq_prepare_constants(*[t.data_ptr() for t in args], bits, d, buf.data_ptr(), nbytes,
                                             _stream_ptr(dev)))
    return buf


def prepared_constants(kc=None, vc=None) -> torch.Tensor:
    """The device buffer of operand images and fp32 constants for this compressor pair (or one compressor),
    built on first use and kept until one of the constants is replaced or moved."""
    owner = kc if kc is not None else vc
    key = (id(kc) if kc else 0, id(vc) if vc else 0)
    ver = (kc._version if kc else 0, vc._version if vc else 0)
    cache = owner.__dict__.setdefault("_prepared", {})
    hit = cache.get(key)
    if hit is None or hit[0] != ver:
        if kc is not None and vc is not None and (kc.bits != vc.bits or kc.head_dim != vc.head_dim):
            raise ValueError("key and value compressors must share bit width and head_dim")
        cache[key] = hit = (ver, _prepare(kc, vc, owner.bits, owner.head_dim, owner.Pi.device))
    return hit[1]


_WORKSPACES: dict = {}


def _workspace(dev, nbytes: int) -> torch.Tensor:
    """Scratch for one call.  One buffer per (device, stream) is kept and grown: calls on a stream run in order,
    so they can share it; during stream capture a fresh tensor is taken from the graph's pool instead."""
    nbytes = max(int(nbytes), 256)
    if torch.cuda.is_current_stream_capturing():
        return torch.empty(nbytes, dtype=torch.uint8, device=dev)
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), _stream_ptr(dev))
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < nbytes:
        _WORKSPACES[key] = ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    return ws


def _packed_buffers(kc, vc, B: int, H: int, S: int, D: int, dev):
    ck = cv = None
    n = B * H * S
    if kc is not None:
        ck = {"packed_key_indices": torch.empty((n, D * kc.mse_bits // 8), dtype=torch.uint8, device=dev),
              "packed_qjl_signs": torch.empty((n, D // 8), dtype=torch.uint8, device=dev),
              "residual_norm": torch.empty((B, H, S), dtype=torch.float16, device=dev),
              "vec_norms": torch.empty((B, H, S), dtype=torch.float16, device=dev), "shape": (B, H, S, D)}
    if vc is not None:
        cv = {"packed_indices": torch.empty((n, D * vc.bits // 8), dtype=torch.uint8, device=dev),
              "vec_norms": torch.empty((n,), dtype=torch.float16, device=dev), "shape": (B, H, S, D)}
    return ck, cv


@torch.no_grad()
def compress_kv(keys, values, key_compressor=None, val_compressor=None):
    """Compress keys and values [B, H, S, D] in ONE launch (either may be None): what the family adapters do with
    `key_compressor.compress(k)` and `val_compressor.compress(v)` back to back (families/llama.py:103-104 of
    the reference).  Returns (compressed_keys, compressed_values) in the packed layout of `compress`."""
    kc, vc = (key_compressor if keys is not None else None), (val_compressor if values is not None else None)
    ref = keys if keys is not None else values
    if ref is None or (kc is None and vc is None):
        raise ValueError("nothing to compress")
    _require_cuda(ref, "states")
    for comp in (kc, vc):
        if comp is not None:
            comp._check_device(ref)
    B, H, S, D = ref.shape
    owner = kc or vc
    if D != owner.head_dim or (keys is not None and values is not None and values.shape != keys.shape):
        raise ValueError(f"expected [B, H, S, {owner.head_dim}] keys and values of one shape")
    k = _rows_view(keys) if kc is not None else None
    v = _rows_view(values) if vc is not None else None
    if k is not None and v is not None and k.dtype != v.dtype:
        v = v.to(k.dtype)
    x = k if k is not None else v
    dev = x.device
    ck, cv = _packed_buffers(kc, vc, B, H, S, D, dev)
    consts = prepared_constants(kc, vc)
    ks = k.stride() if k is not None else (0, 0, D, 1)
    vs = v.stride() if v is not None else (0, 0, D, 1)
    _lib.check(_lib.lib.tq_compress_kv(
        k.data_ptr() if k is not None else None, v.data_ptr() if v is not None else None, _DTYPES[x.dtype],
        B, H, S, D, ks[0], ks[1], ks[2], vs[0], vs[1], vs[2], consts.data_ptr(), owner.bits,
        ck["packed_key_indices"].data_ptr() if ck else None, ck["packed_qjl_signs"].data_ptr() if ck else None,
        ck["vec_norms"].data_ptr() if ck else None, ck["residual_norm"].data_ptr() if ck else None,
        cv["packed_indices"].data_ptr() if cv else None, cv["vec_norms"].data_ptr() if cv else None,
        S, 0, resolve_mode(x.dtype, owner.mode), _stream_ptr(dev)))
    return ck, cv


class TurboQuantCompressorV2(_Constants):
    """Key compressor: (bits-1)-bit Lloyd-Max indices of the rotated unit vector plus a
    1-bit QJL sketch of the residual (compressors.py:36-224)."""

    _tensor_attrs = ("Pi", "PiT", "S", "S_eff", "centroids", "boundaries")

    def __init__(self, head_dim: int, bits: int, seed: int, device: str = "cuda", use_triton: bool = True,
                 mode: str | None = None):
        if head_dim not in (64, 128):
            raise ValueError(f"head_dim {head_dim} unsupported by the CUDA kernels (64 or 128)")
        if bits not in (2, 3, 4):
            raise ValueError(f"bits must be 2, 3 or 4, got {bits}")
        self.head_dim, self.bits, self.mse_bits = head_dim, bits, max(bits - 1, 1)
        self.use_triton = use_triton  # accepted for call compatibility; there is one backend
        self.mode = mode
        self.Pi = _haar_rotation(head_dim, seed)
        self.PiT = self.Pi.T.contiguous()
        self.centroids = lloyd_max_centroids(head_dim, self.mse_bits)
        self.boundaries = midpoints(self.centroids)
        g = torch.Generator(device="cpu").manual_seed(seed + 10000)
        self.S = torch.randn(head_dim, head_dim, generator=g)
        self.S_eff = self.S @ self.Pi.T  # sketch matrix in rotated coordinates
        self.to(device)

    @torch.no_grad()
    def compress(self, states: torch.Tensor) -> dict:
        """[B, H, S, D] -> packed dict (one fused kernel)."""
        if states.dim() != 4 or states.shape[-1] != self.head_dim:
            raise ValueError(f"expected [B, H, S, {self.head_dim}] states, got {tuple(states.shape)}")
        return compress_kv(states, None, key_compressor=self)[0]

    @torch.no_grad()
    def asymmetric_attention_scores(self, queries: torch.Tensor, compressed: dict) -> torch.Tensor:
        """Unscaled, unmasked estimator scores fp32 [B, Hq, Sq, Sk] (compressors.py:163-224).
        Materialises the whole matrix; the adapters use `fused_attention` instead."""
        _require_cuda(queries, "queries")
        self._check_device(queries)
        B, Hq, Sq, D = queries.shape
        Bk, Hkv, Sk, Dk = compressed["shape"]
        if (Bk, Dk) != (B, D) or D != self.head_dim:
            raise ValueError(f"queries {tuple(queries.shape)} do not match compressed keys {compressed['shape']}")
        compressed = _dense_packed(compressed, _KEY_ARRAYS)
        q = _rows_view(queries)
        dev = q.device
        scores = torch.empty((B, Hq, Sq, Sk), dtype=torch.float32, device=dev)
        ws_bytes = _lib.lib.tq_attention_workspace_bytes(B, Hq, Sq, D, _lib.TQ_MODE_FP32)
        ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
        _lib.check(_lib.lib.tq_attention_scores(
            q.data_ptr(), _DTYPES[q.dtype], B, Hq, Sq, D, q.stride(0), q.stride(1), q.stride(2), Hkv, Sk,
            compressed["packed_key_indices"].data_ptr(), compressed["packed_qjl_signs"].data_ptr(),
            compressed["vec_norms"].data_ptr(), compressed["residual_norm"].data_ptr(),
            self.Pi.data_ptr(), self.S_eff.data_ptr(), self.centroids.data_ptr(), self.bits,
            scores.data_ptr(), ws.data_ptr(), ws.numel(), _lib.TQ_MODE_FP32, _stream_ptr(dev)))
        return scores


class TurboQuantCompressorMSE(_Constants):
    """Value compressor: `bits`-bit Lloyd-Max indices of the rotated unit vector
    (compressors.py:227-317)."""

    _tensor_attrs = ("Pi", "PiT", "centroids", "boundaries")

    def __init__(self, head_dim: int, bits: int, seed: int, device: str = "cuda", use_triton: bool = True,
                 mode: str | None = None):
        if head_dim not in (64, 128):
            raise ValueError(f"head_dim {head_dim} unsupported by the CUDA kernels (64 or 128)")
        if bits not in (2, 3, 4):
            raise ValueError(f"bits must be 2, 3 or 4, got {bits}")
        self.head_dim, self.bits = head_dim, bits
        self.use_triton = use_triton
        self.mode = mode
        self.Pi = _haar_rotation(head_dim, seed)
        self.PiT = self.Pi.T.contiguous()
        self.centroids = lloyd_max_centroids(head_dim, bits)
        self.boundaries = midpoints(self.centroids)
        self.to(device)

    @torch.no_grad()
    def compress(self, states: torch.Tensor) -> dict:
        if states.dim() != 4 or states.shape[-1] != self.head_dim:
            raise ValueError(f"expected [B, H, S, {self.head_dim}] states, got {tuple(states.shape)}")
        return compress_kv(None, states, val_compressor=self)[1]

    @torch.no_grad()
    def decompress(self, compressed: dict) -> torch.Tensor:
        """packed dict -> fp32 [B, H, S, D] (compressors.py:296-317)."""
        B, H, S, D = compressed["shape"]
        compressed = _dense_packed(compressed, _VALUE_ARRAYS)
        idx = compressed["packed_indices"]
        _require_cuda(idx, "compressed values")
        self._check_device(idx)
        out = torch.empty((B, H, S, D), dtype=torch.float32, device=idx.device)
        _lib.check(_lib.lib.tq_decompress_values(
            idx.data_ptr(), compressed["vec_norms"].data_ptr(), B * H * S, D, self.Pi.data_ptr(),
            self.centroids.data_ptr(), self.bits, out.data_ptr(), _stream_ptr(idx.device)))
        return out


def _mask_args(attention_mask, B: int, Sq: int, Sk: int, dev):
    """A mask broadcastable to [B, 1, Sq, Sk] as (tensor, pointer, batch stride, row stride) of an additive
    fp32 tensor with unit inner stride; (None, None, 0, 0) for no mask.

    Floating-point masks are additive (0 = visible, large negative = hidden), as HF's eager path builds them.
    Boolean masks mean True = visible, which is what HF's sdpa path hands over for padded batches; they are
    turned into the additive form here.  Integer masks are refused: their meaning would be a guess."""
    if attention_mask is None:
        return None, None, 0, 0
    mk = attention_mask
    if mk.dim() == 4:
        if mk.shape[1] != 1:
            raise ValueError("per-head masks are not supported; expected [B, 1, Sq, Sk]")
        mk = mk[:, 0]
    elif mk.dim() == 2:
        mk = mk.unsqueeze(0)
    if mk.dtype == torch.bool:
        keep = mk.to(device=dev)
        mk = torch.zeros(keep.shape, dtype=torch.float32, device=dev).masked_fill_(~keep, torch.finfo(torch.float32).min)
    elif mk.dtype.is_floating_point:
        mk = mk.to(device=dev, dtype=torch.float32)
    else:
        raise TypeError(f"attention mask of dtype {mk.dtype} is ambiguous: pass a bool mask (True = visible) or an "
                        "additive floating-point mask")
    if mk.shape[-2:] != (Sq, Sk) or mk.shape[0] not in (1, B):
        raise ValueError(f"mask shape {tuple(attention_mask.shape)} does not broadcast to [B,1,{Sq},{Sk}]")
    if mk.stride(-1) != 1:
        mk = mk.contiguous()
    return mk, mk.data_ptr(), (mk.stride(0) if mk.shape[0] == B and B > 1 else 0), mk.stride(1)


@torch.no_grad()
def fused_attention(q: torch.Tensor, compressed_k: dict, compressed_v: dict,
                    key_compressor: TurboQuantCompressorV2, val_compressor: TurboQuantCompressorMSE,
                    causal: bool = True, attention_mask: torch.Tensor | None = None,
                    sm_scale: float | None = None, mode: str | None = None) -> torch.Tensor:
    """softmax(scores * sm_scale + mask) @ V_hat from packed K and V: the attention core of
    the family adapters (families/llama.py:100-114 of the reference) as one fused pass.

    q [B, Hq, Sq, D]; the compressed tensors hold Hkv heads with Hq % Hkv == 0 (query head h
    reads KV head h // (Hq // Hkv), the `repeat_interleave` grouping).  `attention_mask` is an
    optional additive mask broadcastable to [B, 1, Sq, Sk].  Returns [B, Hq, Sq, D] in q.dtype (stored
    position-major, i.e. contiguous after `.transpose(1, 2)`).
    """
    _require_cuda(q, "q")
    key_compressor._check_device(q)
    val_compressor._check_device(q)
    B, Hq, Sq, D = q.shape
    Bk, Hkv, Sk, Dk = compressed_k["shape"]
    if compressed_v["shape"] != compressed_k["shape"] or (Bk, Dk) != (B, D):
        raise ValueError("q, compressed keys and compressed values disagree on shape")
    if key_compressor.bits != val_compressor.bits:
        raise ValueError("key and value compressors must use the same bit width")
    compressed_k, compressed_v = _dense_packed(compressed_k, _KEY_ARRAYS), _dense_packed(compressed_v, _VALUE_ARRAYS)
    qv = _rows_view(q)
    dev = qv.device
    m = resolve_mode(qv.dtype, mode or key_compressor.mode)
    # [B, Hq, Sq, D] as a view of a [B, Sq, Hq, D] buffer: the adapters' `out.transpose(1, 2).reshape(B, Sq, Hq * D)`
    # in front of the output projection is then a view, not a copy (the kernels write through the strides)
    out = torch.empty((B, Sq, Hq, D), dtype=qv.dtype, device=dev).transpose(1, 2)
    consts = prepared_constants(key_compressor, val_compressor)
    ws = _workspace(dev, _lib.lib.tq_attention_prepared_workspace_bytes(B, Hq, Sq, Hkv, Sk, Sk, D, m))
    mk, mask_ptr, msb, msq = _mask_args(attention_mask, B, Sq, Sk, dev)  # mk keeps the converted mask alive
    scale = float(sm_scale) if sm_scale is not None else 1.0 / math.sqrt(D)
    _lib.check(_lib.lib.tq_attention_fwd_prepared(
        qv.data_ptr(), _DTYPES[qv.dtype], B, Hq, Sq, D, qv.stride(0), qv.stride(1), qv.stride(2), Hkv, Sk, Sk,
        compressed_k["packed_key_indices"].data_ptr(), compressed_k["packed_qjl_signs"].data_ptr(),
        compressed_k["vec_norms"].data_ptr(), compressed_k["residual_norm"].data_ptr(),
        compressed_v["packed_indices"].data_ptr(), compressed_v["vec_norms"].data_ptr(),
        consts.data_ptr(), key_compressor.bits, scale, 1 if causal else 0, mask_ptr, msb, msq,
        out.data_ptr(), out.stride(0), out.stride(1), out.stride(2),
        ws.data_ptr(), ws.numel(), m, _stream_ptr(dev)))
    return out


def device_fault_count(device=None) -> int:
    """Expired bounded device-side waits since the library was loaded (0 when healthy)."""
    import ctypes

    n = ctypes.c_int64(0)
    dev = torch.device(device if device is not None else "cuda")
    with torch.cuda.device(dev):  # the counter read is the one call that goes by the current device
        _lib.check(_lib.lib.tq_device_fault_count(_stream_ptr(dev), ctypes.byref(n)))
    return int(n.value)
