"""Helpers shared by the GPU parity tests: oracle parameters, their twins on the device,
and thin wrappers that call the C ABI through ctypes with torch tensors as buffers."""

from __future__ import annotations

import numpy as np
import torch

from oracle import tq_oracle as orc

_PARAM_CACHE: dict = {}


def oracle_params(d: int, bits: int, key_seed: int = 42, val_seed: int = 10042):
    key = (d, bits, key_seed, val_seed)
    if key not in _PARAM_CACHE:
        _PARAM_CACHE[key] = (orc.make_key_params(d, bits, key_seed), orc.make_value_params(d, bits, val_seed))
    return _PARAM_CACHE[key]


def device_compressors(d: int, bits: int, key_seed: int = 42, val_seed: int = 10042, mode=None):
    """Product compressors whose constants are overwritten with the oracle's, so that both
    sides work from identical matrices and codebooks."""
    from turboquant_b200 import TurboQuantCompressorMSE, TurboQuantCompressorV2

    kp, vp = oracle_params(d, bits, key_seed, val_seed)
    kc = TurboQuantCompressorV2(d, bits, key_seed, device="cuda", mode=mode)
    vc = TurboQuantCompressorMSE(d, bits, val_seed, device="cuda", mode=mode)
    # .contiguous(): the Q factor of torch.linalg.qr comes back column-major
    kc.Pi, kc.S, kc.S_eff = kp.Pi.contiguous().cuda(), kp.S.contiguous().cuda(), kp.S_eff.contiguous().cuda()
    kc.PiT = kc.Pi.T.contiguous()
    kc.centroids, kc.boundaries = kp.centroids.contiguous().cuda(), kp.boundaries.contiguous().cuda()
    vc.Pi, vc.PiT = vp.Pi.contiguous().cuda(), vp.Pi.T.contiguous().cuda()
    vc.centroids, vc.boundaries = vp.centroids.contiguous().cuda(), vp.boundaries.contiguous().cuda()
    return kc, vc


def oracle_key_dict_to_device(ck: dict) -> dict:
    """The oracle's packed bytes and fp16 norms as the dict the product consumes."""
    B, H, S, D = ck["shape"]
    return {"packed_key_indices": torch.from_numpy(ck["packed_key_indices"]).cuda(),
            "packed_qjl_signs": torch.from_numpy(ck["packed_qjl_signs"]).cuda(),
            "residual_norm": ck["residual_norm"].cuda().contiguous(),
            "vec_norms": ck["vec_norms"].cuda().contiguous(), "shape": (B, H, S, D)}


def oracle_value_dict_to_device(cv: dict) -> dict:
    return {"packed_indices": torch.from_numpy(cv["packed_indices"]).cuda(),
            "vec_norms": cv["vec_norms"].cuda().contiguous(), "shape": cv["shape"]}


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """Norm-wise relative error ||a-b|| / ||b||."""
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def oracle_attention_from_packed(q, ck, cv, kp, vp, causal=True, mask=None):
    """fp32 attention output computed on the CPU from the oracle's packed bytes:
    softmax(scores/sqrt(d) + mask) @ V_hat, with GQA grouping of heads."""
    B, Hq, Sq, D = q.shape
    Hkv, Sk = ck["shape"][1], ck["shape"][2]
    g = Hq // Hkv
    out = torch.empty(B, Hq, Sq, D)
    vals = orc.values_from_packed(cv["packed_indices"], cv["vec_norms"], vp, cv["shape"])
    idx = ck["packed_key_indices"].reshape(B, Hkv, Sk, -1)
    sgn = ck["packed_qjl_signs"].reshape(B, Hkv, Sk, -1)
    for h in range(Hq):
        j = h // g
        sc = orc.scores_from_packed(q[:, h:h + 1].float(), idx[:, j:j + 1], sgn[:, j:j + 1],
                                    ck["vec_norms"][:, j:j + 1], ck["residual_norm"][:, j:j + 1],
                                    kp, (B, 1, Sk, D))
        sc = sc / D ** 0.5
        if causal:
            sc = sc + orc.causal_mask(Sq, Sk)
        if mask is not None:
            sc = sc + mask
        out[:, h:h + 1] = torch.softmax(sc, dim=-1) @ vals[:, j:j + 1]
    return out
