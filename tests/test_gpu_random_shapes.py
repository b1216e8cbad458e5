"""Seeded random sweeps over shapes, head groupings, dtypes, layouts and masks: the tensor-core path against the
independent fp32 CUDA-core kernel (both consume the same packed bytes), the compressed cache filled in random
chunks against one-shot compression, and tensor-core compression against the fp32 parity kernels.  (A sweep of
this kind found a one-token cache being gathered as a strided view.)"""

import random

import pytest
import torch

from helpers import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _compressors(d, bits, cache={}):
    from turboquant_b200 import TurboQuantCompressorMSE, TurboQuantCompressorV2
    if (d, bits) not in cache:
        cache[(d, bits)] = (TurboQuantCompressorV2(d, bits, 42, device=DEV), TurboQuantCompressorMSE(d, bits, 10042, device=DEV))
    return cache[(d, bits)]


def test_random_attention_shapes_tensor_core_vs_fp32_kernel():
    from turboquant_b200 import compress_kv, device_fault_count, fused_attention
    rng = random.Random(1)
    for it in range(160):
        d, bits = rng.choice([64, 128]), rng.choice([2, 3, 4])
        Hkv, G, B = rng.choice([1, 2, 3]), rng.choice([1, 2, 3, 4, 5, 8]), rng.choice([1, 2, 3])
        Hq = Hkv * G
        Sk = rng.choice([1, 2, 17, 63, 64, 65, 127, 128, 129, 200, 255, 256, 257, 300, 511, 513, 700, 1025])
        causal = rng.random() < 0.7
        Sq = rng.choice([s for s in [1, 2, 5, 16, 17, 64, 100, 128, 129, Sk] if s <= Sk]) if causal \
            else rng.choice([1, 3, 17, 64, 130, 200])
        dtype = rng.choice([torch.bfloat16, torch.bfloat16, torch.float16])
        g = torch.Generator(device=DEV).manual_seed(it)
        if rng.random() < 0.5:   # the [B, H, S, D] view of a [B, S, H, D] projection output
            q = torch.randn(B, Sq, Hq, d, generator=g, device=DEV).to(dtype).transpose(1, 2)
        else:
            q = torch.randn(B, Hq, Sq, d, generator=g, device=DEV).to(dtype)
        k = torch.randn(B, Hkv, Sk, d, generator=g, device=DEV).to(dtype)
        v = torch.randn(B, Hkv, Sk, d, generator=g, device=DEV).to(dtype)
        kc, vc = _compressors(d, bits)
        ck, cv = compress_kv(k, v, kc, vc)
        mask = None
        if rng.random() < 0.3:
            mask = torch.zeros(B, 1, Sq, Sk, device=DEV)
            pad = rng.randint(0, max(0, Sk - 1) // 2)
            if pad:
                mask[-1, :, :, :pad] = torch.finfo(torch.float32).min
        a = fused_attention(q, ck, cv, kc, vc, causal=causal, attention_mask=mask, mode="bf16")
        b = fused_attention(q, ck, cv, kc, vc, causal=causal, attention_mask=mask, mode="fp32")
        case = (it, d, bits, B, Hq, Hkv, Sq, Sk, causal, dtype, mask is not None)
        assert torch.isfinite(a).all(), case
        assert rel_err(a, b) < 1e-2, (case, rel_err(a, b))
    assert device_fault_count(DEV) == 0


def test_random_cache_chunks_against_one_shot_compression():
    from turboquant_b200 import CompressedKVCache, compress_kv, fused_attention
    rng = random.Random(3)
    for it in range(60):
        d, bits = rng.choice([64, 128]), rng.choice([2, 3, 4])
        Hkv, G, B = rng.choice([1, 2, 4]), rng.choice([1, 2, 4, 8]), rng.choice([1, 2, 3])
        total, dtype = rng.choice([5, 64, 129, 300, 700]), rng.choice([torch.bfloat16, torch.float16])
        kc, vc = _compressors(d, bits)
        g = torch.Generator(device=DEV).manual_seed(it)
        k = torch.randn(B, Hkv, total, d, generator=g, device=DEV).to(dtype)
        v = torch.randn(B, Hkv, total, d, generator=g, device=DEV).to(dtype)
        cache = CompressedKVCache(kc, vc, B, Hkv, total + rng.randint(0, 100), device=DEV)
        pos = 0
        while pos < total:
            n = min(rng.choice([1, 1, 2, 7, 64, 200]), total - pos)
            cache.append(k[:, :, pos:pos + n], v[:, :, pos:pos + n])
            pos += n
            if rng.random() < 0.5 or pos == total:
                Sq = min(n, rng.choice([1, 1, 2, n]))
                q = torch.randn(B, Hkv * G, Sq, d, generator=g, device=DEV).to(dtype)
                got = cache.attend(q, causal=True)
                ck, cv = compress_kv(k[:, :, :pos], v[:, :, :pos], kc, vc)
                want = fused_attention(q, ck, cv, kc, vc, causal=True, mode="fp32")
                case = (it, d, bits, B, Hkv * G, Hkv, total, pos, Sq, dtype)
                assert torch.isfinite(got).all(), case
                assert rel_err(got, want) < 1e-2, (case, rel_err(got, want))


def test_random_compression_layouts_tensor_core_vs_fp32_kernels():
    from turboquant_b200 import compress_kv
    rng = random.Random(11)

    def differ(a, b):
        return float((a != b).float().mean())

    for it in range(80):
        d, bits = rng.choice([64, 128]), rng.choice([2, 3, 4])
        H, B = rng.choice([1, 2, 3, 8]), rng.choice([1, 2, 3])
        S = rng.choice([1, 2, 63, 127, 128, 129, 255, 257, 300, 1000, 2049])
        dtype = rng.choice([torch.bfloat16, torch.bfloat16, torch.float16])
        layout = rng.choice(["bhsd", "bshd", "padded"])
        g = torch.Generator(device=DEV).manual_seed(it)

        def states():
            if layout == "bhsd":
                return torch.randn(B, H, S, d, generator=g, device=DEV).to(dtype)
            if layout == "bshd":
                return torch.randn(B, S, H, d, generator=g, device=DEV).to(dtype).transpose(1, 2)
            return torch.randn(B, H, S + 5, d + 16, generator=g, device=DEV).to(dtype)[:, :, 2:2 + S, 8:8 + d]

        k, v = states(), states()
        kc, vc = _compressors(d, bits)
        ck, cv = compress_kv(k, v, kc, vc)                                             # tensor-core mode
        ck2, cv2 = compress_kv(k.float().contiguous(), v.float().contiguous(), kc, vc)  # fp32 parity kernels
        case = (it, d, bits, B, H, S, dtype, layout)
        # index bytes differ only where a coordinate sits within rounding of a boundary; sign bits likewise
        assert differ(ck["packed_key_indices"], ck2["packed_key_indices"]) < 2e-3, case
        assert differ(cv["packed_indices"], cv2["packed_indices"]) < 2e-3, case
        assert differ(ck["packed_qjl_signs"], ck2["packed_qjl_signs"]) < 2e-2, case
        for a, b in ((ck["vec_norms"], ck2["vec_norms"]), (ck["residual_norm"], ck2["residual_norm"]),
                     (cv["vec_norms"], cv2["vec_norms"])):
            assert float((a.float() - b.float()).abs().max() / b.float().abs().max()) < 2e-3, case
