"""Persistent compressed KV cache: tokens appended step by step and attended in place by the split-KV kernel
give what the reference's cache-less flow gives (compress the whole prefix again, attend over it:
src/transformers_turboquant/patch.py:80-81, families/llama.py:100-114)."""

import pytest
import torch

from helpers import (device_compressors, oracle_attention_from_packed, oracle_key_dict_to_device, oracle_params,
                     oracle_value_dict_to_device, rel_err)
from oracle import tq_oracle as orc

pytestmark = pytest.mark.gpu


def _tokens(B, H, S, d, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, H, S, d, generator=g)
    x[..., :4] *= 8.0  # outlier channels, as in LLM keys
    return x.to(torch.bfloat16)


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_generation_loop_matches_recompression(bits):
    from turboquant_b200 import CompressedKVCache, fused_attention
    d, B, Hq, Hkv, prefill, steps, cap = 128, 2, 8, 2, 300, 6, 333
    kc, vc = device_compressors(d, bits, mode="bf16")
    k, v = _tokens(B, Hkv, prefill + steps, d, 1).cuda(), _tokens(B, Hkv, prefill + steps, d, 2).cuda()
    q = _tokens(B, Hq, prefill + steps, d, 3).cuda()
    cache = CompressedKVCache(kc, vc, B, Hkv, cap)
    cache.append(k[:, :, :prefill], v[:, :, :prefill])
    # prefill-sized queries over the cache take the gather path
    want = fused_attention(q[:, :, :prefill], kc.compress(k[:, :, :prefill]), vc.compress(v[:, :, :prefill]), kc, vc)
    assert torch.equal(cache.attend(q[:, :, :prefill]), want)
    for t in range(prefill, prefill + steps):
        cache.append(k[:, :, t:t + 1], v[:, :, t:t + 1])
        assert len(cache) == t + 1
        got = cache.attend(q[:, :, t:t + 1])
        # the reference's flow: everything compressed again, one query row over t + 1 keys
        ck, cv = kc.compress(k[:, :, :t + 1]), vc.compress(v[:, :, :t + 1])
        assert torch.equal(cache.key_indices[:, :, :t + 1].reshape(-1, ck["packed_key_indices"].shape[1]),
                           ck["packed_key_indices"])
        assert torch.equal(cache.value_norms[:, :, :t + 1].reshape(-1), cv["vec_norms"])
        want = fused_attention(q[:, :, t:t + 1], ck, cv, kc, vc, causal=True)
        assert got.shape == want.shape and got.dtype == torch.bfloat16
        assert torch.equal(got, want)  # same kernel, same split of the same bytes; only the row stride differs
    with pytest.raises(ValueError):
        cache.append(k[:, :, :cap], v[:, :, :cap])


@pytest.mark.parametrize("n_keys,Sq", [(1, 1), (5, 1), (63, 2), (130, 4), (1000, 3)])
def test_cached_attention_against_oracle_any_length(n_keys, Sq):
    """Short and ragged caches (the split-KV kernel serves every length when the rows are strided), several new
    positions at once (causal among themselves), against the oracle on the oracle's own packed bytes."""
    from turboquant_b200 import CompressedKVCache
    d, bits, B, Hq, Hkv, cap = 128, 3, 2, 8, 2, 1024
    kp, vp = oracle_params(d, bits)
    kc, vc = device_compressors(d, bits, mode="bf16")
    k, v = _tokens(B, Hkv, n_keys, d, 10 + n_keys), _tokens(B, Hkv, n_keys, d, 20 + n_keys)
    q = _tokens(B, Hq, Sq, d, 30 + n_keys)
    ok, ov = orc.key_compress(k, kp), orc.value_compress(v, vp)
    want = oracle_attention_from_packed(q, ok, ov, kp, vp, causal=True)
    cache = CompressedKVCache(kc, vc, B, Hkv, cap)
    # store the oracle's bytes so that both sides attend over identical packed data
    n = n_keys
    dk, dv = oracle_key_dict_to_device(ok), oracle_value_dict_to_device(ov)
    cache.key_indices[:, :, :n] = dk["packed_key_indices"].view(B, Hkv, n, -1)
    cache.key_signs[:, :, :n] = dk["packed_qjl_signs"].view(B, Hkv, n, -1)
    cache.key_norms[:, :, :n] = dk["vec_norms"].view(B, Hkv, n)
    cache.key_residual_norms[:, :, :n] = dk["residual_norm"].view(B, Hkv, n)
    cache.value_indices[:, :, :n] = dv["packed_indices"].view(B, Hkv, n, -1)
    cache.value_norms[:, :, :n] = dv["vec_norms"].view(B, Hkv, n)
    cache.length = n
    got = cache.attend(q.cuda(), causal=True)
    assert rel_err(got, want) < 1e-2, rel_err(got, want)   # the bf16-mode bound


@pytest.mark.parametrize("Sq", [1, 3])
def test_cached_attention_with_padding_mask(Sq):
    """Left-padded batch: an additive mask (the large negative HF builds) over the cache, in place, against the
    oracle with the same mask."""
    from turboquant_b200 import CompressedKVCache
    d, bits, B, Hq, Hkv, n, cap = 128, 3, 2, 8, 2, 500, 640
    kp, vp = oracle_params(d, bits)
    kc, vc = device_compressors(d, bits, mode="bf16")
    k, v, q = _tokens(B, Hkv, n, d, 41), _tokens(B, Hkv, n, d, 42), _tokens(B, Hq, Sq, d, 43)
    ok, ov = orc.key_compress(k, kp), orc.value_compress(v, vp)
    mask = torch.zeros(B, 1, Sq, n)
    mask[1, :, :, :37] = torch.finfo(torch.float32).min   # sequence 1 starts with 37 padding tokens
    want = oracle_attention_from_packed(q, ok, ov, kp, vp, causal=True, mask=mask)
    cache = CompressedKVCache(kc, vc, B, Hkv, cap)
    dk, dv = oracle_key_dict_to_device(ok), oracle_value_dict_to_device(ov)
    cache.key_indices[:, :, :n] = dk["packed_key_indices"].view(B, Hkv, n, -1)
    cache.key_signs[:, :, :n] = dk["packed_qjl_signs"].view(B, Hkv, n, -1)
    cache.key_norms[:, :, :n] = dk["vec_norms"].view(B, Hkv, n)
    cache.key_residual_norms[:, :, :n] = dk["residual_norm"].view(B, Hkv, n)
    cache.value_indices[:, :, :n] = dv["packed_indices"].view(B, Hkv, n, -1)
    cache.value_norms[:, :, :n] = dv["vec_norms"].view(B, Hkv, n)
    cache.length = n
    got = cache.attend(q.cuda(), causal=True, attention_mask=mask.cuda())
    assert rel_err(got, want) < 1e-2, rel_err(got, want)   # the bf16-mode bound
    unmasked = cache.attend(q.cuda(), causal=True)
    assert rel_err(got[1], unmasked[1]) > 1e-3  # the mask does something


def test_fully_masked_row_averages_uniformly():
    """A query row that sees only masked keys (a padding position) gets the uniform average of the values, as
    with the prefill kernels and a softmax over equal finite scores -- not NaN and not zero."""
    from turboquant_b200 import CompressedKVCache, fused_attention
    d, bits, B, Hq, Hkv, n = 128, 3, 1, 4, 2, 320
    kc, vc = device_compressors(d, bits, mode="bf16")
    k, v, q = _tokens(B, Hkv, n, d, 51).cuda(), _tokens(B, Hkv, n, d, 52).cuda(), _tokens(B, Hq, 1, d, 53).cuda()
    cache = CompressedKVCache(kc, vc, B, Hkv, 400)
    cache.append(k, v)
    mask = torch.full((B, 1, 1, n), torch.finfo(torch.float32).min, device="cuda")
    got = cache.attend(q, causal=True, attention_mask=mask)
    assert torch.isfinite(got).all()
    # uniform weights: every query head of a KV head gets the same mean of the decompressed values
    want = vc.decompress(vc.compress(v)).mean(dim=2, keepdim=True).repeat_interleave(Hq // Hkv, dim=1)
    assert rel_err(got, want) < 2e-2, rel_err(got, want)


@pytest.mark.parametrize("d", [64, 128])
def test_single_token_cache_through_the_gather_path(d):
    """One token per head in a cache with room for more: the prefix gathered for the prefill kernels must be a
    dense copy (for a single token `reshape` alone returns a view whose rows are a whole capacity apart).  fp32
    queries take the gather path at both head dimensions."""
    from turboquant_b200 import CompressedKVCache, compress_kv, fused_attention
    bits, B, Hq, Hkv = 3, 3, 4, 2
    kc, vc = device_compressors(d, bits)
    g = torch.Generator(device="cuda").manual_seed(d)
    k = torch.randn(B, Hkv, 1, d, generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn(B, Hkv, 1, d, generator=g, device="cuda").to(torch.bfloat16)
    q = torch.randn(B, Hq, 1, d, generator=g, device="cuda")
    cache = CompressedKVCache(kc, vc, B, Hkv, 64, device="cuda")
    cache.append(k, v)
    ck, cv = compress_kv(k, v, kc, vc)
    for query, tol in ((q, 1e-6), (q.to(torch.bfloat16), 1e-6 if d == 64 else 1e-2)):
        # same kernel on both sides through the gather path; at head_dim 128 a 16-bit query reads the cache in place
        # with the split-KV kernel instead
        got = cache.attend(query, causal=True)
        want = fused_attention(query, ck, cv, kc, vc, causal=True)
        assert rel_err(got, want) < tol, rel_err(got, want)
    # and the consumers of a compressed dictionary refuse arrays that do not match its shape
    with pytest.raises(ValueError):
        fused_attention(q, dict(ck, packed_key_indices=ck["packed_key_indices"][:-1]), cv, kc, vc)
