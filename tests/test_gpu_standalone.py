"""Standalone quantiser API on the GPU against the reference's CPU outputs (tests/golden/standalone.npz,
made by tests/golden/make_golden.py) and the oracle's wire format.

The d x d rotation runs as a GPU matmul, whose rounding differs from the CPU's in the last bit, so a
coordinate within ~1e-6 of a decision boundary may take the neighbouring index, and a sketch projection
within ~1e-5 of zero the other sign: both are counted and bounded, everything else is exact."""

import os

import numpy as np
import pytest
import torch

from oracle import tq_oracle as orc

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(__file__), "golden", "standalone.npz"))


@pytest.mark.parametrize("b", [1, 2, 3, 4, 8])
def test_pack_unpack_quantize_dequantize_wrappers(b):
    from turboquant_b200.kernels import lloyd_max_dequantize, lloyd_max_quantize, pack_bits, unpack_bits
    rng = np.random.default_rng(b)
    idx = rng.integers(0, 1 << b, size=(300, 128), dtype=np.int32)
    packed = pack_bits(torch.from_numpy(idx).cuda(), b)
    assert packed.dtype == torch.uint8 and np.array_equal(packed.cpu().numpy(), orc.pack_bits(idx, b))
    assert np.array_equal(unpack_bits(packed, b, 128).cpu().numpy(), idx)
    if b <= 4:
        from turboquant_b200.scalar_codebook import solve_lloyd_max
        cen, bnd = solve_lloyd_max(128, b)
        y = torch.from_numpy(rng.standard_normal((300, 128)).astype(np.float32) / np.sqrt(128))
        q = lloyd_max_quantize(y.cuda(), bnd.cuda(), b)
        want = torch.searchsorted(bnd, y).numpy().astype(np.int32)
        assert np.array_equal(unpack_bits(q, b, 128).cpu().numpy(), want)
        deq = lloyd_max_dequantize(q, cen.half().cuda(), b, 128)
        assert deq.dtype == torch.float16 and torch.equal(deq.cpu(), cen.half()[torch.from_numpy(want).long()])


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_mse_and_prod_quantisers_match_reference(bits):
    from turboquant_b200 import TurboQuantMSE, TurboQuantProd
    x, y = torch.from_numpy(G["x"]).cuda(), torch.from_numpy(G["y"]).cuda()
    mse = TurboQuantMSE(128, bits, seed=42)
    x_hat, idx = mse(x)
    flips = float((idx.cpu().numpy() != G[f"mse_idx_b{bits}"]).mean())
    assert idx.shape == x.shape and flips < 1e-3, flips
    assert float((x_hat.cpu() - torch.from_numpy(G[f"mse_xhat_b{bits}"])).norm() / torch.from_numpy(G[f"mse_xhat_b{bits}"]).norm()) < 2e-3
    assert torch.equal(mse.dequantize(mse.quantize_packed(x)), mse.dequantize(idx))       # packed and index forms agree

    prod = TurboQuantProd(128, bits, seed=42)
    c = prod.quantize(x)
    same_idx = c["mse_indices"].cpu().numpy() == G[f"prod_idx_b{bits}"]
    rows_ok = same_idx.all(axis=1)                     # rows whose indices all agree have the same residual
    assert rows_ok.mean() > 0.9
    sure = np.abs(G[f"prod_proj_b{bits}"]) > 1e-4
    got_s, want_s = c["qjl_signs"].cpu().numpy().astype(np.int8), G[f"prod_signs_b{bits}"]
    assert np.array_equal(got_s[rows_ok][sure[rows_ok]], want_s[rows_ok][sure[rows_ok]])
    assert np.allclose(c["residual_norm"].cpu().numpy()[rows_ok], G[f"prod_rnorm_b{bits}"][rows_ok], rtol=1e-4)
    ip = prod.inner_product(y, c).cpu().numpy()
    assert np.allclose(ip[rows_ok], G[f"prod_ip_b{bits}"][rows_ok], atol=5e-3)
    # the estimator tracks the true inner products (its variance grows as the bit budget shrinks)
    true_ip = (G["x"] * G["y"]).sum(-1)
    assert np.corrcoef(ip, true_ip)[0, 1] > (0.5 if bits == 2 else 0.8)


def test_kv_cache_matches_reference():
    from turboquant_b200 import TurboQuantKVCache
    x, y = torch.from_numpy(G["x"]).cuda(), torch.from_numpy(G["y"]).cuda()
    cache = TurboQuantKVCache(128, 128, bits=3, seed=42)
    cache.append(x[:40], y[:40])
    cache.append(x[40:], y[40:])
    assert len(cache) == 96
    mem = cache.memory_usage_bits()
    assert [mem["key_bits"], mem["value_bits"], mem["total_bits"], mem["fp16_bits"]] == G["cache_mem"].tolist()
    sc = cache.attention_scores(y[:1]).cpu().numpy()
    assert sc.shape == G["cache_scores"].shape
    assert np.mean(np.abs(sc - G["cache_scores"]) < 5e-3) > 0.9
    vals = cache.get_values().cpu()
    want = torch.from_numpy(G["cache_values"])
    assert float((vals - want).norm() / want.norm()) < 5e-3


def test_kernel_level_scores_from_prerotated_queries(golden_comp):
    """`kernels.asymmetric_attention_scores` takes queries already rotated (q Pi^T) and S_eff."""
    from helpers import device_compressors, oracle_key_dict_to_device, oracle_params, rel_err
    from turboquant_b200.kernels import asymmetric_attention_scores
    d, bits = 128, 3
    kp, _ = oracle_params(d, bits)
    q = torch.from_numpy(golden_comp[f"q_d{d}"])
    k = torch.from_numpy(golden_comp[f"k_d{d}"])
    ok = orc.key_compress(k, kp)
    want = orc.scores_from_packed(q, ok["packed_key_indices"], ok["packed_qjl_signs"], ok["vec_norms"],
                                  ok["residual_norm"], kp, ok["shape"])
    kc, _ = device_compressors(d, bits)
    dk = oracle_key_dict_to_device(ok)
    B, H, S, _ = ok["shape"]
    q_rot = (q.cuda().float() @ kc.Pi.T)
    import math
    got = asymmetric_attention_scores(
        q_rot, dk["packed_key_indices"].view(B, H, S, -1), dk["packed_qjl_signs"].view(B, H, S, -1),
        dk["residual_norm"], kc.centroids.unsqueeze(0).expand(H, -1), kc.S_eff, dk["vec_norms"], bits,
        math.sqrt(math.pi / 2) / d)
    assert got.shape == want.shape and rel_err(got.cpu(), want) < 1e-5
    twice = asymmetric_attention_scores(
        q_rot, dk["packed_key_indices"].view(B, H, S, -1), dk["packed_qjl_signs"].view(B, H, S, -1),
        dk["residual_norm"], kc.centroids, kc.S_eff, dk["vec_norms"], bits, 2 * math.sqrt(math.pi / 2) / d)
    zero = asymmetric_attention_scores(
        q_rot, dk["packed_key_indices"].view(B, H, S, -1), dk["packed_qjl_signs"].view(B, H, S, -1),
        dk["residual_norm"], kc.centroids, kc.S_eff, dk["vec_norms"], bits, 0.0)
    assert rel_err((twice - zero).cpu(), 2 * (got - zero).cpu()) < 1e-5    # the correction term scales with coeff
