"""Host side of the standalone quantiser API (solver, names, argument checks) against the reference's
own values (tests/golden/constants.npz, standalone.npz).  No GPU needed."""

import numpy as np
import pytest
import torch


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("bits", [1, 2, 3, 4])
def test_solver_matches_reference_to_the_bit(d, bits, golden_constants):
    from turboquant_b200.scalar_codebook import solve_lloyd_max
    cen, bnd = solve_lloyd_max(d, bits)
    assert cen.dtype == torch.float32 and bnd.dtype == torch.float32
    assert np.array_equal(cen.numpy(), golden_constants[f"lm_centroids_d{d}_b{bits}"])
    assert np.array_equal(bnd.numpy(), golden_constants[f"lm_boundaries_d{d}_b{bits}"])
    assert np.allclose(cen.numpy(), -cen.numpy()[::-1], atol=1e-7)          # symmetric codebook


def test_exact_beta_codebook_is_close_to_the_gaussian_one():
    from turboquant_b200.scalar_codebook import solve_lloyd_max
    g, _ = solve_lloyd_max(128, 3)
    e, _ = solve_lloyd_max(128, 3, use_exact=True)
    assert e.shape == g.shape and float((e - g).abs().max()) < 2e-3 and float((e - g).abs().max()) > 0


def test_codebook_cpu_semantics_and_distortion():
    from turboquant_b200.scalar_codebook import LloydMaxCodebook
    g = np.load(__import__("os").path.join(__import__("os").path.dirname(__file__), "golden", "standalone.npz"))
    cb = LloydMaxCodebook(128, 3)
    assert cb.n_levels == 8 and abs(cb.distortion - float(g["codebook_distortion_d128_b3"])) < 1e-12
    x = torch.from_numpy(g["x"])
    idx = cb.quantize(x)                      # CPU tensors: the reference's integer-index contract
    assert np.array_equal(idx.numpy().astype(np.int32), g["codebook_idx"])
    assert torch.equal(cb.dequantize(idx), cb.centroids[idx])
    assert "LloydMaxCodebook(d=128, bits=3" in repr(cb)


def test_reference_import_names_resolve():
    import turboquant_pytorch as tp
    from turboquant_pytorch.kernels import (asymmetric_attention_scores, lloyd_max_dequantize,  # noqa: F401
                                            lloyd_max_quantize, pack_bits, unpack_bits)
    from turboquant_pytorch.lloyd_max import LloydMaxCodebook, solve_lloyd_max  # noqa: F401
    from turboquant_pytorch.turboquant import TurboQuantKVCache, TurboQuantMSE, TurboQuantProd  # noqa: F401
    for name in ("TurboQuantMSE", "TurboQuantProd", "TurboQuantKVCache", "LloydMaxCodebook", "solve_lloyd_max",
                 "TurboQuantCompressorV2", "TurboQuantCompressorMSE"):
        assert hasattr(tp, name)


def test_rotation_and_sketch_generators_match_reference_constants():
    from turboquant_b200.quantizers import generate_qjl_matrix, generate_rotation_matrix
    pi = generate_rotation_matrix(128, seed=42, device="cpu")
    assert np.allclose(pi[0, :4].numpy(), [0.174885, 0.120727, 0.085467, -0.145567], atol=1e-6)
    assert torch.allclose(pi @ pi.T, torch.eye(128), atol=1e-5)
    s = generate_qjl_matrix(128, seed=10042, device="cpu")
    assert np.allclose(s[0, :4].numpy(), [1.190396, -0.725117, 0.403278, 0.173541], atol=1e-6)


def test_kernels_refuse_cpu_tensors_and_bad_shapes():
    from turboquant_b200 import kernels as k
    with pytest.raises((RuntimeError, ValueError)):
        k.pack_bits(torch.zeros(4, 128, dtype=torch.int32), 3)           # not on a CUDA device
    with pytest.raises((RuntimeError, ValueError)):
        k.lloyd_max_quantize(torch.zeros(4, 128), torch.zeros(7), 3)
