"""Wire-format kernels on the GPU against the golden fixtures and the oracle: bit-exact."""

import numpy as np
import pytest
import torch

from oracle import tq_oracle as orc

pytestmark = pytest.mark.gpu


def _lib():
    from turboquant_b200 import _lib
    return _lib


def _stream():
    return torch.cuda.current_stream().cuda_stream


def gpu_pack(idx: np.ndarray, b: int) -> np.ndarray:
    L = _lib()
    n, d = idx.shape
    src = torch.from_numpy(idx.astype(np.int32)).cuda()
    out = torch.empty((n, d * b // 8), dtype=torch.uint8, device="cuda")
    L.check(L.lib.tq_pack_bits(src.data_ptr(), n, d, b, out.data_ptr(), _stream()))
    return out.cpu().numpy()


def gpu_unpack(packed: np.ndarray, b: int, d: int) -> np.ndarray:
    L = _lib()
    n = packed.shape[0]
    src = torch.from_numpy(packed).cuda()
    out = torch.empty((n, d), dtype=torch.int32, device="cuda")
    L.check(L.lib.tq_unpack_bits(src.data_ptr(), n, d, b, out.data_ptr(), _stream()))
    return out.cpu().numpy()


@pytest.mark.parametrize("b", range(1, 9))
def test_pack_unpack_golden(b, golden_wire):
    idx = golden_wire[f"idx_b{b}"].astype(np.int32)
    packed = gpu_pack(idx, b)
    assert np.array_equal(packed, golden_wire[f"packed_b{b}"])
    assert np.array_equal(gpu_unpack(packed, b, idx.shape[1]), idx)


@pytest.mark.parametrize("b", [1, 2, 3, 4])
@pytest.mark.parametrize("n,d", [(1, 64), (7, 128), (1000, 128), (4097, 64)])
def test_pack_random_and_extremes(b, n, d):
    rng = np.random.default_rng(b * 1000 + n)
    idx = rng.integers(0, 1 << b, size=(n, d), dtype=np.int32)
    idx[0, :] = (1 << b) - 1
    idx[-1, :] = 0
    packed = gpu_pack(idx, b)
    assert np.array_equal(packed, orc.pack_bits(idx, b))
    assert np.array_equal(gpu_unpack(packed, b, d), idx)


def test_pack_known_byte_and_empty():
    assert gpu_pack(np.array([[0xA, 0x5] + [0] * 6], dtype=np.int32), 4)[0, 0] == 0x5A
    L = _lib()
    assert L.lib.tq_pack_bits(None, 0, 128, 3, None, _stream()) == 0


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("b_eff", [1, 2, 3, 4])
def test_quantize_dequantize_golden(d, b_eff, golden_wire, golden_constants):
    """Bit-exact on identical fp32 rotated inputs, exact boundary hits and zeros included."""
    L = _lib()
    rot = torch.from_numpy(golden_wire[f"rot_d{d}_b{b_eff}"]).cuda()
    bounds = torch.from_numpy(golden_constants[f"lm_boundaries_d{d}_b{b_eff}"]).cuda()
    cents = torch.from_numpy(golden_constants[f"lm_centroids_d{d}_b{b_eff}"]).cuda()
    n = rot.shape[0]
    out = torch.empty((n, d * b_eff // 8), dtype=torch.uint8, device="cuda")
    L.check(L.lib.tq_quantize_rotated(rot.data_ptr(), n, d, bounds.data_ptr(), b_eff, out.data_ptr(), _stream()))
    assert np.array_equal(out.cpu().numpy(), golden_wire[f"qpacked_d{d}_b{b_eff}"])
    deq = torch.empty((n, d), dtype=torch.float32, device="cuda")
    L.check(L.lib.tq_dequantize(out.data_ptr(), n, d, cents.data_ptr(), b_eff, deq.data_ptr(), _stream()))
    assert np.array_equal(deq.half().cpu().numpy(), golden_wire[f"deq_d{d}_b{b_eff}"])
    assert np.array_equal(deq.cpu().numpy(), orc.dequantize_packed(out.cpu().numpy(), cents.cpu(), b_eff, d).numpy())


@pytest.mark.parametrize("d,b_eff", [(128, 1), (128, 2), (128, 3), (128, 4), (64, 2)])
def test_quantize_large_bit_exact(d, b_eff):
    """4096 x d and a ragged 100003-row case: every packed byte equals the oracle's."""
    L = _lib()
    cents = orc.solve_codebook(d, b_eff)
    bounds = ((cents[:-1] + cents[1:]) / 2).contiguous()
    for n in (4096, 100003 if d == 128 and b_eff == 2 else 513):
        g = torch.Generator().manual_seed(n + b_eff)
        rot = torch.randn(n, d, generator=g) / d ** 0.5
        out = torch.empty((n, d * b_eff // 8), dtype=torch.uint8, device="cuda")
        r = rot.cuda()
        L.check(L.lib.tq_quantize_rotated(r.data_ptr(), n, d, bounds.cuda().data_ptr(), b_eff, out.data_ptr(), _stream()))
        assert np.array_equal(out.cpu().numpy(), orc.quantize_packed(rot, bounds, b_eff))
