"""Fused compression kernels against the reference-generated fixtures and the oracle."""

import numpy as np
import pytest
import torch

from helpers import device_compressors, oracle_params
from oracle import tq_oracle as orc

pytestmark = pytest.mark.gpu


def _bit_mismatch(a: np.ndarray, b: np.ndarray) -> float:
    return float(np.unpackbits(np.bitwise_xor(a, b)).mean())


def _index_mismatch(packed_a, packed_b, bits, d) -> float:
    ia = orc.unpack_bits(packed_a, bits, d)
    ib = orc.unpack_bits(packed_b, bits, d)
    assert np.abs(ia - ib).max() <= 1, "an index moved by more than one level"
    return float((ia != ib).mean())


def _fp16_close(a: torch.Tensor, b: torch.Tensor, ulps=1) -> bool:
    """fp16 values equal up to `ulps` units in the last place (norms are reduced in a
    different order on the GPU)."""
    ai = a.cpu().contiguous().view(torch.int16).int()
    bi = b.cpu().contiguous().view(torch.int16).int()
    return int((ai - bi).abs().max()) <= ulps


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("bits", [2, 3, 4])
def test_compress_matches_reference_fixture(d, bits, golden_comp):
    """Same fp32 inputs (zero vector and outlier channel included) as the reference run."""
    tag = f"d{d}_bits{bits}"
    k = torch.from_numpy(golden_comp[f"k_d{d}"]).cuda()
    v = torch.from_numpy(golden_comp[f"v_d{d}"]).cuda()
    kc, vc = device_compressors(d, bits, mode="fp32")
    ck, cv = kc.compress(k), vc.compress(v)
    B, H, S, _ = k.shape
    assert ck["shape"] == (B, H, S, d) and ck["packed_key_indices"].shape == (B * H * S, d * (bits - 1) // 8)
    assert ck["packed_qjl_signs"].shape == (B * H * S, d // 8) and ck["vec_norms"].dtype == torch.float16
    # indices: bit-exact
    assert np.array_equal(ck["packed_key_indices"].cpu().numpy(), golden_comp[f"packed_idx_{tag}"])
    ref_v = orc.pack_bits(golden_comp[f"v_indices_{tag}"].astype(np.int32), bits)
    assert np.array_equal(cv["packed_indices"].cpu().numpy(), ref_v)
    # QJL sign bits: equal except where the projection is ~0 (the zero vector's 'd' bits are
    # sign(0) >= 0 on both sides); allow a 1e-4 fraction for near-zero projections
    assert _bit_mismatch(ck["packed_qjl_signs"].cpu().numpy(), golden_comp[f"packed_sgn_{tag}"]) <= 1e-4
    assert _fp16_close(ck["residual_norm"], torch.from_numpy(golden_comp[f"residual_norm_{tag}"]))
    assert _fp16_close(cv["vec_norms"], torch.from_numpy(golden_comp[f"v_norms_{tag}"]))
    # value decompression
    rec = vc.decompress(cv)
    assert rec.shape == (B, H, S, d) and rec.dtype == torch.float32
    ref = torch.from_numpy(golden_comp[f"v_recon_{tag}"])
    assert float((rec.cpu() - ref).abs().max()) <= 2e-3 * float(ref.abs().max())  # 1 fp16 ulp of the norm


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d,bits", [(128, 2), (128, 3), (128, 4), (64, 3)])
def test_compress_vs_oracle_random(dtype, d, bits):
    """[2, 4, 257, d] in every input type, with outlier channels; strided (transposed) input."""
    g = torch.Generator().manual_seed(11)
    B, H, S = 2, 4, 257
    k = torch.randn(B, S, H, d, generator=g)
    k[..., 5] *= 8
    v = torch.randn(B, S, H, d, generator=g)
    k, v = k.to(dtype), v.to(dtype)
    kp, vp = oracle_params(d, bits)
    ok = orc.key_compress(k.transpose(1, 2), kp)
    ov = orc.value_compress(v.transpose(1, 2), vp)
    kc, vc = device_compressors(d, bits, mode="fp32")
    ck = kc.compress(k.cuda().transpose(1, 2))      # non-contiguous view, read in place
    cv = vc.compress(v.cuda().transpose(1, 2))
    n_coord = B * H * S * d
    mk = _index_mismatch(ck["packed_key_indices"].cpu().numpy(), ok["packed_key_indices"], bits - 1, d)
    mv = _index_mismatch(cv["packed_indices"].cpu().numpy(), ov["packed_indices"], bits, d)
    assert mk <= 2.0 / n_coord + 1e-6 and mv <= 2.0 / n_coord + 1e-6, (mk, mv)
    assert _bit_mismatch(ck["packed_qjl_signs"].cpu().numpy(), ok["packed_qjl_signs"]) <= 5e-5
    assert _fp16_close(ck["vec_norms"], ok["vec_norms"]) and _fp16_close(ck["residual_norm"], ok["residual_norm"])
    assert _fp16_close(cv["vec_norms"], ov["vec_norms"])


@pytest.mark.parametrize("S", [1, 7, 63, 64, 65, 129])
def test_compress_ragged_lengths(S):
    d, bits = 128, 3
    g = torch.Generator().manual_seed(S)
    k = torch.randn(1, 3, S, d, generator=g)
    kp, vp = oracle_params(d, bits)
    kc, vc = device_compressors(d, bits, mode="fp32")
    ck, cv = kc.compress(k.cuda()), vc.compress(k.cuda())
    ok, ov = orc.key_compress(k, kp), orc.value_compress(k, vp)
    assert np.array_equal(ck["packed_key_indices"].cpu().numpy(), ok["packed_key_indices"])
    assert np.array_equal(cv["packed_indices"].cpu().numpy(), ov["packed_indices"])
    assert _bit_mismatch(ck["packed_qjl_signs"].cpu().numpy(), ok["packed_qjl_signs"]) <= 1e-3


def test_compress_empty_and_zero_vectors():
    kc, vc = device_compressors(128, 3, mode="fp32")
    e = kc.compress(torch.zeros(2, 0, 5, 128, device="cuda"))
    assert e["packed_key_indices"].shape == (0, 32) and e["shape"] == (2, 0, 5, 128)
    z = kc.compress(torch.zeros(1, 1, 3, 128, device="cuda"))
    kp, _ = oracle_params(128, 3)
    oz = orc.key_compress(torch.zeros(1, 1, 3, 128), kp)
    assert np.array_equal(z["packed_key_indices"].cpu().numpy(), oz["packed_key_indices"])
    assert np.array_equal(z["packed_qjl_signs"].cpu().numpy(), oz["packed_qjl_signs"])
    assert float(z["vec_norms"].float().abs().max()) == 0.0 and float(z["residual_norm"].float().abs().max()) == 0.0


@pytest.mark.parametrize("d,bits", [(128, 2), (128, 3), (128, 4), (64, 2), (64, 3), (64, 4)])
def test_tensor_core_compress_vs_oracle(d, bits):
    """bf16 inputs in bf16 mode run the tcgen05 kernel (rotation and sketch as split-bf16 MMAs).  Its
    operands carry ~16 mantissa bits, so a coordinate within ~1e-6 of a boundary may move by one
    level and a projection within rounding of zero may flip its sign bit: bounded here."""
    g = torch.Generator().manual_seed(100 + d + bits)
    B, H, S = 2, 3, 1500                       # 9000 vectors: ragged last tile, several tiles per CTA
    k = torch.randn(B, S, H, d, generator=g)
    k[..., 7] *= 8
    k[0, 5] = 0.0                              # zero vectors
    v = torch.randn(B, S, H, d, generator=g)
    k, v = k.to(torch.bfloat16), v.to(torch.bfloat16)
    kp, vp = oracle_params(d, bits)
    ok = orc.key_compress(k.transpose(1, 2), kp)
    ov = orc.value_compress(v.transpose(1, 2), vp)
    kc, vc = device_compressors(d, bits, mode="bf16")
    ck = kc.compress(k.cuda().transpose(1, 2))   # strided view, read in place
    cv = vc.compress(v.cuda().transpose(1, 2))
    mk = _index_mismatch(ck["packed_key_indices"].cpu().numpy(), ok["packed_key_indices"], bits - 1, d)
    mv = _index_mismatch(cv["packed_indices"].cpu().numpy(), ov["packed_indices"], bits, d)
    assert mk <= 3e-5 and mv <= 3e-5, (mk, mv)
    assert _bit_mismatch(ck["packed_qjl_signs"].cpu().numpy(), ok["packed_qjl_signs"]) <= 2e-4
    assert _fp16_close(ck["vec_norms"], ok["vec_norms"]) and _fp16_close(ck["residual_norm"], ok["residual_norm"])
    assert _fp16_close(cv["vec_norms"], ov["vec_norms"])
    # and against the fp32 kernel on the same device data
    kc32, vc32 = device_compressors(d, bits, mode="fp32")
    c32 = kc32.compress(k.cuda().transpose(1, 2))
    assert _index_mismatch(ck["packed_key_indices"].cpu().numpy(), c32["packed_key_indices"].cpu().numpy(), bits - 1, d) <= 3e-5


@pytest.mark.parametrize("S", [1, 127, 128, 129])
def test_tensor_core_compress_ragged(S):
    d, bits = 128, 3
    k = torch.randn(1, 2, S, d, generator=torch.Generator().manual_seed(S)).to(torch.bfloat16)
    kp, vp = oracle_params(d, bits)
    kc, vc = device_compressors(d, bits, mode="bf16")
    ck, cv = kc.compress(k.cuda()), vc.compress(k.cuda())
    ok, ov = orc.key_compress(k, kp), orc.value_compress(k, vp)
    assert _index_mismatch(ck["packed_key_indices"].cpu().numpy(), ok["packed_key_indices"], bits - 1, d) <= 1e-3
    assert _index_mismatch(cv["packed_indices"].cpu().numpy(), ov["packed_indices"], bits, d) <= 1e-3
    assert _bit_mismatch(ck["packed_qjl_signs"].cpu().numpy(), ok["packed_qjl_signs"]) <= 2e-3


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_fused_kv_launch_equals_one_sided_launches(bits):
    """`compress_kv` (keys and values in one launch: every CTA walks key tiles, swaps its constant operands, then
    walks value tiles) gives the bytes of the two one-sided calls, on more tiles than there are SMs, a ragged
    last tile per head and strided [B, S, H, d] inputs; and the oracle's within the tensor-core bounds."""
    from turboquant_b200 import compress_kv
    d, B, H, S = 128, 2, 8, 4100               # 2 x 8 x 33 = 528 tiles per side
    g = torch.Generator().manual_seed(bits)
    k = torch.randn(B, S, H, d, generator=g)
    k[..., 3] *= 8
    v = torch.randn(B, S, H, d, generator=g)
    k, v = k.to(torch.bfloat16).cuda().transpose(1, 2), v.to(torch.bfloat16).cuda().transpose(1, 2)
    kc, vc = device_compressors(d, bits, mode="bf16")
    ck, cv = compress_kv(k, v, kc, vc)
    ck1, cv1 = kc.compress(k), vc.compress(v)
    for name in ("packed_key_indices", "packed_qjl_signs", "vec_norms", "residual_norm"):
        assert torch.equal(ck[name], ck1[name]), name
    for name in ("packed_indices", "vec_norms"):
        assert torch.equal(cv[name], cv1[name]), name
    # one (batch, head) against the oracle
    kp, vp = oracle_params(d, bits)
    ok = orc.key_compress(k[1:2, 5:6].cpu(), kp)
    ov = orc.value_compress(v[1:2, 5:6].cpu(), vp)
    sel = slice((1 * H + 5) * S, (1 * H + 6) * S)
    assert _index_mismatch(ck["packed_key_indices"][sel].cpu().numpy(), ok["packed_key_indices"], bits - 1, d) <= 1e-4
    assert _index_mismatch(cv["packed_indices"][sel].cpu().numpy(), ov["packed_indices"], bits, d) <= 1e-4
    assert _bit_mismatch(ck["packed_qjl_signs"][sel].cpu().numpy(), ok["packed_qjl_signs"]) <= 5e-4
    assert _fp16_close(ck["vec_norms"][1, 5], ok["vec_norms"][0, 0]) and _fp16_close(cv["vec_norms"][sel], ov["vec_norms"])


def test_prepared_constants_follow_replaced_tensors():
    """The per-pair constants buffer is rebuilt when a compressor's constant is replaced (tests overwrite them
    with the oracle's) and reused otherwise."""
    from turboquant_b200 import TurboQuantCompressorMSE, TurboQuantCompressorV2, prepared_constants
    kc = TurboQuantCompressorV2(128, 3, 42, device="cuda")
    vc = TurboQuantCompressorMSE(128, 3, 10042, device="cuda")
    a = prepared_constants(kc, vc)
    assert prepared_constants(kc, vc) is a
    x = torch.randn(1, 1, 64, 128, device="cuda").to(torch.bfloat16)
    before = kc.compress(x)["packed_key_indices"].clone()
    kc.Pi = kc.Pi.flip(0).contiguous()          # another rotation
    assert prepared_constants(kc, vc) is not a
    assert not torch.equal(kc.compress(x)["packed_key_indices"], before)
