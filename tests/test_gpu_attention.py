"""Estimator scores and fused attention on the GPU, fed with the ORACLE's packed bytes so
that both sides consume identical compressed data.

Tolerances (norm-wise relative error ||a-b||/||b||): 1e-4 in fp32 mode, 1e-2 in bf16 mode."""

import numpy as np
import pytest
import torch

from helpers import (device_compressors, oracle_attention_from_packed, oracle_key_dict_to_device, oracle_params,
                     oracle_value_dict_to_device, rel_err)
from pathlib import Path

from oracle import tq_oracle as orc

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu
TOL = {"fp32": 1e-4, "bf16": 1e-2}


def _case(B, Hq, Hkv, Sq, Sk, d, seed=0, dtype=torch.float32, outliers=True):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, Sq, d, generator=g).to(dtype)
    k = torch.randn(B, Hkv, Sk, d, generator=g)
    if outliers:
        k[..., torch.randperm(d, generator=g)[:4]] *= 8
    v = torch.randn(B, Hkv, Sk, d, generator=g)
    return q, k.to(dtype), v.to(dtype)


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("bits", [2, 3, 4])
def test_scores_match_reference_fixture(d, bits, golden_comp):
    """Scores from the reference run's own packed bytes vs (a) the fp32 evaluation of the
    estimator and (b) the reference's literal PyTorch-branch scores (fp16 k_mse storage)."""
    tag = f"d{d}_bits{bits}"
    kp, _ = oracle_params(d, bits)
    q = torch.from_numpy(golden_comp[f"q_d{d}"])
    k = torch.from_numpy(golden_comp[f"k_d{d}"])
    ok = orc.key_compress(k, kp)
    kc, _ = device_compressors(d, bits)
    sc = kc.asymmetric_attention_scores(q.cuda(), oracle_key_dict_to_device(ok)).cpu()
    want = orc.scores_from_packed(q, ok["packed_key_indices"], ok["packed_qjl_signs"], ok["vec_norms"],
                                  ok["residual_norm"], kp, ok["shape"])
    assert sc.shape == want.shape and sc.dtype == torch.float32
    assert rel_err(sc, want) < 1e-5
    assert rel_err(sc, torch.from_numpy(golden_comp[f"scores_{tag}"])) < 1e-3    # fp16 k_mse in the literal path
    assert float((sc - torch.from_numpy(golden_comp[f"packed_scores_{tag}"])).abs().max()) < 3e-2  # reference's own bar


@pytest.mark.parametrize("mode", ["fp32", "bf16"])
@pytest.mark.parametrize("d,bits", [(128, 3), (128, 2), (128, 4), (64, 3), (64, 2), (64, 4)])
def test_fused_attention_causal_gqa(mode, d, bits):
    B, Hq, Hkv, S = 2, 4, 2, 200   # two query heads per KV head, ragged tile edge
    dtype = torch.float32 if mode == "fp32" else torch.bfloat16
    q, k, v = _case(B, Hq, Hkv, S, S, d, seed=bits, dtype=dtype)
    kp, vp = oracle_params(d, bits)
    ok, ov = orc.key_compress(k, kp), orc.value_compress(v, vp)
    want = oracle_attention_from_packed(q, ok, ov, kp, vp, causal=True)
    from turboquant_b200 import fused_attention
    kc, vc = device_compressors(d, bits, mode=mode)
    out = fused_attention(q.cuda(), oracle_key_dict_to_device(ok), oracle_value_dict_to_device(ov), kc, vc,
                          causal=True, mode=mode)
    assert out.shape == q.shape and out.dtype == dtype
    assert rel_err(out, want) < TOL[mode], rel_err(out, want)


@pytest.mark.parametrize("mode", ["fp32", "bf16"])
@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("Sq,Sk", [(1, 1), (7, 7), (129, 129), (64, 300), (1, 513), (256, 256)])
def test_fused_attention_shapes(mode, Sq, Sk, d):
    bits = 3
    dtype = torch.float32 if mode == "fp32" else torch.bfloat16
    q, k, v = _case(1, 2, 1, Sq, Sk, d, seed=Sq + Sk, dtype=dtype)
    kp, vp = oracle_params(d, bits)
    ok, ov = orc.key_compress(k, kp), orc.value_compress(v, vp)
    want = oracle_attention_from_packed(q, ok, ov, kp, vp, causal=True)
    from turboquant_b200 import fused_attention
    kc, vc = device_compressors(d, bits, mode=mode)
    out = fused_attention(q.cuda(), oracle_key_dict_to_device(ok), oracle_value_dict_to_device(ov), kc, vc, mode=mode)
    assert rel_err(out, want) < TOL[mode], rel_err(out, want)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("Hq,Hkv", [(4, 2), (3, 3)])
def test_tensor_core_mode_converts_other_dtypes_and_follows_strides(dtype, Hq, Hkv, d):
    """bf16 (tensor-core) mode fed fp16 / fp32 queries laid out [B, S, H, D] (the layout the family
    adapters see before their transpose): the kernel converts the rows itself, follows the strides and
    writes the output in the query dtype.  An odd GQA group pairs position blocks instead of heads."""
    bits, B, S = 3, 2, 300
    q, k, v = _case(B, Hq, Hkv, S, S, d, seed=11, dtype=torch.float32)
    kp, vp = oracle_params(d, bits)
    ok, ov = orc.key_compress(k, kp), orc.value_compress(v, vp)
    q = q.to(dtype)
    want = oracle_attention_from_packed(q, ok, ov, kp, vp, causal=True)
    from turboquant_b200 import fused_attention
    kc, vc = device_compressors(d, bits, mode="bf16")
    q_dev = q.permute(0, 2, 1, 3).contiguous().cuda().permute(0, 2, 1, 3)   # [B, H, S, D] view of [B, S, H, D]
    assert not q_dev.is_contiguous()
    out = fused_attention(q_dev, oracle_key_dict_to_device(ok), oracle_value_dict_to_device(ov), kc, vc,
                          causal=True, mode="bf16")
    assert out.dtype == dtype and out.shape == q.shape
    assert rel_err(out, want) < TOL["bf16"], rel_err(out, want)


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("Sq,Sk,causal", [(1, 256, True), (1, 1000, True), (3, 4097, True), (4, 777, False)])
def test_decode_sized_calls_use_the_split_kv_kernel(bits, Sq, Sk, causal):
    """Few query rows per KV head (G * Sq <= 16) against long keys: the split-KV kernel (packed bytes decoded
    straight into mma.sync fragments) against the oracle, ragged key counts and all bit widths."""
    d, B, Hq, Hkv = 128, 2, 8, 2
    q, k, v = _case(B, Hq, Hkv, Sq, Sk, d, seed=100 * bits + Sq, dtype=torch.bfloat16)
    kp, vp = oracle_params(d, bits)
    ok, ov = orc.key_compress(k, kp), orc.value_compress(v, vp)
    want = oracle_attention_from_packed(q, ok, ov, kp, vp, causal=causal)
    from turboquant_b200 import fused_attention
    kc, vc = device_compressors(d, bits, mode="bf16")
    out = fused_attention(q.cuda(), oracle_key_dict_to_device(ok), oracle_value_dict_to_device(ov), kc, vc,
                          causal=causal, mode="bf16")
    assert out.shape == q.shape and out.dtype == torch.bfloat16
    # norms are applied in fp32 and the sign operand is exact in this kernel: measured 4-6e-3 on these shapes
    assert rel_err(out, want) < TOL["bf16"], rel_err(out, want)


@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("mode", ["fp32", "bf16"])
def test_fused_attention_additive_mask_and_noncausal(mode, d):
    """Padding-style additive mask (finite large negative, as HF builds it) and the
    non-causal path."""
    bits, B, S = 3, 2, 150
    dtype = torch.float32 if mode == "fp32" else torch.bfloat16
    q, k, v = _case(B, 2, 2, S, S, d, seed=5, dtype=dtype)
    kp, vp = oracle_params(d, bits)
    ok, ov = orc.key_compress(k, kp), orc.value_compress(v, vp)
    mask = torch.zeros(B, 1, S, S)
    mask[1, :, :, :17] = torch.finfo(torch.float32).min   # batch 1: first 17 keys are padding
    from turboquant_b200 import fused_attention
    kc, vc = device_compressors(d, bits, mode=mode)
    dk, dv = oracle_key_dict_to_device(ok), oracle_value_dict_to_device(ov)
    want = oracle_attention_from_packed(q, ok, ov, kp, vp, causal=True, mask=mask)
    out = fused_attention(q.cuda(), dk, dv, kc, vc, causal=True, attention_mask=mask.cuda(), mode=mode)
    assert rel_err(out[:, :, 17:], want[:, :, 17:]) < TOL[mode]
    # Rows 0..16 of batch 1 see only masked keys.  Their softmax runs over equal finite scores, so the row is a
    # uniform average: of the keys the causal rule leaves visible here, of all keys in the reference (whose
    # causal mask is the same finite value).  Such rows are padding positions; what matters is that they are
    # finite and that both kernels (prefill and split-KV) treat them the same way.
    vals = orc.values_from_packed(ov["packed_indices"], ov["vec_norms"], vp, ov["shape"])  # [B, Hkv, S, d]
    for row in (0, 5, 16):
        uniform = vals[1, :, :row + 1].mean(dim=1)                                         # [Hkv, d]
        assert rel_err(out[1, :, row], uniform) < 2e-2, (row, rel_err(out[1, :, row], uniform))
    want_nc = oracle_attention_from_packed(q, ok, ov, kp, vp, causal=False)
    out_nc = fused_attention(q.cuda(), dk, dv, kc, vc, causal=False, mode=mode)
    assert rel_err(out_nc, want_nc) < TOL[mode]


@pytest.mark.parametrize("mode", ["fp32", "bf16"])
def test_prepare_queries(mode):
    """q_cat = [q Pi^T | coeff q S^T]: the tensor-core row GEMM against fp32 torch."""
    from turboquant_b200 import _lib as L
    d = 128
    kp, _ = oracle_params(d, 3)
    g = torch.Generator().manual_seed(3)
    dtype = torch.float32 if mode == "fp32" else torch.bfloat16
    q = torch.randn(2, 3, 70, d, generator=g).to(dtype)
    want = torch.cat([q.float() @ kp.Pi.T, orc.qjl_coeff(d) * (q.float() @ kp.S.T)], dim=-1).reshape(-1, 2 * d)
    kc, _ = device_compressors(d, 3)
    qd = q.cuda()
    out = torch.empty((2 * 3 * 70, 2 * d), dtype=dtype, device="cuda")
    ws = torch.empty(4 * d * d, dtype=torch.uint8, device="cuda")
    m = L.TQ_MODE_FP32 if mode == "fp32" else L.TQ_MODE_BF16
    L.check(L.lib.tq_prepare_queries(qd.data_ptr(), 0 if mode == "fp32" else 1, 2, 3, 70, d, qd.stride(0), qd.stride(1),
                                     qd.stride(2), kc.Pi.data_ptr(), kc.S_eff.data_ptr(), out.data_ptr(),
                                     ws.data_ptr(), ws.numel(), m, torch.cuda.current_stream().cuda_stream))
    assert rel_err(out[:, :d], want[:, :d]) < (1e-5 if mode == "fp32" else 6e-3)
    assert rel_err(out[:, d:], want[:, d:]) < (1e-5 if mode == "fp32" else 6e-3)


def test_end_to_end_operator_sequence_vs_reference_fixture(golden_family):
    """compress -> fused attention through the product API on the reference GPT-2 adapter's
    inputs, against the reference adapter's output (fp32, bits 2/3/4)."""
    from turboquant_b200 import TurboQuantCompressorMSE, TurboQuantCompressorV2, fused_attention
    g = golden_family
    hidden = torch.from_numpy(g["hidden"]).cuda()
    qkv = hidden @ torch.from_numpy(g["c_attn_w"]).cuda() + torch.from_numpy(g["c_attn_b"]).cuda()
    B, T, E = hidden.shape
    q, k, v = (t.view(B, T, 2, 64).transpose(1, 2) for t in qkv.split(E, dim=2))
    for bits in (2, 3, 4):
        kc = TurboQuantCompressorV2(64, bits, seed=42, device="cuda")
        vc = TurboQuantCompressorMSE(64, bits, seed=10042, device="cuda")
        out = fused_attention(q, kc.compress(k), vc.compress(v), kc, vc, causal=True,
                              attention_mask=torch.from_numpy(g["mask"]).cuda())
        out = out.transpose(1, 2).reshape(B, T, E) @ torch.from_numpy(g["c_proj_w"]).cuda() + torch.from_numpy(g["c_proj_b"]).cuda()
        # the literal reference stores k_mse in fp16 (2e-4 away from the fp32 estimator)
        assert rel_err(out, torch.from_numpy(g[f"out_bits{bits}"])) < 2e-3


def test_no_device_wait_faults():
    from turboquant_b200 import device_fault_count
    assert device_fault_count() == 0


@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("Hq,Hkv", [(8, 2), (3, 3)])
def test_long_sequence_tensor_core_vs_fp32_kernel_and_oracle(Hq, Hkv, d):
    """S = 4096 (64 key tiles, many ring and barrier-phase wrap-arounds, several CTAs per head; head
    pairs for the even group, position-block pairs for MHA), both head dimensions of the SM-pair kernel:
    the tensor-core kernel against the independent fp32 CUDA-core kernel on the whole output, and against
    the oracle on the last 32 query rows of one head."""
    from turboquant_b200 import fused_attention
    bits, B, S = 3, 2, 4096
    g = torch.Generator(device="cuda").manual_seed(7)
    q = torch.randn(B, Hq, S, d, generator=g, device="cuda").to(torch.bfloat16)
    k = torch.randn(B, Hkv, S, d, generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn(B, Hkv, S, d, generator=g, device="cuda").to(torch.bfloat16)
    kc, vc = device_compressors(d, bits)
    ck, cv = kc.compress(k), vc.compress(v)
    out16 = fused_attention(q, ck, cv, kc, vc, causal=True, mode="bf16")
    out32 = fused_attention(q, ck, cv, kc, vc, causal=True, mode="fp32")
    assert rel_err(out16, out32) < TOL["bf16"], rel_err(out16, out32)
    per_row = ((out16.float() - out32.float()).norm(dim=-1) / out32.float().norm(dim=-1)).max()
    assert float(per_row) < 5e-2, float(per_row)          # no single bad row hides in the aggregate
    # oracle on a slice: batch 1, last query head, last 32 rows, from the product's packed bytes
    kp, vp = oracle_params(d, bits)
    hk = (Hq - 1) // (Hq // Hkv)
    sel = slice((1 * Hkv + hk) * S, (1 * Hkv + hk + 1) * S)
    sc = orc.scores_from_packed(q[1:2, -1:, -32:].float().cpu(), ck["packed_key_indices"][sel].cpu().numpy(),
                                ck["packed_qjl_signs"][sel].cpu().numpy(), ck["vec_norms"][1, hk].cpu(),
                                ck["residual_norm"][1, hk].cpu(), kp, (1, 1, S, d))
    vals = orc.values_from_packed(cv["packed_indices"][sel].cpu().numpy(), cv["vec_norms"][sel].cpu(), vp, (1, 1, S, d))
    want = torch.softmax(sc / d ** 0.5 + orc.causal_mask(S, S)[-32:], -1) @ vals
    assert rel_err(out32[1:2, -1:, -32:], want) < 4e-3   # fp32 arithmetic, but the output is stored as bf16 here
    assert rel_err(out16[1:2, -1:, -32:], want) < TOL["bf16"]


@pytest.mark.parametrize("Sq", [1, 200])
def test_compress_and_attention_replay_from_a_cuda_graph(Sq):
    """The whole path (compress keys, compress values, fused attention; prefill- and decode-sized) is
    capturable: no synchronisation, no allocation inside the library, work on the capture stream only.
    A replay on new inputs in the same buffers reproduces the eager result."""
    from turboquant_b200 import fused_attention
    d, bits, B, Hq, Hkv, Sk = 128, 3, 2, 8, 2, 512
    kc, vc = device_compressors(d, bits, mode="bf16")
    q, k, v = (t.cuda() for t in _case(B, Hq, Hkv, Sq, Sk, d, seed=3, dtype=torch.bfloat16))

    def run():
        return fused_attention(q, kc.compress(k), vc.compress(v), kc, vc, causal=True, mode="bf16")

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            run()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out_g = run()
    q2, k2, v2 = (t.cuda() for t in _case(B, Hq, Hkv, Sq, Sk, d, seed=4, dtype=torch.bfloat16))
    q.copy_(q2); k.copy_(k2); v.copy_(v2)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out_g, run())



@pytest.mark.parametrize("Hq,Hkv,Sq", [(2, 2, 1), (4, 2, 8), (16, 1, 1), (8, 1, 2), (3, 3, 5)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_decode_kernel_group_sizes_and_dtypes(Hq, Hkv, Sq, dtype):
    """The split-KV kernel over the group sizes and row counts it accepts (1 to 16 query rows per KV head, one or
    two tiles of eight), fp16 and bf16 queries, a key count that is odd and not a multiple of the block."""
    d, bits, B, Sk = 128, 3, 2, 1531
    q, k, v = _case(B, Hq, Hkv, Sq, Sk, d, seed=7 * Hq + Sq, dtype=torch.float32)
    kp, vp = oracle_params(d, bits)
    ok, ov = orc.key_compress(k, kp), orc.value_compress(v, vp)
    q = q.to(dtype)
    want = oracle_attention_from_packed(q, ok, ov, kp, vp, causal=True)
    from turboquant_b200 import fused_attention
    kc, vc = device_compressors(d, bits, mode="bf16")
    out = fused_attention(q.cuda(), oracle_key_dict_to_device(ok), oracle_value_dict_to_device(ov), kc, vc,
                          causal=True, mode="bf16")
    assert out.dtype == dtype
    assert rel_err(out, want) < TOL["bf16"], rel_err(out, want)


def _oracle_rows(q, ck, cv, kp, vp, b, h, hk, rows, S, d):
    """Oracle attention output of query rows `rows` (a slice) of head h of batch b, from the product's own packed
    bytes of KV head hk: scores over all S keys, causal mask, softmax, P @ V_hat."""
    Hkv = ck["shape"][1]
    sel = slice((b * Hkv + hk) * S, (b * Hkv + hk + 1) * S)
    sc = orc.scores_from_packed(q[b:b + 1, h:h + 1, rows].float().cpu(), ck["packed_key_indices"][sel].cpu().numpy(),
                                ck["packed_qjl_signs"][sel].cpu().numpy(), ck["vec_norms"][b, hk].cpu(),
                                ck["residual_norm"][b, hk].cpu(), kp, (1, 1, S, d))
    vals = orc.values_from_packed(cv["packed_indices"][sel].cpu().numpy(), cv["vec_norms"][sel].cpu(), vp, (1, 1, S, d))
    return torch.softmax(sc / d ** 0.5 + orc.causal_mask(S, S)[rows], -1) @ vals


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_benchmark_shape_s8192_slices_against_oracle(bits):
    """The benchmarked configuration itself (32 query / 8 KV heads, S = 8192, bf16, four key channels per head
    scaled x8 -- the generator of bench.py), one batch element: rows from the end, the middle and the first tile
    of three heads against the oracle, all bit widths."""
    import bench
    from turboquant_b200 import fused_attention
    d, S = 128, 8192
    q, k, v = bench.make_inputs(1, S, torch.device("cuda"), seed=0)
    kc, vc = device_compressors(d, bits)
    ck, cv = kc.compress(k), vc.compress(v)
    out = fused_attention(q, ck, cv, kc, vc, causal=True, mode="bf16")
    kp, vp = oracle_params(d, bits)
    for h, rows in ((31, slice(S - 32, S)), (13, slice(4100, 4132)), (0, slice(0, 32)), (6, slice(127, 130))):
        want = _oracle_rows(q, ck, cv, kp, vp, 0, h, h // 4, rows, S, d)
        err = rel_err(out[0:1, h:h + 1, rows], want)
        assert err < TOL["bf16"], (bits, h, rows, err)


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_scaling_shape_s32768_slices_against_oracle(bits):
    """S = 32768, the sequence length of the multi-GPU scaling configuration: 256 key tiles per query tile, so the
    staging rings and barrier phases wrap four times as often as at S = 8192.  One batch element with two KV
    heads and their eight query heads; rows near the end (all tiles), in the middle and at a ring wrap-around."""
    from turboquant_b200 import fused_attention
    d, S, Hq, Hkv = 128, 32768, 8, 2
    g = torch.Generator(device="cuda").manual_seed(11)
    q = torch.randn(1, Hq, S, d, generator=g, device="cuda").to(torch.bfloat16)
    k = torch.randn(1, Hkv, S, d, generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn(1, Hkv, S, d, generator=g, device="cuda").to(torch.bfloat16)
    kc, vc = device_compressors(d, bits)
    ck, cv = kc.compress(k), vc.compress(v)
    out = fused_attention(q, ck, cv, kc, vc, causal=True, mode="bf16")
    assert torch.isfinite(out.float()).all()
    kp, vp = oracle_params(d, bits)
    for h, rows in ((7, slice(S - 32, S)), (2, slice(20000, 20016)), (5, slice(128 * 3 * 17, 128 * 3 * 17 + 8))):
        want = _oracle_rows(q, ck, cv, kp, vp, 0, h, h // 4, rows, S, d)
        err = rel_err(out[0:1, h:h + 1, rows], want)
        assert err < TOL["bf16"], (bits, h, rows, err)


def test_boolean_mask_means_visible():
    """HF's sdpa path hands over a boolean mask (True = visible) for padded batches; it must act as the additive
    mask with the large negative value at the False entries, in the prefill and in the split-KV kernel."""
    from turboquant_b200 import fused_attention
    d, bits, B, S = 128, 3, 2, 300
    q, k, v = _case(B, 4, 2, S, S, d, seed=21, dtype=torch.bfloat16)
    kc, vc = device_compressors(d, bits, mode="bf16")
    ck, cv = kc.compress(k.cuda()), vc.compress(v.cuda())
    keep = torch.ones(B, 1, S, S, dtype=torch.bool)
    keep[1, :, :, :23] = False
    additive = torch.zeros(B, 1, S, S).masked_fill_(~keep, torch.finfo(torch.float32).min)
    a = fused_attention(q.cuda(), ck, cv, kc, vc, causal=True, attention_mask=keep.cuda())
    b2 = fused_attention(q.cuda(), ck, cv, kc, vc, causal=True, attention_mask=additive.cuda())
    assert torch.equal(a, b2)
    assert rel_err(a[1, :, 23:], fused_attention(q.cuda(), ck, cv, kc, vc, causal=True)[1, :, 23:]) > 1e-3
    # decode-sized: the last query row against all keys
    a1 = fused_attention(q[:, :, -1:].cuda(), ck, cv, kc, vc, causal=True, attention_mask=keep[:, :, -1:].cuda())
    b1 = fused_attention(q[:, :, -1:].cuda(), ck, cv, kc, vc, causal=True, attention_mask=additive[:, :, -1:].cuda())
    assert torch.equal(a1, b1)
    with pytest.raises(TypeError):
        fused_attention(q.cuda(), ck, cv, kc, vc, causal=True, attention_mask=keep.long().cuda())


def test_expired_device_wait_is_reported_as_a_status():
    """The expiry path of the bounded waits, exercised safely: a one-CTA self-test kernel waits (with the wait the
    production kernels use and a short limit) for a barrier nobody arrives on, gives up, returns normally and
    raises the host-visible flag; the host turns that into TQ_ERR_DEVICE_WAIT and an error text.  The self-test
    has a flag of its own: the production fault counter stays 0 and later calls run."""
    import ctypes
    import time
    from turboquant_b200 import _lib, device_fault_count, fused_attention
    kc, vc = device_compressors(128, 3, mode="bf16")
    q, k, v = (t.cuda() for t in _case(1, 2, 1, 64, 64, 128, seed=1, dtype=torch.bfloat16))
    fused_attention(q, kc.compress(k), vc.compress(v), kc, vc)   # the first call on the device installs the status page
    torch.cuda.synchronize()
    waited = ctypes.c_int64(0)
    t0 = time.perf_counter()
    st = _lib.lib.tq_selftest_wait_expiry(torch.cuda.current_stream().cuda_stream, 200_000, ctypes.byref(waited))
    elapsed = time.perf_counter() - t0
    assert st == 5, (st, _lib.last_error())                       # TQ_ERR_DEVICE_WAIT
    assert "gave up" in _lib.last_error() and "self-test" in _lib.last_error()
    assert 200_000 <= waited.value < 50_000_000, waited.value     # it did wait for the limit, and not much longer
    assert elapsed < 1.0, elapsed
    with pytest.raises(_lib.TurboQuantError) as exc:
        _lib.check(st)
    assert exc.value.status == 5
    assert device_fault_count() == 0                              # the production counter is untouched
    out = fused_attention(q, kc.compress(k), vc.compress(v), kc, vc)   # and later calls are served
    assert torch.isfinite(out.float()).all()


def test_tensors_on_a_device_that_is_not_current():
    """A model on cuda:1 while the thread's current device is cuda:0 (device_map splits, a second replica in one
    process): every entry point runs on the device that owns its tensors and leaves the current device alone."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from turboquant_b200 import TurboQuantCompressorMSE, TurboQuantCompressorV2, device_fault_count, fused_attention
    d, bits = 128, 3
    q, k, v = _case(1, 4, 2, 200, 200, d, seed=9, dtype=torch.bfloat16)
    outs = []
    for dev in ("cuda:0", "cuda:1"):
        torch.cuda.set_device(0)
        kc = TurboQuantCompressorV2(d, bits, 42, device=dev)
        vc = TurboQuantCompressorMSE(d, bits, 10042, device=dev)
        qd, kd, vd = (t.to(dev) for t in (q, k, v))
        out = fused_attention(qd, kc.compress(kd), vc.compress(vd), kc, vc, causal=True)
        dec = fused_attention(qd[:, :, -1:], kc.compress(kd), vc.compress(vd), kc, vc, causal=True)
        assert out.device == torch.device(dev) and torch.cuda.current_device() == 0
        # the rotary kernel too
        from turboquant_b200 import rope
        ang = torch.arange(200, dtype=torch.float32)[None, :, None] * torch.linspace(0.01, 1.0, d)[None, None, :]
        rq, rk = rope(qd, kd, ang.cos().to(torch.bfloat16).to(dev), ang.sin().to(torch.bfloat16).to(dev))
        assert rq.device == torch.device(dev) and torch.cuda.current_device() == 0
        outs.append((out.cpu(), dec.cpu(), rq.cpu(), rk.cpu()))
        assert device_fault_count(dev) == 0
    assert all(torch.equal(a, b) for a, b in zip(outs[0], outs[1]))


def test_single_sm_kernel_selected_by_environment():
    """TQ_B200_ATTN=ws (read once per process, hence the child process) routes tensor-core mode to the single-SM
    kernel with its separate query-preparation and back-rotation launches; it must agree with the fp32 kernel
    like the default SM-pair kernel does."""
    import os
    import subprocess
    import sys
    code = """
import sys, torch
sys.path[:0] = [%r, %r]
from turboquant_b200 import fused_attention, TurboQuantCompressorV2, TurboQuantCompressorMSE
for d in (64, 128):
    g = torch.Generator(device="cuda").manual_seed(d)
    q = torch.randn(2, 4, 300, d, generator=g, device="cuda").to(torch.bfloat16)
    k = torch.randn(2, 2, 300, d, generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn(2, 2, 300, d, generator=g, device="cuda").to(torch.bfloat16)
    kc, vc = TurboQuantCompressorV2(d, 3, 42, device="cuda"), TurboQuantCompressorMSE(d, 3, 10042, device="cuda")
    ck, cv = kc.compress(k), vc.compress(v)
    a = fused_attention(q, ck, cv, kc, vc, causal=True, mode="bf16").float()
    b = fused_attention(q, ck, cv, kc, vc, causal=True, mode="fp32").float()
    err = float((a - b).norm() / b.norm())
    assert err < 1e-2, (d, err)
print("agree")
""" % (str(ROOT), str(ROOT / "transformers-turboquant_b200"))
    env = dict(os.environ, TQ_B200_ATTN="ws")
    res = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "agree" in res.stdout, res.stdout + res.stderr
