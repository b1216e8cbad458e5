"""The estimator-quality harness (`turboquant_b200.validate`, the reference's validate script on the CUDA
kernels): compression ratios by bit accounting, and per-layer score cosine / top-k agreement equal to the
oracle's on the same cached keys."""

import pytest
import torch

from oracle import tq_oracle as orc


def test_compression_ratios_by_bit_accounting():
    """32 d / (2 b d + 48) at d = 128: 7.31x, 5.02x, 3.82x for 2, 3, 4 bits (validate.py:137-152 of the reference)."""
    from turboquant_b200.validate import compression_ratio
    assert [round(compression_ratio(b, 128), 2) for b in (2, 3, 4)] == [7.31, 5.02, 3.82]


def test_cli_has_the_validate_command():
    """`validate` is a sub-command of the console entry, as in the reference (cli.py:10-15)."""
    from typer.testing import CliRunner
    from transformers_turboquant.cli import app
    res = CliRunner().invoke(app, ["--help"])
    assert res.exit_code == 0 and "validate" in res.output


@pytest.mark.gpu
def test_layer_metrics_equal_the_oracle():
    """One layer's cached keys through the harness on the GPU and through the oracle on the CPU (same seeds
    layer*1000, last key as proxy query): same cosine to 1e-4, same top-1 / top-5 decisions."""
    from turboquant_b200.validate import layer_metrics
    H, S, D, layer = 2, 384, 128, 3
    g = torch.Generator().manual_seed(5)
    keys = torch.randn(1, H, S, D, generator=g).to(torch.bfloat16)
    keys[..., :4] *= 6.0
    values = torch.randn(1, H, S, D, generator=g).to(torch.bfloat16)
    for bits in (2, 3, 4):
        got = layer_metrics(keys.cuda(), values.cuda(), bits, layer)
        kp = orc.make_key_params(D, bits, layer * 1000)
        ck = orc.key_compress(keys, kp)
        q = keys[:, :, -1:, :]
        est = orc.scores_from_packed(q.float(), ck["packed_key_indices"], ck["packed_qjl_signs"], ck["vec_norms"],
                                     ck["residual_norm"], kp, ck["shape"])[0, :, 0]
        real = (q.float() @ keys.float().transpose(-1, -2))[0, :, 0]
        cos = torch.nn.functional.cosine_similarity(real, est, dim=-1)
        assert torch.allclose(torch.tensor(got["cosine"]), cos, atol=2e-4), (bits, got["cosine"], cos)
        assert got["top1"] == (est.argmax(-1) == real.argmax(-1)).tolist()
        assert got["top5"] == (est.topk(5, dim=-1).indices == real.argmax(-1)[:, None]).any(-1).tolist()


@pytest.mark.gpu
def test_validation_run_on_a_shallow_model():
    """The whole harness on two layers of the Qwen2.5-3B shape at a short context: ratios as above, sane
    quality figures that improve with the bit width."""
    from turboquant_b200.validate import run_validation
    rec = run_validation(bits_list=(2, 3, 4), contexts=(512,), layers=2)
    r = rec["results"]
    assert [r[f"T512_b{b}"]["compression_ratio"] for b in (2, 3, 4)] == [7.31, 5.02, 3.82]
    assert r["T512_b2"]["heads_checked"] == 2 * 2
    assert 0.5 < r["T512_b2"]["score_cosine"] < r["T512_b3"]["score_cosine"] < r["T512_b4"]["score_cosine"] <= 1.0
    assert all(0.0 <= r[k][m] <= 1.0 for k in r for m in ("top1", "top5"))
