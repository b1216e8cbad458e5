"""Host-side plugin API on the CPU: registry, error text, module replacement, seeds."""

import numpy as np
import pytest
import torch

from oracle import tq_oracle as orc


def test_registry_dispatch_and_error_text():
    from turboquant_b200 import (TurboQuantAttentionBase, UnsupportedModelError, get_attention_class,
                                 register_family)
    from turboquant_b200.plugin import _REGISTRY

    for fam in ("gpt2", "qwen2", "llama", "mistral", "deepseek", "deepseek_v2", "deepseek_v3"):
        assert issubclass(get_attention_class(fam), TurboQuantAttentionBase)
    assert get_attention_class("llama") is get_attention_class("mistral")

    @register_family("unit_a", "unit_b")
    class Dummy(TurboQuantAttentionBase):
        ATTENTION_CLASS_NAMES = ("DummyAttention",)

        @classmethod
        def from_original(cls, original, key_compressor, val_compressor):
            return cls()

        def forward(self, hidden_states, **kwargs):
            return hidden_states

    try:
        assert get_attention_class("unit_a") is Dummy and get_attention_class("unit_b") is Dummy
    finally:
        _REGISTRY.pop("unit_a"), _REGISTRY.pop("unit_b")
    with pytest.raises(UnsupportedModelError) as err:
        get_attention_class("not_a_model")
    msg = str(err.value)
    assert "not_a_model" in msg and "Supported:" in msg and "@register_family" in msg
    assert isinstance(err.value, ValueError)


def test_reference_import_names_resolve():
    from transformers_turboquant import apply_turboquant
    from transformers_turboquant.base import TurboQuantAttentionBase
    from transformers_turboquant.registry import get_attention_class
    from turboquant_pytorch.compressors import TurboQuantCompressorMSE, TurboQuantCompressorV2
    import turboquant_b200 as t

    assert apply_turboquant is t.apply_turboquant and TurboQuantAttentionBase is t.TurboQuantAttentionBase
    assert get_attention_class("gpt2") is t.families.gpt2.TurboQuantGPT2Attention
    assert TurboQuantCompressorV2 is t.TurboQuantCompressorV2 and TurboQuantCompressorMSE is t.TurboQuantCompressorMSE


def test_compressor_constants_match_oracle():
    from turboquant_b200 import TurboQuantCompressorMSE, TurboQuantCompressorV2

    kc = TurboQuantCompressorV2(128, 3, seed=45, device="cpu")
    vc = TurboQuantCompressorMSE(128, 3, seed=10045, device="cpu")
    kp, vp = orc.make_key_params(128, 3, 45), orc.make_value_params(128, 3, 10045)
    assert torch.equal(kc.Pi, kp.Pi) and torch.equal(kc.S, kp.S) and torch.equal(kc.centroids, kp.centroids)
    assert torch.equal(kc.boundaries, kp.boundaries) and torch.equal(kc.PiT, kp.Pi.T)
    assert torch.allclose(kc.S_eff, kp.S_eff, atol=1e-6)
    assert torch.equal(vc.Pi, vp.Pi) and torch.equal(vc.centroids, vp.centroids)
    assert (kc.bits, kc.mse_bits, kc.head_dim, vc.bits) == (3, 2, 128, 3)
    with pytest.raises(ValueError):
        TurboQuantCompressorV2(96, 3, 0, device="cpu")
    with pytest.raises(ValueError):
        TurboQuantCompressorMSE(128, 5, 0, device="cpu")
    with pytest.raises(RuntimeError, match="no CPU path"):
        kc.compress(torch.zeros(1, 1, 4, 128))


def _tiny(model_type):
    from transformers import GPT2Config, GPT2LMHeadModel, LlamaConfig, LlamaForCausalLM, Qwen2Config, Qwen2ForCausalLM

    torch.manual_seed(0)
    if model_type == "gpt2":
        return GPT2LMHeadModel(GPT2Config(n_embd=128, n_head=2, n_layer=2, n_positions=32, vocab_size=64)), "GPT2Attention"
    if model_type == "llama":
        return LlamaForCausalLM(LlamaConfig(hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                                            intermediate_size=128, num_hidden_layers=2, vocab_size=64)), "LlamaAttention"
    return Qwen2ForCausalLM(Qwen2Config(hidden_size=256, num_attention_heads=4, num_key_value_heads=2,
                                        intermediate_size=128, num_hidden_layers=2, vocab_size=64)), "Qwen2Attention"


@pytest.mark.parametrize("model_type", ["gpt2", "llama", "qwen2"])
def test_apply_turboquant_replaces_attention(model_type):
    from turboquant_b200 import TurboQuantAttentionBase, apply_turboquant

    model, cls_name = _tiny(model_type)
    n_before = sum(type(m).__name__ == cls_name for m in model.modules())
    assert n_before == 2
    same = apply_turboquant(model, bits=3, seed=42)
    assert same is model and model.config.use_cache is False
    assert not any(type(m).__name__ == cls_name for m in model.modules())
    adapters = [m for m in model.modules() if isinstance(m, TurboQuantAttentionBase)]
    assert len(adapters) == 2
    for i, a in enumerate(adapters):
        ks, vs = orc.layer_seeds(42, i)
        assert torch.equal(a.key_compressor.Pi, orc.rotation_matrix(64, ks))
        assert torch.equal(a.val_compressor.Pi, orc.rotation_matrix(64, vs))
        assert a.key_compressor.bits == 3 and a.val_compressor.bits == 3
    if model_type != "gpt2":
        assert adapters[0].num_heads == 4 and adapters[0].num_key_value_heads == 2
    # casting the model leaves the compressor constants in fp32
    model.to(torch.bfloat16)
    assert adapters[0].key_compressor.Pi.dtype == torch.float32
    assert adapters[0].q_proj.weight.dtype == torch.bfloat16 if model_type != "gpt2" else True


def test_unsupported_model_type_raises():
    from transformers import BertConfig, BertModel
    from turboquant_b200 import UnsupportedModelError, apply_turboquant

    with pytest.raises(UnsupportedModelError):
        apply_turboquant(BertModel(BertConfig(hidden_size=32, num_attention_heads=2, num_hidden_layers=1,
                                              intermediate_size=32, vocab_size=32)))


def test_mask_forms_accepted_by_the_attention_wrapper():
    """Boolean masks mean True = visible (HF's sdpa path), floating-point masks are additive (its eager path),
    integer masks are refused because their meaning would be a guess."""
    import pytest
    import torch
    from turboquant_b200.compressors import _mask_args
    keep = torch.ones(2, 1, 3, 5, dtype=torch.bool)
    keep[1, 0, :, :2] = False
    mk, ptr, sb, sq = _mask_args(keep, 2, 3, 5, "cpu")
    assert mk.dtype == torch.float32 and mk.shape == (2, 3, 5) and (sb, sq) == (15, 5) and ptr == mk.data_ptr()
    assert torch.equal(mk == 0, keep[:, 0]) and float(mk[1, 0, 0]) == torch.finfo(torch.float32).min
    add = torch.zeros(1, 1, 3, 5, dtype=torch.float16)
    mk, _, sb, _ = _mask_args(add, 2, 3, 5, "cpu")
    assert mk.dtype == torch.float32 and sb == 0            # broadcast over the batch
    with pytest.raises(TypeError):
        _mask_args(keep.long(), 2, 3, 5, "cpu")
    with pytest.raises(ValueError):
        _mask_args(torch.zeros(2, 4, 3, 5), 2, 3, 5, "cpu")  # per-head masks
    assert _mask_args(None, 2, 3, 5, "cpu") == (None, None, 0, 0)
