"""The rotary-embedding kernel against HF's apply_rotary_pos_emb (what the reference's adapters call,
families/llama.py:98): bit-identical in every dtype, on the transposed views the adapters hand over."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(B, Hq, Hkv, S, d, dtype, seed, broadcast_batch):
    g = torch.Generator(device="cuda").manual_seed(seed)
    # projection outputs are [B, S, H, d]; the adapters see the [B, H, S, d] view
    q = torch.randn(B, S, Hq, d, generator=g, device="cuda").to(dtype).transpose(1, 2)
    k = torch.randn(B, S, Hkv, d, generator=g, device="cuda").to(dtype).transpose(1, 2)
    pos = torch.arange(S, device="cuda", dtype=torch.float32)[None, :, None] + \
        (0 if broadcast_batch else torch.arange(B, device="cuda", dtype=torch.float32)[:, None, None] * 7)
    inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2, device="cuda", dtype=torch.float32) / d))
    ang = torch.cat([pos * inv, pos * inv], dim=-1)                     # [B or 1, S, d]
    return q, k, ang.cos().to(dtype), ang.sin().to(dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("B,Hq,Hkv,S,d,broadcast", [(2, 8, 2, 300, 128, False), (3, 4, 4, 77, 64, True),
                                                     (1, 32, 8, 1, 128, True), (2, 2, 1, 1025, 96, False)])
def test_rope_equals_hf_bit_for_bit(dtype, B, Hq, Hkv, S, d, broadcast):
    from transformers.models.llama.modeling_llama import apply_rotary_pos_emb
    from turboquant_b200 import rope
    q, k, cos, sin = _inputs(B, Hq, Hkv, S, d, dtype, seed=S + d, broadcast_batch=broadcast)
    want_q, want_k = apply_rotary_pos_emb(q, k, cos, sin)
    got_q, got_k = rope(q, k, cos, sin)
    assert got_q.is_contiguous() and got_k.is_contiguous() and got_q.dtype == dtype
    assert torch.equal(got_q, want_q) and torch.equal(got_k, want_k)


def test_rope_rejects_what_it_does_not_cover():
    from turboquant_b200 import rope
    from turboquant_b200.rotary import rope_applies
    q, k, cos, sin = _inputs(1, 2, 2, 16, 128, torch.bfloat16, seed=1, broadcast_batch=True)
    assert rope_applies(q, k, cos, sin)
    assert not rope_applies(q, k, cos[..., :64], sin[..., :64])          # partial rotary width
    assert not rope_applies(q, k, cos.float(), sin.float())              # mixed dtypes
    with pytest.raises(ValueError):
        rope(q, k, cos[..., :64], sin[..., :64])


def test_llama_adapter_uses_the_kernel_and_keeps_its_output():
    """The LLaMA-style adapters rotate with the kernel; a layer's output is what it is with HF's function."""
    import copy
    from transformers import LlamaConfig, LlamaForCausalLM
    from turboquant_b200 import apply_turboquant
    from turboquant_b200.families import _rope_gqa
    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=512, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                      intermediate_size=512, num_hidden_layers=2, vocab_size=512, max_position_embeddings=512)
    model = apply_turboquant(LlamaForCausalLM(cfg).eval().cuda().to(torch.bfloat16), bits=3, seed=42)
    ids = torch.randint(0, 512, (2, 200), generator=torch.Generator().manual_seed(4)).cuda()
    with torch.no_grad():
        fused = model(input_ids=ids).logits
        from transformers.models.llama.modeling_llama import apply_rotary_pos_emb
        saved = _rope_gqa.RopeGQAAttention.__dict__["_rotary"]   # the staticmethod object itself
        try:
            _rope_gqa.RopeGQAAttention._rotary = staticmethod(lambda q, k, cos, sin: apply_rotary_pos_emb(q, k, cos, sin))
            stock = model(input_ids=ids).logits
        finally:
            _rope_gqa.RopeGQAAttention._rotary = saved
    assert torch.equal(fused, stock)
