"""End-to-end plugin path on small models: `apply_turboquant` on the GPU against the same model on
the CPU whose attention cores are evaluated by the oracle (the reference arithmetic), layer by
layer with the reference's seeds (layer i: keys seed+i, values seed+i+10000)."""

import copy

import pytest
import torch

from helpers import rel_err
from oracle.model_oracle import oracle_model

pytestmark = pytest.mark.gpu


def _oracle_model(model, cls_name, kind, bits, seed):
    return oracle_model(model, cls_name, kind, bits, seed)


def _build(kind):
    from transformers import GPT2Config, GPT2LMHeadModel, LlamaConfig, LlamaForCausalLM, Qwen2Config, Qwen2ForCausalLM
    torch.manual_seed(0)
    if kind == "gpt2":
        cfg = GPT2Config(n_embd=256, n_head=4, n_layer=2, n_positions=128, vocab_size=512,
                         attn_pdrop=0.0, resid_pdrop=0.0, embd_pdrop=0.0)
        return GPT2LMHeadModel(cfg).eval(), "GPT2Attention"
    if kind == "llama":
        cfg = LlamaConfig(hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                          intermediate_size=512, num_hidden_layers=2, vocab_size=512)
        return LlamaForCausalLM(cfg).eval(), "LlamaAttention"
    cfg = Qwen2Config(hidden_size=256, num_attention_heads=4, num_key_value_heads=1, intermediate_size=512,
                      num_hidden_layers=2, vocab_size=512)
    return Qwen2ForCausalLM(cfg).eval(), "Qwen2Attention"


@pytest.mark.parametrize("kind", ["gpt2", "llama", "qwen2"])
@pytest.mark.parametrize("bits", [3, 4])
def test_model_logits_match_oracle_fp32(kind, bits):
    from turboquant_b200 import apply_turboquant
    model, cls_name = _build(kind)
    ids = torch.randint(0, 512, (2, 96), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = _oracle_model(model, cls_name, "gpt2" if kind == "gpt2" else "rope", bits, 42)(ids).logits
        got = apply_turboquant(copy.deepcopy(model).cuda(), bits=bits, seed=42)(ids.cuda()).logits
        plain = model(ids).logits
    # fp32 mode; the literal reference stores k_mse in fp16 (~2e-4 per layer)
    assert rel_err(got, want) < 3e-3, rel_err(got, want)
    # and compression is doing something: the compressed model differs from the uncompressed one
    assert rel_err(got, plain) > 10 * rel_err(got, want)


def test_llama_bf16_is_causal_and_close_to_fp32_mode():
    from turboquant_b200 import apply_turboquant
    model, _ = _build("llama")
    ids = torch.randint(0, 512, (1, 200), generator=torch.Generator().manual_seed(2))
    ids2 = ids.clone()
    ids2[0, -1] = (ids2[0, -1] + 1) % 512
    with torch.no_grad():
        m32 = apply_turboquant(copy.deepcopy(model).cuda(), bits=3, seed=42)
        m16 = apply_turboquant(copy.deepcopy(model).cuda().to(torch.bfloat16), bits=3, seed=42)
        a, b2 = m16(ids.cuda()).logits.float(), m16(ids2.cuda()).logits.float()
        ref = m32(ids.cuda()).logits
    assert torch.isfinite(a).all()
    assert torch.equal(a[:, :-1], b2[:, :-1])         # HF passes no mask under sdpa: causality is ours
    assert not torch.equal(a[:, -1], b2[:, -1])
    assert rel_err(a, ref) < 1e-1                     # whole model (weights included) in bf16 vs fp32


@pytest.mark.parametrize("kind", ["gpt2", "llama"])
def test_single_training_step_completes(kind):
    """The reference's fine-tuning check (tests/test_sft.py:19-43: one optimiser step on a patched
    model finishes) without the trainer or a download.  Compression, scoring and the value
    reconstruction are no-grad in the reference (compressors.py:98,163,270,296), so attention
    output is a constant: the output projection learns, the q/k/v projections receive nothing."""
    from turboquant_b200 import apply_turboquant
    model, _ = _build(kind)
    model = apply_turboquant(copy.deepcopy(model).cuda().to(torch.bfloat16), bits=3, seed=42).train()
    ids = torch.randint(0, 512, (2, 32), generator=torch.Generator().manual_seed(3)).cuda()
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    out_w, in_w = (("c_proj", "c_attn") if kind == "gpt2" else ("o_proj", "q_proj"))
    attn = next(m for m in model.modules() if hasattr(m, "key_compressor"))
    before = getattr(attn, out_w).weight.detach().clone()
    loss = model(input_ids=ids, labels=ids).loss
    assert torch.isfinite(loss)
    loss.backward()
    g = getattr(attn, out_w).weight.grad
    assert g is not None and torch.isfinite(g).all() and g.abs().sum() > 0
    assert getattr(attn, in_w).weight.grad is None
    opt.step()
    assert not torch.equal(before, getattr(attn, out_w).weight.detach())
    assert model.config.use_cache is False


def test_generation_with_the_compressed_cache_matches_recomputation():
    """`apply_turboquant(..., kv_cache_capacity=n)` (an extension: the reference's adapters always run with
    use_cache = False, patch.py:80-81) keeps a CompressedKVCache per layer.  Token-by-token decoding through the
    HF cache protocol must give the logits of the reference flow, which recompresses and re-attends the whole
    prefix for every new token."""
    from transformers import LlamaConfig, LlamaForCausalLM
    from turboquant_b200 import apply_turboquant
    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=512, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                      intermediate_size=512, num_hidden_layers=2, vocab_size=512, max_position_embeddings=512)
    base = LlamaForCausalLM(cfg).eval().cuda().to(torch.bfloat16)
    plain = apply_turboquant(copy.deepcopy(base), bits=3, seed=42)
    cached = apply_turboquant(copy.deepcopy(base), bits=3, seed=42, kv_cache_capacity=400)
    assert plain.config.use_cache is False and cached.config.use_cache is True
    ids = torch.randint(0, 512, (2, 300), generator=torch.Generator().manual_seed(4)).cuda()
    steps = 5
    with torch.no_grad():
        out = cached(input_ids=ids[:, :300 - steps], use_cache=True)
        pkv = out.past_key_values
        assert rel_err(out.logits[:, -1].float(), plain(input_ids=ids[:, :300 - steps]).logits[:, -1].float()) < 1e-6
        for t in range(300 - steps, 300):
            out = cached(input_ids=ids[:, t:t + 1], past_key_values=pkv, use_cache=True)
            want = plain(input_ids=ids[:, :t + 1]).logits[:, -1].float()
            got = out.logits[:, -1].float()
            # one query row per head through the split-KV kernel instead of the last row of a prefill tile
            assert rel_err(got, want) < 3e-2, (t, rel_err(got, want))
        # a second generation starts over: a new HF cache object resets the compressed caches
        again = cached(input_ids=ids[:, :64], use_cache=True).logits[:, -1].float()
        assert rel_err(again, plain(input_ids=ids[:, :64]).logits[:, -1].float()) < 1e-6
        # and generate() runs end to end on it
        gen = cached.generate(ids[:1, :32], max_new_tokens=4, do_sample=False)
        assert gen.shape == (1, 36)


def test_gpt2_generation_with_the_compressed_cache_matches_recomputation():
    """The same extension on the GPT-2 adapter (head_dim 64, learned positions, fused c_attn): token-by-token
    decoding against the compressed cache must give the logits of the cache-less flow, and generate() the same
    greedy tokens."""
    from transformers import GPT2Config, GPT2LMHeadModel
    from turboquant_b200 import apply_turboquant
    torch.manual_seed(0)
    cfg = GPT2Config(n_embd=256, n_head=4, n_layer=2, vocab_size=512, n_positions=512, attn_pdrop=0.0,
                     resid_pdrop=0.0, embd_pdrop=0.0)
    base = GPT2LMHeadModel(cfg).eval().cuda().to(torch.bfloat16)
    plain = apply_turboquant(copy.deepcopy(base), bits=3, seed=42)
    cached = apply_turboquant(copy.deepcopy(base), bits=3, seed=42, kv_cache_capacity=400)
    assert plain.config.use_cache is False and cached.config.use_cache is True
    ids = torch.randint(0, 512, (2, 200), generator=torch.Generator().manual_seed(4)).cuda()
    steps = 4
    with torch.no_grad():
        out = cached(input_ids=ids[:, :200 - steps], use_cache=True)
        pkv = out.past_key_values
        assert rel_err(out.logits[:, -1].float(), plain(input_ids=ids[:, :200 - steps]).logits[:, -1].float()) < 1e-6
        for t in range(200 - steps, 200):
            out = cached(input_ids=ids[:, t:t + 1], past_key_values=pkv, use_cache=True)
            want = plain(input_ids=ids[:, :t + 1]).logits[:, -1].float()
            assert rel_err(out.logits[:, -1].float(), want) < 3e-2, (t, rel_err(out.logits[:, -1].float(), want))
        gen = cached.generate(ids[:1, :32], max_new_tokens=4, do_sample=False, pad_token_id=0)
        want = plain.generate(ids[:1, :32], max_new_tokens=4, do_sample=False, pad_token_id=0)
        assert gen.shape == (1, 36) and torch.equal(gen[:, :33], want[:, :33])  # the first new token comes from the same prefill


def test_generate_without_cache_recomputes_the_whole_sequence():
    """The reference switches `config.use_cache` off (patch.py:80-81); current transformers read the flag from
    `generation_config`, which has to follow, or generate() would hand the adapters single tokens."""
    from turboquant_b200 import apply_turboquant
    model, _ = _build("llama")
    model = apply_turboquant(copy.deepcopy(model).cuda().to(torch.bfloat16), bits=3, seed=42)
    assert model.config.use_cache is False and model.generation_config.use_cache is False
    ids = torch.randint(0, 512, (1, 40), generator=torch.Generator().manual_seed(5)).cuda()
    with torch.no_grad():
        gen = model.generate(ids, max_new_tokens=3, do_sample=False)
        want = ids
        for _ in range(3):
            want = torch.cat([want, model(input_ids=want).logits[:, -1:].argmax(-1)], dim=1)
    assert torch.equal(gen, want)
