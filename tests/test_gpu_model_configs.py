"""The named model configurations through `apply_turboquant` on the GPU, against the oracle model on the CPU.

* GPT-2-small shape (12 layers, 768 wide, 12 heads of 64, 1024 positions, fp32, 3 bits, seed 42): whole-model
  logits against the oracle model, both against uncompressed attention, and the per-layer causal score cosine
  -- the figures the reference's own adapter produces on this configuration (logits rel-err 0.164, top-1
  agreement 0.642, layer cosines 0.909 .. 0.928).
* LLaMA-3-8B layer shape (hidden 4096, 32 query / 8 KV heads of 128, SwiGLU 14336) in bf16, two layers: every
  layer's attention core against the oracle core on the same inputs, and the final logits against the oracle
  model evaluated in fp32.
* A padded batch (attention_mask) through the sdpa path, prefill and cached generation.
"""

import copy

import pytest
import torch

from helpers import rel_err
from oracle import tq_oracle as orc
from oracle.model_oracle import OracleCore, causal_score_cosine, logits_agreement, oracle_model

pytestmark = pytest.mark.gpu

# layer cosines of the reference adapter on the GPT-2-small configuration (estimator vs exact q.k^T, causal
# entries, mean over heads), layers 0..11
REFERENCE_LAYER_COSINES = (0.919, 0.918, 0.922, 0.926, 0.912, 0.910, 0.925, 0.917, 0.925, 0.928, 0.909, 0.909)


def test_gpt2_small_full_forward_matches_oracle_and_reference_figures():
    from transformers import GPT2Config, GPT2LMHeadModel
    from turboquant_b200 import apply_turboquant
    torch.manual_seed(0)
    cfg = GPT2Config(attn_pdrop=0.0, resid_pdrop=0.0, embd_pdrop=0.0)   # 12 layers, 768, 12 heads, d = 64
    model = GPT2LMHeadModel(cfg).eval()
    ids = torch.randint(0, cfg.vocab_size, (1, 1024), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        plain = model(ids).logits
        ref = oracle_model(model, "GPT2Attention", "gpt2", 3, 42)
        cores = [m for m in ref.modules() if isinstance(m, OracleCore)]
        for c in cores:
            c.record = {}
        want = ref(ids).logits
        gpu = apply_turboquant(copy.deepcopy(model).cuda(), bits=3, seed=42)
        assert gpu.config.use_cache is False
        # per-layer estimator scores of the product on the oracle model's own q and k of that layer
        adapters = [m for m in gpu.modules() if hasattr(m, "key_compressor")]
        assert len(adapters) == len(cores) == 12
        got = gpu(ids.cuda()).logits.cpu()
    # whole model, fp32 mode: the literal reference stores k_mse in fp16 (~2e-4 per layer)
    assert rel_err(got, want) < 5e-3, rel_err(got, want)
    vs_plain, ref_vs_plain = logits_agreement(got, plain), logits_agreement(want, plain)
    # the reference's figures for this configuration, from its own adapter on the CPU
    assert abs(ref_vs_plain["rel_err"] - 0.164) < 2e-3 and abs(ref_vs_plain["top1"] - 0.642) < 2e-3
    assert abs(vs_plain["rel_err"] - ref_vs_plain["rel_err"]) < 3e-3, (vs_plain, ref_vs_plain)
    assert abs(vs_plain["cosine"] - ref_vs_plain["cosine"]) < 1e-3
    assert abs(vs_plain["top1"] - ref_vs_plain["top1"]) < 1.5e-2
    for layer, (core, adapter) in enumerate(zip(cores, adapters)):
        q, k = core.record["q"], core.record["k"]
        exact = q @ k.transpose(-1, -2)
        oracle_cos = float(causal_score_cosine(core.record["scores"], exact).mean())
        kc = adapter.key_compressor
        est = kc.asymmetric_attention_scores(q.cuda(), kc.compress(k.cuda())).cpu()
        cos = float(causal_score_cosine(est, exact).mean())
        assert abs(oracle_cos - REFERENCE_LAYER_COSINES[layer]) < 1e-3, (layer, oracle_cos)
        assert abs(cos - oracle_cos) < 1e-3, (layer, cos, oracle_cos)


def _llama8b_layers(n_layers=2, vocab=2048):
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(num_hidden_layers=n_layers, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                      head_dim=128, intermediate_size=14336, vocab_size=vocab, rope_theta=500000.0,
                      max_position_embeddings=1024, initializer_range=0.02)
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg).eval()
    # both sides start from weights that bf16 represents exactly
    with torch.no_grad():
        for p in model.parameters():
            p.copy_(p.to(torch.bfloat16).float())
    return model


def test_llama8b_shaped_bf16_layers_match_oracle():
    """d = 128, bf16, GQA 4:1 (head pairs on the SM-pair kernel), hidden 4096: the production shape class."""
    from turboquant_b200 import apply_turboquant
    from turboquant_b200.families import _rope_gqa
    T = 512
    model = _llama8b_layers()
    ids = torch.randint(0, 2048, (1, T), generator=torch.Generator().manual_seed(0))
    gpu = apply_turboquant(copy.deepcopy(model).cuda().to(torch.bfloat16), bits=3, seed=42)
    adapters = [m for m in gpu.modules() if hasattr(m, "key_compressor")]
    assert len(adapters) == 2 and adapters[0].head_dim == 128 and adapters[0].num_key_value_groups == 4
    # record what each layer's attention core is fed and what it returns
    seen = []
    real = _rope_gqa.fused_attention

    def recording(q, ck, cv, kc, vc, **kw):
        out = real(q, ck, cv, kc, vc, **kw)
        seen.append({"q": q.detach().float().cpu(), "out": out.detach().float().cpu(), "ck": ck, "cv": cv})
        return out

    raw_kv = []
    real_compress = _rope_gqa.compress_kv

    def recording_compress(k, v, kc, vc):
        raw_kv.extend((k.detach().float().cpu(), v.detach().float().cpu()))
        return real_compress(k, v, kc, vc)

    _rope_gqa.fused_attention, _rope_gqa.compress_kv = recording, recording_compress
    try:
        with torch.no_grad():
            got = gpu(ids.cuda()).logits.float().cpu()
    finally:
        _rope_gqa.fused_attention, _rope_gqa.compress_kv = real, real_compress
    assert len(seen) == 2 and len(raw_kv) == 4
    # (1) every layer's attention core against the oracle core on the same bf16 q, k, v
    for layer, rec in enumerate(seen):
        ks, vs = orc.layer_seeds(42, layer)
        kp, vp = orc.make_key_params(128, 3, ks), orc.make_value_params(128, 3, vs)
        k, v = raw_kv[2 * layer], raw_kv[2 * layer + 1]
        want, _ = orc.attention_core(rec["q"], k, v, kp, vp, mask=orc.causal_mask(T, T), literal=False)
        err = rel_err(rec["out"], want)
        assert err < 1e-2, (layer, err)
    # (2) the whole model.  TurboQuant's quantisers are discontinuous, so a perturbation of relative size e in a
    # layer's keys moves a fraction ~e of the index and sign decisions and with them the scores by ~sqrt(e): the
    # bf16 rounding of activations (1e-3..1e-2) is amplified layer by layer, whatever computes the attention.
    # The reference arithmetic itself shows it: the oracle model with bf16 activations against the oracle model
    # in fp32.  The product must agree with the fp32 oracle as well as the bf16 oracle does.
    with torch.no_grad():
        ref = oracle_model(model, "LlamaAttention", "rope", 3, 42)
        want_logits = ref(ids).logits
        ref16 = oracle_model(copy.deepcopy(model).to(torch.bfloat16), "LlamaAttention", "rope", 3, 42)
        want16 = ref16(ids).logits.float()
        plain = model(ids).logits
    agree, agree16 = logits_agreement(got, want_logits), logits_agreement(got, want16)
    oracle_pair = logits_agreement(want16, want_logits)
    ref_vs_plain, got_vs_plain = logits_agreement(want_logits, plain), logits_agreement(got, plain)
    print("llama8b-shaped, 2 layers | product vs fp32 oracle", agree, "| product vs bf16 oracle", agree16,
          "| bf16 oracle vs fp32 oracle", oracle_pair, "| fp32 oracle vs uncompressed", ref_vs_plain,
          "| product vs uncompressed", got_vs_plain)
    assert agree["cosine"] > oracle_pair["cosine"] - 0.05, (agree, oracle_pair)
    # measured: product vs bf16 oracle cosine 0.997 (rel-err 0.076, top-1 0.85); bf16 oracle vs fp32 oracle 0.755;
    # product vs fp32 oracle 0.755; fp32 oracle vs uncompressed 0.593, product vs uncompressed 0.587
    assert agree16["cosine"] > 0.99 and agree16["rel_err"] < 0.15, agree16
    # and the distance to uncompressed attention is the estimator's, not this implementation's
    assert abs(got_vs_plain["cosine"] - ref_vs_plain["cosine"]) < 0.05, (got_vs_plain, ref_vs_plain)


@pytest.mark.parametrize("kind", ["llama", "gpt2"])
def test_padded_batch_through_sdpa_matches_oracle(kind):
    """A left-padded batch: HF's sdpa path hands the adapter a BOOLEAN mask (True = visible), its eager path an
    additive one.  The real (unpadded) positions must match the oracle model, which is built with eager
    attention, and must not depend on what the padding tokens are."""
    from transformers import GPT2Config, GPT2LMHeadModel, LlamaConfig, LlamaForCausalLM
    from turboquant_b200 import apply_turboquant
    torch.manual_seed(0)
    if kind == "gpt2":
        cfg = GPT2Config(n_embd=256, n_head=4, n_layer=2, n_positions=128, vocab_size=512,
                         attn_pdrop=0.0, resid_pdrop=0.0, embd_pdrop=0.0)
        model, cls_name, okind = GPT2LMHeadModel(cfg).eval(), "GPT2Attention", "gpt2"
    else:
        cfg = LlamaConfig(hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                          intermediate_size=512, num_hidden_layers=2, vocab_size=512)
        model, cls_name, okind = LlamaForCausalLM(cfg).eval(), "LlamaAttention", "rope"
    B, T, pad = 2, 96, 29
    ids = torch.randint(0, 512, (B, T), generator=torch.Generator().manual_seed(1))
    am = torch.ones(B, T, dtype=torch.long)
    am[1, :pad] = 0                                   # sequence 1 starts with 29 padding tokens
    ids2 = ids.clone()
    ids2[1, :pad] = (ids2[1, :pad] + 7) % 512         # other padding tokens, same real tokens
    with torch.no_grad():
        eager = copy.deepcopy(model)
        eager.config._attn_implementation = "eager"
        want = oracle_model(eager, cls_name, okind, 3, 42)(ids, attention_mask=am).logits
        gpu = apply_turboquant(copy.deepcopy(model).cuda(), bits=3, seed=42)
        assert gpu.config._attn_implementation == "sdpa"
        got = gpu(ids.cuda(), attention_mask=am.cuda()).logits.cpu()
        got2 = gpu(ids2.cuda(), attention_mask=am.cuda()).logits.cpu()
        unmasked = gpu(ids.cuda()).logits.cpu()
    real = am.bool()
    assert rel_err(got[real], want[real]) < 3e-3, rel_err(got[real], want[real])
    assert rel_err(got2[real], got[real]) < 1e-5      # padding tokens are invisible to real positions
    assert rel_err(unmasked[1, pad:], got[1, pad:]) > 1e-2   # and the mask does something


def test_padded_batch_generation_with_compressed_cache():
    """The same left-padded batch through `kv_cache_capacity` generation: prefill with the mask, then token by
    token with the growing mask; the last-position logits follow the cache-less flow on the full prefix."""
    from transformers import LlamaConfig, LlamaForCausalLM
    from turboquant_b200 import apply_turboquant
    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=512, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                      intermediate_size=512, num_hidden_layers=2, vocab_size=512, max_position_embeddings=512)
    base = LlamaForCausalLM(cfg).eval().cuda().to(torch.bfloat16)
    plain = apply_turboquant(copy.deepcopy(base), bits=3, seed=42)
    cached = apply_turboquant(copy.deepcopy(base), bits=3, seed=42, kv_cache_capacity=400)
    B, T0, steps, pad = 2, 290, 4, 41
    ids = torch.randint(0, 512, (B, T0 + steps), generator=torch.Generator().manual_seed(4)).cuda()
    am = torch.ones(B, T0 + steps, dtype=torch.long, device="cuda")
    am[0, :pad] = 0
    with torch.no_grad():
        out = cached(input_ids=ids[:, :T0], attention_mask=am[:, :T0], use_cache=True)
        pkv = out.past_key_values
        want = plain(input_ids=ids[:, :T0], attention_mask=am[:, :T0]).logits[:, -1].float()
        assert rel_err(out.logits[:, -1].float(), want) < 1e-6
        for t in range(T0, T0 + steps):
            out = cached(input_ids=ids[:, t:t + 1], attention_mask=am[:, :t + 1], past_key_values=pkv, use_cache=True)
            want = plain(input_ids=ids[:, :t + 1], attention_mask=am[:, :t + 1]).logits[:, -1].float()
            assert rel_err(out.logits[:, -1].float(), want) < 3e-2, (t, rel_err(out.logits[:, -1].float(), want))
        # the mask matters: without it sequence 0 attends to its padding
        nomask = plain(input_ids=ids[:, :T0]).logits[0, -1].float()
        assert rel_err(nomask, plain(input_ids=ids[:, :T0], attention_mask=am[:, :T0]).logits[0, -1].float()) > 1e-2


def test_compressed_cache_refuses_a_prefilled_or_interleaved_hf_cache():
    """The compressed caches follow one generation at a time: a cache object the layers have not seen must be
    empty, otherwise the tokens it already counts were never compressed and the step would silently attend over
    the new token alone."""
    from transformers import LlamaConfig, LlamaForCausalLM
    from turboquant_b200 import apply_turboquant
    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=512, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                      intermediate_size=512, num_hidden_layers=2, vocab_size=512, max_position_embeddings=512)
    model = apply_turboquant(LlamaForCausalLM(cfg).eval().cuda().to(torch.bfloat16), bits=3, seed=42,
                             kv_cache_capacity=128)
    ids = torch.randint(0, 512, (1, 40), generator=torch.Generator().manual_seed(5)).cuda()
    with torch.no_grad():
        first = model(input_ids=ids[:, :20], use_cache=True).past_key_values
        second = model(input_ids=ids[:, :30], use_cache=True).past_key_values   # a new generation: fine
        model(input_ids=ids[:, 30:31], past_key_values=second, use_cache=True)  # continues the second
        with pytest.raises(RuntimeError, match="already holds"):
            model(input_ids=ids[:, 20:21], past_key_values=first, use_cache=True)  # back to the first: refused
