"""Estimator-quality harness on the CUDA kernels: the measurements of the reference's validation script
(src/turboquant_pytorch/validate.py:88-231) on a random-init model of the Qwen2.5-3B shape.

The reference loads the Qwen2.5-3B-Instruct checkpoint, feeds it a needle-in-a-haystack prompt, takes every
layer's cached keys and values, compresses them with seeds `layer * 1000` (keys) and `layer * 1000 + 500`
(values) and, with the LAST KEY of each head as a proxy query, compares the estimator's scores with the exact
ones: compression ratio by bit accounting, cosine similarity of the score rows, top-1 agreement and whether the
exact top-1 key is among the estimator's top five, per head and layer.  Checkpoint, tokenizer and prompt are not
available offline, so the model here is random-init (N(0, 0.02), seed 0) and the tokens uniform random; the
prompt-specific "needle rank" has no counterpart.  Everything else follows the reference line by line, with the
compression and the estimator on the GPU kernels.

    python -m turboquant_b200.validate [--contexts 2048 4096 8192] [--bits 2 3 4] [--layers 36]
"""

from __future__ import annotations

import argparse
import json

import torch

from .compressors import TurboQuantCompressorMSE, TurboQuantCompressorV2

QWEN25_3B = dict(num_hidden_layers=36, hidden_size=2048, num_attention_heads=16, num_key_value_heads=2,
                 head_dim=128, intermediate_size=11008, vocab_size=151936)


def compression_ratio(bits: int, d: int) -> float:
    """fp16 K+V bytes over packed bytes, by the reference's bit accounting (validate.py:137-152): keys store
    (bits-1)-bit indices, one sign bit per coordinate and two fp16 norms, values `bits`-bit indices and one."""
    key_bits = d * max(bits - 1, 1) + d + 16 + 16
    val_bits = d * bits + 16
    return 32.0 * d / (key_bits + val_bits)


@torch.no_grad()
def layer_metrics(keys: torch.Tensor, values: torch.Tensor, bits: int, layer: int) -> dict:
    """One layer's cached keys/values [1, H, S, D] -> per-head score cosine, top-1 and top-5 agreement with the
    last key as proxy query (validate.py:121-186).  Seeds as in the reference: layer*1000 / layer*1000+500."""
    B, H, S, D = keys.shape
    dev = str(keys.device)
    kc = TurboQuantCompressorV2(D, bits, seed=layer * 1000, device=dev)
    vc = TurboQuantCompressorMSE(D, bits, seed=layer * 1000 + 500, device=dev)
    ck = kc.compress(keys)
    vc.compress(values)  # compressed as the reference does; only its size enters the metrics
    query = keys[:, :, -1:, :]
    real = torch.matmul(query.float(), keys.float().transpose(-2, -1)).squeeze(-2)[0]   # [H, S]
    est = kc.asymmetric_attention_scores(query, ck).squeeze(-2)[0]
    cos = torch.nn.functional.cosine_similarity(real, est, dim=-1)
    real_top1 = real.argmax(-1)
    top1 = (est.argmax(-1) == real_top1)
    top5 = (est.topk(min(5, S), dim=-1).indices == real_top1[:, None]).any(-1)
    return {"cosine": cos.tolist(), "top1": top1.tolist(), "top5": top5.tolist()}


@torch.no_grad()
def run_validation(bits_list=(2, 3, 4), contexts=(2048, 4096, 8192), layers: int | None = None,
                   device: str = "cuda:0", seed: int = 0, shape: dict | None = None) -> dict:
    """Random-init model of the Qwen2.5-3B shape (bf16), batch 1, uniform random tokens: per context length and
    bit width the compression ratio, mean score cosine, top-1 and top-5 agreement over all heads and layers."""
    from transformers import Qwen2Config, Qwen2ForCausalLM
    shape = dict(shape or QWEN25_3B)
    if layers is not None:
        shape["num_hidden_layers"] = layers
    dev = torch.device(device)
    cfg = Qwen2Config(max_position_embeddings=max(contexts), initializer_range=0.02, **shape)
    torch.manual_seed(seed)
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            model = Qwen2ForCausalLM(cfg).eval()
    finally:
        torch.set_default_dtype(torch.float32)
    results = {}
    for T in contexts:
        ids = torch.randint(0, shape["vocab_size"], (1, T), generator=torch.Generator().manual_seed(seed)).to(dev)
        cache = model(input_ids=ids, use_cache=True, logits_to_keep=1).past_key_values
        n_layers = len(cache.layers)
        for bits in bits_list:
            cos, top1, top5 = [], [], []
            for layer in range(n_layers):
                m = layer_metrics(cache.layers[layer].keys, cache.layers[layer].values, bits, layer)
                cos += m["cosine"]
                top1 += m["top1"]
                top5 += m["top5"]
            results[f"T{T}_b{bits}"] = {
                "compression_ratio": round(compression_ratio(bits, shape["head_dim"]), 2),
                "score_cosine": sum(cos) / len(cos), "top1": sum(top1) / len(top1), "top5": sum(top5) / len(top5),
                "heads_checked": len(cos)}
        del cache
    del model
    torch.cuda.empty_cache()
    return {"metric": "tq_estimator_quality", "unit": "cosine / agreement", "data": "synthetic",
            "config": {"workload": "qwen2.5-3b-shaped random-init model, last key as proxy query",
                       "layers": shape["num_hidden_layers"], "q_heads": shape["num_attention_heads"],
                       "kv_heads": shape["num_key_value_heads"], "head_dim": shape["head_dim"], "batch": 1,
                       "contexts": list(contexts), "bits": list(bits_list),
                       "seeds": "keys layer*1000, values layer*1000+500"},
            "results": results}


def main(argv=None) -> None:
    """Console entry: prints the reference script's summary lines, then the JSON record."""
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--contexts", type=int, nargs="+", default=[2048, 4096, 8192])
    ap.add_argument("--bits", type=int, nargs="+", default=[2, 3, 4])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the 36 of the shape (smoke runs)")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("validate needs a CUDA device: turboquant_b200 has no CPU path")
    rec = run_validation(tuple(args.bits), tuple(args.contexts), args.layers, args.device)
    for T in args.contexts:
        print(f"\nContext {T} tokens")
        for b in args.bits:
            r = rec["results"][f"T{T}_b{b}"]
            print(f"  TQ-{b}bit:  compression {r['compression_ratio']:.2f}x   score cosine {r['score_cosine']:.6f}   "
                  f"top-1 {100 * r['top1']:.1f}%   top-5 {100 * r['top5']:.1f}%   ({r['heads_checked']} heads)")
    print()
    print(json.dumps(rec))


if __name__ == "__main__":
    main()
