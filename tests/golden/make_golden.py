"""Generate the golden fixtures in this directory by running the reference.

Usage (only where the reference checkout exists; the fixtures are committed):

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's Python packages from `<reference>/src`, with no CUDA
device visible so that its pure-PyTorch code paths (including the packed-format
fallbacks of its kernel modules) are the ones that run, feeds them small seeded
inputs and stores inputs and outputs as compressed `.npz` files.  The tests
never import the reference; they read these files.
"""

import os
import sys
import warnings

os.environ["CUDA_VISIBLE_DEVICES"] = ""
warnings.filterwarnings("ignore")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def npy(t):
    if isinstance(t, torch.Tensor):
        return t.detach().cpu().numpy()
    return np.asarray(t)


def main(ref_root: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "src"))
    from turboquant_pytorch.compressors import TurboQuantCompressorMSE, TurboQuantCompressorV2
    from turboquant_pytorch.kernels import (asymmetric_attention_scores, lloyd_max_dequantize,
                                            lloyd_max_quantize, pack_bits, unpack_bits)
    from turboquant_pytorch.lloyd_max import solve_lloyd_max

    torch.manual_seed(0)

    # ---- 1. set-up constants -------------------------------------------------
    consts = {}
    for d in (64, 128):
        for bits in (1, 2, 3, 4):
            cents, bounds = solve_lloyd_max(d, bits)
            consts[f"lm_centroids_d{d}_b{bits}"] = npy(cents)
            consts[f"lm_boundaries_d{d}_b{bits}"] = npy(bounds)
        for bits in (2, 3, 4):
            kc = TurboQuantCompressorV2(d, bits, seed=42, use_triton=False)
            vc = TurboQuantCompressorMSE(d, bits, seed=10042, use_triton=False)
            consts[f"key_centroids_d{d}_bits{bits}"] = npy(kc.centroids)
            consts[f"key_boundaries_d{d}_bits{bits}"] = npy(kc.boundaries)
            consts[f"val_centroids_d{d}_bits{bits}"] = npy(vc.centroids)
            consts[f"val_boundaries_d{d}_bits{bits}"] = npy(vc.boundaries)
        consts[f"Pi_seed42_d{d}"] = npy(kc.Pi)
        consts[f"S_seed42_d{d}"] = npy(kc.S)
        consts[f"Pi_seed10042_d{d}"] = npy(vc.Pi)
    np.savez_compressed(os.path.join(HERE, "constants.npz"), **consts)

    # ---- 2. wire format ------------------------------------------------------
    wire = {}
    gen = torch.Generator().manual_seed(7)
    for b in range(1, 9):
        idx = torch.randint(0, 1 << b, (13, 128), generator=gen, dtype=torch.int32)
        wire[f"idx_b{b}"] = npy(idx).astype(np.uint8)
        wire[f"packed_b{b}"] = npy(pack_bits(idx, b))
        assert torch.equal(unpack_bits(pack_bits(idx, b), b, 128), idx)
    for d in (64, 128):
        for b_eff in (1, 2, 3, 4):
            cents, bounds = solve_lloyd_max(d, b_eff)
            rot = torch.randn(37, d, generator=gen) / d ** 0.5
            rot[0, :] = 0.0                       # exact zero on the middle boundary
            rot[1, : bounds.numel()] = bounds     # exact boundary hits
            rot[2, :] = 10.0
            rot[3, :] = -10.0
            packed = lloyd_max_quantize(rot, bounds, b_eff)
            wire[f"rot_d{d}_b{b_eff}"] = npy(rot)
            wire[f"qpacked_d{d}_b{b_eff}"] = npy(packed)
            wire[f"deq_d{d}_b{b_eff}"] = npy(lloyd_max_dequantize(packed, cents.half(), b_eff, d))
    np.savez_compressed(os.path.join(HERE, "wire_format.npz"), **wire)

    # ---- 3. compressors + estimator -----------------------------------------
    comp = {}
    for d in (64, 128):
        B, H, S, Sq = 2, 2, 33, 9
        k = torch.randn(B, H, S, d, generator=gen)
        k[0, 0, 5] = 0.0                          # a zero vector
        k[:, :, :, 3] *= 8.0                      # an outlier channel
        v = torch.randn(B, H, S, d, generator=gen)
        q = torch.randn(B, H, Sq, d, generator=gen)
        comp[f"k_d{d}"], comp[f"v_d{d}"], comp[f"q_d{d}"] = npy(k), npy(v), npy(q)
        for bits in (2, 3, 4):
            kc = TurboQuantCompressorV2(d, bits, seed=42, use_triton=False)
            vc = TurboQuantCompressorMSE(d, bits, seed=10042, use_triton=False)
            ck = kc.compress(k)
            cv = vc.compress(v)
            tag = f"d{d}_bits{bits}"
            comp[f"k_mse_{tag}"] = npy(ck["k_mse"])
            comp[f"qjl_signs_{tag}"] = npy(ck["qjl_signs"])
            comp[f"residual_norm_{tag}"] = npy(ck["residual_norm"])
            comp[f"scores_{tag}"] = npy(kc.asymmetric_attention_scores(q, ck))
            comp[f"v_indices_{tag}"] = npy(cv["indices"])
            comp[f"v_norms_{tag}"] = npy(cv["vec_norms"])
            comp[f"v_recon_{tag}"] = npy(vc.decompress(cv))

            # the reference's packed-format estimator (its CPU fallback), fed with
            # bytes produced by its own quantise/pack functions
            flat = k.reshape(-1, d).float()
            n = torch.norm(flat, dim=-1, keepdim=True)
            rotated = (flat / (n + 1e-8)) @ kc.Pi.T
            p_idx = lloyd_max_quantize(rotated, kc.boundaries, kc.mse_bits)
            p_sgn = pack_bits((ck["qjl_signs"].reshape(-1, d) > 0).to(torch.int32), 1)
            q_rot = (q.float() @ kc.Pi.T).half()
            s_eff = (kc.S.float() @ kc.Pi.T).half()
            coeff = float(np.sqrt(np.pi / 2) / d)
            packed_scores = asymmetric_attention_scores(
                q_rot, p_idx.reshape(B, H, S, -1), p_sgn.reshape(B, H, S, -1), ck["residual_norm"],
                kc.centroids.half().unsqueeze(0).expand(H, -1).contiguous(), s_eff,
                n.squeeze(-1).half().reshape(B, H, S), bits, coeff)
            comp[f"packed_idx_{tag}"] = npy(p_idx)
            comp[f"packed_sgn_{tag}"] = npy(p_sgn)
            comp[f"packed_scores_{tag}"] = npy(packed_scores)
    np.savez_compressed(os.path.join(HERE, "compressors.npz"), **comp)

    # ---- 4. a family adapter end to end (GPT-2, the one that runs unmodified) --
    from transformers import GPT2Config
    from transformers.models.gpt2.modeling_gpt2 import GPT2Attention
    from transformers_turboquant.families.gpt2 import TurboQuantGPT2Attention

    torch.manual_seed(3)
    cfg = GPT2Config(n_embd=128, n_head=2, n_layer=1, n_positions=64,
                     attn_pdrop=0.0, resid_pdrop=0.0)
    cfg._attn_implementation = "eager"
    attn = GPT2Attention(cfg, layer_idx=0).eval()
    with torch.no_grad():
        for p in attn.parameters():
            p.normal_(0.0, 0.1)
    T = 24
    hidden = torch.randn(2, T, 128)
    mask = torch.full((T, T), float("-inf")).triu(1)[None, None]
    fam = {"hidden": npy(hidden), "mask": npy(mask),
           "c_attn_w": npy(attn.c_attn.weight), "c_attn_b": npy(attn.c_attn.bias),
           "c_proj_w": npy(attn.c_proj.weight), "c_proj_b": npy(attn.c_proj.bias)}
    for bits in (2, 3, 4):
        kc = TurboQuantCompressorV2(64, bits, seed=42, use_triton=False)
        vc = TurboQuantCompressorMSE(64, bits, seed=10042, use_triton=False)
        mod = TurboQuantGPT2Attention.from_original(attn, kc, vc).eval()
        with torch.no_grad():
            out = mod(hidden, attention_mask=mask)[0]
        fam[f"out_bits{bits}"] = npy(out)
    np.savez_compressed(os.path.join(HERE, "family_gpt2.npz"), **fam)

    # ---- 5. standalone quantisers (turboquant.py, lloyd_max.py) on CPU ----------------
    from turboquant_pytorch.lloyd_max import LloydMaxCodebook
    from turboquant_pytorch.turboquant import TurboQuantKVCache, TurboQuantMSE, TurboQuantProd
    sa = {}
    g = torch.Generator().manual_seed(7)
    x = torch.randn(96, 128, generator=g)
    x = x / x.norm(dim=-1, keepdim=True)
    y = torch.randn(96, 128, generator=g)
    sa["x"], sa["y"] = npy(x), npy(y)
    for bits in (2, 3, 4):
        mse = TurboQuantMSE(128, bits, seed=42, device="cpu")
        x_hat, idx = mse(x)
        sa[f"mse_idx_b{bits}"], sa[f"mse_xhat_b{bits}"] = npy(idx).astype(np.int32), npy(x_hat)
        prod = TurboQuantProd(128, bits, seed=42, device="cpu")
        c = prod.quantize(x)
        sa[f"prod_idx_b{bits}"] = npy(c["mse_indices"]).astype(np.int32)
        sa[f"prod_signs_b{bits}"] = npy(c["qjl_signs"]).astype(np.int8)
        sa[f"prod_rnorm_b{bits}"] = npy(c["residual_norm"])
        sa[f"prod_ip_b{bits}"] = npy(prod.inner_product(y, c))
        sa[f"prod_proj_b{bits}"] = npy((x - prod.dequantize(c)) @ prod.S.T)   # to discount sign flips near zero
    cb = LloydMaxCodebook(128, 3, use_triton=False)
    sa["codebook_distortion_d128_b3"] = np.float64(cb.distortion)
    sa["codebook_idx"] = npy(cb.quantize(x * 1.0)).astype(np.int32)
    cache = TurboQuantKVCache(128, 128, bits=3, seed=42, device="cpu")
    cache.append(x[:40], y[:40])
    cache.append(x[40:], y[40:])
    sa["cache_scores"] = npy(cache.attention_scores(y[:1]))
    sa["cache_values"] = npy(cache.get_values())
    mem = cache.memory_usage_bits()
    sa["cache_mem"] = np.array([mem["key_bits"], mem["value_bits"], mem["total_bits"], mem["fp16_bits"]], dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "standalone.npz"), **sa)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
