"""CPU oracle for the TurboQuant KV-compression + compressed-attention path.

TEST INFRASTRUCTURE ONLY.  This module is a CPU restatement of the reference
algorithm (SrzStephen/transformers-turboquant) used as the checker for the CUDA
kernels.  Only the test-suite, the smoke check and the CPU-baseline leg of the
benchmark may import it; the product package never does.

Parity status: PINNED.  `tests/golden/make_golden.py` runs the reference's own
Python implementation and stores its inputs/outputs as fixtures; the
`not gpu` tests check every function below against those fixtures and against
the known-answer constants of the reference (codebook values, first matrix
entries for seed 42, the 0x5A packing example).

Each function cites the reference source it follows, as `path:line` relative to
the reference project root.  Float maths uses torch CPU ops in fp32 (what the
reference itself executes); bit-level work uses numpy.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

QJL_SEED_OFFSET = 10000  # src/turboquant_pytorch/compressors.py:66
VALUE_SEED_OFFSET = 10000  # src/transformers_turboquant/patch.py:72


# --------------------------------------------------------------------------
# Set-up: codebook, rotation, QJL matrix
# --------------------------------------------------------------------------

def solve_codebook(d: int, bits: int) -> torch.Tensor:
    """Lloyd-Max centroids for N(0, 1/d) with 2**bits levels, as fp32.

    Follows src/turboquant_pytorch/compressors.py:72-96 (identical copy at
    :248-268): uniform start inside +-3.5 sigma, cell edges at the midpoints and
    +-10.5 sigma, centroid = E[x | cell] by adaptive quadrature, stop when no
    centroid moves by 1e-10 or after 200 sweeps.
    """
    from scipy import integrate

    levels = 1 << bits
    sigma = 1.0 / math.sqrt(d)
    norm_c = 1.0 / math.sqrt(2.0 * math.pi * sigma ** 2)

    def density(x):
        return norm_c * math.exp(-x * x / (2.0 * sigma ** 2))

    def first_moment(x):
        return x * density(x)

    lo, hi = -3.5 * sigma, 3.5 * sigma
    cents = [lo + (hi - lo) * (j + 0.5) / levels for j in range(levels)]
    for _ in range(200):
        mids = [(cents[j] + cents[j + 1]) / 2.0 for j in range(levels - 1)]
        edges = [lo * 3] + mids + [hi * 3]
        updated = []
        for j in range(levels):
            mass, _ = integrate.quad(density, edges[j], edges[j + 1])
            mom, _ = integrate.quad(first_moment, edges[j], edges[j + 1])
            updated.append(mom / mass if mass > 1e-15 else cents[j])
        shift = max(abs(a - b) for a, b in zip(updated, cents))
        if shift < 1e-10:
            break  # the reference keeps the previous iterate on convergence
        cents = updated
    return torch.tensor(cents, dtype=torch.float32)


def rotation_matrix(d: int, seed: int) -> torch.Tensor:
    """Haar-distributed orthogonal Pi [d, d] fp32.

    src/turboquant_pytorch/compressors.py:50-56: QR of a seeded Gaussian matrix,
    columns flipped so that diag(R) is positive.
    """
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    gauss = torch.randn(d, d, generator=gen)
    q, r = torch.linalg.qr(gauss)
    flip = torch.sign(torch.diag(r))
    flip[flip == 0] = 1.0
    return (q * flip.unsqueeze(0)).contiguous()  # qr hands back a column-major Q


def qjl_matrix(d: int, key_seed: int) -> torch.Tensor:
    """Gaussian sketch matrix S [d, d] fp32, drawn with seed key_seed + 10000.

    src/turboquant_pytorch/compressors.py:65-67.
    """
    gen = torch.Generator(device="cpu")
    gen.manual_seed(key_seed + QJL_SEED_OFFSET)
    return torch.randn(d, d, generator=gen)


@dataclass
class KeyParams:
    """Constants of one key compressor (compressors.py:42-70)."""
    head_dim: int
    bits: int
    Pi: torch.Tensor
    S: torch.Tensor
    centroids: torch.Tensor

    @property
    def mse_bits(self) -> int:
        return max(self.bits - 1, 1)

    @property
    def boundaries(self) -> torch.Tensor:
        return (self.centroids[:-1] + self.centroids[1:]) / 2

    @property
    def S_eff(self) -> torch.Tensor:
        """S @ Pi^T: the sketch matrix seen from rotated coordinates
        (compressors.py:189, tests/test_kernels.py:296-314)."""
        return self.S.float() @ self.Pi.float().T

    def to(self, device) -> "KeyParams":
        """The same constants on another device (the reference's `device=` constructor argument)."""
        return KeyParams(self.head_dim, self.bits, self.Pi.to(device), self.S.to(device), self.centroids.to(device))


@dataclass
class ValueParams:
    """Constants of one value compressor (compressors.py:230-246)."""
    head_dim: int
    bits: int
    Pi: torch.Tensor
    centroids: torch.Tensor

    @property
    def boundaries(self) -> torch.Tensor:
        return (self.centroids[:-1] + self.centroids[1:]) / 2

    def to(self, device) -> "ValueParams":
        return ValueParams(self.head_dim, self.bits, self.Pi.to(device), self.centroids.to(device))


def make_key_params(d: int, bits: int, seed: int) -> KeyParams:
    return KeyParams(d, bits, rotation_matrix(d, seed), qjl_matrix(d, seed),
                     solve_codebook(d, max(bits - 1, 1)))


def make_value_params(d: int, bits: int, seed: int) -> ValueParams:
    return ValueParams(d, bits, rotation_matrix(d, seed), solve_codebook(d, bits))


def layer_seeds(seed: int, layer: int) -> tuple[int, int]:
    """(key seed, value seed) of layer `layer` (patch.py:62-75)."""
    return seed + layer, seed + layer + VALUE_SEED_OFFSET


# --------------------------------------------------------------------------
# Wire format: LSB-first bit stream per row
# --------------------------------------------------------------------------

def packed_cols(d: int, b: int) -> int:
    """Bytes per row for d fields of b bits (kernels/bit_ops.py:162-164)."""
    return (d * b + 7) // 8


def pack_bits(indices: np.ndarray, b: int) -> np.ndarray:
    """int[N, d] -> uint8[N, ceil(d*b/8)].

    Field i occupies stream bits [i*b, i*b+b); stream bit g lives in byte g//8
    at bit g%8 (kernels/bit_ops.py:5-7, :243-286).  Implemented as a flat bit
    matrix so that it shares no structure with the code under test.
    """
    idx = np.asarray(indices).astype(np.int64)
    n, d = idx.shape
    field_bits = (idx[:, :, None] >> np.arange(b)[None, None, :]) & 1  # [N, d, b]
    stream = field_bits.reshape(n, d * b)
    pad = packed_cols(d, b) * 8 - d * b
    if pad:
        stream = np.concatenate([stream, np.zeros((n, pad), dtype=stream.dtype)], axis=1)
    weights = (1 << np.arange(8)).astype(np.int64)
    return (stream.reshape(n, -1, 8) * weights).sum(axis=2).astype(np.uint8)


def unpack_bits(packed: np.ndarray, b: int, d: int) -> np.ndarray:
    """uint8[N, ceil(d*b/8)] -> int32[N, d] (kernels/bit_ops.py:288-326)."""
    p = np.asarray(packed, dtype=np.uint8)
    n = p.shape[0]
    stream = ((p[:, :, None] >> np.arange(8)[None, None, :]) & 1).reshape(n, -1)
    fields = stream[:, : d * b].reshape(n, d, b).astype(np.int64)
    return (fields * (1 << np.arange(b))).sum(axis=2).astype(np.int32)


def quantize_indices(rotated: torch.Tensor, centroids: torch.Tensor) -> torch.Tensor:
    """Nearest-centroid index, first minimum on ties (compressors.py:141-142)."""
    return (rotated.unsqueeze(-1) - centroids).abs().argmin(dim=-1)


def quantize_by_boundaries(rotated: torch.Tensor, boundaries: torch.Tensor) -> torch.Tensor:
    """Index = number of boundaries strictly below y (kernels/quantize.py:334-337,
    pinned by tests/test_kernels.py:108-138)."""
    flat = rotated.reshape(-1).contiguous().float()
    return torch.searchsorted(boundaries.contiguous().float(), flat).reshape(rotated.shape)


def quantize_packed(rotated: torch.Tensor, boundaries: torch.Tensor, b_eff: int) -> np.ndarray:
    """fp32[N, d] -> packed uint8 rows (kernels/quantize.py:299-339)."""
    idx = quantize_by_boundaries(rotated, boundaries)
    return pack_bits(idx.numpy(), b_eff)


def dequantize_packed(packed: np.ndarray, centroids: torch.Tensor, b: int, d: int) -> torch.Tensor:
    """packed rows -> centroid values fp32[N, d] (kernels/quantize.py:341-369,
    without its fp16 table)."""
    idx = torch.from_numpy(unpack_bits(packed, b, d).astype(np.int64))
    return centroids.float()[idx]


# --------------------------------------------------------------------------
# Compressors
# --------------------------------------------------------------------------

def _normalise_rotate(states: torch.Tensor, Pi: torch.Tensor):
    """compressors.py:104-112 / :272-276."""
    d = states.shape[-1]
    flat = states.reshape(-1, d).float()
    norms = torch.norm(flat, dim=-1, keepdim=True)
    rotated = (flat / (norms + 1e-8)) @ Pi.float().T
    return flat, norms, rotated


def key_compress(states: torch.Tensor, P: KeyParams, pack: bool = True) -> dict:
    """Key compression, reference PyTorch branch (compressors.py:98-112, :139-161).
    `pack=False` leaves out the packed wire-format view (host-side numpy work that the
    reference's PyTorch branch does not do): what a timed baseline runs, on any device.

    Returns the reference's dict (`k_mse` fp16, `qjl_signs` int8 +-1,
    `residual_norm` fp16, `shape`) plus the quantities the packed wire format
    stores, derived from the same decisions: `indices` (int64 [N, d]),
    `sign_bits` (uint8 0/1 [N, d]), `vec_norms` fp16, `packed_key_indices`,
    `packed_qjl_signs` (numpy uint8; compressors.py:132-138).
    """
    B, H, S, D = states.shape
    flat, norms, rotated = _normalise_rotate(states, P.Pi)
    idx = quantize_indices(rotated, P.centroids.float())
    k_mse = (P.centroids.float()[idx] @ P.Pi.float()) * norms
    resid = flat - k_mse
    rnorm = torch.norm(resid, dim=-1)
    proj = resid @ P.S.float().T
    bits01 = (proj >= 0)
    if not pack:
        return {"k_mse": k_mse.to(torch.float16).reshape(B, H, S, D),
                "qjl_signs": (bits01.to(torch.int8) * 2 - 1).reshape(B, H, S, D),
                "residual_norm": rnorm.to(torch.float16).reshape(B, H, S), "shape": (B, H, S, D)}
    return {
        "k_mse": k_mse.to(torch.float16).reshape(B, H, S, D),
        "qjl_signs": (bits01.to(torch.int8) * 2 - 1).reshape(B, H, S, D),
        "residual_norm": rnorm.to(torch.float16).reshape(B, H, S),
        "shape": (B, H, S, D),
        # packed-format view of the same decisions
        "indices": idx,
        "sign_bits": bits01.to(torch.uint8),
        "vec_norms": norms.squeeze(-1).to(torch.float16).reshape(B, H, S),
        "packed_key_indices": pack_bits(idx.numpy(), P.mse_bits),
        "packed_qjl_signs": pack_bits(bits01.to(torch.int32).numpy(), 1),
        "k_mse_fp32": k_mse.reshape(B, H, S, D),
        "rotated": rotated,
        "projected": proj,
    }


def value_compress(states: torch.Tensor, P: ValueParams, pack: bool = True) -> dict:
    """Value compression (compressors.py:270-294); `pack` as in key_compress."""
    B, H, S, D = states.shape
    _, norms, rotated = _normalise_rotate(states, P.Pi)
    idx = quantize_indices(rotated, P.centroids.float())
    if not pack:
        return {"indices": idx.to(torch.uint8), "vec_norms": norms.squeeze(-1).to(torch.float16), "shape": (B, H, S, D)}
    return {
        "indices": idx.to(torch.uint8),
        "vec_norms": norms.squeeze(-1).to(torch.float16),
        "shape": (B, H, S, D),
        "packed_indices": pack_bits(idx.numpy(), P.bits),
        "rotated": rotated,
    }


def value_decompress(comp: dict, P: ValueParams) -> torch.Tensor:
    """compressors.py:312-317: centroid lookup, back-rotation, rescale; fp32."""
    B, H, S, D = comp["shape"]
    recon = P.centroids.float()[comp["indices"].long()] @ P.Pi.float()
    return (recon * comp["vec_norms"].float().unsqueeze(-1)).reshape(B, H, S, D)


# --------------------------------------------------------------------------
# Score estimator
# --------------------------------------------------------------------------

def qjl_coeff(m: int) -> float:
    """sqrt(pi/2)/m (compressors.py:219-220)."""
    return math.sqrt(math.pi / 2) / m


def scores_literal(q: torch.Tensor, comp: dict, P: KeyParams) -> torch.Tensor:
    """Reference PyTorch branch, literally (compressors.py:201-224): uses the
    fp16-stored `k_mse`.  fp32 [B, H, Sq, Sk]."""
    qf = q.float()
    term1 = qf @ comp["k_mse"].float().transpose(-2, -1)
    sketch = (qf @ P.S.float().T) @ comp["qjl_signs"].float().transpose(-2, -1)
    return term1 + qjl_coeff(P.S.shape[0]) * sketch * comp["residual_norm"].float().unsqueeze(-2)


def scores_from_packed(q: torch.Tensor, packed_idx: np.ndarray, packed_signs: np.ndarray,
                       vec_norms: torch.Tensor, residual_norm: torch.Tensor,
                       P: KeyParams, shape) -> torch.Tensor:
    """The estimator evaluated in fp32 from the packed wire format, in rotated
    coordinates (kernels/attention.py:380-461 and compressors.py:178-200, with the
    fp16 casts of q_rot, S_eff and the centroid table left out):

        score = n_k * <q Pi^T, C[idx_k]> + coeff * rn_k * <q Pi^T S_eff^T, +-1_k>

    `vec_norms`, `residual_norm` are the stored fp16 values.  This is the
    fp32-mode parity target for the CUDA path, which consumes exactly these bytes.
    """
    B, H, Sk, D = shape
    idx = torch.from_numpy(unpack_bits(packed_idx.reshape(B * H * Sk, -1), P.mse_bits, D).astype(np.int64))
    sgn = torch.from_numpy(unpack_bits(packed_signs.reshape(B * H * Sk, -1), 1, D).astype(np.float32)) * 2 - 1
    k_rot = P.centroids.float()[idx].reshape(B, H, Sk, D)
    sgn = sgn.reshape(B, H, Sk, D)
    q_rot = q.float() @ P.Pi.float().T
    q_s = q_rot @ P.S_eff.T
    term1 = (q_rot @ k_rot.transpose(-2, -1)) * vec_norms.float().reshape(B, H, 1, Sk)
    term2 = (q_s @ sgn.transpose(-2, -1)) * residual_norm.float().reshape(B, H, 1, Sk)
    return term1 + qjl_coeff(D) * term2


def values_from_packed(packed_idx: np.ndarray, vec_norms: torch.Tensor, P: ValueParams, shape) -> torch.Tensor:
    """Packed value rows -> fp32 [B, H, S, D] (compressors.py:301-311 with an fp32 table)."""
    B, H, S, D = shape
    rot = dequantize_packed(packed_idx.reshape(B * H * S, -1), P.centroids, P.bits, D)
    return ((rot @ P.Pi.float()) * vec_norms.float().reshape(-1, 1)).reshape(B, H, S, D)


# --------------------------------------------------------------------------
# Attention core of the family adapters
# --------------------------------------------------------------------------

def causal_mask(sq: int, sk: int, dtype=torch.float32) -> torch.Tensor:
    """Additive mask HF's eager path hands to the adapter: query i (aligned to the
    end of the key sequence) may see keys <= i + sk - sq."""
    i = torch.arange(sq).unsqueeze(1) + (sk - sq)
    j = torch.arange(sk).unsqueeze(0)
    return torch.where(j <= i, 0.0, float("-inf")).to(dtype)


def attention_core(q, k, v, KP: KeyParams, VP: ValueParams, mask=None, literal=True):
    """The body shared by the family adapters (families/llama.py:100-114,
    gpt2.py:90-110): GQA expansion, compress K and V, estimator scores,
    / sqrt(d), + additive mask, fp32 softmax cast to q.dtype, @ decompressed V.

    q [B, Hq, Sq, D]; k, v [B, Hkv, Sk, D]; mask broadcastable to [B, Hq, Sq, Sk]
    or None.  literal=True evaluates scores exactly as the reference's PyTorch
    branch does (fp16 `k_mse`); literal=False evaluates them from the packed
    wire format in fp32.  Returns (out [B, Hq, Sq, D] in q.dtype, scores fp32).
    """
    B, Hq, Sq, D = q.shape
    groups = Hq // k.shape[1]
    k = k.repeat_interleave(groups, dim=1)
    v = v.repeat_interleave(groups, dim=1)
    ck = key_compress(k, KP)
    cv = value_compress(v, VP)
    if literal:
        scores = scores_literal(q, ck, KP)
    else:
        scores = scores_from_packed(q, ck["packed_key_indices"], ck["packed_qjl_signs"],
                                    ck["vec_norms"], ck["residual_norm"], KP, ck["shape"])
    raw = scores
    scores = scores / math.sqrt(D)
    if mask is not None:
        scores = scores + mask
    weights = torch.softmax(scores.float(), dim=-1).to(q.dtype)
    vals = value_decompress(cv, VP).to(q.dtype)
    return weights @ vals, raw


def attention_core_chunked(q, k, v, KP: KeyParams, VP: ValueParams, causal=True,
                           q_chunk=1024, literal=True):
    """attention_core without GQA expansion of the compressed tensors and without
    the full [Sq, Sk] score matrix: same arithmetic per (head, query block), used
    where the literal form would not fit in memory.  Causal only."""
    B, Hq, Sq, D = q.shape
    Hkv, Sk = k.shape[1], k.shape[2]
    groups = Hq // Hkv
    ck = key_compress(k, KP)
    cv = value_compress(v, VP)
    vals = value_decompress(cv, VP).to(q.dtype)  # [B, Hkv, Sk, D]
    out = torch.empty_like(q)
    k_mse = ck["k_mse"].float() if literal else ck["k_mse_fp32"]
    sgn = ck["qjl_signs"].float()
    rn = ck["residual_norm"].float()
    coeff = qjl_coeff(D)
    for h in range(Hq):
        g = h // groups
        for s0 in range(0, Sq, q_chunk):
            s1 = min(s0 + q_chunk, Sq)
            hi = s1 + (Sk - Sq) if causal else Sk
            qf = q[:, h, s0:s1].float()
            sc = qf @ k_mse[:, g, :hi].transpose(-2, -1)
            sc = sc + coeff * ((qf @ KP.S.float().T) @ sgn[:, g, :hi].transpose(-2, -1)) * rn[:, g, None, :hi]
            sc = sc / math.sqrt(D)
            if causal:
                sc = sc + causal_mask(Sq, Sk)[s0:s1, :hi]
            w = torch.softmax(sc, dim=-1).to(q.dtype)
            out[:, h, s0:s1] = w @ vals[:, g, :hi]
    return out
