"""Partitioning of the hot path across the GPUs of one node.

A (batch, KV-head) unit owns its K/V vectors, the G query heads that read them and their output
rows, and the rotation / codebook constants are replicated, so the path shards with no
collective: each process (one per GPU) compresses and attends to a contiguous block of units.
A collective appears only when results are brought together (`gather_rows`, e.g. the logits of an
end-to-end model run); it goes through `torch.distributed` (NCCL on GPUs, gloo in the CPU tests).
"""

from __future__ import annotations

from typing import Callable

import torch


def unit_range(n_units: int, rank: int, world: int) -> tuple[int, int]:
    """Half-open range of units of `rank`: contiguous blocks, sizes differing by at most one,
    the larger blocks first."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside 0..{world - 1}")
    base, extra = divmod(n_units, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_qkv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, rank: int, world: int):
    """The rank's share of q [B, Hq, Sq, D] and k, v [B, Hkv, Sk, D] as views.

    When the batch divides evenly the share is a batch slice (a plain data-parallel replica);
    otherwise units are split below the batch level and every unit becomes a batch element with
    one KV head and its G query heads: q [U, G, Sq, D], k/v [U, 1, Sk, D]."""
    B, Hq, Sq, D = q.shape
    Hkv = k.shape[1]
    if B % world == 0:
        lo, hi = unit_range(B, rank, world)
        return q[lo:hi], k[lo:hi], v[lo:hi]
    G = Hq // Hkv
    lo, hi = unit_range(B * Hkv, rank, world)
    qu = q.reshape(B * Hkv, G, Sq, D)[lo:hi]
    ku = k.reshape(B * Hkv, 1, k.shape[2], D)[lo:hi]
    vu = v.reshape(B * Hkv, 1, v.shape[2], D)[lo:hi]
    return qu, ku, vu


def unshard_output(parts: list[torch.Tensor], B: int, Hq: int) -> torch.Tensor:
    """Inverse of shard_qkv for the per-rank outputs, in rank order -> [B, Hq, Sq, D]."""
    cat = torch.cat(parts, dim=0)
    return cat.reshape(B, Hq, cat.shape[-2], cat.shape[-1])


def sharded_attention(attend: Callable, q, k, v, rank: int, world: int):
    """Run `attend(q_local, k_local, v_local) -> out_local` on this rank's units.  `attend` is
    compress + fused attention in production (see `local_attention`)."""
    ql, kl, vl = shard_qkv(q, k, v, rank, world)
    if ql.shape[0] == 0:
        return ql.new_empty(ql.shape)
    return attend(ql, kl, vl)


def local_attention(key_compressor, val_compressor, causal: bool = True) -> Callable:
    """compress K, compress V, fused attention: the per-rank work of the hot path."""
    from .compressors import compress_kv, fused_attention

    def attend(q, k, v):
        ck, cv = compress_kv(k, v, key_compressor, val_compressor)
        return fused_attention(q, ck, cv, key_compressor, val_compressor, causal=causal)

    return attend


def gather_rows(local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather along dim 0 of tensors whose leading size may differ between ranks (pads to the
    largest, gathers once, trims).  The only collective of an end-to-end run (logits)."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    n = torch.tensor([local.shape[0]], dtype=torch.int64, device=local.device)
    sizes = [torch.zeros_like(n) for _ in range(world)]
    dist.all_gather(sizes, n, group=group)
    sizes = [int(s.item()) for s in sizes]
    width = max(sizes)
    padded = local.new_zeros((width,) + tuple(local.shape[1:]))
    padded[: local.shape[0]] = local
    bufs = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(bufs, padded, group=group)
    return torch.cat([b[:s] for b, s in zip(bufs, sizes)], dim=0)
