"""Multi-rank host logic on the CPU: unit partition, shard / gather round trip with two gloo
ranks, and a rank that never joins (detected on the host by a short process-group timeout)."""

import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_unit_range_is_a_partition():
    from turboquant_b200.sharding import unit_range

    for n in (0, 1, 7, 32, 512):
        for world in (1, 2, 3, 4, 8):
            spans = [unit_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
    with pytest.raises(ValueError):
        unit_range(4, 2, 2)


def _reference_attend(q, k, v):
    """CPU stand-in for compress + fused attention: plain causal GQA attention."""
    g = q.shape[1] // k.shape[1]
    k, v = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
    s = q @ k.transpose(-1, -2) / q.shape[-1] ** 0.5
    s = s + torch.full(s.shape[-2:], float("-inf")).triu(1 + k.shape[2] - q.shape[2])
    return torch.softmax(s, -1) @ v


def _worker(rank, world, port, B, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    from turboquant_b200.sharding import gather_rows, sharded_attention, unshard_output

    g = torch.Generator().manual_seed(0)          # every rank builds the same global problem
    q = torch.randn(B, 4, 9, 16, generator=g)
    k = torch.randn(B, 2, 9, 16, generator=g)
    v = torch.randn(B, 2, 9, 16, generator=g)
    local = sharded_attention(_reference_attend, q, k, v, rank, world)
    flat = gather_rows(local.reshape(-1, 9 * 16))  # the one collective: ragged row gather
    if rank == 0:
        full = unshard_output([flat.reshape(-1, *local.shape[-2:])], B, 4)
        torch.save({"sharded": full, "whole": _reference_attend(q, k, v)}, out_path)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("B", [2, 3])   # even batch: batch slices; odd batch: unit-level split
def test_two_rank_shard_gather_round_trip(B, tmp_path):
    out = str(tmp_path / "res.pt")
    mp.spawn(_worker, args=(2, _free_port(), B, out), nprocs=2, join=True)
    res = torch.load(out)
    assert res["sharded"].shape == res["whole"].shape
    assert torch.allclose(res["sharded"], res["whole"], atol=1e-6)


def _lonely_worker(rank, world, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    from turboquant_b200.sharding import gather_rows

    if rank == 1:          # leaves between steps, with nothing in flight
        return
    try:
        gather_rows(torch.ones(2, 3))
        outcome = "completed"
    except Exception as exc:  # the collective ends with an error instead of hanging
        outcome = type(exc).__name__
    with open(out_path, "w") as fh:
        fh.write(outcome)


def test_missing_rank_is_detected_on_the_host(tmp_path):
    out = str(tmp_path / "outcome.txt")
    mp.spawn(_lonely_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    assert open(out).read() != "completed"
