"""Benchmark of the TurboQuant hot path: fused KV compression + compressed causal attention.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--bits 3]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Workload ("op_level_gqa4_s8192"): bf16 Q [4,32,8192,128], K,V [4,8,8192,128] drawn N(0,1)
with 4 key channels per head scaled x8, rotation/QJL matrices from seed 42, causal, 3-bit by
default.  One step = compress K, compress V, fused attention over the whole batch.  With N
ranks every rank runs this workload on its own (batch x KV-head) shard, no data-path
collective (weak scaling).  Inputs (402 MB) exceed the 126 MB L2, so no flush between
steps.  Prints ONE JSON line on rank 0.

`--impl reference` times the CPU restatement of the reference's PyTorch path (oracle/) on the
host cores, on a bounded sample of the same workload.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import math
import os

# NCCL prints a version banner on STDOUT at its VERSION (and WARN) debug level, and NCCL_DEBUG_FILE does not
# move it; stdout must carry the JSON line only, so that level is lowered before torch loads NCCL.
if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
    os.environ["NCCL_DEBUG"] = "NONE"
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "transformers-turboquant_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

B, HQ, HKV, S, D = 4, 32, 8, 8192, 128
METRIC = "fused_tq_attention_keys_per_s"
UNIT = "keys/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--bits", type=int, default=3)
    ap.add_argument("--seq", type=int, default=S, help="sequence length (default: the named workload)")
    ap.add_argument("--batch", type=int, default=B)
    ap.add_argument("--workload", default="op", choices=["op", "llama8b", "deepseek7b", "quality", "decode"],
                    help="op: the op-level headline workload (default); llama8b / deepseek7b: end-to-end prefill of a "
                         "random-init model of that shape through apply_turboquant; quality: estimator quality "
                         "metrics on a Qwen2.5-3B-shaped attention layer; decode: one new token per sequence against a long "
                         "compressed KV cache (split-KV kernel)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


def make_inputs(batch, seq, device, seed=0):
    """Synthetic stand-in for the named op-level configuration."""
    g = torch.Generator(device=device).manual_seed(seed)
    q = torch.randn(batch, HQ, seq, D, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    k = torch.randn(batch, HKV, seq, D, generator=g, device=device, dtype=torch.float32)
    v = torch.randn(batch, HKV, seq, D, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    cg = torch.Generator().manual_seed(1)
    for h in range(HKV):
        ch = torch.randperm(D, generator=cg)[:4].to(device)
        k[:, h, :, ch] *= 8.0
    return q, k.to(torch.bfloat16), v


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop_evt = threading.Event()
        self.ok = True

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                     nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
                     nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
                     nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
                     nv.nvmlClocksThrottleReasonHwPowerBrakeSlowdown: "hw_power_brake"}
            while not self._stop_evt.is_set():
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                self.reasons.update(n for bit, n in names.items() if mask & bit)
                time.sleep(0.01)
        except Exception as exc:  # NVML missing: report, never fail the run
            self.ok = False
            self.error = repr(exc)

    def finish(self):
        self._stop_evt.set()
        self.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                    "note": getattr(self, "error", "no samples")}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def causal_pairs(batch, seq):
    return batch * HQ * seq * (seq + 1) // 2


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"tflops": p.get("bf16_tflops_sustained", p.get("bf16_tflops")), "hbm_gbs": p.get("hbm_gbs"),
                "source": "measured (MEASURED_PEAKS.json, sustained bf16)"}
    return {"tflops": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


CPU_Q_ROWS = 1024  # query rows of the unit that the CPU sample actually evaluates


def cpu_sample(bits, seq, repeats=1, threads=None):
    """Reference PyTorch path (oracle restatement, literal arithmetic: compress of the
    GQA-expanded K/V, full-width score rows, fp32 softmax, PV) on one (batch, query-head) unit
    of the workload.  Compression is timed on all `seq` keys; the score/softmax/PV part on the
    last CPU_Q_ROWS query rows against all keys and scaled by seq/CPU_Q_ROWS (the reference
    computes every row at full width whatever the mask).  Returns seconds per unit."""
    from oracle import tq_oracle as orc
    threads = threads or os.cpu_count()
    torch.set_num_threads(threads)
    kp, vp = orc.make_key_params(D, bits, 42), orc.make_value_params(D, bits, 10042)
    g = torch.Generator().manual_seed(0)
    rows = min(CPU_Q_ROWS, seq)
    q = torch.randn(1, 1, rows, D, generator=g).to(torch.bfloat16)
    k = torch.randn(1, 1, seq, D, generator=g).to(torch.bfloat16)
    v = torch.randn(1, 1, seq, D, generator=g).to(torch.bfloat16)
    mask = orc.causal_mask(seq, seq)[-rows:]
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        ck, cv = orc.key_compress(k, kp), orc.value_compress(v, vp)
        t1 = time.perf_counter()
        sc = orc.scores_literal(q, ck, kp) / math.sqrt(D) + mask
        w = torch.softmax(sc.float(), dim=-1).to(q.dtype)
        _ = w @ orc.value_decompress(cv, vp).to(q.dtype)
        t2 = time.perf_counter()
        best = min(best, (t1 - t0) + (t2 - t1) * (seq / rows))
    return best, threads


def run_reference(args):
    """The reference arm: CPU, rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    seq, batch = args.seq, args.batch
    cpu_sample(args.bits, min(seq, 1024))  # warm the thread pool and allocator
    for _ in range(max(args.warmup - 1, 0)):
        cpu_sample(args.bits, seq)
    per_unit = sum(cpu_sample(args.bits, seq)[0] for _ in range(args.steps)) / args.steps
    units = batch * HQ  # the reference expands K/V to one copy per query head before compressing
    step_s = per_unit * units
    keys = batch * HKV * seq
    value = keys / step_s
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "op_level_gqa4_s8192", "batch": batch, "q_heads": HQ, "kv_heads": HKV,
                       "seq_len": seq, "head_dim": D, "bits": args.bits, "causal": True},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
                             "sample": f"per step one (batch, query head) unit of {units}: compress of S={seq} keys and "
                                       f"values, score/softmax/PV rows for {min(CPU_Q_ROWS, seq)} of {seq} queries "
                                       "at full width, scaled to the unit and then linearly to the workload"},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


MODEL_SHAPES = {
    # name: (layers, hidden, q heads, kv heads, head_dim, ffn, vocab, rope_theta, global batch, seq)
    "llama8b": (32, 4096, 32, 8, 128, 14336, 128256, 500000.0, 8, 4096),
    "deepseek7b": (30, 4096, 32, 32, 128, 11008, 102400, 10000.0, 16, 4096),
}


def run_model(args):
    """End-to-end prefill tokens/s of a random-init LLaMA-architecture model (bf16, N(0, 0.02) init, uniform
    random tokens) with every attention layer replaced by apply_turboquant(bits, seed=42).  The global
    batch is split over the ranks (full replica per GPU, strong scaling); the only collective is the
    all_gather of the last-token logits, inside the timed region."""
    import turboquant_b200 as tq
    from transformers import LlamaConfig, LlamaForCausalLM
    from turboquant_b200.sharding import gather_rows, unit_range

    L, hid, hq, hkv, hd, ffn, vocab, theta, gbatch, seq = MODEL_SHAPES[args.workload]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    cfg = LlamaConfig(num_hidden_layers=L, hidden_size=hid, num_attention_heads=hq, num_key_value_heads=hkv,
                      head_dim=hd, intermediate_size=ffn, vocab_size=vocab, rope_theta=theta,
                      max_position_embeddings=seq, initializer_range=0.02)
    torch.manual_seed(0)
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(dev):
        model = LlamaForCausalLM(cfg).eval()
    torch.set_default_dtype(torch.float32)
    ids_all = torch.randint(0, vocab, (gbatch, seq), generator=torch.Generator().manual_seed(0))
    lo, hi = unit_range(gbatch, rank, world)
    ids_host = ids_all[lo:hi].pin_memory()

    def forward(m):
        with torch.no_grad():
            ids = ids_host.to(dev, non_blocking=True)
            last = m(ids, logits_to_keep=1).logits[:, -1].float()
            if dist is not None:
                last = gather_rows(last)
            return last.cpu()

    def timed(m, steps, warm):
        for _ in range(warm):
            forward(m)
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            out = forward(m)
        e1.record()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)
        t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), out

    steps, warm = max(1, min(args.steps, 5)), max(1, min(args.warmup, 3))
    ms_plain, logits_plain = timed(model, steps, warm)
    tq.apply_turboquant(model, bits=args.bits, seed=42)
    sampler = ClockSampler(local)
    sampler.start()
    ms_tq, logits_tq = timed(model, steps, warm)
    clocks = sampler.finish()
    if rank == 0:
        cos = torch.nn.functional.cosine_similarity(logits_tq, logits_plain, dim=-1).mean().item()
        line = {"metric": f"{args.workload}_{args.bits}bit_prefill_tok_per_s", "value": gbatch * seq / (ms_tq * 1e-3),
                "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warm, "ms_per_step": ms_tq,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic", "config": {"workload": args.workload, "global_batch": gbatch, "seq_len": seq,
                                                "layers": L, "bits": args.bits, "parallelism": f"dp{world}",
                                                "logits": "last token, all_gather inside the timed region"},
                "clocks": clocks,
                "e2e": {"value": gbatch * seq / (ms_tq * 1e-3), "unit": "tok/s",
                        "h2d_bytes_per_step": ids_host.numel() * 8, "d2h_bytes_per_step": gbatch * vocab * 4},
                "uncompressed_attention_tok_per_s": gbatch * seq / (ms_plain * 1e-3),
                "last_token_logit_cosine_vs_uncompressed": cos, "device_wait_faults": tq.device_fault_count(dev)}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_quality(args):
    """Estimator quality on a Qwen2.5-3B-shaped attention layer (16 query heads, 2 KV heads, d=128), the
    synthetic stand-in for the reference's validate script (validate.py:137-196): compression ratio by bit
    accounting, cosine between estimator and exact score rows, top-1 / top-5 agreement of the per-head
    argmax, with the last key as proxy query.  Random-init projections of N(0,1) hidden states."""
    import turboquant_b200 as tq
    dev = torch.device("cuda", 0)
    out = {}
    for T in (2048, 4096, 8192):
        g = torch.Generator(device=dev).manual_seed(T)
        k = torch.randn(1, 2, T, D, generator=g, device=dev).to(torch.bfloat16)
        q = k[:, :, -1:, :]  # last key as proxy query, per KV head
        exact = (q.float() @ k.float().transpose(-1, -2))[0, :, 0]  # [H, T]
        for bits in (2, 3, 4):
            kc = tq.TurboQuantCompressorV2(D, bits, 0, device=str(dev))
            est = kc.asymmetric_attention_scores(q, kc.compress(k))[0, :, 0]
            cos = torch.nn.functional.cosine_similarity(est, exact, dim=-1).mean().item()
            top1 = (est.argmax(-1) == exact.argmax(-1)).float().mean().item()
            top5 = torch.stack([(exact.argmax(-1)[h] == est[h].topk(5).indices).any() for h in range(2)]).float().mean().item()
            ratio = 32.0 * D / (2 * bits * D + 48)
            out[f"T{T}_b{bits}"] = {"compression_ratio": round(ratio, 2), "score_cosine": cos, "top1": top1, "top5": top5}
    print(json.dumps({"metric": "tq_estimator_quality", "workload": "qwen2.5-3b-shaped attention, synthetic", "results": out}))


def run_decode(args):
    """Decode step against a resident compressed KV cache: one query token per sequence (32 query / 8 KV heads,
    d = 128) attends to Sk = 32768 cached keys, batch 8 — the per-GPU share of the scaling shape K,V
    [64, 8, 32768, 128] over 8 GPUs.  The cache (`CompressedKVCache`, capacity above the keys in use) is filled
    outside the timed region; a step is `cache.attend(q)`.  The work is bound by the packed bytes: per key (16 (b-1) + 16 + 4) + (16 b + 2)."""
    import turboquant_b200 as tq
    from turboquant_b200 import _lib
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    batch, sk, bits = 8, 32768, args.bits
    g = torch.Generator(device=dev).manual_seed(0)
    k = torch.randn(batch, HKV, sk, D, generator=g, device=dev).to(torch.bfloat16)
    v = torch.randn(batch, HKV, sk, D, generator=g, device=dev).to(torch.bfloat16)
    q = torch.randn(batch, HQ, 1, D, generator=g, device=dev).to(torch.bfloat16)
    kc = tq.TurboQuantCompressorV2(D, bits, 42, device=str(dev))
    vc = tq.TurboQuantCompressorMSE(D, bits, 10042, device=str(dev))
    # a persistent cache with room to grow: the kernel reads rows with the capacity as their stride
    cache = tq.CompressedKVCache(kc, vc, batch, HKV, sk + 256, device=dev)
    cache.append(k, v)
    k_new, v_new = k[:, :, -1:].clone(), v[:, :, -1:].clone()
    del k, v

    def timed(steps):
        for _ in range(max(args.warmup, 3)):
            cache.attend(q, causal=True)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            out = cache.attend(q, causal=True)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps, out

    def generation_steps(steps):
        """Append the new token's key and value (two compression launches + six small copies), then attend."""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            cache.append(k_new, v_new)
            cache.attend(q, causal=True)
        e1.record()
        torch.cuda.synchronize()
        cache.length = sk
        return e0.elapsed_time(e1) / steps

    sampler = ClockSampler(0)
    sampler.start()
    ms, out = timed(args.steps)
    clocks = sampler.finish()
    # per-kernel times from a second pass: the profiling events sit between the three launches of a call and
    # keep them from overlapping (programmatic dependent launch), so the timed pass above runs without them
    _lib.check(_lib.lib.tq_profile_begin(max(args.steps, 1) + max(args.warmup, 3)))
    timed(args.steps)
    ms_sum, launches = (ctypes.c_float * 5)(), (ctypes.c_int * 5)()
    _lib.check(_lib.lib.tq_profile_end(ms_sum, launches))
    generation_steps(3)
    gen_ms = generation_steps(min(max(args.steps, 1), 200))
    kern_ms = ms_sum[3] / max(launches[3], 1)
    keys = batch * HKV * sk
    bytes_per_key = (16 * (bits - 1) + 16 + 4) + (16 * bits + 2)
    peaks = measured_peaks()
    achieved = keys * bytes_per_key / (kern_ms * 1e-3) / 1e9
    line = {"metric": "tq_decode_keys_per_s", "value": keys / (ms * 1e-3), "unit": "keys/s", "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "decode_b8_h32_kv8_sk32768", "batch_per_gpu": batch, "q_heads": HQ, "kv_heads": HKV,
                       "new_tokens": 1, "cached_keys": sk, "head_dim": D, "bits": bits,
                       "l2": f"packed cache ({keys * bytes_per_key / 1e6:.0f} MB) exceeds the 126 MB L2; no flush"},
            "clocks": clocks, "gpu_launches": 3 * args.steps,  # per call: query preparation, split-KV kernel, merge + back-rotation
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                         "kernel": "decode_kernel", "ms_per_launch": kern_ms,
                         "peak_source": peaks["source"]},
            "kernel_ms": {"prepare_queries": ms_sum[2] / max(launches[2], 1), "decode": kern_ms,
                          "merge_and_back_rotation": ms_sum[4] / max(launches[4], 1)},
            "generation_step_ms": gen_ms,  # append one token per sequence to the cache, then attend
            "device_wait_faults": tq.device_fault_count(dev), "output_norm": float(out.float().norm())}
    print(json.dumps(line), flush=True)


def main():
    args = parse()
    if args.workload in MODEL_SHAPES:
        return run_model(args)
    if args.workload == "quality":
        return run_quality(args)
    if args.workload == "decode":
        return run_decode(args)
    if args.impl == "reference":
        return run_reference(args)

    import turboquant_b200 as tq
    from turboquant_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    batch, seq, bits = args.batch, args.seq, args.bits
    q, k, v = make_inputs(batch, seq, dev, seed=rank)  # every rank owns its own shard of units
    kc = tq.TurboQuantCompressorV2(D, bits, 42, device=str(dev))
    vc = tq.TurboQuantCompressorMSE(D, bits, 10042, device=str(dev))

    def step(qd, kd, vd):
        ck = kc.compress(kd)
        cv = vc.compress(vd)
        return tq.fused_attention(qd, ck, cv, kc, vc, causal=True)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(args.warmup, 3)):
        out = step(q, k, v)
    barrier()

    sampler = ClockSampler(torch.cuda.current_device() if "CUDA_VISIBLE_DEVICES" not in os.environ else local)
    sampler.start()
    _lib.check(_lib.lib.tq_profile_begin(max(args.steps, 1)))
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        out = step(q, k, v)
    ev1.record()
    barrier()
    ms_sum = (ctypes.c_float * 5)()
    launches = (ctypes.c_int * 5)()
    _lib.check(_lib.lib.tq_profile_end(ms_sum, launches))
    clocks = sampler.finish()
    elapsed_ms = ev0.elapsed_time(ev1)
    t = torch.tensor([elapsed_ms], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    keys_per_rank = batch * HKV * seq
    value = keys_per_rank * world / (ms_per_step * 1e-3)

    # ---- end to end through the public API with pinned host buffers -----------------------
    # Every step copies its q, k, v from pinned host memory to the device, runs compress + fused attention
    # through the public Python API and copies the output back to pinned host memory.  Copies and compute of
    # consecutive steps overlap on three streams (double-buffered device inputs), as a serving loop would.
    e2e = None
    if not args.no_e2e:
        hq, hk, hv = (t_.cpu().pin_memory() for t_ in (q, k, v))
        houts = [torch.empty(out.shape, dtype=out.dtype).pin_memory() for _ in range(2)]
        n_e2e = max(4, min(args.steps, 10))
        s_in, s_run, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        dbuf = [[torch.empty_like(t_) for t_ in (q, k, v)] for _ in range(2)]
        free_in = [torch.cuda.Event() for _ in range(2)]    # device inputs of slot i consumed
        free_out = [torch.cuda.Event() for _ in range(2)]   # host output of slot i written

        def e2e_loop(n):
            outs = []
            for i in range(n):
                sl = i & 1
                with torch.cuda.stream(s_in):
                    s_in.wait_event(free_in[sl])
                    for d_, h_ in zip(dbuf[sl], (hq, hk, hv)):
                        d_.copy_(h_, non_blocking=True)
                    ready = torch.cuda.Event()
                    ready.record(s_in)
                with torch.cuda.stream(s_run):
                    s_run.wait_event(ready)
                    o = step(*dbuf[sl])
                    free_in[sl].record(s_run)
                    done = torch.cuda.Event()
                    done.record(s_run)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(done)
                    s_out.wait_event(free_out[sl])
                    houts[sl].copy_(o, non_blocking=True)
                    free_out[sl].record(s_out)
                outs.append(o)  # keep the device output alive until its copy has been issued and run
            return outs

        for ev in free_in + free_out:
            ev.record(torch.cuda.current_stream(dev))
        barrier()
        e2e_loop(2)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s_in)
        keep = e2e_loop(n_e2e)
        s_out.wait_stream(s_run)
        s_out.wait_stream(s_in)
        e1.record(s_out)
        barrier()
        del keep
        te = torch.tensor([e0.elapsed_time(e1) / n_e2e], device=dev, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e = {"value": keys_per_rank * world / (float(te.item()) * 1e-3), "unit": UNIT,
               "h2d_bytes_per_step": sum(h.numel() * h.element_size() for h in (hq, hk, hv)),
               "d2h_bytes_per_step": houts[0].numel() * houts[0].element_size(), "ms_per_step": float(te.item()),
               "steps": n_e2e, "overlap": "H2D, compute and D2H of consecutive steps on three streams"}

    faults = tq.device_fault_count(dev)
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel (fused attention: tensor-core bound) ---------------
    peaks = measured_peaks()
    attn_ms = ms_sum[3] / max(launches[3], 1)
    # algorithmic flops of the fused kernel: 2d (q.K_hat) + 2d (q_s.sign) + 2d (P.V_hat) per causal pair, plus
    # per query row the preparation q [Pi ; coeff S]^T (2 * 2d * d) and the output back-rotation (2 d^2)
    flops = 6.0 * D * causal_pairs(batch, seq) + 6.0 * D * D * batch * HQ * seq
    achieved = flops / (attn_ms * 1e-3) / 1e12 if attn_ms > 0 else None
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s",
                "frac": (achieved / peaks["tflops"]) if achieved else None,
                # DRAM bytes per launch: ncu capture at batch 1 (74.0 MB read + 29.3 MB written; queries in,
                # outputs out, packed keys and values), which scales with batch
                "traffic": 103.3e6 * batch if (seq == S and D == 128) else None,
                "kernel": "attention_c2_kernel", "ms_per_launch": attn_ms, "peak_source": peaks["source"],
                "kernel_ms": {"compress_keys": ms_sum[0] / max(launches[0], 1),
                              "compress_values": ms_sum[1] / max(launches[1], 1),
                              "prepare_queries": ms_sum[2] / max(launches[2], 1),
                              "attention": attn_ms, "back_rotation": ms_sum[4] / max(launches[4], 1)}}

    cpu = None
    if not args.no_cpu_baseline and world == 1:
        cpu_sample(bits, 1024)
        sec, threads = cpu_sample(bits, seq, repeats=2)
        units = batch * HQ
        cpu = {"value": batch * HKV * seq / (sec * units), "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"one (batch, query head) unit of {units}: compress of S={seq} keys and values, "
                         f"score/softmax/PV rows for {min(CPU_Q_ROWS, seq)} of {seq} queries at full width, scaled to "
                         f"the unit ({sec:.2f} s) and then linearly to the workload; reference PyTorch path"}

    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "op_level_gqa4_s8192", "batch_per_gpu": batch, "q_heads": HQ, "kv_heads": HKV,
                       "seq_len": seq, "head_dim": D, "bits": bits, "causal": True,
                       "l2": "inputs (402 MB per step) exceed the 126 MB L2; no flush",
                       "causal_pairs_per_s": causal_pairs(batch, seq) * world / (ms_per_step * 1e-3)},
            "clocks": clocks, "e2e": e2e, "gpu_launches": (int(sum(launches)) + 3 * args.steps) * world,  # + the three constant-operand builders per step
            "roofline": roofline, "cpu_baseline": cpu, "device_wait_faults": faults}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
