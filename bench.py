#!/usr/bin/env python
"""Benchmark of the paged-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): the Qwen3-8B-shaped paged decode configuration — 32 q heads, 8 kv heads,
head_dim 128, bf16, block_size 16, batch 256, context lengths lognormal (median 1024,
sigma 0.8) clipped to [32, 8192], N(0,1) values, block tables cut from a seeded random
permutation of the pool (~1.5 GB of K/V, far larger than the 126 MB L2, so no flush is
needed between iterations).  One step = what the production caller does per layer
(nanoPD/engine/model_runner.py:188-207): store the new token of every sequence, then attend
with seq_len = position + 1.

Metric: decode-attention HBM GB/s = ALGORITHMIC bytes of the step / step time, where the
bytes count every K/V element once per kv head and real token, plus Q, O, the used table
entries, lengths, and the store's rows (read + written).

With N > 1 (torchrun, one rank per GPU) every rank is an independent decode replica with its
own pool and batch (weak scaling, no data-path collective); value = bytes of all ranks /
max-over-ranks time.

`--impl reference` times the reference's CPU path (the same paged math in PyTorch on the host
cores, through the oracle port) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

from nanopd_b200 import replicas, workloads  # noqa: E402

METRIC = "decode_attn_hbm_gbs"
UNIT = "GB/s"
WORKLOAD = "cfg2: paged decode attention, Qwen3-8B shape (32q/8kv heads, D128, bf16, block 16), batch 256, ctx lognormal(1024, 0.8) in [32, 8192]"


def algorithmic_bytes(ctx_lens, Hq, Hkv, D, B, e=2):
    """Bytes one step must move: attention over len = ctx + 1 tokens plus the one-token store."""
    lens = [int(c) + 1 for c in ctx_lens]
    S = len(lens)
    attn = sum(lens) * 2 * Hkv * D * e + 2 * S * Hq * D * e + sum((l + B - 1) // B for l in lens) * 4 + S * 4
    store = S * Hkv * D * e * 2 * 2 + S * 8
    return attn, store


def measured_peak_gbs():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json, copy bandwidth)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons; keeps the samples taken inside the timed window.

    nvidia-smi needs a few hundred milliseconds to start, so the sampler is started well before
    the timed region and the samples are filtered by their own timestamps afterwards."""
    FIELDS = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.t_begin = self.t_end = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu_index), "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def mark_begin(self):
        self.t_begin = time.time()

    def mark_end(self):
        self.t_end = time.time()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        import datetime
        rows = []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 10:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(parts[2]), float(parts[3]), float(parts[4]),
                             [n for n, v in zip(names, parts[6:10]) if v.lower().startswith("active")]))
            except ValueError:
                continue
        inside = [r for r in rows if self.t_begin is not None and self.t_begin - 0.05 <= r[0] <= self.t_end + 0.05]
        use = inside if inside else rows
        reasons = sorted({n for r in use for n in r[4]})
        return {"sm_mhz": statistics.median(r[1] for r in use) if use else None,
                "sm_max_mhz": max(r[2] for r in use) if use else None,
                "power_w_max": max(r[3] for r in use) if use else None,
                "samples": len(use), "samples_in_timed_window": len(inside), "reasons": reasons}


# ---------------------------------------------------------------------------
# CPU baseline: the reference's paged math in PyTorch on the host cores (oracle port)
# ---------------------------------------------------------------------------
def cpu_reference_sample(batch_cpu, target_seconds=12.0):
    """Chooses a prefix of the batch that takes about target_seconds on this host."""
    from oracle import paged_oracle
    torch.set_num_threads(os.cpu_count() or 1)
    probe = min(8, batch_cpu.query.size(0))
    lens = batch_cpu.seq_lens_after_store
    t0 = time.perf_counter()
    paged_oracle.paged_decode_attention(batch_cpu.query[:probe], batch_cpu.k_cache, batch_cpu.v_cache,
                                        batch_cpu.block_tables[:probe], lens[:probe], batch_cpu.scale)
    dt = time.perf_counter() - t0
    per_token = dt / max(1, int(lens[:probe].sum()))
    budget_tokens = target_seconds / per_token
    csum = torch.cumsum(lens.to(torch.int64), 0)
    n = int((csum <= budget_tokens).sum().item())
    return max(probe, min(n, batch_cpu.query.size(0)))


def cpu_reference_time(batch_cpu, n_seqs, steps, warmup):
    from oracle import paged_oracle
    torch.set_num_threads(os.cpu_count() or 1)
    lens = batch_cpu.seq_lens_after_store[:n_seqs]

    def one():
        kc, vc = batch_cpu.k_cache, batch_cpu.v_cache
        paged_oracle.kv_store(kc, vc, batch_cpu.k_new[:, :n_seqs], batch_cpu.v_new[:, :n_seqs],
                              batch_cpu.block_tables[:n_seqs], batch_cpu.positions[:n_seqs])
        return paged_oracle.paged_decode_attention(batch_cpu.query[:n_seqs], kc, vc,
                                                   batch_cpu.block_tables[:n_seqs], lens, batch_cpu.scale)
    for _ in range(warmup):
        one()
    t0 = time.perf_counter()
    for _ in range(steps):
        one()
    dt = (time.perf_counter() - t0) / steps
    a, s = algorithmic_bytes(batch_cpu.ctx_lens[:n_seqs].tolist(), batch_cpu.num_q_heads, batch_cpu.num_kv_heads,
                             batch_cpu.head_dim, batch_cpu.block_size)
    return (a + s) / dt / 1e9, dt


def config_block(ctx, S, Hq, Hkv, D, world):
    """The ``config`` object of the bench line; both arms print the same keys."""
    return {"workload": WORKLOAD, "batch_per_gpu": S, "tokens_per_gpu": int(sum(ctx)) + S,
            "kv_bytes_per_gpu": int(sum(c + 1 for c in ctx)) * 2 * Hkv * D * 2,
            "l2": "inputs (1.5 GB per GPU) exceed the 126 MB L2; no flush between iterations",
            "parallelism": f"{world} independent decode replicas (batch-sharded, no collective)"}


def run_reference_arm(args):
    """The reference's CPU path (the oracle port of its paged math in PyTorch) on the box's host cores, all
    threads, on the same workload, metric and unit; rank 0 only.  Exactly ``--steps`` timed and ``--warmup``
    untimed passes; a pass covers the whole batch when ``steps + warmup`` such passes end within about three
    minutes, otherwise a prefix of it, which the line states."""
    rank, _, world = replicas.env_world()
    if rank != 0:
        return 0
    batch = workloads.make_config2(device="cpu", seed=args.seed, batch=args.batch)
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    n = cpu_reference_sample(batch, target_seconds=150.0 / (steps + warmup))
    gbs, dt = cpu_reference_time(batch, n, steps, warmup)
    cores = os.cpu_count() or 1
    whole = n == batch.query.size(0)
    sample = (f"{'all' if whole else 'first'} {n} of {args.batch} sequences "
              f"({int(batch.seq_lens_after_store[:n].sum())} tokens) per step")
    ctx = batch.ctx_lens.tolist()
    cfg = config_block(ctx, len(ctx), batch.num_q_heads, batch.num_kv_heads, batch.head_dim, args.gpus)
    cfg["sample"] = sample
    line = {
        "impl": "reference", "metric": METRIC, "value": round(gbs, 4), "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": cfg,
        "cpu_baseline": {"value": round(gbs, 4), "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": round(gbs, 4), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "cpu_arm": "one process on rank 0 using all host cores, whatever --gpus says: the value does not grow with N",
    }
    print(json.dumps(line), flush=True)
    return 0



# ---------------------------------------------------------------------------
# Secondary workload: configuration 3, chunked prefill over paged K/V (tensor-core bound)
# ---------------------------------------------------------------------------
def measured_peak_tflops():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["bf16_tflops"]), "measured (MEASURED_PEAKS.json, cuBLAS bf16 burst)"
        except Exception:
            pass
    return 1590.0, "fallback (1.59 PFLOP/s, earlier measurement on this pool)"


def prefill_flops(chunks, Hq, D):
    return sum(4 * Hq * D * (c.num_tokens * c.start_position + c.num_tokens * (c.num_tokens + 1) // 2) for c in chunks)


def build_prefill_call(mixed, chunks, dev):
    """Packs the given chunks for one paged_prefill_attention call."""
    max_blk = max(c.block_table.numel() for c in chunks)
    bt = torch.zeros(len(chunks), max_blk, dtype=torch.int32, device=dev)
    for i, c in enumerate(chunks):
        bt[i, :c.block_table.numel()] = c.block_table
    q = torch.cat([c.query for c in chunks]).contiguous()
    offsets, tokens, starts, off = [], [], [], 0
    for c in chunks:
        offsets.append(off), tokens.append(c.num_tokens), starts.append(c.start_position)
        off += c.num_tokens
    return q, bt, offsets, tokens, starts


def run_prefill_workload(args, paged_kernels, dev, timed):
    """All 512-token chunks of configuration 3's four prompts in one call (a whole chunked prefill
    of the prompts for one layer), and one mixed step: one chunk per prompt + the 128 decode sequences."""
    m = workloads.make_config3(device=dev, seed=args.seed)
    d = m.decode
    Hq, D, B = d.num_q_heads, d.head_dim, d.block_size
    for c in m.chunks:      # the chunks' K/V rows go into the pages first, as the caller does
        n = c.num_tokens
        pos = torch.arange(c.start_position, c.start_position + n, dtype=torch.int32, device=dev)
        paged_kernels.paged_kv_store(d.k_cache, d.v_cache, c.k_new, c.v_new, c.block_table.unsqueeze(0).expand(n, -1), pos)
    q, bt, offs, toks, starts = build_prefill_call(m, m.chunks, dev)
    out = torch.empty_like(q)
    fn_all = lambda: paged_kernels.paged_prefill_attention(out, q, d.k_cache, d.v_cache, bt, offs, toks, starts,
                                                           d.scale, B, bt.size(1))
    for _ in range(3):
        fn_all()
    steps = max(3, min(args.steps, 20))
    if args.profile:
        for _ in range(2):
            fn_all()
        torch.cuda.synchronize()
        return {"profile_run": True, "flops_per_launch": prefill_flops(m.chunks, Hq, D)}
    ms_all = timed(fn_all, steps)
    flops_all = prefill_flops(m.chunks, Hq, D)
    # mixed step: the last chunk of every prompt + decode batch
    last = [c for i, c in enumerate(m.chunks) if i + 1 == len(m.chunks) or m.chunks[i + 1].start_position == 0]
    q2, bt2, offs2, toks2, starts2 = build_prefill_call(m, last, dev)
    out2 = torch.empty_like(q2)
    dec_out = torch.empty_like(d.query)
    seq_lens = d.seq_lens_after_store.contiguous()

    def mixed_step():
        paged_kernels.paged_prefill_attention(out2, q2, d.k_cache, d.v_cache, bt2, offs2, toks2, starts2, d.scale, B, bt2.size(1))
        paged_kernels.paged_kv_store(d.k_cache, d.v_cache, d.k_new, d.v_new, d.block_tables, d.positions)
        paged_kernels.paged_attention_forward(dec_out, d.query, d.k_cache, d.v_cache, d.block_tables, seq_lens,
                                              d.scale, B, d.max_blocks)
    for _ in range(3):
        mixed_step()
    ms_mixed = timed(mixed_step, steps)
    # the same mixed step with the two attention kernels side by side on two streams, each on its share of the SMs
    from nanopd_b200 import paged_forward
    P2, Dn2 = q2.size(0), d.query.size(0)
    sc = paged_forward.StepContext(
        num_prefill_tokens=P2, num_decode_tokens=Dn2, block_size=B, prefill_tables=bt2, prefill_offsets=offs2,
        prefill_tokens=toks2, prefill_starts=starts2, decode_tables=d.block_tables, decode_positions=d.positions,
        decode_seq_lens=seq_lens,
        prefill_score_pairs=sum(n * s0 + n * (n + 1) // 2 for n, s0 in zip(toks2, starts2)),
        decode_context_tokens=int(seq_lens.sum().item()))
    q_all = torch.cat([q2, d.query]).contiguous()
    out_all = torch.empty_like(q_all)
    sm_share = paged_forward._sm_split(sc, Hq, d.num_kv_heads, D, 2, torch.cuda.get_device_properties(dev).multi_processor_count)

    def mixed_step_overlapped():
        paged_kernels.paged_kv_store(d.k_cache, d.v_cache, d.k_new, d.v_new, d.block_tables, d.positions)
        paged_forward._attend(sc, out_all, q_all, d.k_cache, d.v_cache, d.scale, True)
    for _ in range(3):
        mixed_step_overlapped()
    ms_mixed_overlapped = timed(mixed_step_overlapped, steps)
    ms_last = timed(lambda: paged_kernels.paged_prefill_attention(out2, q2, d.k_cache, d.v_cache, bt2, offs2, toks2,
                                                                  starts2, d.scale, B, bt2.size(1)), steps)
    peak, src = measured_peak_tflops()
    tf = flops_all / (ms_all * 1e-3) / 1e12
    return {"prompt_lens": m.prompt_lens, "chunks": len(m.chunks), "flops_all_chunks": flops_all,
            "all_chunks_ms": round(ms_all, 4), "tflops": round(tf, 1), "peak_tflops": peak, "peak_source": src,
            "frac_of_peak": round(tf / peak, 4),
            "last_chunks_ms": round(ms_last, 4),
            "last_chunks_tflops": round(prefill_flops(last, Hq, D) / (ms_last * 1e-3) / 1e12, 1),
            "mixed_step_ms": round(ms_mixed, 4),
            "mixed_step_two_streams_ms": round(ms_mixed_overlapped, 4), "prefill_sm_share": sm_share,
            "mixed_step": "last 512-token chunk of each of 4 prompts + store + decode attention of 128 sequences"}


def graph_device_time_us(fns, dev, replays=5):
    """Device time per call of the calls in ``fns``, recorded once each in ONE CUDA graph and replayed: the
    Python call overhead of microsecond-sized launches is not part of the number."""
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        for fn in fns[:3]:
            fn()
    side.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        for fn in fns:
            fn()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (replays * len(fns)) * 1e3


def run_shim_host_cost(paged_kernels, dev, calls=3000):
    """Host time per call of the two reference ops at the reference's operating size (16 running sequences,
    nanoPD/engine/engine.py:21): wall time of issuing ``calls`` eager calls, the GPU kept far from being the
    bottleneck by the small batch, so the figure is the Python shim + ctypes + launch."""
    b = workloads.make_decode_batch([200] * 16, 32, 8, 128, 16, torch.bfloat16, device=dev, seed=1)
    out = torch.zeros_like(b.query)
    lens = b.seq_lens_after_store.contiguous()
    res = {}
    for name, fn in (("paged_kv_store", lambda: paged_kernels.paged_kv_store(b.k_cache, b.v_cache, b.k_new, b.v_new,
                                                                             b.block_tables, b.positions)),
                     ("paged_attention_forward", lambda: paged_kernels.paged_attention_forward(
                         out, b.query, b.k_cache, b.v_cache, b.block_tables, lens, b.scale, 16, b.max_blocks))):
        for _ in range(50):
            fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(calls):
            fn()
        host = time.perf_counter() - t0
        torch.cuda.synchronize()
        total = time.perf_counter() - t0
        res[name] = {"host_us_per_call": round(host / calls * 1e6, 2), "us_per_call_until_gpu_idle": round(total / calls * 1e6, 2)}
    res["batch"] = "16 sequences of 200 tokens, Qwen3-8B shape"
    return res


def run_store_kernel_timing(paged_kernels, b, positions, dev):
    """Device time of the KV store kernel: the decode step's 256 tokens, and an 8192-token prompt.  Sources rotate
    over buffers larger than L2 inside one CUDA graph; GB/s counts the rows read and written plus 8 bytes of
    table/position per token."""
    Hkv, D, B = b.num_kv_heads, b.head_dim, b.block_size
    peak = measured_peak_gbs()[0]
    out = {}
    for label, T, nbuf in (("decode_256_tokens", b.query.size(0), 160), ("prompt_8192_tokens", 8192, 6)):
        srcs = [(torch.randn(Hkv, T, D, device=dev).to(b.k_cache.dtype), torch.randn(Hkv, T, D, device=dev).to(b.k_cache.dtype))
                for _ in range(nbuf)]
        if T == b.query.size(0):
            bt, pos = b.block_tables, positions
        else:
            per = T // b.query.size(0)
            bt = b.block_tables.repeat_interleave(per, dim=0)
            pos = (torch.clamp(positions - per, min=0).repeat_interleave(per) +
                   torch.arange(per, device=dev, dtype=torch.int32).repeat(b.query.size(0)))
        fns = [(lambda k=k, v=v: paged_kernels.paged_kv_store(b.k_cache, b.v_cache, k, v, bt, pos)) for k, v in srcs]
        us = graph_device_time_us(fns, dev)
        nbytes = T * Hkv * D * 2 * 2 * 2 + 8 * T
        out[label] = {"us": round(us, 2), "algorithmic_bytes": nbytes, "gbs": round(nbytes / us / 1e3, 1),
                      "frac_of_hbm_peak": round(nbytes / us / 1e3 / peak, 3),
                      "source_buffers_rotated": nbuf, "rotated_source_bytes": nbuf * T * Hkv * D * 2 * 2}
        del srcs
    out["timing"] = "one CUDA graph with one launch per source buffer, 5 replays, CUDA events"
    return out


def run_config1(paged_kernels, dev, seed, copies=64, cpu_reps=20):
    """Configuration 1 (Qwen2-1.5B shape, 8 sequences, fp16, 256-block pool): one step = store the new token of
    every sequence + decode attention.  GPU: device time per step from one CUDA graph that walks 64 independently
    drawn copies of the configuration (170 MB of pools, more than the L2).  CPU: the oracle port of the
    reference's PyTorch path on all host cores, the whole configuration, median of 20 repetitions."""
    from oracle import paged_oracle
    b0 = workloads.make_config1(device="cpu", seed=seed)
    on_dev = workloads.DecodeBatch(**{f: (getattr(b0, f).to(dev) if torch.is_tensor(getattr(b0, f)) else getattr(b0, f))
                                      for f in b0.__dataclass_fields__})
    batches = [on_dev] + [workloads.make_config1(device=dev, seed=seed + i) for i in range(1, copies)]
    outs = [torch.zeros_like(bb.query) for bb in batches]
    lens = [bb.seq_lens_after_store.contiguous() for bb in batches]

    def one(i):
        bb = batches[i]
        paged_kernels.paged_kv_store(bb.k_cache, bb.v_cache, bb.k_new, bb.v_new, bb.block_tables, bb.positions)
        paged_kernels.paged_attention_forward(outs[i], bb.query, bb.k_cache, bb.v_cache, bb.block_tables, lens[i],
                                              bb.scale, bb.block_size, bb.max_blocks)
    us = graph_device_time_us([(lambda i=i: one(i)) for i in range(copies)], dev)
    a, st = algorithmic_bytes(b0.ctx_lens.tolist(), b0.num_q_heads, b0.num_kv_heads, b0.head_dim, b0.block_size)
    torch.set_num_threads(os.cpu_count() or 1)
    times = []
    for _ in range(cpu_reps + 2):
        t0 = time.perf_counter()
        paged_oracle.kv_store(b0.k_cache, b0.v_cache, b0.k_new, b0.v_new, b0.block_tables, b0.positions)
        want = paged_oracle.paged_decode_attention(b0.query, b0.k_cache, b0.v_cache, b0.block_tables,
                                                   b0.seq_lens_after_store, b0.scale)
        times.append(time.perf_counter() - t0)
    cpu_s = statistics.median(times[2:])
    err = (outs[0].float().cpu() - want).abs().max().item()      # copy 0 is the seed the CPU ran
    return {"workload": "cfg1: Qwen2-1.5B shape (12q/2kv heads, D128, fp16, block 16), 8 sequences, ctx U[16,512], 256-block pool",
            "tokens": int(b0.seq_lens_after_store.sum()), "algorithmic_bytes_per_step": a + st,
            "gpu_us_per_step": round(us, 2), "gpu_gbs": round((a + st) / us / 1e3, 1),
            "gpu_timing": f"one CUDA graph over {copies} copies of the configuration ({copies * 2 * 256 * 2 * 16 * 128 * 2 >> 20} MiB of pools), 5 replays",
            "cpu_ms_per_step_median": round(cpu_s * 1e3, 3), "cpu_repetitions": cpu_reps, "cpu_cores": os.cpu_count() or 1,
            "cpu_gbs": round((a + st) / cpu_s / 1e9, 3), "cpu_kind": "port (oracle restatement of the reference's PyTorch path)",
            "max_abs_error_vs_oracle": round(err, 6)}

def run_reference_grid(args, paged_kernels, dev):
    """The shape grid of the reference's own micro-benchmark (nanoPD/paged_attention/tests/
    benchmark_paged_attention_optim.py:110-137: small uniform-length batches, and whole-prompt stores), as device
    time per launch: 20 launches captured in one CUDA graph, so the Python call overhead of these microsecond-sized
    problems is not part of the number.  The reference prints such a table at run time and publishes none."""
    attn_cfgs = [(1, 32, 32, 128, 128, 16, torch.float16), (1, 32, 32, 128, 512, 16, torch.float16),
                 (1, 32, 32, 128, 1024, 16, torch.float16), (8, 32, 32, 128, 256, 16, torch.float16),
                 (16, 32, 32, 128, 256, 16, torch.float16), (32, 32, 32, 128, 256, 16, torch.float16),
                 (1, 32, 8, 128, 512, 16, torch.float16), (8, 32, 8, 128, 512, 16, torch.float16),
                 (16, 32, 8, 128, 512, 16, torch.float16), (8, 32, 32, 128, 256, 16, torch.bfloat16)]
    store_cfgs = [(8, 128, 128, 16, torch.float16), (8, 512, 128, 16, torch.float16), (8, 1024, 128, 16, torch.float16),
                  (8, 2048, 128, 16, torch.float16), (8, 512, 128, 32, torch.float16), (32, 512, 128, 16, torch.float16),
                  (8, 512, 128, 16, torch.bfloat16)]
    inner = 20

    def graph_time(fn):
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(3):
                fn()
        side.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for _ in range(inner):
                fn()
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (5 * inner) * 1e3          # microseconds per launch

    rows_a, rows_s = [], []
    for (S, Hq, Hkv, D, L, B, dt) in attn_cfgs:
        b = workloads.make_decode_batch([L] * S, Hq, Hkv, D, B, dt, device=dev, seed=args.seed)
        out = torch.zeros_like(b.query)
        us = graph_time(lambda: paged_kernels.paged_attention_forward(out, b.query, b.k_cache, b.v_cache, b.block_tables,
                                                                      b.ctx_lens, b.scale, B, b.max_blocks))
        by, _ = algorithmic_bytes([L] * S, Hq, Hkv, D, B)
        rows_a.append({"num_seqs": S, "heads": Hq, "kv_heads": Hkv, "head_size": D, "seq_len": L, "block": B,
                       "dtype": str(dt).replace("torch.", ""), "us": round(us, 2), "gbs": round(by / us / 1e3, 1),
                       "tflops_reference_formula": round(S * Hq * 4 * L * D / us / 1e6, 3)})
    for (Hkv, T, D, B, dt) in store_cfgs:
        nblk = (T + B - 1) // B
        kc = torch.zeros(nblk, Hkv, B, D, dtype=dt, device=dev)
        vc = torch.zeros_like(kc)
        k_src = torch.randn(Hkv, T, D, device=dev).to(dt)
        v_src = torch.randn(Hkv, T, D, device=dev).to(dt)
        table = torch.arange(nblk, dtype=torch.int32, device=dev).unsqueeze(0).expand(T, -1)
        pos = torch.arange(T, dtype=torch.int32, device=dev)
        us = graph_time(lambda: paged_kernels.paged_kv_store(kc, vc, k_src, v_src, table, pos))
        written = 2 * T * Hkv * D * 2
        rows_s.append({"kv_heads": Hkv, "seq_len": T, "head_dim": D, "block": B, "dtype": str(dt).replace("torch.", ""),
                       "us": round(us, 2), "gbs_written_reference_formula": round(written / us / 1e3, 1)})
    return {"attention": rows_a, "kv_store": rows_s, "timing": f"{inner} launches per CUDA graph, 5 replays, CUDA events",
            "device_status": paged_kernels.check_status(dev, raise_on_error=False)}


def run_model_tables(args, dev, timed):
    """The reference's model-level timing tables (nanoPD/cost_model/record_no_kvstorekernel_naive_pagedattention.txt:
    T_decode(kv_len, batch), T_prefill(L), extra decode latency from a co-scheduled prompt chunk; measured there
    on an RTX 4090 with real Qwen3-8B weights) on the random-init stack of the same shape around this library."""
    import numpy as np
    from nanopd_b200 import decoder_step
    free, _ = torch.cuda.mem_get_info(dev)
    if free < 60 * (1 << 30):
        return {"skipped": f"only {free >> 30} GiB free on the device"}
    shape = decoder_step.DecoderShape()
    B, pool_blocks = 16, 6144
    model = decoder_step.SyntheticDecoder(dev, shape, torch.bfloat16, seed=args.seed, max_position=16384 + 64)
    k_cache = torch.empty(shape.num_layers, pool_blocks, shape.num_kv_heads, B, shape.head_dim, dtype=torch.bfloat16, device=dev)
    v_cache = torch.empty_like(k_cache)
    for li in range(shape.num_layers):
        k_cache[li].normal_()
        v_cache[li].normal_()
    rng = np.random.default_rng(args.seed)

    def tables_for(batch, kv_len, headroom=16):
        nblk = (kv_len + headroom + B - 1) // B
        perm = rng.permutation(pool_blocks)[:batch * nblk].astype(np.int32).reshape(batch, nblk)
        return perm

    t_decode = {}
    for batch in (1, 4, 8, 16, 32):
        for kv in (128, 512, 1024, 2048):
            tb = torch.from_numpy(tables_for(batch, kv)).to(dev)
            ctx = torch.full((batch,), kv, dtype=torch.int32, device=dev)
            model.attach_batch(k_cache, v_cache, tb, ctx, torch.randint(0, shape.vocab, (batch,), device=dev))
            model.capture()
            model.replay()
            t_decode[f"B{batch}_kv{kv}"] = round(timed(model.replay, 5), 3)
    t_prefill = {}
    for L in (64, 128, 256, 512, 1024, 2048, 8192, 16384):
        table = tables_for(1, L, 0)[0].tolist()
        ctx = {"num_prefill_tokens": L, "num_decode_tokens": 0, "decodes": [],
               "prefills": [{"block_table": table, "start_position": 0, "num_tokens": L}]}
        toks = torch.randint(0, shape.vocab, (L,), device=dev)
        fn = lambda: model.mixed_step(ctx, toks, k_cache, v_cache)
        fn()
        t_prefill[f"L{L}"] = round(timed(fn, 3 if L <= 2048 else 2), 3)
    interference = {}
    for batch in (4, 16):
        kv = 1024
        tb = tables_for(batch, kv)
        decodes = [{"block_table": tb[i].tolist(), "position": kv} for i in range(batch)]
        d_ctx = {"num_prefill_tokens": 0, "num_decode_tokens": batch, "prefills": [], "decodes": decodes}
        d_toks = torch.randint(0, shape.vocab, (batch,), device=dev)
        fn_d = lambda: model.mixed_step(d_ctx, d_toks, k_cache, v_cache)
        fn_d()
        base = timed(fn_d, 3)
        for chunk in (64, 128, 256, 512):
            table = tables_for(1, chunk, 0)[0].tolist()
            m_ctx = {"num_prefill_tokens": chunk, "num_decode_tokens": batch, "decodes": decodes,
                     "prefills": [{"block_table": table, "start_position": 0, "num_tokens": chunk}]}
            m_toks = torch.randint(0, shape.vocab, (chunk + batch,), device=dev)
            fn_m = lambda: model.mixed_step(m_ctx, m_toks, k_cache, v_cache)
            fn_m()
            interference[f"B{batch}_chunk{chunk}"] = round(timed(fn_m, 3) - base, 3)
        interference[f"B{batch}_decode_only_eager_ms"] = round(base, 3)
    import paged_kernels
    status = paged_kernels.check_status(dev, raise_on_error=False)
    del model, k_cache, v_cache
    torch.cuda.empty_cache()
    return {"model": "Qwen3-8B shape, random init, bf16", "unit": "ms per step",
            "t_decode_graph": t_decode, "t_prefill_eager": t_prefill, "extra_decode_ms_from_prompt_chunk": interference,
            "reference_rtx4090_fp16_ms": {
                "source": "nanoPD/cost_model/record_no_kvstorekernel_naive_pagedattention.txt:5-88 (other hardware, real weights)",
                "t_decode": {"B1_kv128": 49.0, "B1_kv2048": 64.3, "B8_kv1024": 83.9, "B32_kv128": 192.2, "B32_kv2048": 226.7},
                "t_prefill": {"L64": 218, "L128": 394, "L256": 742, "L512": 1442, "L1024": 2847, "L2048": 5641},
                "extra_decode_ms_from_prompt_chunk": {"chunk64": 179, "chunk128": 352, "chunk256": 702, "chunk512": 1400}},
            "device_status": status}


def run_model_workload(args, dev, timed, batch, seed):
    """Decode tokens/s at model level: a random-init stack of Qwen3-8B shape (36 layers) around the paged kernels,
    configuration 2's batch (256 sequences, lognormal contexts) in a 36-layer pool, every step one token per
    sequence; the whole step replayed as one CUDA graph.  Returns per-GPU numbers; the caller aggregates."""
    import numpy as np
    from nanopd_b200 import decoder_step
    free, _ = torch.cuda.mem_get_info(dev)
    if free < 95 * (1 << 30):
        return {"skipped": f"only {free >> 30} GiB free on the device"}
    shape = decoder_step.DecoderShape()
    B, headroom = 16, 24
    ctx = workloads.config2_lens(batch=batch, seed=seed)
    nblk = (np.asarray(ctx, dtype=np.int64) + headroom + B - 1) // B
    pool_blocks = int(nblk.sum())
    rng = np.random.default_rng(seed)
    perm = rng.permutation(pool_blocks)
    tables = np.zeros((len(ctx), int(nblk.max())), dtype=np.int32)
    o = 0
    for i, n in enumerate(nblk.tolist()):
        tables[i, :n] = perm[o:o + n]
        o += n
    model = decoder_step.SyntheticDecoder(dev, shape, torch.bfloat16, seed=seed, max_position=8192 + 64)
    k_cache = torch.empty(shape.num_layers, pool_blocks, shape.num_kv_heads, B, shape.head_dim, dtype=torch.bfloat16, device=dev)
    v_cache = torch.empty_like(k_cache)
    for li in range(shape.num_layers):       # layer by layer: bounded temporaries
        k_cache[li].normal_()
        v_cache[li].normal_()
    ctx_t = torch.from_numpy(np.asarray(ctx, dtype=np.int32)).to(dev)
    tokens = torch.randint(0, shape.vocab, (len(ctx),), device=dev)
    model.attach_batch(k_cache, v_cache, torch.from_numpy(tables).to(dev), ctx_t, tokens)
    n_eager, n_graph = 2, 8
    model.step()                                                  # warm-up (cuBLAS handles, workspaces)
    ms_eager = timed(model.step, n_eager)
    model.capture()
    model.replay()
    ms_graph = timed(model.replay, n_graph)
    status = 0
    import paged_kernels
    status = paged_kernels.check_status(dev, raise_on_error=False)
    S = len(ctx)
    kv_bytes_step = int(sum(int(c) for c in ctx)) * 2 * shape.num_kv_heads * shape.head_dim * 2 * shape.num_layers
    res = {"model": "Qwen3-8B shape, random init (36 layers, hidden 4096, FFN 12288, 32q/8kv x 128, vocab 151936), bf16",
           "batch": S, "context_tokens": int(sum(int(c) for c in ctx)),
           "params": shape.param_count, "kv_pool_gb": round(2 * k_cache.numel() * 2 / 1e9, 1),
           "graph_ms_per_step": round(ms_graph, 3), "eager_ms_per_step": round(ms_eager, 3),
           "tok_s": round(S / (ms_graph * 1e-3), 1), "tok_s_eager": round(S / (ms_eager * 1e-3), 1),
           "kv_bytes_per_step": kv_bytes_step, "weight_bytes_per_step": 2 * (shape.param_count - shape.vocab * shape.hidden),
           "library_launches_per_step": model.launches_per_step(),
           "sampling": "top_k_sample, top_k = 1, one launch per step, tokens stay on the device", "device_status": status,
           "steps_timed": n_graph, "tokens_advance_in_place": True}
    del model, k_cache, v_cache
    torch.cuda.empty_cache()
    return res



# ---------------------------------------------------------------------------
# NVLink parity, visible in the bench line: every migrated block, and the whole hand-off against the oracle
# ---------------------------------------------------------------------------
def nvlink_parity(src_dev: int, dst_dev: int, seed: int = 0):
    """(i) 1024 block-scattered blocks x 36 layers pulled from ``src_dev`` to OTHER ids on ``dst_dev``: every
    migrated block is compared with its source, and every block that was not a destination must be untouched.
    (ii) The hand-off end to end: a prompt's K/V stored into the source pool (store kernel), its pages moved to
    other ids of the destination pool (migration kernel), one more token stored there and decode attention over
    the moved pages compared with the CPU oracle evaluated on the prompt laid out contiguously."""
    import paged_kernels
    from nanopd_b200 import kv_transfer
    from oracle import paged_oracle
    res = {"from_gpu": src_dev, "to_gpu": dst_dev}
    g = torch.Generator().manual_seed(seed)
    sd, dd = f"cuda:{src_dev}", f"cuda:{dst_dev}"
    L, nb, Hkv, B, D = 36, 1024, 8, 16, 128
    src_k = torch.empty(L, nb, Hkv, B, D, dtype=torch.bfloat16, device=sd).normal_()
    src_v = torch.empty_like(src_k).normal_()
    dst_nb = nb + 64
    dst_k = torch.zeros(L, dst_nb, Hkv, B, D, dtype=torch.bfloat16, device=dd)
    dst_v = torch.zeros_like(dst_k)
    src_ids = torch.randperm(nb, generator=g)[:960]
    dst_ids = torch.randperm(dst_nb, generator=g)[:960]
    torch.cuda.synchronize(src_dev)
    kv_transfer.transfer_kv(src_k, src_v, dst_k, dst_v, src_ids.tolist(), dst_block_table=dst_ids.tolist())
    torch.cuda.synchronize(dst_dev)
    ok = True
    for sc, dc in ((src_k, dst_k), (src_v, dst_v)):
        for lo in range(0, 960, 240):                       # in slabs, through the copy engine: an independent path
            want = sc[:, src_ids[lo:lo + 240].to(sd)].to(dd)
            ok = ok and torch.equal(dc[:, dst_ids[lo:lo + 240].to(dd)], want)
        rest = torch.ones(dst_nb, dtype=torch.bool)
        rest[dst_ids] = False
        ok = ok and int(torch.count_nonzero(dc[:, rest.to(dd)])) == 0
    res["blocks_compared"] = 960 * L * 2
    res["every_migrated_block_equal"] = bool(ok)
    del src_k, src_v, dst_k, dst_v
    # (ii) store -> migrate to other ids -> store one more token -> decode attention, against the oracle
    L2, Hq, n_prompt = 2, 32, 2003
    nblk = (n_prompt + 1 + B - 1) // B
    k_prompt = torch.randn(L2, Hkv, n_prompt, D, generator=g).to(torch.bfloat16)
    v_prompt = torch.randn(L2, Hkv, n_prompt, D, generator=g).to(torch.bfloat16)
    pk = torch.zeros(L2, 160, Hkv, B, D, dtype=torch.bfloat16, device=sd)
    pv = torch.zeros_like(pk)
    p_ids = torch.randperm(160, generator=g)[:nblk].tolist()
    with torch.cuda.device(src_dev):
        table = torch.tensor(p_ids, dtype=torch.int32, device=sd)
        for li in range(L2):
            paged_kernels.paged_kv_store(pk[li], pv[li], k_prompt[li].to(sd), v_prompt[li].to(sd), table, 0)
    torch.cuda.synchronize(src_dev)
    dk = torch.randn(L2, 256, Hkv, B, D, device=dd).to(torch.bfloat16)
    dv = torch.randn(L2, 256, Hkv, B, D, device=dd).to(torch.bfloat16)
    d_ids = torch.randperm(256, generator=g)[:nblk].tolist()
    kv_transfer.transfer_kv(pk, pv, dk, dv, p_ids, dst_block_table=d_ids)
    q = torch.randn(1, Hq, D, generator=g).to(torch.bfloat16)
    k_new = torch.randn(L2, Hkv, 1, D, generator=g).to(torch.bfloat16)
    v_new = torch.randn(L2, Hkv, 1, D, generator=g).to(torch.bfloat16)
    out = torch.zeros(L2, 1, Hq, D, dtype=torch.bfloat16, device=dd)
    with torch.cuda.device(dst_dev):
        t2 = torch.tensor([d_ids], dtype=torch.int32, device=dd)
        pos = torch.tensor([n_prompt], dtype=torch.int32, device=dd)
        for li in range(L2):
            paged_kernels.paged_kv_store(dk[li], dv[li], k_new[li].to(dd), v_new[li].to(dd), t2, pos)
            paged_kernels.paged_attention_forward(out[li], q.to(dd), dk[li], dv[li], t2, pos + 1, D ** -0.5, B, t2.size(1))
    torch.cuda.synchronize(dst_dev)
    worst = 0.0
    for li in range(L2):
        kc = torch.zeros(nblk, Hkv, B, D, dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        ids = torch.arange(nblk, dtype=torch.int32)
        paged_oracle.kv_store(kc, vc, torch.cat((k_prompt[li], k_new[li]), dim=1), torch.cat((v_prompt[li], v_new[li]), dim=1),
                              ids.unsqueeze(0).expand(n_prompt + 1, -1), torch.arange(n_prompt + 1, dtype=torch.int32))
        want = paged_oracle.paged_decode_attention(q, kc, vc, ids.unsqueeze(0), torch.tensor([n_prompt + 1], dtype=torch.int32),
                                                   D ** -0.5)
        worst = max(worst, (out[li].float().cpu() - want).abs().max().item())
    res["handoff_attention_max_abs_error_vs_oracle"] = round(worst, 6)
    res["tolerance"] = 1e-2
    status = 0
    for d in {src_dev, dst_dev}:
        status |= paged_kernels.check_status(f"cuda:{d}", raise_on_error=False)
    res["device_status"] = status
    res["pass"] = bool(ok and worst <= 1e-2 and status == 0)
    return res


def disagg_splits(n_gpus: int):
    """Prefill:decode splits measured on n GPUs (configuration 5 names 1:7, 2:6 and 4:4 on eight)."""
    if n_gpus >= 8:
        return [(1, 7), (2, 6), (4, 4)]
    if n_gpus >= 4:
        return [(1, 3), (2, 2)]
    if n_gpus >= 2:
        return [(1, 1)]
    return [(1, 1)]                     # one GPU plays both roles (a functional run: no link is crossed)


def run_disagg_workload(args, n_gpus: int, requests_per_prefill_gpu: int = 12):
    """Configuration 5: disaggregated prefill/decode of the random-init Qwen3-8B stack on the GPUs of one box, one
    process, one thread per GPU.  Prompts uniform in [2048, 16384] tokens, 128 output tokens each.  Returns the
    ``disagg`` block of the bench line."""
    from nanopd_b200 import serving
    n_gpus = max(1, min(n_gpus, torch.cuda.device_count()))
    out = {"workload": "cfg5: prompts U[2048,16384], 128 output tokens, Qwen3-8B shape random init bf16, "
                       "KV 147456 B/token, block 16", "gpus": n_gpus, "process_model": "one process, one thread per GPU"}
    ids = list(range(n_gpus))
    if n_gpus >= 2:
        out["nvlink_parity"] = nvlink_parity(1, 0, seed=args.seed)
        peak = serving.measure_peer_copy_peak(1, 0)
        out["peer_copy_peak"] = {k: (round(v, 2) if isinstance(v, float) else v) for k, v in peak.items()}
        out["link_sharing"] = serving.measure_link_sharing(ids)
        for key, val in out["link_sharing"].items():
            if isinstance(val, dict):
                val["aggregate_over_one_link_peak"] = round(val["aggregate_gbs"] / peak["gbs"], 3)
    models = serving.build_models(ids, seed=args.seed)
    shape = next(iter(models.values())).shape
    out["splits"] = {}
    for (np_, nd) in disagg_splits(n_gpus):
        pg = ids[:np_]
        dg = ids[np_:np_ + nd] if n_gpus >= 2 else ids[:1]
        entry = {}
        for layerwise in (False, True):
            name = "pull_layer_by_layer" if layerwise else "pull_after_prefill"
            # a verification pass (also the warm-up): every block is kept and compared on both sides afterwards
            reqs = serving.disagg_requests(6 * np_, shape.vocab, args.seed + 1)
            ver = serving.run_disagg_split(models, pg, dg, reqs, layerwise, verify=True)
            reqs = serving.disagg_requests(requests_per_prefill_gpu * np_, shape.vocab, args.seed)
            run = serving.run_disagg_split(models, pg, dg, reqs, layerwise)
            run["verification_pass"] = {"requests": ver["requests"], "pages_equal_on_both_sides": ver["pages_equal_on_both_sides"],
                                        "device_status": ver["device_status"]}
            if "peer_copy_peak" in out and "pull_gbs_per_request" in run:
                run["pull_median_over_link_peak"] = round(run["pull_gbs_per_request"]["median"] / out["peer_copy_peak"]["gbs"], 3)
            entry[name] = run
        out["splits"][f"{np_}:{nd}"] = entry
    del models
    for i in ids:
        with torch.cuda.device(i):
            torch.cuda.empty_cache()
    return out


def run_poisson_workload(args, dev, rates=(2, 4, 8, 16, 32), horizon_s: float = 6.0):
    """Configuration 4 on one GPU: continuous batching of the random-init Qwen3-8B stack under Poisson arrivals.
    Prompts lognormal(median 512, sigma 0.8 — the configuration names no sigma; configuration 2's is used) clipped
    to [16, 4096], outputs geometric(mean 256) capped at 1024.  Arrivals stop after ``horizon_s`` seconds; the run
    lasts until the last request has finished."""
    from nanopd_b200 import serving
    free, _ = torch.cuda.mem_get_info(dev)
    if free < 80 * (1 << 30):
        return {"skipped": f"only {free >> 30} GiB free on the device"}
    idx = torch.device(dev).index or 0
    model = serving.build_models([idx], seed=args.seed)[idx]
    out = {"workload": "cfg4: Poisson arrivals, prompts lognormal(512, 0.8) in [16,4096], outputs geometric(256) <= 1024, "
                       "Qwen3-8B shape random init bf16, collocated continuous batching on one GPU",
           "arrival_window_s": horizon_s, "slots": 256, "prefill_token_budget_per_step": 2048, "rates": {}}
    worker = None
    fig, worker = serving.run_poisson(model, 8.0, 1.0, args.seed + 99, worker=worker)      # warm-up (cuBLAS, workspaces)
    for lam in rates:
        fig, worker = serving.run_poisson(model, float(lam), horizon_s, args.seed, worker=worker)
        out["rates"][str(lam)] = fig
    model.detach_batch()
    del worker, model
    torch.cuda.empty_cache()
    return out


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def run_sampler_workload(dev, timed, rows, vocab=151936):
    """Batched top-k sampling over one step's logits (``rows`` x the Qwen3 vocabulary, bf16).  Five buffers (389 MB
    at 256 rows, larger than L2) are taken in turn inside one CUDA graph, so neither L2 nor the host's launch rate
    enters the figure.  The library kernels torch would run for the same job stand beside it."""
    from nanopd_b200 import sampling
    nbuf = 5
    logit_bufs = [(2.5 * torch.randn(rows, vocab, device=dev)).to(torch.bfloat16) for _ in range(nbuf)]
    uni = torch.rand(rows, device=dev)
    tok = torch.empty(rows, dtype=torch.int64, device=dev)
    bytes_s = rows * vocab * 2 + rows * 12
    peak = measured_peak_gbs()[0]
    entry = {"rows": rows, "vocab": vocab, "dtype": "bf16", "algorithmic_bytes": bytes_s}
    side = torch.cuda.Stream(device=dev)
    for k in (1, 10):
        with torch.cuda.stream(side):
            sampling.top_k_sample(logit_bufs[0], k, uniforms=uni, out=tok)
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for lb in logit_bufs:
                    sampling.top_k_sample(lb, k, uniforms=uni, out=tok)
        graph.replay()
        ms = timed(graph.replay, 10) / nbuf
        entry[f"top_{k}"] = {"us": round(ms * 1e3, 2), "gbs": round(bytes_s / (ms * 1e-3) / 1e9, 1),
                             "frac_of_hbm_peak": round(bytes_s / (ms * 1e-3) / 1e9 / peak, 3)}
    turn = iter(range(10 ** 9))
    for name, fn in (("torch_argmax_us", lambda: torch.argmax(logit_bufs[next(turn) % nbuf], dim=-1)),
                     ("torch_topk_10_us", lambda: torch.topk(logit_bufs[next(turn) % nbuf], 10))):
        for _ in range(3):
            fn()
        entry[name] = round(timed(fn, 20) * 1e3, 2)
    entry["status"] = sampling.check_status(dev, raise_on_error=False)
    return entry


def run_gpu_arm(args):
    import paged_kernels                      # raises if the CUDA library is missing: no fallback
    from nanopd_b200 import kv_transfer

    rank, local_rank, world = replicas.init_process_group("nccl")
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE {world}", file=sys.stderr)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    steps, warmup = args.steps, max(3, args.warmup)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()

    def timed(fn, n):
        """n calls of fn between two events on the current stream; returns ms per call."""
        replicas.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        replicas.barrier()
        return e0.elapsed_time(e1) / n

    if args.workload == "reference-grid":
        res = run_reference_grid(args, paged_kernels, dev)
        if rank == 0:
            sampler.stop()
            print(json.dumps({"workload": "the reference micro-benchmark's shape grid (secondary, not the headline metric)", **res}), flush=True)
        if world > 1:
            torch.distributed.destroy_process_group()
        return 0

    if args.workload == "model-tables":
        res = run_model_tables(args, dev, timed)
        if rank == 0:
            sampler.stop()
            print(json.dumps({"workload": "model-level timing tables (secondary, not the headline metric)", **res}), flush=True)
        if world > 1:
            torch.distributed.destroy_process_group()
        return 0

    if args.workload == "model":
        res = run_model_workload(args, dev, timed, args.batch, args.seed)
        ms = replicas.max_over_ranks(res.get("graph_ms_per_step", 0.0), dev)
        toks = replicas.sum_over_ranks(res.get("batch", 0), dev)
        if rank == 0:
            sampler.stop()
            if ms > 0:
                res["n_gpus"] = world
                res["tok_s_all_gpus"] = round(toks / (ms * 1e-3), 1)
            print(json.dumps({"workload": "decode tokens/s at model level (secondary, not the headline metric)", **res}), flush=True)
        if world > 1:
            torch.distributed.destroy_process_group()
        return 0

    if args.workload == "disagg":
        # one process drives all the GPUs, one thread per GPU, as the reference does; other ranks wait on the host
        replicas.host_barrier()
        if rank == 0:
            res = run_disagg_workload(args, args.gpus)
            sampler.stop()
            print(json.dumps({"workload": "disaggregated prefill/decode (secondary, not the headline metric)", **res}), flush=True)
        replicas.host_barrier()
        if world > 1:
            torch.distributed.destroy_process_group()
        return 0

    if args.workload == "poisson":
        res = run_poisson_workload(args, dev)
        agg = {}
        for lam, fig in res.get("rates", {}).items():
            agg[lam] = replicas.sum_over_ranks(float(fig["output_tok_s"]), dev)
        if rank == 0:
            sampler.stop()
            res["n_gpus"] = world
            res["output_tok_s_all_replicas"] = {k: round(v, 1) for k, v in agg.items()}
            print(json.dumps({"workload": "continuous batching under Poisson arrivals, one replica per GPU "
                                          "(secondary, not the headline metric)", **res}), flush=True)
        if world > 1:
            torch.distributed.destroy_process_group()
        return 0

    if args.workload == "sampler":
        res = run_sampler_workload(dev, timed, args.batch)
        if rank == 0:
            sampler.stop()
            print(json.dumps({"workload": "batched top-k sampling of one step (secondary, not the headline metric)", **res}), flush=True)
        if world > 1:
            torch.distributed.destroy_process_group()
        return 0

    if args.workload == "prefill":
        res = run_prefill_workload(args, paged_kernels, dev, timed)
        res["device_status"] = paged_kernels.check_status(dev, raise_on_error=False)
        if rank == 0:
            sampler.stop()
            print(json.dumps({"workload": "cfg3 chunked prefill (secondary, not the headline metric)", **res}), flush=True)
        return 0

    # every replica gets the same draw of lengths and tables: per-GPU work is identical (weak scaling)
    b = workloads.make_config2(device=dev, seed=args.seed, batch=args.batch)
    S, Hq, Hkv, D, B = b.query.size(0), b.num_q_heads, b.num_kv_heads, b.head_dim, b.block_size
    ctx = b.ctx_lens.cpu().tolist()
    attn_bytes, store_bytes = algorithmic_bytes(ctx, Hq, Hkv, D, B)
    step_bytes = attn_bytes + store_bytes
    positions = b.positions.contiguous()
    seq_lens = b.seq_lens_after_store.contiguous()
    out = torch.zeros_like(b.query)
    max_blk = b.max_blocks

    def step():
        paged_kernels.paged_kv_store(b.k_cache, b.v_cache, b.k_new, b.v_new, b.block_tables, positions)
        paged_kernels.paged_attention_forward(out, b.query, b.k_cache, b.v_cache, b.block_tables, seq_lens,
                                              b.scale, B, max_blk, max_ctas=args.max_ctas)

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    if args.profile:
        for _ in range(steps):
            step()
        torch.cuda.synchronize()
        print(json.dumps({"profile_run": True, "steps": steps, "batch": S, "attention_bytes_per_launch": attn_bytes}))
        if rank == 0:
            sampler.stop()
        return 0

    sampler.mark_begin()
    # The timed region is exactly `steps` steps between a barrier + synchronize on both sides.  It is short (a few
    # milliseconds at the default sizes), so the block is repeated and the median block is reported, with the spread.
    blocks = max(1, args.repeats)
    step_blocks = sorted(timed(step, steps) for _ in range(blocks))
    ms_step = statistics.median(step_blocks)
    # the attention kernel alone (streaming + in-kernel merge of split sequences): the launch the roofline is quoted on
    attn_fn = lambda: paged_kernels.paged_attention_forward(
        out, b.query, b.k_cache, b.v_cache, b.block_tables, seq_lens, b.scale, B, max_blk)
    attn_blocks = sorted(timed(attn_fn, steps) for _ in range(blocks))
    ms_attn = statistics.median(attn_blocks)
    ms_stream = ms_attn
    ms_store_host = timed(lambda: paged_kernels.paged_kv_store(
        b.k_cache, b.v_cache, b.k_new, b.v_new, b.block_tables, positions), steps)

    # ---- end to end through the public op with HOST buffers ----
    # All of the step's host inputs live in ONE pinned staging buffer and cross PCIe in ONE copy; the
    # device-side tensors the ops receive are views of its device twin.
    parts = dict(q=b.query, k_new=b.k_new, v_new=b.v_new, bt=b.block_tables, pos=positions, sl=seq_lens)
    sizes = {k: (v.numel() * v.element_size() + 255) // 256 * 256 for k, v in parts.items()}
    h2d = sum(sizes.values())
    stage_host = torch.empty(h2d, dtype=torch.uint8).pin_memory()
    stage_dev = torch.empty(h2d, dtype=torch.uint8, device=dev)
    dbuf, off = {}, 0
    for k, v in parts.items():
        nbytes = v.numel() * v.element_size()
        stage_host[off:off + nbytes].copy_(v.contiguous().view(-1).view(torch.uint8).cpu())
        dbuf[k] = stage_dev[off:off + nbytes].view(v.dtype).view(v.shape)
        off += sizes[k]
    out_host = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    d2h = out_host.numel() * out_host.element_size()

    def e2e_step():
        stage_dev.copy_(stage_host, non_blocking=True)
        paged_kernels.paged_kv_store(b.k_cache, b.v_cache, dbuf["k_new"], dbuf["v_new"], dbuf["bt"], dbuf["pos"])
        paged_kernels.paged_attention_forward(out, dbuf["q"], b.k_cache, b.v_cache, dbuf["bt"], dbuf["sl"],
                                              b.scale, B, max_blk)
        out_host.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()     # the host consumes the result every step

    for _ in range(3):
        e2e_step()
    ms_e2e_eager = timed(e2e_step, steps)

    # The same four operations recorded once in a CUDA graph and replayed: one submission per step instead of four
    # (what a serving loop with fixed buffer addresses does).  The copies stay inside the step and the host still
    # waits for the result every step.
    ms_e2e_graph = None
    try:
        side_e = torch.cuda.Stream(device=dev)
        side_e.wait_stream(torch.cuda.current_stream(dev))
        graph_e = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side_e):
            e2e_step()                                  # the stream's workspace exists before the capture
            with torch.cuda.graph(graph_e, stream=side_e):
                stage_dev.copy_(stage_host, non_blocking=True)
                paged_kernels.paged_kv_store(b.k_cache, b.v_cache, dbuf["k_new"], dbuf["v_new"], dbuf["bt"], dbuf["pos"])
                paged_kernels.paged_attention_forward(out, dbuf["q"], b.k_cache, b.v_cache, dbuf["bt"], dbuf["sl"],
                                                      b.scale, B, max_blk)
                out_host.copy_(out, non_blocking=True)
        torch.cuda.synchronize(dev)

        def e2e_graph_step():
            graph_e.replay()
            torch.cuda.current_stream().synchronize()

        out_host.zero_()
        for _ in range(3):
            e2e_graph_step()
        if torch.equal(out_host, out.cpu()):
            ms_e2e_graph = timed(e2e_graph_step, steps)
        del graph_e                                     # it holds the staging buffers' addresses; they are freed below
    except Exception as exc:  # noqa: BLE001
        print(f"e2e graph variant skipped: {exc}", file=sys.stderr)
        ms_e2e_graph = None
    # Pipelined: two staging buffers on the device; the upload of step i+1's inputs runs on a copy stream while step i's
    # kernels run, as a serving loop does when the next step's inputs do not depend on this step's output.  Every step
    # still uploads one set of inputs (3.67 MB), runs store + attention on it, downloads its output (2 MB) and has the
    # host wait for that output; the timed region holds exactly `steps` uploads, steps and downloads.
    ms_e2e_pipe = ms_e2e_pipe_graph = None
    try:
        copy_stream = torch.cuda.Stream(device=dev)
        main_stream = torch.cuda.current_stream(dev)
        stage2 = [stage_dev, torch.empty_like(stage_dev)]
        views2 = []
        for sd in stage2:
            vw, off2 = {}, 0
            for k_, v_ in parts.items():
                nbytes = v_.numel() * v_.element_size()
                vw[k_] = sd[off2:off2 + nbytes].view(v_.dtype).view(v_.shape)
                off2 += sizes[k_]
            views2.append(vw)
        uploaded = [torch.cuda.Event(), torch.cuda.Event()]
        consumed = [torch.cuda.Event(), torch.cuda.Event()]
        for ev in consumed:
            ev.record(main_stream)
        state = {"i": 0}

        def upload(buf):
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(consumed[buf])          # the kernels that read this buffer two steps ago
                stage2[buf].copy_(stage_host, non_blocking=True)
                uploaded[buf].record(copy_stream)

        def e2e_pipelined_step():
            cur = state["i"] & 1
            upload(cur ^ 1)                                    # the next step's inputs, behind this step's kernels
            main_stream.wait_event(uploaded[cur])
            vw = views2[cur]
            paged_kernels.paged_kv_store(b.k_cache, b.v_cache, vw["k_new"], vw["v_new"], vw["bt"], vw["pos"])
            paged_kernels.paged_attention_forward(out, vw["q"], b.k_cache, b.v_cache, vw["bt"], vw["sl"], b.scale, B, max_blk)
            consumed[cur].record(main_stream)
            out_host.copy_(out, non_blocking=True)
            main_stream.synchronize()                          # the host consumes the result every step
            state["i"] += 1

        upload(0)
        out_host.zero_()
        for _ in range(4):
            e2e_pipelined_step()
        if torch.equal(out_host, out.cpu()):
            ms_e2e_pipe = timed(e2e_pipelined_step, steps)
        torch.cuda.synchronize(dev)
        # The same pipeline as two CUDA graphs (one per staging buffer) replayed in turn: inside a graph the upload of
        # the next step's inputs is a branch beside this step's store, attention and download; one submission per step.
        try:
            cap = torch.cuda.Stream(device=dev)
            cap.wait_stream(main_stream)
            graphs = []
            with torch.cuda.stream(cap):
                for cur in (0, 1):
                    vw = views2[cur]
                    paged_kernels.paged_kv_store(b.k_cache, b.v_cache, vw["k_new"], vw["v_new"], vw["bt"], vw["pos"])
                    paged_kernels.paged_attention_forward(out, vw["q"], b.k_cache, b.v_cache, vw["bt"], vw["sl"], b.scale, B, max_blk)
                cap.synchronize()
                for cur in (0, 1):
                    g_ = torch.cuda.CUDAGraph()
                    vw = views2[cur]
                    with torch.cuda.graph(g_, stream=cap):
                        copy_stream.wait_stream(cap)
                        with torch.cuda.stream(copy_stream):
                            stage2[cur ^ 1].copy_(stage_host, non_blocking=True)
                        paged_kernels.paged_kv_store(b.k_cache, b.v_cache, vw["k_new"], vw["v_new"], vw["bt"], vw["pos"])
                        paged_kernels.paged_attention_forward(out, vw["q"], b.k_cache, b.v_cache, vw["bt"], vw["sl"], b.scale, B, max_blk)
                        out_host.copy_(out, non_blocking=True)
                        cap.wait_stream(copy_stream)
                    graphs.append(g_)
            torch.cuda.synchronize(dev)
            stage2[0].copy_(stage_host)
            gstate = {"i": 0}

            def e2e_pipelined_graph_step():
                graphs[gstate["i"] & 1].replay()
                torch.cuda.current_stream().synchronize()
                gstate["i"] += 1

            out_host.zero_()
            for _ in range(4):
                e2e_pipelined_graph_step()
            if torch.equal(out_host, out.cpu()):
                ms_e2e_pipe_graph = timed(e2e_pipelined_graph_step, steps)
            torch.cuda.synchronize(dev)
            del graphs
        except Exception as exc:  # noqa: BLE001
            print(f"e2e pipelined graph variant skipped: {exc}", file=sys.stderr)
        del stage2, views2
    except Exception as exc:  # noqa: BLE001
        print(f"e2e pipelined variant skipped: {exc}", file=sys.stderr)
        ms_e2e_pipe = None
    e2e_how = "eager: four calls of the public API per step"
    ms_e2e = ms_e2e_eager
    if ms_e2e_graph is not None and ms_e2e_graph < ms_e2e:
        ms_e2e, e2e_how = ms_e2e_graph, "the four calls of the public API recorded in a CUDA graph, one replay per step"
    if ms_e2e_pipe is not None and ms_e2e_pipe < ms_e2e:
        ms_e2e, e2e_how = ms_e2e_pipe, ("eager calls of the public API, two staging buffers: the upload of the next step's "
                                        "inputs overlaps this step's kernels")
    if ms_e2e_pipe_graph is not None and ms_e2e_pipe_graph < ms_e2e:
        ms_e2e, e2e_how = ms_e2e_pipe_graph, ("two staging buffers and one CUDA graph per buffer, replayed in turn: the upload "
                                              "of the next step's inputs is a branch beside this step's store, attention "
                                              "and download")
    sampler.mark_end()
    clocks = sampler.stop() if rank == 0 else None

    status = paged_kernels.check_status(dev, raise_on_error=False)

    # ---- aggregate over replicas: total bytes / slowest rank ----
    tot_bytes = replicas.sum_over_ranks(step_bytes, dev)
    ms_step_max = replicas.max_over_ranks(ms_step, dev)
    ms_e2e_max = replicas.max_over_ranks(ms_e2e, dev)
    ms_stream_max = replicas.max_over_ranks(ms_stream, dev)

    extras = {}
    cpu_baseline = None
    if not args.no_model:
        # decode tokens/s at model level, on every rank (replicas): aggregate = all sequences / slowest rank
        try:
            del stage_dev, dbuf
            torch.cuda.empty_cache()
            md = run_model_workload(args, dev, timed, args.batch, args.seed)
        except Exception as exc:  # noqa: BLE001
            md = {"error": str(exc)[:300]}
        ms_model = replicas.max_over_ranks(float(md.get("graph_ms_per_step", 0.0)), dev)
        toks_model = replicas.sum_over_ranks(int(md.get("batch", 0)) if ms_model > 0 else 0, dev)
        if ms_model > 0 and "tok_s" in md:
            md["n_gpus"] = world
            md["tok_s_all_gpus"] = round(toks_model / (ms_model * 1e-3), 1)
        extras["model_decode"] = md
        # continuous batching under Poisson arrivals (configuration 4), two of the five rates; one replica per GPU
        try:
            torch.cuda.empty_cache()
            po = run_poisson_workload(args, dev, rates=(8, 32), horizon_s=4.0)
        except Exception as exc:  # noqa: BLE001
            po = {"error": str(exc)[:300]}
        for lam in ("8", "32"):
            tok = float(po.get("rates", {}).get(lam, {}).get("output_tok_s", 0.0))
            tot = replicas.sum_over_ranks(tok, dev)
            if "rates" in po and lam in po["rates"]:
                po["rates"][lam]["output_tok_s_all_replicas"] = round(tot, 1)
        po["n_gpus"] = world
        po["all_rates"] = "python bench.py --workload poisson sweeps 2, 4, 8, 16, 32 req/s"
        extras["poisson"] = po
    if world > 1:
        # Page migration over NVLink: rank 0 pulls 1024 blocks x 36 layers (2.4 GB, one 16k-token request of
        # the Qwen3-8B layout) from the next GPU's pool into its own while the other ranks wait — on the host, not
        # in an NCCL barrier, whose kernel would sit on their GPUs beside the kernels rank 0 launches there.
        torch.cuda.empty_cache()
        replicas.host_barrier()
        if rank == 0:
            try:
                peer = (local_rank + 1) % torch.cuda.device_count()
                L_m, nb_m = 36, 1024
                src_k = torch.empty(L_m, nb_m, Hkv, B, D, dtype=torch.bfloat16, device=f"cuda:{peer}").normal_()
                src_v = torch.empty(L_m, nb_m, Hkv, B, D, dtype=torch.bfloat16, device=f"cuda:{peer}").normal_()
                dst_k = torch.empty(L_m, nb_m, Hkv, B, D, dtype=torch.bfloat16, device=dev)
                dst_v = torch.empty_like(dst_k)
                ids = torch.randperm(nb_m).tolist()
                torch.cuda.synchronize(peer)
                fn = lambda: kv_transfer.transfer_kv(src_k, src_v, dst_k, dst_v, ids)
                fn()
                torch.cuda.synchronize(dev)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(5):
                    fn()
                e1.record()
                torch.cuda.synchronize(dev)
                ms_mig = e0.elapsed_time(e1) / 5
                mig_bytes = kv_transfer.migration_bytes(nb_m, src_k)
                # the same pull on a side stream while the decode step loop runs on the main stream
                side = torch.cuda.Stream(device=dev)
                side.wait_stream(torch.cuda.current_stream(dev))
                n_during = 24
                evs = [torch.cuda.Event(enable_timing=True) for _ in range(n_during + 1)]
                m0, m1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                with torch.cuda.stream(side):
                    m0.record()
                for _ in range(3):
                    kv_transfer.transfer_kv(src_k, src_v, dst_k, dst_v, ids, stream=side)
                with torch.cuda.stream(side):
                    m1.record()
                evs[0].record()
                for i in range(n_during):
                    step()
                    evs[i + 1].record()
                torch.cuda.synchronize(dev)
                t_mig_busy = m0.elapsed_time(m1) / 3
                # steps that ended inside the migration window
                t_end, inside = 0.0, []
                for i in range(n_during):
                    dt = evs[i].elapsed_time(evs[i + 1])
                    t_end += dt
                    if t_end <= 3 * t_mig_busy:
                        inside.append(dt)
                sel_d = torch.tensor(ids, device=dev)
                ok = True
                for lo in range(0, nb_m, 256):             # every migrated block, against a copy-engine copy of its source
                    part = sel_d[lo:lo + 256]
                    ok = ok and torch.equal(dst_k[:, part], src_k[:, part.to(src_k.device)].to(dev))
                    ok = ok and torch.equal(dst_v[:, part], src_v[:, part.to(src_v.device)].to(dev))
                from nanopd_b200 import serving
                peak_m = serving.measure_peer_copy_peak(peer, local_rank)
                extras["migrate_nvlink"] = {"gbs_one_direction": round(mig_bytes / (ms_mig * 1e-3) / 1e9, 1),
                                            "ms": round(ms_mig, 3), "bytes": mig_bytes, "blocks": nb_m, "layers": L_m,
                                            "from_gpu": peer, "to_gpu": local_rank,
                                            "data_check": bool(ok), "data_check_blocks": nb_m * L_m * 2,
                                            "gbs_while_decoding": round(mig_bytes / (t_mig_busy * 1e-3) / 1e9, 1),
                                            "decode_step_ms_during_migration": round(sum(inside) / max(1, len(inside)), 4),
                                            "decode_step_ms_alone": round(ms_step, 4),
                                            "peak_gbs": round(peak_m["gbs"], 1), "peak_source": "measured in this run: " + peak_m["how"],
                                            "frac_of_peer_copy_peak": round(mig_bytes / (ms_mig * 1e-3) / 1e9 / peak_m["gbs"], 3)}
                del src_k, src_v, dst_k, dst_v
            except Exception as exc:  # noqa: BLE001
                extras["migrate_nvlink_error"] = str(exc)[:200]
            if not args.no_model:
                try:
                    del b, out
                    torch.cuda.empty_cache()
                    extras["disagg"] = run_disagg_workload(args, world)
                except Exception as exc:  # noqa: BLE001
                    import traceback
                    extras["disagg_error"] = (str(exc)[:300] + " | " + traceback.format_exc()[-600:])
        replicas.host_barrier()
    if rank == 0 and world == 1:
        # secondary kernels, timed briefly
        extras["attention_ms"] = round(ms_attn, 4)
        extras["store_host_call_ms"] = round(ms_store_host, 4)     # back-to-back eager calls: the Python shim, not the kernel
        try:
            extras["kv_store_kernel"] = run_store_kernel_timing(paged_kernels, b, positions, dev)
        except Exception as exc:  # noqa: BLE001
            extras["kv_store_kernel_error"] = str(exc)[:200]
        try:
            extras["shim_host_cost"] = run_shim_host_cost(paged_kernels, dev)
        except Exception as exc:  # noqa: BLE001
            extras["shim_host_cost_error"] = str(exc)[:200]
        try:
            extras["cfg1"] = run_config1(paged_kernels, dev, args.seed)
        except Exception as exc:  # noqa: BLE001
            extras["cfg1_error"] = str(exc)[:200]
        try:
            # fused QK-norm + rotary + store: the decode batch (one token per sequence) and an 8192-token prefill
            for label, T_f in (("decode_256_tokens", S), ("prefill_8192_tokens", 8192)):
                qkv = torch.randn(T_f, (Hq + 2 * Hkv) * D, device=dev).to(torch.bfloat16)
                q_f = qkv[:, :Hq * D].view(T_f, Hq, D)
                k_f = qkv[:, Hq * D:(Hq + Hkv) * D].view(T_f, Hkv, D)
                v_f = qkv[:, (Hq + Hkv) * D:].view(T_f, Hkv, D)
                cs = torch.randn(T_f, D, device=dev).to(torch.bfloat16)
                wn = torch.ones(D, dtype=torch.bfloat16, device=dev)
                q_o = torch.empty(T_f, Hq, D, dtype=torch.bfloat16, device=dev)
                if T_f == S:
                    bt_f, pos_f = b.block_tables, positions
                else:       # tokens spread over the batch's sequences, T_f / S consecutive positions each
                    per = T_f // S
                    bt_f = b.block_tables.repeat_interleave(per, dim=0)
                    pos_f = (torch.clamp(positions - per, min=0).repeat_interleave(per) +
                             torch.arange(per, device=dev, dtype=torch.int32).repeat(S))
                fn_f = lambda: paged_kernels.paged_qk_norm_rope_store(q_f, k_f, v_f, cs, cs, b.k_cache, b.v_cache, bt_f,
                                                                      pos_f, wn, wn, 1e-6, q_out=q_o)
                for _ in range(3):
                    fn_f()
                ms_f = timed(fn_f, min(steps, 50))
                bytes_f = 2 * T_f * (Hq + 2 * Hkv) * D * 2 + 2 * T_f * D * 2 + 8 * T_f
                extras.setdefault("fused_norm_rope_store", {})[label] = {
                    "ms": round(ms_f, 4), "gbs": round(bytes_f / (ms_f * 1e-3) / 1e9, 1), "algorithmic_bytes": bytes_f}
            del qkv, q_o
        except Exception as exc:  # noqa: BLE001
            extras["fused_norm_rope_store_error"] = str(exc)[:200]
        try:
            extras["top_k_sample"] = run_sampler_workload(dev, timed, S)
        except Exception as exc:  # noqa: BLE001
            extras["top_k_sample_error"] = str(exc)[:200]
        try:
            # the same launch on the interleaved cache layouts of the reference's split-K op
            k_il = b.k_cache.view(b.k_cache.size(0), Hkv, B, D // 8, 8).permute(0, 1, 3, 2, 4).contiguous()
            v_il = b.v_cache.permute(0, 1, 3, 2).contiguous()
            fn_il = lambda: paged_kernels.paged_attention_forward(out, b.query, k_il, v_il, b.block_tables, seq_lens,
                                                                  b.scale, B, max_blk)
            for _ in range(3):
                fn_il()
            extras["attention_interleaved_layout_ms"] = round(timed(fn_il, min(steps, 50)), 4)
            del k_il, v_il
        except Exception as exc:  # noqa: BLE001
            extras["interleaved_error"] = str(exc)[:200]
        try:
            L, nb = 36, 96
            pool_k = torch.randn(L, nb, Hkv, B, D, device=dev).to(torch.bfloat16)
            pool_v = torch.randn(L, nb, Hkv, B, D, device=dev).to(torch.bfloat16)
            dst_k, dst_v = torch.empty_like(pool_k), torch.empty_like(pool_v)
            ids = torch.randperm(nb)[:64].to(torch.int32).to(dev)
            fn = lambda: paged_kernels.paged_kv_migrate(pool_k, pool_v, dst_k, dst_v, ids, max_ctas=96)
            for _ in range(3):
                fn()
            ms_mig = timed(fn, 10)
            mig_bytes = kv_transfer.migration_bytes(64, pool_k)
            extras["migrate_same_gpu_gbs_one_direction"] = round(mig_bytes / (ms_mig * 1e-3) / 1e9, 1)
            del pool_k, pool_v, dst_k, dst_v
        except Exception as exc:  # noqa: BLE001
            extras["migrate_error"] = str(exc)[:200]
        try:
            torch.cuda.empty_cache()
            extras["prefill_cfg3"] = run_prefill_workload(args, paged_kernels, dev, timed)
        except Exception as exc:  # noqa: BLE001
            extras["prefill_error"] = str(exc)[:200]
        # CPU baseline on a bounded sample of the same workload
        bc = workloads.DecodeBatch(**{f: (getattr(b, f).cpu() if torch.is_tensor(getattr(b, f)) else getattr(b, f))
                                      for f in b.__dataclass_fields__})
        n = cpu_reference_sample(bc, target_seconds=10.0)
        gbs, dt = cpu_reference_time(bc, n, 1, 0)
        cpu_baseline = {"value": round(gbs, 4), "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port",
                        "sample": f"first {n} of {S} sequences ({int(bc.seq_lens_after_store[:n].sum())} tokens), "
                                  f"one pass, {dt:.2f} s"}

    if rank == 0:
        peak, peak_src = measured_peak_gbs()
        achieved = attn_bytes / (ms_stream_max * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": round(tot_bytes / (ms_step_max * 1e-3) / 1e9, 2), "unit": UNIT,
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": round(ms_step_max, 5),
            "timed_blocks": {"blocks": blocks, "steps_per_block": steps, "reported": "median block (max over ranks)",
                             "ms_per_step_min": round(step_blocks[0], 5), "ms_per_step_max": round(step_blocks[-1], 5),
                             "attention_launch_ms_min": round(attn_blocks[0], 5),
                             "attention_launch_ms_max": round(attn_blocks[-1], 5), "rank": 0},
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": config_block(ctx, S, Hq, Hkv, D, world),
            "e2e": {"value": round(tot_bytes / (ms_e2e_max * 1e-3) / 1e9, 2), "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": round(ms_e2e_max, 5),
                    "submission": e2e_how, "eager_ms_per_step": round(ms_e2e_eager, 5),
                    "graph_ms_per_step": None if ms_e2e_graph is None else round(ms_e2e_graph, 5),
                    "pipelined_ms_per_step": None if ms_e2e_pipe is None else round(ms_e2e_pipe, 5),
                    "pipelined_graph_ms_per_step": None if ms_e2e_pipe_graph is None else round(ms_e2e_pipe_graph, 5)},
            "gpu_launches": 2 * steps,
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4),
                         # DRAM bytes per launch: dram__bytes_read.sum + dram__bytes_write.sum of the ncu capture of a
                         # batch-64 case of the same kernel (372.72 MB + 5.92 MB for 369.46 MB of algorithmic bytes),
                         # scaled by the algorithmic bytes of this launch (traffic grows in proportion)
                         "traffic": int(attn_bytes * (372.716032 + 5.916160) / 369.46), "traffic_source": "profiles/decode_stream_batch64_ncu_full.md",
                         "peak_source": peak_src,
                         "kernel": "paged_decode_stream_kernel<bf16,128,1>",
                         "algorithmic_bytes_per_launch": attn_bytes, "launch_ms": round(ms_stream_max, 5)},
            "cpu_baseline": cpu_baseline,
            "clocks": clocks,
            "device_status": status,
            "other": extras,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--repeats", type=int, default=25,
                    help="how many times the timed block of --steps steps is repeated (median, min and max are reported)")
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--workload", choices=["decode", "prefill", "model", "model-tables", "reference-grid", "sampler", "disagg", "poisson"],
                    default="decode",
                    help="decode = the headline configuration 2 (default); prefill = configuration 3's chunked prefill")
    ap.add_argument("--max-ctas", type=int, default=0,
                    help="cap the decode-attention grid (0 = one CTA per SM): the launch shape a mixed step uses when "
                         "it shares the SMs with a prompt chunk; for profiling that instance")
    ap.add_argument("--profile", action="store_true",
                    help="only warm up and run the timed step loop (for short ncu captures); prints no bench line")
    ap.add_argument("--no-model", action="store_true",
                    help="skip the model-level measurements (decode tokens/s, Poisson arrivals, disaggregated serving; "
                         "they need ~75 GB of device memory)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback "
                         "(use --impl reference for the CPU baseline)")
    return run_gpu_arm(args)


if __name__ == "__main__":
    sys.exit(main())
