"""Measurement drivers for the two serving layouts built on ``workers``: disaggregated prefill/decode across the
GPUs of one box, and continuous batching under Poisson arrivals on one GPU.  ``bench.py`` calls these and prints
their results; the reference's counterparts are its load generators (nanoPD/benchmark/benchmark.py,
nanoPD/benchmark/benchmark_poisson.py), which need checkpoints and a tokenizer and print no kernel-level figures.

Workloads are synthetic and seeded: random token ids, prompt and output lengths drawn from the distributions the
benchmark configurations name.
"""
from __future__ import annotations

import statistics
import threading
import time
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from . import decoder_step, kv_transfer, paged_kernels, workers


def _pct(values: Sequence[float], q: float) -> float:
    v = sorted(values)
    if not v:
        return float("nan")
    return v[min(len(v) - 1, int(round(q * (len(v) - 1))))]


def build_models(device_ids: Sequence[int], shape=None, dtype=torch.bfloat16, seed: int = 0, top_k: int = 10,
                 max_position: int = 16384 + 1024 + 64) -> Dict[int, decoder_step.SyntheticDecoder]:
    """One random-init replica per GPU (the same weights everywhere: same seed), built in parallel threads."""
    shape = shape or decoder_step.DecoderShape()
    out: Dict[int, decoder_step.SyntheticDecoder] = {}
    errors: List[BaseException] = []

    def make(i):
        try:
            with torch.cuda.device(i):
                out[i] = decoder_step.SyntheticDecoder(torch.device("cuda", i), shape, dtype, seed=seed,
                                                       max_position=max_position, top_k=top_k)
                torch.cuda.synchronize(i)
        except BaseException as exc:  # noqa: BLE001
            errors.append(exc)

    threads = [threading.Thread(target=make, args=(i,)) for i in device_ids]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise errors[0]
    return out


# ---------------------------------------------------------------------------------------------------------------
# NVLink figures measured in the run
# ---------------------------------------------------------------------------------------------------------------
def measure_peer_copy_peak(src_dev: int, dst_dev: int, nbytes: int = 1 << 30, repeats: int = 5) -> Dict[str, float]:
    """One contiguous device-to-device copy through the copy engine (``Tensor.copy_`` between two GPUs), timed with
    events on the destination: the link peak the migration kernel is compared with."""
    src = torch.empty(nbytes, dtype=torch.uint8, device=f"cuda:{src_dev}").fill_(1)
    dst = torch.empty(nbytes, dtype=torch.uint8, device=f"cuda:{dst_dev}")
    torch.cuda.synchronize(src_dev)
    best = float("inf")
    with torch.cuda.device(dst_dev):
        dst.copy_(src)
        torch.cuda.synchronize(dst_dev)
        for _ in range(repeats):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            dst.copy_(src)
            e1.record()
            torch.cuda.synchronize(dst_dev)
            best = min(best, e0.elapsed_time(e1))
    del src, dst
    return {"gbs": nbytes / (best * 1e-3) / 1e9, "ms": best, "bytes": nbytes, "from_gpu": src_dev, "to_gpu": dst_dev,
            "how": "Tensor.copy_ of one contiguous buffer between two GPUs (copy engine), best of %d" % repeats}


def measure_link_sharing(device_ids: Sequence[int], blocks: int = 512, layers: int = 36, hkv: int = 8, bs: int = 16,
                         d: int = 128, repeats: int = 3) -> Dict[str, object]:
    """The migration kernel when links are shared: k decode GPUs pulling from ONE prefill GPU at the same time
    (that GPU's egress is shared), and one decode GPU pulling from k prefill GPUs at the same time (its ingress is
    shared).  Each pull moves ``blocks`` block-scattered blocks of all layers.  Every pull is timed by events on its
    own stream; the aggregate is all bytes over the host-clock window from the first launch to the end of the last
    pull (the pulls run on different GPUs, whose events cannot be compared), best of ``repeats``."""
    ids = list(device_ids)
    pools = {}
    for i in ids:
        k = torch.empty(layers, blocks, hkv, bs, d, dtype=torch.bfloat16, device=f"cuda:{i}").normal_()
        pools[i] = (k, torch.empty_like(k).normal_(), torch.empty_like(k), torch.empty_like(k))
    g = torch.Generator().manual_seed(0)
    perm = torch.randperm(blocks, generator=g).to(torch.int32)
    perm_dev = {i: perm.to(f"cuda:{i}") for i in ids}          # block lists resident on every destination
    nbytes = kv_transfer.migration_bytes(blocks, pools[ids[0]][0])
    for i in ids:
        torch.cuda.synchronize(i)

    def run(pairs):
        """pairs: (src_dev, dst_dev) pulls started together; returns (per-pull ms from events on each pull's own
        stream, milliseconds from the first launch to the end of the last pull by the host's clock)."""
        streams = {p: torch.cuda.Stream(device=f"cuda:{p[1]}") for p in pairs}
        best = None
        for _ in range(repeats + 1):
            evs = {}
            for i in ids:
                torch.cuda.synchronize(i)
            t0 = time.perf_counter()
            for p in pairs:                         # enqueue everything first, then wait
                s, t = p
                with torch.cuda.device(t):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(streams[p])
                    kv_transfer.transfer_kv(pools[s][0], pools[s][1], pools[t][2], pools[t][3], perm_dev[t], stream=streams[p])
                    e1.record(streams[p])
                    evs[p] = (e0, e1)
            for p in pairs:
                streams[p].synchronize()
            window = (time.perf_counter() - t0) * 1e3
            ms = [evs[p][0].elapsed_time(evs[p][1]) for p in pairs]
            if best is None or window < best[1]:
                best = (ms, window)
        return best

    out: Dict[str, object] = {"bytes_per_pull": nbytes, "blocks": blocks, "layers": layers,
                              "aggregate": "all bytes / host-clock window from the first launch to the end of the last pull"}
    src = ids[0]
    for k in (1, 2, 4, 7):
        if k > len(ids) - 1:
            break
        ms, window = run([(src, t) for t in ids[1:1 + k]])
        out[f"fan_out_{k}"] = {"aggregate_gbs": round(k * nbytes / (window * 1e-3) / 1e9, 1),
                               "per_pull_gbs": [round(nbytes / (m * 1e-3) / 1e9, 1) for m in ms]}
    dst = ids[0]
    for k in (2, 4, 7):
        if k > len(ids) - 1:
            break
        ms, window = run([(s, dst) for s in ids[1:1 + k]])
        out[f"fan_in_{k}"] = {"aggregate_gbs": round(k * nbytes / (window * 1e-3) / 1e9, 1),
                              "per_pull_gbs": [round(nbytes / (m * 1e-3) / 1e9, 1) for m in ms]}
    del pools
    for i in ids:
        with torch.cuda.device(i):
            torch.cuda.empty_cache()
    return out


# ---------------------------------------------------------------------------------------------------------------
# Disaggregated prefill / decode
# ---------------------------------------------------------------------------------------------------------------
def disagg_requests(num: int, vocab: int, seed: int, lo: int = 2048, hi: int = 16384, output_len: int = 128):
    """Prompt lengths uniform in [lo, hi], ``output_len`` output tokens each, random token ids (pinned)."""
    rng = np.random.default_rng(seed)
    lens = rng.integers(lo, hi + 1, size=num)
    g = torch.Generator().manual_seed(seed)
    return [workers.Request(i, torch.randint(0, vocab, (int(n),), generator=g).pin_memory(), output_len)
            for i, n in enumerate(lens)]


def run_disagg_split(models: Dict[int, decoder_step.SyntheticDecoder], prefill_gpus: Sequence[int],
                     decode_gpus: Sequence[int], requests: List[workers.Request], layerwise: bool,
                     prefill_blocks: int = 8192, decode_blocks: int = 12288, capacity: int = 32,
                     max_context: int = 16384 + 128, token_budget: int = 16384, verify: bool = False) -> Dict[str, object]:
    """Serves ``requests`` with the given GPUs as prefill and decode workers and returns the figures of the run.
    ``verify`` keeps every block after use and compares each request's prompt pages on the two sides bit for bit
    (pools must then hold the whole run)."""
    pws = [workers.PrefillWorker(models[i], prefill_blocks, top_k=10, seed=i) for i in prefill_gpus]
    dws = [workers.DecodeWorker(models[i], decode_blocks, capacity=capacity, max_context=max_context) for i in decode_gpus]
    for w in dws:
        w.record_steps = True
        w.keep_blocks = verify
    for w in pws:
        w.keep_blocks = verify
    sched = workers.DisaggregatedScheduler(pws, dws, token_budget=token_budget, layerwise=layerwise)
    for r in requests:
        sched.add_request(r)
    t0 = time.perf_counter()
    done = sched.run_until_done(timeout=600)
    wall = time.perf_counter() - t0
    prompt_tokens = sum(r.prompt_len for r in done)
    out_tokens = sum(r.output_len for r in done)
    mig_bytes = sum(r.stats["migrated_bytes"] for r in done)
    exposed = [r.stats["exposed_transfer_ms"] for r in done]
    prefill_window = max(r.stats["t_first_token"] for r in done)
    res: Dict[str, object] = {
        "prefill_gpus": list(prefill_gpus), "decode_gpus": list(decode_gpus), "layerwise_pull": layerwise,
        "requests": len(done), "prompt_tokens": prompt_tokens, "output_tokens": out_tokens, "wall_s": round(wall, 3),
        # the run ends with the decode of the last request (its 127 steps after the last prompt): prompt throughput is
        # taken over the window in which prompts were computed, up to the arrival of the last one's pages
        "prefill_window_s": round(prefill_window, 3), "prefill_tok_s": round(prompt_tokens / prefill_window, 1),
        "output_tok_s": round(out_tokens / wall, 1),
        "prefill_ms_per_request_median": round(statistics.median(r.stats["prefill_ms"] for r in done), 2),
        "migrated_bytes": mig_bytes, "migrated_gb_per_request_mean": round(mig_bytes / len(done) / 1e9, 3),
        "exposed_transfer_ms": {"median": round(statistics.median(exposed), 3), "p95": round(_pct(exposed, 0.95), 3),
                                "max": round(max(exposed), 3)},
    }
    if not layerwise:
        rates = [r.stats["migrated_bytes"] / (r.stats["transfer_ms"] * 1e-3) / 1e9 for r in done]
        res["pull_gbs_per_request"] = {"median": round(statistics.median(rates), 1), "min": round(min(rates), 1),
                                       "max": round(max(rates), 1)}
    busy, quiet, batch = [], [], []
    for w in dws:
        for a, b, pending, active in w.step_events:
            (busy if pending else quiet).append(a.elapsed_time(b))
            batch.append(active)
    res["decode_step_ms"] = {"while_a_pull_is_pending": round(statistics.median(busy), 3) if busy else None,
                             "otherwise": round(statistics.median(quiet), 3) if quiet else None,
                             "steps": len(busy) + len(quiet), "mean_running_requests": round(sum(batch) / max(1, len(batch)), 2)}
    status = 0
    for w in pws + dws:
        status |= paged_kernels.check_status(w.device, raise_on_error=False)
    res["device_status"] = status
    if verify:
        ok = True
        for r in done:
            pw = r.prefill_worker
            n_full = r.prompt_len // pw.block_size
            dwk = r.decode_worker
            src = torch.tensor(r.src_blocks[:n_full], device=pw.device)
            dst = torch.tensor(r.dst_blocks[:n_full], device=dwk.device)
            for sc, dc in ((pw.k_cache, dwk.k_cache), (pw.v_cache, dwk.v_cache)):
                ok = ok and torch.equal(sc[:, src].to(dwk.device), dc[:, dst])
        res["pages_equal_on_both_sides"] = bool(ok)
    for w in dws:
        w.model.detach_batch()
        w.slots = None
    for w in pws + dws:
        del w.k_cache, w.v_cache
    del pws, dws, sched
    for i in set(prefill_gpus) | set(decode_gpus):
        with torch.cuda.device(i):
            torch.cuda.empty_cache()
    return res


# ---------------------------------------------------------------------------------------------------------------
# Continuous batching under Poisson arrivals
# ---------------------------------------------------------------------------------------------------------------
def poisson_requests(rate: float, horizon_s: float, vocab: int, seed: int, median_prompt: int = 512,
                     sigma: float = 0.8, lo: int = 16, hi: int = 4096, mean_output: int = 256, cap_output: int = 1024):
    """Arrivals of a Poisson process of ``rate`` requests/s over ``horizon_s`` seconds; prompt lengths lognormal
    (median ``median_prompt``, sigma ``sigma``) clipped to [lo, hi]; output lengths geometric with mean
    ``mean_output`` capped at ``cap_output``; random token ids."""
    rng = np.random.default_rng(seed)
    t, arrivals = 0.0, []
    while True:
        t += rng.exponential(1.0 / rate)
        if t >= horizon_s:
            break
        arrivals.append(t)
    g = torch.Generator().manual_seed(seed)
    reqs = []
    for i, at in enumerate(arrivals):
        n = int(np.clip(round(float(np.exp(rng.normal(np.log(median_prompt), sigma)))), lo, hi))
        out = int(min(rng.geometric(1.0 / mean_output), cap_output))
        reqs.append(workers.Request(i, torch.randint(0, vocab, (n,), generator=g).pin_memory(), out, arrival=at))
    return reqs


def run_poisson(model, rate: float, horizon_s: float, seed: int, num_blocks: int = 20480, capacity: int = 256,
                token_budget: int = 2048, max_chunk: int = 2048, worker: Optional[workers.CollocatedWorker] = None):
    """One arrival rate on one GPU: returns throughput and latency figures (and the worker, for reuse)."""
    if worker is None:
        worker = workers.CollocatedWorker(model, num_blocks, capacity=capacity, max_context=4096 + 1024,
                                          token_budget=token_budget, max_chunk=max_chunk, top_k=10, seed=seed)
    worker.finished, worker.decode_tokens, worker.prefill_tokens = [], 0, 0
    reqs = poisson_requests(rate, horizon_s, model.shape.vocab, seed)
    res = workers.serve_open_loop(worker, reqs, drain_timeout=120.0)
    served = [r for r in reqs if "latency_s" in r.stats]
    ttft = [r.stats["ttft_s"] * 1e3 for r in served]
    tpot = [r.stats["tpot_s"] * 1e3 for r in served if "tpot_s" in r.stats]
    out_tokens = sum(r.output_len for r in served)
    figures = {
        "rate_req_s": rate, "horizon_s": horizon_s, "requests": len(reqs), "finished": len(served),
        "wall_s": round(res["wall_s"], 3), "prompt_tokens": sum(r.prompt_len for r in served), "output_tokens": out_tokens,
        "output_tok_s": round(out_tokens / res["wall_s"], 1),
        "ttft_ms": {"median": round(statistics.median(ttft), 2), "p95": round(_pct(ttft, 0.95), 2)} if ttft else None,
        "ms_per_output_token": {"median": round(statistics.median(tpot), 3), "p95": round(_pct(tpot, 0.95), 3)} if tpot else None,
        "device_status": paged_kernels.check_status(model.device, raise_on_error=False),
    }
    return figures, worker
