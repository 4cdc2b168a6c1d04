"""GPU: the ops called from several Python threads at once, as the reference's scheduler drives its workers
(nanoPD/router/central_scheduler.py:132-135, 281-283: one thread per worker, each bound to its own GPU).
Each thread works on its own stream (and on its own GPU when two are present); the results must equal those of
the same calls made one after another."""
import threading

import pytest
import torch

from nanopd_b200 import workloads

pytestmark = pytest.mark.gpu


def _one_worker(kernels, dev, seed, rounds, use_stream):
    """``rounds`` times: store a fresh token in every sequence's next slot, attend over it; returns every round's
    output."""
    torch.cuda.set_device(dev)
    b = workloads.make_decode_batch([300 + 97 * i for i in range(12)], 16, 4, 128, 16, torch.bfloat16, device=dev,
                                    seed=seed, pool_blocks=700)
    g = torch.Generator().manual_seed(seed)
    outs = []
    stream = torch.cuda.Stream(device=dev) if use_stream else torch.cuda.current_stream(dev)
    stream.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.device(dev), torch.cuda.stream(stream):
        positions = b.ctx_lens.clone()
        for _ in range(rounds):
            k_new = torch.randn(4, 12, 128, generator=g).to(torch.bfloat16).to(dev, non_blocking=False)
            v_new = torch.randn(4, 12, 128, generator=g).to(torch.bfloat16).to(dev, non_blocking=False)
            q = torch.randn(12, 16, 128, generator=g).to(torch.bfloat16).to(dev, non_blocking=False)
            kernels.paged_kv_store(b.k_cache, b.v_cache, k_new, v_new, b.block_tables, positions)
            out = torch.zeros_like(q)
            kernels.paged_attention_forward(out, q, b.k_cache, b.v_cache, b.block_tables, positions + 1, b.scale, 16,
                                            b.block_tables.size(1))
            outs.append(out)
        stream.synchronize()
    return [o.cpu() for o in outs]


def test_two_threads_give_the_serial_results(kernels):
    ndev = torch.cuda.device_count()
    devs = ["cuda:0", "cuda:1" if ndev >= 2 else "cuda:0"]
    rounds = 25
    serial = [_one_worker(kernels, devs[i], seed=100 + i, rounds=rounds, use_stream=True) for i in range(2)]
    results, errors = [None, None], []

    def run(i):
        try:
            results[i] = _one_worker(kernels, devs[i], seed=100 + i, rounds=rounds, use_stream=True)
        except Exception as exc:  # noqa: BLE001
            errors.append(exc)

    threads = [threading.Thread(target=run, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=300)
    assert not errors, errors
    for i in range(2):
        assert results[i] is not None and len(results[i]) == rounds
        for got, want in zip(results[i], serial[i]):
            assert torch.equal(got, want)
    for d in set(devs):
        assert kernels.check_status(d, raise_on_error=False) == 0
