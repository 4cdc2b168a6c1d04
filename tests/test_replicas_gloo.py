"""CPU, world_size 2 over gloo: the batch-sharded decode path needs no data-path collective —
each replica evaluates its own sequences and the gathered rows equal the 1-replica result."""
import os
import sys
from pathlib import Path

import torch
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    from nanopd_b200 import replicas, workloads
    from oracle import paged_oracle

    r, _, w = replicas.init_process_group("gloo")
    assert (r, w) == (rank, world)
    b = workloads.make_decode_batch([33, 7, 120, 64, 5], 8, 2, 64, 16, torch.float16, seed=3)
    q, bt, sl = replicas.shard_batch_rows([b.query, b.block_tables, b.ctx_lens], rank, world)
    local = paged_oracle.paged_decode_attention(q, b.k_cache, b.v_cache, bt, sl, b.scale)
    replicas.barrier()
    replicas.host_barrier()          # the host-side barrier the benchmark uses around its one-rank phases
    full = replicas.gather_rows(local, world)
    # plumbing used by the benchmark: max of per-rank time, sum of per-rank work
    assert replicas.max_over_ranks(float(rank + 1)) == float(world)
    assert replicas.sum_over_ranks(float(local.size(0))) == 5.0
    if rank == 0:
        want = paged_oracle.paged_decode_attention(b.query, b.k_cache, b.v_cache, b.block_tables, b.ctx_lens, b.scale)
        torch.save({"ok": bool(torch.equal(full, want))}, os.path.join(out_dir, "result.pt"))
    dist.destroy_process_group()


def test_two_replicas_reproduce_single_replica(tmp_path):
    port = 29600 + (os.getpid() % 300)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert torch.load(tmp_path / "result.pt")["ok"]
