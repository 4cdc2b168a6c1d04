"""CPU: the host logic of the workers — block pools, the slot table that mirrors the device-resident decode
batch, the planning of a prefill step, and the scheduler's choice of a batch and of a decode worker."""
import numpy as np
import pytest
import torch

from nanopd_b200 import workers


def test_block_pool_is_a_stack_like_the_reference_allocator():
    """nanoPD/block_manager/block_manager.py:9-34: ``pop()`` from the end, freed blocks go back on top."""
    pool = workers.BlockPool(8)
    assert pool.num_free == 7                      # block 0 is the parking block of idle slots
    a = pool.allocate(3)
    assert a == [7, 6, 5]
    pool.free([6])
    assert pool.allocate(2) == [6, 4]
    assert pool.try_allocate(10) is None
    with pytest.raises(MemoryError):
        pool.allocate(10)
    assert 0 not in pool.allocate(pool.num_free)


def test_slot_table_mirrors_what_the_device_does():
    t = workers.SlotTable(capacity=4, max_blocks_per_seq=6, block_size=16)
    s0 = t.admit("a", [9, 8, 7], context_len=40, decode_steps=3)
    s1 = t.admit("b", [5], context_len=3, decode_steps=1)
    assert t.num_active == 2 and t.dirty_rows == {s0, s1} and t.dirty_state
    assert t.tables[s0].tolist() == [9, 8, 7, 0, 0, 0]
    assert (t.positions[s0], t.seq_lens[s0], t.active[s0]) == (40, 41, 1)
    t.dirty_rows.clear()
    t.dirty_state = False
    finished = t.advance()                          # the step a replay performs: active rows move by one
    assert finished == [s1] and t.positions[s0] == 41 and t.seq_lens[s0] == 42
    assert t.positions[[i for i in range(4) if i not in (s0, s1)]].tolist() == [0, 0]     # idle rows stay parked
    assert t.retire(s1) == "b"
    assert t.seq_lens[s1] == 0 and t.active[s1] == 0 and not t.tables[s1].any() and s1 in t.dirty_rows
    assert t.advance() == [] and t.advance() == [s0]
    with pytest.raises(ValueError):
        t.admit("c", [1], context_len=10, decode_steps=10)        # table too short for the tokens to come
    with pytest.raises(ValueError):
        t.admit("c", list(range(7)), context_len=1, decode_steps=1)
    for name in "cde":
        t.admit(name, [1, 2], 1, 1)
    with pytest.raises(RuntimeError):
        t.admit("f", [1, 2], 1, 1)


def _req(rid, n, out=8, arrival=0.0):
    return workers.Request(rid, torch.zeros(n, dtype=torch.int64), out, arrival)


def test_plan_prefill_step_takes_several_chunks_within_the_budget():
    """The reference's scheduler plans one chunk per step (nanoPD/engine/scheduler.py:70-101); here as many as the
    token budget holds, in arrival order, continuing half-done prompts first."""
    a, b, c = _req(0, 3000), _req(1, 700), _req(2, 5000)
    a.prefilled = 2048
    plan = workers.plan_prefill_step([a, b, c], token_budget=4096, max_chunk=2048)
    assert [(r.rid, start, n) for r, start, n in plan] == [(0, 2048, 952), (1, 0, 700), (2, 0, 2048)]
    plan = workers.plan_prefill_step([c, b], token_budget=1024, max_chunk=0)
    assert [(r.rid, start, n) for r, start, n in plan] == [(2, 0, 5000)]            # the first chunk always goes
    plan = workers.plan_prefill_step([b, c], token_budget=1024, max_chunk=0)
    assert [(r.rid, start, n) for r, start, n in plan] == [(1, 0, 700), (2, 0, 324)]
    done = _req(3, 10)
    done.prefilled = 10
    assert workers.plan_prefill_step([done], 100) == []


class _FakeDecode:
    def __init__(self, blocks, slots):
        self.pool = workers.BlockPool(blocks)
        self.slots_left = slots

    def try_reserve(self, req):
        need = (req.prompt_len + req.decode_steps + 15) // 16
        if self.slots_left == 0:
            return False
        got = self.pool.try_allocate(need)
        if got is None:
            return False
        self.slots_left -= 1
        req.dst_blocks, req.decode_worker = got, self
        return True


class _FakePrefill:
    def __init__(self, blocks):
        self.pool = workers.BlockPool(blocks)

    def blocks_for(self, n):
        return (n + 15) // 16


def test_scheduler_batches_within_budget_and_reserves_on_the_emptiest_decode_worker():
    d0, d1 = _FakeDecode(200, 4), _FakeDecode(400, 4)
    sched = workers.DisaggregatedScheduler([_FakePrefill(1000)], [d0, d1], token_budget=4096)
    for rid, n in enumerate([2000, 1500, 1000, 2000]):
        sched.add_request(_req(rid, n))
    batch = sched._take_batch(sched.prefill_workers[0])
    assert [r.rid for r in batch] == [0, 1]                 # 2000 + 1500 fit the budget, + 1000 does not
    assert batch[0].decode_worker is d1 and len(batch[0].dst_blocks) == (2000 + 7 + 15) // 16
    assert batch[1].decode_worker is d1                     # still the one with more free blocks
    batch = sched._take_batch(sched.prefill_workers[0])
    assert [r.rid for r in batch] == [2, 3] and {r.decode_worker for r in batch} <= {d0, d1}
    assert sched._take_batch(sched.prefill_workers[0]) == []


def test_scheduler_waits_when_no_decode_worker_has_room():
    d0 = _FakeDecode(20, 1)
    sched = workers.DisaggregatedScheduler([_FakePrefill(1000)], [d0], token_budget=10 ** 6)
    sched.add_request(_req(0, 100))
    sched.add_request(_req(1, 100))
    assert [r.rid for r in sched._take_batch(sched.prefill_workers[0])] == [0]       # one slot only
    assert sched._take_batch(sched.prefill_workers[0]) == []
    d0.slots_left = 1                                                                 # a request finished
    assert [r.rid for r in sched._take_batch(sched.prefill_workers[0])] == [1]
    # the prefill pool is checked too
    small = workers.DisaggregatedScheduler([_FakePrefill(4)], [_FakeDecode(100, 4)], token_budget=10 ** 6)
    small.add_request(_req(0, 100))
    assert small._take_batch(small.prefill_workers[0]) == []


def test_requests_not_yet_arrived_are_left_waiting():
    sched = workers.DisaggregatedScheduler([_FakePrefill(100)], [_FakeDecode(100, 4)])
    sched.add_request(_req(0, 10, arrival=1e9))
    import time
    sched._t0 = time.perf_counter()
    assert sched._take_batch(sched.prefill_workers[0]) == []


def test_synthetic_request_streams_follow_the_named_distributions():
    """Configuration 4: Poisson arrivals, lognormal prompts clipped to [16, 4096], geometric outputs capped at 1024;
    configuration 5: prompts uniform in [2048, 16384], 128 output tokens.  Seeded, so two draws agree."""
    pin = torch.Tensor.pin_memory
    torch.Tensor.pin_memory = lambda self, *a, **k: self          # no CUDA here: pinning is a no-op for this check
    try:
        from nanopd_b200 import serving
        a = serving.poisson_requests(32.0, 20.0, 1000, seed=3)
        b = serving.poisson_requests(32.0, 20.0, 1000, seed=3)
        d = serving.disagg_requests(200, 1000, seed=3)
    finally:
        torch.Tensor.pin_memory = pin
    assert [r.prompt_len for r in a] == [r.prompt_len for r in b] and [r.arrival for r in a] == [r.arrival for r in b]
    n = len(a)
    assert 500 < n < 780                                            # 32 req/s over 20 s
    arrivals = np.array([r.arrival for r in a])
    assert (np.diff(arrivals) > 0).all() and arrivals[-1] < 20.0
    lens = np.array([r.prompt_len for r in a])
    assert lens.min() >= 16 and lens.max() <= 4096 and 400 < np.median(lens) < 650
    outs = np.array([r.output_len for r in a])
    assert outs.min() >= 1 and outs.max() <= 1024 and 200 < outs.mean() < 320
    dl = np.array([r.prompt_len for r in d])
    assert dl.min() >= 2048 and dl.max() <= 16384 and 8000 < dl.mean() < 10400 and all(r.output_len == 128 for r in d)
    assert all(int(r.prompt.max()) < 1000 and r.prompt.dtype == torch.int64 for r in d[:5])
