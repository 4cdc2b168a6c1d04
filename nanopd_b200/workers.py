"""Prefill and decode workers around the paged kernels: the disaggregated layout and continuous batching.

The reference runs one Python process with one thread per worker GPU (nanoPD/router/central_scheduler.py:99-135,
281-283).  Its ``PrefillWorker`` computes whole prompts and hands ``(first_token, block_table, k_cache, v_cache)``
to the scheduler after an unconditional copy of the pages to pinned host memory and a device-wide synchronise
(nanoPD/workers/prefill_worker.py:92-112); its ``DecodeWorker`` pulls the pages on a transfer stream, polls the
transfer's event and decodes the running sequences step by step (nanoPD/workers/decode_worker.py:39-126).  Both
share ONE ``BlockSpaceManager``, so a request occupies the same block ids on every GPU
(central_scheduler.py:99-117).

The classes here keep those roles and method names and change what limited them:

* every GPU has its own allocator (``BlockPool``); a hand-off carries the source ids and the decode side places the
  pages at ids of its own (``npd_kv_migrate`` takes the two lists);
* the prefill side neither extracts to host memory nor synchronises: a hand-off carries a CUDA event recorded
  behind the prompt's last store, and the first token stays on the device;
* with ``layerwise=True`` every layer's pages are pulled as soon as that layer's store has been issued, so that
  the migration hides behind the remaining layers and only the last layer's pages are left when the prompt ends;
* the decode side is a table of SLOTS replayed as one CUDA graph per step: requests are admitted into and retired
  from slots between replays by rewriting the slot's table row, position and length in place;
* ``CollocatedWorker`` (the reference's ``Engine.step`` loop, nanoPD/engine/engine.py:42-113) admits several
  prompt chunks per step within a token budget (``Scheduler.schedule`` admits at most one,
  nanoPD/engine/scheduler.py:70-101).

The model is the random-init stack of ``decoder_step.SyntheticDecoder``; the host logic (``BlockPool``,
``SlotTable``, ``plan_prefill_step``) has no CUDA in it and is tested on the CPU.
"""
from __future__ import annotations

import threading
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import kv_transfer, sampling


# ---------------------------------------------------------------------------------------------------------------
# Host logic
# ---------------------------------------------------------------------------------------------------------------
class BlockPool:
    """Free list of one GPU's physical blocks: a stack, like the reference's ``BlockAllocator``
    (nanoPD/block_manager/block_manager.py:9-34: the block freed last is handed out first), thread-safe because a
    decode thread returns blocks that a prefill thread allocates.  The first ``reserved`` ids are never handed
    out: block 0 is where idle decode slots park their writes."""

    def __init__(self, num_blocks: int, reserved: int = 1):
        if num_blocks <= reserved:
            raise ValueError("the pool needs more blocks than it reserves")
        self.num_blocks = num_blocks
        self._free: List[int] = list(range(reserved, num_blocks))
        self._lock = threading.Lock()

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self, n: int) -> List[int]:
        with self._lock:
            if n > len(self._free):
                raise MemoryError(f"OOM: {n} blocks wanted, {len(self._free)} free")      # block_manager.py:22-23
            return [self._free.pop() for _ in range(n)]

    def try_allocate(self, n: int) -> Optional[List[int]]:
        with self._lock:
            if n > len(self._free):
                return None
            return [self._free.pop() for _ in range(n)]

    def free(self, ids: Sequence[int]) -> None:
        with self._lock:
            self._free.extend(int(i) for i in ids)


class SlotTable:
    """Host mirror of a decode worker's slots.

    A slot is one row of the device-resident batch state (block-table row, position of the token being fed,
    ``seq_len = position + 1``, an ``active`` flag).  The device advances active rows by one per step on its own;
    this mirror advances in the same way, so it always knows the device's values without reading them back, and
    only rows that change hands are uploaded."""

    def __init__(self, capacity: int, max_blocks_per_seq: int, block_size: int):
        self.capacity, self.max_blocks, self.block_size = capacity, max_blocks_per_seq, block_size
        self.tables = np.zeros((capacity, max_blocks_per_seq), dtype=np.int32)
        self.positions = np.zeros(capacity, dtype=np.int32)
        self.seq_lens = np.zeros(capacity, dtype=np.int32)
        self.active = np.zeros(capacity, dtype=np.int32)
        self.steps_left = np.zeros(capacity, dtype=np.int64)
        self.owner: List[object] = [None] * capacity
        self._free = list(range(capacity - 1, -1, -1))
        self.dirty_rows: set = set()        # table rows to upload
        self.dirty_state = False            # positions / seq_lens / active to upload

    @property
    def num_active(self) -> int:
        return self.capacity - len(self._free)

    @property
    def has_free_slot(self) -> bool:
        return bool(self._free)

    def admit(self, owner, block_table: Sequence[int], context_len: int, decode_steps: int) -> int:
        """A request with ``context_len`` tokens in the pages; its next token is fed at position ``context_len``
        and ``decode_steps`` steps follow.  The table must have room for all of them."""
        if not self._free:
            raise RuntimeError("no free decode slot")
        if decode_steps < 1:
            raise ValueError("a slot is for requests with at least one decode step")
        if len(block_table) > self.max_blocks:
            raise ValueError("block table longer than the slot's row")
        if len(block_table) * self.block_size < context_len + decode_steps:
            raise ValueError("block table too short for the tokens to come")
        slot = self._free.pop()
        self.tables[slot] = 0
        self.tables[slot, :len(block_table)] = np.asarray(block_table, dtype=np.int32)
        self.positions[slot] = context_len
        self.seq_lens[slot] = context_len + 1
        self.active[slot] = 1
        self.steps_left[slot] = decode_steps
        self.owner[slot] = owner
        self.dirty_rows.add(slot)
        self.dirty_state = True
        return slot

    def advance(self) -> List[int]:
        """What one step does to the device state; returns the slots whose last step this was."""
        self.positions += self.active
        self.seq_lens += self.active
        self.steps_left -= self.active
        return [int(s) for s in np.nonzero((self.active == 1) & (self.steps_left <= 0))[0]]

    def retire(self, slot: int):
        owner = self.owner[slot]
        self.owner[slot] = None
        self.tables[slot] = 0               # back to the parking block
        self.positions[slot] = self.seq_lens[slot] = self.active[slot] = 0
        self.steps_left[slot] = 0
        self._free.append(slot)
        self.dirty_rows.add(slot)
        self.dirty_state = True
        return owner


@dataclass
class Request:
    """One request of a synthetic workload: prompt token ids and the number of output tokens it will produce
    (the first comes from the prefill, the others from decode steps)."""
    rid: int
    prompt: torch.Tensor                  # int64 [n] on the host (pinned when it is to be copied asynchronously)
    output_len: int
    arrival: float = 0.0                  # seconds after the start of the run
    # filled in as the request moves
    prefilled: int = 0                    # prompt tokens whose K/V are in the pages (chunked prefill)
    src_blocks: Optional[List[int]] = None
    dst_blocks: Optional[List[int]] = None
    decode_worker: Optional["DecodeWorker"] = None
    prefill_worker: Optional["PrefillWorker"] = None
    stats: Dict[str, float] = field(default_factory=dict)

    @property
    def prompt_len(self) -> int:
        return int(self.prompt.numel())

    @property
    def decode_steps(self) -> int:
        return max(0, self.output_len - 1)


def plan_prefill_step(waiting: Sequence[Request], token_budget: int, max_chunk: int = 0) -> List[Tuple[Request, int, int]]:
    """Which prompt tokens the next prefill step computes: requests in arrival order, each contributing its next
    ``min(remaining, max_chunk or remaining)`` tokens, until ``token_budget`` tokens are planned (the first chunk
    is always taken, whatever its size).  Returns ``(request, start_position, num_tokens)`` triples — several per
    step, where the reference's scheduler takes one (nanoPD/engine/scheduler.py:70-101)."""
    plan, used = [], 0
    for req in waiting:
        left = req.prompt_len - req.prefilled
        if left <= 0:
            continue
        n = min(left, max_chunk) if max_chunk > 0 else left
        if plan and used + n > token_budget:
            n = token_budget - used
            if n <= 0:
                break
        plan.append((req, req.prefilled, n))
        used += n
        if used >= token_budget:
            break
    return plan


# ---------------------------------------------------------------------------------------------------------------
# Hand-off
# ---------------------------------------------------------------------------------------------------------------
@dataclass
class Handoff:
    """What the prefill side gives the decode side for one request: the reference's tuple
    ``(first_token, block_table, buf, k_cache, v_cache)`` (nanoPD/workers/prefill_worker.py:92-112) without the
    pinned buffer, plus the event behind the prompt's last store and a way to give the source blocks back."""
    request: Request
    first_token: torch.Tensor             # int64 [1] on the prefill GPU (never read by the host)
    block_table: List[int]                # source block ids
    k_cache: torch.Tensor
    v_cache: torch.Tensor
    ready: torch.cuda.Event               # the pages are complete on the prefill GPU
    release: Callable[[], None]           # returns the source blocks to the prefill GPU's pool
    pulled_layerwise: bool = False        # the decode side has already been told to pull every layer


class PrefillWorker:
    """Computes prompts on one GPU and hands their pages over (nanoPD/workers/prefill_worker.py:13-118)."""

    def __init__(self, model, num_blocks: int, block_size: int = 16, top_k: int = 10, seed: int = 0):
        s = model.shape
        self.model, self.device, self.block_size, self.top_k = model, model.device, block_size, top_k
        self.k_cache = torch.zeros(s.num_layers, num_blocks, s.num_kv_heads, block_size, s.head_dim,
                                   dtype=model.dtype, device=self.device)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.pool = BlockPool(num_blocks)
        self.stream = torch.cuda.Stream(device=self.device)
        self.generator = torch.Generator(device=self.device)
        self.generator.manual_seed(seed)
        self._busy = False
        self.keep_blocks = False            # verification runs: source blocks are not reused after the hand-off

    def blocks_for(self, prompt_len: int) -> int:
        return (prompt_len + self.block_size - 1) // self.block_size

    def prefill_batch(self, requests: Sequence[Request], after_layer=None):
        """All prompts packed into one forward (prefill_worker.py:29-89).  Returns the first tokens (int64
        ``[len(requests)]`` on the device) and the block tables; nothing waits for the GPU."""
        self._busy = True
        try:
            prefills, tables = [], []
            for req in requests:
                table = self.pool.allocate(self.blocks_for(req.prompt_len))     # MemoryError when full
                req.src_blocks = table
                tables.append(table)
                prefills.append({"block_table": table, "start_position": 0, "num_tokens": req.prompt_len})
            total = sum(r.prompt_len for r in requests)
            ctx = {"num_prefill_tokens": total, "num_decode_tokens": 0, "prefills": prefills, "decodes": []}
            with torch.cuda.device(self.device), torch.cuda.stream(self.stream):
                ids = torch.cat([r.prompt for r in requests]) if len(requests) > 1 else requests[0].prompt
                ids = ids.to(self.device, non_blocking=True)
                logits = self.model.mixed_step(ctx, ids, self.k_cache, self.v_cache, after_layer=after_layer)
                uniforms = None
                if self.top_k > 1:
                    uniforms = torch.rand(len(requests), dtype=torch.float32, device=self.device, generator=self.generator)
                first = sampling.top_k_sample(logits, self.top_k, uniforms=uniforms)
            return first, tables
        finally:
            self._busy = False

    def prefill_batch_and_extract(self, requests: Sequence[Request], layerwise_to=None) -> List[Handoff]:
        """Prefill, then one hand-off per request (prefill_worker.py:92-112), with no copy to host memory and no
        synchronise: ``Handoff.ready`` is recorded on this worker's stream behind the last store.

        ``layerwise_to`` — a callable ``(request, layer, event)`` — is invoked for every request after every
        layer's store has been issued, with an event recorded at that point: the decode side uses it to pull
        that layer's pages while the later layers still compute."""
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record(self.stream)
        hook = None
        if layerwise_to is not None:
            def hook(layer):
                ev = torch.cuda.Event()
                ev.record(self.stream)
                for req in requests:
                    layerwise_to(req, layer, ev)
        first, tables = self.prefill_batch(requests, after_layer=hook)
        t1.record(self.stream)
        ready = torch.cuda.Event()
        ready.record(self.stream)
        out = []
        for i, (req, table) in enumerate(zip(requests, tables)):
            req.prefilled = req.prompt_len
            req.stats["_prefill_events"] = (t0, t1)
            req.stats["prefill_batch_tokens"] = sum(r.prompt_len for r in requests)
            out.append(Handoff(req, first[i:i + 1], table, self.k_cache, self.v_cache, ready,
                               release=(lambda: None) if self.keep_blocks else (lambda t=table: self.pool.free(t)),
                               pulled_layerwise=layerwise_to is not None))
        return out


class DecodeSlots:
    """The device side of ``SlotTable``: the slot tensors a ``SyntheticDecoder`` steps over, and their upload."""

    def __init__(self, model, k_cache, v_cache, capacity: int, max_blocks_per_seq: int, block_size: int):
        self.model, self.device = model, model.device
        self.table = SlotTable(capacity, max_blocks_per_seq, block_size)
        dev = self.device
        zeros = torch.zeros(capacity, dtype=torch.int32, device=dev)
        model.attach_batch(k_cache, v_cache, torch.zeros(capacity, max_blocks_per_seq, dtype=torch.int32, device=dev),
                           zeros, torch.zeros(capacity, dtype=torch.int64, device=dev), active=zeros.clone())
        model.capture()                     # all slots idle: the recorded step works for any later occupancy

    def flush(self) -> None:
        """Uploads what changed since the last step (on the current stream, from pinned snapshots)."""
        t, m = self.table, self.model
        if t.dirty_rows:
            rows = sorted(t.dirty_rows)
            snap = torch.from_numpy(t.tables[rows].copy()).pin_memory()
            idx = torch.tensor(rows, dtype=torch.int64).pin_memory().to(self.device, non_blocking=True)
            m.block_tables.index_copy_(0, idx, snap.to(self.device, non_blocking=True))
            t.dirty_rows.clear()
        if t.dirty_state:
            state = torch.from_numpy(np.stack([t.positions, t.seq_lens, t.active])).pin_memory().to(self.device, non_blocking=True)
            m.positions.copy_(state[0])
            m.seq_lens.copy_(state[1])
            m.active.copy_(state[2])
            t.dirty_state = False


class DecodeWorker:
    """Receives pages and decodes on one GPU (nanoPD/workers/decode_worker.py:19-126)."""

    def __init__(self, model, num_blocks: int, capacity: int = 32, max_context: int = 16384 + 128,
                 block_size: int = 16, migrate_ctas: int = 0):
        s = model.shape
        self.model, self.device, self.block_size = model, model.device, block_size
        self.k_cache = torch.zeros(s.num_layers, num_blocks, s.num_kv_heads, block_size, s.head_dim,
                                   dtype=model.dtype, device=self.device)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.pool = BlockPool(num_blocks)
        self.compute_stream = torch.cuda.Stream(device=self.device)
        self.migrate_ctas = migrate_ctas
        # One transfer stream (and one marker stream) per SOURCE GPU: a stream runs its waits in order, so pulls
        # from two prefill GPUs on one stream would hold each other up behind events of the slower prompt.
        self._streams: Dict[int, Tuple[torch.cuda.Stream, torch.cuda.Stream]] = {}
        self._pending: List[Tuple[Handoff, torch.cuda.Event]] = []
        max_blocks = (max_context + block_size - 1) // block_size
        with torch.cuda.device(self.device), torch.cuda.stream(self.compute_stream):
            self.slots = DecodeSlots(model, self.k_cache, self.v_cache, capacity, max_blocks, block_size)
        self.compute_stream.synchronize()
        self._lock = threading.Lock()       # prefill threads call receive_*; the decode thread calls step
        self._reserved_slots = 0
        self._layer_lists: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        self.finished: List[Request] = []
        self.step_events: List[Tuple[torch.cuda.Event, torch.cuda.Event, bool, int]] = []
        self.record_steps = False
        # verification runs: keep finished requests' blocks, and copy every step's tokens to pinned host memory
        self.keep_blocks = False
        self.record_tokens = False
        self._inflight: Deque[torch.cuda.Event] = deque()      # events behind the last few steps (host pacing)

    # ---- admission control: a request reserves its blocks and a slot before its prefill starts ----
    def blocks_for(self, req: Request) -> int:
        return (req.prompt_len + req.decode_steps + self.block_size - 1) // self.block_size

    def try_reserve(self, req: Request) -> bool:
        with self._lock:
            if self.slots.table.num_active + self._reserved_slots >= self.slots.table.capacity:
                return False
            blocks = self.pool.try_allocate(self.blocks_for(req))
            if blocks is None:
                return False
            self._reserved_slots += 1
            req.dst_blocks, req.decode_worker = blocks, self
            return True

    def _streams_for(self, src_device: torch.device) -> Tuple[torch.cuda.Stream, torch.cuda.Stream]:
        pair = self._streams.get(src_device.index)
        if pair is None:
            pair = self._streams[src_device.index] = (torch.cuda.Stream(device=self.device),
                                                      torch.cuda.Stream(device=self.device))
        return pair

    @property
    def num_pending(self) -> int:
        return len(self._pending)

    # ---- receiving ----
    def receive_kv_async(self, handoff: Handoff) -> str:
        """Pulls the request's pages into this GPU's pool at the ids reserved for it and queues it for promotion
        (decode_worker.py:39-59).  Returns at once; the transfer waits for ``handoff.ready`` on the GPU."""
        req = handoff.request
        n = len(handoff.block_table)
        with self._lock, torch.cuda.device(self.device):
            transfer_stream, marker_stream = self._streams_for(handoff.k_cache.device)
            e_ready, e0, e1 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            marker_stream.wait_event(handoff.ready)
            e_ready.record(marker_stream)                          # when the prompt was done, on this GPU's clock
            if handoff.pulled_layerwise:
                # every layer has been queued on the transfer stream already; only completion is left to mark
                self._layer_lists.pop(req.rid, None)
                path = "p2p"
                e0 = req.stats.get("_first_layer_event", e0)
            else:
                transfer_stream.wait_event(handoff.ready)
                e0.record(transfer_stream)
                path = kv_transfer.transfer_kv(handoff.k_cache, handoff.v_cache, self.k_cache, self.v_cache,
                                               handoff.block_table, stream=transfer_stream,
                                               dst_block_table=req.dst_blocks[:n], max_ctas=self.migrate_ctas)
            e1.record(transfer_stream)
            transfer_stream.wait_event(handoff.ready)              # the first token is sampled after the last store
            done = torch.cuda.Event()
            done.record(transfer_stream)
            req.stats["_transfer_events"] = (e_ready, e0, e1)
            req.stats["migrated_bytes"] = kv_transfer.migration_bytes(n, self.k_cache)
            self._pending.append((handoff, done))
        return path

    def receive_layer(self, req: Request, layer: int, after: torch.cuda.Event) -> None:
        """Layer-wise variant: pull layer ``layer`` of the request's pages once ``after`` (recorded on the prefill
        GPU behind that layer's store) has completed.  Called by the prefill thread, layer by layer."""
        worker = req.prefill_worker
        n = len(req.src_blocks)
        transfer_stream, _ = self._streams_for(worker.device)
        with self._lock, torch.cuda.device(self.device), torch.cuda.stream(transfer_stream):
            lists = self._layer_lists.get(req.rid)
            if lists is None:
                src = torch.tensor(req.src_blocks, dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
                dst = torch.tensor(req.dst_blocks[:n], dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
                lists = self._layer_lists[req.rid] = (src, dst)
            transfer_stream.wait_event(after)
            if layer == 0:
                e0 = torch.cuda.Event(enable_timing=True)
                e0.record(transfer_stream)
                req.stats["_first_layer_event"] = e0
            kv_transfer.transfer_kv(worker.k_cache[layer:layer + 1], worker.v_cache[layer:layer + 1],
                                    self.k_cache[layer:layer + 1], self.v_cache[layer:layer + 1], lists[0],
                                    stream=transfer_stream, dst_block_table=lists[1], max_ctas=self.migrate_ctas)

    def _promote_ready(self) -> int:
        """Requests whose pages have arrived move into slots (decode_worker.py:61-68); no host wait."""
        ready, still = [], []
        with self._lock:
            for handoff, event in self._pending:
                if event.query():
                    self.compute_stream.wait_event(event)        # kernels launched from now on see the pages
                    ready.append(handoff)
                else:
                    still.append((handoff, event))
            self._pending = still
        for handoff in ready:
            req = handoff.request
            handoff.release()                                     # the prefill GPU may reuse the source blocks
            req.stats["t_first_token"] = time.perf_counter()
            with self._lock:                                      # the reservation becomes a slot in one step
                self._reserved_slots -= 1
                slot = (self.slots.table.admit(req, req.dst_blocks, req.prompt_len, req.decode_steps)
                        if req.decode_steps > 0 else None)
            if slot is None:
                self._finish(req)
                continue
            self.model.token_ids[slot:slot + 1].copy_(handoff.first_token, non_blocking=True)
            if self.record_tokens:
                first = torch.empty(1, dtype=torch.int64, pin_memory=True)
                first.copy_(self.model.token_ids[slot:slot + 1], non_blocking=True)
                req.stats["_tokens"] = [first]
        return len(ready)

    def _finish(self, req: Request) -> None:
        req.stats["t_done"] = time.perf_counter()
        if not self.keep_blocks:
            self.pool.free(req.dst_blocks)
        self.finished.append(req)

    def step(self) -> List[Request]:
        """One decode step for every running request (decode_worker.py:70-126).  Returns the requests that
        finished with it."""
        with torch.cuda.device(self.device), torch.cuda.stream(self.compute_stream):
            self._promote_ready()
            self.slots.flush()              # also when the last request has just left: the slots go back to parked
            if self.slots.table.num_active == 0:
                return []
            if self.record_steps:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(self.compute_stream)
            self.model.replay()
            if self.record_steps:
                b.record(self.compute_stream)
                self.step_events.append((a, b, self.num_pending > 0, self.slots.table.num_active))
            if self.record_tokens:
                toks = torch.empty(self.slots.table.capacity, dtype=torch.int64, pin_memory=True)
                toks.copy_(self.model.token_ids, non_blocking=True)
                for slot, owner in enumerate(self.slots.table.owner):
                    if owner is not None:
                        owner.stats["_tokens"].append(toks[slot:slot + 1])
            done = []
            for slot in self.slots.table.advance():
                req = self.slots.table.retire(slot)
                self._finish(req)
                done.append(req)
            # Pace the host: at most a few steps queued ahead, so that admissions take effect promptly
            self._pace()
            return done

    def park(self) -> None:
        """Uploads pending slot changes (after the last request has left, this parks every slot again)."""
        with torch.cuda.device(self.device), torch.cuda.stream(self.compute_stream):
            self.slots.flush()

    def _pace(self, ahead: int = 2) -> None:
        ev = torch.cuda.Event()
        ev.record(self.compute_stream)
        self._inflight.append(ev)
        while len(self._inflight) > ahead:
            self._inflight.popleft().synchronize()

    @property
    def idle(self) -> bool:
        return self.slots.table.num_active == 0 and self.num_pending == 0 and self._reserved_slots == 0


# ---------------------------------------------------------------------------------------------------------------
# Disaggregated serving: prefill GPUs feed decode GPUs
# ---------------------------------------------------------------------------------------------------------------
class DisaggregatedScheduler:
    """Prefill workers and decode workers in one process, one thread per worker, as the reference's
    ``CentralScheduler`` drives its disaggregated path (nanoPD/router/central_scheduler.py:128-135, 202-340):
    waiting requests are given to the first free prefill worker, their pages are handed to a decode worker, which
    promotes them into its running batch while it steps.  A request reserves its destination blocks and slot on
    the decode worker with the most free blocks BEFORE its prefill starts, so a finished prompt never waits for
    room (the reference re-queues on shortage, central_scheduler.py:244-259)."""

    def __init__(self, prefill_workers: Sequence[PrefillWorker], decode_workers: Sequence[DecodeWorker],
                 token_budget: int = 16384, layerwise: bool = False):
        self.prefill_workers, self.decode_workers = list(prefill_workers), list(decode_workers)
        self.token_budget, self.layerwise = token_budget, layerwise
        self._waiting: Deque[Request] = deque()
        self._lock = threading.Lock()
        self._errors: List[BaseException] = []
        self._total = 0
        self._t0 = 0.0

    def add_request(self, req: Request) -> None:
        self._waiting.append(req)
        self._total += 1

    def _take_batch(self, pw: PrefillWorker) -> List[Request]:
        """Requests for one prefill forward: in arrival order, within the token budget, each with room reserved on
        a decode worker and in this worker's pool."""
        batch, used, blocks = [], 0, 0
        now = time.perf_counter() - self._t0
        with self._lock:
            while self._waiting:
                req = self._waiting[0]
                if req.arrival > now:
                    break
                if batch and used + req.prompt_len > self.token_budget:
                    break
                if blocks + pw.blocks_for(req.prompt_len) > pw.pool.num_free:
                    break
                target = max(self.decode_workers, key=lambda d: d.pool.num_free)
                if not target.try_reserve(req):
                    others = [d for d in self.decode_workers if d is not target]
                    if not any(d.try_reserve(req) for d in sorted(others, key=lambda d: -d.pool.num_free)):
                        break
                self._waiting.popleft()
                batch.append(req)
                used += req.prompt_len
                blocks += pw.blocks_for(req.prompt_len)
        return batch

    def _prefill_loop(self, pw: PrefillWorker) -> None:
        try:
            torch.cuda.set_device(pw.device)
            while True:
                batch = self._take_batch(pw)
                if not batch:
                    with self._lock:
                        if not self._waiting:
                            return
                    time.sleep(0.0005)
                    continue
                for req in batch:
                    req.stats["t_prefill_start"] = time.perf_counter()
                    req.prefill_worker = pw
                hook = (lambda req, layer, ev: req.decode_worker.receive_layer(req, layer, ev)) if self.layerwise else None
                for handoff in pw.prefill_batch_and_extract(batch, layerwise_to=hook):
                    handoff.request.decode_worker.receive_kv_async(handoff)
        except BaseException as exc:  # noqa: BLE001
            self._errors.append(exc)

    def _decode_loop(self, dw: DecodeWorker, stop: threading.Event) -> None:
        try:
            torch.cuda.set_device(dw.device)
            while not stop.is_set():
                dw.step()
                if dw.slots.table.num_active == 0:
                    time.sleep(0.0002)
        except BaseException as exc:  # noqa: BLE001
            self._errors.append(exc)

    def run_until_done(self, timeout: float = 600.0) -> List[Request]:
        """Serves every added request; returns them with their ``stats`` filled in (times in seconds since the
        start; ``prefill_ms``, ``transfer_ms`` and ``exposed_transfer_ms`` from CUDA events)."""
        stop = threading.Event()
        for d in self.decode_workers:
            d.finished = []
        self._t0 = time.perf_counter()
        threads = [threading.Thread(target=self._prefill_loop, args=(pw,), daemon=True) for pw in self.prefill_workers]
        threads += [threading.Thread(target=self._decode_loop, args=(dw, stop), daemon=True) for dw in self.decode_workers]
        for t in threads:
            t.start()
        deadline = time.perf_counter() + timeout
        while time.perf_counter() < deadline and not self._errors:
            if sum(len(d.finished) for d in self.decode_workers) >= self._total:
                break
            time.sleep(0.002)
        stop.set()
        for t in threads:
            t.join(timeout=30)
        for d in self.decode_workers:
            if hasattr(d, "park"):
                d.park()
        for w in list(self.prefill_workers) + list(self.decode_workers):
            torch.cuda.synchronize(w.device)
        if self._errors:
            raise self._errors[0]
        done = [r for d in self.decode_workers for r in d.finished]
        if len(done) < self._total:
            raise RuntimeError(f"only {len(done)} of {self._total} requests finished within {timeout} s")
        for req in done:
            finalize_stats(req, self._t0)
        return done


def finalize_stats(req: Request, t0: float) -> None:
    """Turns the CUDA events a request collected into milliseconds and drops the event objects."""
    st = req.stats
    ev = st.pop("_prefill_events", None)
    if ev is not None:
        st["prefill_ms"] = ev[0].elapsed_time(ev[1])
    ev = st.pop("_transfer_events", None)
    if ev is not None:
        e_ready, e0, e1 = ev
        st["transfer_ms"] = e0.elapsed_time(e1)                    # first byte requested .. last byte landed
        st["exposed_transfer_ms"] = max(0.0, e_ready.elapsed_time(e1))   # prompt finished .. pages complete
    st.pop("_first_layer_event", None)
    for key in ("t_prefill_start", "t_first_token", "t_done"):
        if key in st:
            st[key] -= t0


# ---------------------------------------------------------------------------------------------------------------
# Collocated serving: prefill chunks and decode steps on one GPU, continuous batching
# ---------------------------------------------------------------------------------------------------------------
class CollocatedWorker:
    """One GPU that prefills and decodes (the reference's ``CollocatedWorker`` around ``Engine.step``,
    nanoPD/workers/collocated_worker.py:14-15, nanoPD/engine/engine.py:42-113).  Every step first computes the
    prompt chunks planned by ``plan_prefill_step`` (several prompts and chunks per step, within ``token_budget``),
    eagerly, then replays the captured decode step over the slots.  Requests enter the slots when their last chunk
    is done and leave when their output is complete; both happen between replays, by rewriting slot rows."""

    def __init__(self, model, num_blocks: int, capacity: int = 256, max_context: int = 4096 + 1024,
                 block_size: int = 16, token_budget: int = 4096, max_chunk: int = 2048, top_k: int = 10, seed: int = 0):
        s = model.shape
        self.model, self.device, self.block_size = model, model.device, block_size
        self.token_budget, self.max_chunk, self.top_k = token_budget, max_chunk, top_k
        self.k_cache = torch.zeros(s.num_layers, num_blocks, s.num_kv_heads, block_size, s.head_dim,
                                   dtype=model.dtype, device=self.device)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.pool = BlockPool(num_blocks)
        self.stream = torch.cuda.Stream(device=self.device)
        max_blocks = (max_context + block_size - 1) // block_size
        with torch.cuda.device(self.device), torch.cuda.stream(self.stream):
            self.slots = DecodeSlots(model, self.k_cache, self.v_cache, capacity, max_blocks, block_size)
        self.stream.synchronize()
        self.generator = torch.Generator(device=self.device)
        self.generator.manual_seed(seed)
        self.waiting: Deque[Request] = deque()       # arrived, prompt not fully prefilled
        self.finished: List[Request] = []
        self.decode_tokens = 0
        self.prefill_tokens = 0

    def add_request(self, req: Request) -> None:
        self.waiting.append(req)

    def _admit_blocks(self) -> List[Request]:
        """Requests at the head of the queue that may start (blocks for prompt + output and a slot in sight)."""
        started = []
        free_slots = self.slots.table.capacity - self.slots.table.num_active - sum(1 for r in self.waiting if r.dst_blocks)
        for req in self.waiting:
            if req.dst_blocks is not None:
                continue
            if free_slots <= 0:
                break
            need = (req.prompt_len + req.decode_steps + self.block_size - 1) // self.block_size
            blocks = self.pool.try_allocate(need)
            if blocks is None:
                break
            req.dst_blocks = blocks
            free_slots -= 1
            started.append(req)
        return started

    def step(self) -> List[Request]:
        """One scheduler step; returns the requests that finished with it."""
        now = time.perf_counter()
        done: List[Request] = []
        with torch.cuda.device(self.device), torch.cuda.stream(self.stream):
            self._admit_blocks()
            plan = plan_prefill_step([r for r in self.waiting if r.dst_blocks is not None], self.token_budget, self.max_chunk)
            if plan:
                prefills, ids = [], []
                for req, start, n in plan:
                    req.stats.setdefault("t_prefill_start", now)
                    prefills.append({"block_table": req.dst_blocks, "start_position": start, "num_tokens": n})
                    ids.append(req.prompt[start:start + n])
                total = sum(n for _, _, n in plan)
                ctx = {"num_prefill_tokens": total, "num_decode_tokens": 0, "prefills": prefills, "decodes": []}
                tok = (torch.cat(ids) if len(ids) > 1 else ids[0]).to(self.device, non_blocking=True)
                logits = self.model.mixed_step(ctx, tok, self.k_cache, self.v_cache)
                uniforms = None
                if self.top_k > 1:
                    uniforms = torch.rand(len(plan), dtype=torch.float32, device=self.device, generator=self.generator)
                first = sampling.top_k_sample(logits, self.top_k, uniforms=uniforms)
                self.prefill_tokens += total
                for i, (req, start, n) in enumerate(plan):
                    req.prefilled = start + n
                    if req.prefilled < req.prompt_len:
                        continue
                    self.waiting.remove(req)
                    ev = torch.cuda.Event()
                    ev.record(self.stream)
                    req.stats["_first_token_event"] = ev
                    if req.decode_steps == 0:
                        self._finish(req)
                        done.append(req)
                        continue
                    slot = self.slots.table.admit(req, req.dst_blocks, req.prompt_len, req.decode_steps)
                    self.model.token_ids[slot:slot + 1].copy_(first[i:i + 1])
            if self.slots.table.num_active:
                self.slots.flush()
                self.model.replay()
                self.decode_tokens += self.slots.table.num_active
                for slot in self.slots.table.advance():
                    req = self.slots.table.retire(slot)
                    self._finish(req)
                    done.append(req)
        return done

    def _finish(self, req: Request) -> None:
        ev = torch.cuda.Event()
        ev.record(self.stream)
        req.stats["_done_event"] = ev
        self.pool.free(req.dst_blocks)
        self.finished.append(req)

    @property
    def idle(self) -> bool:
        return not self.waiting and self.slots.table.num_active == 0


def serve_open_loop(worker: CollocatedWorker, requests: Sequence[Request], drain_timeout: float = 120.0) -> Dict[str, float]:
    """Feeds ``requests`` to ``worker`` at their arrival times (an open loop: arrivals do not wait for the server,
    as in the reference's Poisson benchmark, nanoPD/benchmark/benchmark_poisson.py:108-147) and steps it until all
    have finished.  Completion times are taken from CUDA events by a watcher that polls them between steps, so the
    serving loop itself never waits for the GPU except to keep at most two steps queued."""
    pending = deque(sorted(requests, key=lambda r: r.arrival))
    inflight: Deque[torch.cuda.Event] = deque()
    watch: List[Request] = []
    t0 = time.perf_counter()
    first_done: Dict[int, float] = {}
    all_done: Dict[int, float] = {}

    def poll():
        now = time.perf_counter() - t0
        for req in list(watch):
            ev = req.stats.get("_first_token_event")
            if ev is not None and req.rid not in first_done and ev.query():
                first_done[req.rid] = now
            ev = req.stats.get("_done_event")
            if ev is not None and ev.query():
                all_done[req.rid] = now
                first_done.setdefault(req.rid, now)
                watch.remove(req)

    total = len(pending)
    deadline = None
    while len(all_done) < total:
        now = time.perf_counter() - t0
        while pending and pending[0].arrival <= now:
            req = pending.popleft()
            worker.add_request(req)
            watch.append(req)
        if worker.idle:
            poll()
            if pending:
                time.sleep(min(0.001, max(0.0, pending[0].arrival - now)))
            elif len(all_done) < total:
                time.sleep(0.0005)
            continue
        worker.step()
        ev = torch.cuda.Event()
        ev.record(worker.stream)
        inflight.append(ev)
        while len(inflight) > 2:
            inflight.popleft().synchronize()
        poll()
        if not pending and deadline is None:
            deadline = time.perf_counter() + drain_timeout
        if deadline is not None and time.perf_counter() > deadline:
            break
    torch.cuda.synchronize(worker.device)
    poll()
    wall = time.perf_counter() - t0
    for req in requests:
        req.stats.pop("_first_token_event", None)
        req.stats.pop("_done_event", None)
        if req.rid in all_done:
            req.stats["ttft_s"] = first_done[req.rid] - req.arrival
            req.stats["latency_s"] = all_done[req.rid] - req.arrival
            if req.decode_steps > 0:
                req.stats["tpot_s"] = (all_done[req.rid] - first_done[req.rid]) / req.decode_steps
    return {"wall_s": wall, "finished": len(all_done), "submitted": total}
