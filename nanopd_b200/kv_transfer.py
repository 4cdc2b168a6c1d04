"""Prefill -> decode KV page migration: a drop-in for the reference's ``workers/kv_transfer`` module.

Same names as there (nanoPD/workers/kv_transfer.py:6-83): ``_check_p2p``, ``PinnedKVBuffer``,
``extract_kv_to_pinned``, ``load_kv_from_pinned``, ``transfer_kv`` — the names the reference's workers import
at module load (workers/prefill_worker.py:10, workers/decode_worker.py:11).

The reference copies a request's pages block by block with ``Tensor.copy_`` — two calls per block, each a
strided copy of ``[layers]`` chunks — when the two GPUs can reach each other, and relays through a pinned host
buffer otherwise.  Here every one of those loops is ONE kernel launch (``paged_kv_migrate``): the kernel walks
all (block, layer, K|V) units itself.  Between two GPUs it runs on the destination GPU's stream (the
``transfer_stream`` that ``DecodeWorker.receive_kv_async`` passes, workers/decode_worker.py:47-58) and pulls the
pages over NVLink; completion is the CUDA event the caller records on that stream afterwards, exactly as in the
reference.  For the pinned relay one side of the copy is the pinned buffer, which the kernel reaches over PCIe
through the unified address space.
"""
from __future__ import annotations

from contextlib import nullcontext
from typing import List, Optional, Sequence

import torch

from . import paged_kernels


def _check_p2p(src_device: torch.device, dst_device: torch.device) -> bool:
    """Same answer as the reference's probe (nanoPD/workers/kv_transfer.py:6-14)."""
    if src_device == dst_device:
        return False
    if src_device.type != "cuda" or dst_device.type != "cuda":
        return False
    try:
        return torch.cuda.can_device_access_peer(dst_device.index, src_device.index)
    except Exception:
        return False


class PinnedKVBuffer:
    """Pinned host staging for one request's pages, ``k`` and ``v`` of shape
    ``[num_layers, num_block, num_kv_heads, block_size, head_dim]`` (nanoPD/workers/kv_transfer.py:17-41; same
    constructor arguments, same two attributes)."""

    def __init__(self, num_layers: int, num_block: int, num_kv_heads: int, block_size: int, head_dim: int,
                 dtype=torch.float16):
        shape = (num_layers, num_block, num_kv_heads, block_size, head_dim)
        self.k = torch.empty(shape, dtype=dtype, pin_memory=True)
        self.v = torch.empty(shape, dtype=dtype, pin_memory=True)

    @staticmethod
    def from_runner(runner, num_blocks: int) -> "PinnedKVBuffer":
        """Sized from a runner's pools (``runner.k_cache`` ``[L, blocks, Hkv, B, D]``, ``num_kv_heads``,
        ``block_size``, ``head_dim``).  The buffer takes the pool's dtype; the reference hard-wires float16,
        which is also the only dtype its runner allocates (nanoPD/engine/model_runner.py:24-31)."""
        return PinnedKVBuffer(num_layers=runner.k_cache.shape[0], num_block=num_blocks,
                              num_kv_heads=runner.num_kv_heads, block_size=runner.block_size,
                              head_dim=runner.head_dim, dtype=runner.k_cache.dtype)


def _relay_grid(max_ctas: int) -> int:
    # negative = the load/store kernel (the only one that touches host memory); 32 CTAs x 256 threads keep
    # about 1 MB in flight, several times what a PCIe link needs
    return -abs(max_ctas) if max_ctas else -32


def extract_kv_to_pinned(k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: Sequence[int],
                         buf: PinnedKVBuffer, stream: Optional[torch.cuda.Stream] = None, wait: bool = True,
                         max_ctas: int = 0) -> None:
    """``buf.k[:, i] = k_cache[:, block_table[i]]`` (and V) for every block of the request
    (nanoPD/workers/kv_transfer.py:44-52), as one launch on ``stream`` (default: the current stream of the
    pool's device).  The reference's copies block the host one by one; here the host waits once, after the
    launch, unless ``wait=False`` (then order later readers of ``buf`` behind the stream yourself)."""
    n = len(block_table)
    if n > buf.k.size(1):
        raise RuntimeError(f"pinned buffer holds {buf.k.size(1)} blocks, the request has {n}")
    dev = k_cache.device
    ctx = torch.cuda.stream(stream) if stream is not None else nullcontext()
    with torch.cuda.device(dev), ctx:
        paged_kernels.paged_kv_migrate(k_cache, v_cache, buf.k, buf.v, block_table, list(range(n)),
                                       max_ctas=_relay_grid(max_ctas))
        if wait:
            torch.cuda.current_stream(dev).synchronize()


def load_kv_from_pinned(k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: Sequence[int],
                        buf: PinnedKVBuffer, stream: Optional[torch.cuda.Stream] = None, max_ctas: int = 0) -> None:
    """``k_cache[:, block_table[i]] = buf.k[:, i]`` (and V) (nanoPD/workers/kv_transfer.py:55-66), one launch.
    With a ``stream`` the call is asynchronous on it, as the reference's ``non_blocking`` copies are; without one
    the host waits for the copy, as it does there."""
    n = len(block_table)
    if n > buf.k.size(1):
        raise RuntimeError(f"pinned buffer holds {buf.k.size(1)} blocks, the request has {n}")
    dev = k_cache.device
    ctx = torch.cuda.stream(stream) if stream is not None else nullcontext()
    with torch.cuda.device(dev), ctx:
        paged_kernels.paged_kv_migrate(buf.k, buf.v, k_cache, v_cache, list(range(n)), block_table,
                                       max_ctas=_relay_grid(max_ctas))
        if stream is None:
            torch.cuda.current_stream(dev).synchronize()


def transfer_kv(src_k, src_v, dst_k, dst_v, block_table, stream=None, buf=None,
                dst_block_table=None, max_ctas: int = 0) -> str:
    """Copy blocks ``block_table`` of the 5-D pools ``src_*`` into ``dst_*``; returns the path taken, ``"p2p"``
    or ``"pinned_relay"`` as the reference does (nanoPD/workers/kv_transfer.py:69-83).

    Pools are ``[layers, blocks, Hkv, B, D]``.  ``block_table`` is a list of ids or an int32 tensor on the
    destination device.  ``dst_block_table`` (an addition) lets the decode replica place the pages at ids of its
    own allocator; by default the ids are equal on both sides as in the reference, which shares one
    BlockSpaceManager (nanoPD/router/central_scheduler.py:99-117).  Two GPUs with peer access — every pair on
    an NVSwitch box — take the direct path; so do two pools on one GPU (a device-to-device gather; the reference
    would relay those through the host).  Without peer access the pages come from ``buf``, which
    ``extract_kv_to_pinned`` filled, and a missing ``buf`` raises, as the reference's assertion does.
    """
    src_device, dst_device = src_k.device, dst_k.device
    ctx = torch.cuda.stream(stream) if stream is not None else nullcontext()
    if src_device != dst_device and not _check_p2p(src_device, dst_device):
        if buf is None:
            raise RuntimeError(f"no peer access from {dst_device} to {src_device} and no pinned buffer to relay through")
        if dst_block_table is not None:
            block_table = dst_block_table
        load_kv_from_pinned(dst_k, dst_v, list(block_table) if not torch.is_tensor(block_table) else block_table.tolist(),
                            buf, stream=stream)
        return "pinned_relay"
    if max_ctas == 0:
        # 64 single-warp CTAs fill an NVLink; a pool-to-pool copy inside one GPU has 3x the bandwidth to fill
        max_ctas = 64 if src_device != dst_device else 96
    with torch.cuda.device(dst_device), ctx:
        if src_device != dst_device:
            paged_kernels.enable_peer_access(src_device.index)
        paged_kernels.paged_kv_migrate(src_k, src_v, dst_k, dst_v, block_table, dst_block_table, max_ctas=max_ctas)
    return "p2p"


class KVReceiver:
    """The receiving half of the hand-over, as ``DecodeWorker`` keeps it (``receive_kv_async`` and
    ``_promote_ready``, nanoPD/workers/decode_worker.py:36-68): transfers are issued on a stream of their own on
    the destination GPU, each followed by an event; ``promote_ready`` returns, without blocking, the requests
    whose pages have arrived, in the order they were issued.  Scheduling stays with the caller."""

    def __init__(self, dst_k: torch.Tensor, dst_v: torch.Tensor, max_ctas: int = 0):
        self.dst_k, self.dst_v = dst_k, dst_v
        self.device = dst_k.device
        self.transfer_stream = torch.cuda.Stream(device=self.device)
        self.max_ctas = max_ctas
        self._pending: List[tuple] = []

    def receive_kv_async(self, group, block_table, buf=None, src_k: torch.Tensor = None,
                         src_v: torch.Tensor = None, dst_block_table=None, after=None) -> str:
        """Starts pulling ``block_table`` of ``src_k`` / ``src_v`` into this replica's pools and returns the path
        taken.  The call only enqueues work: block lists travel through pinned memory with a non-blocking copy, so
        it returns while earlier transfers are still in flight.  The source pages must be complete either on the
        stream that is current on the destination device (the transfer stream waits for it), as after the prefill
        worker's synchronise, or at ``after`` — a CUDA event recorded on the prefill GPU behind the last store,
        which the transfer stream then waits for instead of the host."""
        self.transfer_stream.wait_stream(torch.cuda.current_stream(self.device))
        if after is not None:
            self.transfer_stream.wait_event(after)
        path = transfer_kv(src_k, src_v, self.dst_k, self.dst_v, block_table, stream=self.transfer_stream, buf=buf,
                           dst_block_table=dst_block_table, max_ctas=self.max_ctas)
        event = torch.cuda.Event()
        self.transfer_stream.record_event(event)
        self._pending.append((group, event))
        return path

    def promote_ready(self) -> list:
        """Requests whose transfer has completed since the last call (``event.query()``, no host wait).  The compute
        stream is made to wait for each completed event, so kernels launched afterwards see the pages."""
        ready, still = [], []
        for group, event in self._pending:
            if event.query():
                torch.cuda.current_stream(self.device).wait_event(event)
                ready.append(group)
            else:
                still.append((group, event))
        self._pending = still
        return ready

    @property
    def num_pending(self) -> int:
        return len(self._pending)


def migration_bytes(num_blocks: int, pool: torch.Tensor) -> int:
    """Algorithmic bytes of one request's migration: blocks x layers x 2 (K, V) x block bytes."""
    L = pool.size(0)
    block_bytes = pool[0, 0].numel() * pool.element_size()
    return num_blocks * L * 2 * block_bytes
