"""Prefill -> decode KV page migration with the reference's ``transfer_kv`` signature.

The reference copies a request's pages block by block with ``Tensor.copy_`` when the two
GPUs can reach each other, and relays through a pinned host buffer otherwise
(nanoPD/workers/kv_transfer.py:69-83).  On an NVSwitch box every GPU reaches every peer, so
this module keeps only the direct path and does it in ONE kernel launch per request
(``paged_kv_migrate``) instead of two ``copy_`` calls per block.

The kernel runs on the destination GPU's stream (the ``transfer_stream`` that
``DecodeWorker.receive_kv_async`` passes, nanoPD/workers/decode_worker.py:47-58) and pulls
the pages over NVLink with plain loads; completion is the CUDA event the caller records on
that stream afterwards, exactly as in the reference.
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


def transfer_kv(src_k, src_v, dst_k, dst_v, block_table: Sequence[int], stream=None, buf=None,
                dst_block_table: Optional[Sequence[int]] = None, max_ctas: int = 0) -> str:
    """Copy blocks ``block_table`` of the 5-D pools ``src_*`` into ``dst_*``; returns ``"p2p"``.

    Pools are ``[layers, blocks, Hkv, B, D]``.  ``dst_block_table`` (an addition) lets the
    decode replica place the pages at ids of its own allocator; by default the ids are
    equal on both sides as in the reference, which shares one BlockSpaceManager
    (nanoPD/router/central_scheduler.py:99-117).  ``buf`` is accepted for signature
    compatibility and ignored: there is no pinned-host relay here, and a pair of GPUs
    without peer access raises RuntimeError instead of silently taking a slower path.
    Also works when both pools live on one GPU (a plain device-to-device gather).
    """
    src_device, dst_device = src_k.device, dst_k.device
    if src_device != dst_device and not _check_p2p(src_device, dst_device):
        raise RuntimeError(f"no peer access from {dst_device} to {src_device}: page migration needs NVLink/P2P")
    if max_ctas == 0:
        # 64 single-warp CTAs fill an NVLink; a pool-to-pool copy inside one GPU has 3x the bandwidth to fill
        max_ctas = 64 if src_device != dst_device else 96
    ctx = torch.cuda.stream(stream) if stream is not None else nullcontext()
    with torch.cuda.device(dst_device), ctx:
        if src_device != dst_device:
            paged_kernels.enable_peer_access(src_device.index)
        paged_kernels.paged_kv_migrate(src_k, src_v, dst_k, dst_v, list(block_table),
                                       None if dst_block_table is None else list(dst_block_table),
                                       max_ctas=max_ctas)
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

    def receive_kv_async(self, group, block_table: Sequence[int], buf=None, src_k: torch.Tensor = None,
                         src_v: torch.Tensor = None, dst_block_table: Optional[Sequence[int]] = None) -> str:
        """Starts pulling ``block_table`` of ``src_k`` / ``src_v`` into this replica's pools and returns the path
        taken (always ``"p2p"``).  The source pages must already be complete on the stream that is current on the
        destination device (the transfer stream waits for it), as after the prefill worker's synchronise."""
        self.transfer_stream.wait_stream(torch.cuda.current_stream(self.device))
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
