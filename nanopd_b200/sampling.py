"""Batched sampling of one step's tokens on the device.

The reference samples one sequence at a time — ``top_k_sample(logit, top_k=1)`` of
nanoPD/engine/model_runner.py:279-284 returns a 0-d tensor that its callers read back with
``.item()`` (nanoPD/engine/engine.py:100-106, nanoPD/workers/decode_worker.py:110,
nanoPD/workers/prefill_worker.py:79).  ``top_k_sample`` here keeps that name, argument order and
default, accepts the same 1-D ``logit`` and returns the same 0-d tensor; given the 2-D logits of a
whole step it returns one token per row from a single launch, with no host synchronisation.
The randomness is a vector of uniform numbers (drawn from ``generator`` or passed in), so a test can
reproduce a draw exactly; the reference draws from torch's global generator through ``torch.multinomial``.
"""
from __future__ import annotations

import threading
from typing import Dict, Optional, Tuple

import torch

from . import _lib

_C = _lib.load()
_DTYPE_CODE = {torch.float16: _lib.NPD_DTYPE_F16, torch.bfloat16: _lib.NPD_DTYPE_BF16,
               torch.float32: _lib.NPD_DTYPE_F32}
MAX_TOP_K = 64

# One zeroed workspace per (device, stream): the kernel leaves its arrival counters at zero, so the buffer
# is reusable by every later call on that stream; it only ever grows.
_lock = threading.Lock()
_workspaces: Dict[Tuple[int, int], torch.Tensor] = {}


def _workspace(device: torch.device, stream_handle: int, nbytes: int) -> torch.Tensor:
    key = (device.index, stream_handle)
    with _lock:
        ws = _workspaces.get(key)
        if ws is None or ws.numel() < nbytes:
            ws = torch.zeros(nbytes, dtype=torch.uint8, device=device)
            _workspaces[key] = ws
        return ws


def check_status(device=None, raise_on_error: bool = True) -> int:
    """Reads and clears the status words of the sampler's workspaces on ``device`` (synchronises).  The only bit
    the sampler raises is the wait time-out (4); the workspace is zeroed again when it is seen."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    with _lock:
        items = [w for (d, _), w in _workspaces.items() if d == idx]
    bits = 0
    for ws in items:
        word = int(ws[:4].view(torch.int32).item())
        if word:
            bits |= word
            ws.zero_()
            torch.cuda.synchronize(idx)
    if bits and raise_on_error:
        raise RuntimeError(f"nanopd_b200 sampler device status: {bits}")
    return bits


def top_k_sample(logit: torch.Tensor, top_k: int = 1, uniforms: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Token ids (int64) drawn from the ``top_k`` largest logits of every row.

    ``logit``: [V] (returns a 0-d tensor, as the reference does) or [T, V] (returns [T]); fp16, bf16 or
    fp32 on a CUDA device, last dimension contiguous.  ``uniforms``: float32 [T] in [0, 1); drawn with
    ``generator`` when absent and ``top_k > 1``.  ``out``: int64 [T] to write into."""
    if not logit.is_cuda:
        raise RuntimeError("top_k_sample: logit must be a CUDA tensor (this library has no CPU path)")
    if logit.dtype not in _DTYPE_CODE:
        raise RuntimeError(f"top_k_sample: unsupported dtype {logit.dtype}")
    single = logit.dim() == 1
    rows = logit.unsqueeze(0) if single else logit
    if rows.dim() != 2 or rows.stride(1) != 1:
        raise RuntimeError("top_k_sample: logit must be [V] or [T, V] with a contiguous last dimension")
    T, V = rows.shape
    top_k = int(top_k)
    if not 1 <= top_k <= MAX_TOP_K:
        raise RuntimeError(f"top_k_sample: top_k must be in [1, {MAX_TOP_K}]")
    if top_k > V:
        raise RuntimeError("top_k_sample: top_k exceeds the vocabulary")       # torch.topk raises here too
    dev = rows.device
    if out is None:
        out = torch.empty(T, dtype=torch.int64, device=dev)
    elif out.dtype != torch.int64 or out.numel() != T or not out.is_contiguous() or out.device != dev:
        raise RuntimeError("top_k_sample: out must be a contiguous int64 tensor with one element per row")
    if T == 0:
        return out
    if top_k > 1:
        if uniforms is None:
            uniforms = torch.rand(T, dtype=torch.float32, device=dev, generator=generator)
        elif (uniforms.dtype != torch.float32 or uniforms.numel() != T or not uniforms.is_contiguous()
              or uniforms.device != dev):
            raise RuntimeError("top_k_sample: uniforms must be a contiguous float32 tensor with one element per row")
    row_stride = rows.stride(0) if T > 1 else max(V, rows.stride(0))
    handle = torch.cuda.current_stream(dev).cuda_stream
    with torch.cuda.device(dev):
        ws = _workspace(dev, handle, _C.npd_top_k_sample_workspace_bytes(T, V, top_k))
        _lib.check(_C.npd_top_k_sample(out.data_ptr(), rows.data_ptr(),
                                       uniforms.data_ptr() if top_k > 1 else None, T, V, row_stride, top_k,
                                       _DTYPE_CODE[rows.dtype], ws.data_ptr(), ws.numel(), handle))
    return out[0] if single else out
