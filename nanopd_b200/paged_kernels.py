"""Drop-in for the reference's ``paged_kernels`` extension module, on top of the C ABI.

``paged_attention_forward`` and ``paged_kv_store`` keep the positional signatures the
reference binds (nanoPD/paged_attention/csrc/attention/paged_attention_bindings.cpp:6-14,
nanoPD/paged_attention/csrc/kvstore/paged_kv_store_bindings.cpp:4-11), so
``ModelRunner.paged_forward`` (nanoPD/engine/model_runner.py:94,146,189,270) can import this
module unchanged.  ``paged_prefill_attention`` and ``paged_kv_migrate`` are additions.

Everything launches asynchronously on the current stream of the tensors' device and
returns ``None``; argument errors raise ``RuntimeError`` like the reference's TORCH_CHECKs.
Device-side anomalies (an out-of-range block id, a length beyond the table) never fault:
the kernels skip the access and set a status word that :func:`check_status` reads.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Dict, Optional, Sequence, Tuple

import torch

from . import _lib

_DTYPE_CODE = {torch.float16: _lib.NPD_DTYPE_F16, torch.bfloat16: _lib.NPD_DTYPE_BF16,
               torch.float32: _lib.NPD_DTYPE_F32}

_C = _lib.load()   # raises ImportError when the CUDA library is missing: no fallback path


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


# ---------------------------------------------------------------------------
# Per-(device, stream) workspace.  The reference's split-K op allocates three temporaries
# and syncs on every call (paged_attention_optimized_ops.cu:43-57); here one zeroed buffer
# per device and stream is kept and grown on demand.  Several Python threads, each bound
# to its own GPU, may call in concurrently (nanoPD/router/central_scheduler.py:132-135).
# ---------------------------------------------------------------------------
_ws_lock = threading.Lock()
_workspaces: Dict[Tuple[int, int], torch.Tensor] = {}


def _workspace(device: torch.device, stream_handle: int, nbytes: int) -> torch.Tensor:
    key = (device.index, stream_handle)
    ws = _workspaces.get(key)                 # dict reads are atomic under the GIL: the common case takes no lock
    if ws is not None and ws.numel() >= nbytes:
        return ws
    with _ws_lock:
        ws = _workspaces.get(key)
        if ws is None or ws.numel() < nbytes:
            grown = torch.zeros(max(nbytes, 256), dtype=torch.uint8, device=device)
            if ws is not None:
                grown[:4].copy_(ws[:4])       # carry the status word over, on the device (no host wait)
            _workspaces[key] = ws = grown
        return ws


def release_workspaces(device=None) -> None:
    """Drops the cached per-stream workspaces of ``device`` (default: all devices), e.g. after destroying the
    streams they belonged to.  Synchronises the devices concerned first; the next call on a stream makes a new one."""
    with _ws_lock:
        idx = None if device is None else torch.device(device).index
        keys = [k for k in _workspaces if idx is None or k[0] == idx]
        for d in {k[0] for k in keys}:
            torch.cuda.synchronize(d)
        for k in keys:
            del _workspaces[k]


def check_status(device=None, raise_on_error: bool = True) -> int:
    """Reads (and clears) the device-side status words of ``device`` (default: current).

    Returns the OR of the NPD_STATUS_* bits seen since the last call; raises RuntimeError
    for a non-zero word unless ``raise_on_error`` is false.  Synchronises the streams involved.
    """
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    bits = 0
    with _ws_lock:
        items = [(k, w) for k, w in _workspaces.items() if k[0] == idx]
    with torch.cuda.device(idx):
        for (_, stream_handle), ws in items:
            out = ctypes.c_int32(0)
            _lib.check(_C.npd_read_status(ws.data_ptr(), ctypes.byref(out), stream_handle))
            bits |= out.value
            if out.value & _lib.NPD_STATUS_WAIT_TIMEOUT:
                ws.zero_()          # a launch that gave up may have left arrival tickets behind
                torch.cuda.synchronize(idx)
    if bits and raise_on_error:
        names = [n for n, b in (("bad block id", 1), ("bad position / seq_len", 2), ("wait time-out", 4)) if bits & b]
        raise RuntimeError("nanopd_b200 device status: " + ", ".join(names))
    return bits


def _stream_handle(device: torch.device) -> int:
    return _raw_stream(device.index)


try:
    _raw_stream = torch._C._cuda_getCurrentRawStream       # the current stream's handle without building a Stream object
except AttributeError:                                     # pragma: no cover
    def _raw_stream(device_index: int) -> int:
        return torch.cuda.current_stream(device_index).cuda_stream


# ---------------------------------------------------------------------------
# Validated call shapes.  The reference's caller is eager and small (at most 16 running sequences,
# nanoPD/engine/engine.py:21), where the host cost of a call matters as much as the kernel.  Every op therefore
# remembers the call shapes it has validated: the key is what the checks look at (shape, strides, dtype and device
# of every tensor, and the integer arguments), the value the scalar arguments of the C call.  A repeated shape skips
# the checks; a new one takes the checks and is remembered if it needed no conversion.
# ---------------------------------------------------------------------------
_PLAN_LIMIT = 1024
_store_plans: Dict[tuple, tuple] = {}
_attn_plans: Dict[tuple, tuple] = {}
_rope_plans: Dict[tuple, tuple] = {}


def _sig(*tensors) -> tuple:
    return tuple([(t.shape, t.stride(), t.dtype, t.device) for t in tensors])


def _remember(table: Dict[tuple, tuple], key: tuple, plan: tuple) -> None:
    if len(table) >= _PLAN_LIMIT:
        table.clear()
    table[key] = plan


def _call(dev_index: int, fn, *args) -> None:
    """The C call with ``dev_index`` current (switching only when it is not)."""
    if torch.cuda.current_device() == dev_index:
        rc = fn(*args)
    else:
        with torch.cuda.device(dev_index):
            rc = fn(*args)
    if rc:
        _lib.check(rc)


def _ws_ptr(dev_index: int, handle: int, nbytes: int):
    ws = _workspaces.get((dev_index, handle))
    if ws is None or ws.numel() < nbytes:
        ws = _workspace(torch.device("cuda", dev_index), handle, nbytes)
    return ws


def _cache_geometry(cache: torch.Tensor, name: str):
    _require(cache.dim() == 4, f"{name} must be [num_blocks, num_kv_heads, block_size, head_dim]")
    nb, hkv, bs, d = cache.shape
    _require(cache.stride(3) == 1 and cache.stride(2) == d and cache.stride(1) == bs * d,
             f"{name}: the last three dims must be contiguous")
    return nb, hkv, bs, d, cache.stride(0)


# ---------------------------------------------------------------------------
# (1) KV store
# ---------------------------------------------------------------------------
def paged_kv_store(k_cache, v_cache, k_src, v_src, block_tables, positions) -> None:
    """Scatter new K/V rows into their block slots, in place.

    Same contract as the reference op (nanoPD/paged_attention/csrc/kvstore/paged_kv_store.h:23-27,
    paged_kv_store_ops.cu:7-50): caches ``[blocks, Hkv, B, D]``, sources ``[Hkv, T, D]``,
    ``block_tables`` int32 ``[T, max_blk]`` with one row per token (a stride-0 ``expand`` of a
    single row is accepted as is), ``positions`` int32 ``[T]`` absolute positions.

    The call shape the reference's own tests still use is accepted too
    (tests/test_paged_kernels.py:280,311): sources ``[1, Hkv, T, D]``, a 1-D block table of
    the sequence and an ``int`` start position, meaning token ``t`` sits at ``start + t``.
    """
    key = None
    if type(positions) is not int:
        try:
            key = _sig(k_cache, v_cache, k_src, v_src, block_tables, positions)
        except AttributeError:
            key = None
        plan = _store_plans.get(key) if key is not None else None
        if plan is not None:
            dev_index = plan[0]
            handle = _raw_stream(dev_index)
            _call(dev_index, _C.npd_kv_store, k_cache.data_ptr(), v_cache.data_ptr(), k_src.data_ptr(), v_src.data_ptr(),
                  block_tables.data_ptr(), positions.data_ptr(), *plan[1:], _ws_ptr(dev_index, handle, 256).data_ptr(), handle)
            return
    given = (k_src, v_src, block_tables, positions)
    _require(k_src.is_cuda, "k src is must be on CUDA")
    _require(v_src.is_cuda, "v src is must be on CUDA")
    if k_src.dim() == 4 and k_src.size(0) == 1:
        k_src, v_src = k_src[0], v_src[0]
    _require(k_src.dim() == 3, "k_src must be [num_kv_heads, num_tokens, head_dim]")
    _require(v_src.shape == k_src.shape, "k_src and v_src must have the same shape")
    _require(k_cache.is_cuda and v_cache.is_cuda and k_cache.device == k_src.device == v_cache.device,
             "caches and sources must be on the same CUDA device")
    dev = k_src.device
    hkv, T, d = k_src.shape
    if isinstance(positions, int):
        positions = torch.arange(positions, positions + T, dtype=torch.int32, device=dev)
    if block_tables.dim() == 1:
        block_tables = block_tables.unsqueeze(0).expand(T, -1)
    _require(block_tables.dtype == torch.int32 and positions.dtype == torch.int32,
             "block_tables and positions must be int32")
    _require(block_tables.dim() == 2 and block_tables.size(0) == T and positions.dim() == 1 and positions.numel() == T,
             "block_tables must be [num_tokens, max_blocks] and positions [num_tokens]")
    _require(block_tables.device == dev and positions.device == dev, "index tensors must be on the cache device")
    _require(k_cache.dtype == v_cache.dtype == k_src.dtype == v_src.dtype, "cache and source dtypes differ")
    _require(k_cache.dtype in _DTYPE_CODE, f"unsupported dtype {k_cache.dtype}")
    nb, chkv, bs, cd, cstride = _cache_geometry(k_cache, "k_cache")
    _require(_cache_geometry(v_cache, "v_cache") == (nb, chkv, bs, cd, cstride), "k_cache and v_cache layouts differ")
    _require(chkv == hkv and cd == d, "source heads / head_dim do not match the cache")
    _require(k_src.stride(2) == 1 and v_src.stride(2) == 1, "sources need a contiguous last dim")
    # The stride of a size-1 dimension means nothing (torch leaves whatever the producing view had, e.g. on the
    # decode branch's [Hkv, 1, D] slices, nanoPD/engine/model_runner.py:190-193): only real strides must agree.
    def _strides(t):
        return (t.stride(0) if hkv > 1 else T * d, t.stride(1) if T > 1 else d)
    if _strides(k_src) != _strides(v_src):
        k_src, v_src = k_src.contiguous(), v_src.contiguous()
    src_head_stride, src_token_stride = _strides(k_src)
    if block_tables.stride(1) != 1 and block_tables.size(1) > 1:
        block_tables = block_tables.contiguous()
    if positions.stride(0) != 1:
        positions = positions.contiguous()
    if T == 0:
        return
    plan = (dev.index, T, hkv, d, bs, nb, block_tables.size(1), cstride, src_head_stride, src_token_stride,
            block_tables.stride(0), _DTYPE_CODE[k_cache.dtype])
    if key is not None and all(a is b for a, b in zip(given, (k_src, v_src, block_tables, positions))):
        _remember(_store_plans, key, plan)
    handle = _raw_stream(dev.index)
    _call(dev.index, _C.npd_kv_store, k_cache.data_ptr(), v_cache.data_ptr(), k_src.data_ptr(), v_src.data_ptr(),
          block_tables.data_ptr(), positions.data_ptr(), *plan[1:], _ws_ptr(dev.index, handle, 256).data_ptr(), handle)


# ---------------------------------------------------------------------------
# (1b) fused QK-norm + rotary embedding + KV store
# ---------------------------------------------------------------------------
def paged_qk_norm_rope_store(q, k, v, cos, sin, k_cache, v_cache, block_tables, positions,
                             q_norm_weight=None, k_norm_weight=None, eps: float = 1e-6, q_out=None):
    """Per-head RMSNorm (when weights are given) and rotary embedding of Q and K, K and V written into
    their block slots, in one launch.

    Stands for the passes the reference runs between the projections and the store
    (nanoPD/engine/model_runner.py:97-115, then paged_kv_store at :142-149 / :188-194), with the
    rounding steps of the Hugging Face modules it calls.  ``q`` ``[T, Hq, D]``, ``k``/``v``
    ``[T, Hkv, D]`` token-major (views into a fused projection output are fine: only the last two
    dims must be contiguous); ``cos``/``sin`` ``[T, D]`` (or ``[1, T, D]``) in the tensors' dtype;
    ``block_tables`` int32 one row per token, ``positions`` int32 ``[T]`` as for ``paged_kv_store``.
    Returns the rotated queries ``[T, Hq, D]`` (``q_out``, default: in place over ``q``) — the layout
    ``paged_attention_forward`` and ``paged_prefill_attention`` take.
    """
    if q_out is None:
        q_out = q
    try:
        key = (_sig(q, k, v, cos, sin, k_cache, v_cache, block_tables, positions, q_out),
               None if q_norm_weight is None else _sig(q_norm_weight),
               None if k_norm_weight is None else _sig(k_norm_weight))
    except AttributeError:
        key = None
    plan = _rope_plans.get(key) if key is not None else None
    if plan is not None:
        dev_index = plan[0]
        handle = _raw_stream(dev_index)
        _call(dev_index, _C.npd_qk_norm_rope_store, q_out.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
              None if q_norm_weight is None else q_norm_weight.data_ptr(),
              None if k_norm_weight is None else k_norm_weight.data_ptr(),
              cos.data_ptr(), sin.data_ptr(), float(eps), k_cache.data_ptr(), v_cache.data_ptr(),
              block_tables.data_ptr(), positions.data_ptr(), *plan[1:], _ws_ptr(dev_index, handle, 256).data_ptr(), handle)
        return q_out
    given = (cos, sin, block_tables, positions)
    _require(q.is_cuda and k.is_cuda and v.is_cuda, "q, k and v must be on CUDA")
    _require(q.dim() == 3 and k.dim() == 3 and v.dim() == 3, "q must be [T, Hq, D] and k, v [T, Hkv, D]")
    T, hq, d = q.shape
    _require(k.shape == v.shape and k.size(0) == T and k.size(2) == d, "k and v must be [T, Hkv, D] with q's T and D")
    hkv = k.size(1)
    dev = q.device
    if cos.dim() == 3 and cos.size(0) == 1:
        cos, sin = cos[0], sin[0]
    _require(cos.shape == sin.shape and cos.dim() == 2 and cos.size(1) == d and cos.size(0) in (1, T),
             "cos and sin must be [T, D]")
    _require(q_out.shape == q.shape, "q_out must have q's shape")
    for name, t_ in (("q", q), ("k", k), ("v", v), ("q_out", q_out)):
        _require(t_.stride(2) == 1 and t_.stride(1) == d, f"{name}: the last two dims must be contiguous")
    _require(cos.stride(1) == 1 and sin.stride(1) == 1 and cos.stride(0) == sin.stride(0), "cos/sin rows must be contiguous")
    _require(q.dtype in (torch.float16, torch.bfloat16), f"unsupported dtype {q.dtype}")
    _require(all(t_.dtype == q.dtype for t_ in (k, v, cos, sin, q_out, k_cache, v_cache)), "dtypes differ")
    _require(all(t_.device == dev for t_ in (k, v, cos, sin, q_out, k_cache, v_cache, block_tables, positions)),
             "all tensors must be on the same CUDA device")
    for w_ in (q_norm_weight, k_norm_weight):
        _require(w_ is None or (w_.dtype == q.dtype and w_.device == dev and w_.numel() == d and w_.is_contiguous()),
                 "norm weights must be contiguous [D] tensors of q's dtype")
    if block_tables.dim() == 1:
        block_tables = block_tables.unsqueeze(0).expand(T, -1)
    _require(block_tables.dtype == torch.int32 and positions.dtype == torch.int32,
             "block_tables and positions must be int32")
    _require(block_tables.dim() == 2 and block_tables.size(0) == T and positions.dim() == 1 and positions.numel() == T,
             "block_tables must be [num_tokens, max_blocks] and positions [num_tokens]")
    nb, chkv, bs, cd, cstride = _cache_geometry(k_cache, "k_cache")
    _require(_cache_geometry(v_cache, "v_cache") == (nb, chkv, bs, cd, cstride), "k_cache and v_cache layouts differ")
    _require(chkv == hkv and cd == d, "k/v heads / head_dim do not match the cache")
    if block_tables.stride(1) != 1 and block_tables.size(1) > 1:
        block_tables = block_tables.contiguous()
    if positions.stride(0) != 1:
        positions = positions.contiguous()
    if T == 0:
        return q_out
    plan = (dev.index, T, hq, hkv, d, bs, nb, block_tables.size(1), cstride, q.stride(0), k.stride(0), v.stride(0),
            q_out.stride(0), 0 if cos.size(0) == 1 else cos.stride(0), block_tables.stride(0), _DTYPE_CODE[q.dtype])
    if key is not None and all(a is b for a, b in zip(given, (cos, sin, block_tables, positions))):
        _remember(_rope_plans, key, plan)
    handle = _raw_stream(dev.index)
    _call(dev.index, _C.npd_qk_norm_rope_store, q_out.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
          None if q_norm_weight is None else q_norm_weight.data_ptr(),
          None if k_norm_weight is None else k_norm_weight.data_ptr(),
          cos.data_ptr(), sin.data_ptr(), float(eps), k_cache.data_ptr(), v_cache.data_ptr(),
          block_tables.data_ptr(), positions.data_ptr(), *plan[1:], _ws_ptr(dev.index, handle, 256).data_ptr(), handle)
    return q_out


# ---------------------------------------------------------------------------
# (2) decode attention
# ---------------------------------------------------------------------------
def paged_attention_forward(out, query, key_cache, value_cache, block_tables, seq_lens,
                            scale: float, block_size: int, max_num_blocks_per_seq: int,
                            _flags: int = 0, max_ctas: int = 0) -> None:
    """``out[s, h] = softmax(scale * q[s, h] . K_s^T) . V_s`` over paged K/V, written in place.

    Same contract as the reference op (nanoPD/paged_attention/csrc/attention/paged_attention.h:24-34,
    paged_attention_ops.cu:7-59): ``out``/``query`` ``[S, Hq, D]`` contiguous, caches
    ``[blocks, Hkv, B, D]``, ``block_tables`` int32 ``[S, max_num_blocks_per_seq]`` zero padded,
    ``seq_lens`` int32 ``[S]``; int64 index tensors raise RuntimeError as they do there
    (pinned by tests/test_paged_kernels.py:218-227).  As in the reference's pointer math
    (paged_attention_kernel.cu:72), row ``s`` of a contiguous table starts at
    ``s * max_num_blocks_per_seq``.

    The interleaved layouts the reference's split-K op and its kernel tests use are accepted under the
    same name (csrc/paged_attention_optimized/paged_attention_optimized_ops.cu:33-34,
    tests/test_paged_kernels.py:39-56): a 5-D ``key_cache`` ``[blocks, Hkv, D/8, B, 8]`` goes with a
    ``value_cache`` ``[blocks, Hkv, D, B]``.

    ``max_ctas`` (an addition, 0 = one CTA per SM) caps the persistent grid so that the call can share the GPU
    with another kernel on a second stream (see ``paged_forward.paged_attention_step``).
    """
    try:
        key = (_sig(out, query, key_cache, value_cache, block_tables, seq_lens), block_size, max_num_blocks_per_seq,
               _flags, max_ctas)
    except AttributeError:
        key = None
    plan = _attn_plans.get(key) if key is not None else None
    if plan is not None:
        dev_index, need, flags = plan[0], plan[1], plan[2]
        handle = _raw_stream(dev_index)
        ws = _ws_ptr(dev_index, handle, need)
        _call(dev_index, _C.npd_paged_decode_attention, out.data_ptr(), query.data_ptr(), key_cache.data_ptr(),
              value_cache.data_ptr(), block_tables.data_ptr(), seq_lens.data_ptr(), float(scale), *plan[3:],
              ws.data_ptr(), ws.numel(), flags, handle)
        return
    _require(query.is_cuda, "query is must be on CUDA")
    _require(query.dim() == 3, "query must be [num seqs, num_heads, head_size]")
    _require(key_cache.dim() in (4, 5), "key_cache must be [num_blocks, num_kv_heads, block_size, head_size] "
                                        "or [num_blocks, num_kv_heads, head_size/8, block_size, 8]")
    interleaved = key_cache.dim() == 5
    _require(block_tables.dtype == torch.int32, "block_tables must be int32")
    _require(seq_lens.dtype == torch.int32, "seq_lens must be int32")
    dev = query.device
    S, hq, d = query.shape
    _require(out.shape == query.shape and out.dtype == query.dtype and out.device == dev,
             "out must match query in shape, dtype and device")
    _require(query.is_contiguous() and out.is_contiguous(), "query and out must be contiguous")
    _require(query.dtype in (torch.float16, torch.bfloat16),
             f"paged_attention_forward supports float16 and bfloat16, got {query.dtype}")
    _require(key_cache.dtype == query.dtype and value_cache.dtype == query.dtype, "cache dtype differs from query")
    _require(key_cache.device == dev and value_cache.device == dev and block_tables.device == dev
             and seq_lens.device == dev, "all tensors must be on the query's device")
    if interleaved:
        nb, hkv, pieces, bs, x = key_cache.shape
        _require(x == 8 and pieces * x == d, "interleaved key_cache must be [blocks, Hkv, head_size/8, block_size, 8]")
        _require(value_cache.dim() == 4 and tuple(value_cache.shape) == (nb, hkv, d, bs),
                 "interleaved value_cache must be [blocks, Hkv, head_size, block_size]")
        _require(key_cache[0].is_contiguous() and value_cache[0].is_contiguous()
                 and key_cache.stride(0) == value_cache.stride(0), "interleaved caches must be contiguous per block")
        cd, cstride = d, key_cache.stride(0)
        _flags = int(_flags) | _lib.NPD_DECODE_KV_INTERLEAVED
    else:
        nb, hkv, bs, cd, cstride = _cache_geometry(key_cache, "key_cache")
        _require(_cache_geometry(value_cache, "value_cache") == (nb, hkv, bs, cd, cstride),
                 "key_cache and value_cache layouts differ")
    _require(cd == d, "head_size of query and cache differ")
    _require(int(block_size) == bs, f"block_size argument {block_size} != cache block size {bs}")
    _require(hq % hkv == 0, "num_heads must be a multiple of num_kv_heads")
    _require(seq_lens.dim() == 1 and seq_lens.numel() == S and seq_lens.stride(0) == 1, "seq_lens must be contiguous [S]")
    max_blk = int(max_num_blocks_per_seq)
    _require(max_blk >= 1, "max_num_blocks_per_seq must be positive")
    if block_tables.dim() == 2 and block_tables.stride(1) == 1 and not block_tables.is_contiguous():
        row_stride = block_tables.stride(0)          # a row-strided view: honour it
        _require(block_tables.size(1) >= max_blk, "block_tables rows shorter than max_num_blocks_per_seq")
    else:
        _require(block_tables.is_contiguous(), "block_tables must be contiguous")
        row_stride = max_blk                         # the reference's flat indexing
        _require(block_tables.numel() >= S * max_blk, "block_tables smaller than num_seqs * max_num_blocks_per_seq")
    if S == 0:
        return
    need = _C.npd_decode_workspace_bytes(S, hq, hkv, d, dev.index)
    flags = int(_flags) | ((int(max_ctas) & 0xffff) << 8)
    plan = (dev.index, need, flags, S, hq, hkv, d, bs, max_blk, nb, cstride, row_stride, _DTYPE_CODE[query.dtype])
    if key is not None:
        _remember(_attn_plans, key, plan)
    handle = _raw_stream(dev.index)
    ws = _ws_ptr(dev.index, handle, need)
    _call(dev.index, _C.npd_paged_decode_attention, out.data_ptr(), query.data_ptr(), key_cache.data_ptr(),
          value_cache.data_ptr(), block_tables.data_ptr(), seq_lens.data_ptr(), float(scale), *plan[3:],
          ws.data_ptr(), ws.numel(), flags, handle)


# ---------------------------------------------------------------------------
# (3) chunked-prefill attention over paged K/V
# ---------------------------------------------------------------------------
def paged_prefill_attention(out, query, key_cache, value_cache, block_tables,
                            chunk_q_offsets: Sequence[int], chunk_tokens: Sequence[int],
                            chunk_starts: Sequence[int], scale: float, block_size: int,
                            max_num_blocks_per_seq: int, _flags: int = 0, max_ctas: int = 0) -> None:
    """Causal attention of prompt chunks over their paged K/V (the chunk's own rows included).

    Replaces the prefill branch of ``paged_forward`` (nanoPD/engine/model_runner.py:152-169).
    ``query``/``out`` are ``[total_tokens, Hq, D]`` with the chunks packed one after another;
    chunk ``c`` occupies rows ``chunk_q_offsets[c] : + chunk_tokens[c]``, its first token sits
    at absolute position ``chunk_starts[c]`` and row ``c`` of ``block_tables`` (int32
    ``[num_chunks, max_num_blocks_per_seq]``) names its pages.  Store the chunk's K/V with
    :func:`paged_kv_store` first, as the caller does (model_runner.py:132-150).
    """
    _require(query.is_cuda and query.dim() == 3, "query must be a CUDA tensor [tokens, num_heads, head_size]")
    _require(block_tables.dtype == torch.int32 and block_tables.dim() == 2, "block_tables must be int32 [chunks, max_blk]")
    dev = query.device
    total, hq, d = query.shape
    nchunks = len(chunk_tokens)
    _require(len(chunk_q_offsets) == nchunks and len(chunk_starts) == nchunks and block_tables.size(0) == nchunks,
             "one offset, token count, start position and table row per chunk")
    _require(out.shape == query.shape and out.dtype == query.dtype and query.is_contiguous() and out.is_contiguous(),
             "out must match query; both contiguous")
    _require(query.dtype in (torch.float16, torch.bfloat16), f"unsupported dtype {query.dtype}")
    nb, hkv, bs, cd, cstride = _cache_geometry(key_cache, "key_cache")
    _require(_cache_geometry(value_cache, "value_cache") == (nb, hkv, bs, cd, cstride), "cache layouts differ")
    _require(cd == d and int(block_size) == bs and key_cache.dtype == query.dtype == value_cache.dtype,
             "cache does not match query")
    _require(block_tables.stride(1) == 1 or block_tables.size(1) == 1, "block_tables rows must be contiguous")
    max_blk = int(max_num_blocks_per_seq)
    _require(1 <= max_blk <= block_tables.size(1), "max_num_blocks_per_seq out of range")
    for off, n, start in zip(chunk_q_offsets, chunk_tokens, chunk_starts):
        _require(n >= 0 and off >= 0 and off + n <= total and start >= 0, "chunk outside the query tensor")
        _require(start + n <= max_blk * bs, "chunk reaches beyond its block table")
    if nchunks == 0 or total == 0:
        return
    arr = ctypes.c_int32 * nchunks
    handle = _stream_handle(dev)
    with torch.cuda.device(dev):
        need = _C.npd_prefill_workspace_bytes(total, hq, hkv, d, dev.index)
        ws = _workspace(dev, handle, need)
        _lib.check(_C.npd_paged_prefill_attention(
            out.data_ptr(), query.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
            block_tables.data_ptr(), arr(*chunk_q_offsets), arr(*chunk_tokens), arr(*chunk_starts),
            nchunks, float(scale), hq, hkv, d, bs, max_blk, nb, cstride, block_tables.stride(0),
            _DTYPE_CODE[query.dtype], ws.data_ptr(), ws.numel(),
            int(_flags) | ((int(max_ctas) & 0xffff) << 8), handle))


# ---------------------------------------------------------------------------
# (4) KV page migration
# ---------------------------------------------------------------------------
def _pool_geometry(pool: torch.Tensor, name: str):
    _require(pool.dim() == 5, f"{name} must be [layers, blocks, num_kv_heads, block_size, head_dim]")
    L, nb = pool.shape[:2]
    block_elems = pool.shape[2] * pool.shape[3] * pool.shape[4]
    _require(pool[0, 0].is_contiguous(), f"{name}: a block must be contiguous")
    return L, nb, block_elems, pool.stride(0), pool.stride(1)


def _block_list(ids, dev: torch.device) -> torch.Tensor:
    """A block list as an int32 tensor on ``dev``.  A Python list goes through pinned host memory and a
    non-blocking copy on the current stream, so the calling thread never waits behind work already queued on
    that stream (a pageable source would make the copy synchronous with the stream's earlier work)."""
    if torch.is_tensor(ids):
        return ids
    host = torch.tensor(list(ids), dtype=torch.int32)
    if host.numel() == 0:
        return host.to(dev)
    return host.pin_memory().to(dev, non_blocking=True)


def paged_kv_migrate(src_k, src_v, dst_k, dst_v, src_blocks, dst_blocks=None, max_ctas: int = 0) -> None:
    """Copy blocks ``src_blocks[i] -> dst_blocks[i]`` of every layer between two 5-D pools.

    One kernel on the current stream of the CURRENT device, which must be able to address
    both pools (same device, or peer access enabled — see ``kv_transfer.transfer_kv``).  One of the
    two pools may be a PINNED host buffer (``kv_transfer.PinnedKVBuffer``): the kernel then reads or writes
    it over PCIe through the unified address space with plain loads and stores.
    ``src_blocks``/``dst_blocks``: int32 tensors on the current device, or Python lists, which are staged in
    pinned memory and copied there without blocking the host.  ``max_ctas`` > 0 caps the grid of the
    bulk-copy kernel (one warp per CTA; 0 = 64 CTAs) so a side-stream migration leaves the SMs to compute; a
    negative value selects the plain load/store kernel with that many CTAs.
    """
    dev = torch.device("cuda", torch.cuda.current_device())
    L, snb, belems, sls, sbs = _pool_geometry(src_k, "src_k")
    _require(_pool_geometry(src_v, "src_v") == (L, snb, belems, sls, sbs), "src_k and src_v layouts differ")
    L2, dnb, belems2, dls, dbs = _pool_geometry(dst_k, "dst_k")
    _require(_pool_geometry(dst_v, "dst_v") == (L2, dnb, belems2, dls, dbs), "dst_k and dst_v layouts differ")
    _require(L == L2 and belems == belems2 and src_k.dtype == dst_k.dtype == src_v.dtype == dst_v.dtype,
             "source and destination pools differ in layers, block shape or dtype")
    for name, pool in (("src_k", src_k), ("src_v", src_v), ("dst_k", dst_k), ("dst_v", dst_v)):
        _require(pool.is_cuda or pool.is_pinned(), f"{name} must be a CUDA tensor or a pinned host tensor")
    _require(src_k.is_cuda or dst_k.is_cuda, "one of the two pools must be on a GPU")
    src_blocks = _block_list(src_blocks, dev)
    dst_blocks = src_blocks if dst_blocks is None else _block_list(dst_blocks, dev)
    _require(src_blocks.dtype == torch.int32 and dst_blocks.dtype == torch.int32, "block lists must be int32")
    _require(src_blocks.device == dev and dst_blocks.device == dev, "block lists must live on the current device")
    _require(src_blocks.numel() == dst_blocks.numel() and src_blocks.is_contiguous() and dst_blocks.is_contiguous(),
             "block lists must be contiguous and of equal length")
    n = src_blocks.numel()
    if n == 0:
        return
    handle = _stream_handle(dev)
    ws = _workspace(dev, handle, 256)
    _lib.check(_C.npd_kv_migrate(
        src_k.data_ptr(), src_v.data_ptr(), dst_k.data_ptr(), dst_v.data_ptr(),
        src_blocks.data_ptr(), dst_blocks.data_ptr(), n, L, belems, src_k.element_size(),
        sls, sbs, snb, dls, dbs, dnb, int(max_ctas), ws.data_ptr(), handle))


def enable_peer_access(peer_device: int) -> None:
    """Map ``peer_device``'s memory into the current device (idempotent)."""
    _lib.check(_C.npd_enable_peer_access(int(peer_device)))
