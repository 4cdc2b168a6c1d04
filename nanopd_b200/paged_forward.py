"""The attention step of ``ModelRunner.paged_forward`` on top of the paged kernels.

The reference's closure (nanoPD/engine/model_runner.py:117-212) turns the scheduler's context dict
(nanoPD/engine/engine.py:68-90) into device tensors INSIDE every layer: one ``torch.tensor(..., device=)``
per decode sequence and per prompt, 36 times per step with identical content
(model_runner.py:132-140, 176-187).  Here the context is packed ONCE per step — every table, length and
position in one pinned staging buffer and one host-to-device copy — and each layer only launches kernels:

    sc = build_step_context(runner._current_context, device)        # once per step
    attn_out = paged_attention_step(sc, q, k, v, k_cache[layer], v_cache[layer], scale)   # per layer

``paged_attention_step`` replaces the block between the rotary embedding and ``o_proj``
(model_runner.py:117-210): store the new K/V rows, causal attention of the prompt chunks over their
paged K/V (all earlier chunks included), decode attention of the running sequences.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np
import torch

from . import paged_kernels


@dataclass
class StepContext:
    """Device-resident form of one scheduler step (same content as the reference's ``_current_context``)."""
    num_prefill_tokens: int
    num_decode_tokens: int
    block_size: int
    # prompt chunks, packed one after another in the first num_prefill_tokens rows
    prefill_tables: Optional[torch.Tensor] = None      # int32 [chunks, max_blk_p], zero padded
    prefill_positions: Optional[torch.Tensor] = None   # int32 [num_prefill_tokens]
    prefill_offsets: List[int] = field(default_factory=list)
    prefill_tokens: List[int] = field(default_factory=list)
    prefill_starts: List[int] = field(default_factory=list)
    # decode sequences, one token each, in the last num_decode_tokens rows
    decode_tables: Optional[torch.Tensor] = None       # int32 [Dn, max_blk_d], zero padded
    decode_positions: Optional[torch.Tensor] = None    # int32 [Dn]
    decode_seq_lens: Optional[torch.Tensor] = None     # int32 [Dn] = position + 1
    h2d_bytes: int = 0
    # host-side work estimates behind the SM split of a mixed step
    prefill_score_pairs: int = 0                       # sum over prompt chunks of n*start + n(n+1)/2
    decode_context_tokens: int = 0                     # sum over decode sequences of position + 1


def _padded_table(rows: List[List[int]]) -> np.ndarray:
    width = max(1, max(len(r) for r in rows))
    out = np.zeros((len(rows), width), dtype=np.int32)
    for i, r in enumerate(rows):
        out[i, :len(r)] = r
    return out


def build_step_context(ctx: Dict, device, block_size: int = 16) -> StepContext:
    """Packs the scheduler's context dict for the device with a single host-to-device copy.

    ``ctx`` has the reference's schema (nanoPD/engine/engine.py:68-90, model_runner.py:32-46):
    ``num_prefill_tokens``, ``num_decode_tokens``, ``prefills`` (list of ``block_table``,
    ``start_position``, ``num_tokens``) and ``decodes`` (list of ``block_table``, ``position``).
    Decode tables are zero padded to the longest one and ``seq_lens = position + 1``, exactly what
    the reference builds per layer (model_runner.py:176-187).
    """
    device = torch.device(device)
    prefills, decodes = ctx.get("prefills", []), ctx.get("decodes", [])
    num_p, num_d = int(ctx["num_prefill_tokens"]), int(ctx["num_decode_tokens"])
    if sum(int(p["num_tokens"]) for p in prefills) != num_p:
        raise RuntimeError("num_prefill_tokens does not match the prefill entries")
    if len(decodes) != num_d:
        raise RuntimeError("num_decode_tokens does not match the decode entries")

    parts: Dict[str, np.ndarray] = {}
    sc = StepContext(num_prefill_tokens=num_p, num_decode_tokens=num_d, block_size=block_size)
    if prefills:
        parts["prefill_tables"] = _padded_table([list(p["block_table"]) for p in prefills])
        pos, off = [], 0
        for p in prefills:
            n, start = int(p["num_tokens"]), int(p["start_position"])
            if start + n > len(p["block_table"]) * block_size:
                raise RuntimeError("a prefill chunk reaches beyond its block table")
            pos.append(np.arange(start, start + n, dtype=np.int32))
            sc.prefill_offsets.append(off)
            sc.prefill_tokens.append(n)
            sc.prefill_starts.append(start)
            sc.prefill_score_pairs += n * start + n * (n + 1) // 2
            off += n
        parts["prefill_positions"] = np.concatenate(pos) if pos else np.zeros(0, np.int32)
    if decodes:
        parts["decode_tables"] = _padded_table([list(d["block_table"]) for d in decodes])
        positions = np.asarray([int(d["position"]) for d in decodes], dtype=np.int32)
        for d, p in zip(decodes, positions):
            if p // block_size >= len(d["block_table"]):
                raise RuntimeError("a decode position lies beyond its block table")
        parts["decode_positions"] = positions
        parts["decode_seq_lens"] = positions + 1
        sc.decode_context_tokens = int(positions.sum()) + len(decodes)

    # one staging buffer, 256-byte aligned sections, one copy
    offsets, total = {}, 0
    for name, arr in parts.items():
        offsets[name] = total
        total += (arr.nbytes + 255) // 256 * 256
    sc.h2d_bytes = total
    if total == 0:
        return sc
    stage = torch.empty(total, dtype=torch.uint8)
    if device.type == "cuda":
        stage = stage.pin_memory()
    host = stage.numpy()
    for name, arr in parts.items():
        host[offsets[name]:offsets[name] + arr.nbytes] = arr.reshape(-1).view(np.uint8)
    dev_buf = stage.to(device, non_blocking=True)
    for name, arr in parts.items():
        view = dev_buf[offsets[name]:offsets[name] + arr.nbytes].view(torch.int32).view(arr.shape)
        setattr(sc, name, view)
    sc._staging = (stage, dev_buf)      # keeps the pinned buffer alive until the copy has run
    return sc


# ---- a mixed step on two streams ---------------------------------------------------------------------------
# The prompt chunks' attention is tensor-bound and the decode batch's HBM-bound; both kernels are persistent with
# one CTA per SM.  Run one after the other, each leaves the other's resource idle.  In a mixed step they are
# launched side by side instead, each capped to its share of the SMs; the split minimises the longer of the two
# estimated times.
_PREFILL_FLOPS_PER_S = 1.1e15      # measured rates of the two kernels on a B200, only used for the split
_DECODE_BYTES_PER_S = 6.0e12
_MIN_OVERLAP_SECONDS = 15e-6       # below this much estimated work on either side, fork and join cost more than they save
_side_streams: Dict[int, "torch.cuda.Stream"] = {}


def _sm_split(sc: StepContext, hq: int, hkv: int, d: int, elem: int, sms: int) -> Optional[int]:
    """Of ``sms`` SMs, how many the prompt chunks get in a mixed step (the rest go to the decode batch);
    None = run the two kernels in turn."""
    if sc.num_prefill_tokens == 0 or sc.num_decode_tokens == 0 or sms < 64:
        return None
    t_p = 4.0 * hq * d * sc.prefill_score_pairs / _PREFILL_FLOPS_PER_S
    t_d = 2.0 * hkv * d * elem * sc.decode_context_tokens / _DECODE_BYTES_PER_S
    if min(t_p, t_d) < _MIN_OVERLAP_SECONDS:
        return None
    # The decode kernel switches to 12 warps per CTA on a capped grid and then keeps HBM saturated down to about
    # two thirds of the SMs (measured: 243 us on 100 of 148 SMs against 240 on all of them), below that its time
    # grows in proportion; the chunk kernel's time is inversely proportional to its share throughout.
    knee = int(sms * 0.68)
    best, best_t = None, t_p + t_d
    for share in range(16, sms - 31, 4):
        left = sms - share
        t = max(t_d * (1.0 if left >= knee else knee / left), t_p * sms / share)
        if t < best_t:
            best, best_t = share, t
    return best


def _attend(sc: StepContext, out, q_tokens_major, k_cache, v_cache, scale, overlap: bool):
    """Prompt-chunk attention over rows [:P] and decode attention over rows [P:] of token-major queries."""
    P, Dn = sc.num_prefill_tokens, sc.num_decode_tokens
    bs = k_cache.size(2)
    _, hq, d = q_tokens_major.shape
    dev = q_tokens_major.device
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    share = _sm_split(sc, hq, k_cache.size(1), d, q_tokens_major.element_size(), sms) if overlap else None

    def prefill(max_ctas=0):
        paged_kernels.paged_prefill_attention(out[:P], q_tokens_major[:P], k_cache, v_cache, sc.prefill_tables,
                                              sc.prefill_offsets, sc.prefill_tokens, sc.prefill_starts,
                                              scale, bs, sc.prefill_tables.size(1), max_ctas=max_ctas)

    def decode(max_ctas=0):
        paged_kernels.paged_attention_forward(out[P:], q_tokens_major[P:], k_cache, v_cache, sc.decode_tables,
                                              sc.decode_seq_lens, scale, bs, sc.decode_tables.size(1),
                                              max_ctas=max_ctas)

    if share is None:
        if P > 0:
            prefill()
        if Dn > 0:
            decode()
        return
    main = torch.cuda.current_stream(dev)
    side = _side_streams.get(dev.index)
    if side is None:
        side = _side_streams[dev.index] = torch.cuda.Stream(device=dev)
    side.wait_stream(main)                       # the stores and q are ready
    with torch.cuda.stream(side):
        prefill(max_ctas=share)
    decode(max_ctas=sms - share)
    main.wait_stream(side)


def paged_attention_step(sc: StepContext, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                         k_cache: torch.Tensor, v_cache: torch.Tensor, scale: float,
                         overlap: bool = True) -> torch.Tensor:
    """Store + attention of one layer for one step.

    ``q`` is ``[1, Hq, total, D]``, ``k``/``v`` ``[1, Hkv, total, D]`` after the rotary embedding (the tensors
    the reference holds at model_runner.py:115); the first ``num_prefill_tokens`` columns are the packed
    prompt chunks, the rest one token per decode sequence.  ``k_cache``/``v_cache`` are the layer's
    ``[blocks, Hkv, B, D]`` pools.  Returns ``[1, total, Hq*D]`` like the reference's ``attn_out``
    (model_runner.py:210) — with one difference the reference's tests do not cover: a chunk with
    ``start_position > 0`` attends to the earlier chunks' keys in the pages as well.
    In a mixed step the two attention kernels run side by side on two streams, each on its share of the SMs
    (``overlap=False`` runs them in turn).
    """
    P, Dn = sc.num_prefill_tokens, sc.num_decode_tokens
    total = P + Dn
    _, hq, tq, d = q.shape
    if tq != total or k.size(2) != total or v.size(2) != total:
        raise RuntimeError("q/k/v token count does not match the step context")
    out = torch.empty(total, hq, d, dtype=q.dtype, device=q.device)
    if P > 0:
        for i, (off, n) in enumerate(zip(sc.prefill_offsets, sc.prefill_tokens)):
            # the prompt's table row, read in place for every token of the chunk (stride-0 expand)
            paged_kernels.paged_kv_store(k_cache, v_cache, k[0, :, off:off + n], v[0, :, off:off + n],
                                         sc.prefill_tables[i:i + 1].expand(n, -1), sc.prefill_positions[off:off + n])
    if Dn > 0:
        paged_kernels.paged_kv_store(k_cache, v_cache, k[0, :, P:], v[0, :, P:], sc.decode_tables, sc.decode_positions)
    _attend(sc, out, q[0].transpose(0, 1).contiguous(), k_cache, v_cache, scale, overlap)
    return out.view(1, total, hq * d)


def paged_attention_step_fused(sc: StepContext, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                               cos: torch.Tensor, sin: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                               scale: float, q_norm_weight=None, k_norm_weight=None, eps: float = 1e-6,
                               overlap: bool = True) -> torch.Tensor:
    """The same step starting one stage earlier: from the projection outputs.

    ``q`` ``[total, Hq, D]``, ``k``/``v`` ``[total, Hkv, D]`` are the token-major views of ``q_proj``/``k_proj``/
    ``v_proj`` (nanoPD/engine/model_runner.py:84-99) — or of one fused projection — BEFORE the per-head norm and
    the rotary embedding; ``cos``/``sin`` ``[total, D]`` are the rotary tables of the step's positions.  Norm,
    rotary embedding and the store run as one launch per prompt chunk plus one for all decode tokens
    (``paged_qk_norm_rope_store``), the rotated queries stay token-major, and the attention kernels read them
    in place: no transposes, no ``contiguous()`` copies.  Returns ``[1, total, Hq*D]``.
    """
    P, Dn = sc.num_prefill_tokens, sc.num_decode_tokens
    total = P + Dn
    tq, hq, d = q.shape
    if tq != total or k.size(0) != total or v.size(0) != total:
        raise RuntimeError("q/k/v token count does not match the step context")
    if cos.dim() == 3:
        cos, sin = cos[0], sin[0]
    bs = k_cache.size(2)
    out = torch.empty(total, hq, d, dtype=q.dtype, device=q.device)
    q_rot = torch.empty(total, hq, d, dtype=q.dtype, device=q.device)
    for i, (off, n) in enumerate(zip(sc.prefill_offsets, sc.prefill_tokens)):
        paged_kernels.paged_qk_norm_rope_store(
            q[off:off + n], k[off:off + n], v[off:off + n], cos[off:off + n], sin[off:off + n], k_cache, v_cache,
            sc.prefill_tables[i:i + 1].expand(n, -1), sc.prefill_positions[off:off + n],
            q_norm_weight, k_norm_weight, eps, q_out=q_rot[off:off + n])
    if Dn > 0:
        paged_kernels.paged_qk_norm_rope_store(
            q[P:], k[P:], v[P:], cos[P:], sin[P:], k_cache, v_cache, sc.decode_tables, sc.decode_positions,
            q_norm_weight, k_norm_weight, eps, q_out=q_rot[P:])
    _attend(sc, out, q_rot, k_cache, v_cache, scale, overlap)
    return out.view(1, total, hq * d)
