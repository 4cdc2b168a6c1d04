"""CPU oracle for the paged-attention hot path (TEST INFRASTRUCTURE, not product code).

This file restates, in plain PyTorch on the CPU, the arithmetic of the reference
project's paged-attention path.  Only the test-suite, the smoke check and the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark may import it; the
shipped package never does and fails loudly when its CUDA library is missing.

Parity pin: ``paged_decode_attention`` is checked bit-for-bit (fp32 result and the
dtype-rounded result) against the reference's own ``ref_paged_attention``
(nanoPD/paged_attention/tests/test_paged_kernels.py:63-95), imported from the
reference tree by ``tests/golden/make_golden.py``, which also writes the committed
fixtures under ``tests/golden/``.  ``kv_store`` is pinned by the mapping the
reference's store tests assert (test_paged_kernels.py:272-355).  The chunked-prefill
function has no reference implementation that reads earlier chunks from the pages
(nanoPD/engine/model_runner.py:152-168 attends to the current chunk only); for
``start_position == 0`` it is pinned against that SDPA call, for later chunks parity
is unpinned and this oracle defines the value.

``qk_norm_rope_store`` restates arithmetic that lives in a third-party dependency of the
reference, Hugging Face transformers (``Qwen3RMSNorm.forward``, ``apply_rotary_pos_emb`` and
``rotate_half`` of ``transformers/models/qwen3/modeling_qwen3.py``; the reference pins no version,
README "transformers", the fixtures were made with 5.5.0), at the reference's call sites
nanoPD/engine/model_runner.py:97-115.  It is pinned bit for bit against those functions by
``tests/golden/make_golden_rope.py`` and the fixture ``tests/golden/qk_norm_rope_cases.npz``.

``top_k_candidates`` / ``top_k_sample`` restate ``top_k_sample`` of nanoPD/engine/model_runner.py:279-284
(nan_to_num, ``torch.topk``, softmax over the k values in the logits' dtype, one multinomial draw).
The k values, their ids and the probabilities are pinned bit for bit against those torch calls by
``tests/golden/make_golden_sampling.py`` (fixture ``tests/golden/top_k_sample_cases.npz``), and the
``top_k = 1`` result against the reference function itself.  The draw cannot be pinned: the
reference takes it from torch's global generator.  Here it is the inverse CDF of a uniform number
the caller supplies, over the same probabilities.

Every function cites the reference file:line it follows.
"""
from __future__ import annotations

import math
from typing import Sequence

import torch
import torch.nn.functional as F


# ---------------------------------------------------------------------------
# Sampling
# ---------------------------------------------------------------------------
def top_k_candidates(logits, top_k):
    """The k candidates of every row and their probabilities (nanoPD/engine/model_runner.py:280-282).

    logits [T, V] (fp16 / bf16 / fp32).  Returns (values [T, k] in the logits' dtype, ids int64 [T, k],
    probabilities [T, k] in the logits' dtype).  Candidates are ordered by value, largest first, equal
    values by the lower id first (``torch.topk`` leaves that order unspecified)."""
    x = torch.nan_to_num(logits, nan=0.0, posinf=1e4, neginf=-1e4)
    order = torch.sort(x.float(), dim=-1, descending=True, stable=True).indices[:, :top_k]
    vals = torch.gather(x, 1, order)
    probs = torch.softmax(vals, dim=-1)
    return vals, order, probs


def top_k_sample(logits, top_k, uniforms=None):
    """One draw per row from the top-k distribution (nanoPD/engine/model_runner.py:279-284).

    The draw is the inverse CDF of ``uniforms[t]`` in [0, 1): the first candidate whose running fp32 sum
    of probabilities exceeds ``uniforms[t]`` times the total.  ``top_k == 1`` needs no uniform number and
    returns the arg-max, which is what the reference's default returns."""
    import numpy as np
    _, ids, probs = top_k_candidates(logits, top_k)
    T = logits.size(0)
    out = torch.empty(T, dtype=torch.int64)
    u = torch.zeros(T) if uniforms is None else uniforms.float().cpu()
    for t in range(T):
        c = np.cumsum(probs[t].float().numpy(), dtype=np.float32)
        target = np.float32(u[t].item()) * c[-1]
        j = int(np.searchsorted(c, target, side="right"))
        out[t] = ids[t, min(j, top_k - 1)]
    return out


# ---------------------------------------------------------------------------
# KV store
# ---------------------------------------------------------------------------
def kv_store(k_cache, v_cache, k_src, v_src, block_tables, positions):
    """Scatter new K/V rows into block slots, in place.

    Follows nanoPD/paged_attention/csrc/kvstore/paged_kv_store_kernel.cu:40-57 and the
    indexed-assignment loop in nanoPD/docs/en/03-cuda_kernels_en.md:71-78:
    token ``t`` of head ``h`` goes to
    ``cache[block_tables[t, positions[t] // B], h, positions[t] % B, :]``.

    k_cache, v_cache : [blocks, Hkv, B, D]
    k_src, v_src     : [Hkv, T, D]
    block_tables     : int32 [T, max_blk]  (one row per token)
    positions        : int32 [T]
    """
    B = k_cache.size(2)
    T = k_src.size(1)
    pos = positions.to(torch.int64)
    blk_idx = pos // B
    off = pos % B
    phys = block_tables.to(torch.int64)[torch.arange(T), blk_idx]
    # Later tokens win when two tokens name the same slot, as a serial loop would.
    for t in range(T):
        k_cache[phys[t], :, off[t], :] = k_src[:, t, :]
        v_cache[phys[t], :, off[t], :] = v_src[:, t, :]


# ---------------------------------------------------------------------------
# QK-norm + rotary embedding + store (the passes in front of the store)
# ---------------------------------------------------------------------------
def rms_norm_heads(x, weight, eps):
    """Per-head RMSNorm as the reference's q_norm / k_norm apply it (model_runner.py:101-104 calling
    transformers' Qwen3RMSNorm): fp32 statistics, result rounded to the input dtype, then multiplied
    by the weight in that dtype."""
    x32 = x.to(torch.float32)
    var = x32.pow(2).mean(-1, keepdim=True)
    return weight * (x32 * torch.rsqrt(var + eps)).to(x.dtype)


def rotate_half(x):
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def rotary(x, cos, sin):
    """x: [T, H, D]; cos, sin: [T, D] in x's dtype.  ``(x * cos) + (rotate_half(x) * sin)`` evaluated in
    the tensor dtype, each product and the sum rounded (model_runner.py:110-115 calling transformers'
    apply_rotary_pos_emb)."""
    c, s_ = cos.unsqueeze(1), sin.unsqueeze(1)
    return (x * c) + (rotate_half(x) * s_)


def qk_norm_rope_store(q, k, v, cos, sin, k_cache, v_cache, block_tables, positions,
                       q_norm_weight=None, k_norm_weight=None, eps=1e-6):
    """q [T,Hq,D], k/v [T,Hkv,D] token-major.  Returns the rotated queries [T,Hq,D]; K (normed and
    rotated) and V go to their block slots with ``kv_store`` (model_runner.py:97-115 then :142-149)."""
    if q_norm_weight is not None:
        q = rms_norm_heads(q, q_norm_weight, eps)
    if k_norm_weight is not None:
        k = rms_norm_heads(k, k_norm_weight, eps)
    q_rot = rotary(q, cos, sin)
    k_rot = rotary(k, cos, sin)
    kv_store(k_cache, v_cache, k_rot.transpose(0, 1), v.transpose(0, 1), block_tables, positions)
    return q_rot


# ---------------------------------------------------------------------------
# Decode attention
# ---------------------------------------------------------------------------
def _gather_sequence(cache, block_table_row, slen, block_size):
    """[Hkv, slen, D] view of one sequence's pages (test_paged_kernels.py:79-85)."""
    nblocks = (slen + block_size - 1) // block_size
    ids = block_table_row[:nblocks].to(torch.int64)
    pages = cache.index_select(0, ids)               # [nblocks, Hkv, B, D]
    pages = pages.permute(1, 0, 2, 3).reshape(cache.size(1), nblocks * block_size, cache.size(3))
    return pages[:, :slen, :]


def paged_decode_attention(query, key_cache, value_cache, block_tables, seq_lens, scale):
    """fp32 result of one-token-per-sequence attention over paged K/V.

    Follows ``ref_paged_attention`` (nanoPD/paged_attention/tests/test_paged_kernels.py:63-95;
    same math at tests/test_paged_attention.py:33-71): gather the sequence's blocks,
    truncate to seq_len, cast to fp32, repeat K/V for grouped heads
    (kv head of q head h is ``h // (Hq // Hkv)``), ``bmm * scale -> softmax -> bmm``.
    Returns fp32 ``[S, Hq, D]`` (the reference's value *before* its final cast to the
    query dtype; ``.to(query.dtype)`` of this equals the reference's return value).
    """
    S, Hq, D = query.shape
    Hkv = key_cache.size(1)
    B = key_cache.size(2)
    group = Hq // Hkv
    out = torch.empty(S, Hq, D, dtype=torch.float32)
    for s in range(S):
        slen = int(seq_lens[s])
        keys = _gather_sequence(key_cache, block_tables[s], slen, B).float()
        values = _gather_sequence(value_cache, block_tables[s], slen, B).float()
        keys = keys.repeat_interleave(group, dim=0)      # [Hq, slen, D]
        values = values.repeat_interleave(group, dim=0)
        q = query[s].unsqueeze(1).float()                # [Hq, 1, D]
        attn = torch.bmm(q, keys.transpose(1, 2)) * scale
        attn = F.softmax(attn, dim=-1)
        out[s] = torch.bmm(attn, values).squeeze(1)
    return out


# ---------------------------------------------------------------------------
# Chunked-prefill attention over paged K/V
# ---------------------------------------------------------------------------
def paged_prefill_attention(query, key_cache, value_cache, block_table, start_position, scale):
    """fp32 causal attention of a chunk's queries over positions [0, start+n).

    query : [n, Hq, D], token i sits at absolute position ``start_position + i`` and
    attends to keys ``0 .. start_position + i`` read from the pages named by
    ``block_table`` (the chunk's own K/V must already be stored, as the caller does at
    nanoPD/engine/model_runner.py:132-150 before attending).  For
    ``start_position == 0`` this equals the reference's prefill branch
    (model_runner.py:152-168: ``-inf`` upper-triangular mask, ``repeat_interleave`` of
    K/V over the group, ``scaled_dot_product_attention``); for later chunks the
    reference ignores earlier pages, so this function defines the value.
    Returns fp32 ``[n, Hq, D]``.
    """
    n, Hq, D = query.shape
    Hkv = key_cache.size(1)
    B = key_cache.size(2)
    group = Hq // Hkv
    total = start_position + n
    keys = _gather_sequence(key_cache, block_table, total, B).float()
    values = _gather_sequence(value_cache, block_table, total, B).float()
    keys = keys.repeat_interleave(group, dim=0)          # [Hq, total, D]
    values = values.repeat_interleave(group, dim=0)
    q = query.float().transpose(0, 1)                    # [Hq, n, D]
    scores = torch.bmm(q, keys.transpose(1, 2)) * scale  # [Hq, n, total]
    qpos = torch.arange(start_position, total).unsqueeze(1)
    kpos = torch.arange(total).unsqueeze(0)
    scores = scores.masked_fill((kpos > qpos).unsqueeze(0), float("-inf"))
    probs = F.softmax(scores, dim=-1)
    return torch.bmm(probs, values).transpose(0, 1).contiguous()


def reference_prefill_sdpa(q_p, k_p, v_p, chunk_lens: Sequence[int], scale):
    """The reference's packed prefill attention exactly as it calls it.

    nanoPD/engine/model_runner.py:152-169: q_p ``[1, Hq, P, D]``, k_p/v_p
    ``[1, Hkv, P, D]`` hold the packed prompts; a dense ``P x P`` mask is ``-inf``
    everywhere except a causal lower triangle per prompt.  Used by the oracle's own
    tests to pin ``paged_prefill_attention`` at ``start_position == 0``.
    """
    P = q_p.size(2)
    group = q_p.size(1) // k_p.size(1)
    mask = torch.full((P, P), float("-inf"), dtype=q_p.dtype)
    off = 0
    for L in chunk_lens:
        mask[off:off + L, off:off + L] = torch.triu(
            torch.full((L, L), float("-inf"), dtype=q_p.dtype), diagonal=1)
        off += L
    k_ex = k_p.repeat_interleave(group, dim=1)
    v_ex = v_p.repeat_interleave(group, dim=1)
    out = F.scaled_dot_product_attention(q_p, k_ex, v_ex, attn_mask=mask, scale=scale)
    return out.transpose(1, 2).reshape(1, P, -1)


# ---------------------------------------------------------------------------
# KV page migration
# ---------------------------------------------------------------------------
def kv_migrate(src_k, src_v, dst_k, dst_v, src_blocks, dst_blocks=None):
    """Copy the named blocks of every layer from the source pool to the destination pool.

    Follows ``transfer_kv`` (nanoPD/workers/kv_transfer.py:73-79): for each block id,
    ``dst[:, bid] = src[:, bid]`` on 5-D pools ``[L, blocks, Hkv, B, D]``.  The
    reference uses the same id on both sides; ``dst_blocks`` lets the ids differ.
    """
    if dst_blocks is None:
        dst_blocks = src_blocks
    for sb, db in zip(src_blocks, dst_blocks):
        dst_k[:, int(db)].copy_(src_k[:, int(sb)])
        dst_v[:, int(db)].copy_(src_v[:, int(sb)])


def extract_kv_to_buffer(k_cache, v_cache, block_table, buf_k, buf_v):
    """The sending half of the pinned relay (nanoPD/workers/kv_transfer.py:44-52):
    ``buf[:, i] = cache[:, block_table[i]]`` on ``[L, blocks, Hkv, B, D]`` tensors."""
    for i, bid in enumerate(block_table):
        buf_k[:, i].copy_(k_cache[:, int(bid)])
        buf_v[:, i].copy_(v_cache[:, int(bid)])


def load_kv_from_buffer(k_cache, v_cache, block_table, buf_k, buf_v):
    """The receiving half of the pinned relay (nanoPD/workers/kv_transfer.py:55-66):
    ``cache[:, block_table[i]] = buf[:, i]``."""
    for i, bid in enumerate(block_table):
        k_cache[:, int(bid)].copy_(buf_k[:, i])
        v_cache[:, int(bid)].copy_(buf_v[:, i])


# ---------------------------------------------------------------------------
# Algorithmic work (the figures the benchmark's roofline uses)
# ---------------------------------------------------------------------------
def decode_algorithmic_bytes(seq_lens, Hq, Hkv, D, block_size, elem_bytes=2):
    """K/V counted once per kv head and per real token, plus Q, O, tables and lengths."""
    lens = [int(x) for x in seq_lens]
    S = len(lens)
    kv = sum(lens) * 2 * Hkv * D * elem_bytes
    qo = 2 * S * Hq * D * elem_bytes
    tables = sum((l + block_size - 1) // block_size for l in lens) * 4 + S * 4
    return kv + qo + tables


def prefill_algorithmic_flops(n, start, Hq, D):
    """Causal flops of one chunk: 4 * Hq * D * sum_{i<n} (start + i + 1)."""
    return 4 * Hq * D * (n * start + n * (n + 1) // 2)


def default_scale(head_dim):
    return 1.0 / math.sqrt(head_dim)
