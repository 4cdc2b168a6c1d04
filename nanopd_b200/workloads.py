"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

The reference measures on no public dataset: its tests and benches build inputs with
``torch.manual_seed`` + ``torch.randn`` (nanoPD/paged_attention/tests/test_paged_kernels.py:102-139).
These builders do the same for the five named configurations: N(0,1) values cast to the
working dtype, ragged context lengths, and block tables cut from a seeded random
permutation of the block pool (the reference's allocator hands out ids from a LIFO free
list, nanoPD/block_manager/block_manager.py:16-26; a permutation is the adversarial case).

Lengths and permutations come from ``numpy.random.default_rng(seed)`` on the host, so they
are identical on every device; tensor values come from a ``torch.Generator`` on the target
device (CPU values and CUDA values differ, which is fine: parity tests build on the CPU and
copy to the GPU).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np
import torch


@dataclass
class DecodeBatch:
    """One decode step over a paged pool, in the layout the ops take."""
    query: torch.Tensor          # [S, Hq, D]
    k_cache: torch.Tensor        # [blocks, Hkv, B, D]
    v_cache: torch.Tensor
    block_tables: torch.Tensor   # int32 [S, max_blk], zero padded
    ctx_lens: torch.Tensor       # int32 [S]  tokens already in the pool
    k_new: torch.Tensor          # [Hkv, S, D]  the step's new token per sequence
    v_new: torch.Tensor
    scale: float
    block_size: int
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    name: str = ""

    @property
    def positions(self) -> torch.Tensor:
        """Slot of the new token (== ctx_len), as the caller passes it to the store."""
        return self.ctx_lens

    @property
    def seq_lens_after_store(self) -> torch.Tensor:
        """``position + 1``: what the caller hands to attention after the store
        (nanoPD/engine/model_runner.py:183)."""
        return self.ctx_lens + 1

    @property
    def max_blocks(self) -> int:
        return self.block_tables.size(1)


@dataclass
class PrefillChunk:
    query: torch.Tensor          # [n, Hq, D]
    k_new: torch.Tensor          # [Hkv, n, D]
    v_new: torch.Tensor
    block_table: torch.Tensor    # int32 [nblk]
    start_position: int
    num_tokens: int


@dataclass
class MixedBatch:
    """Chunked prefill of several prompts co-scheduled with a decode batch on one pool."""
    chunks: List[PrefillChunk]
    decode: DecodeBatch
    prompt_lens: List[int] = field(default_factory=list)


def _randn(shape, dtype, device, gen, chunk_elems=1 << 27):
    """N(0,1) in fp32 cast to dtype, generated in slabs so the fp32 temporary stays small."""
    out = torch.empty(shape, dtype=dtype, device=device)
    flat = out.view(-1)
    n = flat.numel()
    for lo in range(0, n, chunk_elems):
        hi = min(n, lo + chunk_elems)
        flat[lo:hi] = torch.randn(hi - lo, generator=gen, device=device, dtype=torch.float32).to(dtype)
    return out


def _tables_from_permutation(nblocks_per_seq, perm, device):
    S = len(nblocks_per_seq)
    max_blk = max(1, int(max(nblocks_per_seq)))
    bt = np.zeros((S, max_blk), dtype=np.int32)
    off = 0
    for s, nb in enumerate(nblocks_per_seq):
        bt[s, :nb] = perm[off:off + nb]
        off += nb
    return torch.from_numpy(bt).to(device)


def poison_unwritten_slots(batch: DecodeBatch, value=float("nan")):
    """Overwrite every pool slot no sequence has written with ``value`` (NaN by default).

    An attention kernel that reads a slot at or beyond a sequence's length, or a block
    no table names, then shows NaN in its output.  Slot ``ctx_len`` (the one the store
    is about to fill) is poisoned too.
    """
    B = batch.block_size
    blocks = batch.k_cache.size(0)
    written = torch.zeros(blocks, B, dtype=torch.bool)
    bt = batch.block_tables.cpu()
    lens = batch.ctx_lens.cpu().tolist()
    for s, l in enumerate(lens):
        nfull, rem = divmod(l, B)
        if nfull:
            written[bt[s, :nfull].long()] = True
        if rem:
            written[int(bt[s, nfull]), :rem] = True
    mask = (~written).to(batch.k_cache.device)
    batch.k_cache.permute(0, 2, 1, 3)[mask] = value
    batch.v_cache.permute(0, 2, 1, 3)[mask] = value
    return batch


def make_decode_batch(ctx_lens, num_q_heads, num_kv_heads, head_dim, block_size, dtype,
                      device="cpu", seed=0, pool_blocks: Optional[int] = None,
                      permute=True, name="") -> DecodeBatch:
    """Pool + tables for the given context lengths; every table has room for one more token."""
    rng = np.random.default_rng(seed)
    ctx = np.asarray(ctx_lens, dtype=np.int64)
    S = len(ctx)
    nblk = (ctx + 1 + block_size - 1) // block_size
    need = int(nblk.sum())
    if pool_blocks is None:
        pool_blocks = need
    if need > pool_blocks:
        raise ValueError(f"contexts need {need} blocks, pool has {pool_blocks}")
    perm = rng.permutation(pool_blocks) if permute else np.arange(pool_blocks)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    bt = _tables_from_permutation(nblk.tolist(), perm, device)
    shape = (pool_blocks, num_kv_heads, block_size, head_dim)
    return DecodeBatch(
        query=_randn((S, num_q_heads, head_dim), dtype, device, gen),
        k_cache=_randn(shape, dtype, device, gen),
        v_cache=_randn(shape, dtype, device, gen),
        block_tables=bt,
        ctx_lens=torch.from_numpy(ctx.astype(np.int32)).to(device),
        k_new=_randn((num_kv_heads, S, head_dim), dtype, device, gen),
        v_new=_randn((num_kv_heads, S, head_dim), dtype, device, gen),
        scale=float(head_dim) ** -0.5,
        block_size=block_size, num_q_heads=num_q_heads, num_kv_heads=num_kv_heads,
        head_dim=head_dim, name=name)


def config1_lens(seed=0):
    """8 context lengths uniform in [16, 512] that fit a 256-block pool at block size 16."""
    rng = np.random.default_rng(seed)
    while True:
        ctx = rng.integers(16, 513, size=8)
        if int(((ctx + 1 + 15) // 16).sum()) <= 256:
            return ctx


def make_config1(device="cpu", seed=0) -> DecodeBatch:
    """Qwen2-1.5B attention shape: 12 q heads, 2 kv heads, D 128, fp16, block 16, 8 sequences."""
    return make_decode_batch(config1_lens(seed), 12, 2, 128, 16, torch.float16,
                             device=device, seed=seed, pool_blocks=256,
                             name="cfg1-qwen2-1.5b-s8-fp16")


def config2_lens(batch=256, seed=0):
    """Lognormal (median 1024, sigma 0.8) context lengths clipped to [32, 8192]."""
    rng = np.random.default_rng(seed)
    ctx = np.rint(np.exp(rng.normal(np.log(1024.0), 0.8, size=batch)))
    return np.clip(ctx, 32, 8192).astype(np.int64)


def make_config2(device="cpu", seed=0, batch=256) -> DecodeBatch:
    """Qwen3-8B attention shape: 32 q heads, 8 kv heads, D 128, bf16, block 16, batch 256."""
    return make_decode_batch(config2_lens(batch, seed), 32, 8, 128, 16, torch.bfloat16,
                             device=device, seed=seed,
                             name=f"cfg2-qwen3-8b-s{batch}-bf16-lognormal")


def make_config3(device="cpu", seed=0, num_prompts=4, prompt_lo=1024, prompt_hi=4096,
                 chunk=512, num_decode=128, decode_lo=256, decode_hi=4096,
                 dtype=torch.bfloat16) -> MixedBatch:
    """Chunked prefill (512-token chunks) of 4 prompts plus 128 decode sequences, Qwen3-8B shape.

    Prompt pages live in the same pool as the decode sequences' pages; each chunk carries
    its own new K/V rows, to be stored before the chunk attends (the caller's order,
    nanoPD/engine/model_runner.py:132-168).
    """
    Hq, Hkv, D, B = 32, 8, 128, 16
    rng = np.random.default_rng(seed + 7919)
    prompt_lens = rng.integers(prompt_lo, prompt_hi + 1, size=num_prompts).tolist()
    dec_ctx = rng.integers(decode_lo, decode_hi + 1, size=num_decode)
    dec_nblk = (dec_ctx + 1 + B - 1) // B
    prm_nblk = [(l + B - 1) // B for l in prompt_lens]
    pool_blocks = int(dec_nblk.sum()) + sum(prm_nblk)
    perm = rng.permutation(pool_blocks)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    shape = (pool_blocks, Hkv, B, D)
    k_cache = _randn(shape, dtype, device, gen)
    v_cache = _randn(shape, dtype, device, gen)
    dec_bt = _tables_from_permutation(dec_nblk.tolist(), perm, device)
    decode = DecodeBatch(
        query=_randn((num_decode, Hq, D), dtype, device, gen),
        k_cache=k_cache, v_cache=v_cache, block_tables=dec_bt,
        ctx_lens=torch.from_numpy(dec_ctx.astype(np.int32)).to(device),
        k_new=_randn((Hkv, num_decode, D), dtype, device, gen),
        v_new=_randn((Hkv, num_decode, D), dtype, device, gen),
        scale=float(D) ** -0.5, block_size=B, num_q_heads=Hq, num_kv_heads=Hkv, head_dim=D,
        name="cfg3-decode-part")
    chunks: List[PrefillChunk] = []
    off = int(dec_nblk.sum())
    for L, nb in zip(prompt_lens, prm_nblk):
        table = torch.from_numpy(perm[off:off + nb].astype(np.int32)).to(device)
        off += nb
        for start in range(0, L, chunk):
            n = min(chunk, L - start)
            chunks.append(PrefillChunk(
                query=_randn((n, Hq, D), dtype, device, gen),
                k_new=_randn((Hkv, n, D), dtype, device, gen),
                v_new=_randn((Hkv, n, D), dtype, device, gen),
                block_table=table, start_position=start, num_tokens=n))
    return MixedBatch(chunks=chunks, decode=decode, prompt_lens=prompt_lens)


def shard_sequences(num_seqs: int, rank: int, world_size: int) -> range:
    """Contiguous batch shard of a decode batch for one replica (no data-path collective)."""
    base, rem = divmod(num_seqs, world_size)
    lo = rank * base + min(rank, rem)
    return range(lo, lo + base + (1 if rank < rem else 0))
