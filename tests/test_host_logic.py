"""CPU: host-side logic — workload builders, sharding, argument checks of the drop-in ops."""
import numpy as np
import pytest
import torch

from nanopd_b200 import workloads


def test_config1_shape_and_determinism():
    a = workloads.make_config1(seed=0)
    b = workloads.make_config1(seed=0)
    assert a.query.shape == (8, 12, 128) and a.query.dtype == torch.float16
    assert a.k_cache.shape == (256, 2, 16, 128)
    assert torch.equal(a.query, b.query) and torch.equal(a.block_tables, b.block_tables)
    lens = a.ctx_lens.tolist()
    assert all(16 <= l <= 512 for l in lens)
    # tables are disjoint slices of a permutation of the pool and have room for one more token
    used = []
    for s, l in enumerate(lens):
        nb = (l + 1 + 15) // 16
        used += a.block_tables[s, :nb].tolist()
        assert a.block_tables[s, nb:].eq(0).all()
    assert len(set(used)) == len(used) and max(used) < 256


def test_config2_length_distribution():
    lens = workloads.config2_lens(256, seed=0)
    assert lens.min() >= 32 and lens.max() <= 8192 and len(lens) == 256
    assert 700 < np.median(lens) < 1500


def test_config3_structure():
    m = workloads.make_config3(seed=0, num_prompts=2, prompt_lo=40, prompt_hi=90, chunk=32,
                               num_decode=3, decode_lo=5, decode_hi=40)
    assert len(m.prompt_lens) == 2
    for L in m.prompt_lens:
        chunks = [c for c in m.chunks if c.block_table.numel() == (L + 15) // 16]
        assert sum(c.num_tokens for c in chunks) >= L or len(set(m.prompt_lens)) == 1
    starts = [c.start_position for c in m.chunks]
    assert 0 in starts and all(s % 32 == 0 for s in starts)
    all_ids = torch.cat([m.decode.block_tables.flatten()] + [c.block_table for c in m.chunks])
    assert int(all_ids.max()) < m.decode.k_cache.size(0)


def test_poison_marks_only_unwritten_slots():
    b = workloads.make_decode_batch([5, 16, 17], 4, 2, 64, 16, torch.float16, seed=1)
    workloads.poison_unwritten_slots(b)
    for s, l in enumerate(b.ctx_lens.tolist()):
        for pos in range(l):
            blk = int(b.block_tables[s, pos // 16])
            assert not torch.isnan(b.k_cache[blk, :, pos % 16]).any()
        blk = int(b.block_tables[s, l // 16])
        assert torch.isnan(b.v_cache[blk, :, l % 16]).all()


@pytest.mark.parametrize("n,world", [(256, 1), (256, 2), (256, 8), (10, 4), (3, 8)])
def test_shard_sequences_partitions_the_batch(n, world):
    seen = []
    for r in range(world):
        seen += list(workloads.shard_sequences(n, r, world))
    assert seen == list(range(n))
    sizes = [len(workloads.shard_sequences(n, r, world)) for r in range(world)]
    assert max(sizes) - min(sizes) <= 1


def test_ops_reject_cpu_tensors_with_runtime_error():
    import paged_kernels
    q = torch.zeros(1, 4, 128, dtype=torch.float16)
    kc = torch.zeros(2, 4, 16, 128, dtype=torch.float16)
    bt = torch.zeros(1, 1, dtype=torch.int32)
    sl = torch.ones(1, dtype=torch.int32)
    with pytest.raises(RuntimeError):
        paged_kernels.paged_attention_forward(torch.zeros_like(q), q, kc, kc, bt, sl, 1.0, 16, 1)
    with pytest.raises(RuntimeError):
        paged_kernels.paged_kv_store(kc, kc, torch.zeros(4, 1, 128, dtype=torch.float16),
                                     torch.zeros(4, 1, 128, dtype=torch.float16), bt, sl)


def test_kv_transfer_exports_the_reference_module_names():
    """The reference's workers import these at module load (nanoPD/workers/prefill_worker.py:10,
    nanoPD/workers/decode_worker.py:11)."""
    from nanopd_b200.kv_transfer import (PinnedKVBuffer, _check_p2p, extract_kv_to_pinned,  # noqa: F401
                                         load_kv_from_pinned, transfer_kv)
    import inspect
    assert list(inspect.signature(transfer_kv).parameters)[:7] == ["src_k", "src_v", "dst_k", "dst_v", "block_table",
                                                                   "stream", "buf"]
    assert list(inspect.signature(extract_kv_to_pinned).parameters)[:4] == ["k_cache", "v_cache", "block_table", "buf"]
    assert list(inspect.signature(load_kv_from_pinned).parameters)[:5] == ["k_cache", "v_cache", "block_table", "buf",
                                                                          "stream"]
    assert list(inspect.signature(PinnedKVBuffer.__init__).parameters)[1:] == ["num_layers", "num_block", "num_kv_heads",
                                                                               "block_size", "head_dim", "dtype"]


def test_both_module_names_of_the_reference_resolve_to_this_implementation():
    """``paged_kernels`` is what ``ModelRunner.paged_forward`` imports (nanoPD/engine/model_runner.py:94,270),
    ``paged_attn`` what the older kernel tests import (nanoPD/paged_attention/tests/test_paged_attention.py:18);
    the positional signature of the attention op is the reference's."""
    import inspect

    import paged_attn
    import paged_kernels
    assert paged_attn.paged_attention_forward is paged_kernels.paged_attention_forward
    assert list(inspect.signature(paged_kernels.paged_attention_forward).parameters)[:9] == [
        "out", "query", "key_cache", "value_cache", "block_tables", "seq_lens", "scale", "block_size",
        "max_num_blocks_per_seq"]
    assert list(inspect.signature(paged_kernels.paged_kv_store).parameters) == [
        "k_cache", "v_cache", "k_src", "v_src", "block_tables", "positions"]
