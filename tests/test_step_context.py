"""CPU: the once-per-step packing of the scheduler's context dict reproduces what the reference builds per
layer (nanoPD/engine/model_runner.py:132-140, 176-187)."""
import pytest
import torch

from nanopd_b200 import paged_forward


def _reference_decode_tensors(decodes):
    """The reference's own loop, on the CPU."""
    max_blocks = max(len(d["block_table"]) for d in decodes)
    block_tables = torch.zeros(len(decodes), max_blocks, dtype=torch.int32)
    seq_lens = torch.zeros(len(decodes), dtype=torch.int32)
    for i, d in enumerate(decodes):
        bt = d["block_table"]
        block_tables[i, :len(bt)] = torch.tensor(bt, dtype=torch.int32)
        seq_lens[i] = d["position"] + 1
    positions = torch.tensor([d["position"] for d in decodes], dtype=torch.int32)
    return block_tables, seq_lens, positions


def test_decode_tables_equal_the_reference_loop():
    decodes = [{"block_table": [7, 3, 9], "position": 40}, {"block_table": [1], "position": 0},
               {"block_table": [5, 6, 2, 8, 4], "position": 79}]
    ctx = {"num_prefill_tokens": 0, "num_decode_tokens": 3, "prefills": [], "decodes": decodes}
    sc = paged_forward.build_step_context(ctx, "cpu")
    bt, sl, pos = _reference_decode_tensors(decodes)
    assert torch.equal(sc.decode_tables, bt) and torch.equal(sc.decode_seq_lens, sl)
    assert torch.equal(sc.decode_positions, pos)
    assert sc.prefill_tables is None and sc.num_decode_tokens == 3


def test_prefill_chunks_are_packed_in_order():
    prefills = [{"block_table": [4, 1, 0], "start_position": 0, "num_tokens": 40},
                {"block_table": [9, 8, 7, 6, 5], "start_position": 64, "num_tokens": 10}]
    ctx = {"num_prefill_tokens": 50, "num_decode_tokens": 1, "prefills": prefills,
           "decodes": [{"block_table": [2, 3], "position": 17}]}
    sc = paged_forward.build_step_context(ctx, "cpu")
    assert sc.prefill_offsets == [0, 40] and sc.prefill_tokens == [40, 10] and sc.prefill_starts == [0, 64]
    assert sc.prefill_tables.tolist() == [[4, 1, 0, 0, 0], [9, 8, 7, 6, 5]]
    # positions as the reference's per-prompt arange (model_runner.py:134-138)
    assert sc.prefill_positions.tolist() == list(range(40)) + list(range(64, 74))
    assert sc.decode_seq_lens.tolist() == [18]
    assert sc.h2d_bytes > 0 and sc.h2d_bytes % 256 == 0


def test_inconsistent_contexts_raise():
    with pytest.raises(RuntimeError):
        paged_forward.build_step_context({"num_prefill_tokens": 5, "num_decode_tokens": 0,
                                          "prefills": [{"block_table": [0], "start_position": 0, "num_tokens": 4}],
                                          "decodes": []}, "cpu")
    with pytest.raises(RuntimeError):   # position beyond the table
        paged_forward.build_step_context({"num_prefill_tokens": 0, "num_decode_tokens": 1, "prefills": [],
                                          "decodes": [{"block_table": [0], "position": 16}]}, "cpu")
    with pytest.raises(RuntimeError):   # chunk beyond the table
        paged_forward.build_step_context({"num_prefill_tokens": 20, "num_decode_tokens": 0,
                                          "prefills": [{"block_table": [0], "start_position": 0, "num_tokens": 20}],
                                          "decodes": []}, "cpu")


def _ctx(chunk_tokens, chunk_start, decode_positions):
    prefills = [{"block_table": list(range(400)), "start_position": chunk_start, "num_tokens": chunk_tokens}] if chunk_tokens else []
    decodes = [{"block_table": list(range(400)), "position": p} for p in decode_positions]
    return {"num_prefill_tokens": chunk_tokens, "num_decode_tokens": len(decodes), "prefills": prefills, "decodes": decodes}


def test_sm_split_of_a_mixed_step():
    split = lambda ctx: paged_forward._sm_split(paged_forward.build_step_context(ctx, "cpu"), 32, 8, 128, 2, 148)
    assert split(_ctx(0, 0, [1000] * 64)) is None                     # decode only
    assert split(_ctx(512, 2048, [])) is None                         # prefill only
    assert split(_ctx(16, 0, [5] * 4)) is None                        # too little work to pay for a fork and join
    # configuration 3's shape: a 512-token chunk deep into its prompt + 128 long decode sequences
    share = split(_ctx(512, 2048, [2200] * 128))
    assert share is not None and 16 <= share <= 148 - 32
    assert 148 - share >= 100                                         # decode keeps enough SMs to stay HBM-bound
    # more prompt work moves SMs to the chunk kernel, never the other way
    shares = [split(_ctx(512, start, [2200] * 128)) for start in (2048, 4096, 5600)]
    assert shares == sorted(shares)
    assert paged_forward._sm_split(paged_forward.build_step_context(_ctx(512, 2048, [2200] * 128), "cpu"), 32, 8, 128, 2, 32) is None
