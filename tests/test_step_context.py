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
