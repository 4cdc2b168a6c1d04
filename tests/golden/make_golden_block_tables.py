"""Generates tests/golden/block_manager_tables.json by driving the REFERENCE's own allocator.

Run where the reference checkout is at hand, its path in NANOPD_REFERENCE:
    NANOPD_REFERENCE=<checkout> python tests/golden/make_golden_block_tables.py

It imports ``BlockSpaceManager`` and ``Sequence`` from nanoPD/block_manager (pure Python) and plays a small
serving scenario through them — prompts allocated one after another (the free list is a stack, so the first
sequence gets the highest ids, block_manager.py:16-26), a sequence freed and its ids handed to the next one,
``append_slot`` growth at block boundaries during decode (block_manager.py:72-98), and a ``fork`` whose child
shares every block of its parent until its first ``append_slot`` copies the last one
(block_manager.py:91-96,100-105).  What the kernels would be given at every step — the block table and position
of every running sequence, and the (old, new) pairs of copy-on-write — is written down as the fixture.
"""
import json
import os
import sys
from pathlib import Path

if "NANOPD_REFERENCE" not in os.environ:
    sys.exit("set NANOPD_REFERENCE to the reference checkout")
REF = Path(os.environ["NANOPD_REFERENCE"]) / "nanoPD"
sys.path.insert(0, str(REF))
from block_manager.block_manager import BlockSpaceManager  # noqa: E402
from block_manager.sequence import Sequence, SequenceGroup  # noqa: E402

BLOCK, POOL = 16, 48
OUT = Path(__file__).resolve().parent / "block_manager_tables.json"


def main():
    bm = BlockSpaceManager(block_size=BLOCK, num_gpu_blocks=POOL)
    seqs = {}

    def admit(seq_id, prompt_len):
        seq = Sequence(seq_id, list(range(1000 * seq_id, 1000 * seq_id + prompt_len)), BLOCK)
        group = SequenceGroup(str(seq_id), [seq])
        assert bm.can_allocate(group)
        bm.allocate(group)
        seq.num_computed_tokens = prompt_len            # what prefill leaves behind (prefill_worker.py:80)
        seqs[seq_id] = seq
        return {"seq_id": seq_id, "prompt_len": prompt_len, "block_table": bm.get_block_table(seq)}

    events = []
    events.append({"kind": "prefill", **admit(0, 37)})
    events.append({"kind": "prefill", **admit(1, 16)})
    events.append({"kind": "prefill", **admit(2, 100)})
    events.append({"kind": "prefill", **admit(3, 1)})
    bm.free(seqs.pop(1))                                # its block goes back on top of the stack
    events.append({"kind": "free", "seq_id": 1})
    events.append({"kind": "prefill", **admit(4, 64)})  # takes the freed id first

    def decode_step(ids):
        step = {"kind": "decode", "decodes": [], "copy_on_write": []}
        for sid in ids:
            seq = seqs[sid]
            cow = bm.append_slot(seq)                   # decode_worker.py:79
            if cow is not None:
                step["copy_on_write"].append({"seq_id": sid, "old": cow[0], "new": cow[1]})
            step["decodes"].append({"seq_id": sid, "block_table": bm.get_block_table(seq),
                                    "position": seq.num_computed_tokens})
            seq.append_token_id(7)
            seq.num_computed_tokens += 1                # decode_worker.py:112
        events.append(step)

    for _ in range(14):                                 # seq 3 crosses a block boundary at position 16, seq 0 at 48
        decode_step([0, 2, 3, 4])
    # fork: the child shares all of its parent's blocks
    parent = seqs[2]
    child = Sequence(5, [], BLOCK)
    child.num_computed_tokens = parent.num_computed_tokens
    bm.fork(parent, child)
    seqs[5] = child
    events.append({"kind": "fork", "parent": 2, "child": 5, "tokens_shared": parent.num_computed_tokens,
                   "block_table": bm.get_block_table(child)})
    for _ in range(4):                                  # the first step copies the shared last block for the
        decode_step([0, 2, 5, 3, 4])                    # sequence that appends first
    free_after = bm.num_free_blocks
    OUT.write_text(json.dumps({"block_size": BLOCK, "num_blocks": POOL, "events": events,
                               "free_blocks_at_end": free_after}, indent=1))
    n_cow = sum(len(e.get("copy_on_write", [])) for e in events)
    print(f"wrote {OUT.name}: {len(events)} events, {n_cow} copy-on-write pairs, {free_after} blocks free at the end")


if __name__ == "__main__":
    main()
