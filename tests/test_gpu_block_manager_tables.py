"""Block tables produced by the reference's own ``BlockSpaceManager`` (nanoPD/block_manager/block_manager.py:56-115)
fed to the store and decode-attention ops.

The fixture tests/golden/block_manager_tables.json was written by tests/golden/make_golden_block_tables.py, which
drives the reference's allocator through a small serving scenario: stack-ordered ids (the first sequence holds the
highest), ids of a freed sequence handed to the next one, growth by ``append_slot`` during decode, and a fork whose
child names the same physical blocks as its parent until copy-on-write separates the last one.  Every step is run
on the GPU with exactly those tables and compared with the oracle evaluated on each sequence's tokens laid out
contiguously, so a wrong table walk cannot hide."""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from nanopd_b200 import kv_transfer, paged_forward
from oracle import paged_oracle

FIXTURE = json.loads((Path(__file__).resolve().parent / "golden" / "block_manager_tables.json").read_text())


def test_fixture_shows_the_allocator_behaviours():
    """CPU: the fixture really contains what it is for."""
    ev = FIXTURE["events"]
    prefills = [e for e in ev if e["kind"] == "prefill"]
    assert prefills[0]["block_table"] == [47, 46, 45]                    # stack order: highest ids first
    freed = prefills[1]["block_table"][0]
    assert prefills[4]["block_table"][0] == freed                        # a freed id is reused first
    fork = next(e for e in ev if e["kind"] == "fork")
    parent_table = next(d for e in ev if e["kind"] == "decode" for d in e["decodes"] if d["seq_id"] == fork["parent"])
    assert fork["block_table"][:7] == parent_table["block_table"][:7]    # shared physical blocks
    cows = [c for e in ev if e["kind"] == "decode" for c in e["copy_on_write"]]
    assert len(cows) == 1 and cows[0]["old"] != cows[0]["new"]
    grown = [len(d["block_table"]) for e in ev if e["kind"] == "decode" for d in e["decodes"] if d["seq_id"] == 3]
    assert grown[0] == 1 and grown[-1] == 2                              # append_slot grew it at position 16
    for e in ev:
        for d in e.get("decodes", []):
            assert all(0 <= b < FIXTURE["num_blocks"] for b in d["block_table"])
            assert d["position"] // FIXTURE["block_size"] < len(d["block_table"])


def test_step_context_packs_the_tables_like_the_reference_caller():
    """CPU: ``build_step_context`` on a recorded step gives the zero-padded table, ``seq_lens = position + 1`` and
    positions the reference builds per layer (nanoPD/engine/model_runner.py:176-187)."""
    step = [e for e in FIXTURE["events"] if e["kind"] == "decode"][-1]
    ctx = {"num_prefill_tokens": 0, "num_decode_tokens": len(step["decodes"]), "prefills": [],
           "decodes": [{"block_table": d["block_table"], "position": d["position"]} for d in step["decodes"]]}
    sc = paged_forward.build_step_context(ctx, "cpu", block_size=FIXTURE["block_size"])
    max_blocks = max(len(d["block_table"]) for d in step["decodes"])
    want = torch.zeros(len(step["decodes"]), max_blocks, dtype=torch.int32)
    for i, d in enumerate(step["decodes"]):
        want[i, :len(d["block_table"])] = torch.tensor(d["block_table"], dtype=torch.int32)
    assert torch.equal(sc.decode_tables, want)
    assert sc.decode_seq_lens.tolist() == [d["position"] + 1 for d in step["decodes"]]
    assert sc.decode_positions.tolist() == [d["position"] for d in step["decodes"]]


def _oracle_row(q, k_log, v_log, B, scale):
    """Decode attention of one sequence whose tokens sit in consecutive blocks 0, 1, 2, ... of a private pool."""
    Hkv, n, D = k_log.shape
    nblk = (n + B - 1) // B
    kc = torch.zeros(nblk, Hkv, B, D, dtype=k_log.dtype)
    vc = torch.zeros_like(kc)
    ids = torch.arange(nblk, dtype=torch.int32)
    paged_oracle.kv_store(kc, vc, k_log, v_log, ids.unsqueeze(0).expand(n, -1), torch.arange(n, dtype=torch.int32))
    return paged_oracle.paged_decode_attention(q, kc, vc, ids.unsqueeze(0), torch.tensor([n], dtype=torch.int32), scale)


@pytest.mark.gpu
def test_allocator_tables_through_store_and_attention(kernels):
    from conftest import TOL
    dtype = torch.float16
    B, nb = FIXTURE["block_size"], FIXTURE["num_blocks"]
    Hq, Hkv, D = 8, 2, 128
    scale = D ** -0.5
    g = torch.Generator().manual_seed(77)
    dev = "cuda:0"
    k_cache = torch.full((nb, Hkv, B, D), float("nan"), dtype=dtype, device=dev)       # unwritten slots are poison
    v_cache = torch.full_like(k_cache, float("nan"))
    pool_k, pool_v = k_cache.unsqueeze(0), v_cache.unsqueeze(0)                        # [1, blocks, ...] views
    logical = {}                                                                       # seq id -> (k, v) [Hkv, n, D]
    steps_checked = 0
    for e in FIXTURE["events"]:
        if e["kind"] == "prefill":
            n = e["prompt_len"]
            k = torch.randn(Hkv, n, D, generator=g).to(dtype)
            v = torch.randn(Hkv, n, D, generator=g).to(dtype)
            logical[e["seq_id"]] = (k, v)
            bt = torch.tensor(e["block_table"], dtype=torch.int32, device=dev)
            # the caller's prefill store: the prompt's table repeated per token (nanoPD/engine/model_runner.py:132-150)
            kernels.paged_kv_store(k_cache, v_cache, k.to(dev), v.to(dev), bt.unsqueeze(0).expand(n, -1),
                                   torch.arange(n, dtype=torch.int32, device=dev))
        elif e["kind"] == "free":
            del logical[e["seq_id"]]
        elif e["kind"] == "fork":
            pk, pv = logical[e["parent"]]
            assert pk.size(1) == e["tokens_shared"]
            logical[e["child"]] = (pk.clone(), pv.clone())
        else:
            for c in e["copy_on_write"]:        # the copy append_slot asks its caller for (block_manager.py:72-81)
                kv_transfer.transfer_kv(pool_k, pool_v, pool_k, pool_v, [c["old"]], dst_block_table=[c["new"]])
            decodes = e["decodes"]
            Dn = len(decodes)
            q = torch.randn(Dn, Hq, D, generator=g).to(dtype)
            k_new = torch.randn(Hkv, Dn, D, generator=g).to(dtype)
            v_new = torch.randn(Hkv, Dn, D, generator=g).to(dtype)
            # tables, lengths and positions as the reference's decode branch packs them (model_runner.py:176-187)
            max_blocks = max(len(d["block_table"]) for d in decodes)
            tables = torch.zeros(Dn, max_blocks, dtype=torch.int32)
            for i, d in enumerate(decodes):
                tables[i, :len(d["block_table"])] = torch.tensor(d["block_table"], dtype=torch.int32)
            positions = torch.tensor([d["position"] for d in decodes], dtype=torch.int32)
            tables_d, pos_d = tables.to(dev), positions.to(dev)
            kernels.paged_kv_store(k_cache, v_cache, k_new.to(dev), v_new.to(dev), tables_d, pos_d)
            out = torch.zeros(Dn, Hq, D, dtype=dtype, device=dev)
            kernels.paged_attention_forward(out, q.to(dev), k_cache, v_cache, tables_d, pos_d + 1, scale, B, max_blocks)
            out = out.float().cpu()
            for i, d in enumerate(decodes):
                k_log, v_log = logical[d["seq_id"]]
                assert k_log.size(1) == d["position"], "the fixture's position is the sequence's token count"
                k_log = torch.cat((k_log, k_new[:, i:i + 1]), dim=1)
                v_log = torch.cat((v_log, v_new[:, i:i + 1]), dim=1)
                logical[d["seq_id"]] = (k_log, v_log)
                want = _oracle_row(q[i:i + 1], k_log, v_log, B, scale)
                err = (out[i:i + 1] - want).abs().max().item()
                assert err <= TOL[dtype], f"sequence {d['seq_id']} at position {d['position']}: max-abs error {err}"
            steps_checked += 1
    assert steps_checked == 18
    # the pages themselves: every sequence's tokens sit bit-exactly where its final table says
    last = [e for e in FIXTURE["events"] if e["kind"] == "decode"][-1]
    kc, vc = k_cache.cpu(), v_cache.cpu()
    for d in last["decodes"]:
        k_log, v_log = logical[d["seq_id"]]
        for t in range(k_log.size(1)):
            blk, off = d["block_table"][t // B], t % B
            assert torch.equal(kc[blk, :, off], k_log[:, t]) and torch.equal(vc[blk, :, off], v_log[:, t])
