"""GPU: paged decode attention through the C ABI against the fp32 oracle.

Tolerance (max-abs against the fp32-accumulated oracle): 2e-3 for fp16, 1e-2 for bf16."""
import math
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN, TOL, load_decode_cases
from nanopd_b200 import workloads
from oracle import paged_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
CASES = load_decode_cases()


def run_kernel(kernels, q, kc, vc, bt, sl, scale, block_size=None):
    """Same wrapper as the reference's run_kernel (model_runner.py:269-277)."""
    out = torch.zeros_like(q)
    kernels.paged_attention_forward(out, q, kc, vc, bt, sl, scale, block_size or kc.size(2), bt.size(1))
    torch.cuda.synchronize()
    return out


def check(kernels, q, kc, vc, bt, sl, scale, tol=None):
    want = paged_oracle.paged_decode_attention(q, kc, vc, bt, sl, scale)
    got = run_kernel(kernels, q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), sl.to(DEV), scale).float().cpu()
    assert torch.isfinite(got).all()
    err = (got - want).abs().max().item()
    assert err <= (tol or TOL[q.dtype]), f"max abs err {err}"
    return err


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_golden_reference_cases(kernels, case):
    """Inputs and outputs produced by the reference's own ref_paged_attention."""
    got = run_kernel(kernels, case["q"].to(DEV), case["k"].to(DEV), case["v"].to(DEV),
                     case["block_tables"].to(DEV), case["seq_lens"].to(DEV), case["scale"]).float().cpu()
    assert (got - case["out_fp32"]).abs().max().item() <= TOL[case["dtype"]]
    # and the reference tests' own criterion (atol = rtol = 1e-2 on the rounded output)
    torch.testing.assert_close(got, case["ref_out"].float(), atol=1e-2, rtol=1e-2)


def _inputs(S, Hq, Hkv, D, lens, B, dtype, seed=42, permute=True, extra_blocks=3):
    b = workloads.make_decode_batch([l - 1 for l in lens], Hq, Hkv, D, B, dtype, seed=seed, permute=permute,
                                    pool_blocks=sum((l + B - 1) // B for l in lens) + extra_blocks)
    return b.query, b.k_cache, b.v_cache, b.block_tables, torch.tensor(lens, dtype=torch.int32), b.scale


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("S,Hq,Hkv,lens", [(1, 1, 1, [8]), (3, 4, 4, [32, 48, 64]), (2, 32, 8, [64, 48])])
def test_reference_case_list(kernels, dtype, S, Hq, Hkv, lens):
    """The case list of the reference tests (test_paged_kernels.py:160-189) on permuted tables."""
    check(kernels, *_inputs(S, Hq, Hkv, 128, lens, 16, dtype))


@pytest.mark.parametrize("seq_len", [1, 2, 15, 16, 17, 31, 32, 33, 64, 128, 512, 1000])
def test_various_seq_lens(kernels, seq_len):
    check(kernels, *_inputs(1, 4, 4, 128, [seq_len], 16, torch.float16))


@pytest.mark.parametrize("block_size", [4, 8, 16, 32])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_block_sizes(kernels, block_size, dtype):
    check(kernels, *_inputs(4, 4, 4, 128, [48, 32, 7, 131], block_size, dtype))


@pytest.mark.parametrize("S,Hq,Hkv,D,B,lens", [
    (8, 12, 2, 128, 16, [16, 100, 512, 333, 1, 47, 250, 64]),          # the shape of configuration 1
    (16, 32, 8, 128, 16, [200] * 16),                                  # the reference's operating size; one sequence is emptied below
    (1, 32, 8, 128, 16, [1024]),                                       # the longest context the small form takes
    (2, 32, 8, 128, 16, [1025, 3]),                                    # one token more: both runs take the streaming form
    (3, 40, 2, 128, 16, [5, 700, 33]),                                 # group 20: two virtual kv heads per head
    (5, 8, 2, 256, 32, [31, 32, 33, 1000, 7]),
    (4, 16, 16, 64, 8, [9, 130, 77, 1500]),
])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_small_batch_form_and_streaming_form_agree(kernels, S, Hq, Hkv, D, B, lens, dtype):
    """Small batches of short sequences take the form with one CTA per (sequence, kv head) and a merge in shared
    memory; the private flag bit 2 forces the streaming form (equal-work split, merge through the workspace) on the
    same inputs.  Both must match the oracle; their results differ at most by the order of the merges."""
    q, kc, vc, bt, sl, scale = _inputs(S, Hq, Hkv, D, lens, B, dtype)
    if S == 16:
        sl[5] = 0                                                       # an empty sequence: a zero row
    want = paged_oracle.paged_decode_attention(q, kc, vc, bt, sl, scale)
    qd, kd, vd, btd, sld = q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), sl.to(DEV)
    outs = []
    for flags in (0, 4):
        out = torch.full_like(qd, float("nan"))
        kernels.paged_attention_forward(out, qd, kd, vd, btd, sld, scale, B, btd.size(1), _flags=flags)
        torch.cuda.synchronize()
        got = out.float().cpu()
        assert torch.isfinite(got).all()
        assert (got - want).abs().max().item() <= TOL[dtype]
        outs.append(got)
    assert (outs[0] - outs[1]).abs().max().item() <= TOL[dtype]


@pytest.mark.parametrize("D", [64, 128, 256])
def test_block_size_4(kernels, D):
    """Blocks of 4 tokens (the smallest size of the reference's kernel tests,
    nanoPD/paged_attention/tests/test_paged_attention.py:192-203): four TMA boxes of 4 rows per 16-token tile."""
    check(kernels, *_inputs(3, 8, 2, D, [24, 16, 77], 4, torch.float16))
    check(kernels, *_inputs(2, 4, 4, D, [3, 130], 4, torch.bfloat16))


@pytest.mark.parametrize("D", [64, 128, 256])
def test_head_dims(kernels, D):
    check(kernels, *_inputs(3, 8, 2, D, [100, 17, 260], 16, torch.float16))


@pytest.mark.parametrize("Hq,Hkv", [(1, 1), (6, 1), (8, 1), (12, 2), (12, 1), (16, 1), (32, 2), (24, 1), (32, 1), (5, 1), (20, 1)])
def test_group_sizes(kernels, Hq, Hkv):
    """Groups of 1..32 q heads per kv head, including ones that need two head tiles or a split."""
    check(kernels, *_inputs(3, Hq, Hkv, 128, [77, 16, 300], 16, torch.bfloat16))


def test_config1_store_then_attend_matches_reference_golden(kernels):
    """Configuration 1 in the caller's order: store the new token, then attend with position+1."""
    z = np.load(GOLDEN / "config1_reference_out.npz")
    b = workloads.make_config1(seed=0)
    kc, vc = b.k_cache.to(DEV), b.v_cache.to(DEV)
    bt = b.block_tables.to(DEV)
    kernels.paged_kv_store(kc, vc, b.k_new.to(DEV), b.v_new.to(DEV), bt, b.positions.to(DEV))
    got = run_kernel(kernels, b.query.to(DEV), kc, vc, bt, b.seq_lens_after_store.to(DEV), b.scale).float().cpu()
    assert (got - torch.from_numpy(z["out_fp32"])).abs().max().item() <= TOL[torch.float16]


def test_unwritten_slots_are_never_read(kernels):
    """NaN in every slot beyond a sequence's length and in every unnamed block must not reach the output."""
    b = workloads.make_decode_batch([5, 16, 17, 100, 1, 255], 8, 2, 128, 16, torch.float16, seed=4,
                                    pool_blocks=40)
    workloads.poison_unwritten_slots(b)
    check(kernels, b.query, b.k_cache, b.v_cache, b.block_tables, b.ctx_lens, b.scale)


def test_empty_and_ragged_batch(kernels):
    """Length 0 gives a zero row (the reference kernel's behaviour); neighbours are unaffected."""
    q, kc, vc, bt, sl, scale = _inputs(5, 8, 2, 128, [40, 1, 300, 1, 16], 16, torch.bfloat16)
    sl = torch.tensor([40, 0, 300, 0, 16], dtype=torch.int32)
    out = torch.full_like(q, 7.0).to(DEV)
    kernels.paged_attention_forward(out, q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), sl.to(DEV), scale, 16, bt.size(1))
    got = out.float().cpu()
    assert got[1].eq(0).all() and got[3].eq(0).all()
    keep = [0, 2, 4]
    want = paged_oracle.paged_decode_attention(q[keep], kc, vc, bt[keep], sl[keep], scale)
    assert (got[keep] - want).abs().max().item() <= TOL[torch.bfloat16]


def test_long_sequences_split_across_many_workers(kernels):
    """Two 8192-token sequences on one kv head: every (sequence, head) is cut into many partials."""
    check(kernels, *_inputs(2, 4, 1, 128, [8192, 5000], 16, torch.bfloat16))


def test_single_long_sequence_mha(kernels):
    check(kernels, *_inputs(1, 2, 2, 128, [20000], 16, torch.float16))


def test_layer_slice_and_padded_tables(kernels):
    """Caches as slices of a 5-D pool; table rows wider than needed, padding never dereferenced."""
    q, kc, vc, bt, sl, scale = _inputs(3, 8, 4, 128, [33, 70, 5], 16, torch.float16)
    pool_k = torch.full((2,) + tuple(kc.shape), float("nan"), dtype=kc.dtype, device=DEV)
    pool_v = torch.full_like(pool_k, float("nan"))
    pool_k[1], pool_v[1] = kc.to(DEV), vc.to(DEV)
    wide = torch.full((3, bt.size(1) + 9), 2 ** 30, dtype=torch.int32)     # poison padding ids
    for s, l in enumerate(sl.tolist()):
        n = (l + 15) // 16
        wide[s, :n] = bt[s, :n]
    got = run_kernel(kernels, q.to(DEV), pool_k[1], pool_v[1], wide.to(DEV), sl.to(DEV), scale).float().cpu()
    want = paged_oracle.paged_decode_attention(q, kc, vc, bt, sl, scale)
    assert (got - want).abs().max().item() <= TOL[torch.float16]


def test_bad_dtypes_raise_runtime_error(kernels):
    """int64 index tensors raise, as the reference pins (test_paged_kernels.py:218-227)."""
    q, kc, vc, bt, sl, scale = [t.to(DEV) if torch.is_tensor(t) else t
                                for t in _inputs(1, 4, 4, 128, [16], 16, torch.float16)]
    out = torch.zeros_like(q)
    with pytest.raises(RuntimeError):
        kernels.paged_attention_forward(out, q, kc, vc, bt.to(torch.int64), sl, scale, 16, bt.size(1))
    with pytest.raises(RuntimeError):
        kernels.paged_attention_forward(out, q, kc, vc, bt, sl.to(torch.int64), scale, 16, bt.size(1))
    with pytest.raises(RuntimeError):
        kernels.paged_attention_forward(out, q, kc.unsqueeze(0), vc, bt, sl, scale, 16, bt.size(1))
    with pytest.raises(RuntimeError):
        kernels.paged_attention_forward(out, q.float(), kc.float(), vc.float(), bt, sl, scale, 16, bt.size(1))


def test_out_of_range_block_id_is_flagged_not_dereferenced(kernels):
    """A table entry outside the pool is redirected to a zero-filled tile and the status word set."""
    q, kc, vc, bt, sl, scale = _inputs(2, 4, 4, 128, [40, 20], 16, torch.float16)
    bad = bt.clone()
    bad[1, 0] = kc.size(0) + 100
    out = run_kernel(kernels, q.to(DEV), kc.to(DEV), vc.to(DEV), bad.to(DEV), sl.to(DEV), scale).float().cpu()
    assert kernels.check_status(raise_on_error=False) & 1
    want = paged_oracle.paged_decode_attention(q[:1], kc, vc, bt[:1], sl[:1], scale)
    assert (out[:1] - want).abs().max().item() <= TOL[torch.float16]
    assert torch.isfinite(out).all()


def test_config2_quarter_batch_vs_oracle(kernels):
    """Qwen3-8B shape, lognormal lengths, 64 sequences: full oracle comparison."""
    b = workloads.make_config2(device=DEV, seed=0, batch=64)
    out = run_kernel(kernels, b.query, b.k_cache, b.v_cache, b.block_tables, b.ctx_lens, b.scale).float().cpu()
    want = paged_oracle.paged_decode_attention(b.query.cpu(), b.k_cache.cpu(), b.v_cache.cpu(),
                                               b.block_tables.cpu(), b.ctx_lens.cpu(), b.scale)
    assert (out - want).abs().max().item() <= TOL[torch.bfloat16]


def test_config2_full_size_vs_oracle(kernels):
    """Configuration 2 at full size (batch 256, ~1.5 GB of K/V): every sequence against the oracle, plus two
    size-independent properties: (i) a sequence's row does not depend on what else is in the batch (different
    work partition, same answer); (ii) rows are convex combinations of V rows, so every output lies inside the
    value range."""
    b = workloads.make_config2(device=DEV, seed=0, batch=256)
    out = run_kernel(kernels, b.query, b.k_cache, b.v_cache, b.block_tables, b.ctx_lens, b.scale)
    assert torch.isfinite(out).all()
    pick = [0, 17, 101, 200, 255, int(b.ctx_lens.argmax()), int(b.ctx_lens.argmin())]
    idx = torch.tensor(pick, device=DEV)
    alone = run_kernel(kernels, b.query[idx].contiguous(), b.k_cache, b.v_cache,
                       b.block_tables[idx].contiguous(), b.ctx_lens[idx].contiguous(), b.scale)
    assert (alone.float() - out[idx].float()).abs().max().item() <= 4e-3
    assert out.float().abs().max().item() <= b.v_cache.float().abs().max().item() * 1.01
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    want = paged_oracle.paged_decode_attention(b.query.cpu(), b.k_cache.cpu(), b.v_cache.cpu(),
                                               b.block_tables.cpu(), b.ctx_lens.cpu(), b.scale)
    assert (out.float().cpu() - want).abs().max().item() <= TOL[torch.bfloat16]


def test_skip_merge_flag_only_affects_split_sequences(kernels):
    """The diagnostic flag used by the benchmark to time the streaming kernel alone."""
    q, kc, vc, bt, sl, scale = [t.to(DEV) if torch.is_tensor(t) else t
                                for t in _inputs(2, 4, 4, 128, [30, 50], 16, torch.float16)]
    out = torch.zeros_like(q)
    kernels.paged_attention_forward(out, q, kc, vc, bt, sl, scale, 16, bt.size(1), 1)
    torch.cuda.synchronize()
    assert torch.isfinite(out).all()


def test_more_sequences_than_one_launch_takes(kernels):
    """Batches beyond the shared-memory prefix capacity (4096 sequences) run as consecutive launches over the same
    workspace: 5000 short ragged sequences, some of them empty."""
    torch.manual_seed(41)
    S, Hq, Hkv, D, B = 5000, 4, 2, 64, 16
    lens = torch.randint(0, 41, (S,)).tolist()
    b = workloads.make_decode_batch(lens, Hq, Hkv, D, B, torch.float16, device="cpu", seed=41)
    check(kernels, b.query, b.k_cache, b.v_cache, b.block_tables, b.ctx_lens, b.scale)
    got = run_kernel(kernels, b.query.to(DEV), b.k_cache.to(DEV), b.v_cache.to(DEV), b.block_tables.to(DEV),
                     b.ctx_lens.to(DEV), b.scale)
    empty = (b.ctx_lens == 0)
    assert int(empty.sum()) > 0 and torch.count_nonzero(got[empty.to(DEV)]) == 0


def test_streaming_form_on_the_small_shapes():
    """The golden cases, block sizes, lengths and head counts of this file are batches of short sequences, which
    the launcher gives to the small-batch form; a child process with that form switched off (the library reads
    NPD_DECODE_SMALL once) runs them through the streaming form as well."""
    import os
    import subprocess
    import sys
    from pathlib import Path
    env = dict(os.environ, NPD_DECODE_SMALL="2")
    res = subprocess.run([sys.executable, "-m", "pytest", str(Path(__file__).resolve()), "-q", "-x", "-p", "no:cacheprovider",
                          "-k", "golden or block_size or seq_lens or head_dims or group or empty or poison"],
                         env=env, capture_output=True, text=True, timeout=900, cwd=str(Path(__file__).resolve().parents[1]))
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]
    assert " passed" in res.stdout and "failed" not in res.stdout, res.stdout[-2000:]
