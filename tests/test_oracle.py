"""CPU: the oracle against the reference-generated golden vectors and against itself."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN, load_decode_cases, load_rope_cases, load_sampling_cases
from nanopd_b200 import workloads
from oracle import paged_oracle

CASES = load_decode_cases()


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_decode_oracle_reproduces_reference_bit_for_bit(case):
    got = paged_oracle.paged_decode_attention(case["q"], case["k"], case["v"], case["block_tables"],
                                              case["seq_lens"], case["scale"])
    assert torch.equal(got, case["out_fp32"])
    # the reference returns the value cast to the query dtype (test_paged_kernels.py:95)
    assert torch.equal(got.to(case["dtype"]), case["ref_out"])


def test_config1_oracle_matches_reference_output():
    z = np.load(GOLDEN / "config1_reference_out.npz")
    b = workloads.make_config1(device="cpu", seed=0)
    assert np.array_equal(b.ctx_lens.numpy(), z["ctx_lens"])
    assert np.array_equal(b.block_tables.numpy(), z["block_tables"])
    paged_oracle.kv_store(b.k_cache, b.v_cache, b.k_new, b.v_new, b.block_tables, b.positions)
    got = paged_oracle.paged_decode_attention(b.query, b.k_cache, b.v_cache, b.block_tables,
                                              b.seq_lens_after_store, b.scale)
    assert torch.equal(got, torch.from_numpy(z["out_fp32"]))
    assert torch.equal(got.to(torch.float16).view(torch.int16), torch.from_numpy(z["ref_out"]))


# ---- KV store: the mapping the reference's tests assert (test_paged_kernels.py:272-355) ----
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("start,seq_len,heads,block", [(0, 16, 4, 16), (8, 8, 2, 16), (0, 1, 2, 16),
                                                        (0, 64, 8, 16), (0, 32, 2, 32), (5, 40, 3, 8)])
def test_kv_store_mapping(dtype, start, seq_len, heads, block):
    torch.manual_seed(0)
    D = 128
    nblk = (start + seq_len + block - 1) // block
    k_src = torch.randn(heads, seq_len, D).to(dtype)
    v_src = torch.randn(heads, seq_len, D).to(dtype)
    k_cache = torch.zeros(nblk + 2, heads, block, D, dtype=dtype)
    v_cache = torch.zeros_like(k_cache)
    table = torch.randperm(nblk + 2)[:nblk].to(torch.int32)
    bt = table.unsqueeze(0).expand(seq_len, -1)
    pos = torch.arange(start, start + seq_len, dtype=torch.int32)
    paged_oracle.kv_store(k_cache, v_cache, k_src, v_src, bt, pos)
    for tok in range(seq_len):
        p = start + tok
        phys = int(table[p // block])
        for h in range(heads):
            assert torch.equal(k_cache[phys, h, p % block], k_src[h, tok])
            assert torch.equal(v_cache[phys, h, p % block], v_src[h, tok])
    written = torch.zeros(nblk + 2, block, dtype=torch.bool)
    for tok in range(seq_len):
        p = start + tok
        written[int(table[p // block]), p % block] = True
    assert torch.count_nonzero(k_cache.permute(0, 2, 1, 3)[~written]) == 0


# ---- chunked prefill ----
def _prefill_setup(L, Hq, Hkv, D, B, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    nblk = (L + B - 1) // B
    pool = nblk + 3
    q = torch.randn(L, Hq, D, generator=g).to(dtype)
    k = torch.randn(Hkv, L, D, generator=g).to(dtype)
    v = torch.randn(Hkv, L, D, generator=g).to(dtype)
    table = torch.randperm(pool, generator=g)[:nblk].to(torch.int32)
    k_cache = torch.zeros(pool, Hkv, B, D, dtype=dtype)
    v_cache = torch.zeros_like(k_cache)
    paged_oracle.kv_store(k_cache, v_cache, k, v, table.unsqueeze(0).expand(L, -1),
                          torch.arange(L, dtype=torch.int32))
    return q, k, v, table, k_cache, v_cache


def test_prefill_oracle_equals_reference_sdpa_at_start_zero():
    """For start_position == 0 the oracle must equal the reference's own call
    (dense -inf mask + repeat_interleave + SDPA, model_runner.py:152-169)."""
    L, Hq, Hkv, D, B = 45, 8, 2, 64, 16
    q, k, v, table, kc, vc = _prefill_setup(L, Hq, Hkv, D, B, torch.float32)
    scale = D ** -0.5
    got = paged_oracle.paged_prefill_attention(q, kc, vc, table, 0, scale)
    q_p = q.transpose(0, 1).unsqueeze(0)                     # [1, Hq, P, D]
    want = paged_oracle.reference_prefill_sdpa(q_p, k.unsqueeze(0), v.unsqueeze(0), [L], scale)
    assert torch.allclose(got.reshape(1, L, Hq * D), want, atol=2e-6, rtol=1e-5)


def test_prefill_two_packed_prompts_match_reference_sdpa():
    """Two prompts packed in one forward, as PrefillWorker does (prefill_worker.py:47-64)."""
    Hq, Hkv, D, B = 4, 2, 64, 16
    L1, L2 = 20, 33
    scale = D ** -0.5
    a = _prefill_setup(L1, Hq, Hkv, D, B, torch.float32, seed=1)
    b = _prefill_setup(L2, Hq, Hkv, D, B, torch.float32, seed=2)
    got = torch.cat([paged_oracle.paged_prefill_attention(a[0], a[4], a[5], a[3], 0, scale),
                     paged_oracle.paged_prefill_attention(b[0], b[4], b[5], b[3], 0, scale)])
    q_p = torch.cat([a[0], b[0]]).transpose(0, 1).unsqueeze(0)
    k_p = torch.cat([a[1], b[1]], dim=1).unsqueeze(0)
    v_p = torch.cat([a[2], b[2]], dim=1).unsqueeze(0)
    want = paged_oracle.reference_prefill_sdpa(q_p, k_p, v_p, [L1, L2], scale)
    assert torch.allclose(got.reshape(1, L1 + L2, Hq * D), want, atol=2e-6, rtol=1e-5)


def test_prefill_chunks_compose_to_full_causal_attention():
    L, Hq, Hkv, D, B = 100, 4, 2, 64, 16
    q, k, v, table, kc, vc = _prefill_setup(L, Hq, Hkv, D, B, torch.float32)
    scale = D ** -0.5
    full = paged_oracle.paged_prefill_attention(q, kc, vc, table, 0, scale)
    parts = [paged_oracle.paged_prefill_attention(q[s:s + 32], kc, vc, table, s, scale) for s in range(0, L, 32)]
    assert torch.allclose(torch.cat(parts), full, atol=1e-6)


def test_prefill_last_row_equals_decode():
    """The last query of a chunk sees the same keys as a decode step at that position."""
    L, Hq, Hkv, D, B = 37, 4, 2, 128, 16
    q, k, v, table, kc, vc = _prefill_setup(L, Hq, Hkv, D, B, torch.float16)
    scale = D ** -0.5
    pre = paged_oracle.paged_prefill_attention(q, kc, vc, table, 0, scale)
    dec = paged_oracle.paged_decode_attention(q[-1:], kc, vc, table.unsqueeze(0),
                                              torch.tensor([L], dtype=torch.int32), scale)
    assert torch.allclose(pre[-1], dec[0], atol=1e-5)


# ---- migration ----
def test_kv_migrate_copies_named_blocks_only():
    torch.manual_seed(0)
    L, nb, Hkv, B, D = 3, 10, 2, 16, 64
    src_k, src_v = torch.randn(L, nb, Hkv, B, D), torch.randn(L, nb, Hkv, B, D)
    dst_k, dst_v = torch.zeros(L, nb, Hkv, B, D), torch.zeros(L, nb, Hkv, B, D)
    paged_oracle.kv_migrate(src_k, src_v, dst_k, dst_v, [7, 2, 5])
    for bid in range(nb):
        if bid in (7, 2, 5):
            assert torch.equal(dst_k[:, bid], src_k[:, bid]) and torch.equal(dst_v[:, bid], src_v[:, bid])
        else:
            assert torch.count_nonzero(dst_k[:, bid]) == 0 and torch.count_nonzero(dst_v[:, bid]) == 0
    dst2_k, dst2_v = torch.zeros_like(dst_k), torch.zeros_like(dst_v)
    paged_oracle.kv_migrate(src_k, src_v, dst2_k, dst2_v, [7, 2], [0, 9])
    assert torch.equal(dst2_k[:, 0], src_k[:, 7]) and torch.equal(dst2_v[:, 9], src_v[:, 2])


def test_algorithmic_bytes_formula():
    # Qwen3-8B shape: 4096 bytes per context token (K and V, 8 kv heads, 128, bf16)
    b = paged_oracle.decode_algorithmic_bytes([100, 33], 32, 8, 128, 16)
    assert b == 133 * 4096 + 2 * 2 * 32 * 128 * 2 + (7 + 3) * 4 + 2 * 4
    assert paged_oracle.prefill_algorithmic_flops(512, 0, 32, 128) == 4 * 32 * 128 * (512 * 513 // 2)


@pytest.mark.parametrize("case", load_rope_cases(), ids=lambda c: c["name"])
def test_norm_and_rotary_oracle_reproduce_transformers_bit_for_bit(case):
    q, k = case["q"], case["k"]
    if case["with_norm"]:
        q = paged_oracle.rms_norm_heads(q, case["q_norm_weight"], 1e-6)
        k = paged_oracle.rms_norm_heads(k, case["k_norm_weight"], 1e-6)
    assert torch.equal(paged_oracle.rotary(q, case["cos"], case["sin"]), case["q_ref"])
    assert torch.equal(paged_oracle.rotary(k, case["cos"], case["sin"]), case["k_ref"])


def test_qk_norm_rope_store_oracle_puts_rows_in_their_slots():
    case = load_rope_cases()[0]
    T, Hkv, D = case["k"].shape
    B, pool = 16, 12
    torch.manual_seed(0)
    v = torch.randn(T, Hkv, D).to(case["dtype"])
    kc = torch.zeros(pool, Hkv, B, D, dtype=case["dtype"])
    vc = torch.zeros_like(kc)
    table = torch.randperm(pool)[:4].to(torch.int32)
    positions = torch.arange(10, 10 + T, dtype=torch.int32)          # crosses from block 0 into block 1
    q_rot = paged_oracle.qk_norm_rope_store(case["q"], case["k"], v, case["cos"], case["sin"], kc, vc,
                                            table.unsqueeze(0).expand(T, -1), positions,
                                            case["q_norm_weight"], case["k_norm_weight"], 1e-6)
    assert torch.equal(q_rot, case["q_ref"])
    for t in range(T):
        pos = 10 + t
        blk, off = int(table[pos // B]), pos % B
        assert torch.equal(kc[blk, :, off], case["k_ref"][t]) and torch.equal(vc[blk, :, off], v[t])
    assert int((kc != 0).any(-1).sum()) == T * Hkv


@pytest.mark.parametrize("case", load_sampling_cases(), ids=lambda c: c["name"])
def test_sampling_oracle_matches_torch_topk_softmax_and_the_reference_top_1(case):
    """Fixture made by tests/golden/make_golden_sampling.py from torch.nan_to_num / topk / softmax and the
    reference's top_k_sample (nanoPD/engine/model_runner.py:279-284): values and probabilities bit for bit,
    ids on the rows whose k-th value is not tied, the top-1 token wherever the maximum is unique."""
    vals, ids, probs = paged_oracle.top_k_candidates(case["logits"], case["top_k"])
    assert torch.equal(vals, case["values"])
    assert torch.equal(probs, case["probabilities"])
    rows = case["untied_rows"]
    assert torch.equal(ids[rows], case["ids"][rows])
    greedy = paged_oracle.top_k_sample(case["logits"], 1)
    assert torch.equal(greedy[case["top_1_unique"]], case["reference_top_1"][case["top_1_unique"]])


def test_sampling_oracle_draw_is_the_inverse_cdf():
    logits = torch.tensor([[0.0, 1.0, 3.0, 2.0, -1.0]])
    p = torch.softmax(torch.tensor([3.0, 2.0, 1.0]), 0)
    for u, want in ((0.0, 2), (float(p[0]) - 1e-3, 2), (float(p[0]) + 1e-3, 3), (float(p[0] + p[1]) + 1e-3, 1),
                    (0.9999, 1)):
        assert int(paged_oracle.top_k_sample(logits, 3, torch.tensor([u]))[0]) == want
    assert int(paged_oracle.top_k_sample(logits, 1)[0]) == 2
    ties = torch.zeros(1, 6)
    assert paged_oracle.top_k_candidates(ties, 3)[1].tolist() == [[0, 1, 2]]       # equal values: the lower id first
