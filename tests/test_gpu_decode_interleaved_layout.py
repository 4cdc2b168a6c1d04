"""GPU: decode attention on the interleaved cache layouts of the reference's split-K op — K
[blocks, Hkv, D/8, B, 8], V [blocks, Hkv, D, B] — which the reference's own kernel tests pass under the same op
name (nanoPD/paged_attention/tests/test_paged_kernels.py:39-56, 118-150).  Same golden cases, same oracle, and the
result must equal the standard-layout kernel's bit for bit (same tiles, same MMA order)."""
import pytest
import torch

from conftest import TOL, load_decode_cases
from nanopd_b200 import paged_kernels, workloads
from oracle import paged_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def interleave_k(k_std):
    nb, hkv, bs, d = k_std.shape
    return k_std.view(nb, hkv, bs, d // 8, 8).permute(0, 1, 3, 2, 4).contiguous()


def transpose_v(v_std):
    return v_std.permute(0, 1, 3, 2).contiguous()


@pytest.mark.parametrize("case", load_decode_cases(), ids=lambda c: c["name"])
def test_golden_cases_in_interleaved_layout(kernels, case):
    q, k, v = case["q"].to(DEV), case["k"].to(DEV), case["v"].to(DEV)
    bt, sl = case["block_tables"].to(DEV), case["seq_lens"].to(DEV)
    B = k.size(2)
    out_std = torch.zeros_like(q)
    out_il = torch.zeros_like(q)
    if B < 8:
        # a V row of a block is then B * 2 = 8 bytes, below the 16 bytes of the smallest TMA box row: refused
        with pytest.raises(RuntimeError):
            paged_kernels.paged_attention_forward(out_il, q, interleave_k(k), transpose_v(v), bt, sl, case["scale"], B, bt.size(1))
        return
    # the interleaved layouts always take the streaming form of the kernel: bit-equality holds against the standard
    # layout in the same form (private flag bit 2), the small-batch form cuts and merges a sequence differently
    paged_kernels.paged_attention_forward(out_std, q, k, v, bt, sl, case["scale"], B, bt.size(1), _flags=4)
    paged_kernels.paged_attention_forward(out_il, q, interleave_k(k), transpose_v(v), bt, sl, case["scale"], B, bt.size(1))
    torch.cuda.synchronize()
    assert torch.equal(out_il, out_std)
    err = (out_il.float().cpu() - case["out_fp32"]).abs().max().item()
    assert err <= TOL[case["dtype"]], err
    assert torch.allclose(out_il.float().cpu(), case["ref_out"].float(), atol=1e-2, rtol=1e-2)   # the reference tests' own bound


@pytest.mark.parametrize("D,B,Hq,Hkv", [(64, 8, 4, 2), (64, 16, 8, 8), (128, 8, 12, 2), (128, 32, 32, 8),
                                        (256, 16, 8, 2), (256, 32, 4, 4), (128, 16, 40, 2)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_shapes_ragged_lengths_and_poisoned_tails(kernels, D, B, Hq, Hkv, dtype):
    torch.manual_seed(D + B + Hq)
    lens = [1, B - 1, B, B + 1, 3 * B + 5, 130, 257, 0]
    b = workloads.make_decode_batch(lens, Hq, Hkv, D, B, dtype, device="cpu", seed=7)
    want = paged_oracle.paged_decode_attention(b.query, b.k_cache, b.v_cache, b.block_tables, b.ctx_lens, b.scale)
    workloads.poison_unwritten_slots(b)              # NaN in every slot past a sequence's end
    q, bt, sl = b.query.to(DEV), b.block_tables.to(DEV), b.ctx_lens.to(DEV)
    out = torch.full_like(q, float("nan"))
    paged_kernels.paged_attention_forward(out, q, interleave_k(b.k_cache.to(DEV)), transpose_v(b.v_cache.to(DEV)),
                                          bt, sl, b.scale, B, bt.size(1))
    torch.cuda.synchronize()
    assert not torch.isnan(out).any()
    err = (out.float().cpu() - want).abs().max().item()
    assert err <= TOL[dtype], err
    assert torch.count_nonzero(out[-1]) == 0          # the empty sequence gets a zero row
    assert paged_kernels.check_status(DEV, raise_on_error=False) == 0


def test_config2_slice_equals_standard_layout(kernels):
    b = workloads.make_config2(device=DEV, seed=0, batch=48)
    out_std = torch.zeros_like(b.query)
    out_il = torch.zeros_like(b.query)
    B = b.block_size
    paged_kernels.paged_attention_forward(out_std, b.query, b.k_cache, b.v_cache, b.block_tables, b.ctx_lens,
                                          b.scale, B, b.max_blocks, _flags=4)
    paged_kernels.paged_attention_forward(out_il, b.query, interleave_k(b.k_cache), transpose_v(b.v_cache),
                                          b.block_tables, b.ctx_lens, b.scale, B, b.max_blocks)
    torch.cuda.synchronize()
    assert torch.equal(out_il, out_std)


def test_mismatched_interleaved_shapes_raise(kernels):
    q = torch.zeros(1, 4, 128, dtype=torch.float16, device=DEV)
    k5 = torch.zeros(2, 4, 16, 16, 8, dtype=torch.float16, device=DEV)
    v_std = torch.zeros(2, 4, 16, 128, dtype=torch.float16, device=DEV)       # standard V with interleaved K
    bt = torch.zeros(1, 1, dtype=torch.int32, device=DEV)
    sl = torch.ones(1, dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError):
        paged_kernels.paged_attention_forward(torch.zeros_like(q), q, k5, v_std, bt, sl, 1.0, 16, 1)
    with pytest.raises(RuntimeError):
        paged_kernels.paged_attention_forward(torch.zeros_like(q), q, k5[..., :4], v_std.permute(0, 1, 3, 2).contiguous(),
                                              bt, sl, 1.0, 16, 1)
