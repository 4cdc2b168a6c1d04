"""GPU: the fused QK-norm + rotary embedding + KV store against the oracle and against the
transformers-generated fixture.  The page mapping is exact; values may differ from the 16-bit
reference arithmetic by one rounding step where the fp32 mean of squares is summed in another order
(the kernel reduces across a warp), so the comparison allows one step of the dtype on a small fraction
of elements and nothing more; without norm weights the result is bit-exact."""
import pytest
import torch

from conftest import load_rope_cases
from nanopd_b200 import paged_kernels
from oracle import paged_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def check_close(got, want, what):
    """Equal except where one operand of the rotation was rounded the other way: the difference is then at most
    one step of the dtype at the operands' magnitude (|x| < 8 here; the sum itself may be much smaller, so this is
    an absolute bound, not a count of representable values), on a small fraction of the elements."""
    step = {torch.float16: 2.0 ** -8, torch.bfloat16: 2.0 ** -5}[want.dtype]
    got = got.cpu()
    diff = (got.float() - want.float()).abs()
    assert float(diff.max()) <= step, f"{what}: max abs difference {float(diff.max())}"
    assert float((got != want).float().mean()) < 0.02, f"{what}: {(got != want).float().mean():.4f} of the elements differ"


@pytest.mark.parametrize("case", load_rope_cases(), ids=lambda c: c["name"])
def test_fixture_cases(kernels, case):
    dtype = case["dtype"]
    T, Hq, D = case["q"].shape
    Hkv = case["k"].size(1)
    B, pool = 16, 3000 // 16 + 2
    torch.manual_seed(1)
    v = torch.randn(T, Hkv, D).to(dtype)
    kc = torch.zeros(pool, Hkv, B, D, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    table = torch.randperm(pool).to(torch.int32)
    positions = case["positions"]
    dev = lambda t: None if t is None else t.to(DEV)
    q_dev = case["q"].to(DEV)
    q_out = paged_kernels.paged_qk_norm_rope_store(q_dev, dev(case["k"]), dev(v), dev(case["cos"]), dev(case["sin"]),
                                                   kc, vc, table.to(DEV), positions.to(DEV),
                                                   dev(case["q_norm_weight"]), dev(case["k_norm_weight"]), 1e-6)
    torch.cuda.synchronize()
    assert q_out.data_ptr() == q_dev.data_ptr()                       # in place by default
    check_close(q_out, case["q_ref"], "q")
    kc_h, vc_h = kc.cpu(), vc.cpu()
    for t in range(T):
        pos = int(positions[t])
        blk, off = int(table[pos // B]), pos % B
        check_close(kc_h[blk, :, off], case["k_ref"][t], f"k row {t}")
        assert torch.equal(vc_h[blk, :, off], v[t])
    assert int((kc_h != 0).any(-1).sum()) == T * Hkv                  # nothing else was written
    assert int((vc_h != 0).any(-1).sum()) == T * Hkv


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("D", [64, 128, 256])
def test_fused_projection_views_and_separate_output(kernels, dtype, D):
    torch.manual_seed(5)
    T, Hq, Hkv, B = 33, 8, 2, 16
    pool = 40
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D).to(dtype)                # one fused projection output
    q = qkv[:, :Hq * D].view(T, Hq, D)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
    ang = torch.rand(T, D // 2) * 6.28
    cos = torch.cat((ang.cos(), ang.cos()), -1).to(dtype)
    sin = torch.cat((ang.sin(), ang.sin()), -1).to(dtype)
    qw = (1 + 0.1 * torch.randn(D)).to(dtype)
    kw = (1 + 0.1 * torch.randn(D)).to(dtype)
    # three sequences: decode-like tokens at arbitrary positions
    tables = torch.randperm(pool)[:T * 1].to(torch.int32).view(T, 1)
    tables = torch.cat((tables, torch.zeros(T, 2, dtype=torch.int32)), 1)
    positions = torch.randint(0, B, (T,), dtype=torch.int32)

    kc_ref = torch.zeros(pool, Hkv, B, D, dtype=dtype)
    vc_ref = torch.zeros_like(kc_ref)
    q_ref = paged_oracle.qk_norm_rope_store(q, k, v, cos, sin, kc_ref, vc_ref, tables, positions, qw, kw, 1e-6)

    qkv_d = qkv.to(DEV)
    q_d = qkv_d[:, :Hq * D].view(T, Hq, D)
    k_d = qkv_d[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
    v_d = qkv_d[:, (Hq + Hkv) * D:].view(T, Hkv, D)
    kc = torch.zeros(pool, Hkv, B, D, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    q_out = torch.empty(T, Hq, D, dtype=dtype, device=DEV)
    ret = paged_kernels.paged_qk_norm_rope_store(q_d, k_d, v_d, cos.to(DEV), sin.to(DEV), kc, vc, tables.to(DEV),
                                                 positions.to(DEV), qw.to(DEV), kw.to(DEV), 1e-6, q_out=q_out)
    torch.cuda.synchronize()
    assert ret is q_out and torch.equal(qkv_d.cpu(), qkv)             # inputs untouched with a separate output
    check_close(q_out, q_ref, "q")
    check_close(kc, kc_ref, "k cache")
    assert torch.equal(vc.cpu(), vc_ref)
    # in place over the strided view of the fused buffer (q_out aliases q, the default): the rotated queries replace
    # the q columns, the k and v columns of the buffer stay as they were
    kc.zero_(), vc.zero_()
    ret = paged_kernels.paged_qk_norm_rope_store(q_d, k_d, v_d, cos.to(DEV), sin.to(DEV), kc, vc, tables.to(DEV),
                                                 positions.to(DEV), qw.to(DEV), kw.to(DEV), 1e-6)
    torch.cuda.synchronize()
    assert ret.data_ptr() == q_d.data_ptr() and ret.stride(0) == (Hq + 2 * Hkv) * D
    check_close(ret, q_ref, "q in place")
    assert torch.equal(qkv_d[:, Hq * D:].cpu(), qkv[:, Hq * D:])
    check_close(kc, kc_ref, "k cache (in-place run)")
    assert paged_kernels.check_status(DEV, raise_on_error=False) == 0


def test_no_norm_matches_plain_store_of_rotated_keys(kernels):
    """Without norm weights the K rows in the pages must equal paged_kv_store of the oracle's rotated keys."""
    torch.manual_seed(6)
    T, Hq, Hkv, D, B, pool = 20, 4, 4, 128, 16, 8
    dtype = torch.float16
    q, k, v = (torch.randn(T, h, D).to(dtype) for h in (Hq, Hkv, Hkv))
    ang = torch.rand(T, D // 2) * 6.28
    cos = torch.cat((ang.cos(), ang.cos()), -1).to(dtype)
    sin = torch.cat((ang.sin(), ang.sin()), -1).to(dtype)
    table = torch.tensor([3, 6], dtype=torch.int32)
    kc = torch.zeros(pool, Hkv, B, D, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    positions = torch.arange(5, 5 + T, dtype=torch.int32)
    paged_kernels.paged_qk_norm_rope_store(q.to(DEV), k.to(DEV), v.to(DEV), cos.to(DEV), sin.to(DEV), kc, vc,
                                           table.to(DEV), positions.to(DEV))
    kc2 = torch.zeros_like(kc)
    vc2 = torch.zeros_like(kc)
    k_rot = paged_oracle.rotary(k, cos, sin)
    paged_kernels.paged_kv_store(kc2, vc2, k_rot.transpose(0, 1).contiguous().to(DEV),
                                 v.transpose(0, 1).contiguous().to(DEV), table.to(DEV), 5)
    torch.cuda.synchronize()
    assert torch.equal(kc, kc2) and torch.equal(vc, vc2)              # no norm: every step is exactly rounded


def test_bad_arguments_raise(kernels):
    T, Hq, Hkv, D, B = 4, 4, 2, 128, 16
    mk = lambda *s, dt=torch.float16: torch.zeros(*s, dtype=dt, device=DEV)
    q, k, v, cos, sin = mk(T, Hq, D), mk(T, Hkv, D), mk(T, Hkv, D), mk(T, D), mk(T, D)
    kc, vc = mk(4, Hkv, B, D), mk(4, Hkv, B, D)
    bt = torch.zeros(T, 2, dtype=torch.int32, device=DEV)
    pos = torch.zeros(T, dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError):
        paged_kernels.paged_qk_norm_rope_store(q, k, v, cos, sin, kc, vc, bt.long(), pos)
    with pytest.raises(RuntimeError):
        paged_kernels.paged_qk_norm_rope_store(q, k, v, cos[:, :64], sin[:, :64], kc, vc, bt, pos)
    with pytest.raises(RuntimeError):
        paged_kernels.paged_qk_norm_rope_store(q.float(), k, v, cos, sin, kc, vc, bt, pos)
    with pytest.raises(RuntimeError):
        paged_kernels.paged_qk_norm_rope_store(q, k, v, cos, sin, kc, vc, bt, pos, q_norm_weight=mk(64))
    # a position beyond the table is flagged, not written
    pos_bad = torch.full((T,), 5 * B, dtype=torch.int32, device=DEV)
    paged_kernels.paged_qk_norm_rope_store(q, k, v, cos, sin, kc, vc, bt, pos_bad)
    assert paged_kernels.check_status(DEV, raise_on_error=False) != 0
