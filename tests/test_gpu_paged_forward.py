"""GPU: one mixed scheduler step (prompt chunks + decode sequences) through paged_attention_step, against the
oracle applied in the caller's order (store, then attend)."""
import pytest
import torch

from conftest import TOL
from nanopd_b200 import paged_forward
from oracle import paged_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_mixed_step_matches_oracle(kernels, dtype):
    torch.manual_seed(3)
    Hq, Hkv, D, B, pool = 8, 2, 128, 16, 64
    # existing context in the pool: prompt 1 has 70 tokens cached already (an earlier chunk), decodes have history
    k_cache = torch.randn(pool, Hkv, B, D).to(dtype)
    v_cache = torch.randn(pool, Hkv, B, D).to(dtype)
    perm = torch.randperm(pool).tolist()
    prefills = [{"block_table": perm[0:3], "start_position": 0, "num_tokens": 40},
                {"block_table": perm[3:10], "start_position": 70, "num_tokens": 33}]
    decodes = [{"block_table": perm[10:14], "position": 50}, {"block_table": perm[14:15], "position": 0},
               {"block_table": perm[15:25], "position": 159}]
    P, Dn = 73, 3
    ctx = {"num_prefill_tokens": P, "num_decode_tokens": Dn, "prefills": prefills, "decodes": decodes}
    q = torch.randn(1, Hq, P + Dn, D).to(dtype)
    k = torch.randn(1, Hkv, P + Dn, D).to(dtype)
    v = torch.randn(1, Hkv, P + Dn, D).to(dtype)
    scale = D ** -0.5

    # ---- oracle, in the caller's order ----
    kc_ref, vc_ref = k_cache.clone(), v_cache.clone()
    want = torch.zeros(P + Dn, Hq, D)
    off = 0
    for pinfo in prefills:
        n, start = pinfo["num_tokens"], pinfo["start_position"]
        bt = torch.tensor(pinfo["block_table"], dtype=torch.int32)
        paged_oracle.kv_store(kc_ref, vc_ref, k[0, :, off:off + n], v[0, :, off:off + n],
                              bt.unsqueeze(0).expand(n, -1), torch.arange(start, start + n, dtype=torch.int32))
        off += n
    off = 0
    for pinfo in prefills:
        n, start = pinfo["num_tokens"], pinfo["start_position"]
        bt = torch.tensor(pinfo["block_table"], dtype=torch.int32)
        want[off:off + n] = paged_oracle.paged_prefill_attention(q[0, :, off:off + n].transpose(0, 1), kc_ref, vc_ref,
                                                                 bt, start, scale)
        off += n
    sc_cpu = paged_forward.build_step_context(ctx, "cpu")
    paged_oracle.kv_store(kc_ref, vc_ref, k[0, :, P:], v[0, :, P:], sc_cpu.decode_tables, sc_cpu.decode_positions)
    want[P:] = paged_oracle.paged_decode_attention(q[0, :, P:].transpose(0, 1), kc_ref, vc_ref, sc_cpu.decode_tables,
                                                   sc_cpu.decode_seq_lens, scale)

    # ---- CUDA path ----
    sc = paged_forward.build_step_context(ctx, DEV)
    kc, vc = k_cache.to(DEV), v_cache.to(DEV)
    got = paged_forward.paged_attention_step(sc, q.to(DEV), k.to(DEV), v.to(DEV), kc, vc, scale)
    torch.cuda.synchronize()
    assert got.shape == (1, P + Dn, Hq * D)
    assert torch.equal(kc.cpu(), kc_ref) and torch.equal(vc.cpu(), vc_ref)          # stores are bit-exact
    err = (got.float().cpu().view(P + Dn, Hq, D) - want).abs().max().item()
    assert err <= TOL[dtype], err


def test_decode_only_and_prefill_only_steps(kernels):
    torch.manual_seed(4)
    Hq, Hkv, D, B, pool = 4, 4, 128, 16, 16
    k_cache = torch.zeros(pool, Hkv, B, D, dtype=torch.float16, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    scale = D ** -0.5
    # a 20-token prompt, then one decode step on it: the decode row must equal the oracle over 21 keys
    table = [5, 2]
    q = torch.randn(1, Hq, 20, D, device=DEV).half()
    k = torch.randn(1, Hkv, 20, D, device=DEV).half()
    v = torch.randn(1, Hkv, 20, D, device=DEV).half()
    sc = paged_forward.build_step_context({"num_prefill_tokens": 20, "num_decode_tokens": 0, "decodes": [],
                                           "prefills": [{"block_table": table, "start_position": 0, "num_tokens": 20}]}, DEV)
    out_p = paged_forward.paged_attention_step(sc, q, k, v, k_cache, v_cache, scale)
    q1 = torch.randn(1, Hq, 1, D, device=DEV).half()
    k1 = torch.randn(1, Hkv, 1, D, device=DEV).half()
    v1 = torch.randn(1, Hkv, 1, D, device=DEV).half()
    sc1 = paged_forward.build_step_context({"num_prefill_tokens": 0, "num_decode_tokens": 1, "prefills": [],
                                            "decodes": [{"block_table": table, "position": 20}]}, DEV)
    out_d = paged_forward.paged_attention_step(sc1, q1, k1, v1, k_cache, v_cache, scale)
    torch.cuda.synchronize()
    bt = torch.tensor([table], dtype=torch.int32)
    want_d = paged_oracle.paged_decode_attention(q1[0].transpose(0, 1).cpu(), k_cache.cpu(), v_cache.cpu(), bt,
                                                 torch.tensor([21], dtype=torch.int32), scale)
    assert (out_d.view(1, Hq, D).float().cpu() - want_d).abs().max().item() <= TOL[torch.float16]
    want_p = paged_oracle.paged_prefill_attention(q[0].transpose(0, 1).cpu(), k_cache.cpu(), v_cache.cpu(), bt[0], 0, scale)
    assert (out_p.view(20, Hq, D).float().cpu() - want_p).abs().max().item() <= TOL[torch.float16]


def test_fused_step_equals_unfused_step_on_rotated_inputs(kernels):
    """paged_attention_step_fused (norm + rotary + store in one launch) against paged_attention_step fed with
    the oracle's normed and rotated tensors: same pages (up to one rounding step of the norm) and same output."""
    torch.manual_seed(9)
    dtype = torch.bfloat16
    Hq, Hkv, D, B, pool = 8, 2, 128, 16, 48
    perm = torch.randperm(pool).tolist()
    prefills = [{"block_table": perm[0:4], "start_position": 16, "num_tokens": 37}]
    decodes = [{"block_table": perm[4:8], "position": 49}, {"block_table": perm[8:9], "position": 3}]
    P, Dn = 37, 2
    total = P + Dn
    ctx = {"num_prefill_tokens": P, "num_decode_tokens": Dn, "prefills": prefills, "decodes": decodes}
    k_cache = torch.randn(pool, Hkv, B, D).to(dtype)
    v_cache = torch.randn(pool, Hkv, B, D).to(dtype)
    q = torch.randn(total, Hq, D).to(dtype)
    k = torch.randn(total, Hkv, D).to(dtype)
    v = torch.randn(total, Hkv, D).to(dtype)
    pos = torch.tensor(list(range(16, 16 + 37)) + [49, 3], dtype=torch.float32)
    inv_freq = 1.0 / (1e6 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = pos[:, None] * inv_freq[None, :]
    cos = torch.cat((ang.cos(), ang.cos()), -1).to(dtype)
    sin = torch.cat((ang.sin(), ang.sin()), -1).to(dtype)
    qw = (1 + 0.1 * torch.randn(D)).to(dtype)
    kw = (1 + 0.1 * torch.randn(D)).to(dtype)
    scale = D ** -0.5

    q_rot = paged_oracle.rotary(paged_oracle.rms_norm_heads(q, qw, 1e-6), cos, sin)
    k_rot = paged_oracle.rotary(paged_oracle.rms_norm_heads(k, kw, 1e-6), cos, sin)
    sc = paged_forward.build_step_context(ctx, DEV)
    kc1, vc1 = k_cache.to(DEV), v_cache.to(DEV)
    want = paged_forward.paged_attention_step(sc, q_rot.transpose(0, 1).unsqueeze(0).to(DEV),
                                              k_rot.transpose(0, 1).unsqueeze(0).to(DEV),
                                              v.transpose(0, 1).unsqueeze(0).to(DEV), kc1, vc1, scale)
    kc2, vc2 = k_cache.to(DEV), v_cache.to(DEV)
    got = paged_forward.paged_attention_step_fused(sc, q.to(DEV), k.to(DEV), v.to(DEV), cos.to(DEV), sin.to(DEV),
                                                   kc2, vc2, scale, qw.to(DEV), kw.to(DEV), 1e-6)
    torch.cuda.synchronize()
    assert torch.equal(vc1, vc2)
    assert (kc1.float() - kc2.float()).abs().max().item() <= 2 ** -5          # one bf16 step at |x| < 8
    assert float((kc1 != kc2).float().mean()) < 0.01
    assert (got.float() - want.float()).abs().max().item() <= TOL[dtype]


def test_mixed_step_on_two_streams_equals_the_step_in_turn(kernels, monkeypatch):
    """The side-by-side launch of the two attention kernels (each on its share of the SMs) gives what running them
    one after the other gives, and both match the oracle."""
    monkeypatch.setattr(paged_forward, "_MIN_OVERLAP_SECONDS", 0.0)      # force the two-stream path at test size
    torch.manual_seed(12)
    dtype = torch.bfloat16
    Hq, Hkv, D, B = 8, 2, 128, 16
    n_chunk, start = 150, 310
    dec_pos = [700, 33, 1500, 64, 255, 1023, 12, 480]
    nblk_p = (start + n_chunk + B - 1) // B
    nblk_d = [(p + 1 + B - 1) // B for p in dec_pos]
    pool = nblk_p + sum(nblk_d) + 4
    perm = torch.randperm(pool).tolist()
    prefills = [{"block_table": perm[:nblk_p], "start_position": start, "num_tokens": n_chunk}]
    decodes, o = [], nblk_p
    for p_, n_ in zip(dec_pos, nblk_d):
        decodes.append({"block_table": perm[o:o + n_], "position": p_})
        o += n_
    P, Dn = n_chunk, len(dec_pos)
    ctx = {"num_prefill_tokens": P, "num_decode_tokens": Dn, "prefills": prefills, "decodes": decodes}
    k_cache = torch.randn(pool, Hkv, B, D).to(dtype)
    v_cache = torch.randn(pool, Hkv, B, D).to(dtype)
    q = torch.randn(1, Hq, P + Dn, D).to(dtype)
    k = torch.randn(1, Hkv, P + Dn, D).to(dtype)
    v = torch.randn(1, Hkv, P + Dn, D).to(dtype)
    scale = D ** -0.5
    sc = paged_forward.build_step_context(ctx, DEV)
    assert paged_forward._sm_split(sc, Hq, Hkv, D, 2, 148) is not None
    outs = []
    for overlap in (False, True):
        kc, vc = k_cache.to(DEV), v_cache.to(DEV)
        outs.append(paged_forward.paged_attention_step(sc, q.to(DEV), k.to(DEV), v.to(DEV), kc, vc, scale, overlap=overlap))
        torch.cuda.synchronize()
    assert torch.equal(outs[0][:, :P], outs[1][:, :P])                     # prompt rows: same kernel, same tiles
    assert (outs[0].float() - outs[1].float()).abs().max().item() <= TOL[dtype]

    kc_ref, vc_ref = k_cache.clone(), v_cache.clone()
    bt = torch.tensor(prefills[0]["block_table"], dtype=torch.int32)
    paged_oracle.kv_store(kc_ref, vc_ref, k[0, :, :P], v[0, :, :P], bt.unsqueeze(0).expand(P, -1),
                          torch.arange(start, start + P, dtype=torch.int32))
    sc_cpu = paged_forward.build_step_context(ctx, "cpu")
    paged_oracle.kv_store(kc_ref, vc_ref, k[0, :, P:], v[0, :, P:], sc_cpu.decode_tables, sc_cpu.decode_positions)
    want = torch.zeros(P + Dn, Hq, D)
    want[:P] = paged_oracle.paged_prefill_attention(q[0, :, :P].transpose(0, 1), kc_ref, vc_ref, bt, start, scale)
    want[P:] = paged_oracle.paged_decode_attention(q[0, :, P:].transpose(0, 1), kc_ref, vc_ref, sc_cpu.decode_tables,
                                                   sc_cpu.decode_seq_lens, scale)
    err = (outs[1].float().cpu().view(P + Dn, Hq, D) - want).abs().max().item()
    assert err <= TOL[dtype], err


def test_prefill_in_the_same_step_does_not_change_the_decode_rows(kernels):
    """The reference's engine test asks that a mixed batch leaves the decode tokens unchanged
    (nanoPD/engine/test/test_mixed_batch.py:10-30).  Here: the decode rows of a mixed step, run in turn, equal the
    rows of the same decode batch stepped alone, bit for bit; with the two kernels side by side (another split of
    the decode work) they agree within the attention tolerance."""
    torch.manual_seed(21)
    dtype = torch.float16
    Hq, Hkv, D, B, pool = 12, 2, 128, 16, 40
    perm = torch.randperm(pool).tolist()
    decodes = [{"block_table": perm[0:6], "position": 90}, {"block_table": perm[6:7], "position": 7},
               {"block_table": perm[7:17], "position": 150}]
    prefills = [{"block_table": perm[17:25], "start_position": 32, "num_tokens": 70}]
    Dn, P = len(decodes), 70
    k_cache = torch.randn(pool, Hkv, B, D).to(dtype)
    v_cache = torch.randn(pool, Hkv, B, D).to(dtype)
    q_d, k_d, v_d = (torch.randn(1, h, Dn, D).to(dtype) for h in (Hq, Hkv, Hkv))
    q_p, k_p, v_p = (torch.randn(1, h, P, D).to(dtype) for h in (Hq, Hkv, Hkv))
    scale = D ** -0.5

    def run(ctx, q, k, v, overlap):
        sc = paged_forward.build_step_context(ctx, DEV)
        kc, vc = k_cache.to(DEV), v_cache.to(DEV)
        out = paged_forward.paged_attention_step(sc, q.to(DEV), k.to(DEV), v.to(DEV), kc, vc, scale, overlap=overlap)
        torch.cuda.synchronize()
        return out[0].cpu()

    alone = run({"num_prefill_tokens": 0, "num_decode_tokens": Dn, "prefills": [], "decodes": decodes}, q_d, k_d, v_d, False)
    mixed_ctx = {"num_prefill_tokens": P, "num_decode_tokens": Dn, "prefills": prefills, "decodes": decodes}
    cat = lambda a, b: torch.cat((a, b), dim=2)
    in_turn = run(mixed_ctx, cat(q_p, q_d), cat(k_p, k_d), cat(v_p, v_d), False)
    assert torch.equal(in_turn[P:], alone)
    prev = paged_forward._MIN_OVERLAP_SECONDS
    paged_forward._MIN_OVERLAP_SECONDS = 0.0
    try:
        side_by_side = run(mixed_ctx, cat(q_p, q_d), cat(k_p, k_d), cat(v_p, v_d), True)
    finally:
        paged_forward._MIN_OVERLAP_SECONDS = prev
    assert torch.equal(side_by_side[:P], in_turn[:P])
    assert (side_by_side[P:].float() - alone.float()).abs().max().item() <= TOL[dtype]
