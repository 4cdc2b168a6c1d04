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
