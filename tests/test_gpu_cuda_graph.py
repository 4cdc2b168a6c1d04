"""GPU: the decode step (store the new token, then attend) captured once in a CUDA graph and replayed while
positions, lengths, queries and new K/V rows change in place — the way a serving loop would run it
(the reference rebuilds and re-copies its tables in every layer, nanoPD/engine/model_runner.py:176-187).
Each replay is checked against the oracle applied in the caller's order."""
import pytest
import torch

from conftest import TOL
from nanopd_b200 import paged_kernels, workloads
from oracle import paged_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_decode_step_graph_replays_follow_the_positions(kernels, dtype):
    torch.manual_seed(11)
    S, Hq, Hkv, D, B = 12, 8, 2, 128, 16
    steps = 3
    ctx = torch.randint(1, 200, (S,))
    ctx[0], ctx[1] = 15, 16                       # one sequence crosses a block boundary during the replays
    nblk = [(int(c) + steps + B - 1) // B for c in ctx]
    pool = sum(nblk) + 3
    perm = torch.randperm(pool)
    tables = torch.zeros(S, max(nblk), dtype=torch.int32)
    o = 0
    for i, n in enumerate(nblk):
        tables[i, :n] = perm[o:o + n].to(torch.int32)
        o += n
    k_cache = torch.randn(pool, Hkv, B, D).to(dtype)
    v_cache = torch.randn(pool, Hkv, B, D).to(dtype)
    scale = D ** -0.5

    kc, vc, bt = k_cache.to(DEV), v_cache.to(DEV), tables.to(DEV)
    q = torch.zeros(S, Hq, D, dtype=dtype, device=DEV)
    k_new = torch.zeros(Hkv, S, D, dtype=dtype, device=DEV)
    v_new = torch.zeros_like(k_new)
    positions = ctx.to(torch.int32).to(DEV)
    seq_lens = positions + 1
    out = torch.zeros_like(q)

    def step():
        paged_kernels.paged_kv_store(kc, vc, k_new, v_new, bt, positions)
        paged_kernels.paged_attention_forward(out, q, kc, vc, bt, seq_lens, scale, B, bt.size(1))

    # warm up on the capture stream (its workspace is created here, outside the capture), then capture
    side = torch.cuda.Stream(device=DEV)
    side.wait_stream(torch.cuda.current_stream())
    kc_keep, vc_keep = kc.clone(), vc.clone()
    with torch.cuda.stream(side):
        step()
    side.synchronize()
    kc.copy_(kc_keep), vc.copy_(vc_keep)          # undo the warm-up's store
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        step()
    kc.copy_(kc_keep), vc.copy_(vc_keep)
    torch.cuda.synchronize()

    kc_ref, vc_ref = k_cache.clone(), v_cache.clone()
    pos_ref = ctx.to(torch.int32).clone()
    for it in range(steps):
        q_h = torch.randn(S, Hq, D).to(dtype)
        k_h = torch.randn(Hkv, S, D).to(dtype)
        v_h = torch.randn(Hkv, S, D).to(dtype)
        q.copy_(q_h), k_new.copy_(k_h), v_new.copy_(v_h)
        positions.copy_(pos_ref)
        seq_lens.copy_(pos_ref + 1)
        graph.replay()
        torch.cuda.synchronize()
        paged_oracle.kv_store(kc_ref, vc_ref, k_h, v_h, tables, pos_ref)
        want = paged_oracle.paged_decode_attention(q_h, kc_ref, vc_ref, tables, pos_ref + 1, scale)
        assert torch.equal(kc.cpu(), kc_ref) and torch.equal(vc.cpu(), vc_ref), f"replay {it}: store differs"
        err = (out.float().cpu() - want).abs().max().item()
        assert err <= TOL[dtype], (it, err)
        pos_ref += 1
    assert paged_kernels.check_status(DEV, raise_on_error=False) == 0


def test_graph_of_configuration1_matches_eager(kernels):
    b = workloads.make_config1(device=DEV, seed=0)
    out_eager = torch.zeros_like(b.query)
    out_graph = torch.zeros_like(b.query)
    B = b.block_size
    paged_kernels.paged_attention_forward(out_eager, b.query, b.k_cache, b.v_cache, b.block_tables, b.ctx_lens,
                                          b.scale, B, b.max_blocks)
    side = torch.cuda.Stream(device=DEV)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        paged_kernels.paged_attention_forward(out_graph, b.query, b.k_cache, b.v_cache, b.block_tables, b.ctx_lens,
                                              b.scale, B, b.max_blocks)
    side.synchronize()
    out_graph.zero_()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        paged_kernels.paged_attention_forward(out_graph, b.query, b.k_cache, b.v_cache, b.block_tables, b.ctx_lens,
                                              b.scale, B, b.max_blocks)
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out_graph, out_eager)
