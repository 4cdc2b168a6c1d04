"""GPU: the prefill and decode workers on a small random-init stack — the disaggregated hand-off (after the prompt,
and layer by layer) and continuous batching on one GPU.  With two GPUs the prefill side runs on cuda:0 and the
decode side on cuda:1 and the pages cross NVLink; with one, both sides share cuda:0."""
import pytest
import torch

from nanopd_b200 import decoder_step, workers

pytestmark = pytest.mark.gpu
SHAPE = decoder_step.DecoderShape(num_layers=3, hidden=256, ffn=512, vocab=1000, num_q_heads=4, num_kv_heads=2,
                                  head_dim=128)
B = 16


def _model(dev, top_k=1):
    return decoder_step.SyntheticDecoder(dev, SHAPE, torch.bfloat16, seed=4, max_position=1024, top_k=top_k)


def _requests(lens, outs, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [workers.Request(i, torch.randint(0, SHAPE.vocab, (n,), generator=g).pin_memory(), o)
            for i, (n, o) in enumerate(zip(lens, outs))]


def _tokens(req):
    return [int(t.item()) for t in req.stats["_tokens"]]


def _prompt_rows(cache, blocks, n):
    """K (or V) of the first n tokens of a request, [L, Hkv, n, D], read through its block list."""
    rows = cache[:, torch.tensor(blocks, device=cache.device)]             # [L, nblk, Hkv, B, D]
    L, nblk, Hkv, Bs, D = rows.shape
    return rows.permute(0, 2, 1, 3, 4).reshape(L, Hkv, nblk * Bs, D)[:, :, :n].cpu()


@pytest.mark.parametrize("layerwise", [False, True])
def test_disaggregated_requests_end_to_end(kernels, layerwise):
    p_dev = torch.device("cuda:0")
    d_dev = torch.device("cuda:1" if torch.cuda.device_count() >= 2 else "cuda:0")
    lens, outs = [50, 300, 129, 16, 211, 77], [6, 4, 9, 1, 5, 7]
    pw = workers.PrefillWorker(_model(p_dev), num_blocks=96, block_size=B, top_k=1)
    dw = workers.DecodeWorker(_model(d_dev), num_blocks=128, capacity=4, max_context=512, block_size=B)
    pw.keep_blocks = dw.keep_blocks = dw.record_tokens = True
    dw.record_steps = True
    sched = workers.DisaggregatedScheduler([pw], [dw], token_budget=400, layerwise=layerwise)
    reqs = _requests(lens, outs)
    for r in reqs:
        sched.add_request(r)
    done = sched.run_until_done(timeout=120)
    assert sorted(r.rid for r in done) == list(range(len(reqs)))
    for r in reqs:
        n, steps = r.prompt_len, r.decode_steps
        # the prompt's pages arrived bit for bit, at the decode side's own ids
        assert len(set(r.dst_blocks)) == len(r.dst_blocks) and 0 not in r.dst_blocks
        assert torch.equal(_prompt_rows(dw.k_cache, r.dst_blocks, n), _prompt_rows(pw.k_cache, r.src_blocks, n))
        assert torch.equal(_prompt_rows(dw.v_cache, r.dst_blocks, n), _prompt_rows(pw.v_cache, r.src_blocks, n))
        # decode wrote exactly positions n .. n+steps-1 of this request (the pools started as zeros)
        cap = len(r.dst_blocks) * B
        tail = _prompt_rows(dw.k_cache, r.dst_blocks, cap)[:, :, n:]
        assert tail[:, :, :steps].abs().sum(dim=(0, 1, 3)).gt(0).all()
        assert not tail[:, :, steps:].any()
        if steps:
            assert len(_tokens(r)) == 1 + steps
        assert r.stats["transfer_ms"] > 0 and r.stats["exposed_transfer_ms"] >= 0 and r.stats["prefill_ms"] > 0
        assert r.stats["migrated_bytes"] == len(r.src_blocks) * SHAPE.num_layers * 2 * SHAPE.num_kv_heads * B * SHAPE.head_dim * 2
    # every decode slot was recycled (six requests through four slots) and left parked
    t = dw.slots.table
    assert t.num_active == 0 and not t.tables.any() and not t.seq_lens.any()
    assert torch.count_nonzero(dw.model.seq_lens) == 0 and torch.count_nonzero(dw.model.active) == 0
    for d in {p_dev, d_dev}:
        assert kernels.check_status(d, raise_on_error=False) == 0

    # the same requests one at a time through the same workers: greedy tokens agree (the split of the attention
    # work differs with the batch, so a rare low-bit difference may flip an arg-max: most, not all, must agree)
    pw.keep_blocks = dw.keep_blocks = False
    alone = _requests(lens, outs)
    for r in alone:
        s1 = workers.DisaggregatedScheduler([pw], [dw], token_budget=400, layerwise=layerwise)
        s1.add_request(r)
        s1.run_until_done(timeout=120)
    same = sum(_tokens(a) == _tokens(b) for a, b in zip(alone, reqs) if a.decode_steps)
    firsts = sum(_tokens(a)[0] == _tokens(b)[0] for a, b in zip(alone, reqs) if a.decode_steps)
    assert firsts >= 4 and same >= 3, (firsts, same)


def test_blocks_and_slots_are_returned(kernels):
    dev = torch.device("cuda:0")
    pw = workers.PrefillWorker(_model(dev), num_blocks=64, block_size=B, top_k=10)
    dw = workers.DecodeWorker(_model(dev, top_k=10), num_blocks=64, capacity=2, max_context=256, block_size=B)
    free_p, free_d = pw.pool.num_free, dw.pool.num_free
    sched = workers.DisaggregatedScheduler([pw], [dw], token_budget=256)
    for r in _requests([100, 30, 200, 64, 10], [3, 3, 3, 3, 3], seed=2):
        sched.add_request(r)
    done = sched.run_until_done(timeout=120)
    assert len(done) == 5 and pw.pool.num_free == free_p and dw.pool.num_free == free_d and dw.idle


def test_collocated_continuous_batching(kernels):
    """Several prompts chunked within a token budget while earlier requests decode; every request produces its
    output length; chunked prompts leave the same pages as whole-prompt prefill."""
    dev = torch.device("cuda:0")
    cw = workers.CollocatedWorker(_model(dev), num_blocks=160, capacity=4, max_context=512, block_size=B,
                                  token_budget=128, max_chunk=96, top_k=1)
    lens, outs = [200, 40, 333, 90, 17, 150], [5, 12, 3, 8, 2, 6]
    reqs = _requests(lens, outs, seed=5)
    for i, r in enumerate(reqs):
        r.arrival = 0.002 * i
    res = workers.serve_open_loop(cw, reqs, drain_timeout=60)
    assert res["finished"] == len(reqs)
    assert cw.prefill_tokens == sum(lens) and cw.decode_tokens == sum(o - 1 for o in outs)
    assert cw.pool.num_free == 159 and cw.idle
    for r in reqs:
        assert r.stats["ttft_s"] > 0 and r.stats["latency_s"] >= r.stats["ttft_s"]
    # whole-prompt prefill of the longest prompt in a fresh worker leaves the same K/V rows as the chunked run:
    # the chunk kernel reads earlier chunks from the pages, so later layers' K/V agree to rounding
    pw = workers.PrefillWorker(_model(dev), num_blocks=64, block_size=B, top_k=1)
    whole = _requests(lens, outs, seed=5)[2]
    pw.prefill_batch([whole])
    torch.cuda.synchronize()
    cw2 = workers.CollocatedWorker(_model(dev), num_blocks=160, capacity=4, max_context=512, block_size=B,
                                   token_budget=128, max_chunk=96, top_k=1)
    again = _requests(lens, outs, seed=5)[2]
    again.output_len = 1
    cw2.add_request(again)
    while not cw2.idle:
        cw2.step()
    torch.cuda.synchronize()
    a = _prompt_rows(pw.k_cache, whole.src_blocks, 333).float()
    b = _prompt_rows(cw2.k_cache, again.dst_blocks, 333).float()
    assert torch.equal(a[0], b[0])                                   # layer 0 does not depend on attention
    assert (a - b).abs().max().item() <= 0.25 and (a - b).abs().mean().item() <= 5e-3
    assert kernels.check_status(dev, raise_on_error=False) == 0
