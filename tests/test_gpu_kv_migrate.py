"""GPU: KV page migration through the C ABI — bit-exact against the oracle."""
import pytest
import torch

from nanopd_b200 import kv_transfer
from oracle import paged_oracle

pytestmark = pytest.mark.gpu


def _pools(L, nb, Hkv, B, D, dtype, device, seed):
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(L, nb, Hkv, B, D, generator=g).to(dtype)
    v = torch.randn(L, nb, Hkv, B, D, generator=g).to(dtype)
    return k, v, k.to(device), v.to(device)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("max_ctas", [0, 1, 4, -8])
def test_same_ids_like_the_reference(kernels, dtype, max_ctas):
    """transfer_kv with equal ids on both sides (kv_transfer.py:73-79), both pools on one GPU."""
    L, nb, Hkv, B, D = 4, 24, 8, 16, 128
    sk, sv, dsk, dsv = _pools(L, nb, Hkv, B, D, dtype, "cuda:0", 0)
    dk, dv, ddk, ddv = _pools(L, nb, Hkv, B, D, dtype, "cuda:0", 1)
    table = [5, 17, 3, 22, 0]
    path = kv_transfer.transfer_kv(dsk, dsv, ddk, ddv, table, max_ctas=max_ctas)
    assert path == "p2p"
    paged_oracle.kv_migrate(sk, sv, dk, dv, table)
    torch.cuda.synchronize()
    assert torch.equal(ddk.cpu(), dk) and torch.equal(ddv.cpu(), dv)


def test_different_ids_and_side_stream(kernels):
    L, nb, Hkv, B, D = 3, 16, 2, 16, 64
    sk, sv, dsk, dsv = _pools(L, nb, Hkv, B, D, torch.float16, "cuda:0", 2)
    dk = torch.zeros(L, 9, Hkv, B, D, dtype=torch.float16)
    dv = torch.zeros_like(dk)
    ddk, ddv = dk.to("cuda:0"), dv.to("cuda:0")
    stream = torch.cuda.Stream(device="cuda:0")
    stream.wait_stream(torch.cuda.current_stream())
    kv_transfer.transfer_kv(dsk, dsv, ddk, ddv, [1, 15, 7], stream=stream, dst_block_table=[8, 0, 4])
    ev = torch.cuda.Event()
    stream.record_event(ev)          # completion as in DecodeWorker.receive_kv_async
    ev.synchronize()
    paged_oracle.kv_migrate(sk, sv, dk, dv, [1, 15, 7], [8, 0, 4])
    assert torch.equal(ddk.cpu(), dk) and torch.equal(ddv.cpu(), dv)
    torch.cuda.synchronize()


def test_request_sized_migration_roundtrip(kernels):
    """A 2048-token request at the Qwen3-8B layout (36 layers, 128 blocks of 32 KiB per layer and tensor):
    migrate there and back, the pool must be unchanged (round-trip property)."""
    L, nb, Hkv, B, D = 36, 160, 8, 16, 128
    src_k = torch.randn(L, nb, Hkv, B, D, device="cuda:0").bfloat16()
    src_v = torch.randn(L, nb, Hkv, B, D, device="cuda:0").bfloat16()
    mid_k, mid_v = torch.zeros_like(src_k), torch.zeros_like(src_v)
    back_k, back_v = torch.zeros_like(src_k), torch.zeros_like(src_v)
    ids = torch.randperm(nb)[:128].tolist()
    there = torch.randperm(nb)[:128].tolist()
    kv_transfer.transfer_kv(src_k, src_v, mid_k, mid_v, ids, dst_block_table=there)
    kv_transfer.transfer_kv(mid_k, mid_v, back_k, back_v, there, dst_block_table=ids)
    torch.cuda.synchronize()
    sel = torch.tensor(ids, device="cuda:0")
    assert torch.equal(back_k[:, sel], src_k[:, sel]) and torch.equal(back_v[:, sel], src_v[:, sel])
    rest = torch.ones(nb, dtype=torch.bool, device="cuda:0")
    rest[sel] = False
    assert torch.count_nonzero(back_k[:, rest]) == 0


@pytest.mark.parametrize("block_shape,dtype", [((1, 16, 64), torch.float16),     # 2 KiB units: one small piece each
                                               ((8, 32, 128), torch.bfloat16),   # 64 KiB units: two pieces each
                                               ((5, 16, 72), torch.float16)])    # 11 520-byte units
def test_unit_sizes(kernels, block_shape, dtype):
    Hkv, B, D = block_shape
    L, nb = 3, 12
    sk, sv, dsk, dsv = _pools(L, nb, Hkv, B, D, dtype, "cuda:0", 9)
    dk, dv = torch.zeros_like(sk), torch.zeros_like(sv)
    ddk, ddv = dk.to("cuda:0"), dv.to("cuda:0")
    kv_transfer.transfer_kv(dsk, dsv, ddk, ddv, [0, 11, 5, 6, 2], dst_block_table=[4, 3, 2, 1, 0], max_ctas=3)
    paged_oracle.kv_migrate(sk, sv, dk, dv, [0, 11, 5, 6, 2], [4, 3, 2, 1, 0])
    torch.cuda.synchronize()
    assert torch.equal(ddk.cpu(), dk) and torch.equal(ddv.cpu(), dv)


def test_migration_overlaps_decode_attention(kernels):
    """Migration on a side stream while decode attention runs on the main stream: both results are exact
    (the migrated blocks are disjoint from the ones the decode batch reads, as the allocator guarantees)."""
    from nanopd_b200 import workloads
    b = workloads.make_decode_batch([700, 1500, 64, 3000], 32, 8, 128, 16, torch.bfloat16, device="cuda:0", seed=5,
                                    pool_blocks=400)
    want = torch.zeros_like(b.query)
    kernels.paged_attention_forward(want, b.query, b.k_cache, b.v_cache, b.block_tables, b.ctx_lens, b.scale, 16,
                                    b.block_tables.size(1))
    L = 4
    src_k = torch.randn(L, 400, 8, 16, 128, device="cuda:0").bfloat16()
    src_v = torch.randn(L, 400, 8, 16, 128, device="cuda:0").bfloat16()
    dst_k, dst_v = torch.zeros_like(src_k), torch.zeros_like(src_v)
    ids = torch.randperm(400)[:300].tolist()
    side = torch.cuda.Stream(device="cuda:0")
    side.wait_stream(torch.cuda.current_stream())
    out = torch.zeros_like(b.query)
    for _ in range(3):
        kv_transfer.transfer_kv(src_k, src_v, dst_k, dst_v, ids, stream=side, max_ctas=8)
        kernels.paged_attention_forward(out, b.query, b.k_cache, b.v_cache, b.block_tables, b.ctx_lens, b.scale, 16,
                                        b.block_tables.size(1))
    torch.cuda.synchronize()
    assert torch.equal(out, want)
    sel = torch.tensor(ids, device="cuda:0")
    assert torch.equal(dst_k[:, sel], src_k[:, sel]) and torch.equal(dst_v[:, sel], src_v[:, sel])


def test_bad_block_id_is_skipped(kernels):
    L, nb, Hkv, B, D = 2, 4, 2, 16, 64
    sk, sv, dsk, dsv = _pools(L, nb, Hkv, B, D, torch.float16, "cuda:0", 3)
    ddk, ddv = torch.zeros_like(dsk), torch.zeros_like(dsv)
    kv_transfer.transfer_kv(dsk, dsv, ddk, ddv, [1, 99])
    assert kernels.check_status(raise_on_error=False) == 1
    assert torch.equal(ddk[:, 1], dsk[:, 1]) and torch.count_nonzero(ddk[:, [0, 2, 3]]) == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_to_peer_pull_over_nvlink(kernels):
    """Prefill pool on cuda:0, decode pool on cuda:1, pulled by a kernel on cuda:1's stream.
    Plain peer loads only."""
    L, nb, Hkv, B, D = 4, 32, 8, 16, 128
    sk, sv, dsk, dsv = _pools(L, nb, Hkv, B, D, torch.bfloat16, "cuda:0", 4)
    ddk = torch.zeros(L, nb, Hkv, B, D, dtype=torch.bfloat16, device="cuda:1")
    ddv = torch.zeros_like(ddk)
    torch.cuda.synchronize("cuda:0")
    stream = torch.cuda.Stream(device="cuda:1")
    table = [3, 30, 11, 12]
    assert kv_transfer.transfer_kv(dsk, dsv, ddk, ddv, table, stream=stream) == "p2p"
    stream.synchronize()
    dk, dv = torch.zeros_like(sk), torch.zeros_like(sv)
    paged_oracle.kv_migrate(sk, sv, dk, dv, table)
    assert torch.equal(ddk.cpu(), dk) and torch.equal(ddv.cpu(), dv)
    with torch.cuda.device(1):
        assert kernels.check_status(raise_on_error=False) == 0


@pytest.mark.parametrize("two_gpus", [False, True])
def test_prefill_here_decode_there(kernels, two_gpus):
    """The disaggregated hand-off end to end at the attention level: a prompt's K/V is written into the prefill
    side's pool (store kernel), its pages move to OTHER block ids of the decode side's pool (migration kernel, over
    NVLink when two GPUs are present), and decode attention over the moved pages — after storing one more token
    there — matches the oracle run on the prompt as a whole."""
    if two_gpus and torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from conftest import TOL
    paged_kernels = kernels
    from nanopd_b200 import kv_transfer
    from oracle import paged_oracle
    torch.manual_seed(31)
    dtype = torch.bfloat16
    p_dev, d_dev = "cuda:0", ("cuda:1" if two_gpus else "cuda:0")
    L, Hq, Hkv, D, B = 2, 8, 2, 128, 16
    n_prompt = 203
    nblk = (n_prompt + 1 + B - 1) // B
    p_pool, d_pool = 40, 64
    k_prompt = torch.randn(L, Hkv, n_prompt, D).to(dtype)
    v_prompt = torch.randn(L, Hkv, n_prompt, D).to(dtype)
    # prefill side: store the prompt layer by layer
    pk_cache = torch.zeros(L, p_pool, Hkv, B, D, dtype=dtype, device=p_dev)
    pv_cache = torch.zeros_like(pk_cache)
    src_ids = torch.randperm(p_pool)[:nblk].tolist()
    with torch.cuda.device(p_dev):
        for li in range(L):
            paged_kernels.paged_kv_store(pk_cache[li], pv_cache[li], k_prompt[li].to(p_dev), v_prompt[li].to(p_dev),
                                         torch.tensor(src_ids, dtype=torch.int32, device=p_dev), 0)
    torch.cuda.synchronize(p_dev)
    # decode side: pull the pages into its own ids
    dk_cache = torch.randn(L, d_pool, Hkv, B, D, device=d_dev).to(dtype)       # other requests' pages
    dv_cache = torch.randn(L, d_pool, Hkv, B, D, device=d_dev).to(dtype)
    dst_ids = torch.randperm(d_pool)[:nblk].tolist()
    assert kv_transfer.transfer_kv(pk_cache, pv_cache, dk_cache, dv_cache, src_ids, dst_block_table=dst_ids) == "p2p"
    # one decode step there: store token n_prompt, attend over n_prompt + 1 tokens
    q = torch.randn(1, Hq, D).to(dtype)
    k_new, v_new = torch.randn(L, Hkv, 1, D).to(dtype), torch.randn(L, Hkv, 1, D).to(dtype)
    table = torch.tensor([dst_ids], dtype=torch.int32, device=d_dev)
    pos = torch.tensor([n_prompt], dtype=torch.int32, device=d_dev)
    out = torch.zeros(L, 1, Hq, D, dtype=dtype, device=d_dev)
    with torch.cuda.device(d_dev):
        for li in range(L):
            paged_kernels.paged_kv_store(dk_cache[li], dv_cache[li], k_new[li].to(d_dev), v_new[li].to(d_dev), table, pos)
            paged_kernels.paged_attention_forward(out[li], q.to(d_dev), dk_cache[li], dv_cache[li], table, pos + 1,
                                                  D ** -0.5, B, table.size(1))
    torch.cuda.synchronize(d_dev)
    # oracle: the same sequence in one contiguous pool
    for li in range(L):
        kc = torch.zeros(nblk, Hkv, B, D, dtype=dtype)
        vc = torch.zeros_like(kc)
        ids = torch.arange(nblk, dtype=torch.int32)
        k_all = torch.cat((k_prompt[li], k_new[li]), dim=1)
        v_all = torch.cat((v_prompt[li], v_new[li]), dim=1)
        paged_oracle.kv_store(kc, vc, k_all, v_all, ids.unsqueeze(0).expand(n_prompt + 1, -1),
                              torch.arange(n_prompt + 1, dtype=torch.int32))
        want = paged_oracle.paged_decode_attention(q, kc, vc, ids.unsqueeze(0), torch.tensor([n_prompt + 1], dtype=torch.int32),
                                                   D ** -0.5)
        assert (out[li].float().cpu() - want).abs().max().item() <= TOL[dtype]
        # the moved pages are bit-identical to what the prefill side wrote
        assert torch.equal(dk_cache[li, dst_ids[0]].cpu(), pk_cache[li, src_ids[0]].cpu())
    for d in {p_dev, d_dev}:
        assert paged_kernels.check_status(d, raise_on_error=False) == 0


def test_receiver_promotes_requests_as_their_pages_arrive(kernels):
    """The receiving half as DecodeWorker keeps it (nanoPD/workers/decode_worker.py:36-68): three requests issued
    on the transfer stream, promoted without a host wait once their events have completed, pages exact and placed
    at the destination allocator's ids."""
    torch.manual_seed(21)
    L, nb, Hkv, B, D = 4, 64, 2, 16, 128
    src_k = torch.randn(L, nb, Hkv, B, D, device="cuda:0").to(torch.float16)
    src_v = torch.randn(L, nb, Hkv, B, D, device="cuda:0").to(torch.float16)
    dst_k, dst_v = torch.zeros_like(src_k), torch.zeros_like(src_v)
    rx = kv_transfer.KVReceiver(dst_k, dst_v)
    requests = {"a": ([3, 9, 27], [0, 1, 2]), "b": ([5, 6], [10, 11]), "c": (list(range(30, 50)), list(range(40, 60)))}
    for name, (src_ids, dst_ids) in requests.items():
        assert rx.receive_kv_async(name, src_ids, src_k=src_k, src_v=src_v, dst_block_table=dst_ids) == "p2p"
    assert rx.num_pending == 3
    promoted = []
    for _ in range(10000):
        promoted += rx.promote_ready()
        if rx.num_pending == 0:
            break
    assert promoted == ["a", "b", "c"] and rx.num_pending == 0
    # the compute stream waited for the events: a kernel launched now sees the pages
    for src_ids, dst_ids in requests.values():
        assert torch.equal(dst_k[:, dst_ids], src_k[:, src_ids]) and torch.equal(dst_v[:, dst_ids], src_v[:, src_ids])
    untouched = [i for i in range(nb) if i not in sum((d for _, d in requests.values()), [])]
    assert not dst_k[:, untouched].any()
    assert kernels.check_status("cuda:0", raise_on_error=False) == 0
