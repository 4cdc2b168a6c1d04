"""GPU: ``nanopd_b200.kv_transfer`` as a drop-in for the reference's ``workers/kv_transfer`` module —
the pinned relay (``PinnedKVBuffer``, ``extract_kv_to_pinned``, ``load_kv_from_pinned``,
nanoPD/workers/kv_transfer.py:17-66), a receive call that does not block the host, and the bounded wait of the
migration kernel.  Everything goes through the C ABI; results are compared with the oracle bit for bit."""
import ctypes
import time

import pytest
import torch

from nanopd_b200 import _lib, kv_transfer
from oracle import paged_oracle

pytestmark = pytest.mark.gpu


def _pool(L, nb, Hkv, B, D, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(L, nb, Hkv, B, D, generator=g).to(dtype), torch.randn(L, nb, Hkv, B, D, generator=g).to(dtype))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_pool_to_pinned_to_other_pool(kernels, dtype):
    """Prefill pool -> pinned buffer -> decode pool, the reference's relay path, against the oracle."""
    L, nb, Hkv, B, D = 5, 40, 8, 16, 128
    sk, sv = _pool(L, nb, Hkv, B, D, dtype, 0)
    dk, dv = _pool(L, nb, Hkv, B, D, dtype, 1)
    dsk, dsv, ddk, ddv = sk.cuda(), sv.cuda(), dk.cuda(), dv.cuda()
    table = [7, 39, 0, 22, 21, 3, 18]
    buf = kv_transfer.PinnedKVBuffer(L, len(table), Hkv, B, D, dtype=dtype)
    assert buf.k.is_pinned() and buf.v.is_pinned() and tuple(buf.k.shape) == (L, len(table), Hkv, B, D)
    buf.k.fill_(7), buf.v.fill_(7)
    kv_transfer.extract_kv_to_pinned(dsk, dsv, table, buf)          # returns after the host can read the buffer
    want_k, want_v = torch.zeros_like(buf.k), torch.zeros_like(buf.v)
    paged_oracle.extract_kv_to_buffer(sk, sv, table, want_k, want_v)
    assert torch.equal(buf.k, want_k) and torch.equal(buf.v, want_v)

    stream = torch.cuda.Stream()
    kv_transfer.load_kv_from_pinned(ddk, ddv, table, buf, stream=stream)
    stream.synchronize()
    paged_oracle.load_kv_from_buffer(dk, dv, table, want_k, want_v)
    assert torch.equal(ddk.cpu(), dk) and torch.equal(ddv.cpu(), dv)
    # the two halves together are the reference's transfer: same result as oracle.kv_migrate
    dk2, dv2 = _pool(L, nb, Hkv, B, D, dtype, 1)
    paged_oracle.kv_migrate(sk, sv, dk2, dv2, table)
    assert torch.equal(dk, dk2) and torch.equal(dv, dv2)


def test_buffer_larger_than_the_request_and_from_runner(kernels):
    class Runner:                      # the attributes PinnedKVBuffer.from_runner reads
        num_kv_heads, block_size, head_dim = 2, 16, 64
        k_cache = torch.zeros(3, 8, 2, 16, 64, dtype=torch.float16, device="cuda")
    sk, sv = _pool(3, 8, 2, 16, 64, torch.float16, 5)
    buf = kv_transfer.PinnedKVBuffer.from_runner(Runner, num_blocks=6)
    assert tuple(buf.k.shape) == (3, 6, 2, 16, 64) and buf.k.dtype == torch.float16
    buf.k.zero_(), buf.v.zero_()
    kv_transfer.extract_kv_to_pinned(sk.cuda(), sv.cuda(), [4, 1], buf)
    assert torch.equal(buf.k[:, 0], sk[:, 4]) and torch.equal(buf.v[:, 1], sv[:, 1]) and not buf.k[:, 2:].any()
    with pytest.raises(RuntimeError):
        kv_transfer.extract_kv_to_pinned(sk.cuda(), sv.cuda(), list(range(7)), buf)


def test_transfer_kv_relays_through_the_buffer_without_peer_access(kernels, monkeypatch):
    """With no peer access transfer_kv takes the buffer path and says so, as the reference does
    (nanoPD/workers/kv_transfer.py:80-83).  Peer access is always there on an NVSwitch box, so the probe is
    made to answer no; both pools then sit on cuda:0 but are treated as two devices."""
    L, nb, Hkv, B, D = 2, 12, 2, 16, 128
    sk, sv = _pool(L, nb, Hkv, B, D, torch.bfloat16, 2)
    dk, dv = _pool(L, nb, Hkv, B, D, torch.bfloat16, 3)
    dsk, dsv, ddk, ddv = sk.cuda(), sv.cuda(), dk.cuda(), dv.cuda()
    table = [11, 2, 5]
    buf = kv_transfer.PinnedKVBuffer(L, len(table), Hkv, B, D, dtype=torch.bfloat16)
    kv_transfer.extract_kv_to_pinned(dsk, dsv, table, buf)

    class OtherDevice:                      # a source the destination cannot reach
        device = torch.device("cuda", 99)
    monkeypatch.setattr(kv_transfer, "_check_p2p", lambda s, d: False)
    assert kv_transfer.transfer_kv(OtherDevice, OtherDevice, ddk, ddv, table, buf=buf) == "pinned_relay"
    with pytest.raises(RuntimeError):
        kv_transfer.transfer_kv(OtherDevice, OtherDevice, ddk, ddv, table, buf=None)
    paged_oracle.kv_migrate(sk, sv, dk, dv, table)
    assert torch.equal(ddk.cpu(), dk) and torch.equal(ddv.cpu(), dv)


def test_receive_returns_while_an_earlier_transfer_is_in_flight(kernels):
    """receive_kv_async only enqueues: with the transfer stream kept busy for about 0.3 s, two receive calls given
    Python lists return in a fraction of that, with the first request's event still pending."""
    L, nb, Hkv, B, D = 2, 32, 2, 16, 128
    sk, sv = _pool(L, nb, Hkv, B, D, torch.float16, 8)
    dsk, dsv = sk.cuda(), sv.cuda()
    ddk, ddv = torch.zeros_like(dsk), torch.zeros_like(dsv)
    rx = kv_transfer.KVReceiver(ddk, ddv)
    rx.receive_kv_async("warm", [0], src_k=dsk, src_v=dsv, dst_block_table=[0])     # workspace, pinned cache, peer maps
    torch.cuda.synchronize()
    assert rx.promote_ready() == ["warm"]
    clock_khz = torch.cuda.get_device_properties(0).clock_rate
    with torch.cuda.stream(rx.transfer_stream):
        torch.cuda._sleep(int(0.3 * clock_khz * 1e3))          # a bounded busy kernel ahead of the transfers
    t0 = time.perf_counter()
    rx.receive_kv_async("a", list(range(1, 17)), src_k=dsk, src_v=dsv, dst_block_table=list(range(1, 17)))
    rx.receive_kv_async("b", [20, 21], src_k=dsk, src_v=dsv, dst_block_table=[30, 31])
    host_seconds = time.perf_counter() - t0
    still_running = rx.promote_ready() == [] and rx.num_pending == 2
    torch.cuda.synchronize()
    assert host_seconds < 0.1, f"two receive calls held the host for {host_seconds:.3f} s"
    assert still_running, "the earlier work on the transfer stream had already finished: nothing was shown"
    assert rx.promote_ready() == ["a", "b"]
    assert torch.equal(ddk[:, 1:17], dsk[:, 1:17]) and torch.equal(ddv[:, 30:32], dsv[:, 20:22])


def test_bounded_wait_of_the_migration_kernel(kernels):
    """One load is announced to its barrier but never issued and the wait limit is set to about a millisecond: the
    CTA that owns it gives up, reports NPD_STATUS_WAIT_TIMEOUT and returns; every other CTA finishes its share;
    check_status cleans up; the next ordinary migration is exact."""
    lib = _lib.load()
    L, nb, Hkv, B, D = 2, 16, 2, 16, 128
    sk, sv = _pool(L, nb, Hkv, B, D, torch.float16, 13)
    dsk, dsv = sk.cuda(), sv.cuda()
    ddk, ddv = torch.zeros_like(dsk), torch.zeros_like(dsv)
    ids = torch.arange(nb, dtype=torch.int32, device="cuda")
    status = torch.zeros(64, dtype=torch.int32, device="cuda")
    belems = Hkv * B * D
    grid = 4
    withheld = 6                                   # piece 6 belongs to CTA 6 % 4 = 2
    stream = torch.cuda.current_stream().cuda_stream
    t0 = time.perf_counter()
    _lib.check(lib.npd_testing_kv_migrate_withheld(
        dsk.data_ptr(), dsv.data_ptr(), ddk.data_ptr(), ddv.data_ptr(), ids.data_ptr(), ids.data_ptr(), nb, L,
        belems, 2, dsk.stride(0), dsk.stride(1), nb, ddk.stride(0), ddk.stride(1), nb, grid, status.data_ptr(),
        stream, withheld, 2_000_000))
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0
    assert int(status[0].item()) == _lib.NPD_STATUS_WAIT_TIMEOUT
    # a unit is one 8 KiB piece here; piece p = (pair, layer, K|V) in that order, CTA c copies pieces c, c+4, ...
    pieces = [(pair, layer, kv) for pair in range(nb) for layer in range(L) for kv in range(2)]
    for i, (pair, layer, kv) in enumerate(pieces):
        got, want = (ddv if kv else ddk)[layer, pair], (dsv if kv else dsk)[layer, pair]
        if i % grid != withheld % grid or i < withheld:
            assert torch.equal(got, want), f"piece {i} of a CTA that did not time out"
        else:
            assert not got.any(), f"piece {i} lies behind the withheld one in its CTA's sequence"
    # the same through the module: the status word of the stream's workspace is read, reported and cleaned
    kernels.paged_kv_migrate(dsk.view(L, nb, Hkv, B, D), dsv, ddk, ddv, [1], [1])       # creates the workspace
    torch.cuda.synchronize()
    from nanopd_b200 import paged_kernels as shim
    ws = shim._workspaces[(0, stream)]
    _lib.check(lib.npd_testing_kv_migrate_withheld(
        dsk.data_ptr(), dsv.data_ptr(), ddk.data_ptr(), ddv.data_ptr(), ids.data_ptr(), ids.data_ptr(), nb, L,
        belems, 2, dsk.stride(0), dsk.stride(1), nb, ddk.stride(0), ddk.stride(1), nb, grid, ws.data_ptr(),
        stream, withheld, 2_000_000))
    with pytest.raises(RuntimeError, match="wait time-out"):
        kernels.check_status()
    assert kernels.check_status(raise_on_error=False) == 0
    ddk.zero_(), ddv.zero_()
    kv_transfer.transfer_kv(dsk, dsv, ddk, ddv, list(range(nb)))
    torch.cuda.synchronize()
    assert torch.equal(ddk, dsk) and torch.equal(ddv, dsv)
