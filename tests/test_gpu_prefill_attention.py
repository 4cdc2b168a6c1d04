"""GPU: chunked-prefill causal attention over paged K/V (tcgen05 path) against the fp32 oracle.

Tolerance (max-abs against the fp32-accumulated oracle): 2e-3 for fp16, 1e-2 for bf16."""
import pytest
import torch

from conftest import TOL
from nanopd_b200 import workloads
from oracle import paged_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def build_prompt(L, Hq, Hkv, D, B, dtype, seed=0, extra_blocks=3, poison=False):
    """A prompt of L tokens whose K/V already sit in the pages (stored with the oracle on the CPU)."""
    g = torch.Generator().manual_seed(seed)
    nblk = (L + B - 1) // B
    pool = nblk + extra_blocks
    q = torch.randn(L, Hq, D, generator=g).to(dtype)
    k = torch.randn(Hkv, L, D, generator=g).to(dtype)
    v = torch.randn(Hkv, L, D, generator=g).to(dtype)
    table = torch.randperm(pool, generator=g)[:nblk].to(torch.int32)
    fill = float("nan") if poison else 0.0
    k_cache = torch.full((pool, Hkv, B, D), fill, dtype=dtype)
    v_cache = torch.full((pool, Hkv, B, D), fill, dtype=dtype)
    paged_oracle.kv_store(k_cache, v_cache, k, v, table.unsqueeze(0).expand(L, -1), torch.arange(L, dtype=torch.int32))
    return q, table, k_cache, v_cache


def run_chunks(kernels, q_rows, k_cache, v_cache, tables, offsets, tokens, starts, scale, B):
    out = torch.zeros_like(q_rows)
    kernels.paged_prefill_attention(out, q_rows, k_cache, v_cache, tables, offsets, tokens, starts, scale, B,
                                    tables.size(1))
    torch.cuda.synchronize()
    return out


def check_single(kernels, L, start, n, Hq, Hkv, B, dtype, seed=0, poison=False, D=128):
    """Chunk [start, start+n) of an L-token prompt; keys beyond start+n exist in the pool but must be ignored."""
    q, table, kc, vc = build_prompt(L, Hq, Hkv, D, B, dtype, seed=seed, poison=poison)
    if poison:   # the contract only promises keys < start+n: poison everything later as well
        for pos in range(start + n, L):
            kc[int(table[pos // B]), :, pos % B] = float("nan")
            vc[int(table[pos // B]), :, pos % B] = float("nan")
    scale = D ** -0.5
    qc = q[start:start + n].contiguous()
    want = paged_oracle.paged_prefill_attention(qc, kc, vc, table, start, scale)
    got = run_chunks(kernels, qc.to(DEV), kc.to(DEV), vc.to(DEV), table.unsqueeze(0).to(DEV),
                     [0], [n], [start], scale, B).float().cpu()
    assert torch.isfinite(got).all()
    err = (got - want).abs().max().item()
    assert err <= TOL[dtype], f"max abs err {err}"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("L,start,n", [(32, 0, 32), (128, 0, 128), (200, 0, 200), (300, 128, 100), (700, 512, 188),
                                       (64, 0, 1), (130, 129, 1), (1024, 512, 512)])
def test_single_chunk_group4(kernels, dtype, L, start, n):
    check_single(kernels, L, start, n, 8, 2, 16, dtype)


@pytest.mark.parametrize("Hq,Hkv", [(1, 1), (2, 1), (4, 4), (8, 1), (12, 2), (16, 1), (32, 8)])
def test_group_sizes(kernels, Hq, Hkv):
    check_single(kernels, 333, 100, 233, Hq, Hkv, 16, torch.bfloat16, seed=3)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_block_size_32(kernels, dtype):
    check_single(kernels, 500, 200, 300, 8, 2, 32, dtype, seed=5)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("L,start,n,poison", [(500, 200, 300, False), (77, 0, 77, True), (1100, 1000, 100, True),
                                              (264, 256, 8, False)])
def test_block_size_8(kernels, dtype, L, start, n, poison):
    """Blocks of 8 tokens (what the decode kernel also takes): a 16-key row group of a K/V tile then lies in two
    blocks and is fetched as two boxes of 8 rows."""
    check_single(kernels, L, start, n, 8, 2, 8, dtype, seed=6, poison=poison)


@pytest.mark.parametrize("D,Hq,Hkv", [(64, 4, 4), (128, 8, 2), (256, 4, 1)])
@pytest.mark.parametrize("L,start,n,poison", [(500, 200, 300, False), (77, 0, 77, True), (264, 256, 8, False)])
def test_block_size_4(kernels, D, Hq, Hkv, L, start, n, poison):
    """Blocks of 4 tokens, the smallest size the decode kernel takes: a 16-key row group is four boxes of 4 rows
    (64 boxes per 128-key tile, two copy instructions per producer warp)."""
    check_single(kernels, L, start, n, Hq, Hkv, 4, torch.float16, seed=16, poison=poison, D=D)
    check_single(kernels, L, start, n, Hq, Hkv, 4, torch.bfloat16, seed=17, poison=poison, D=D)


def test_unwritten_slots_are_never_used(kernels):
    """NaN everywhere outside keys [0, start+n): later tokens of the prompt, the tail of the last page
    and unused blocks must not reach the output."""
    check_single(kernels, 300, 90, 75, 8, 2, 16, torch.float16, seed=7, poison=True)
    check_single(kernels, 140, 0, 130, 4, 1, 16, torch.bfloat16, seed=8, poison=True)


def test_several_chunks_in_one_call(kernels):
    """Two prompts packed in one forward (as PrefillWorker does, prefill_worker.py:47-64) plus a later chunk
    of a third one; each chunk has its own table row."""
    D, B, Hq, Hkv = 128, 16, 8, 2
    scale = D ** -0.5
    specs = [(150, 0, 150, 11), (90, 0, 90, 12), (400, 256, 144, 13)]      # (L, start, n, seed)
    prompts = [build_prompt(L, Hq, Hkv, D, B, torch.bfloat16, seed=s) for L, _, _, s in specs]
    # one shared pool: concatenate the per-prompt pools and shift the ids
    base, tables, kcs, vcs = 0, [], [], []
    for (_, table, kc, vc) in prompts:
        tables.append(table + base)
        kcs.append(kc)
        vcs.append(vc)
        base += kc.size(0)
    kc, vc = torch.cat(kcs), torch.cat(vcs)
    max_blk = max(t.numel() for t in tables)
    bt = torch.zeros(len(specs), max_blk, dtype=torch.int32)
    for i, t in enumerate(tables):
        bt[i, :t.numel()] = t
    q_rows = torch.cat([p[0][st:st + n] for p, (_, st, n, _) in zip(prompts, specs)])
    offsets, tokens, starts = [], [], []
    off = 0
    for (_, st, n, _) in specs:
        offsets.append(off), tokens.append(n), starts.append(st)
        off += n
    got = run_chunks(kernels, q_rows.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), offsets, tokens, starts, scale, B)
    got = got.float().cpu()
    for i, (_, st, n, _) in enumerate(specs):
        want = paged_oracle.paged_prefill_attention(q_rows[offsets[i]:offsets[i] + n], kc, vc, tables[i], st, scale)
        assert (got[offsets[i]:offsets[i] + n] - want).abs().max().item() <= TOL[torch.bfloat16]


def test_many_items_of_a_single_half_step(kernels):
    """64 short prompts (33-64 tokens, so every work item is ONE 64-key half-step per query tile) in one launch,
    a few items per SM in a row: a softmax group then finishes its next item before the epilogue warps have
    written the one before, the case its hand-over has to wait for."""
    D, B, Hq, Hkv = 128, 16, 32, 8
    scale = D ** -0.5
    lens = [33 + (7 * i) % 32 for i in range(64)]
    prompts = [build_prompt(L, Hq, Hkv, D, B, torch.bfloat16, seed=100 + i, extra_blocks=1) for i, L in enumerate(lens)]
    base, tables, kcs, vcs = 0, [], [], []
    for (_, table, kc, vc) in prompts:
        tables.append(table + base)
        kcs.append(kc)
        vcs.append(vc)
        base += kc.size(0)
    kc, vc = torch.cat(kcs), torch.cat(vcs)
    max_blk = max(t.numel() for t in tables)
    bt = torch.zeros(len(lens), max_blk, dtype=torch.int32)
    for i, t in enumerate(tables):
        bt[i, :t.numel()] = t
    q_rows = torch.cat([p[0] for p in prompts])
    offsets, off = [], 0
    for L in lens:
        offsets.append(off)
        off += L
    starts = [0] * len(lens)
    for _ in range(3):      # the hand-over depends on timing: more than one launch
        got = run_chunks(kernels, q_rows.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), offsets, lens, starts, scale, B)
    assert kernels.check_status(DEV, raise_on_error=False) == 0
    got = got.float().cpu()
    for i, L in enumerate(lens):
        want = paged_oracle.paged_prefill_attention(q_rows[offsets[i]:offsets[i] + L], kc, vc, tables[i], 0, scale)
        # rows that see only a few keys are as large as the values themselves (|x| up to 4, where one bf16 rounding
        # step is 0.016): the absolute tolerance of the other tests plus half a rounding step of the result
        err = (got[offsets[i]:offsets[i] + L] - want).abs()
        assert (err <= TOL[torch.bfloat16] + want.abs() * 2.0 ** -8).all(), err.max().item()


def test_store_then_prefill_chunks_compose(kernels):
    """The caller's order on the GPU: store each 128-token chunk, then attend; the rows of all chunks
    together equal full causal attention over the prompt."""
    D, B, Hq, Hkv, L, chunk = 128, 16, 8, 2, 384, 128
    torch.manual_seed(21)
    q = torch.randn(L, Hq, D).half()
    k = torch.randn(Hkv, L, D).half()
    v = torch.randn(Hkv, L, D).half()
    nblk = L // B
    table = torch.randperm(nblk + 4)[:nblk].to(torch.int32)
    kc = torch.zeros(nblk + 4, Hkv, B, D, dtype=torch.float16, device=DEV)
    vc = torch.zeros_like(kc)
    scale = D ** -0.5
    outs = []
    for s in range(0, L, chunk):
        pos = torch.arange(s, s + chunk, dtype=torch.int32, device=DEV)
        kernels.paged_kv_store(kc, vc, k[:, s:s + chunk].contiguous().to(DEV), v[:, s:s + chunk].contiguous().to(DEV),
                               table.to(DEV).unsqueeze(0).expand(chunk, -1), pos)
        outs.append(run_chunks(kernels, q[s:s + chunk].contiguous().to(DEV), kc, vc, table.unsqueeze(0).to(DEV),
                               [0], [chunk], [s], scale, B))
    got = torch.cat(outs).float().cpu()
    want = paged_oracle.paged_prefill_attention(q, kc.cpu(), vc.cpu(), table, 0, scale)
    assert (got - want).abs().max().item() <= TOL[torch.float16]


def test_config3_every_chunk_vs_oracle(kernels):
    """Configuration 3 (Qwen3-8B shape, 512-token chunks over existing paged K/V): EVERY chunk of every prompt
    against the oracle, all of them in one call."""
    m = workloads.make_config3(device="cpu", seed=0)
    kc, vc = m.decode.k_cache, m.decode.v_cache
    # the prompts' K/V: store every chunk (oracle on CPU keeps the test independent of the store kernel)
    for ch in m.chunks:
        n = ch.num_tokens
        paged_oracle.kv_store(kc, vc, ch.k_new, ch.v_new, ch.block_table.unsqueeze(0).expand(n, -1),
                              torch.arange(ch.start_position, ch.start_position + n, dtype=torch.int32))
    chunks = list(m.chunks)
    torch.set_num_threads(max(1, __import__("os").cpu_count() or 1))
    max_blk = max(c.block_table.numel() for c in chunks)
    bt = torch.zeros(len(chunks), max_blk, dtype=torch.int32)
    for i, c in enumerate(chunks):
        bt[i, :c.block_table.numel()] = c.block_table
    q_rows = torch.cat([c.query for c in chunks])
    offsets, tokens, starts, off = [], [], [], 0
    for c in chunks:
        offsets.append(off), tokens.append(c.num_tokens), starts.append(c.start_position)
        off += c.num_tokens
    scale = m.decode.scale
    got = run_chunks(kernels, q_rows.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), offsets, tokens, starts, scale, 16)
    got = got.float().cpu()
    assert torch.isfinite(got).all()
    for i, c in enumerate(chunks):
        want = paged_oracle.paged_prefill_attention(c.query, kc, vc, c.block_table, c.start_position, scale)
        err = (got[offsets[i]:offsets[i] + c.num_tokens] - want).abs().max().item()
        assert err <= TOL[torch.bfloat16], f"chunk start {c.start_position}: {err}"


def test_argument_errors(kernels):
    q = torch.zeros(16, 8, 128, dtype=torch.float16, device=DEV)
    kc = torch.zeros(4, 2, 16, 128, dtype=torch.float16, device=DEV)
    bt = torch.zeros(1, 4, dtype=torch.int32, device=DEV)
    out = torch.zeros_like(q)
    with pytest.raises(RuntimeError):
        kernels.paged_prefill_attention(out, q, kc, kc, bt.long(), [0], [16], [0], 1.0, 16, 4)
    with pytest.raises(RuntimeError):   # chunk beyond its table
        kernels.paged_prefill_attention(out, q, kc, kc, bt, [0], [16], [60], 1.0, 16, 4)
    with pytest.raises(RuntimeError):   # chunk outside q
        kernels.paged_prefill_attention(out, q, kc, kc, bt, [8], [16], [0], 1.0, 16, 4)
    kc2 = torch.zeros(16, 2, 2, 128, dtype=torch.float16, device=DEV)
    with pytest.raises(RuntimeError):   # block size 2 is outside the kernel's set (4, 8, 16, 32)
        kernels.paged_prefill_attention(out, q, kc2, kc2, torch.zeros(1, 8, dtype=torch.int32, device=DEV), [0], [16], [0], 1.0, 2, 8)


def test_more_chunks_than_one_launch_takes(kernels):
    """A call with more prompt chunks than fit the kernel's parameter arrays (64) is split into launches: 150 short
    prompts, whole-prompt prefill of each (the packing PrefillWorker uses, nanoPD/workers/prefill_worker.py:47-64)."""
    torch.manual_seed(42)
    dtype, Hq, Hkv, D, B = torch.float16, 4, 2, 128, 16
    n_prompts = 150
    lens = torch.randint(1, 50, (n_prompts,)).tolist()
    nblk = [(l + B - 1) // B for l in lens]
    pool = sum(nblk) + 2
    perm = torch.randperm(pool)
    tables = torch.zeros(n_prompts, max(nblk), dtype=torch.int32)
    kc = torch.zeros(pool, Hkv, B, D, dtype=dtype)
    vc = torch.zeros_like(kc)
    qs, want, offs, o, pb = [], [], [], 0, 0
    scale = D ** -0.5
    for i, (l, nb) in enumerate(zip(lens, nblk)):
        tables[i, :nb] = perm[pb:pb + nb].to(torch.int32)
        pb += nb
        q = torch.randn(l, Hq, D).to(dtype)
        k = torch.randn(Hkv, l, D).to(dtype)
        v = torch.randn(Hkv, l, D).to(dtype)
        paged_oracle.kv_store(kc, vc, k, v, tables[i:i + 1].expand(l, -1), torch.arange(l, dtype=torch.int32))
        qs.append(q)
        offs.append(o)
        o += l
    for i, l in enumerate(lens):
        want.append(paged_oracle.paged_prefill_attention(qs[i], kc, vc, tables[i], 0, scale))
    got = run_chunks(kernels, torch.cat(qs).to(DEV), kc.to(DEV), vc.to(DEV), tables.to(DEV), offs, lens, [0] * n_prompts,
                     scale, B).float().cpu()
    err = (got - torch.cat(want)).abs().max().item()
    assert err <= TOL[dtype], err


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("L,start,n,Hq,Hkv,B", [(40, 0, 40, 8, 2, 16), (300, 128, 100, 32, 8, 16), (700, 512, 188, 16, 4, 32),
                                                (1500, 1000, 500, 14, 2, 16), (260, 0, 260, 4, 4, 16)])
def test_head_dim_64(kernels, dtype, L, start, n, Hq, Hkv, B):
    """The 64-wide variant of the kernel (one 64-element half per tile; Llama-3.2-1B / Qwen2-0.5B head size)."""
    check_single(kernels, L, start, n, Hq, Hkv, B, dtype, seed=L, D=64)
    check_single(kernels, L, start, n, Hq, Hkv, B, dtype, seed=L + 1, poison=True, D=64)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("L,start,n,Hq,Hkv,B", [(200, 0, 200, 4, 1, 16), (700, 512, 188, 8, 2, 16), (130, 129, 1, 4, 2, 32),
                                                (1024, 512, 512, 4, 1, 16), (300, 100, 150, 2, 2, 8), (65, 0, 65, 16, 1, 16)])
def test_head_dim_256(kernels, dtype, L, start, n, Hq, Hkv, B):
    """head_dim 256 (what the decode kernel also takes): one query tile per work item, K/V tiles of 64 keys."""
    check_single(kernels, L, start, n, Hq, Hkv, B, dtype, seed=9, poison=(start > 0), D=256)


def test_head_dim_96_is_refused(kernels):
    q = torch.zeros(4, 2, 96, dtype=torch.float16, device=DEV)
    kc = torch.zeros(2, 2, 16, 96, dtype=torch.float16, device=DEV)
    with pytest.raises(RuntimeError, match="head_dim"):
        kernels.paged_prefill_attention(torch.zeros_like(q), q, kc, kc.clone(), torch.zeros(1, 1, dtype=torch.int32, device=DEV),
                                        [0], [4], [0], 1.0, 16, 1)
