"""GPU: paged KV store through the C ABI — bit-exact against the oracle."""
import pytest
import torch

from nanopd_b200 import workloads
from oracle import paged_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run_both(kernels, k_cache, v_cache, k_src, v_src, bt, pos):
    kc_ref, vc_ref = k_cache.clone(), v_cache.clone()
    paged_oracle.kv_store(kc_ref, vc_ref, k_src, v_src, bt, pos)
    kc, vc = k_cache.to(DEV), v_cache.to(DEV)
    kernels.paged_kv_store(kc, vc, k_src.to(DEV), v_src.to(DEV), bt.to(DEV), pos.to(DEV))
    torch.cuda.synchronize()
    assert torch.equal(kc.cpu().view(torch.int16) if kc.element_size() == 2 else kc.cpu(),
                       kc_ref.view(torch.int16) if kc_ref.element_size() == 2 else kc_ref)
    assert torch.equal(vc.cpu().view(torch.int16) if vc.element_size() == 2 else vc.cpu(),
                       vc_ref.view(torch.int16) if vc_ref.element_size() == 2 else vc_ref)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("heads,T,D,B,start", [(4, 16, 128, 16, 0), (2, 8, 128, 16, 8), (2, 1, 128, 16, 0),
                                               (8, 64, 128, 16, 0), (2, 32, 128, 32, 0), (3, 40, 64, 8, 5),
                                               (8, 512, 128, 16, 1000), (1, 7, 256, 16, 3)])
def test_prefill_style_store_is_bit_exact(kernels, dtype, heads, T, D, B, start):
    """One prompt: the table repeated per token, positions start..start+T (model_runner.py:132-150)."""
    torch.manual_seed(0)
    nblk = (start + T + B - 1) // B
    pool = nblk + 5
    k_src, v_src = torch.randn(heads, T, D).to(dtype), torch.randn(heads, T, D).to(dtype)
    k_cache = torch.randn(pool, heads, B, D).to(dtype)       # pre-existing content must survive
    v_cache = torch.randn(pool, heads, B, D).to(dtype)
    table = torch.randperm(pool)[:nblk].to(torch.int32)
    bt = table.unsqueeze(0).expand(T, -1).contiguous()
    pos = torch.arange(start, start + T, dtype=torch.int32)
    _run_both(kernels, k_cache, v_cache, k_src, v_src, bt, pos)


def test_expanded_table_needs_no_copy(kernels):
    """A stride-0 expand of one table row is read in place."""
    torch.manual_seed(1)
    heads, T, D, B = 2, 20, 128, 16
    k_src, v_src = torch.randn(heads, T, D).half(), torch.randn(heads, T, D).half()
    k_cache, v_cache = torch.zeros(4, heads, B, D).half(), torch.zeros(4, heads, B, D).half()
    table = torch.tensor([3, 1], dtype=torch.int32)
    pos = torch.arange(T, dtype=torch.int32)
    kc_ref, vc_ref = k_cache.clone(), v_cache.clone()
    paged_oracle.kv_store(kc_ref, vc_ref, k_src, v_src, table.unsqueeze(0).expand(T, -1), pos)
    kc, vc = k_cache.to(DEV), v_cache.to(DEV)
    kernels.paged_kv_store(kc, vc, k_src.to(DEV), v_src.to(DEV), table.to(DEV).unsqueeze(0).expand(T, -1), pos.to(DEV))
    assert torch.equal(kc.cpu(), kc_ref) and torch.equal(vc.cpu(), vc_ref)


def test_decode_style_store_config1(kernels):
    """Configuration 1: one new token per sequence into its next slot (model_runner.py:188-194)."""
    b = workloads.make_config1(seed=0)
    _run_both(kernels, b.k_cache, b.v_cache, b.k_new, b.v_new, b.block_tables, b.positions)


def test_decode_style_store_config2_shape(kernels):
    b = workloads.make_config2(seed=1, batch=64)
    _run_both(kernels, b.k_cache, b.v_cache, b.k_new, b.v_new, b.block_tables, b.positions)


def test_strided_source_views(kernels):
    """k_src as a non-contiguous [Hkv, T, D] view of a [T, Hkv, D] projection output."""
    torch.manual_seed(2)
    heads, T, D, B = 4, 33, 128, 16
    proj_k, proj_v = torch.randn(T, heads, D).half(), torch.randn(T, heads, D).half()
    k_cache, v_cache = torch.zeros(6, heads, B, D).half(), torch.zeros(6, heads, B, D).half()
    bt = torch.randperm(6)[:3].to(torch.int32).unsqueeze(0).expand(T, -1).contiguous()
    pos = torch.arange(T, dtype=torch.int32)
    kc_ref, vc_ref = k_cache.clone(), v_cache.clone()
    paged_oracle.kv_store(kc_ref, vc_ref, proj_k.transpose(0, 1), proj_v.transpose(0, 1), bt, pos)
    kc, vc = k_cache.to(DEV), v_cache.to(DEV)
    kernels.paged_kv_store(kc, vc, proj_k.to(DEV).transpose(0, 1), proj_v.to(DEV).transpose(0, 1), bt.to(DEV), pos.to(DEV))
    assert torch.equal(kc.cpu(), kc_ref) and torch.equal(vc.cpu(), vc_ref)


def test_layer_slice_of_a_5d_pool(kernels):
    """The production caller passes runner.k_cache[layer_idx] (model_runner.py:147)."""
    torch.manual_seed(3)
    L, pool, heads, B, D, T = 3, 8, 2, 16, 128, 5
    k_pool = torch.zeros(L, pool, heads, B, D, dtype=torch.bfloat16, device=DEV)
    v_pool = torch.zeros_like(k_pool)
    k_src, v_src = torch.randn(heads, T, D).bfloat16(), torch.randn(heads, T, D).bfloat16()
    bt = torch.tensor([[4, 2]], dtype=torch.int32).expand(T, -1).contiguous()
    pos = torch.arange(14, 14 + T, dtype=torch.int32)
    kernels.paged_kv_store(k_pool[1], v_pool[1], k_src.to(DEV), v_src.to(DEV), bt.to(DEV), pos.to(DEV))
    kc_ref, vc_ref = torch.zeros(pool, heads, B, D).bfloat16(), torch.zeros(pool, heads, B, D).bfloat16()
    paged_oracle.kv_store(kc_ref, vc_ref, k_src, v_src, bt, pos)
    assert torch.equal(k_pool[1].cpu(), kc_ref) and torch.equal(v_pool[1].cpu(), vc_ref)
    assert torch.count_nonzero(k_pool[0]) == 0 and torch.count_nonzero(k_pool[2]) == 0


def test_reference_test_call_shape(kernels):
    """The older call shape the reference's own tests use (test_paged_kernels.py:280,311):
    sources [1, Hkv, T, D], a 1-D block table and an int start position."""
    torch.manual_seed(0)
    heads, T, D, B, start = 2, 8, 128, 16, 8
    k_src = torch.randn(1, heads, T, D, dtype=torch.float16, device=DEV)
    v_src = torch.randn(1, heads, T, D, dtype=torch.float16, device=DEV)
    k_cache = torch.zeros(1, heads, B, D, dtype=torch.float16, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    table = torch.arange(1, dtype=torch.int32, device=DEV)
    kernels.paged_kv_store(k_cache, v_cache, k_src, v_src, table, start)
    torch.cuda.synchronize()
    for tok in range(T):
        for h in range(heads):
            assert torch.equal(k_cache[0, h, start + tok], k_src[0, h, tok])
            assert torch.equal(v_cache[0, h, start + tok], v_src[0, h, tok])


def test_bad_block_id_is_skipped_and_flagged(kernels):
    """An id outside the pool never reaches memory: the row is skipped and the status word set."""
    heads, T, D, B = 2, 3, 128, 16
    k_cache = torch.zeros(2, heads, B, D, dtype=torch.float16, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    src = torch.ones(heads, T, D, dtype=torch.float16, device=DEV)
    bt = torch.tensor([[0], [7], [1]], dtype=torch.int32, device=DEV)      # 7 is out of range
    pos = torch.tensor([0, 1, 2], dtype=torch.int32, device=DEV)
    kernels.paged_kv_store(k_cache, v_cache, src, src, bt, pos)
    assert kernels.check_status(raise_on_error=False) == 1
    assert k_cache[0, :, 0].eq(1).all() and k_cache[1, :, 2].eq(1).all()
    assert k_cache.sum().item() == 2 * heads * D
    with pytest.raises(RuntimeError):
        kernels.paged_kv_store(k_cache, v_cache, src, src, bt.long(), pos)


def test_large_store_roundtrip_property(kernels):
    """Full-size property: storing then gathering returns the source (512-token chunk, Qwen3-8B shape)."""
    torch.manual_seed(5)
    heads, T, D, B = 8, 4096, 128, 16
    pool = 600
    k_src = torch.randn(heads, T, D, device=DEV).bfloat16()
    v_src = torch.randn(heads, T, D, device=DEV).bfloat16()
    k_cache = torch.zeros(pool, heads, B, D, dtype=torch.bfloat16, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    table = torch.randperm(pool, device=DEV)[:T // B].to(torch.int32)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    kernels.paged_kv_store(k_cache, v_cache, k_src, v_src, table.unsqueeze(0).expand(T, -1), pos)
    back_k = k_cache[table.long()].permute(1, 0, 2, 3).reshape(heads, T, D)
    back_v = v_cache[table.long()].permute(1, 0, 2, 3).reshape(heads, T, D)
    assert torch.equal(back_k, k_src) and torch.equal(back_v, v_src)


def test_single_token_sources_with_leftover_strides(kernels):
    """The reference's decode branch hands over ``[Hkv, 1, D]`` slices whose size-1 dimension keeps the stride of
    the view it came from (``v`` is a transposed view, ``k`` a fresh tensor, nanoPD/engine/model_runner.py:104-115,
    190-193): torch calls both contiguous, their strides differ, and the store must take them."""
    Hkv, D, B = 4, 128, 16
    torch.manual_seed(3)
    k = torch.randn(1, Hkv, 1, D, device="cuda").half()                                 # strides (.., D, D, 1)
    v = torch.randn(1, 1, Hkv, D, device="cuda").half().transpose(1, 2)                 # strides (.., D, Hkv*D, 1)
    k_src, v_src = k.squeeze(0).contiguous(), v.squeeze(0).contiguous()
    assert k_src.stride() != v_src.stride() and k_src.is_contiguous() and v_src.is_contiguous()
    kc = torch.zeros(3, Hkv, B, D, dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    table = torch.tensor([[2, 0, 1]], dtype=torch.int32, device="cuda")
    pos = torch.tensor([21], dtype=torch.int32, device="cuda")
    kernels.paged_kv_store(kc, vc, k_src, v_src, table, pos)
    torch.cuda.synchronize()
    assert torch.equal(kc[0, :, 5], k_src[:, 0]) and torch.equal(vc[0, :, 5], v_src[:, 0])
    assert int(torch.count_nonzero(kc)) == int(torch.count_nonzero(k_src))
