"""GPU: the decode-attention entry point that brings its own scratch memory.

``npd_paged_decode_attention_static`` exists for hosts that cannot allocate device memory at
call time (all HBM already given to the KV pool and weights, a no-allocation step loop, a
foreign runtime without a device allocator).  It must give the same rows as the workspace
variant, and both must agree with the CPU oracle.  The file name sorts last on purpose: a run that stops at the first failure has by
then run every other test.  The test passes alone in a fresh process and after the others —
it calls the entry point twice in a row, the second time on a different batch, so a scratch
array that carried state from one call into the next would show.
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from conftest import TOL
from nanopd_b200 import _lib, workloads
from oracle import paged_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _static_call(lib, out, b, seq_lens, status):
    nb, hkv, bs, d = b.k_cache.shape
    return lib.npd_paged_decode_attention_static(
        out.data_ptr(), b.query.data_ptr(), b.k_cache.data_ptr(), b.v_cache.data_ptr(),
        b.block_tables.data_ptr(), seq_lens.data_ptr(), float(b.scale),
        b.query.size(0), b.num_q_heads, hkv, d, bs, b.block_tables.size(1), nb,
        b.k_cache.stride(0), b.block_tables.stride(0), _lib.NPD_DTYPE_BF16 if b.query.dtype == torch.bfloat16
        else _lib.NPD_DTYPE_F16, status.data_ptr(), 0, torch.cuda.current_stream().cuda_stream)


def _to_device(b):
    for f in ("query", "k_cache", "v_cache", "block_tables", "ctx_lens"):
        setattr(b, f, getattr(b, f).to(DEV))
    return b


def test_static_scratch_entry_point_matches_workspace_entry_point(kernels):
    lib = _lib.load()
    assert lib.npd_decode_static_scratch_bytes() == 32 << 20
    torch.cuda.set_device(0)
    batches = [
        # long sequences on few heads: most (sequence, head) pairs are cut into partials,
        # so the scratch really is used
        _to_device(workloads.make_decode_batch([8191, 3000, 40, 4999], 8, 2, 128, 16, torch.bfloat16, seed=11)),
        _to_device(workloads.make_decode_batch([100, 17, 2047, 1, 700, 333], 12, 2, 128, 16, torch.float16, seed=12)),
    ]
    for b in batches:
        seq_lens = (b.ctx_lens + 1).contiguous()
        want = torch.zeros_like(b.query)
        kernels.paged_attention_forward(want, b.query, b.k_cache, b.v_cache, b.block_tables, seq_lens,
                                        b.scale, b.block_size, b.block_tables.size(1))
        got = torch.full_like(b.query, float("nan"))
        status = torch.full((1,), -1, dtype=torch.int32, device=DEV)
        before = torch.cuda.memory_allocated()
        rc = _static_call(lib, got, b, seq_lens, status)
        assert rc == _lib.NPD_OK, lib.npd_last_error()
        assert torch.cuda.memory_allocated() == before        # nothing taken from torch's allocator either
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.isfinite(got).all()
        # same kernels, same work split: the two entry points agree far inside the oracle tolerance
        assert (got.float() - want.float()).abs().max().item() <= TOL[b.query.dtype]
        # and the entry point's rows are right in their own right: against the fp32 CPU oracle
        oracle = paged_oracle.paged_decode_attention(b.query.cpu(), b.k_cache.cpu(), b.v_cache.cpu(),
                                                     b.block_tables.cpu(), seq_lens.cpu(), b.scale)
        assert (got.float().cpu() - oracle).abs().max().item() <= TOL[b.query.dtype]


def test_static_scratch_rejects_shapes_beyond_its_size():
    lib = _lib.load()
    torch.cuda.set_device(0)
    # zero heads: refused before anything is launched
    rc = lib.npd_paged_decode_attention_static(None, None, None, None, None, None, 1.0, 4, 0, 2, 128, 16, 4, 8,
                                               4096, 4, _lib.NPD_DTYPE_F16, None, 0, None)
    assert rc == _lib.NPD_ERR_INVALID_ARG
    # Every supported shape fits the array on a 148-SM GPU, so the limit is reached through the launcher's grid
    # override (a tuning knob read from the environment once per process, hence the child process): the scratch
    # need then outgrows the array and the call must say so instead of running past the end.  Nothing is launched.
    code = ("import sys; sys.path.insert(0, %r)\n"
            "from nanopd_b200 import _lib\n"
            "lib = _lib.load()\n"
            "rc = lib.npd_paged_decode_attention_static(None, None, None, None, None, None, 1.0, 4, 32, 2, 128, 16, 4, 8,"
            " 4096, 4, _lib.NPD_DTYPE_F16, None, 0, None)\n"
            "print(rc, lib.npd_last_error().decode())\n") % str(Path(__file__).resolve().parents[1])
    res = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, NPD_DECODE_CTAS="512"),
                         capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    rc, message = res.stdout.strip().split(" ", 1)
    assert int(rc) == _lib.NPD_ERR_WORKSPACE and "scratch" in message
