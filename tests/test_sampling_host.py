"""Host side of the batched sampler, without a GPU: the library loads, the workspace size is computable and
the module refuses what it cannot serve (there is no CPU path)."""
import pytest
import torch

from nanopd_b200 import _lib, sampling


def test_workspace_size_needs_no_device():
    lib = _lib.load()
    head = lib.npd_top_k_sample_workspace_bytes(0, 151936, 10)
    assert head == 65536                                        # the status word and the arrival counters only
    small = lib.npd_top_k_sample_workspace_bytes(1, 151936, 10)
    large = lib.npd_top_k_sample_workspace_bytes(256, 151936, 64)
    assert head < small <= large
    # one list of k (value, id) pairs per part of a row, at most 1024 / k parts per row
    assert large <= head + 256 * 1024 * 8
    # more rows than one launch serves reuse the same lists
    assert lib.npd_top_k_sample_workspace_bytes(10 ** 6, 151936, 10) == lib.npd_top_k_sample_workspace_bytes(16320, 151936, 10)


def test_cpu_tensors_and_bad_arguments_are_refused():
    logits = torch.randn(4, 1024)
    with pytest.raises(RuntimeError, match="CUDA"):
        sampling.top_k_sample(logits)
    with pytest.raises(RuntimeError, match="CUDA"):
        sampling.top_k_sample(logits[0], top_k=10)


def test_entry_point_validates_before_it_touches_a_device():
    lib = _lib.load()
    # top_k outside [1, 64], an unknown dtype code, a vocabulary smaller than top_k: refused with a message
    for rows, vocab, k, dtype in ((4, 1024, 0, 1), (4, 1024, 65, 1), (4, 1024, 10, 7), (4, 8, 10, 1)):
        rc = lib.npd_top_k_sample(None, None, None, rows, vocab, vocab, k, dtype, None, 0, None)
        assert rc != 0
        assert b"npd_top_k_sample" in lib.npd_last_error()
    assert lib.npd_top_k_sample(None, None, None, 0, 1024, 1024, 1, 1, None, 0, None) == 0     # no rows: nothing to do
