"""Top-level alias for the module name the reference's older kernel tests import
(``import paged_attn`` in nanoPD/paged_attention/tests/test_paged_attention.py:18 and the benchmark beside it,
whose ``paged_attn.paged_attention_forward(out, q, key_cache, value_cache, block_tables, seq_lens, scale,
block_size, max_blocks_per_seq)`` is the call ``paged_kernels`` later kept): the same implementation."""
from nanopd_b200.paged_kernels import check_status, paged_attention_forward  # noqa: F401
