"""Top-level alias so that ``import paged_kernels`` — the module name the reference's
``ModelRunner.paged_forward`` imports (nanoPD/engine/model_runner.py:94,270) — resolves to
this repository's implementation when the repository root is on ``sys.path``."""
from nanopd_b200.paged_kernels import (  # noqa: F401
    check_status,
    enable_peer_access,
    paged_attention_forward,
    paged_kv_migrate,
    paged_kv_store,
    paged_prefill_attention,
    paged_qk_norm_rope_store,
)
