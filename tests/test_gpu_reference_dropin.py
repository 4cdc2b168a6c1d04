"""GPU: the reference's OWN code run against this repository's ``paged_kernels`` module.

Needs a checkout of the reference, its path in NANOPD_REFERENCE (the variable the fixture generators under
tests/golden/ use); skipped where there is none.  Nothing of the reference is copied here: its files are run
where they lie.

1. ``nanoPD/paged_attention/tests/test_paged_kernels.py`` — the reference's kernel tests (5-D K / transposed-V
   caches, the older ``paged_kv_store`` call shape, int64 tables must raise) — run unchanged in a child pytest with
   this repository's root first on the module path, so ``import paged_kernels`` finds this implementation.
2. ``ModelRunner`` 's monkey-patch (``_patch_attention_layers`` / ``paged_forward``,
   nanoPD/engine/model_runner.py:48-213) applied to a small random-init Qwen3 model built from a config (the
   constructor's tokenizer and checkpoint download, :8-13, is the only part bypassed): one whole-prompt prefill and
   several decode steps must give the logits of the same weights run by Hugging Face's own attention with its own
   KV cache."""
import copy
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
REF = os.environ.get("NANOPD_REFERENCE")
pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not REF or not (Path(REF) / "nanoPD").is_dir(),
                                 reason="set NANOPD_REFERENCE to a checkout of the reference")]


def test_reference_kernel_tests_pass_unchanged(tmp_path):
    test_file = Path(REF) / "nanoPD" / "paged_attention" / "tests" / "test_paged_kernels.py"
    env = dict(os.environ, PYTHONPATH=str(ROOT) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    res = subprocess.run([sys.executable, "-m", "pytest", str(test_file), "-q", "-p", "no:cacheprovider",
                          "--rootdir", str(tmp_path), "-c", os.devnull],
                         cwd=tmp_path, env=env, capture_output=True, text=True, timeout=900)
    tail = res.stdout[-3000:] + res.stderr[-2000:]
    assert res.returncode == 0, tail
    summary = [ln for ln in res.stdout.splitlines() if " passed" in ln]
    assert summary and "skipped" not in summary[-1] and "failed" not in summary[-1], tail
    print(summary[-1])


def _small_qwen3(device, dtype):
    from transformers import Qwen3Config, Qwen3ForCausalLM
    cfg = Qwen3Config(vocab_size=1024, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=512,
                      rope_theta=1e6, tie_word_embeddings=False)
    torch.manual_seed(0)
    model = Qwen3ForCausalLM(cfg).to(device=device, dtype=dtype)
    model.eval()
    return model


def _patched_runner(model, device, max_blocks, block_size):
    """A ``ModelRunner`` with everything its constructor sets after loading the checkpoint
    (nanoPD/engine/model_runner.py:14-47), around ``model``."""
    sys.path.insert(0, str(Path(REF) / "nanoPD"))
    if str(ROOT) not in sys.path:
        sys.path.insert(0, str(ROOT))
    from engine.model_runner import ModelRunner
    cfg = model.config
    runner = ModelRunner.__new__(ModelRunner)
    runner.device = device
    runner.tokenizer = None
    runner.model = model
    runner.num_heads = cfg.num_attention_heads
    runner.num_kv_heads = cfg.num_key_value_heads
    runner.head_dim = cfg.head_dim
    runner.block_size = block_size
    runner.k_cache = torch.zeros(cfg.num_hidden_layers, max_blocks, runner.num_kv_heads, block_size, runner.head_dim,
                                 dtype=torch.float16, device=device)
    runner.v_cache = torch.zeros_like(runner.k_cache)
    runner._current_context = None
    runner._patch_attention_layers()
    return runner


def test_reference_paged_forward_matches_hugging_face_cache():
    device = "cuda:0"
    block_size, max_blocks = 16, 32
    hf_model = _small_qwen3(device, torch.float16)
    runner = _patched_runner(copy.deepcopy(hf_model), device, max_blocks, block_size)
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, 1024, (1, 45), generator=g).to(device)
    block_table = [29, 3, 17, 8, 30]                      # room for 80 tokens, ids out of order

    with torch.inference_mode():
        # prefill: the reference's own entry point for a whole prompt (model_runner.py:217-240)
        runner._current_context = {"num_prefill_tokens": 45, "num_decode_tokens": 0, "decodes": [],
                                   "prefills": [{"block_table": block_table, "start_position": 0, "num_tokens": 45}]}
        pos = torch.arange(45, device=device).unsqueeze(0)
        got = runner.model(prompt, position_ids=pos, use_cache=False).logits[0, -1].float()
        ref = hf_model(prompt, position_ids=pos, use_cache=True)
        past = ref.past_key_values
        want = ref.logits[0, -1].float()
        scale = want.abs().max().item()
        assert (got - want).abs().max().item() <= 2e-2 * scale, "prefill logits"
        token = want.argmax().view(1, 1)
        for step in range(12):                             # crosses the block boundary at position 48
            position = 45 + step
            runner._current_context = {"num_prefill_tokens": 0, "num_decode_tokens": 1, "prefills": [],
                                       "decodes": [{"block_table": block_table, "position": position}]}
            pos = torch.tensor([[position]], device=device)
            got = runner.model(token, position_ids=pos, use_cache=False).logits[0, 0].float()
            ref = hf_model(token, position_ids=pos, past_key_values=past, use_cache=True)
            past = ref.past_key_values
            want = ref.logits[0, 0].float()
            err = (got - want).abs().max().item()
            assert err <= 2e-2 * want.abs().max().item(), f"decode step {step}: max-abs logit error {err}"
            assert int(got.argmax()) == int(want.argmax())
            token = want.argmax().view(1, 1)
    import paged_kernels
    assert paged_kernels.check_status(device, raise_on_error=False) == 0
