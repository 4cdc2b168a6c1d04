"""GPU: the reference's OWN code run against this repository's ``paged_kernels`` module.

Needs a checkout of the reference, its path in NANOPD_REFERENCE (the variable the fixture generators under
tests/golden/ use); skipped where there is none.  Nothing of the reference is copied here: its files are run
where they lie.

1. ``nanoPD/paged_attention/tests/test_paged_kernels.py`` — the reference's kernel tests (5-D K / transposed-V
   caches, the older ``paged_kv_store`` call shape, int64 tables must raise) — and ``test_paged_attention.py``
   beside it (the older module name ``paged_attn``; block sizes 4 to 32) run unchanged in a child pytest with
   this repository's root first on the module path, so ``import paged_kernels`` / ``import paged_attn`` find this
   implementation.
2. ``ModelRunner`` 's monkey-patch (``_patch_attention_layers`` / ``paged_forward``,
   nanoPD/engine/model_runner.py:48-213) applied to a small random-init Qwen3 model built from a config (the
   constructor's tokenizer and checkpoint download, :8-13, is the only part bypassed): one whole-prompt prefill and
   several decode steps must give the logits of the same weights run by Hugging Face's own attention with its own
   KV cache.
3. The reference's workers (``PrefillWorker.prefill_batch_and_extract``, ``DecodeWorker.receive_kv_async`` and
   ``step``) with this repository's ``kv_transfer`` under the module name they import: prefill of two prompts in one
   forward, extract, hand-over, six decode steps; the tokens equal Hugging Face's greedy generation."""
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


@pytest.mark.parametrize("name", ["test_paged_kernels.py", "test_paged_attention.py"])
def test_reference_kernel_tests_pass_unchanged(tmp_path, name):
    test_file = Path(REF) / "nanoPD" / "paged_attention" / "tests" / name
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


def test_reference_workers_hand_over_through_this_kv_transfer(monkeypatch):
    """The reference's own ``PrefillWorker.prefill_batch_and_extract`` and ``DecodeWorker.receive_kv_async`` /
    ``step`` (nanoPD/workers/prefill_worker.py:92-112, decode_worker.py:39-126), run where they lie, with this
    repository's ``kv_transfer`` under the module name they import and its ``paged_kernels`` behind their runners:
    two prompts are prefilled in one forward, extracted, handed over and decoded for several steps.  Sampling is
    made greedy in both workers so that the tokens can be compared with Hugging Face's own generation."""
    import types
    device = "cuda:0"
    block_size, max_blocks = 16, 64
    sys.path.insert(0, str(Path(REF) / "nanoPD"))
    if str(ROOT) not in sys.path:
        sys.path.insert(0, str(ROOT))
    import nanopd_b200.kv_transfer as ours
    monkeypatch.setitem(sys.modules, "workers.kv_transfer", ours)          # what `from workers.kv_transfer import` finds
    from block_manager.block_manager import BlockSpaceManager
    from block_manager.sequence import Sequence, SequenceGroup
    import workers.prefill_worker as ref_prefill
    import workers.decode_worker as ref_decode
    assert ref_prefill.extract_kv_to_pinned is ours.extract_kv_to_pinned and ref_decode.transfer_kv is ours.transfer_kv
    greedy = lambda logit, top_k=10: logit.argmax()
    monkeypatch.setattr(ref_prefill, "top_k_sample", greedy)
    monkeypatch.setattr(ref_decode, "top_k_sample", greedy)

    hf_model = _small_qwen3(device, torch.float16)
    bm = BlockSpaceManager(block_size=block_size, num_gpu_blocks=max_blocks)      # one manager for both workers, as there
    pre = ref_prefill.PrefillWorker.__new__(ref_prefill.PrefillWorker)
    pre.device, pre.block_manager, pre.block_size, pre._busy = device, bm, block_size, False
    pre.runner = _patched_runner(copy.deepcopy(hf_model), device, max_blocks, block_size)
    dec = ref_decode.DecodeWorker.__new__(ref_decode.DecodeWorker)
    dec.device, dec.block_manager, dec.block_size = device, bm, block_size
    dec.runner = _patched_runner(copy.deepcopy(hf_model), device, max_blocks, block_size)
    dec.runner.tokenizer = types.SimpleNamespace(eos_token_id=-1)
    dec.running, dec.finished, dec._pending = [], [], []
    dec.compute_stream = torch.cuda.Stream(device=device)
    dec.transfer_stream = torch.cuda.Stream(device=device)

    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (45, 70)]
    groups = [SequenceGroup(str(i), [Sequence(i, p, block_size)]) for i, p in enumerate(prompts)]
    steps = 6
    with torch.inference_mode():
        results = pre.prefill_batch_and_extract(groups)
        for group, (first_token, block_table, buf, src_k, src_v) in zip(groups, results):
            # the extract: the pinned buffer holds the request's blocks, layer by layer
            for i, blk in enumerate(block_table):
                assert torch.equal(buf.k[:, i], src_k[:, blk].cpu()) and torch.equal(buf.v[:, i], src_v[:, blk].cpu())
            path = dec.receive_kv_async(group, block_table, buf, src_k=src_k, src_v=src_v)
            assert path in ("p2p", "pinned_relay")
        torch.cuda.synchronize(device)
        for group, (_, block_table, _, src_k, src_v) in zip(groups, results):
            idx = torch.tensor(block_table, device=device)
            assert torch.equal(dec.runner.k_cache[:, idx], src_k[:, idx]) and torch.equal(dec.runner.v_cache[:, idx], src_v[:, idx])
        produced = {0: [results[0][0]], 1: [results[1][0]]}
        for _ in range(steps):
            for group, tok in dec.step():
                produced[int(group.request_id)].append(tok)
        # Hugging Face's own greedy generation from the same weights
        for i, prompt in enumerate(prompts):
            ids = torch.tensor([prompt], device=device)
            ref = hf_model(ids, use_cache=True)
            past, want = ref.past_key_values, [int(ref.logits[0, -1].argmax())]
            for _ in range(steps):
                ref = hf_model(torch.tensor([[want[-1]]], device=device), past_key_values=past, use_cache=True)
                past = ref.past_key_values
                want.append(int(ref.logits[0, 0].argmax()))
            assert produced[i] == want, (i, produced[i], want)
    import paged_kernels
    assert paged_kernels.check_status(device, raise_on_error=False) == 0
