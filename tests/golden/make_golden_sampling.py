"""Generates tests/golden/top_k_sample_cases.npz from the calls the reference's sampler makes
(nanoPD/engine/model_runner.py:279-284): ``torch.nan_to_num``, ``torch.topk`` and ``torch.softmax`` on the
CPU, and the reference's own ``top_k_sample`` (imported from the reference tree) for its default
``top_k = 1``, whose result does not depend on the random generator.  The oracle must reproduce the k
values and the probabilities BIT FOR BIT, the ids wherever the k-th value is not tied, and the
``top_k = 1`` token (checked here and again by tests/test_oracle.py on the committed fixture).
Run:  python tests/golden/make_golden_sampling.py <path to the reference checkout>
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import paged_oracle  # noqa: E402

OUT = Path(__file__).resolve().parent
if len(sys.argv) < 2:
    sys.exit("usage: make_golden_sampling.py <path to the reference checkout>")
REFERENCE = Path(sys.argv[1])


def bits(t):
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.contiguous().view(torch.int16).numpy()
    return t.contiguous().numpy()


# (name, rows, vocabulary, top_k, dtype, scale of the logits)
CASES = [
    ("f32_k10", 6, 5000, 10, torch.float32, 3.0),
    ("bf16_k10", 6, 20000, 10, torch.bfloat16, 3.0),
    ("f16_k10", 6, 20000, 10, torch.float16, 3.0),
    ("bf16_k64", 4, 40000, 64, torch.bfloat16, 2.0),
    ("f32_k1", 8, 3000, 1, torch.float32, 1.0),
    ("f16_k3_specials", 6, 2048, 3, torch.float16, 1.0),
]


def main():
    sys.path.insert(0, str(REFERENCE / "nanoPD"))
    from engine.model_runner import top_k_sample as reference_top_k_sample

    store = {"names": np.array([c[0] for c in CASES]), "torch_version": np.array(torch.__version__)}
    for seed, (name, T, V, k, dtype, spread) in enumerate(CASES):
        torch.manual_seed(300 + seed)
        logits = (spread * torch.randn(T, V)).to(dtype)
        if "specials" in name:
            logits[0, 5] = float("nan")
            logits[1, 17] = float("inf")
            logits[2, 33] = float("-inf")
            logits[3, 100] = float("inf")
            logits[3, 200] = float("inf")           # a tie at the top: the lower id comes first
            logits[4, :] = float("-inf")            # every logit replaced by the same value
            logits[4, 1000] = -20000.0                # a finite logit below the replacement value
        x = torch.nan_to_num(logits, nan=0.0, posinf=1e4, neginf=-1e4)
        vals, ids = torch.topk(x, k)
        probs = torch.softmax(vals, dim=-1)
        greedy = torch.stack([reference_top_k_sample(logits[t]) for t in range(T)])

        o_vals, o_ids, o_probs = paged_oracle.top_k_candidates(logits, k)
        assert torch.equal(o_vals, vals), name
        assert torch.equal(o_probs, probs), name
        untied = torch.ones(T, dtype=torch.bool)
        for t in range(T):
            kth = vals[t, -1]
            untied[t] = (x[t] == kth).sum() == 1 and vals[t].unique().numel() == k
        assert torch.equal(o_ids[untied], ids[untied]), name
        o_greedy = paged_oracle.top_k_sample(logits, 1)
        top_unique = torch.tensor([(x[t] == x[t].max()).sum().item() == 1 for t in range(T)])
        assert torch.equal(o_greedy[top_unique], greedy[top_unique]), name

        store[f"{name}/logits"] = bits(logits)
        store[f"{name}/dtype"] = np.array(str(dtype).replace("torch.", ""))
        store[f"{name}/top_k"] = np.array(k)
        store[f"{name}/values"] = bits(vals)
        store[f"{name}/ids"] = ids.numpy()
        store[f"{name}/probabilities"] = bits(probs)
        store[f"{name}/untied_rows"] = untied.numpy()
        store[f"{name}/reference_top_1"] = greedy.numpy()
        store[f"{name}/top_1_unique"] = top_unique.numpy()
        print(f"{name}: oracle == torch.topk / softmax bit for bit; {int(untied.sum())}/{T} rows untied; "
              f"top-1 == reference on {int(top_unique.sum())}/{T} rows")
    np.savez_compressed(OUT / "top_k_sample_cases.npz", **store)
    print("wrote", OUT / "top_k_sample_cases.npz")


if __name__ == "__main__":
    main()
