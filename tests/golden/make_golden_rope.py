"""Generates tests/golden/qk_norm_rope_cases.npz with the Hugging Face transformers functions the
reference calls in front of the KV store (nanoPD/engine/model_runner.py:97-115): ``Qwen3RMSNorm``,
``Qwen3RotaryEmbedding`` and ``apply_rotary_pos_emb`` of transformers' Qwen3 model, evaluated on the
CPU in fp16 and bf16.  The oracle must reproduce them BIT FOR BIT (checked here and again by
tests/test_oracle.py on the committed fixture).  Run:  python tests/golden/make_golden_rope.py
"""
import sys
from pathlib import Path

import numpy as np
import torch
import transformers
from transformers.models.qwen3 import modeling_qwen3 as hf
from transformers.models.qwen3.configuration_qwen3 import Qwen3Config

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import paged_oracle  # noqa: E402

OUT = Path(__file__).resolve().parent


def bits(t):
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.contiguous().view(torch.int16).numpy()
    return t.contiguous().numpy()


# (name, T, Hq, Hkv, D, dtype, with_norm)
CASES = [
    ("qwen3_bf16", 7, 8, 2, 128, torch.bfloat16, True),
    ("qwen3_f16", 5, 4, 4, 128, torch.float16, True),
    ("qwen2_f16_no_norm", 6, 12, 2, 128, torch.float16, False),
    ("d64_bf16", 4, 4, 2, 64, torch.bfloat16, True),
]


def main():
    store = {"names": np.array([c[0] for c in CASES]), "transformers_version": np.array(transformers.__version__)}
    for seed, (name, T, Hq, Hkv, D, dtype, with_norm) in enumerate(CASES):
        torch.manual_seed(100 + seed)
        cfg = Qwen3Config(hidden_size=Hq * D, num_attention_heads=Hq, num_key_value_heads=Hkv, head_dim=D,
                          rope_theta=1e6, max_position_embeddings=4096)
        rope = hf.Qwen3RotaryEmbedding(cfg)
        positions = torch.randint(0, 3000, (T,))
        q = torch.randn(1, T, Hq, D).to(dtype)
        k = torch.randn(1, T, Hkv, D).to(dtype)
        cos, sin = rope(q, positions.unsqueeze(0))                    # [1, T, D] in q's dtype
        qn, kn = q, k
        qw = kw = None
        if with_norm:
            qnorm, knorm = hf.Qwen3RMSNorm(D, eps=1e-6).to(dtype), hf.Qwen3RMSNorm(D, eps=1e-6).to(dtype)
            with torch.no_grad():
                qnorm.weight.copy_((1 + 0.1 * torch.randn(D)).to(dtype))
                knorm.weight.copy_((1 + 0.1 * torch.randn(D)).to(dtype))
                qn, kn = qnorm(q), knorm(k)
            qw, kw = qnorm.weight.detach(), knorm.weight.detach()
        # the reference's order: norm on [1, T, H, D], transpose to [1, H, T, D], rotary with unsqueeze_dim=1
        q_hf, k_hf = hf.apply_rotary_pos_emb(qn.transpose(1, 2), kn.transpose(1, 2), cos, sin)
        q_ref = q_hf.transpose(1, 2)[0].contiguous()                   # [T, Hq, D]
        k_ref = k_hf.transpose(1, 2)[0].contiguous()

        # the oracle on the same inputs
        q_o = q[0]
        k_o = k[0]
        if with_norm:
            q_o = paged_oracle.rms_norm_heads(q_o, qw, 1e-6)
            k_o = paged_oracle.rms_norm_heads(k_o, kw, 1e-6)
        q_o = paged_oracle.rotary(q_o, cos[0], sin[0])
        k_o = paged_oracle.rotary(k_o, cos[0], sin[0])
        assert torch.equal(q_o, q_ref) and torch.equal(k_o, k_ref), f"{name}: oracle differs from transformers"

        store[f"{name}/is_bf16"] = np.array(dtype == torch.bfloat16)
        store[f"{name}/with_norm"] = np.array(with_norm)
        store[f"{name}/q"] = bits(q[0])
        store[f"{name}/k"] = bits(k[0])
        store[f"{name}/cos"] = bits(cos[0])
        store[f"{name}/sin"] = bits(sin[0])
        store[f"{name}/positions"] = positions.to(torch.int32).numpy()
        if with_norm:
            store[f"{name}/q_norm_weight"] = bits(qw)
            store[f"{name}/k_norm_weight"] = bits(kw)
        store[f"{name}/q_ref"] = bits(q_ref)
        store[f"{name}/k_ref"] = bits(k_ref)
        print(f"{name}: oracle == transformers {transformers.__version__} bit for bit")
    np.savez_compressed(OUT / "qk_norm_rope_cases.npz", **store)
    print("wrote", OUT / "qk_norm_rope_cases.npz")


if __name__ == "__main__":
    main()
