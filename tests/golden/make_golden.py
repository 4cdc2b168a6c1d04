"""Generates tests/golden/*.npz by running the REFERENCE's own CPU path.

Run where the reference checkout is at hand, its path in NANOPD_REFERENCE:
    NANOPD_REFERENCE=<checkout> python tests/golden/make_golden.py

It imports ``ref_paged_attention`` and the input builder ``make_attn_inputs`` from
nanoPD/paged_attention/tests/test_paged_kernels.py (the module imports without the CUDA
extension and accepts device="cpu"), evaluates them on small seeded cases, checks that
``oracle/paged_oracle.py`` reproduces the reference BIT FOR BIT on each, and stores inputs
and outputs.  The committed fixtures let the same check run where the reference tree is
absent (the GPU box, CI).  16-bit tensors are stored as their int16 bit patterns.
"""
import importlib.util
import os
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import paged_oracle  # noqa: E402
from nanopd_b200 import workloads  # noqa: E402

if "NANOPD_REFERENCE" not in os.environ:
    sys.exit("set NANOPD_REFERENCE to the reference checkout")
REF = Path(os.environ["NANOPD_REFERENCE"])
OUT = Path(__file__).resolve().parent


def load_reference_tests():
    path = REF / "nanoPD" / "paged_attention" / "tests" / "test_paged_kernels.py"
    spec = importlib.util.spec_from_file_location("ref_test_paged_kernels", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.contiguous().view(torch.int16).numpy()
    return t.contiguous().numpy()


# (name, num_seqs, Hq, Hkv, D, seq_lens, block_size, dtype) — the reference's case list
# (test_paged_kernels.py:160-209) at fixture-friendly sizes, plus ragged/GQA mixes.
CASES = [
    ("single_f16", 1, 1, 1, 128, [8], 16, torch.float16),
    ("single_bf16", 1, 1, 1, 128, [8], 16, torch.bfloat16),
    ("multi_f16", 3, 4, 4, 128, [32, 48, 64], 16, torch.float16),
    ("multi_bf16", 3, 4, 4, 128, [32, 48, 64], 16, torch.bfloat16),
    ("gqa32_8_f16", 2, 32, 8, 128, [20, 9], 16, torch.float16),
    ("gqa12_2_bf16", 3, 12, 2, 128, [70, 1, 33], 16, torch.bfloat16),
    ("lens_f16", 6, 2, 1, 128, [1, 15, 16, 17, 32, 64], 16, torch.float16),
    ("len512_f16", 1, 2, 1, 128, [512], 16, torch.float16),
    ("block32_f16", 2, 4, 4, 128, [48, 32], 32, torch.float16),
    ("block8_d64_f16", 2, 4, 2, 64, [9, 24], 8, torch.float16),
    # the smallest block of the older test file beside it (test_paged_attention.py:192-203)
    ("block4_d64_f16", 2, 4, 4, 64, [24, 16], 4, torch.float16),
    ("block4_gqa_bf16", 2, 8, 2, 128, [7, 41], 4, torch.bfloat16),
]


def main():
    ref = load_reference_tests()
    arrays = {}
    names = []
    for name, S, hq, hkv, D, lens, B, dtype in CASES:
        q, k_std, v_std, _k5, _vt, bt, sl, scale, max_blocks = ref.make_attn_inputs(
            S, hq, hkv, D, lens, B, dtype, device="cpu", seed=42)
        want = ref.ref_paged_attention(q, k_std, v_std, bt, sl, scale)          # dtype-rounded
        got32 = paged_oracle.paged_decode_attention(q, k_std, v_std, bt, sl, scale)
        assert torch.equal(got32.to(dtype), want), f"oracle != reference on {name}"
        names.append(name)
        arrays[f"{name}/q"] = bits(q)
        arrays[f"{name}/k"] = bits(k_std)
        arrays[f"{name}/v"] = bits(v_std)
        arrays[f"{name}/block_tables"] = bt.numpy()
        arrays[f"{name}/seq_lens"] = sl.numpy()
        arrays[f"{name}/scale"] = np.float32(scale)
        arrays[f"{name}/is_bf16"] = np.bool_(dtype == torch.bfloat16)
        arrays[f"{name}/ref_out"] = bits(want)          # the reference's return value
        arrays[f"{name}/out_fp32"] = got32.numpy()      # its fp32 value before the final cast
        print(f"{name}: reference == oracle (bit-exact), out {tuple(want.shape)}")
    arrays["names"] = np.array(names)
    np.savez_compressed(OUT / "decode_reference_cases.npz", **arrays)

    # Configuration 1 (Qwen2-1.5B shape, 8 sequences, fp16): inputs are regenerated from the
    # seed by nanopd_b200.workloads; only the reference's output is stored.
    b = workloads.make_config1(device="cpu", seed=0)
    paged_oracle.kv_store(b.k_cache, b.v_cache, b.k_new, b.v_new, b.block_tables, b.positions)
    sl = b.seq_lens_after_store
    want = ref.ref_paged_attention(b.query, b.k_cache, b.v_cache, b.block_tables, sl, b.scale)
    got32 = paged_oracle.paged_decode_attention(b.query, b.k_cache, b.v_cache, b.block_tables, sl, b.scale)
    assert torch.equal(got32.to(b.query.dtype), want), "oracle != reference on configuration 1"
    np.savez_compressed(OUT / "config1_reference_out.npz", ref_out=bits(want), out_fp32=got32.numpy(),
                        ctx_lens=b.ctx_lens.numpy(), block_tables=b.block_tables.numpy())
    print("config1: reference == oracle (bit-exact)")


if __name__ == "__main__":
    main()
