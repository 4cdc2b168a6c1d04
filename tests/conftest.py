"""Shared fixtures.  Tests marked ``gpu`` need a B200 and call the CUDA path through the
C ABI; everything else runs on the CPU (oracle vs. golden vectors, host logic, symbol export)."""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"

# max-abs tolerances against the fp32-accumulated oracle
TOL = {torch.float16: 2e-3, torch.bfloat16: 1e-2}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def _from_bits(a: np.ndarray, bf16: bool) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(a))
    if t.dtype == torch.int16:
        return t.view(torch.bfloat16 if bf16 else torch.float16)
    return t


def load_decode_cases():
    """The reference-generated decode cases of tests/golden/decode_reference_cases.npz."""
    z = np.load(GOLDEN / "decode_reference_cases.npz")
    cases = []
    for name in z["names"].tolist():
        bf16 = bool(z[f"{name}/is_bf16"])
        cases.append(dict(
            name=name,
            dtype=torch.bfloat16 if bf16 else torch.float16,
            q=_from_bits(z[f"{name}/q"], bf16), k=_from_bits(z[f"{name}/k"], bf16),
            v=_from_bits(z[f"{name}/v"], bf16),
            block_tables=torch.from_numpy(z[f"{name}/block_tables"]),
            seq_lens=torch.from_numpy(z[f"{name}/seq_lens"]),
            scale=float(z[f"{name}/scale"]),
            ref_out=_from_bits(z[f"{name}/ref_out"], bf16),
            out_fp32=torch.from_numpy(z[f"{name}/out_fp32"])))
    return cases


def load_rope_cases():
    """The transformers-generated norm + rotary cases of tests/golden/qk_norm_rope_cases.npz."""
    z = np.load(GOLDEN / "qk_norm_rope_cases.npz")
    cases = []
    for name in z["names"].tolist():
        bf16 = bool(z[f"{name}/is_bf16"])
        with_norm = bool(z[f"{name}/with_norm"])
        c = dict(name=name, dtype=torch.bfloat16 if bf16 else torch.float16, with_norm=with_norm,
                 positions=torch.from_numpy(z[f"{name}/positions"]))
        for key in ("q", "k", "cos", "sin", "q_ref", "k_ref"):
            c[key] = _from_bits(z[f"{name}/{key}"], bf16)
        for key in ("q_norm_weight", "k_norm_weight"):
            c[key] = _from_bits(z[f"{name}/{key}"], bf16) if with_norm else None
        cases.append(c)
    return cases


def load_sampling_cases():
    """The torch.topk / softmax / reference top-1 cases of tests/golden/top_k_sample_cases.npz."""
    z = np.load(GOLDEN / "top_k_sample_cases.npz")
    dtypes = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}
    cases = []
    for name in z["names"].tolist():
        dtype = dtypes[str(z[f"{name}/dtype"])]

        def tensor(key):
            a = z[f"{name}/{key}"]
            return torch.from_numpy(a.copy()) if dtype == torch.float32 else torch.from_numpy(a.copy()).view(dtype)

        cases.append(dict(name=name, dtype=dtype, top_k=int(z[f"{name}/top_k"]), logits=tensor("logits"),
                          values=tensor("values"), probabilities=tensor("probabilities"),
                          ids=torch.from_numpy(z[f"{name}/ids"]),
                          untied_rows=torch.from_numpy(z[f"{name}/untied_rows"]),
                          reference_top_1=torch.from_numpy(z[f"{name}/reference_top_1"]),
                          top_1_unique=torch.from_numpy(z[f"{name}/top_1_unique"])))
    return cases


@pytest.fixture(autouse=True)
def _first_gpu_is_current():
    """Every test starts with device 0 current, whatever an earlier test on a box with several GPUs left behind
    (a worker of tests/test_gpu_threads.py binds its thread — the main thread, in the serial half — to its GPU)."""
    if torch.cuda.is_available():
        torch.cuda.set_device(0)
    yield


@pytest.fixture(scope="session")
def decode_cases():
    return load_decode_cases()


@pytest.fixture()
def kernels():
    """The drop-in module; importing it loads the CUDA library (no fallback)."""
    import paged_kernels
    yield paged_kernels
    if torch.cuda.is_available():
        # every GPU test must leave the device-side status word clean
        assert paged_kernels.check_status(raise_on_error=False) == 0
