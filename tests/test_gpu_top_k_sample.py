"""Batched top-k sampling against the oracle (oracle/paged_oracle.py: top_k_candidates, top_k_sample — the
restatement of nanoPD/engine/model_runner.py:279-284).  The candidates and their order are checked exactly:
a uniform number in the middle of a candidate's CDF interval must return exactly that candidate.  Random
uniform numbers are checked with a tolerance of one rounding step of the probabilities at the interval's ends
(the kernel's exp and the oracle's may differ by an ulp before the rounding to the logits' dtype)."""
import numpy as np
import pytest
import torch

from conftest import load_sampling_cases
from oracle import paged_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def sampling():
    from nanopd_b200 import sampling as module
    return module


def cdf_of(probs):
    c = np.cumsum(probs.float().numpy(), axis=-1, dtype=np.float32)
    return c, c[:, -1]


def check_every_candidate(sampling, logits, top_k, rows=None):
    """Draws at the midpoint of every candidate's interval and expects exactly the oracle's candidate."""
    _, ids, probs = paged_oracle.top_k_candidates(logits, top_k)
    c, total = cdf_of(probs)
    T = logits.size(0)
    dev_logits = logits.to(DEV)
    ulp = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11, torch.float32: 1e-6}[logits.dtype]
    checked = 0
    for j in range(top_k):
        lo = c[:, j - 1] if j else np.zeros(T, np.float32)
        wide = (c[:, j] - lo) / total > 3 * ulp              # the midpoint is further from both ends than any rounding
        u = torch.from_numpy(((lo + c[:, j]) / 2 / total).astype(np.float32)).clamp_(0, 0.99999)
        got = sampling.top_k_sample(dev_logits, top_k, uniforms=u.to(DEV)).cpu()
        sel = torch.from_numpy(wide)
        if rows is not None:
            sel &= rows
        assert torch.equal(got[sel], ids[:, j][sel]), f"candidate {j}"
        checked += int(sel.sum())
    return checked


def check_draws(sampling, logits, top_k, uniforms):
    _, ids, probs = paged_oracle.top_k_candidates(logits, top_k)
    c, total = cdf_of(probs)
    got = sampling.top_k_sample(logits.to(DEV), top_k, uniforms=uniforms.to(DEV)).cpu()
    want = paged_oracle.top_k_sample(logits, top_k, uniforms)
    step = 2.0 ** -7 if logits.dtype != torch.float32 else 1e-5
    exact = 0
    for t in range(logits.size(0)):
        if got[t] == want[t]:
            exact += 1
            continue
        where = (ids[t] == got[t]).nonzero()
        assert where.numel() == 1, f"row {t}: token {int(got[t])} is not one of the k candidates"
        j = int(where[0])
        target = np.float32(uniforms[t].item()) * total[t]
        lo = c[t, j - 1] if j else np.float32(0)
        assert lo - step * total[t] <= target <= c[t, j] + step * total[t], f"row {t}: candidate {j} for u={uniforms[t]}"
    return exact


@pytest.mark.parametrize("case", load_sampling_cases(), ids=lambda c: c["name"])
def test_golden_cases(sampling, case):
    logits, k = case["logits"], case["top_k"]
    assert check_every_candidate(sampling, logits, k) > 0
    got = sampling.top_k_sample(logits.to(DEV)).cpu()                       # the reference's default: top_k = 1
    sel = case["top_1_unique"]
    assert torch.equal(got[sel], case["reference_top_1"][sel])
    assert torch.equal(got, paged_oracle.top_k_sample(logits, 1))


@pytest.mark.parametrize("dtype,rows", [(torch.bfloat16, 48), (torch.float16, 16), (torch.float32, 16)])
def test_qwen3_vocabulary(sampling, dtype, rows):
    torch.manual_seed(5)
    V = 151936
    logits = (2.5 * torch.randn(rows, V)).to(dtype)
    u = torch.rand(rows)
    exact = check_draws(sampling, logits, 10, u)
    assert exact >= rows - 2
    assert torch.equal(sampling.top_k_sample(logits.to(DEV)).cpu(), paged_oracle.top_k_sample(logits, 1))
    assert check_every_candidate(sampling, logits[:8], 10) > 20


def test_top_k_64(sampling):
    torch.manual_seed(6)
    logits = torch.randn(12, 70000).to(torch.bfloat16)
    assert check_every_candidate(sampling, logits, 64) > 100
    check_draws(sampling, logits, 64, torch.rand(12))


def test_special_values_and_ties(sampling):
    """NaN → 0, ±inf → ±1e4 in the logits' dtype; equal values by the lower id; rows that defeat the bound
    (all logits equal, or a handful of distinct values) take the arg-max rounds."""
    torch.manual_seed(7)
    for dtype in (torch.float16, torch.bfloat16, torch.float32):
        V = 40000
        logits = torch.randn(10, V).to(dtype)
        logits[0, 39999] = float("nan")
        logits[0, :39999] = -1.0                                         # the NaN, read as 0, wins
        logits[1, 123] = float("inf")
        logits[1, 20000] = float("inf")                                  # tie at the top
        logits[2, :] = float("-inf")
        logits[2, 777] = -20000.0                                        # below the replaced -inf: never drawn
        logits[3, :] = 0.5                                               # every logit equal: ids 0..k-1
        logits[4] = torch.randint(-3, 4, (V,)).to(dtype)                 # seven distinct values
        logits[5, :] = float("nan")
        logits[6, 16384:] = 9.0                                          # a run of equal values over two slices
        logits[7, 5] = 10048.0                                           # a finite logit above the replacement
        logits[7, 9] = float("inf")
        _, ids, _ = paged_oracle.top_k_candidates(logits, 5)
        assert ids[0, 0] == 39999 and ids[1].tolist()[:2] == [123, 20000] and ids[3].tolist() == [0, 1, 2, 3, 4]
        assert ids[2, 0] == 0 and 777 not in ids[2].tolist() and ids[7, 0] == 5
        assert check_every_candidate(sampling, logits, 5) >= 30
        assert torch.equal(sampling.top_k_sample(logits.to(DEV)).cpu(), ids[:, 0])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_scattered_ties_at_the_top_go_to_the_lowest_id(sampling, dtype):
    """The largest value several times in a row, far apart: whichever CTA, warp or slice meets which copy first,
    top_k = 1 returns the lowest id and top_k = 4 the four lowest, in order."""
    torch.manual_seed(12)
    V, rows = 151936, 24
    logits = torch.randn(rows, V).to(dtype)
    want = []
    for r in range(rows):
        ids = torch.randperm(V)[:6].sort().values
        logits[r, ids] = 30.0
        logits[r, ids[2]] = -0.0 if r % 5 == 0 else 30.0          # a zero of either sign is no tie-breaker
        want.append(ids.tolist())
    zero_row = torch.full((V,), -1.0).to(dtype)
    zero_row[[140000, 17, 90000]] = torch.tensor([0.0, -0.0, 0.0]).to(dtype)
    logits[0] = zero_row
    dev_logits = logits.to(DEV)
    got = sampling.top_k_sample(dev_logits).cpu()
    _, ids, _ = paged_oracle.top_k_candidates(logits, 4)
    assert torch.equal(got, ids[:, 0])
    assert got[0] == 17 and all(int(got[r]) == want[r][0] for r in range(1, rows))
    u = torch.full((rows,), 0.999)
    assert torch.equal(sampling.top_k_sample(dev_logits, 4, uniforms=u.to(DEV)).cpu(), paged_oracle.top_k_sample(logits, 4, u))


@pytest.mark.parametrize("vocab", [5, 64, 1000, 16384, 16392, 32768 + 24, 49160])
def test_ragged_vocabularies(sampling, vocab):
    torch.manual_seed(vocab)
    k = min(5, vocab)
    logits = torch.randn(6, vocab + 8 - vocab % 8 if vocab % 8 else vocab).to(torch.float16)[:, :vocab]
    wide = logits.clone()                                                  # rows of the oracle's view
    dev = torch.full((6, logits.stride(0)), float("inf"), dtype=torch.float16, device=DEV)   # padding must not be read
    dev[:, :vocab] = logits.to(DEV)
    view = dev[:, :vocab]
    _, ids, probs = paged_oracle.top_k_candidates(wide, k)
    got = sampling.top_k_sample(view).cpu()
    assert torch.equal(got, ids[:, 0])
    c, total = cdf_of(probs)
    u = torch.from_numpy(((c[:, k - 2] + c[:, k - 1]) / 2 / total).astype(np.float32)) if k > 1 else torch.zeros(6)
    got = sampling.top_k_sample(view, k, uniforms=u.to(DEV)).cpu()
    wide_enough = torch.from_numpy((c[:, k - 1] - (c[:, k - 2] if k > 1 else 0)) / total > 2.0 ** -4)
    assert torch.equal(got[wide_enough], ids[:, k - 1][wide_enough])


def test_one_row_is_the_reference_signature(sampling):
    """top_k_sample(logit[V], top_k) → 0-d int64 tensor, as nanoPD/engine/model_runner.py:279-284 returns."""
    torch.manual_seed(8)
    logit = torch.randn(1001)                                               # an odd length: one row needs no alignment
    got = sampling.top_k_sample(logit.to(DEV))
    assert got.dim() == 0 and got.dtype == torch.int64 and int(got) == int(logit.argmax())
    got = sampling.top_k_sample(logit.to(DEV), top_k=10)
    assert got.dim() == 0 and int(got) in torch.topk(logit, 10).indices.tolist()


def test_many_rows_follow_the_distribution(sampling):
    """20 000 rows (more than one launch's 16 384) of the same logits: the frequencies of the five candidates
    follow the softmax within four standard deviations; the generator makes the draw reproducible."""
    torch.manual_seed(9)
    row = torch.randn(1024).to(torch.bfloat16)
    n = 20000
    logits = row.unsqueeze(0).expand(n, -1).contiguous().to(DEV)
    g = torch.Generator(device=DEV).manual_seed(11)
    got = sampling.top_k_sample(logits, 5, generator=g)
    again = sampling.top_k_sample(logits, 5, generator=torch.Generator(device=DEV).manual_seed(11))
    assert torch.equal(got, again)
    _, ids, probs = paged_oracle.top_k_candidates(row.unsqueeze(0), 5)
    p = probs[0].float() / probs[0].float().sum()
    counts = torch.stack([(got.cpu() == i).sum() for i in ids[0]]).float()
    assert int(counts.sum()) == n
    sigma = torch.sqrt(n * p * (1 - p))
    assert torch.all((counts - n * p).abs() <= 4 * sigma + 1), (counts, n * p)


def test_workspace_is_reusable_across_shapes(sampling):
    torch.manual_seed(10)
    for rows, vocab, k in [(3, 50000, 10), (300, 2048, 3), (1, 151936, 64), (40, 50000, 1), (3, 50000, 10)]:
        logits = torch.randn(rows, vocab).to(torch.bfloat16)
        check_draws(sampling, logits, k, torch.rand(rows))


def test_status_word_stays_clear(sampling):
    sampling.top_k_sample(torch.randn(4, 40000, device=DEV), 3, uniforms=torch.rand(4, device=DEV))
    assert sampling.check_status(DEV, raise_on_error=False) == 0


def test_argument_errors(sampling):
    logits = torch.randn(4, 1024, device=DEV)
    with pytest.raises(RuntimeError):
        sampling.top_k_sample(logits.cpu())
    with pytest.raises(RuntimeError):
        sampling.top_k_sample(logits.to(torch.float64))
    with pytest.raises(RuntimeError):
        sampling.top_k_sample(logits, 0)
    with pytest.raises(RuntimeError):
        sampling.top_k_sample(logits, 65)
    with pytest.raises(RuntimeError):
        sampling.top_k_sample(logits[:, :8], 10)
    with pytest.raises(RuntimeError):
        sampling.top_k_sample(logits, 5, uniforms=torch.rand(3, device=DEV))
    with pytest.raises(RuntimeError):
        sampling.top_k_sample(logits.t())
    assert sampling.top_k_sample(logits[:0]).numel() == 0
