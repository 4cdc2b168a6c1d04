"""GPU: the decode-step harness (random-init decoder stack around the paged kernels) — one step against a CPU
restatement built from the oracle, and CUDA-graph replays against eager steps."""
import pytest
import torch
import torch.nn.functional as F

from nanopd_b200 import decoder_step, paged_kernels
from oracle import paged_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SHAPE = decoder_step.DecoderShape(num_layers=2, hidden=256, ffn=512, vocab=1000, num_q_heads=4, num_kv_heads=2,
                                  head_dim=64, rope_theta=1e4)


SHAPE128 = decoder_step.DecoderShape(num_layers=2, hidden=256, ffn=512, vocab=1000, num_q_heads=4, num_kv_heads=2,
                                     head_dim=128, rope_theta=1e4)


def make_batch(dtype, steps_ahead=4, seed=0, shape=SHAPE):
    SHAPE = shape
    torch.manual_seed(seed)
    B = 16
    ctx = torch.tensor([5, 31, 16, 70], dtype=torch.int32)
    nblk = [(int(c) + steps_ahead + B) // B for c in ctx]
    pool = sum(nblk) + 2
    perm = torch.randperm(pool)
    tables = torch.zeros(len(ctx), max(nblk), dtype=torch.int32)
    o = 0
    for i, n in enumerate(nblk):
        tables[i, :n] = perm[o:o + n].to(torch.int32)
        o += n
    kc = torch.randn(SHAPE.num_layers, pool, SHAPE.num_kv_heads, B, SHAPE.head_dim).to(dtype)
    vc = torch.randn(SHAPE.num_layers, pool, SHAPE.num_kv_heads, B, SHAPE.head_dim).to(dtype)
    tokens = torch.randint(0, SHAPE.vocab, (len(ctx),))
    return kc, vc, tables, ctx, tokens


def cpu_step(model, kc, vc, tables, ctx, tokens):
    """The same step on the CPU: fp32 GEMMs on the 16-bit weights, the oracle for norm/rotary/store/attention."""
    s, dt = model.shape, model.dtype
    cpu = lambda t: t.detach().cpu()
    x = cpu(model.embed)[tokens].float()
    pos = ctx.long()
    cos, sin = cpu(model.cos_table)[pos], cpu(model.sin_table)[pos]
    hq_d, hkv_d = s.num_q_heads * s.head_dim, s.num_kv_heads * s.head_dim
    S = tokens.numel()
    for li, L in enumerate(model.layers):
        h = F.rms_norm(x, (s.hidden,), cpu(L["in_norm"]).float(), s.eps).to(dt)
        qkv = F.linear(h.float(), cpu(L["w_qkv"]).float()).to(dt)
        q = qkv[:, :hq_d].view(S, s.num_q_heads, s.head_dim)
        k = qkv[:, hq_d:hq_d + hkv_d].view(S, s.num_kv_heads, s.head_dim)
        v = qkv[:, hq_d + hkv_d:].view(S, s.num_kv_heads, s.head_dim)
        q_rot = paged_oracle.qk_norm_rope_store(q, k, v, cos, sin, kc[li], vc[li], tables, ctx,
                                                cpu(L["q_norm"]), cpu(L["k_norm"]), s.eps)
        attn = paged_oracle.paged_decode_attention(q_rot, kc[li], vc[li], tables, ctx + 1, model.scale).to(dt)
        x = x + F.linear(attn.view(S, hq_d).float(), cpu(L["w_o"]).float())
        h = F.rms_norm(x, (s.hidden,), cpu(L["post_norm"]).float(), s.eps).to(dt)
        gu = F.linear(h.float(), cpu(L["w_gate_up"]).float())
        x = x + F.linear((F.silu(gu[:, :s.ffn]) * gu[:, s.ffn:]).to(dt).float(), cpu(L["w_down"]).float())
    return F.linear(F.rms_norm(x, (s.hidden,), cpu(model.final_norm).float(), s.eps).to(dt).float(), cpu(model.lm_head).float())


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_one_step_matches_cpu_restatement(kernels, dtype):
    model = decoder_step.SyntheticDecoder(DEV, SHAPE, dtype, seed=1, max_position=256)
    kc, vc, tables, ctx, tokens = make_batch(dtype)
    kc_d, vc_d = kc.to(DEV), vc.to(DEV)
    model.attach_batch(kc_d, vc_d, tables.to(DEV), ctx.to(DEV), tokens.to(DEV))
    model.step()
    torch.cuda.synchronize()
    want = cpu_step(model, kc, vc, tables, ctx, tokens)            # also writes the reference pages
    got = model.logits.float().cpu()
    cos_sim = F.cosine_similarity(got, want, dim=-1)
    assert float(cos_sim.min()) > 0.995, cos_sim
    # layer 0's new K/V rows come straight from the embedding: same slots, values within the dtype's rounding
    assert (kc_d[0].float().cpu() - kc[0].float()).abs().max().item() < 0.05
    assert torch.equal(model.positions.cpu(), ctx + 1) and torch.equal(model.seq_lens.cpu(), ctx + 2)
    # the sampled tokens: the reference's default top_k = 1 (nanoPD/engine/model_runner.py:279-284) over the step's logits
    assert torch.equal(model.token_ids.cpu(), paged_oracle.top_k_sample(model.logits.cpu(), 1))
    assert paged_kernels.check_status(DEV, raise_on_error=False) == 0


def test_graph_replays_equal_eager_steps(kernels):
    dtype = torch.bfloat16
    model = decoder_step.SyntheticDecoder(DEV, SHAPE, dtype, seed=2, max_position=256)
    kc, vc, tables, ctx, tokens = make_batch(dtype, seed=3)
    model.attach_batch(kc.to(DEV), vc.to(DEV), tables.to(DEV), ctx.to(DEV), tokens.to(DEV))
    eager_tokens = []
    for _ in range(3):
        model.step()
        eager_tokens.append(model.token_ids.clone())
    kc_eager = model.k_cache.clone()

    model.attach_batch(kc.to(DEV), vc.to(DEV), tables.to(DEV), ctx.to(DEV), tokens.to(DEV))
    model.capture()
    for i in range(3):
        model.replay()
        torch.cuda.synchronize()
        assert torch.equal(model.token_ids, eager_tokens[i]), f"replay {i}"
    assert torch.equal(model.k_cache, kc_eager)
    assert torch.equal(model.positions.cpu(), ctx + 3)
    assert model.launches_per_step() == 2 * SHAPE.num_layers + 1


def test_top_k_10_steps_in_a_graph_draw_fresh_numbers(kernels):
    """With top_k = 10 (what the reference's workers pass, nanoPD/workers/decode_worker.py:110) the captured step
    refreshes its uniform numbers inside the graph: every replayed token is one of the ten candidates of that
    step's logits, and two replays do not reuse the numbers."""
    dtype = torch.bfloat16
    model = decoder_step.SyntheticDecoder(DEV, SHAPE, dtype, seed=6, max_position=256, top_k=10)
    kc, vc, tables, ctx, tokens = make_batch(dtype, seed=7)
    model.attach_batch(kc.to(DEV), vc.to(DEV), tables.to(DEV), ctx.to(DEV), tokens.to(DEV))
    model.capture()
    seen = []
    for _ in range(3):
        model.replay()
        torch.cuda.synchronize()
        _, ids, _ = paged_oracle.top_k_candidates(model.logits.cpu(), 10)
        assert all(int(t) in ids[i].tolist() for i, t in enumerate(model.token_ids.cpu()))
        seen.append(model.uniforms.clone())
    assert not torch.equal(seen[0], seen[1]) and not torch.equal(seen[1], seen[2])


def test_mixed_step_decode_rows_equal_the_decode_only_step(kernels):
    """A step with a prompt chunk next to the decode batch gives the decode sequences the logits the decode-only
    step gives them, and a prompt processed in two chunks ends in the same logits as in one."""
    dtype = torch.bfloat16
    model = decoder_step.SyntheticDecoder(DEV, SHAPE128, dtype, seed=4, max_position=512)
    kc, vc, tables, ctx, tokens = make_batch(dtype, seed=5, shape=SHAPE128)
    B = 16
    decodes = [{"block_table": tables[i, :(int(ctx[i]) + B) // B].tolist(), "position": int(ctx[i])} for i in range(len(ctx))]
    # a prompt in pool blocks nobody else uses
    pool = kc.size(1)
    extra = 6
    kc = torch.cat((kc, torch.zeros(kc.size(0), extra, *kc.shape[2:], dtype=dtype)), dim=1)
    vc = torch.cat((vc, torch.zeros(vc.size(0), extra, *vc.shape[2:], dtype=dtype)), dim=1)
    prompt_table = list(range(pool, pool + extra))
    prompt = torch.randint(0, SHAPE128.vocab, (70,))
    dec_ctx = {"num_prefill_tokens": 0, "num_decode_tokens": len(decodes), "prefills": [], "decodes": decodes}
    mixed_ctx = {"num_prefill_tokens": 70, "num_decode_tokens": len(decodes), "decodes": decodes,
                 "prefills": [{"block_table": prompt_table, "start_position": 0, "num_tokens": 70}]}
    alone = model.mixed_step(dec_ctx, tokens.to(DEV), kc.to(DEV), vc.to(DEV), overlap=False)
    kc_m, vc_m = kc.to(DEV), vc.to(DEV)
    mixed = model.mixed_step(mixed_ctx, torch.cat((prompt, tokens)).to(DEV), kc_m, vc_m, overlap=False)
    torch.cuda.synchronize()
    assert mixed.shape == (1 + len(decodes), SHAPE128.vocab)
    # GEMMs over another row count may pick another algorithm: same values up to the dtype's rounding
    assert F.cosine_similarity(mixed[1:].float(), alone.float(), dim=-1).min().item() > 0.999

    # the same prompt in two chunks (40 + 30 tokens): the second chunk reads the first one's pages
    kc_c, vc_c = kc.to(DEV), vc.to(DEV)
    first = {"num_prefill_tokens": 40, "num_decode_tokens": 0, "decodes": [],
             "prefills": [{"block_table": prompt_table, "start_position": 0, "num_tokens": 40}]}
    second = {"num_prefill_tokens": 30, "num_decode_tokens": 0, "decodes": [],
              "prefills": [{"block_table": prompt_table, "start_position": 40, "num_tokens": 30}]}
    model.mixed_step(first, prompt[:40].to(DEV), kc_c, vc_c)
    chunked = model.mixed_step(second, prompt[40:].to(DEV), kc_c, vc_c)
    torch.cuda.synchronize()
    assert F.cosine_similarity(chunked[0].float(), mixed[0].float(), dim=-1).item() > 0.999
    assert (kc_c[:, pool:].float() - kc_m[:, pool:].float()).abs().max().item() < 0.1     # same pages either way
    assert paged_kernels.check_status(DEV, raise_on_error=False) == 0
