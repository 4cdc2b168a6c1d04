"""A random-init decoder stack of Qwen3 shape around the paged kernels: the measurement harness for decode
tokens/s at model level.

It runs what ``ModelRunner`` runs per decode step (nanoPD/engine/model_runner.py:75-212 inside the Hugging Face
layer loop, then sampling at :279-284) with this library as the attention block: per layer RMSNorm → one fused
QKV projection → ``paged_qk_norm_rope_store`` → ``paged_attention_forward`` → output projection → MLP.  The
projections are plain library GEMMs (``torch.nn.functional.linear``); block tables, positions and lengths live on
the device for the whole run and advance in place, so a step has no host→device traffic and the whole step —
36 layers, sampling (``sampling.top_k_sample``, one launch for the batch, tokens stay on the device) and the
advance of the positions — is one CUDA graph.

Weights are random (there are no checkpoints here); shapes default to Qwen3-8B (36 layers, hidden 4096, FFN 12288,
32 query / 8 KV heads of 128, vocabulary 151 936, rope theta 1e6).  ``top_k`` defaults to 1 as the reference's
``top_k_sample`` does (one call and one ``.item()`` per sequence there, model_runner.py:279-284, engine.py:100-106).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn.functional as F

from . import paged_kernels, sampling


@dataclass
class DecoderShape:
    num_layers: int = 36
    hidden: int = 4096
    ffn: int = 12288
    vocab: int = 151936
    num_q_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    rope_theta: float = 1e6
    eps: float = 1e-6
    qk_norm: bool = True

    @property
    def param_count(self) -> int:
        qkv = self.hidden * (self.num_q_heads + 2 * self.num_kv_heads) * self.head_dim
        o = self.num_q_heads * self.head_dim * self.hidden
        mlp = 3 * self.hidden * self.ffn
        return self.num_layers * (qkv + o + mlp + 2 * self.hidden + 2 * self.head_dim) + 2 * self.vocab * self.hidden + self.hidden


class SyntheticDecoder:
    """Weights + per-step buffers on one device.  ``attach_batch`` binds a decode batch (block tables, context
    lengths, KV pools of all layers); ``step`` runs one token for every sequence and advances the batch."""

    def __init__(self, device, shape: Optional[DecoderShape] = None, dtype=torch.bfloat16, seed: int = 0,
                 max_position: int = 16384, top_k: int = 1):
        self.shape = s = shape or DecoderShape()
        self.top_k = int(top_k)
        self.device = torch.device(device)
        self.dtype = dtype
        gen = torch.Generator(device=self.device)
        gen.manual_seed(seed)

        def w(*dims, std):
            return (torch.randn(*dims, device=self.device, dtype=torch.float32, generator=gen) * std).to(dtype)

        qkv_out = (s.num_q_heads + 2 * s.num_kv_heads) * s.head_dim
        self.embed = w(s.vocab, s.hidden, std=0.02)
        self.lm_head = w(s.vocab, s.hidden, std=0.02)
        self.final_norm = torch.ones(s.hidden, device=self.device, dtype=dtype)
        self.layers: List[dict] = []
        for _ in range(s.num_layers):
            self.layers.append(dict(
                in_norm=torch.ones(s.hidden, device=self.device, dtype=dtype),
                post_norm=torch.ones(s.hidden, device=self.device, dtype=dtype),
                w_qkv=w(qkv_out, s.hidden, std=s.hidden ** -0.5),
                w_o=w(s.hidden, s.num_q_heads * s.head_dim, std=(s.num_q_heads * s.head_dim) ** -0.5 / 6),
                w_gate_up=w(2 * s.ffn, s.hidden, std=s.hidden ** -0.5),
                w_down=w(s.hidden, s.ffn, std=s.ffn ** -0.5 / 6),
                q_norm=torch.ones(s.head_dim, device=self.device, dtype=dtype) if s.qk_norm else None,
                k_norm=torch.ones(s.head_dim, device=self.device, dtype=dtype) if s.qk_norm else None,
            ))
        # rotary tables as the Hugging Face rotary module builds them: fp32 angles, cos/sin cast to the model dtype
        inv_freq = 1.0 / (s.rope_theta ** (torch.arange(0, s.head_dim, 2, dtype=torch.float32, device=self.device) / s.head_dim))
        ang = torch.arange(max_position, dtype=torch.float32, device=self.device)[:, None] * inv_freq[None, :]
        emb = torch.cat((ang, ang), dim=-1)
        self.cos_table = emb.cos().to(dtype)
        self.sin_table = emb.sin().to(dtype)
        self.max_position = max_position
        self.scale = s.head_dim ** -0.5
        self._graph = None

    # ---- batch state -------------------------------------------------------------------------------------
    def attach_batch(self, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor,
                     ctx_lens: torch.Tensor, token_ids: torch.Tensor, active: Optional[torch.Tensor] = None) -> None:
        """``k_cache``/``v_cache`` ``[L, blocks, Hkv, B, D]`` (the reference's pool layout, model_runner.py:24-31),
        ``block_tables`` int32 ``[S, max_blk]`` with room for the tokens to come, ``ctx_lens`` int32 ``[S]`` tokens
        already in the pool, ``token_ids`` int64 ``[S]`` the tokens to feed first.

        ``active`` (int32 ``[S]`` of 0/1, optional) turns the batch into a table of SLOTS for continuous batching:
        a step advances only the rows whose entry is 1.  An idle slot keeps ``seq_lens == 0`` (its attention row is
        zero) and position 0 of whatever block its table row names, so give idle rows a block nobody reads.  The
        four state tensors (``block_tables``, ``positions``, ``seq_lens``, ``active``) and ``token_ids`` may be
        rewritten in place between steps — also between replays of a captured step."""
        s = self.shape
        if k_cache.dim() != 5 or k_cache.size(0) != s.num_layers or k_cache.size(2) != s.num_kv_heads or k_cache.size(4) != s.head_dim:
            raise RuntimeError("k_cache must be [num_layers, blocks, Hkv, B, D] for this decoder's shape")
        self.k_cache, self.v_cache = k_cache, v_cache
        self.block_size = k_cache.size(3)
        self.block_tables = block_tables
        self.positions = ctx_lens.clone()                       # slot of the token being fed
        self.active = active
        self.seq_lens = ctx_lens + 1 if active is None else (ctx_lens + 1) * active
        self.token_ids = token_ids.clone()
        S = token_ids.numel()
        self.q_rot = torch.empty(S, s.num_q_heads, s.head_dim, dtype=self.dtype, device=self.device)
        self.attn_out = torch.empty_like(self.q_rot)
        self.uniforms = torch.zeros(S, dtype=torch.float32, device=self.device)
        self._graph = None

    def detach_batch(self) -> None:
        """Drops the batch state, the pools and the captured step (and with it the memory the capture holds)."""
        self._graph = None
        for name in ("k_cache", "v_cache", "block_tables", "positions", "seq_lens", "active", "token_ids", "q_rot",
                     "attn_out", "uniforms", "logits"):
            if hasattr(self, name):
                delattr(self, name)

    # ---- one decode step -----------------------------------------------------------------------------------
    def _forward(self) -> None:
        s = self.shape
        S = self.token_ids.numel()
        hq_d, hkv_d = s.num_q_heads * s.head_dim, s.num_kv_heads * s.head_dim
        x = self.embed.index_select(0, self.token_ids)
        cos = self.cos_table.index_select(0, self.positions)
        sin = self.sin_table.index_select(0, self.positions)
        max_blk = self.block_tables.size(1)
        for li, L in enumerate(self.layers):
            h = F.rms_norm(x, (s.hidden,), L["in_norm"], s.eps)
            qkv = F.linear(h, L["w_qkv"])
            q = qkv[:, :hq_d].view(S, s.num_q_heads, s.head_dim)
            k = qkv[:, hq_d:hq_d + hkv_d].view(S, s.num_kv_heads, s.head_dim)
            v = qkv[:, hq_d + hkv_d:].view(S, s.num_kv_heads, s.head_dim)
            paged_kernels.paged_qk_norm_rope_store(q, k, v, cos, sin, self.k_cache[li], self.v_cache[li],
                                                   self.block_tables, self.positions, L["q_norm"], L["k_norm"],
                                                   s.eps, q_out=self.q_rot)
            paged_kernels.paged_attention_forward(self.attn_out, self.q_rot, self.k_cache[li], self.v_cache[li],
                                                  self.block_tables, self.seq_lens, self.scale, self.block_size, max_blk)
            x = x + F.linear(self.attn_out.view(S, hq_d), L["w_o"])
            h = F.rms_norm(x, (s.hidden,), L["post_norm"], s.eps)
            gu = F.linear(h, L["w_gate_up"])
            x = x + F.linear(F.silu(gu[:, :s.ffn]) * gu[:, s.ffn:], L["w_down"])
        logits = F.linear(F.rms_norm(x, (s.hidden,), self.final_norm, s.eps), self.lm_head)
        self.logits = logits
        if self.top_k > 1:
            self.uniforms.uniform_()
        sampling.top_k_sample(logits, self.top_k, uniforms=self.uniforms if self.top_k > 1 else None,
                              out=self.token_ids)
        if self.active is None:
            self.positions.add_(1)
            self.seq_lens.add_(1)
        else:
            self.positions.add_(self.active)
            self.seq_lens.add_(self.active)

    def step(self) -> None:
        """One token for every sequence, eagerly (one launch per op)."""
        self._forward()

    def capture(self) -> None:
        """Captures ``step`` in a CUDA graph (after one eager warm-up on the capture stream, which is undone by
        moving the positions back; the slot it wrote is rewritten by the first replay)."""
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        keep = self.token_ids.clone()
        with torch.cuda.stream(side):
            self._forward()
            self.positions.sub_(1 if self.active is None else self.active)
            self.seq_lens.sub_(1 if self.active is None else self.active)
            self.token_ids.copy_(keep)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            self._forward()                 # recorded, not run: the batch state is still the restored one
        torch.cuda.synchronize(self.device)
        self._graph = graph

    def replay(self) -> None:
        if self._graph is None:
            raise RuntimeError("capture() first")
        self._graph.replay()

    def launches_per_step(self) -> int:
        """This library's kernels per step: one fused norm/rotary/store and one attention launch per layer, and
        the sampler."""
        return 2 * self.shape.num_layers + 1

    # ---- one scheduler step with prompt chunks and decode sequences -----------------------------------------
    def mixed_step(self, ctx: dict, token_ids: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                   overlap: bool = True, after_layer=None) -> torch.Tensor:
        """Runs the scheduler's step ``ctx`` (the reference's context dict, nanoPD/engine/engine.py:68-90) through
        all layers: ``token_ids`` int64 ``[num_prefill_tokens + num_decode_tokens]`` are the packed prompt-chunk
        tokens followed by one token per decode sequence, ``k_cache``/``v_cache`` the ``[L, blocks, Hkv, B, D]``
        pools.  Tables and positions go to the device once (``build_step_context``); every layer then runs the
        fused norm/rotary/store launches and the two attention kernels (side by side in a mixed step).  Returns
        the logits of the last token of every prompt chunk followed by those of the decode sequences, as the
        reference samples them (nanoPD/engine/engine.py:96-108).  Eager: the chunk lists are host data.
        ``after_layer(layer_index)`` is called once the launches of a layer's store and attention have been
        issued — the hook a prefill worker uses to start moving that layer's pages to the decode GPU while the
        remaining layers still compute."""
        from . import paged_forward
        s = self.shape
        sc = paged_forward.build_step_context(ctx, self.device, block_size=k_cache.size(3))
        total = sc.num_prefill_tokens + sc.num_decode_tokens
        if token_ids.numel() != total:
            raise RuntimeError("token_ids does not match the step's token count")
        pos_parts = [t for t in (sc.prefill_positions, sc.decode_positions) if t is not None]
        positions = torch.cat(pos_parts) if len(pos_parts) > 1 else pos_parts[0]
        cos = self.cos_table.index_select(0, positions)
        sin = self.sin_table.index_select(0, positions)
        hq_d, hkv_d = s.num_q_heads * s.head_dim, s.num_kv_heads * s.head_dim
        x = self.embed.index_select(0, token_ids)
        for li, L in enumerate(self.layers):
            h = F.rms_norm(x, (s.hidden,), L["in_norm"], s.eps)
            qkv = F.linear(h, L["w_qkv"])
            q = qkv[:, :hq_d].view(total, s.num_q_heads, s.head_dim)
            k = qkv[:, hq_d:hq_d + hkv_d].view(total, s.num_kv_heads, s.head_dim)
            v = qkv[:, hq_d + hkv_d:].view(total, s.num_kv_heads, s.head_dim)
            attn = paged_forward.paged_attention_step_fused(sc, q, k, v, cos, sin, k_cache[li], v_cache[li], self.scale,
                                                            L["q_norm"], L["k_norm"], s.eps, overlap=overlap)
            if after_layer is not None:
                after_layer(li)
            x = x + F.linear(attn.view(total, hq_d), L["w_o"])
            h = F.rms_norm(x, (s.hidden,), L["post_norm"], s.eps)
            gu = F.linear(h, L["w_gate_up"])
            x = x + F.linear(F.silu(gu[:, :s.ffn]) * gu[:, s.ffn:], L["w_down"])
        last_rows = [off + n - 1 for off, n in zip(sc.prefill_offsets, sc.prefill_tokens)]
        last_rows += list(range(sc.num_prefill_tokens, total))
        rows = torch.tensor(last_rows, dtype=torch.int64).pin_memory().to(self.device, non_blocking=True)
        return F.linear(F.rms_norm(x.index_select(0, rows), (s.hidden,), self.final_norm, s.eps), self.lm_head)
