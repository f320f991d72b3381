"""CPU restatement of the reference's paged spiking-Qwen2 forward (TEST INFRASTRUCTURE ONLY).

What it follows, by path inside HzAybars/Spikeinfer v0.3.0:
  * ``FastSpikingQwenModel.forward_paged`` / ``FastSpikingQwenDecoderLayer.forward_paged`` /
    ``FastSpikingQwenAttention.spike_qkv`` / ``FastSpikingQwenMLP.forward``
    (spikeinfer/modeling_fast.py:275-319, :206-211, :121-135, :186-190);
  * ``paged_attention`` (spikeinfer/attention.py:111-180): pack + index_copy_ of K/V, decode rows
    through the CPU decode attention, prefill chunks through gather + SDPA with an offset causal mask;
  * ``ModelRunner.prepare`` (spikeinfer/engine/model_runner.py:66-138) for the batch metadata;
  * Qwen2 RMSNorm / rotary embedding as the reference takes them from transformers 4.57
    (fp32 variance, ``weight * x.to(dtype)``; ``(x * cos) + (rotate_half(x) * sin)`` in the model dtype).

Weights are a plain ``dict[str, Tensor]`` keyed like the reference's ``state_dict``.  Pinned by
``tests/golden/engine_tiny.pt`` (greedy tokens, logits and packed-cache digests the reference itself
produced for the tiny configuration), checked in ``tests/test_model_oracle.py``.  Only ``tests/``,
``__graft_entry__.smoke()`` and the CPU-baseline / reference arms of ``bench.py`` may import this.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from . import torch_oracle as orc


@dataclass
class ModelShape:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    T: int = 4
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    tie_word_embeddings: bool = True


@dataclass
class Meta:
    """Same fields as the reference's AttentionMetadata (spikeinfer/attention.py:33-55)."""

    slot_mapping: torch.Tensor
    block_size: int
    num_decode_tokens: int = 0
    block_tables: torch.Tensor | None = None
    seq_lens: torch.Tensor | None = None
    prefill_query_starts: list = field(default_factory=list)
    prefill_query_lens: list = field(default_factory=list)
    prefill_context_lens: list = field(default_factory=list)
    prefill_block_tables: list = field(default_factory=list)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    dtype = x.dtype
    h = x.to(torch.float32)
    var = h.pow(2).mean(-1, keepdim=True)
    h = h * torch.rsqrt(var + eps)
    return weight * h.to(dtype)


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float, dtype: torch.dtype):
    """cos/sin [n_tok, head_dim] as Qwen2RotaryEmbedding computes them (fp32 angles, cast to dtype)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).to(torch.float32) / head_dim))
    freqs = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def causal_offset_mask(q_len: int, total: int, dtype: torch.dtype) -> torch.Tensor:
    mask = torch.full((q_len, total), float("-inf"), dtype=dtype)
    return torch.triu(mask, diagonal=total - q_len + 1)


def paged_attention(q_spk, k_spk, v_spk, k_cache, v_cache, meta: Meta, hq: int, hkv: int, d: int):
    """q/k/v spikes [T, H, n_tok, D] -> context [T, n_tok, H_q*D]; writes K/V into the caches."""
    T, n_tok = q_spk.shape[0], q_spk.shape[2]
    k_cache.index_copy_(2, meta.slot_mapping, orc.pack_spikes(k_spk))
    v_cache.index_copy_(2, meta.slot_mapping, orc.pack_spikes(v_spk))
    out = torch.empty((T, n_tok, hq, d), dtype=q_spk.dtype)
    n_dec = meta.num_decode_tokens
    if n_dec:
        q_dec = orc.pack_spikes(q_spk[:, :, :n_dec].permute(0, 2, 1, 3))
        out[:, :n_dec] = orc.paged_spike_attn_decode_batched(
            q_dec, k_cache, v_cache, meta.block_tables, meta.seq_lens, d, meta.block_size, hq, hkv,
            dtype=out.dtype)
    for i in range(len(meta.prefill_query_lens)):
        start, q_len = meta.prefill_query_starts[i], meta.prefill_query_lens[i]
        total = meta.prefill_context_lens[i] + q_len
        table = meta.prefill_block_tables[i]
        k_all = orc.gather_kv_unpacked(k_cache, table, total, d, meta.block_size, q_spk.dtype)
        v_all = orc.gather_kv_unpacked(v_cache, table, total, d, meta.block_size, q_spk.dtype)
        o = F.scaled_dot_product_attention(
            q_spk[:, :, start:start + q_len], k_all, v_all,
            attn_mask=causal_offset_mask(q_len, total, q_spk.dtype), enable_gqa=hq != hkv)
        out[:, start:start + q_len] = o.permute(0, 2, 1, 3)
    return out.view(T, n_tok, hq * d)


def forward_paged(w: dict, shape: ModelShape, input_ids, positions, k_caches, v_caches, meta: Meta,
                  capture: dict | None = None) -> torch.Tensor:
    """Rate-coded hidden states [n_tok, hidden] of one engine step.  ``capture`` (optional) receives the
    per-layer LIF input currents and spikes, for feeding the CUDA kernels identical inputs in tests."""
    T, hq, hkv, d = shape.T, shape.num_attention_heads, shape.num_key_value_heads, shape.head_dim
    n_tok = input_ids.shape[0]
    embeds = F.embedding(input_ids, w["model.embed_tokens.weight"])
    cos, sin = rope_cos_sin(positions, d, shape.rope_theta, embeds.dtype)
    cos_b, sin_b = cos[None, None], sin[None, None]  # broadcast over [T, H, n_tok, D]
    h = embeds.unsqueeze(0).expand(T, n_tok, -1).contiguous()
    for i in range(shape.num_hidden_layers):
        p = f"model.layers.{i}."
        x = rms_norm(h, w[p + "input_layernorm.weight"], shape.rms_norm_eps)
        q = F.linear(x, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.q_proj.bias"])
        k = F.linear(x, w[p + "self_attn.k_proj.weight"], w[p + "self_attn.k_proj.bias"])
        v = F.linear(x, w[p + "self_attn.v_proj.weight"], w[p + "self_attn.v_proj.bias"])
        q = q.view(T, n_tok, hq, d).permute(0, 2, 1, 3)
        k = k.view(T, n_tok, hkv, d).permute(0, 2, 1, 3)
        v = v.view(T, n_tok, hkv, d).permute(0, 2, 1, 3)
        q_pre, k_pre = q, k
        q = (q * cos_b) + (rotate_half(q) * sin_b)
        k = (k * cos_b) + (rotate_half(k) * sin_b)
        spikes = {}
        for name, cur in (("q", q), ("k", k), ("v", v)):
            s, _ = orc.lif_multistep(cur, w[p + f"self_attn.lif_{name}.lif.beta"],
                                     w[p + f"self_attn.lif_{name}.lif.threshold"])
            spikes[name] = s
        if capture is not None:
            capture[i] = dict(q_cur=q, k_cur=k, v_cur=v, q_pre=q_pre, k_pre=k_pre, cos=cos, sin=sin,
                              **{f"{n}_spk": s for n, s in spikes.items()})
        ctx = paged_attention(spikes["q"], spikes["k"], spikes["v"], k_caches[i], v_caches[i], meta, hq, hkv, d)
        h = h + F.linear(ctx, w[p + "self_attn.o_proj.weight"])
        x = rms_norm(h, w[p + "post_attention_layernorm.weight"], shape.rms_norm_eps)
        gate = F.linear(x, w[p + "mlp.gate_proj.weight"])
        gate_spk, _ = orc.lif_multistep(gate, w[p + "mlp.lif_gate.lif.beta"], w[p + "mlp.lif_gate.lif.threshold"])
        if capture is not None:
            capture[i].update(gate_cur=gate, gate_spk=gate_spk, ctx=ctx)
        h = h + F.linear(gate_spk * F.linear(x, w[p + "mlp.up_proj.weight"]), w[p + "mlp.down_proj.weight"])
    return rms_norm(h, w["model.norm.weight"], shape.rms_norm_eps).mean(dim=0)


def compute_logits(w: dict, shape: ModelShape, hidden, indices=None) -> torch.Tensor:
    if indices is not None:
        hidden = hidden.index_select(0, indices)
    head = w["model.embed_tokens.weight"] if shape.tie_word_embeddings else w["lm_head.weight"]
    return F.linear(hidden, head)


def init_weights(shape: ModelShape, seed: int = 0, dtype: torch.dtype = torch.float32, std: float = 0.02,
                 beta: float = 0.9, threshold: float = 1.0) -> dict:
    """Seeded random-init weights keyed like the reference's state_dict: normal(0, std) matrices and
    embeddings, zero biases, unit norm weights, constant LIF beta / threshold."""
    g = torch.Generator(device="cpu").manual_seed(seed)

    def mat(*size):
        return (torch.randn(size, generator=g, dtype=torch.float32) * std).to(dtype)

    hq, hkv, d, hid, inter = (shape.num_attention_heads, shape.num_key_value_heads, shape.head_dim,
                              shape.hidden_size, shape.intermediate_size)
    w = {"model.embed_tokens.weight": mat(shape.vocab_size, hid)}
    for i in range(shape.num_hidden_layers):
        p = f"model.layers.{i}."
        w[p + "self_attn.q_proj.weight"] = mat(hq * d, hid)
        w[p + "self_attn.q_proj.bias"] = torch.zeros(hq * d, dtype=dtype)
        w[p + "self_attn.k_proj.weight"] = mat(hkv * d, hid)
        w[p + "self_attn.k_proj.bias"] = torch.zeros(hkv * d, dtype=dtype)
        w[p + "self_attn.v_proj.weight"] = mat(hkv * d, hid)
        w[p + "self_attn.v_proj.bias"] = torch.zeros(hkv * d, dtype=dtype)
        w[p + "self_attn.o_proj.weight"] = mat(hid, hq * d)
        for n in ("q", "k", "v"):
            w[p + f"self_attn.lif_{n}.lif.beta"] = torch.full((d,), beta)
            w[p + f"self_attn.lif_{n}.lif.threshold"] = torch.full((d,), threshold)
        w[p + "mlp.gate_proj.weight"] = mat(inter, hid)
        w[p + "mlp.up_proj.weight"] = mat(inter, hid)
        w[p + "mlp.down_proj.weight"] = mat(hid, inter)
        w[p + "mlp.lif_gate.lif.beta"] = torch.full((inter,), beta)
        w[p + "mlp.lif_gate.lif.threshold"] = torch.full((inter,), threshold)
        w[p + "input_layernorm.weight"] = torch.ones(hid, dtype=dtype)
        w[p + "post_attention_layernorm.weight"] = torch.ones(hid, dtype=dtype)
    w["model.norm.weight"] = torch.ones(hid, dtype=dtype)
    if not shape.tie_word_embeddings:
        w["lm_head.weight"] = mat(shape.vocab_size, hid)
    return w


def randomize_lif(w: dict, seed: int = 1) -> None:
    """Per-channel beta ~ U[0,1), threshold ~ U[0.1,0.6): dense enough spiking that every LIF site and the
    per-channel broadcast are really exercised (what the reference's test fixture does, tests/conftest.py:49-60)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    for k in sorted(w):
        if k.endswith("lif.beta"):
            w[k] = torch.rand(w[k].shape, generator=g)
        elif k.endswith("lif.threshold"):
            w[k] = torch.rand(w[k].shape, generator=g) * 0.5 + 0.1


class PagedRun:
    """Minimal continuous-batching driver over forward_paged: chunk-free prefill of every prompt in one
    step, then greedy decode steps, with the reference's allocator and metadata rules."""

    def __init__(self, w: dict, shape: ModelShape, num_blocks: int, block_size: int, max_model_len: int):
        self.w, self.shape = w, shape
        self.block_size = block_size
        self.num_blocks = num_blocks
        self.pad_block = num_blocks - 1
        self.max_blocks = math.ceil(max_model_len / block_size)
        self.mgr = orc.BlockManager(num_blocks - 1, block_size)
        W = orc.packed_width(shape.head_dim)
        mk = lambda: torch.zeros((shape.T, shape.num_key_value_heads, num_blocks * block_size, W), dtype=torch.int32)
        self.k = [mk() for _ in range(shape.num_hidden_layers)]
        self.v = [mk() for _ in range(shape.num_hidden_layers)]
        self.tables: list[list[int]] = []
        self.computed: list[int] = []
        self.tokens: list[list[int]] = []

    def prefill(self, prompts: list[list[int]], capture: dict | None = None) -> torch.Tensor:
        ids, pos, slots, starts, lens, ctxs, tabs, sample = [], [], [], [], [], [], [], []
        for prompt in prompts:
            table: list[int] = []
            assert self.mgr.allocate(table, 0, len(prompt))
            starts.append(len(ids))
            ids += prompt
            pos += range(len(prompt))
            slots += self.mgr.slot_mapping(table, 0, len(prompt))
            lens.append(len(prompt))
            ctxs.append(0)
            tabs.append(torch.tensor(table, dtype=torch.int32))
            sample.append(len(ids) - 1)
            self.tables.append(table)
            self.computed.append(len(prompt))
            self.tokens.append(list(prompt))
        meta = Meta(slot_mapping=torch.tensor(slots, dtype=torch.int64), block_size=self.block_size,
                    prefill_query_starts=starts, prefill_query_lens=lens, prefill_context_lens=ctxs,
                    prefill_block_tables=tabs)
        hidden = forward_paged(self.w, self.shape, torch.tensor(ids), torch.tensor(pos), self.k, self.v, meta, capture)
        logits = compute_logits(self.w, self.shape, hidden, torch.tensor(sample)).float()
        self._accept(logits)
        return logits

    def decode(self, capture: dict | None = None) -> torch.Tensor:
        n = len(self.tables)
        for t, c in zip(self.tables, self.computed):
            assert self.mgr.allocate(t, c, 1)
        pos, slots, bt, lens = orc.prepare_decode(self.tables, self.computed, self.max_blocks, self.pad_block,
                                                  self.block_size)
        meta = Meta(slot_mapping=slots, block_size=self.block_size, num_decode_tokens=n, block_tables=bt, seq_lens=lens)
        ids = torch.tensor([t[-1] for t in self.tokens])
        hidden = forward_paged(self.w, self.shape, ids, pos, self.k, self.v, meta, capture)
        self.computed = [c + 1 for c in self.computed]
        logits = compute_logits(self.w, self.shape, hidden).float()
        self._accept(logits)
        return logits

    def _accept(self, logits: torch.Tensor) -> None:
        for toks, t in zip(self.tokens, logits.argmax(dim=-1).tolist()):
            toks.append(t)
