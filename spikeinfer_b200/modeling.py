"""Layer-major, T-batched spiking Qwen2 decoder for the paged engine (CUDA).

The computation is the reference's ``FastSpikingQwenModel.forward_paged``
(``spikeinfer/modeling_fast.py:275-319``: embed -> [RMSNorm -> q/k/v projections -> RoPE -> LIF ->
paged spike attention -> o_proj -> RMSNorm -> LIF-gated MLP] x layers -> RMSNorm -> mean over T) with
the hot-path call sites replaced:

* q/k/v projections are one GEMM over concatenated weights; RoPE is applied to its q and k columns;
* LIF of q, k and v + bit-pack + K/V scatter into the paged pool is one launch
  (:func:`spikeinfer_b200.attention.fused_qkv_attention`) instead of three ``lif_multistep``, three
  ``pack_spikes`` and two ``index_copy_`` (``modeling_fast.py:132-134``, ``attention.py:138-148``);
* decode rows attend through the popcount kernel;
* RoPE (``modeling_fast.py:89-99``) is applied to the q and k currents inside that launch, with every
  operation rounded to the model dtype as the eager expression does;
* the gate LIF and the ``gate_spk * up_proj(x)`` product (``modeling_fast.py:186-190``) are one launch
  that never writes the dense gate spikes;
* each residual add + RMSNorm pair is one launch.

Dense GEMMs stay PyTorch (cuBLAS), as do the embedding lookup, the final mean over T and argmax.  Weights are a
``dict[str, Tensor]`` keyed exactly like the reference's ``state_dict``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import _lib
from .attention import AttentionMetadata, fused_qkv_attention
from .kernels import add_rms_norm, lif_gate_mul


@dataclass
class SpikingQwenConfig:
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

    @classmethod
    def qwen2_5_0p5b(cls) -> "SpikingQwenConfig":
        return cls(vocab_size=151936, hidden_size=896, intermediate_size=4864, num_hidden_layers=24,
                   num_attention_heads=14, num_key_value_heads=2, head_dim=64)

    @classmethod
    def tiny(cls) -> "SpikingQwenConfig":
        return cls(vocab_size=32000, hidden_size=256, intermediate_size=1024, num_hidden_layers=4,
                   num_attention_heads=4, num_key_value_heads=2, head_dim=64)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Qwen2RMSNorm: fp32 variance, ``weight * normalised.to(dtype)``."""
    dtype = x.dtype
    h = x.to(torch.float32)
    h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    return weight * h.to(dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


class SpikingQwenModel:
    """Inference-only model over a weights dict; every tensor lives on ``device``."""

    def __init__(self, config: SpikingQwenConfig, weights: dict, device: str | torch.device = "cuda",
                 dtype: torch.dtype | None = None, tp_group=None) -> None:
        """``tp_group``: a ``torch.distributed`` process group when ``config``/``weights`` are one rank's shard
        of a head-sharded model (see :mod:`spikeinfer_b200.tensor_parallel`); the partial outputs of
        ``o_proj`` and ``down_proj`` are then summed over the group."""
        self.config = config
        self.tp_group = tp_group
        self.device = torch.device(device)
        _lib.require_cuda(torch.empty(0, device=self.device), "SpikingQwenModel device")
        c = config
        get = lambda k: weights[k].to(device=self.device, dtype=dtype or weights[k].dtype)
        f32 = lambda k: weights[k].to(device=self.device, dtype=torch.float32).contiguous()
        self.embed = get("model.embed_tokens.weight")
        self.dtype = self.embed.dtype
        self.lm_head = self.embed if c.tie_word_embeddings else get("lm_head.weight")
        self.norm = get("model.norm.weight")
        self.layers = []
        for i in range(c.num_hidden_layers):
            p = f"model.layers.{i}."
            a = p + "self_attn."
            self.layers.append(dict(
                ln1=get(p + "input_layernorm.weight"), ln2=get(p + "post_attention_layernorm.weight"),
                w_qkv=torch.cat([get(a + "q_proj.weight"), get(a + "k_proj.weight"), get(a + "v_proj.weight")]).contiguous(),
                b_qkv=torch.cat([get(a + "q_proj.bias"), get(a + "k_proj.bias"), get(a + "v_proj.bias")]).contiguous(),
                w_o=get(a + "o_proj.weight"),
                lif_q=(f32(a + "lif_q.lif.beta"), f32(a + "lif_q.lif.threshold")),
                lif_k=(f32(a + "lif_k.lif.beta"), f32(a + "lif_k.lif.threshold")),
                lif_v=(f32(a + "lif_v.lif.beta"), f32(a + "lif_v.lif.threshold")),
                w_gate_up=torch.cat([get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight")]).contiguous(),
                w_down=get(p + "mlp.down_proj.weight"),
                lif_gate=(f32(p + "mlp.lif_gate.lif.beta"), f32(p + "mlp.lif_gate.lif.threshold")),
            ))
        half = torch.arange(0, c.head_dim, 2, dtype=torch.int64, device=self.device).to(torch.float32)
        self.inv_freq = 1.0 / (c.rope_theta ** (half / c.head_dim))
        self.rope_table: torch.Tensor | None = None

    def validate_thresholds(self) -> bool:
        """threshold > 0 at every LIF site (checked once at load, never per call)."""
        for i, layer in enumerate(self.layers):
            for site in ("lif_q", "lif_k", "lif_v", "lif_gate"):
                th = layer[site][1]
                if not bool(torch.all(th > 0)):
                    raise ValueError(f"lif_multistep requires threshold > 0; violated at layer {i} {site} "
                                     f"(min={th.min().item():.4g})")
        return True

    def _reduce(self, partial: torch.Tensor) -> torch.Tensor:
        """Sum a row-sharded projection's partial outputs over the tensor-parallel group (NCCL all-reduce)."""
        if self.tp_group is not None:
            torch.distributed.all_reduce(partial, group=self.tp_group)
        return partial

    def _rope_direct(self, positions: torch.Tensor):
        freqs = positions.to(torch.float32)[:, None] * self.inv_freq[None, :]
        emb = torch.cat((freqs, freqs), dim=-1)
        return emb.cos().to(self.dtype), emb.sin().to(self.dtype)

    def build_rope_table(self, max_positions: int) -> None:
        """Tabulate the rotary factors of positions ``0 .. max_positions - 1`` with the very operations
        :meth:`rope` would run per step, so that a step needs one gather instead of seven small launches and
        gets bit-identical factors.  Positions beyond the table must not be fed afterwards."""
        cos, sin = self._rope_direct(torch.arange(max_positions, device=self.device))
        self.rope_table = torch.stack((cos, sin), dim=1).contiguous()  # [max_positions, 2, head_dim]

    def rope(self, positions: torch.Tensor):
        """``(cos, sin)``, each ``[n_tok, head_dim]`` in the model dtype (rows may be strided)."""
        if self.rope_table is not None:
            rows = self.rope_table.index_select(0, positions)
            return rows[:, 0], rows[:, 1]
        return self._rope_direct(positions)

    @torch.no_grad()
    def forward_paged(self, input_ids, positions, kv_caches, meta: AttentionMetadata, T: int | None = None):
        """``input_ids``/``positions`` ``[n_tok]`` (decode tokens first); ``kv_caches`` per layer ``(k, v)``.
        Returns rate-coded hidden states ``[n_tok, hidden]``."""
        c = self.config
        T = T or c.T
        hq, hkv, d = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        n_tok = input_ids.shape[0]
        embeds = F.embedding(input_ids, self.embed)
        rope = self.rope(positions)  # (cos, sin), each [n_tok, D]
        h = embeds.unsqueeze(0).expand(T, n_tok, -1).contiguous()
        delta = None
        for i, L in enumerate(self.layers):
            x = add_rms_norm(h, delta, L["ln1"], c.rms_norm_eps)  # h <- h + delta, x = norm(h)
            qkv = F.linear(x, L["w_qkv"], L["b_qkv"])  # [T, n_tok, (hq + 2 hkv) d]
            ctx = fused_qkv_attention(qkv, L["lif_q"], L["lif_k"], L["lif_v"], kv_caches[i][0], kv_caches[i][1],
                                      meta, hq, hkv, d, rope=rope)
            delta = self._reduce(F.linear(ctx, L["w_o"]))
            x = add_rms_norm(h, delta, L["ln2"], c.rms_norm_eps)
            gu = F.linear(x, L["w_gate_up"])  # [T, n_tok, 2 * inter]
            act = lif_gate_mul(gu[..., : c.intermediate_size], gu[..., c.intermediate_size:], *L["lif_gate"])
            delta = self._reduce(F.linear(act, L["w_down"]))
        return add_rms_norm(h, delta, self.norm, c.rms_norm_eps).mean(dim=0)

    @torch.no_grad()
    def compute_logits(self, hidden: torch.Tensor, indices: torch.Tensor | None = None) -> torch.Tensor:
        """Project only the rows that are sampled (row selection before ``lm_head``)."""
        if indices is not None:
            hidden = hidden.index_select(0, indices)
        return F.linear(hidden, self.lm_head)
