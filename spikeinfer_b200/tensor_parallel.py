"""Head-sharded tensor parallelism for the larger (7B-shape) configuration.

The reference is single-GPU; this is new design.  Within a tensor-parallel group of ``size`` GPUs the
q/k/v and gate/up projections are split column-wise by KV-head group (every rank keeps
``H_q/size`` query heads with their ``H_kv/size`` KV heads and ``intermediate/size`` MLP channels; the
per-channel LIF parameters of the gate split with its columns, those of q/k/v are per head-dim channel
and are replicated), ``o_proj`` and ``down_proj`` are split row-wise (input features), and their
partial outputs are summed with one NCCL all-reduce each (two per layer).  Embedding, norms and
``lm_head`` are replicated.  Every rank runs the hot-path kernels unchanged on its head shard, with a
page pool that holds only its KV heads; block tables and slots are identical on all ranks of a group
because they follow the same allocation sequence, so no metadata is exchanged.
"""
from __future__ import annotations

import dataclasses

import torch


def shard_config(config, size: int):
    """The per-rank model shape of a ``size``-way head-sharded group."""
    if config.num_key_value_heads % size or config.num_attention_heads % size or config.intermediate_size % size:
        raise ValueError(f"heads ({config.num_attention_heads}/{config.num_key_value_heads}) and MLP width "
                         f"({config.intermediate_size}) must divide by the group size {size}")
    return dataclasses.replace(
        config, num_attention_heads=config.num_attention_heads // size,
        num_key_value_heads=config.num_key_value_heads // size, intermediate_size=config.intermediate_size // size)


def shard_weights(weights: dict, config, rank: int, size: int) -> dict:
    """Slice a full ``state_dict``-style weights dict down to what ``rank`` of ``size`` owns."""
    if not 0 <= rank < size:
        raise ValueError(f"rank {rank} outside group of {size}")
    local = shard_config(config, size)
    d = config.head_dim
    q_rows = slice(rank * local.num_attention_heads * d, (rank + 1) * local.num_attention_heads * d)
    kv_rows = slice(rank * local.num_key_value_heads * d, (rank + 1) * local.num_key_value_heads * d)
    mlp = slice(rank * local.intermediate_size, (rank + 1) * local.intermediate_size)
    out = {}
    for name, w in weights.items():
        if name.endswith(("q_proj.weight", "q_proj.bias")):
            out[name] = w[q_rows]
        elif name.endswith(("k_proj.weight", "k_proj.bias", "v_proj.weight", "v_proj.bias")):
            out[name] = w[kv_rows]
        elif name.endswith("o_proj.weight"):
            out[name] = w[:, q_rows]
        elif name.endswith(("gate_proj.weight", "up_proj.weight")):
            out[name] = w[mlp]
        elif name.endswith("down_proj.weight"):
            out[name] = w[:, mlp]
        elif "mlp.lif_gate.lif." in name:
            out[name] = w[mlp]
        else:
            out[name] = w  # embedding, norms, lm_head, per-head-dim LIF parameters: replicated
    return {k: v.contiguous() for k, v in out.items()}
