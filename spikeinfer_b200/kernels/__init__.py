"""CUDA operators with the reference's kernel-level surface (``spikeinfer/kernels/__init__.py``)."""
from .lif import (
    HARD_ZERO,
    SUBTRACT_DELAYED,
    LifSiteSpec,
    lif_gate_mul,
    lif_multistep,
    lif_pack,
    lif_pack_scatter,
    validate_thresholds,
)
from .norm import add_rms_norm
from .sampling import argmax_rows, argmax_workspace_bytes
from .packing import BITS_PER_WORD, pack_spikes, packed_bytes_per_token, packed_width, unpack_spikes
from .spike_attention import (
    gather_kv_unpacked,
    gather_kv_unpacked_batch,
    paged_spike_attn_decode,
    paged_spike_attn_decode_noalloc,
    qk_scores,
)

__all__ = [
    "lif_multistep",
    "validate_thresholds",
    "lif_pack_scatter",
    "lif_pack",
    "lif_gate_mul",
    "add_rms_norm",
    "argmax_rows",
    "argmax_workspace_bytes",
    "LifSiteSpec",
    "SUBTRACT_DELAYED",
    "HARD_ZERO",
    "pack_spikes",
    "unpack_spikes",
    "packed_width",
    "packed_bytes_per_token",
    "BITS_PER_WORD",
    "paged_spike_attn_decode",
    "paged_spike_attn_decode_noalloc",
    "gather_kv_unpacked",
    "gather_kv_unpacked_batch",
    "qk_scores",
]
