"""B200-native (sm_100a) implementation of the spiking decode hot path of HzAybars/Spikeinfer.

Three hand-written CUDA kernels behind the reference's Python operator surface: paged popcount
decode attention, fused T-step LIF + bit-pack + paged-pool scatter, and an on-GPU decode metadata
builder.  The operators run on CUDA tensors only; there is no CPU or Triton path.
"""
from . import kernels
from .kernels import (
    BITS_PER_WORD,
    gather_kv_unpacked,
    lif_multistep,
    lif_pack,
    lif_pack_scatter,
    pack_spikes,
    packed_bytes_per_token,
    packed_width,
    paged_spike_attn_decode,
    unpack_spikes,
    validate_thresholds,
)

__version__ = "0.1.0"

__all__ = [
    "kernels",
    "lif_multistep",
    "lif_pack",
    "lif_pack_scatter",
    "validate_thresholds",
    "pack_spikes",
    "unpack_spikes",
    "packed_width",
    "packed_bytes_per_token",
    "BITS_PER_WORD",
    "paged_spike_attn_decode",
    "gather_kv_unpacked",
]
