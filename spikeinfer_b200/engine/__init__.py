"""Decode-side engine pieces: the paged spike pool, the block allocator and the on-GPU batch state."""
from .batch_state import DecodeBatchState
from .block_manager import BlockManager
from .spike_cache import PagedSpikeCache

__all__ = ["DecodeBatchState", "BlockManager", "PagedSpikeCache", "SpikeDecodeEngine"]


def __getattr__(name):
    if name == "SpikeDecodeEngine":  # imported lazily: it pulls in the model
        from .decode_engine import SpikeDecodeEngine

        return SpikeDecodeEngine
    raise AttributeError(name)
