"""Decode-side engine pieces: the paged spike pool, the on-GPU batch state and its host-side block ledger."""
from .batch_state import DecodeBatchState
from .block_ledger import BlockLedger
from .spike_cache import PagedSpikeCache

__all__ = ["DecodeBatchState", "BlockLedger", "PagedSpikeCache", "SpikeDecodeEngine"]


def __getattr__(name):
    if name == "SpikeDecodeEngine":  # imported lazily: it pulls in the model
        from .decode_engine import SpikeDecodeEngine

        return SpikeDecodeEngine
    raise AttributeError(name)
