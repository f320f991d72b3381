"""Host-side physical block allocator, same contract as ``spikeinfer/engine/block_manager.py``.

Used for prefill-time allocation and as the host mirror of the device free list kept by
:class:`~spikeinfer_b200.engine.batch_state.DecodeBatchState`: allocation is a pure function of
sequence lengths, so the host can follow the device without reading it back.
"""
from __future__ import annotations


class BlockManager:
    def __init__(self, num_blocks: int, block_size: int) -> None:
        if num_blocks < 1:
            raise ValueError(f"need at least one block, got {num_blocks}")
        self.num_blocks = num_blocks
        self.block_size = block_size
        self._free = list(range(num_blocks - 1, -1, -1))  # popped from the tail: 0, 1, 2, ...

    @property
    def num_free_blocks(self) -> int:
        return len(self._free)

    @property
    def num_used_blocks(self) -> int:
        return self.num_blocks - len(self._free)

    @property
    def utilization(self) -> float:
        return self.num_used_blocks / self.num_blocks

    def blocks_for(self, num_tokens: int) -> int:
        return -(-num_tokens // self.block_size)

    def blocks_needed(self, seq, num_new_tokens: int) -> int:
        return max(0, self.blocks_for(seq.num_computed_tokens + num_new_tokens) - len(seq.block_table))

    def can_allocate(self, seq, num_new_tokens: int) -> bool:
        return self.blocks_needed(seq, num_new_tokens) <= len(self._free)

    def allocate(self, seq, num_new_tokens: int) -> bool:
        """Grow ``seq.block_table`` for ``num_new_tokens`` more tokens; all or nothing."""
        need = self.blocks_needed(seq, num_new_tokens)
        if need > len(self._free):
            return False
        seq.block_table.extend(self._free.pop() for _ in range(need))
        return True

    def free(self, seq) -> None:
        self._free.extend(seq.block_table)
        seq.block_table = []

    def reset(self) -> None:
        self._free = list(range(self.num_blocks - 1, -1, -1))

    def slot_mapping(self, seq, start: int, count: int) -> list[int]:
        bs = self.block_size
        return [seq.block_table[p // bs] * bs + p % bs for p in range(start, start + count)]
