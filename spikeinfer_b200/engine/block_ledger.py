"""Host-side ledger of the device free-block stack.

The decode engine allocates on the GPU (``DecodeBatchState``: ``take`` at admission, one block per row
that crosses a page boundary in ``advance``, everything back at ``release``).  How MANY blocks each of
those steps moves is a pure function of sequence lengths, so the host can keep the count without
reading the device: that is what admission control needs (the reference's scheduler asks
``BlockManager.can_allocate`` before it admits, ``spikeinfer/engine/block_manager.py:47-48, called at scheduler.py:160``; here the
question is answered from this ledger, and the block ids themselves never leave the GPU).
"""
from __future__ import annotations


class BlockLedger:
    def __init__(self, num_alloc_blocks: int, block_size: int, max_blocks_per_seq: int) -> None:
        """``num_alloc_blocks`` excludes the reserved pad block."""
        if num_alloc_blocks < 0 or block_size < 1 or max_blocks_per_seq < 1:
            raise ValueError("invalid pool geometry")
        self.num_alloc_blocks = num_alloc_blocks
        self.block_size = block_size
        self.max_blocks_per_seq = max_blocks_per_seq
        self.free = num_alloc_blocks
        self.seq_lens: dict[int, int] = {}  # active row -> cached length

    def blocks_for(self, num_tokens: int) -> int:
        return -(-num_tokens // self.block_size)

    @property
    def max_seq_len(self) -> int:
        return self.max_blocks_per_seq * self.block_size

    def admission_error(self, prompt_lens: list[int]) -> str | None:
        """Why this group of prompts cannot be admitted right now, or None if it can."""
        for n in prompt_lens:
            if n < 1:
                return "empty prompt"
            if n > self.max_seq_len:
                return f"prompt of {n} tokens exceeds max_model_len {self.max_seq_len}"
        need = sum(self.blocks_for(n) for n in prompt_lens)
        if need > self.free:
            return f"prompts need {need} blocks, {self.free} are free"
        return None

    def admit(self, row: int, seq_len: int) -> None:
        if row in self.seq_lens:
            raise RuntimeError(f"row {row} is still active")
        self.free -= self.blocks_for(seq_len)
        self.seq_lens[row] = seq_len

    def blocks_next_step(self) -> int:
        """Blocks the next ``advance`` will pop: one per active row whose length sits on a page boundary
        and whose table still has room."""
        bs = self.block_size
        return sum(1 for n in self.seq_lens.values() if n % bs == 0 and n // bs < self.max_blocks_per_seq)

    def advance(self) -> None:
        """Mirror of one ``DecodeBatchState.advance``: rows are served in row order; a row that finds the list
        empty, or whose table is full, stays where it is."""
        bs = self.block_size
        for row in sorted(self.seq_lens):
            n = self.seq_lens[row]
            if n // bs >= self.max_blocks_per_seq:
                continue
            if n % bs == 0:
                if self.free == 0:
                    continue
                self.free -= 1
            self.seq_lens[row] = n + 1

    def release(self, row: int) -> None:
        n = self.seq_lens.pop(row)
        self.free += min(self.blocks_for(n), self.max_blocks_per_seq)


def row_buckets(max_rows: int) -> list[int]:
    """Row counts a decode step can be captured for: the powers of two up to ``max_rows``, and ``max_rows``
    itself (the reference keeps such a list of batch-size buckets, ``spikeinfer/config.py:118-126``)."""
    if max_rows < 1:
        raise ValueError("max_rows must be at least 1")
    return sorted({min(1 << i, max_rows) for i in range(max_rows.bit_length() + 1)})


def covering_bucket(buckets: list[int], rows_in_use) -> int:
    """Smallest bucket that covers every row in use (rows are handed out lowest first, so a bucket of b rows
    runs rows 0..b-1); the largest bucket when none does."""
    top = max(rows_in_use, default=-1) + 1
    for b in buckets:
        if b >= top:
            return b
    return buckets[-1]
