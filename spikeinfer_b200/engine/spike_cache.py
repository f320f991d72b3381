"""The paged, bit-packed spike K/V pool (contract of ``spikeinfer/engine/spike_cache.py:20-101``).

Per layer two ``int32`` pools addressed ``[T, H_kv, num_slots, W]``; a block is ``block_size``
consecutive slots; the last block is reserved for the padding rows of graph-captured decode
batches and is never handed to the allocator.

Two memory layouts give the same logical tensors:

* ``"reference"``: each pool is its own contiguous ``[T, H_kv, num_slots, W]`` slab, exactly the
  reference's layout (one page is 128 B at W=2, block 16).
* ``"page_major"``: one buffer per layer laid out ``[num_blocks, T, H_kv, 2(K|V), block_size, W]``,
  so everything a page holds for one layer (all timesteps, heads, K and V) is one contiguous
  2 KB run at the 0.5B shape.  ``k``/``v`` are then strided views with an explicit block axis,
  ``[T, H_kv, num_blocks, block_size, W]``; the kernels take the strides.
"""
from __future__ import annotations

import torch

from ..kernels.packing import packed_width


class PagedSpikeCache:
    def __init__(self, num_layers: int, timesteps: int, num_kv_heads: int, head_dim: int, num_blocks: int,
                 block_size: int, device: str | torch.device = "cuda", layout: str = "reference") -> None:
        if num_blocks < 2:
            raise ValueError("need at least 2 blocks (one is reserved for padding)")
        if block_size < 1 or block_size & (block_size - 1):
            raise ValueError(f"block_size must be a power of two, got {block_size}")
        if layout not in ("reference", "page_major"):
            raise ValueError(f"unknown layout {layout!r}")
        self.num_layers = num_layers
        self.timesteps = timesteps
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.num_blocks = num_blocks
        self.block_size = block_size
        self.words = packed_width(head_dim)
        self.layout = layout
        self.device = torch.device(device)
        T, H, W = timesteps, num_kv_heads, self.words
        self.k, self.v, self._buffers = [], [], []
        for _ in range(num_layers):
            if layout == "reference":
                k = torch.zeros((T, H, num_blocks * block_size, W), dtype=torch.int32, device=self.device)
                v = torch.zeros_like(k)
                self._buffers += [k, v]
            else:
                buf = torch.zeros((num_blocks, T, H, 2, block_size, W), dtype=torch.int32, device=self.device)
                k = buf[:, :, :, 0].permute(1, 2, 0, 3, 4)
                v = buf[:, :, :, 1].permute(1, 2, 0, 3, 4)
                self._buffers.append(buf)
            self.k.append(k)
            self.v.append(v)
        self.layers = list(zip(self.k, self.v))

    def scatter_strides(self, pool: torch.Tensor) -> tuple[int, int, int]:
        """(t, slot, head) element strides for writing word rows by flat slot index.  Only the
        reference layout has a uniform slot stride; page-major pools are written block-wise."""
        if pool.ndim != 4:
            raise ValueError("flat slot addressing needs the reference layout")
        return pool.stride(0), pool.stride(2), pool.stride(1)

    @staticmethod
    def bytes_per_block(num_layers: int, timesteps: int, num_kv_heads: int, head_dim: int, block_size: int) -> int:
        return 2 * num_layers * timesteps * num_kv_heads * block_size * packed_width(head_dim) * 4

    @property
    def nbytes(self) -> int:
        return self.bytes_per_block(self.num_layers, self.timesteps, self.num_kv_heads, self.head_dim,
                                    self.block_size) * self.num_blocks

    @property
    def num_allocatable_blocks(self) -> int:
        return self.num_blocks - 1

    @property
    def pad_block(self) -> int:
        return self.num_blocks - 1

    @property
    def pad_slot(self) -> int:
        return self.pad_block * self.block_size

    @property
    def capacity_tokens(self) -> int:
        return self.num_allocatable_blocks * self.block_size

    def logical(self, pool: torch.Tensor) -> torch.Tensor:
        """The pool as a contiguous ``[T, H_kv, num_slots, W]`` tensor (for checks and prefill reads)."""
        if pool.ndim == 4:
            return pool
        T, H, nb, bs, W = pool.shape
        return pool.reshape(T, H, nb * bs, W)

    def reset(self) -> None:
        for t in self._buffers:
            t.zero_()
