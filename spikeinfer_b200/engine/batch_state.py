"""Device-resident decode batch state driven by the on-GPU metadata builder.

Replaces, for decode steps, ``ModelRunner.prepare`` (spikeinfer/engine/model_runner.py:66-138) and the
static-buffer refresh of ``CUDAGraphRunner.replay`` (:275-287): ``advance()`` is one kernel with fixed
launch arguments that reads and writes only device memory, so it is recorded at the head of the
captured decode graph and a replay needs no host-built tensor.  ``admit`` / ``release`` / ``take_blocks``
run between steps when the scheduler adds or retires a sequence.
"""
from __future__ import annotations

import torch

from .. import _lib


class DecodeBatchState:
    def __init__(self, max_rows: int, max_blocks: int, num_blocks: int, block_size: int,
                 device: str | torch.device = "cuda") -> None:
        """``num_blocks`` counts the pool's blocks including the reserved pad block (the last one)."""
        if num_blocks < 2:
            raise ValueError("need at least 2 blocks (one is reserved for padding)")
        self.device = torch.device(device)
        _lib.require_cuda(torch.empty(0, device=self.device), "DecodeBatchState device")
        self.max_rows, self.max_blocks = max_rows, max_blocks
        self.num_blocks, self.block_size = num_blocks, block_size
        self.pad_block = num_blocks - 1
        d = self.device
        self.free_list = torch.empty(num_blocks - 1, dtype=torch.int32, device=d)
        self._free_count = torch.zeros(1, dtype=torch.int32, device=d)
        self.active = torch.zeros(max_rows, dtype=torch.int32, device=d)
        self.seq_lens = torch.ones(max_rows, dtype=torch.int32, device=d)
        self.positions = torch.zeros(max_rows, dtype=torch.int64, device=d)
        self.slot_mapping = torch.zeros(max_rows, dtype=torch.int64, device=d)
        self.block_tables = torch.zeros((max_rows, max_blocks), dtype=torch.int32, device=d)
        self.input_ids = torch.zeros(max_rows, dtype=torch.int64, device=d)
        self.next_tokens = torch.zeros(max_rows, dtype=torch.int64, device=d)
        self.status = torch.zeros(1, dtype=torch.int32, device=d)
        self._lib = _lib.load()
        self.reset()

    def _stream(self) -> int:
        return _lib.current_stream(self.device)

    def reset(self) -> None:
        with torch.cuda.device(self.device):
            rc = self._lib.spk_meta_init(
                self.free_list.data_ptr(), self._free_count.data_ptr(), self.num_blocks - 1,
                self.active.data_ptr(), self.seq_lens.data_ptr(), self.positions.data_ptr(),
                self.slot_mapping.data_ptr(), self.block_tables.data_ptr(), self.input_ids.data_ptr(),
                self.max_rows, self.max_blocks, self.pad_block, self.block_size, self._stream())
        _lib.check(rc, "spk_meta_init")
        self.next_tokens.zero_()
        self.status.zero_()

    def advance(self, rows: int | None = None) -> None:
        """One decode step for every active row among the first ``rows`` (default: all rows).  Graph-capturable:
        no host-dependent argument.  Rows beyond ``rows`` must be inactive."""
        rows = self.max_rows if rows is None else rows
        if not 0 < rows <= self.max_rows:
            raise ValueError(f"rows must be in 1..{self.max_rows}")
        with torch.cuda.device(self.device):
            rc = self._lib.spk_meta_advance(
                self.free_list.data_ptr(), self._free_count.data_ptr(), self.active.data_ptr(),
                self.seq_lens.data_ptr(), self.positions.data_ptr(), self.slot_mapping.data_ptr(),
                self.block_tables.data_ptr(), self.input_ids.data_ptr(), self.next_tokens.data_ptr(),
                rows, self.max_blocks, self.pad_block, self.block_size, self.status.data_ptr(),
                self._stream())
        _lib.check(rc, "spk_meta_advance")

    def take_blocks(self, count: int) -> torch.Tensor:
        """Pop ``count`` blocks from the device free list (allocation order) into a new int32 tensor."""
        # pad-block filled: if the device list turns out short (status POOL_EXHAUSTED) the entries stay harmless
        dst = torch.full((count,), self.pad_block, dtype=torch.int32, device=self.device)
        with torch.cuda.device(self.device):
            rc = self._lib.spk_meta_take(self.free_list.data_ptr(), self._free_count.data_ptr(), count,
                                         dst.data_ptr(), self.status.data_ptr(), self._stream())
        _lib.check(rc, "spk_meta_take")
        return dst

    def admit(self, row: int, table: torch.Tensor, seq_len: int, last_token: int) -> None:
        """Install a prefilled sequence (its blocks already taken) in ``row``."""
        if table.dtype != torch.int32 or not table.is_cuda:
            table = table.to(device=self.device, dtype=torch.int32)
        table = table.contiguous()
        with torch.cuda.device(self.device):
            rc = self._lib.spk_meta_admit(
                row, table.data_ptr(), seq_len, last_token, self.active.data_ptr(), self.seq_lens.data_ptr(),
                self.positions.data_ptr(), self.slot_mapping.data_ptr(), self.block_tables.data_ptr(),
                self.input_ids.data_ptr(), self.next_tokens.data_ptr(), self.max_rows, self.max_blocks,
                self.pad_block, self.block_size, self.status.data_ptr(), self._stream())
        _lib.check(rc, "spk_meta_admit")

    def release(self, row: int) -> None:
        """Retire ``row``: its blocks return to the free list in table order."""
        with torch.cuda.device(self.device):
            rc = self._lib.spk_meta_release(
                row, self.free_list.data_ptr(), self._free_count.data_ptr(), self.active.data_ptr(),
                self.seq_lens.data_ptr(), self.positions.data_ptr(), self.slot_mapping.data_ptr(),
                self.block_tables.data_ptr(), self.max_rows, self.max_blocks, self.pad_block,
                self.block_size, self.num_blocks - 1, self.status.data_ptr(), self._stream())
        _lib.check(rc, "spk_meta_release")

    def free_count(self) -> int:
        """Number of free blocks (synchronises; for tests and host-side accounting only)."""
        return int(self._free_count.item())

    def check_status(self) -> None:
        """Raise if a kernel flagged an anomaly since the last check (synchronises)."""
        bits = int(self.status.item())
        if bits:
            self.status.zero_()
            names = [n for n, b in (("bad block", _lib.STATUS_BAD_BLOCK), ("bad seq_len", _lib.STATUS_BAD_SEQ_LEN),
                                    ("bad slot", _lib.STATUS_BAD_SLOT), ("pool exhausted", _lib.STATUS_POOL_EXHAUSTED),
                                    ("block table full", _lib.STATUS_TABLE_FULL),
                                    ("free list overflow", _lib.STATUS_FREE_LIST_OVERFLOW),
                                    ("row busy", _lib.STATUS_ROW_BUSY),
                                    ("device wait expired", _lib.STATUS_DEVICE_WAIT_EXPIRED)) if bits & b]
            raise _lib.SpkError("device status: " + ", ".join(names))
