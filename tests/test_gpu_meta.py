"""GPU parity: the on-device decode metadata builder against the oracle's BlockManager / prepare_decode
(the reference's host-side allocator and runner, block_manager.py:50-77, model_runner.py:66-138)."""
from __future__ import annotations

import pytest
import torch

from oracle import torch_oracle as orc
from spikeinfer_b200 import _lib
from spikeinfer_b200.engine.batch_state import DecodeBatchState

pytestmark = pytest.mark.gpu


def test_trace_matches_host_allocator(dev):
    bs, num_blocks, max_rows, max_blocks = 4, 13, 8, 8  # last block = pad
    state = DecodeBatchState(max_rows=max_rows, max_blocks=max_blocks, num_blocks=num_blocks, block_size=bs, device=dev)
    mgr = orc.BlockManager(num_blocks - 1, bs)
    tables = {}
    computed = {}
    # admit three prefilled sequences into rows 0, 2, 5 (prompt lengths 5, 9, 2)
    for row, plen, tok in ((0, 5, 11), (2, 9, 22), (5, 2, 33)):
        t = []
        assert mgr.allocate(t, 0, plen)
        got = state.take_blocks(mgr.blocks_for(plen))
        assert got.tolist() == t, "device free list hands out blocks in a different order"
        state.admit(row, got, plen, tok)
        tables[row], computed[row] = t, plen
    assert state.free_count() == len(mgr.free_list)
    next_tokens = torch.arange(100, 100 + max_rows, dtype=torch.int64, device=dev)
    for step in range(7):
        rows = sorted(tables)
        for r in rows:  # host allocator: row order
            assert mgr.allocate(tables[r], computed[r], 1)
        pos, slots, bt, lens = orc.prepare_decode([tables[r] for r in rows], [computed[r] for r in rows],
                                                  max_blocks, num_blocks - 1, bs)
        state.next_tokens.copy_(next_tokens + step)
        state.advance()
        for i, r in enumerate(rows):
            assert state.positions[r].item() == pos[i].item()
            assert state.slot_mapping[r].item() == slots[i].item()
            assert state.seq_lens[r].item() == lens[i].item()
            assert state.block_tables[r].tolist() == bt[i].tolist()
            assert state.input_ids[r].item() == 100 + r + step
            computed[r] += 1
        for r in range(max_rows):
            if r not in tables:  # pad rows stay parked on the pad block, as the graph runner keeps them
                assert state.seq_lens[r].item() == 1 and state.slot_mapping[r].item() == (num_blocks - 1) * bs
                assert (state.block_tables[r] == num_blocks - 1).all()
        assert state.free_count() == len(mgr.free_list)
        assert state.free_list[: state.free_count()].tolist() == mgr.free_list
        if step == 3:  # sequence in row 2 finishes: blocks go back in table order
            mgr.free(tables.pop(2))
            computed.pop(2)
            state.release(2)
            assert state.free_list[: state.free_count()].tolist() == mgr.free_list
    assert state.status.item() == 0


def test_pool_exhaustion_and_full_table_are_flagged(dev):
    state = DecodeBatchState(max_rows=4, max_blocks=2, num_blocks=3, block_size=2, device=dev)
    state.admit(0, state.take_blocks(1), 2, 1)  # needs a new block at the next step
    state.admit(1, state.take_blocks(1), 2, 1)  # pool now empty
    state.advance()
    assert state.status.item() & _lib.STATUS_POOL_EXHAUSTED
    assert state.seq_lens[:2].tolist() == [2, 2], "a row that got no block must not advance"
    assert state.slot_mapping[0].item() == 2 * 2  # parked on the pad slot
    state.status.zero_()
    state2 = DecodeBatchState(max_rows=2, max_blocks=1, num_blocks=4, block_size=2, device=dev)
    state2.admit(0, state2.take_blocks(1), 2, 1)
    state2.advance()
    assert state2.status.item() & _lib.STATUS_TABLE_FULL
    assert state2.seq_lens[0].item() == 2


def test_release_past_capacity_and_admit_into_a_busy_row_are_flagged(dev):
    """A free count that was not kept in step with the tables must not push past the list; a row that still holds
    a sequence keeps it."""
    state = DecodeBatchState(max_rows=2, max_blocks=4, num_blocks=5, block_size=2, device=dev)
    table = state.take_blocks(2)
    state.admit(0, table, 4, 7)
    assert state.free_count() == 2
    state._free_count.fill_(4)          # host-side injection: pretend nothing was ever taken
    before = state.free_list.clone()
    state.release(0)
    assert state.status.item() & _lib.STATUS_FREE_LIST_OVERFLOW
    assert torch.equal(state.free_list, before) and state.free_count() == 4, "nothing may be pushed"
    assert state.active[0].item() == 0, "the row is retired all the same"
    state.status.zero_()
    state.reset()
    t0 = state.take_blocks(1)
    state.admit(1, t0, 2, 5)
    row_before = state.block_tables[1].clone()
    state.admit(1, state.take_blocks(1), 1, 9)   # the row is busy
    assert state.status.item() & _lib.STATUS_ROW_BUSY
    assert torch.equal(state.block_tables[1], row_before) and state.seq_lens[1].item() == 2
    assert state.input_ids[1].item() == 5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_argmax_rows_matches_torch(dtype, dev):
    """Greedy sampling kernel against torch.argmax: ragged vocabulary sizes, ties (first index wins, bf16 makes
    plenty), a strided view, -inf rows, and NaN counting as the maximum."""
    from spikeinfer_b200 import kernels
    g = torch.Generator().manual_seed(7)
    for rows, cols in ((1, 1), (3, 17), (64, 151936), (5, 4097)):
        x = torch.randn(rows, cols, generator=g).to(dtype).to(dev)
        assert torch.equal(kernels.argmax_rows(x), x.argmax(dim=-1))
    x = torch.randn(8, 5000, generator=g).to(dtype).to(dev)
    x[0] = 1.5                      # all equal: index 0
    x[1, 4000:] = 99.0              # a plateau: its first element
    x[2] = float("-inf")            # nothing beats the first element
    x[3, 777] = float("nan")        # NaN is the maximum
    x[4, 12] = float("nan"); x[4, 4900] = float("nan")
    want = x.argmax(dim=-1)
    assert want[:5].tolist() == [0, 4000, 0, 777, 12]
    assert torch.equal(kernels.argmax_rows(x), want)
    wide = torch.randn(6, 9000, generator=g).to(dtype).to(dev)
    view = wide[:, :7001]           # row stride 9000, 7001 columns
    out = torch.empty(6, dtype=torch.int64, device=dev)
    ws = torch.empty(kernels.argmax_workspace_bytes(6), dtype=torch.uint8, device=dev)
    assert kernels.argmax_rows(view, out=out, workspace=ws) is out
    assert torch.equal(out, view.argmax(dim=-1))
    with pytest.raises(ValueError):
        kernels.argmax_rows(wide.t())
