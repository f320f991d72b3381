"""Host-side behaviour of the operator wrappers that needs no GPU: shapes, errors, and that a CPU
tensor is refused loudly (there is no CPU path in the product)."""
from __future__ import annotations

import pytest
import torch

from spikeinfer_b200 import _lib, kernels
from spikeinfer_b200.kernels.packing import _leading_dims


@pytest.mark.parametrize("channels", [1, 31, 32, 33, 63, 64, 128, 4864])
def test_packed_width(channels):
    assert kernels.packed_width(channels) == (channels + 31) // 32


def test_packed_bytes_per_token():
    assert kernels.packed_bytes_per_token(24, 4, 2, 64) == 3072
    assert kernels.BITS_PER_WORD == 32


def test_leading_dims_merge_and_drop():
    x = torch.empty(4, 1, 14, 8, 64)
    assert _leading_dims(x) == ([4 * 14 * 8], [64])
    y = x.permute(0, 1, 3, 2, 4)  # [4,1,8,14,64], strided
    assert _leading_dims(y) == ([4, 8, 14], [14 * 8 * 64, 64, 8 * 64])
    assert _leading_dims(y, first=1) == ([8, 14], [64, 8 * 64])


def test_cpu_tensors_are_refused(lib):
    x = torch.ones(2, 64)
    with pytest.raises(_lib.SpkError, match="no CPU path"):
        kernels.pack_spikes(x)
    with pytest.raises(_lib.SpkError, match="no CPU path"):
        kernels.unpack_spikes(torch.zeros(2, 2, dtype=torch.int32), 64)
    with pytest.raises(_lib.SpkError, match="no CPU path"):
        kernels.lif_multistep(torch.zeros(4, 2, 64), torch.ones(64), torch.ones(64))
    q = torch.zeros(4, 1, 14, 2, dtype=torch.int32)
    c = torch.zeros(4, 2, 64, 2, dtype=torch.int32)
    with pytest.raises(_lib.SpkError, match="no CPU path"):
        kernels.paged_spike_attn_decode(q, c, c, torch.zeros(1, 4, dtype=torch.int32),
                                        torch.ones(1, dtype=torch.int32), 64, 16, 14, 2)


def test_reference_error_behaviour():
    q = torch.zeros(4, 1, 14, 2, dtype=torch.int32)
    c = torch.zeros(4, 2, 64, 2, dtype=torch.int32)
    t = torch.zeros(1, 4, dtype=torch.int32)
    n = torch.ones(1, dtype=torch.int32)
    with pytest.raises(ValueError, match="q has 2 words, expected 4"):
        kernels.paged_spike_attn_decode(q, c, c, t, n, 128, 16, 14, 2)
    with pytest.raises(ValueError, match="q has 14 heads, expected 7"):
        kernels.paged_spike_attn_decode(q, c, c, t, n, 64, 16, 7, 1)
    with pytest.raises(ValueError, match="expected 4 words"):
        kernels.unpack_spikes(torch.zeros(1, 2, dtype=torch.int32), 128)
    with pytest.raises(AssertionError):
        kernels.lif_multistep(torch.zeros(4), torch.ones(1), torch.ones(1))
    with pytest.raises(AssertionError, match="beta/threshold must match"):
        kernels.lif_multistep(torch.zeros(4, 2, 64), torch.ones(63), torch.ones(64))


def test_validate_thresholds():
    class Lif(torch.nn.Module):
        def __init__(self, th):
            super().__init__()
            self.threshold = torch.nn.Parameter(torch.tensor(th))
            self.beta = torch.nn.Parameter(torch.tensor([0.9] * len(th)))

    class Site(torch.nn.Module):
        def __init__(self, th):
            super().__init__()
            self.lif = Lif(th)

    good = torch.nn.Sequential(Site([0.5, 1.0]), Site([0.1, 0.2]))
    assert kernels.validate_thresholds(good) is True
    bad = torch.nn.Sequential(Site([0.5, 1.0]), Site([0.0, 0.2]))
    with pytest.raises(ValueError, match="threshold > 0"):
        kernels.validate_thresholds(bad)


def test_build_prefill_rows_turns_chunks_into_decode_rows():
    """Every prefill token becomes a decode row of length context + index + 1 over its sequence's table."""
    from spikeinfer_b200.attention import AttentionMetadata, build_prefill_rows
    meta = AttentionMetadata(
        slot_mapping=torch.zeros(1 + 3 + 2, dtype=torch.int64), block_size=4, num_decode_tokens=1,
        prefill_query_starts=[1, 4], prefill_query_lens=[3, 2], prefill_context_lens=[0, 5],
        prefill_block_tables=[torch.tensor([7], dtype=torch.int32), torch.tensor([2, 9], dtype=torch.int32)])
    build_prefill_rows(meta, pad_block=31)
    assert meta.prefill_row_lens.tolist() == [1, 2, 3, 6, 7]
    assert meta.prefill_row_tables.tolist() == [[7, 31]] * 3 + [[2, 9]] * 2
    assert meta.prefill_row_tables.dtype == torch.int32 and meta.prefill_row_tables.is_contiguous()
    # chunks out of place, or a table too short for the context, are refused
    bad = AttentionMetadata(slot_mapping=torch.zeros(3, dtype=torch.int64), block_size=4, num_decode_tokens=0,
                            prefill_query_starts=[1], prefill_query_lens=[2], prefill_context_lens=[0],
                            prefill_block_tables=[torch.tensor([0], dtype=torch.int32)])
    with pytest.raises(ValueError):
        build_prefill_rows(bad)
    short = AttentionMetadata(slot_mapping=torch.zeros(2, dtype=torch.int64), block_size=4, num_decode_tokens=0,
                              prefill_query_starts=[0], prefill_query_lens=[2], prefill_context_lens=[7],
                              prefill_block_tables=[torch.tensor([0, 1], dtype=torch.int32)])
    with pytest.raises(ValueError):
        build_prefill_rows(short)
    # no prefill chunks: nothing to do
    none = AttentionMetadata(slot_mapping=torch.zeros(1, dtype=torch.int64), block_size=4, num_decode_tokens=1)
    assert build_prefill_rows(none).prefill_row_tables is None


def test_block_ledger_counts_follow_the_allocation_rules():
    """The host ledger moves as many blocks as the device does: ceil(len / bs) at admission, one per row on a
    page boundary per step (row order, none when the list is empty or the table is full), all back at release."""
    from spikeinfer_b200.engine.block_ledger import BlockLedger
    led = BlockLedger(num_alloc_blocks=6, block_size=4, max_blocks_per_seq=3)
    assert led.admission_error([5, 4]) is None
    assert "exceeds max_model_len" in led.admission_error([13])
    assert "need 7 blocks" in led.admission_error([12, 12, 4])
    assert "empty prompt" in led.admission_error([0])
    led.admit(0, 5)   # 2 blocks
    led.admit(1, 4)   # 1 block, sits on a boundary
    assert led.free == 3 and led.blocks_next_step() == 1
    led.advance()     # row 1 pops a block
    assert led.free == 2 and led.seq_lens == {0: 6, 1: 5}
    for _ in range(2):
        led.advance()
    assert led.seq_lens == {0: 8, 1: 7} and led.free == 2
    led.advance()     # row 0 crosses into its third block
    assert led.free == 1 and led.seq_lens == {0: 9, 1: 8}
    led.advance()     # row 1 too
    assert led.free == 0
    for _ in range(3):
        led.advance()
    assert led.seq_lens == {0: 12, 1: 12}
    led.advance()     # both tables full: nobody moves, nothing is popped
    assert led.seq_lens == {0: 12, 1: 12} and led.free == 0
    with pytest.raises(RuntimeError):
        led.admit(0, 1)
    led.release(0)
    assert led.free == 3 and 0 not in led.seq_lens
    # an empty list parks the row that needs a block, as the device does
    led2 = BlockLedger(num_alloc_blocks=1, block_size=2, max_blocks_per_seq=4)
    led2.admit(3, 2)
    led2.advance()
    assert led2.seq_lens[3] == 2 and led2.free == 0


def test_row_buckets_and_the_covering_bucket():
    from spikeinfer_b200.engine.block_ledger import covering_bucket, row_buckets

    assert row_buckets(1) == [1]
    assert row_buckets(8) == [1, 2, 4, 8]
    assert row_buckets(48) == [1, 2, 4, 8, 16, 32, 48]
    assert row_buckets(64) == [1, 2, 4, 8, 16, 32, 64]
    b = row_buckets(48)
    assert covering_bucket(b, []) == 1                  # an idle engine runs the smallest graph
    assert covering_bucket(b, [0]) == 1
    assert covering_bucket(b, [0, 1]) == 2
    assert covering_bucket(b, [5]) == 8                 # the highest row in use decides, not the count
    assert covering_bucket(b, {0: 10, 32: 7}) == 48     # dict of row -> length, as the ledger keeps it
    assert covering_bucket(b, range(48)) == 48
    assert covering_bucket([48], [0]) == 48             # buckets switched off
    with pytest.raises(ValueError):
        row_buckets(0)
