"""The CPU oracle against outputs of the reference itself (tests/golden/, made by make_golden.py).

The cases restate what the reference's own tests cover: packing round trips and known answers
(tests/test_packing.py:26-98), LIF incl. the threshold-boundary stress (tests/test_lif_kernel.py),
paged attention over scrambled tables, ragged lengths, GQA ratios and head dims
(tests/test_spike_attention.py, tests/test_cpu_backend.py), the slot walk and the allocator.
"""
from __future__ import annotations

import pytest
import torch

import cases
from oracle import torch_oracle as orc


# ------------------------------------------------------------------ packing
@pytest.mark.parametrize("channels", cases.PACK_CHANNELS)
def test_pack_matches_reference(channels, golden):
    g = golden("packing")[channels]
    x = cases.pack_case(channels)
    assert cases.digest(x) == g["digest"], "seeded inputs differ from the ones the fixture was made with"
    words = orc.pack_spikes(x)
    assert words.dtype == torch.int32 and words.shape == (3, 5, orc.packed_width(channels))
    assert torch.equal(words, g["words"])
    assert torch.equal(orc.unpack_spikes(words, channels), x)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.uint8])
def test_pack_roundtrip_dtypes(dtype):
    x = cases.pack_case(63).to(dtype)
    assert torch.equal(orc.unpack_spikes(orc.pack_spikes(x), 63, dtype), x)


def test_pack_known_answers(golden):
    g = golden("packing")
    assert orc.pack_spikes(torch.ones(1, 32)).item() == -1 == g["all_ones_32"].item()
    assert torch.equal(orc.pack_spikes(torch.ones(1, 33)), g["tail_33"])
    assert int(orc.pack_spikes(torch.ones(1, 33))[0, 1]) == 1
    assert torch.equal(orc.pack_spikes(torch.tensor([[0.0, 0.5, 0.0, 2.0]])), g["graded"])
    for ch in (0, 1, 31, 32, 63):
        x = torch.zeros(1, 64)
        x[0, ch] = 1
        w = orc.pack_spikes(x)[0]
        assert (int(w[ch // 32]) & 0xFFFFFFFF) == 1 << (ch % 32) and int(w[1 - ch // 32]) == 0
    assert orc.packed_bytes_per_token(24, 4, 2, 64) == 3072 == g["bytes_per_token_0p5b"]
    with pytest.raises(ValueError, match="expected 4 words"):
        orc.unpack_spikes(orc.pack_spikes(torch.ones(1, 64)), 128)


# ------------------------------------------------------------------ LIF
@pytest.mark.parametrize("name", list(cases.LIF_CASES) + ["boundary"])
def test_lif_matches_reference(name, golden):
    g = golden("lif")[name]
    c = cases.lif_boundary_case() if name == "boundary" else cases.lif_case(**cases.LIF_CASES[name])
    assert cases.digest(c["x"].float(), c["beta"], c["threshold"]) == g["digest"]
    spikes, mem = orc.lif_multistep(c["x"], c["beta"], c["threshold"], mem0=c["mem0"], out_dtype=torch.uint8)
    assert torch.equal(orc.pack_spikes(spikes), g["packed"])
    assert torch.equal(mem, g["membrane"])


def test_lif_hard_zero_definition():
    # parity unpinned: the reference has no hard reset; this pins the oracle's own definition.
    x = torch.tensor([[[0.6]], [[0.6]], [[0.1]], [[2.0]]])
    s, u = orc.lif_multistep(x, torch.tensor([1.0]), torch.tensor([1.0]), reset_mode=orc.HARD_ZERO)
    assert s.flatten().tolist() == [0.0, 1.0, 0.0, 1.0]
    assert u.item() == 0.0


# ------------------------------------------------------------------ attention
@pytest.mark.parametrize("name", list(cases.ATTENTION_CASES))
def test_attention_matches_reference(name, golden):
    g = golden("attention")[name]
    case = cases.attention_case(**cases.ATTENTION_CASES[name])
    assert cases.digest(case["q_packed"], case["k_cache"], case["v_cache"], case["block_tables"]) == g["digest"]
    got = orc.paged_spike_attn_decode(**case)
    torch.testing.assert_close(got, g["out_ref"], rtol=1e-5, atol=1e-6)
    fast = orc.paged_spike_attn_decode_batched(**case)
    torch.testing.assert_close(fast, g["out_ref"], rtol=1e-5, atol=1e-6)


def test_scores_are_exact_integers():
    """popc(q & k) on packed words equals the dense dot product exactly (tests/test_cpu_backend.py:165-181)."""
    case = cases.attention_case(**cases.ATTENTION_CASES["ragged"])
    s = orc.qk_scores(**{k: case[k] for k in ("q_packed", "k_cache", "block_tables", "seq_lens", "head_dim",
                                             "block_size", "num_q_heads", "num_kv_heads")})
    for i, length in enumerate(case["seq_lens"].tolist()):
        q = orc.unpack_spikes(case["q_packed"][:, i], 64)
        k = orc.gather_kv_unpacked(case["k_cache"], case["block_tables"][i], length, 64, 16).repeat_interleave(7, 1)
        dense = torch.einsum("thd,thsd->ths", q, k)
        assert torch.equal(dense.to(torch.int32), s[:, i, :, :length])
        assert (s[:, i, :, length:] == -1).all()
    assert s.max() <= 64


def test_gather_and_slot_walk(golden):
    g = golden("attention")
    case = cases.attention_case(**cases.ATTENTION_CASES["ragged"])
    got = orc.gather_kv_unpacked(case["k_cache"], case["block_tables"][3], 97, 64, 16)
    assert torch.equal(got.to(torch.uint8), g["gather_ragged_3"])
    tables = torch.tensor([[3, 1, 7], [5, 2, 0]], dtype=torch.int32)
    assert torch.equal(orc.slot_matrix(tables, 10, 4), g["slot_matrix"])
    assert orc.slot_matrix(tables, 10, 4).tolist() == [
        [12, 13, 14, 15, 4, 5, 6, 7, 28, 29],
        [20, 21, 22, 23, 8, 9, 10, 11, 0, 1],
    ]


def test_attention_isolation_and_padding_tail():
    """Unowned blocks and the tail of the last block never influence the output."""
    case = cases.attention_case(seq_lens=[9, 25, 41, 3])
    before = orc.paged_spike_attn_decode(**case)
    bs = case["block_size"]
    owned = set()
    for i, length in enumerate(case["seq_lens"].tolist()):
        owned.update(case["block_tables"][i, : (length + bs - 1) // bs].tolist())
    for blk in range(case["k_cache"].shape[2] // bs):
        if blk not in owned:
            case["k_cache"][:, :, blk * bs:(blk + 1) * bs] = -1
            case["v_cache"][:, :, blk * bs:(blk + 1) * bs] = -1
    for i, length in enumerate(case["seq_lens"].tolist()):
        if length % bs:
            last = int(case["block_tables"][i, (length - 1) // bs])
            case["k_cache"][:, :, last * bs + length % bs:(last + 1) * bs] = -1
            case["v_cache"][:, :, last * bs + length % bs:(last + 1) * bs] = -1
    assert torch.equal(orc.paged_spike_attn_decode(**case), before)


# ------------------------------------------------------------------ allocator
def test_block_manager_trace(golden):
    g = golden("block_manager")
    mgr = orc.BlockManager(12, 4)
    tables = [[], [], []]
    computed = [0, 0, 0]
    trace = g["trace"]
    ok = [mgr.allocate(t, 0, n) for t, n in zip(tables, (5, 9, 2))]
    computed = [5, 9, 2]
    assert ok == trace[0]["ok"] and tables == trace[0]["tables"] and mgr.free_list == trace[0]["free"]
    for step in range(6):
        ok = [mgr.allocate(t, c, 1) for t, c in zip(tables, computed)]
        slots = [mgr.slot_mapping(t, c, 1)[0] for t, c in zip(tables, computed)]
        computed = [c + 1 for c in computed]
        ref = trace[1 + step]
        assert ok == ref["ok"] and tables == ref["tables"] and slots == ref["slots"] and mgr.free_list == ref["free"]
        pos, slot_t, bt, lens = orc.prepare_decode(tables, [c - 1 for c in computed], 8, 11, 4)
        assert slot_t.tolist() == slots and lens.tolist() == computed
    mgr.free(tables[1])
    assert tables == trace[7]["tables"] and mgr.free_list == trace[7]["free"]
    assert mgr.allocate(tables[1], computed[1], 6) == trace[8]["ok"]  # preempted row re-grows to 21 tokens
    assert tables == trace[8]["tables"] and mgr.free_list == trace[8]["free"]
    table = [5, 2, 7]
    known = [orc.BlockManager(8, 4).slot_mapping(table, a, b) for a, b in ((0, 4), (4, 4), (8, 2), (3, 3))]
    assert known == g["slot_known"] == [[20, 21, 22, 23], [8, 9, 10, 11], [28, 29], [23, 8, 9]]
