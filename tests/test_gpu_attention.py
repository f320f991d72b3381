"""GPU parity: paged popcount decode attention against the CPU oracle and the golden fixtures.

Scores are compared exactly (integers); attention outputs to the reference's own bar for its
kernel, 1e-5 of the largest magnitude in fp32 (tests/test_spike_attention.py:28,74-78), and to 1e-3
for bf16 output.  Isolation and padding-tail checks are bit-exact, as in the reference.
"""
from __future__ import annotations

import pytest
import torch

import cases
from conftest import to_dev
from oracle import torch_oracle as orc
from spikeinfer_b200 import _lib, kernels

pytestmark = pytest.mark.gpu

REL_TOL = 1e-5  # fp32 output, max-norm relative
REL_TOL_BF16 = 1e-3  # bf16 output vs the oracle rounded to bf16, plus one bf16 ulp of rounding slack


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    scale = want.abs().max().clamp(min=1e-6)
    return ((got.float() - want.float()).abs().max() / scale).item()


def within_bf16_bar(got16: torch.Tensor, want: torch.Tensor) -> bool:
    """16-bit output: within 1e-3 of the largest magnitude before rounding, plus the rounding to bf16 itself
    (half a step of the value, 2^-9 relative; 2^-8 allows the step a 1e-3 difference can push a value over)."""
    scale = want.abs().max().clamp(min=1e-6)
    return bool(((got16.float() - want).abs() <= REL_TOL_BF16 * scale + want.abs() * 2.0 ** -8).all())


def run(case, dev, **kw):
    return kernels.paged_spike_attn_decode(**to_dev(case, dev), **kw)


@pytest.mark.parametrize("name", list(cases.ATTENTION_CASES))
def test_matches_oracle_and_golden(name, dev, golden):
    case = cases.attention_case(**cases.ATTENTION_CASES[name])
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    got = run(case, dev, status=status).cpu()
    assert torch.isfinite(got).all()
    want = orc.paged_spike_attn_decode(**case)
    assert rel_err(got, want) < REL_TOL, f"vs oracle: {rel_err(got, want):.2e}"
    assert rel_err(got, golden("attention")[name]["out_ref"]) < REL_TOL
    assert status.item() == 0


@pytest.mark.parametrize("block_size", [1, 2, 8, 16, 32, 64, 128])
def test_block_sizes(block_size, dev):
    case = cases.attention_case(seq_lens=[1, 5, 40, 97, 130], block_size=block_size, seed=block_size)
    assert rel_err(run(case, dev).cpu(), orc.paged_spike_attn_decode(**case)) < REL_TOL


def test_scores_are_exact(dev):
    for name in ("ragged", "d128_gqa7", "d96", "long_split"):
        case = cases.attention_case(**cases.ATTENTION_CASES[name])
        keys = ("q_packed", "k_cache", "block_tables", "seq_lens", "head_dim", "block_size", "num_q_heads", "num_kv_heads")
        want = orc.qk_scores(**{k: case[k] for k in keys})
        got = kernels.qk_scores(**to_dev({k: case[k] for k in keys}, dev))
        assert torch.equal(got.cpu(), want), name


def test_all_zero_query_gives_the_mean_of_the_values(dev):
    case = cases.attention_case(seq_lens=[40, 17, 5], block_size=32)
    case["q_packed"] = torch.zeros_like(case["q_packed"])
    got = run(case, dev).cpu()
    assert torch.isfinite(got).all()
    assert rel_err(got, orc.paged_spike_attn_decode(**case)) < REL_TOL
    v = orc.gather_kv_unpacked(case["v_cache"], case["block_tables"][1], 17, 64, 32)  # [T, Hkv, 17, D]
    torch.testing.assert_close(got[:, 1, 0], v[:, 0].mean(dim=1), rtol=1e-5, atol=1e-6)


def test_all_ones_query_and_keys(dev):
    """Largest possible scores (64) everywhere: the fixed softmax bound must not overflow or lose weight."""
    case = cases.attention_case(seq_lens=[33, 2], head_dim=128, num_q_heads=7, num_kv_heads=1)
    case["q_packed"] = torch.full_like(case["q_packed"], -1)
    got = run(case, dev).cpu()
    assert rel_err(got, orc.paged_spike_attn_decode(**case)) < REL_TOL
    case["k_cache"] = torch.full_like(case["k_cache"], -1)
    got = run(case, dev).cpu()
    assert rel_err(got, orc.paged_spike_attn_decode(**case)) < REL_TOL


def test_only_owned_blocks_and_valid_positions_are_read(dev):
    case = cases.attention_case(seq_lens=[9, 25, 41, 3, 600], max_blocks=64)
    d = to_dev(case, dev)
    before = kernels.paged_spike_attn_decode(**d).clone()
    bs = case["block_size"]
    owned = set()
    for i, length in enumerate(case["seq_lens"].tolist()):
        owned.update(case["block_tables"][i, : (length + bs - 1) // bs].tolist())
    for blk in range(case["k_cache"].shape[2] // bs):
        if blk not in owned:
            d["k_cache"][:, :, blk * bs:(blk + 1) * bs] = -1
            d["v_cache"][:, :, blk * bs:(blk + 1) * bs] = -1
    for i, length in enumerate(case["seq_lens"].tolist()):
        if length % bs:
            last = int(case["block_tables"][i, (length - 1) // bs])
            d["k_cache"][:, :, last * bs + length % bs:(last + 1) * bs] = -1
            d["v_cache"][:, :, last * bs + length % bs:(last + 1) * bs] = -1
    after = kernels.paged_spike_attn_decode(**d)
    assert torch.equal(before, after), "attention read outside the sequence's blocks or past seq_len"


def test_out_argument_strided_view_and_dtypes(dev):
    """The engine passes out=buf[:, :n_dec] (attention.py:157): a strided view in the model dtype."""
    case = cases.attention_case(seq_lens=[1, 5, 40, 97])
    want = orc.paged_spike_attn_decode(**case)
    for dtype, tol in ((torch.float32, REL_TOL), (torch.bfloat16, None), (torch.float16, 1e-3)):
        buf = torch.full((4, 9, 14, 64), 7.0, dtype=dtype, device=dev)
        ret = run(case, dev, out=buf[:, :4])
        assert ret.data_ptr() == buf.data_ptr()
        assert (buf[:, 4:] == 7.0).all(), "wrote past the requested rows"
        got = buf[:, :4].cpu()
        if dtype == torch.bfloat16:
            # within 1e-3 of the fp32 result before rounding => at most one bf16 step from the rounded oracle
            w16 = want.to(torch.bfloat16).float()
            ulp = torch.maximum(w16.abs() * 2.0 ** -7, torch.tensor(1e-30))
            assert ((got.float() - w16).abs() <= ulp).all()
            assert rel_err(got, want) < 2.0 ** -8 + REL_TOL_BF16
        else:
            assert rel_err(got, want) < tol
    assert run(case, dev, dtype=torch.bfloat16).dtype == torch.bfloat16


def test_strided_pool_views(dev):
    """K and V living interleaved in one buffer ([T, H, slots, 2, W]) are addressed through strides."""
    case = cases.attention_case(seq_lens=[30, 7, 70])
    want = orc.paged_spike_attn_decode(**case)
    d = to_dev(case, dev)
    both = torch.stack([d["k_cache"], d["v_cache"]], dim=3).contiguous()  # [T, H, slots, 2, W]
    d["k_cache"], d["v_cache"] = both[:, :, :, 0], both[:, :, :, 1]
    assert not d["k_cache"].is_contiguous()
    assert rel_err(kernels.paged_spike_attn_decode(**d).cpu(), want) < REL_TOL
    # page-major pool with an explicit block axis: [blocks, T, H, 2, bs, W] viewed as [T, H, blocks, bs, W]
    bs = case["block_size"]
    nb = case["k_cache"].shape[2] // bs
    pm = torch.empty(nb, 4, 2, 2, bs, 2, dtype=torch.int32, device=dev)
    pm[:, :, :, 0] = to_dev(case, dev)["k_cache"].view(4, 2, nb, bs, 2).permute(2, 0, 1, 3, 4)
    pm[:, :, :, 1] = to_dev(case, dev)["v_cache"].view(4, 2, nb, bs, 2).permute(2, 0, 1, 3, 4)
    d["k_cache"] = pm[:, :, :, 0].permute(1, 2, 0, 3, 4)
    d["v_cache"] = pm[:, :, :, 1].permute(1, 2, 0, 3, 4)
    assert rel_err(kernels.paged_spike_attn_decode(**d).cpu(), want) < REL_TOL


def test_corrupt_metadata_is_flagged_not_followed(dev):
    """Host-side fault injection: a block id outside the pool and a bad length set status bits; the
    kernel skips the access instead of reading out of bounds."""
    case = cases.attention_case(seq_lens=[20, 40])
    d = to_dev(case, dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    d["block_tables"] = d["block_tables"].clone()
    d["block_tables"][1, 1] = 10_000
    out = kernels.paged_spike_attn_decode(**d, status=status)
    assert status.item() & _lib.STATUS_BAD_BLOCK
    assert torch.isfinite(out).all()
    ok = orc.paged_spike_attn_decode(**case)
    assert rel_err(out[:, 0].cpu(), ok[:, 0]) < REL_TOL  # the healthy row is unaffected
    status.zero_()
    d = to_dev(case, dev)
    d["seq_lens"] = torch.tensor([0, 10_000], dtype=torch.int32, device=dev)
    out = kernels.paged_spike_attn_decode(**d, status=status)
    assert status.item() & _lib.STATUS_BAD_SEQ_LEN
    assert torch.isfinite(out).all() and (out[:, 0] == 0).all()


def test_gather_kv_unpacked(dev, golden):
    case = cases.attention_case(**cases.ATTENTION_CASES["ragged"])
    d = to_dev(case, dev)
    got = kernels.gather_kv_unpacked(d["k_cache"], d["block_tables"][3], 97, 64, 16, torch.float32)
    assert torch.equal(got.cpu().to(torch.uint8), golden("attention")["gather_ragged_3"])
    got = kernels.gather_kv_unpacked(d["v_cache"], d["block_tables"][2], 40, 64, 16, torch.bfloat16)
    want = orc.gather_kv_unpacked(case["v_cache"], case["block_tables"][2], 40, 64, 16, torch.bfloat16)
    assert torch.equal(got.cpu(), want)


@pytest.mark.parametrize("seed", range(16))
def test_random_batches_through_every_work_split(seed, dev):
    """Seeded random batches that land in every way the streaming form splits work: nothing cut and a warp per item
    (tables of up to 768 keys), nothing cut but more items than resident warps, equal step ranges with cut rows and
    the combine pass, and more than 1024 rows (one warp per unit); ragged lengths down to 1, head_dim 64 and 128,
    several GQA ratios and timestep counts, fp32 against the oracle at 1e-5 and bf16 within the 16-bit bar, and the
    same through the overlapped launch."""
    g = cases.gen(1000 + seed)
    pick = lambda xs: xs[int(torch.randint(0, len(xs), (1,), generator=g))]
    head_dim = pick([64, 64, 128])
    hq, hkv = pick([(14, 2), (7, 1), (4, 2), (8, 8), (16, 2), (28, 4)])
    T = pick([1, 4, 4, 8])
    kind = seed % 4
    if kind == 0:      # short tables: nothing is cut, one warp per item
        n, hi, max_blocks = pick([1, 5, 64]), pick([40, 200, 700]), 48
    elif kind == 1:    # short tables, many rows: more items than resident warps
        n, hi, max_blocks = 700, 90, 8
    elif kind == 2:    # long tables: equal step ranges, cut rows, combine pass
        n, hi, max_blocks = pick([2, 9, 24]), pick([900, 2500]), 256
    else:              # beyond 1024 rows: the unit form
        n, hi, max_blocks = 1100, 70, 64
    lens = torch.randint(1, hi + 1, (n,), generator=g).tolist()
    if n > 3:
        lens[0], lens[-1] = hi, 1
    case = cases.attention_case(seq_lens=lens, head_dim=head_dim, num_q_heads=hq, num_kv_heads=hkv, T=T,
                                density=pick([0.1, 0.3]), seed=2000 + seed, max_blocks=max_blocks)
    d = to_dev(case, dev)
    want = orc.paged_spike_attn_decode(**case)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    got = kernels.paged_spike_attn_decode(**d, status=status)
    assert rel_err(got.cpu(), want) < REL_TOL, f"fp32: {rel_err(got.cpu(), want):.2e}"
    got16 = kernels.paged_spike_attn_decode(**d, dtype=torch.bfloat16, status=status)
    assert within_bf16_bar(got16.cpu(), want)
    again = kernels.paged_spike_attn_decode(**d, status=status, overlap_previous=True)
    assert torch.equal(again, got)
    assert status.item() == 0


def test_gather_kv_unpacked_batch_equals_the_per_sequence_read(dev):
    case = cases.attention_case(seq_lens=[40, 97, 64, 130, 40], seed=12)
    d = to_dev(case, dev)
    for cache in ("k_cache", "v_cache"):
        for dtype in (torch.float32, torch.bfloat16):
            got = kernels.gather_kv_unpacked_batch(d[cache], d["block_tables"][[0, 4, 2]], 40, 64, 16, dtype)
            assert got.shape == (3, 4, 2, 40, 64)
            for b, row in enumerate((0, 4, 2)):
                want = orc.gather_kv_unpacked(case[cache], case["block_tables"][row], 40, 64, 16, dtype)
                assert torch.equal(got[b].cpu(), want)
    # a strided view of the tables (row stride above the width) and an empty batch
    wide = d["block_tables"][:, :3]
    got = kernels.gather_kv_unpacked_batch(d["k_cache"], wide, 40, 64, 16, torch.float32)
    assert torch.equal(got[1].cpu(), orc.gather_kv_unpacked(case["k_cache"], case["block_tables"][1], 40, 64, 16, torch.float32))
    assert kernels.gather_kv_unpacked_batch(d["k_cache"], wide[:0], 40, 64, 16, torch.float32).shape[0] == 0
    with pytest.raises(ValueError):
        kernels.gather_kv_unpacked_batch(d["k_cache"], wide, 64, 64, 16, torch.float32)  # 3 pages hold 48 keys


def config2_case(seed=2, n=64, lo=128, hi=4096):
    g = cases.gen(seed)
    lens = torch.randint(lo, hi + 1, (n,), generator=g).tolist()
    return cases.attention_case(seq_lens=lens, density=0.2, seed=seed, spare_blocks=0, max_blocks=hi // 16)


def test_config2_full_size(dev):
    """The kernel-level attention configuration: 64 ragged sequences in [128, 4096], 14/2 heads, D 64, T 4, Bernoulli(0.2) bits,
    16-token pages in a shuffled pool.  fp32 vs the oracle at 1e-5; bf16 within 1e-3; scores exact on a sample;
    and linearity in V as a size-independent property (out(V1 | V2) = out(V1) + out(V2) for disjoint V bits)."""
    case = config2_case()
    d = to_dev(case, dev)
    got = kernels.paged_spike_attn_decode(**d)
    want = orc.paged_spike_attn_decode(**case)
    assert rel_err(got.cpu(), want) < REL_TOL
    got16 = kernels.paged_spike_attn_decode(**d, dtype=torch.bfloat16).cpu()
    assert within_bf16_bar(got16, want)
    mask = torch.tensor([0x0F0F0F0F, 0x33333333], dtype=torch.int32, device=dev)
    d1, d2 = dict(d), dict(d)
    d1["v_cache"] = d["v_cache"] & mask
    d2["v_cache"] = d["v_cache"] & ~mask
    o1, o2 = kernels.paged_spike_attn_decode(**d1), kernels.paged_spike_attn_decode(**d2)
    torch.testing.assert_close(o1 + o2, got, rtol=1e-5, atol=1e-6)
    keys = ("q_packed", "k_cache", "block_tables", "seq_lens", "head_dim", "block_size", "num_q_heads", "num_kv_heads")
    sub = {k: (case[k][:, :4] if k == "q_packed" else case[k][:4] if k in ("block_tables", "seq_lens") else case[k]) for k in keys}
    assert torch.equal(kernels.qk_scores(**to_dev(sub, dev)).cpu(), orc.qk_scores(**sub))


def test_launches_that_overlap_their_predecessor_give_the_same_results(dev):
    """overlap_previous lets a call's prologue run under the launch before it (here: the previous call's combine
    pass, and a kernel that rewrites q).  Lengths and tables are fixed, everything else changes from call to call:
    q is produced by the kernel just before each call, pools and outputs alternate, and the calls share one
    workspace address (the caching allocator hands the same block back).  Every result must equal the one the
    ordinary launch gives, bit for bit."""
    specs = [dict(seq_lens=[700, 130, 1, 1500, 64, 2047], max_blocks=128, seed=41),
             dict(seq_lens=[700, 130, 1, 1500, 64, 2047], max_blocks=128, seed=42, density=0.4)]
    data = [to_dev(cases.attention_case(**s), dev) for s in specs]
    for d in data:
        d["block_tables"], d["seq_lens"] = data[0]["block_tables"], data[0]["seq_lens"]
    want = [kernels.paged_spike_attn_decode(**d) for d in data]
    want16 = [kernels.paged_spike_attn_decode(**d, dtype=torch.bfloat16) for d in data]
    torch.cuda.synchronize(dev)
    for rounds in range(3):
        outs, outs16 = [], []
        for i in range(6):
            d = dict(data[i % 2])
            d["q_packed"] = d["q_packed"] | 0  # q comes out of the kernel launched just before the attention
            outs.append(kernels.paged_spike_attn_decode(**d, overlap_previous=True))
            d["q_packed"] = d["q_packed"] | 0
            outs16.append(kernels.paged_spike_attn_decode(**d, dtype=torch.bfloat16, overlap_previous=True))
        for i in range(6):
            assert torch.equal(outs[i], want[i % 2]) and torch.equal(outs16[i], want16[i % 2])
    # a short batch (no row is cut, no combine pass) behind a kernel that writes q
    short = to_dev(cases.attention_case(seq_lens=[5, 130, 200, 17], max_blocks=16, seed=43), dev)
    ref = kernels.paged_spike_attn_decode(**short)
    for _ in range(4):
        d = dict(short)
        d["q_packed"] = d["q_packed"] | 0
        assert torch.equal(kernels.paged_spike_attn_decode(**d, overlap_previous=True), ref)


def test_general_form_still_serves_every_layout(dev, lib):
    """With the streaming form switched off, the general form takes the same calls (it is what small pages, odd
    strides and head_dim 32 / 96 use): the kernel-level attention configuration against the oracle."""
    assert lib.spk_attn_select_form(_lib.ATTN_FORM_GENERAL) == 0
    try:
        case = config2_case(n=16)
        got = kernels.paged_spike_attn_decode(**to_dev(case, dev)).cpu()
        assert rel_err(got, orc.paged_spike_attn_decode(**case)) < REL_TOL
    finally:
        assert lib.spk_attn_select_form(_lib.ATTN_FORM_AUTO) == 0


def attention_fp64(case):
    """The same softmax-weighted sum in float64 from the unpacked bits: the yardstick for rows so long that the
    fp32 oracle's own rounding (3.8e-5 at 32768 keys) is above the bar."""
    D, Hq, Hkv = case["head_dim"], case["num_q_heads"], case["num_kv_heads"]
    q = orc.unpack_spikes(case["q_packed"], D, torch.float64)  # [T, n, Hq, D]
    T, n_seqs = q.shape[:2]
    out = torch.zeros(q.shape, dtype=torch.float64)
    for n in range(n_seqs):
        length = int(case["seq_lens"][n])
        k = orc.gather_kv_unpacked(case["k_cache"], case["block_tables"][n], length, D, case["block_size"], torch.float64)
        v = orc.gather_kv_unpacked(case["v_cache"], case["block_tables"][n], length, D, case["block_size"], torch.float64)
        qg = q[:, n].view(T, Hkv, Hq // Hkv, D)  # the query heads of a group share their K/V head
        s = torch.einsum("tgrd,tgld->tgrl", qg, k) * D ** -0.5
        out[:, n] = torch.einsum("tgrl,tgld->tgrd", torch.softmax(s, -1), v).reshape(T, Hq, D)
    return out


def test_long_context_shard_shape(dev):
    """The attention of one tensor-parallel shard of the 7B-shape long-context configuration: head_dim 128, 7 query
    heads on 1 KV head, T = 4, a dozen rows with lengths log-uniform in [1k, 32k] plus one of 32768, 16-token pages.
    Rows are cut between many warps and combined.  fp32 output against float64 < 2e-6; bf16 output within 1e-3."""
    import math
    g = cases.gen(55)
    lo, hi = math.log(1024.0), math.log(32768.0)
    lens = torch.exp(torch.rand(11, generator=g) * (hi - lo) + lo).long().clamp(1024, 32768).tolist() + [32768]
    case = cases.attention_case(seq_lens=lens, density=0.15, seed=55, spare_blocks=0, max_blocks=2048,
                                head_dim=128, num_q_heads=7, num_kv_heads=1)
    d = to_dev(case, dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    got = kernels.paged_spike_attn_decode(**d, status=status).cpu().double()
    want = attention_fp64(case)
    err = ((got - want).abs().max() / want.abs().max()).item()
    assert err < 2e-6, f"{err:.2e}"
    got16 = kernels.paged_spike_attn_decode(**d, dtype=torch.bfloat16).cpu()
    assert within_bf16_bar(got16, want.float())
    assert status.item() == 0


@pytest.fixture
def tcgen05_form(lib):
    """Routes eligible calls to the tcgen05 / tensor-memory form for the duration of a test."""
    assert lib.spk_attn_select_form(_lib.ATTN_FORM_TCGEN05) == 0
    yield
    assert lib.spk_attn_select_form(_lib.ATTN_FORM_AUTO) == 0


@pytest.mark.parametrize("name", ["single_token", "ragged", "bs64", "gqa_4_2", "gqa_28_2", "T1", "T8", "long_split", "wide_table"])
def test_tcgen05_form_matches_oracle(name, dev, tcgen05_form):
    """The tcgen05 form (int8 MMAs out of shared memory, int32 sums in tensor memory) on the cases it applies to
    (head_dim 64, 16-bit output): within the 16-bit bar of the oracle, status clean (no expired wait)."""
    case = cases.attention_case(**cases.ATTENTION_CASES[name])
    want = orc.paged_spike_attn_decode(**case)
    for dtype in (torch.bfloat16, torch.float16):
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        got = run(case, dev, dtype=dtype, status=status).cpu()
        assert torch.isfinite(got).all()
        if dtype == torch.bfloat16:
            assert within_bf16_bar(got, want)
        else:
            assert rel_err(got, want) < 1e-3
        assert status.item() == 0


def test_tcgen05_form_config2_and_linearity(dev, tcgen05_form):
    """The kernel-level attention configuration through the tcgen05 form, plus linearity in V: the sums are exact
    integers there, so out(V1 | V2) = out(V1) + out(V2) holds to the rounding of the 16-bit outputs."""
    case = config2_case()
    d = to_dev(case, dev)
    want = orc.paged_spike_attn_decode(**case)
    got = kernels.paged_spike_attn_decode(**d, dtype=torch.bfloat16).cpu()
    assert within_bf16_bar(got, want)
    mask = torch.tensor([0x0F0F0F0F, 0x33333333], dtype=torch.int32, device=dev)
    d1, d2 = dict(d), dict(d)
    d1["v_cache"] = d["v_cache"] & mask
    d2["v_cache"] = d["v_cache"] & ~mask
    o1 = kernels.paged_spike_attn_decode(**d1, dtype=torch.float16).float()
    o2 = kernels.paged_spike_attn_decode(**d2, dtype=torch.float16).float()
    o = kernels.paged_spike_attn_decode(**d, dtype=torch.float16).float()
    torch.testing.assert_close(o1 + o2, o, rtol=0, atol=3 * 2.0 ** -11 * float(o.abs().max()))


def test_form_selector_rejects_unknown_values(lib):
    assert lib.spk_attn_select_form(7) == -6 and lib.spk_attn_select_form(-1) == -6
    assert lib.spk_attn_select_form(_lib.ATTN_FORM_GENERAL) == 0
    assert lib.spk_attn_select_form(_lib.ATTN_FORM_AUTO) == 0


@pytest.mark.parametrize("seq_lens,max_blocks,density", [([32768], 2048, 0.2), ([9000, 2500], 1024, 0.5)])
def test_long_rows_against_float64(seq_lens, max_blocks, density, dev):
    """Accumulation over tens of thousands of keys (tensor-core sums, partial records, combine) stays within
    2e-6 of an exact evaluation; the bf16 and fp32 bars of the short cases are met with room to spare."""
    case = cases.attention_case(seq_lens=seq_lens, density=density, seed=5, spare_blocks=0, max_blocks=max_blocks)
    got = run(case, dev).cpu().double()
    want = attention_fp64(case)
    err = ((got - want).abs().max() / want.abs().max()).item()
    assert err < 2e-6, f"{err:.2e}"


def test_softmax_range_beyond_the_weight_format_is_refused(dev):
    """The library's weights cover exp(-24)..1 of the softmax bound (scale * head_dim <= 24); the reference's
    scale, head_dim^-0.5, is far inside.  A wider range is rejected on the host, nothing is launched."""
    lib = _lib.load()
    case = to_dev(cases.attention_case(seq_lens=[40]), dev)
    q, k, v, tables, lens = (case[n] for n in ("q_packed", "k_cache", "v_cache", "block_tables", "seq_lens"))
    out = torch.full((q.shape[0], 1, case["num_q_heads"], 64), 7.0, device=dev)
    args = [q.data_ptr(), q.stride(0), q.stride(1), q.stride(2),
            k.data_ptr(), k.stride(0), k.stride(1), k.stride(2) * 16, k.stride(2),
            v.data_ptr(), v.stride(0), v.stride(1), v.stride(2) * 16, v.stride(2),
            tables.data_ptr(), tables.stride(0), lens.data_ptr(),
            out.data_ptr(), _lib.F32, out.stride(0), out.stride(1), out.stride(2),
            q.shape[0], 1, case["num_q_heads"], case["num_kv_heads"], 64, 16, tables.shape[1], k.shape[2] // 16]
    tail = [None, 0, None, None]
    assert lib.spk_attn_decode(*args, 0.5, *tail) == -6      # 64 * 0.5 = 32 > 24
    assert lib.spk_attn_decode(*args, -0.1, *tail) == -6
    torch.cuda.synchronize()
    assert (out == 7.0).all()
    assert lib.spk_attn_decode(*args, 0.125, *tail) == 0
    torch.cuda.synchronize()
    assert torch.isfinite(out).all() and not (out == 7.0).all()
