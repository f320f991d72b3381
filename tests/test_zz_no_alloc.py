"""The allocation-free attention entry point (spk_attn_decode_static) against the ordinary one.

It serves callers that cannot hand the kernel a workspace -- a process whose free device memory all
went to the page pool at start-up, or an FFI host holding nothing but raw device pointers -- by keeping
the split-KV partial sums in a fixed 8 MiB array inside the library.  The array is shared by every
call and keeps the previous call's contents, so the check runs twice in a row on different inputs:
stale partial sums must not leak into the second result.  Collected last on purpose (file name), and
it must pass both alone in a fresh process and after every other test.
"""
from __future__ import annotations

import pytest
import torch

import cases
from conftest import to_dev
from oracle import torch_oracle as orc
from spikeinfer_b200 import _lib, kernels

pytestmark = pytest.mark.gpu

REL_TOL = 1e-5  # same bar as tests/test_gpu_attention.py


def rel_err(got, want):
    return ((got.float() - want.float()).abs().max() / want.abs().max().clamp(min=1e-6)).item()


def test_static_scratch_matches_workspace_path_twice_in_a_row(dev, lib):
    assert lib.spk_attn_decode_static_capacity() == 8 << 20
    # first call: long ragged rows (split into key ranges -> scratch in use); second call: other lengths,
    # other bits, fewer rows, so records left by the first call lie where the second one does not write
    specs = [dict(seq_lens=[700, 130, 1, 1500, 64, 2047], max_blocks=128, seed=31),
             dict(seq_lens=[33, 900, 5], max_blocks=128, seed=32, density=0.4)]
    for spec in specs:
        case = cases.attention_case(**spec)
        d = to_dev(case, dev)
        need = lib.spk_attn_decode_workspace_bytes(4, len(spec["seq_lens"]), 14, 2, 64, 16, 128)
        assert 0 < need <= 8 << 20, "the case must exercise the scratch array"
        want = kernels.paged_spike_attn_decode(**d)
        out = torch.full_like(want, float("nan"))
        n_allocs = lambda: torch.cuda.memory_stats(dev).get("allocation.all.allocated", 0)  # monotonic counter
        before = n_allocs()
        got = kernels.paged_spike_attn_decode_noalloc(**d, out=out)
        assert n_allocs() == before, "the no-alloc path asked the allocator for device memory"
        assert got.data_ptr() == out.data_ptr()
        assert torch.isfinite(got).all()
        assert rel_err(got, want) < REL_TOL
        assert rel_err(got.cpu(), orc.paged_spike_attn_decode(**case)) < REL_TOL  # and against the CPU oracle itself
    # bf16 output into a strided view, as the engine passes it
    buf = torch.zeros(4, 5, 14, 64, dtype=torch.bfloat16, device=dev)
    kernels.paged_spike_attn_decode_noalloc(**d, out=buf[:, :3])
    want16 = kernels.paged_spike_attn_decode(**d, dtype=torch.bfloat16)
    assert rel_err(buf[:, :3], want16) < 2.0 ** -7
    assert (buf[:, 3:] == 0).all()


def test_static_scratch_refuses_what_does_not_fit(dev, lib):
    """Beyond the built-in capacity nothing is launched and the error says so."""
    n, max_blocks = 256, 2048  # 256 sequences x 32k keys: partial sums far above 8 MiB
    assert lib.spk_attn_decode_workspace_bytes(4, n, 14, 2, 64, 16, max_blocks) > 8 << 20
    q = torch.zeros(4, n, 14, 2, dtype=torch.int32, device=dev)
    pool = torch.zeros(4, 2, 64, 2, dtype=torch.int32, device=dev)
    tables = torch.zeros(n, max_blocks, dtype=torch.int32, device=dev)
    lens = torch.ones(n, dtype=torch.int32, device=dev)
    out = torch.full((4, n, 14, 64), 3.0, device=dev)
    with pytest.raises(_lib.SpkError, match="built-in array"):
        kernels.paged_spike_attn_decode_noalloc(q, pool, pool, tables, lens, 64, 16, 14, 2, out=out)
    assert (out == 3.0).all()
