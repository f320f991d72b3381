"""Seeded input generators shared by the golden-fixture script, the CPU tests and the GPU parity tests.

All randomness comes from a CPU ``torch.Generator`` so the oracle and the CUDA path see identical
bits.  Shapes and densities follow the reference's own test generators
(tests/test_spike_attention.py:31-71, tests/test_cpu_backend.py:30-69, tests/test_lif_kernel.py:30-41)
without reusing their code.
"""
from __future__ import annotations

import hashlib

import torch

from oracle import torch_oracle as orc


def gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(seed)


def digest(*tensors: torch.Tensor) -> str:
    """Short hash of tensor contents, stored with golden outputs to detect RNG drift."""
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()[:16]


def bernoulli_bits(shape, p: float, g: torch.Generator) -> torch.Tensor:
    return (torch.rand(shape, generator=g) < p).to(torch.float32)


def attention_case(seq_lens, *, head_dim=64, block_size=16, num_q_heads=14, num_kv_heads=2, T=4,
                   density=0.3, q_density=None, seed=0, spare_blocks=3, max_blocks=None):
    """A paged pool with scrambled physical blocks, random spikes everywhere (owned or not), tables
    padded with the reserved last block."""
    g = gen(seed)
    n = len(seq_lens)
    need = [(s + block_size - 1) // block_size for s in seq_lens]
    widest = max(max(need), 1)
    if max_blocks is None:
        max_blocks = widest
    num_blocks = sum(need) + spare_blocks + 1
    num_slots = num_blocks * block_size
    k_cache = orc.pack_spikes(bernoulli_bits((T, num_kv_heads, num_slots, head_dim), density, g))
    v_cache = orc.pack_spikes(bernoulli_bits((T, num_kv_heads, num_slots, head_dim), density, g))
    q = bernoulli_bits((T, n, num_q_heads, head_dim), density if q_density is None else q_density, g)
    order = torch.randperm(num_blocks - 1, generator=g)
    tables = torch.full((n, max_blocks), num_blocks - 1, dtype=torch.int32)
    cur = 0
    for i, nb in enumerate(need):
        tables[i, :nb] = order[cur:cur + nb].to(torch.int32)
        cur += nb
    return dict(
        q_packed=orc.pack_spikes(q), k_cache=k_cache, v_cache=v_cache, block_tables=tables,
        seq_lens=torch.tensor(seq_lens, dtype=torch.int32), head_dim=head_dim, block_size=block_size,
        num_q_heads=num_q_heads, num_kv_heads=num_kv_heads,
    )


ATTENTION_CASES = {
    # name: kwargs of attention_case
    "single_token": dict(seq_lens=[1]),
    "short": dict(seq_lens=[7]),
    "one_block": dict(seq_lens=[16]),
    "block_boundary": dict(seq_lens=[17]),
    "two_blocks_plus_one": dict(seq_lens=[33], block_size=32),
    "ragged": dict(seq_lens=[1, 5, 40, 97]),
    "uniform": dict(seq_lens=[64] * 8, block_size=32),
    "bs64": dict(seq_lens=[128, 3, 65], block_size=64),
    "gqa_4_4": dict(seq_lens=[48], num_q_heads=4, num_kv_heads=4, block_size=32),
    "gqa_8_1": dict(seq_lens=[48, 9], num_q_heads=8, num_kv_heads=1, block_size=32),
    "gqa_16_8": dict(seq_lens=[48], num_q_heads=16, num_kv_heads=8, block_size=32),
    "gqa_4_2": dict(seq_lens=[7, 20, 40, 3], num_q_heads=4, num_kv_heads=2),
    "gqa_6_2": dict(seq_lens=[21, 4], num_q_heads=6, num_kv_heads=2),
    "gqa_28_2": dict(seq_lens=[37], num_q_heads=28, num_kv_heads=2),
    "T1": dict(seq_lens=[5, 61], T=1, block_size=32),
    "T2": dict(seq_lens=[5, 61], T=2, block_size=32),
    "T8": dict(seq_lens=[5, 61], T=8, block_size=32),
    "d32": dict(seq_lens=[10, 33, 50], head_dim=32, num_q_heads=4),
    "d96": dict(seq_lens=[10, 33, 50], head_dim=96, num_q_heads=4),
    "d128": dict(seq_lens=[10, 33, 50], head_dim=128, num_q_heads=4),
    "d128_gqa7": dict(seq_lens=[70, 300], head_dim=128, num_q_heads=7, num_kv_heads=1),
    "dense_q": dict(seq_lens=[40, 17], density=0.4, q_density=0.6, block_size=32),
    "long_split": dict(seq_lens=[700, 130, 1], max_blocks=64),
    "wide_table": dict(seq_lens=[9, 25, 41, 3], max_blocks=256),
}


def lif_case(T, M, N, *, seed, dtype=torch.float32, scale=2.0, with_mem0=False, mid_shape=None):
    """beta in [-1.5, 2.5] (exercises the clamp), threshold in (0.05, 1.0), currents N(0, scale^2)."""
    g = gen(seed)
    beta = torch.rand(N, generator=g) * 4.0 - 1.5
    threshold = torch.rand(N, generator=g) * 0.95 + 0.05
    shape = (T, *(mid_shape or (M,)), N)
    x = (torch.randn(shape, generator=g) * scale).to(dtype)
    mem0 = torch.randn(shape[1:], generator=g) if with_mem0 else None
    return dict(x=x, beta=beta, threshold=threshold, mem0=mem0)


def lif_boundary_case(T=8, M=256, N=64, seed=0):
    """Membrane hovering at the threshold: catches a fused multiply-add (one rounding instead of two)."""
    g = gen(seed)
    x = torch.ones(T, M, N) + torch.randn(T, M, N, generator=g) * 1e-6
    return dict(x=x, beta=torch.full((N,), 0.9), threshold=torch.full((N,), 1.0), mem0=None)


LIF_CASES = {
    "T1_N64": dict(T=1, M=32, N=64, seed=101),
    "T2_N64": dict(T=2, M=32, N=64, seed=102),
    "T4_N64": dict(T=4, M=128, N=64, seed=104),
    "T8_N64": dict(T=8, M=32, N=64, seed=108),
    "T4_N63": dict(T=4, M=32, N=63, seed=163),
    "T4_N4864": dict(T=4, M=4, N=4864, seed=148),
    "T3_N100": dict(T=3, M=5, N=100, seed=131),
    "T4_bf16": dict(T=4, M=32, N=64, seed=216, dtype=torch.bfloat16),
    "T4_mem0": dict(T=4, M=16, N=64, seed=300, with_mem0=True),
    "T4_5d": dict(T=4, M=0, N=64, seed=42, mid_shape=(2, 3, 5)),
}

PACK_CHANNELS = [1, 31, 32, 33, 63, 64, 128, 256, 4864]


def pack_case(channels: int):
    g = gen(channels)
    return bernoulli_bits((3, 5, channels), 0.5, g)
