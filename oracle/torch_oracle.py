"""CPU restatement of the reference's spiking-decode operators (TEST INFRASTRUCTURE ONLY).

This module is the parity oracle: a plain-PyTorch, CPU-only restatement of what
HzAybars/Spikeinfer v0.3.0 computes on the decode hot path.  Nothing in the shipped package
imports it; only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference arms
of ``bench.py`` do, and there only as the checker or as the timed CPU baseline.

Pinning: every function below is checked against outputs of the reference itself (its own CPU
code imported from the reference checkout) through the fixtures in ``tests/golden/`` made by
``tests/golden/make_golden.py``; ``tests/test_oracle_golden.py`` runs those checks.  The one part
that cannot be pinned directly is the snntorch ``Leaky`` neuron (snntorch 1.0.0 is not
installable here): LIF parity is pinned on the reference's own restatement
``lif_multistep_ref`` (spikeinfer/kernels/lif_triton.py:126-138), which the reference's tests
assert bit-equal to snntorch (tests/test_lif_kernel.py:95-112).  The hard-reset LIF mode has no
counterpart in the reference: its oracle is this file alone ("parity unpinned").

Citations are paths inside the reference project.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

BITS_PER_WORD = 32

SUBTRACT_DELAYED = 0
HARD_ZERO = 1


# --------------------------------------------------------------------------- packing
def packed_width(num_channels: int) -> int:
    """spikeinfer/kernels/packing.py:46-48."""
    return (num_channels + BITS_PER_WORD - 1) // BITS_PER_WORD


def pack_spikes(x: torch.Tensor) -> torch.Tensor:
    """[..., C] -> int32 [..., ceil(C/32)], bit i of word w = (x[..., 32w+i] != 0).

    Follows spikeinfer/kernels/packing.py:98-111 (layout :15-23): little-endian within a word,
    zero tail, sign bit used as a value bit.
    """
    c = x.shape[-1]
    w = packed_width(c)
    bits = (x != 0).to(torch.int64)
    if w * 32 != c:
        bits = F.pad(bits, (0, w * 32 - c))
    bits = bits.reshape(*x.shape[:-1], w, 32)
    weights = torch.ones(32, dtype=torch.int64) << torch.arange(32, dtype=torch.int64)
    val = (bits * weights).sum(-1)
    val = torch.where(val >= (1 << 31), val - (1 << 32), val)
    return val.to(torch.int32)


def unpack_spikes(words: torch.Tensor, num_channels: int, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Inverse of pack_spikes; spikeinfer/kernels/packing.py:136-152 (ValueError on a wrong width)."""
    expected = packed_width(num_channels)
    if words.shape[-1] != expected:
        raise ValueError(f"expected {expected} words for {num_channels} channels, got {words.shape[-1]}")
    u = words.to(torch.int64) & 0xFFFFFFFF
    bits = (u.unsqueeze(-1) >> torch.arange(32, dtype=torch.int64)) & 1
    bits = bits.reshape(*words.shape[:-1], expected * 32)
    return bits[..., :num_channels].to(dtype)


def packed_bytes_per_token(num_layers: int, num_timesteps: int, num_kv_heads: int, head_dim: int) -> int:
    """spikeinfer/kernels/packing.py:155-159."""
    return 2 * num_layers * num_timesteps * num_kv_heads * packed_width(head_dim) * 4


# --------------------------------------------------------------------------- LIF
def lif_multistep(x, beta, threshold, mem0=None, out_dtype=None, reset_mode: int = SUBTRACT_DELAYED):
    """T-step LIF over x [T, *mid, N]; returns (spikes [T, *mid, N], final membrane fp32).

    SUBTRACT_DELAYED follows spikeinfer/kernels/lif_triton.py:126-138 (semantics :13-28): fp32
    membrane, beta clamped to [0,1], reset taken from the previous membrane, spike = (u - th) > 0,
    every product and sum a separate fp32 operation.  HARD_ZERO (u <- 0 where the neuron spiked,
    no delayed reset) is this project's own definition.
    """
    T = x.shape[0]
    b = beta.clamp(0, 1).to(torch.float32)
    th = threshold.to(torch.float32)
    if mem0 is None:
        u = torch.zeros(x.shape[1:], dtype=torch.float32)
    else:
        u = mem0.to(torch.float32).clone()
    out_dtype = out_dtype or x.dtype
    spikes = torch.empty(x.shape, dtype=out_dtype)
    for t in range(T):
        cur = x[t].to(torch.float32)
        if reset_mode == SUBTRACT_DELAYED:
            r = ((u - th) > 0).to(torch.float32)
            u = b * u
            u = u + cur
            u = u - r * th
            spikes[t] = ((u - th) > 0).to(out_dtype)
        elif reset_mode == HARD_ZERO:
            u = b * u
            u = u + cur
            s = (u - th) > 0
            spikes[t] = s.to(out_dtype)
            u = torch.where(s, torch.zeros_like(u), u)
        else:
            raise ValueError(f"unknown reset mode {reset_mode}")
    return spikes, u


# --------------------------------------------------------------------------- paged pool walk
def slot_matrix(block_tables: torch.Tensor, length: int, block_size: int) -> torch.Tensor:
    """[n, max_blocks] -> [n, length] physical slots; spikeinfer/kernels/spike_attention_cpu.py:87-100."""
    pos = torch.arange(length, dtype=torch.int64)
    blocks = block_tables.to(torch.int64)[:, pos // block_size]
    return blocks * block_size + (pos % block_size)[None, :]


def gather_kv_unpacked(cache, block_table, seq_len, head_dim, block_size, dtype=torch.float32):
    """One sequence's cached spikes as dense [T, H_kv, S, D]; spikeinfer/kernels/spike_attention.py:224-244."""
    slots = slot_matrix(block_table[None, :], seq_len, block_size)[0]
    return unpack_spikes(cache.index_select(2, slots), head_dim, dtype)


def qk_scores(q_packed, k_cache, block_tables, seq_lens, head_dim, block_size, num_q_heads, num_kv_heads):
    """Exact integer scores popc(q & k): int32 [T, N, H_q, max_len], -1 past each sequence's end.

    The integer half of spikeinfer/kernels/spike_attention.py:114-120, computed on the packed
    words themselves (AND + bit count), independently of the unpack + matmul route.
    """
    T, n, hq, w = q_packed.shape
    n_rep = num_q_heads // num_kv_heads
    lens = seq_lens.tolist()
    max_len = block_tables.shape[1] * block_size
    out = torch.full((T, n, hq, max_len), -1, dtype=torch.int32)
    for i, length in enumerate(lens):
        slots = slot_matrix(block_tables[i : i + 1], length, block_size)[0]
        k = k_cache.index_select(2, slots).to(torch.int64) & 0xFFFFFFFF  # [T, Hkv, S, W]
        k = k.repeat_interleave(n_rep, dim=1)  # [T, Hq, S, W]
        q = (q_packed[:, i].to(torch.int64) & 0xFFFFFFFF)[:, :, None, :]  # [T, Hq, 1, W]
        both = q & k
        cnt = torch.zeros(both.shape[:-1], dtype=torch.int64)
        for b in range(32):
            cnt += ((both >> b) & 1).sum(-1)
        out[:, i, :, :length] = cnt.to(torch.int32)
    return out


def paged_spike_attn_decode(q_packed, k_cache, v_cache, block_tables, seq_lens, head_dim, block_size,
                            num_q_heads, num_kv_heads, dtype=torch.float32):
    """softmax(q.k / sqrt(d)) v per sequence on unpacked spikes, fp32: [T, N, H_q, D].

    Same computation as spikeinfer/kernels/spike_attention.py:247-282 (one sequence at a time,
    K/V repeated over the GQA group), with the softmax written out instead of calling SDPA.
    """
    T, n = q_packed.shape[0], q_packed.shape[1]
    n_rep = num_q_heads // num_kv_heads
    scale = 1.0 / math.sqrt(head_dim)
    out = torch.empty((T, n, num_q_heads, head_dim), dtype=dtype)
    for i in range(n):
        length = int(seq_lens[i])
        q = unpack_spikes(q_packed[:, i], head_dim, torch.float32)  # [T, Hq, D]
        k = gather_kv_unpacked(k_cache, block_tables[i], length, head_dim, block_size)
        v = gather_kv_unpacked(v_cache, block_tables[i], length, head_dim, block_size)
        k = k.repeat_interleave(n_rep, dim=1)
        v = v.repeat_interleave(n_rep, dim=1)
        s = torch.einsum("thd,thsd->ths", q, k) * scale
        p = torch.softmax(s, dim=-1)
        out[:, i] = torch.einsum("ths,thsd->thd", p, v).to(dtype)
    return out


def paged_spike_attn_decode_batched(q_packed, k_cache, v_cache, block_tables, seq_lens, head_dim,
                                    block_size, num_q_heads, num_kv_heads, dtype=torch.float32,
                                    budget_bytes: int = 16 * 2**20):
    """The reference's CPU decode path, restated: sequences grouped under a gather budget, each group
    padded to its longest member, one SDPA call per group with GQA broadcast
    (spikeinfer/kernels/spike_attention_cpu.py:103-222).  This is the form timed as the CPU baseline."""
    T, n, hq, _ = q_packed.shape
    out = torch.empty((T, n, hq, head_dim), dtype=dtype)
    lens = [int(v) for v in seq_lens.tolist()]
    per_key = T * num_kv_heads * head_dim * 4 * 2
    start = 0
    while start < n:
        stop, longest = start + 1, lens[start]
        while stop < n:
            cand = max(longest, lens[stop])
            if (stop + 1 - start) * cand * per_key > budget_bytes:
                break
            longest, stop = cand, stop + 1
        g = stop - start
        slots = slot_matrix(block_tables[start:stop], longest, block_size).reshape(-1)

        def dense(cache):
            words = cache.index_select(2, slots).view(T, num_kv_heads, g, longest, -1)
            words = words.permute(0, 2, 1, 3, 4).reshape(T * g, num_kv_heads, longest, -1)
            return unpack_spikes(words, head_dim, torch.float32)

        q = unpack_spikes(q_packed[:, start:stop], head_dim, torch.float32).reshape(T * g, hq, 1, head_dim)
        mask = None
        group_lens = lens[start:stop]
        if any(v != longest for v in group_lens):
            valid = torch.arange(longest)[None, :] < torch.tensor(group_lens)[:, None]
            mask = torch.zeros((g, longest), dtype=torch.float32).masked_fill_(~valid, float("-inf"))
            mask = mask[None, :, None, None, :].expand(T, g, 1, 1, longest).reshape(T * g, 1, 1, longest)
        ctx = F.scaled_dot_product_attention(q, dense(k_cache), dense(v_cache), attn_mask=mask,
                                             enable_gqa=num_q_heads != num_kv_heads)
        out[:, start:stop] = ctx.view(T, g, hq, head_dim).to(dtype)
        start = stop
    return out


# --------------------------------------------------------------------------- block allocator / metadata
class BlockManager:
    """LIFO block allocator; spikeinfer/engine/block_manager.py:22-81.

    The free list starts as [N-1 .. 0] and is popped from its tail, so blocks are handed out as
    0, 1, 2, ...; freeing appends a sequence's blocks in table order.
    """

    def __init__(self, num_blocks: int, block_size: int) -> None:
        self.num_blocks = num_blocks
        self.block_size = block_size
        self.free_list = list(range(num_blocks - 1, -1, -1))

    def blocks_for(self, num_tokens: int) -> int:
        return (num_tokens + self.block_size - 1) // self.block_size

    def allocate(self, table: list[int], num_computed: int, num_new: int) -> bool:
        need = max(0, self.blocks_for(num_computed + num_new) - len(table))
        if need > len(self.free_list):
            return False
        for _ in range(need):
            table.append(self.free_list.pop())
        return True

    def free(self, table: list[int]) -> None:
        self.free_list.extend(table)
        table.clear()

    def slot_mapping(self, table: list[int], start: int, count: int) -> list[int]:
        return [table[p // self.block_size] * self.block_size + p % self.block_size
                for p in range(start, start + count)]


def prepare_decode(tables: list[list[int]], computed: list[int], max_blocks: int, pad_block: int,
                   block_size: int):
    """Decode-step metadata as the reference's runner builds it (spikeinfer/engine/model_runner.py:66-138):
    positions = computed length, slot of that position, tables padded with the pad block, lens = computed+1."""
    positions = torch.tensor(computed, dtype=torch.int64)
    slots = torch.tensor([t[c // block_size] * block_size + c % block_size for t, c in zip(tables, computed)],
                         dtype=torch.int64)
    padded = [list(t[:max_blocks]) + [pad_block] * (max_blocks - len(t)) for t in tables]
    block_tables = torch.tensor(padded, dtype=torch.int32).reshape(len(tables), max_blocks)
    seq_lens = torch.tensor([c + 1 for c in computed], dtype=torch.int32)
    return positions, slots, block_tables, seq_lens
