"""Paged popcount decode attention over the bit-packed spike cache (CUDA).

``paged_spike_attn_decode`` keeps the signature and the error behaviour of
``spikeinfer/kernels/spike_attention.py:153-221`` of the reference; ``gather_kv_unpacked``
is :224-244.  ``qk_scores`` exposes the exact integer scores for checking.
"""
from __future__ import annotations

import math

import torch

from .. import _lib
from .packing import packed_width


def _pool_strides(cache: torch.Tensor, block_size: int):
    """(s_t, s_h, s_blk, s_slot) of a pool given as ``[T, H_kv, num_slots, W]`` (the reference
    layout, any strides) or as ``[T, H_kv, num_blocks, block_size, W]`` (explicit block axis)."""
    if cache.ndim == 4:
        if cache.stride(3) != 1 and cache.shape[3] > 1:
            raise ValueError("the word axis of a spike cache must be contiguous")
        return cache.stride(0), cache.stride(1), cache.stride(2) * block_size, cache.stride(2), cache.shape[2] // block_size
    if cache.ndim == 5:
        if cache.stride(4) != 1 and cache.shape[4] > 1:
            raise ValueError("the word axis of a spike cache must be contiguous")
        if cache.shape[3] != block_size:
            raise ValueError(f"cache block axis holds {cache.shape[3]} slots, expected {block_size}")
        return cache.stride(0), cache.stride(1), cache.stride(2), cache.stride(3), cache.shape[2]
    raise ValueError(f"spike cache must be 4-D or 5-D, got {cache.ndim}-D")


def paged_spike_attn_decode(
    q_packed: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_tables: torch.Tensor,
    seq_lens: torch.Tensor,
    head_dim: int,
    block_size: int,
    num_q_heads: int,
    num_kv_heads: int,
    out: torch.Tensor | None = None,
    dtype: torch.dtype = torch.float32,
    status: torch.Tensor | None = None,
    overlap_previous: bool = False,
) -> torch.Tensor:
    """One decode step of attention against the paged spike cache.

    q_packed ``int32 [T, N, H_q, W]``; k_cache/v_cache ``int32 [T, H_kv, num_slots, W]`` (strided
    views allowed); block_tables ``int32 [N, max_blocks]``; seq_lens ``int32 [N]`` including the token
    being decoded.  ``out`` (optional, may be a strided view such as ``buf[:, :n_dec]``) receives
    ``[T, N, H_q, head_dim]``; its dtype decides the output type.  Launches on the current stream,
    never synchronises.  ``overlap_previous=True`` lets the launch overlap the kernel before it on the
    stream (it then reads only ``block_tables`` and ``seq_lens`` until that kernel has finished): pass it only
    when those two were complete before that kernel began.
    """
    T, n_seqs, n_heads, words = q_packed.shape
    if words != packed_width(head_dim):
        raise ValueError(f"q has {words} words, expected {packed_width(head_dim)}")
    if n_heads != num_q_heads:
        raise ValueError(f"q has {n_heads} heads, expected {num_q_heads}")
    _lib.require_cuda(q_packed, "paged_spike_attn_decode q_packed")
    dev = q_packed.device
    if out is None:
        out = torch.empty((T, n_seqs, n_heads, head_dim), device=dev, dtype=dtype)
    if T == 0 or n_seqs == 0:
        return out
    if q_packed.stride(3) != 1:
        q_packed = q_packed.contiguous()
    if out.stride(3) != 1:
        raise ValueError("the channel axis of `out` must be contiguous")
    if block_tables.dtype != torch.int32 or seq_lens.dtype != torch.int32:
        raise TypeError("block_tables and seq_lens must be int32")
    if block_tables.stride(1) != 1:
        block_tables = block_tables.contiguous()
    seq_lens = seq_lens.contiguous()
    sk = _pool_strides(k_cache, block_size)
    sv = _pool_strides(v_cache, block_size)
    max_blocks = block_tables.shape[1]
    lib = _lib.load()
    ws_bytes = lib.spk_attn_decode_workspace_bytes(T, n_seqs, num_q_heads, num_kv_heads, head_dim,
                                                   block_size, max_blocks)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev) if ws_bytes > 0 else None
    with torch.cuda.device(dev):
        if overlap_previous:
            lib.spk_attn_overlap_next_call()
        rc = lib.spk_attn_decode(
            q_packed.data_ptr(), q_packed.stride(0), q_packed.stride(1), q_packed.stride(2),
            k_cache.data_ptr(), sk[0], sk[1], sk[2], sk[3],
            v_cache.data_ptr(), sv[0], sv[1], sv[2], sv[3],
            block_tables.data_ptr(), block_tables.stride(0), seq_lens.data_ptr(),
            out.data_ptr(), _lib.dtype_code(out.dtype), out.stride(0), out.stride(1), out.stride(2),
            T, n_seqs, num_q_heads, num_kv_heads, head_dim, block_size, max_blocks, min(sk[4], sv[4]),
            1.0 / math.sqrt(head_dim), _lib.ptr(ws), ws_bytes, _lib.ptr(status),
            _lib.current_stream(dev))
    _lib.check(rc, "spk_attn_decode")
    return out


def qk_scores(q_packed, k_cache, block_tables, seq_lens, head_dim, block_size, num_q_heads,
              num_kv_heads, max_len: int | None = None, status=None) -> torch.Tensor:
    """Exact scores ``popc(q & k)`` as ``int32 [T, N, H_q, max_len]`` (-1 past each sequence's end)."""
    T, n_seqs, n_heads, words = q_packed.shape
    if words != packed_width(head_dim):
        raise ValueError(f"q has {words} words, expected {packed_width(head_dim)}")
    _lib.require_cuda(q_packed, "qk_scores q_packed")
    dev = q_packed.device
    max_blocks = block_tables.shape[1]
    if max_len is None:
        max_len = max_blocks * block_size
    scores = torch.empty((T, n_seqs, n_heads, max_len), dtype=torch.int32, device=dev)
    q_packed = q_packed.contiguous()
    block_tables = block_tables.contiguous()
    sk = _pool_strides(k_cache, block_size)
    lib = _lib.load()
    with torch.cuda.device(dev):
        rc = lib.spk_qk_scores(
            q_packed.data_ptr(), q_packed.stride(0), q_packed.stride(1), q_packed.stride(2),
            k_cache.data_ptr(), sk[0], sk[1], sk[2], sk[3],
            block_tables.data_ptr(), block_tables.stride(0), seq_lens.contiguous().data_ptr(),
            scores.data_ptr(), max_len, T, n_seqs, num_q_heads, num_kv_heads, head_dim, block_size,
            max_blocks, sk[4], _lib.ptr(status), _lib.current_stream(dev))
    _lib.check(rc, "spk_qk_scores")
    return scores


def gather_kv_unpacked(cache: torch.Tensor, block_table: torch.Tensor, seq_len: int, head_dim: int,
                       block_size: int, dtype: torch.dtype, status=None) -> torch.Tensor:
    """Read one sequence's cached spikes back as a dense ``[T, H_kv, seq_len, head_dim]`` (prefill path)."""
    _lib.require_cuda(cache, "gather_kv_unpacked cache")
    T, H = cache.shape[0], cache.shape[1]
    out = torch.empty((T, H, seq_len, head_dim), dtype=dtype, device=cache.device)
    if out.numel() == 0:
        return out
    s = _pool_strides(cache, block_size)
    if block_table.dtype != torch.int32:
        block_table = block_table.to(torch.int32)
    block_table = block_table.contiguous()
    lib = _lib.load()
    with torch.cuda.device(cache.device):
        rc = lib.spk_gather_kv_unpacked(cache.data_ptr(), s[0], s[1], s[2], s[3], block_table.data_ptr(),
                                        seq_len, T, H, head_dim, block_size, s[4], out.data_ptr(),
                                        _lib.dtype_code(dtype), _lib.ptr(status),
                                        _lib.current_stream(cache.device))
    _lib.check(rc, "spk_gather_kv_unpacked")
    return out


def gather_kv_unpacked_batch(cache: torch.Tensor, block_tables: torch.Tensor, seq_len: int, head_dim: int,
                             block_size: int, dtype: torch.dtype, status=None) -> torch.Tensor:
    """:func:`gather_kv_unpacked` for several sequences of the same length in one launch: ``block_tables`` int32
    ``[n_seqs, >= ceil(seq_len / block_size)]`` -> dense ``[n_seqs, T, H_kv, seq_len, head_dim]``."""
    _lib.require_cuda(cache, "gather_kv_unpacked_batch cache")
    T, H = cache.shape[0], cache.shape[1]
    n = block_tables.shape[0]
    out = torch.empty((n, T, H, seq_len, head_dim), dtype=dtype, device=cache.device)
    if out.numel() == 0:
        return out
    if block_tables.dtype != torch.int32 or block_tables.ndim != 2:
        raise TypeError("block_tables must be int32 [n_seqs, blocks]")
    if block_tables.shape[1] * block_size < seq_len:
        raise ValueError("block tables shorter than seq_len")
    if block_tables.stride(1) != 1:
        block_tables = block_tables.contiguous()
    s = _pool_strides(cache, block_size)
    lib = _lib.load()
    with torch.cuda.device(cache.device):
        rc = lib.spk_gather_kv_unpacked_batch(cache.data_ptr(), s[0], s[1], s[2], s[3], block_tables.data_ptr(),
                                              block_tables.stride(0), n, seq_len, T, H, head_dim, block_size, s[4],
                                              out.data_ptr(), _lib.dtype_code(dtype), _lib.ptr(status),
                                              _lib.current_stream(cache.device))
    _lib.check(rc, "spk_gather_kv_unpacked_batch")
    return out


def paged_spike_attn_decode_noalloc(q_packed, k_cache, v_cache, block_tables, seq_lens, head_dim: int,
                                    block_size: int, num_q_heads: int, num_kv_heads: int, out: torch.Tensor,
                                    status: torch.Tensor | None = None) -> torch.Tensor:
    """:func:`paged_spike_attn_decode` for callers that must not allocate.

    Nothing is allocated on the way: ``out`` is required, every tensor must already be laid out as
    the kernel wants it (no ``.contiguous()`` copies are made here), and the split-KV partial sums
    go to the 8 MiB scratch array built into the library instead of a torch workspace.  Meant for a
    server that gave all free device memory to the page pool at start-up, or a host that only holds
    raw device pointers.  Problems whose partial sums do not fit raise :class:`SpkError`; calls on
    one device share the scratch array and must not overlap on the GPU.  The first call on a device
    resolves the array's address: make it at start-up.
    """
    T, n_seqs, n_heads, words = q_packed.shape
    if words != packed_width(head_dim):
        raise ValueError(f"q has {words} words, expected {packed_width(head_dim)}")
    if n_heads != num_q_heads:
        raise ValueError(f"q has {n_heads} heads, expected {num_q_heads}")
    _lib.require_cuda(q_packed, "paged_spike_attn_decode_noalloc q_packed")
    if q_packed.stride(3) != 1 or out.stride(3) != 1 or block_tables.stride(1) != 1 or seq_lens.stride(0) != 1:
        raise ValueError("q_packed, out, block_tables and seq_lens must have a contiguous last axis")
    if block_tables.dtype != torch.int32 or seq_lens.dtype != torch.int32:
        raise TypeError("block_tables and seq_lens must be int32")
    sk = _pool_strides(k_cache, block_size)
    sv = _pool_strides(v_cache, block_size)
    dev = q_packed.device
    lib = _lib.load()
    with torch.cuda.device(dev):
        rc = lib.spk_attn_decode_static(
            q_packed.data_ptr(), q_packed.stride(0), q_packed.stride(1), q_packed.stride(2),
            k_cache.data_ptr(), sk[0], sk[1], sk[2], sk[3],
            v_cache.data_ptr(), sv[0], sv[1], sv[2], sv[3],
            block_tables.data_ptr(), block_tables.stride(0), seq_lens.data_ptr(),
            out.data_ptr(), _lib.dtype_code(out.dtype), out.stride(0), out.stride(1), out.stride(2),
            T, n_seqs, num_q_heads, num_kv_heads, head_dim, block_size, block_tables.shape[1], min(sk[4], sv[4]),
            1.0 / math.sqrt(head_dim), _lib.ptr(status), _lib.current_stream(dev))
    _lib.check(rc, "spk_attn_decode_static")
    return out
