"""Attention against the paged spike cache, with the reference's interface
(``AttentionMetadata`` and ``paged_attention`` of ``spikeinfer/attention.py:33-95, :111-180``).

``paged_attention`` takes dense q/k/v spikes as the reference does and is a drop-in for it.  The model
in :mod:`spikeinfer_b200.modeling` uses :func:`fused_qkv_attention` instead, which starts from the
projection outputs and never materialises dense spikes for decode rows.

Token order in the batch is decodes first, then prefill chunks.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from .kernels import (LifSiteSpec, gather_kv_unpacked, gather_kv_unpacked_batch, lif_pack_scatter, pack_spikes,
                      paged_spike_attn_decode)
from .kernels.packing import packed_width


@dataclass
class AttentionMetadata:
    """Everything attention needs that is not a weight or an activation."""

    slot_mapping: torch.Tensor
    """int64 ``[n_tok]``: physical cache slot of every token of the batch."""
    block_size: int
    num_decode_tokens: int = 0
    block_tables: torch.Tensor | None = None
    """int32 ``[n_dec, max_blocks]``."""
    seq_lens: torch.Tensor | None = None
    """int32 ``[n_dec]``: cached length including the token being decoded."""
    prefill_query_starts: list[int] = field(default_factory=list)
    prefill_query_lens: list[int] = field(default_factory=list)
    prefill_context_lens: list[int] = field(default_factory=list)
    prefill_block_tables: list[torch.Tensor] = field(default_factory=list)
    status: torch.Tensor | None = None
    """Optional int32 ``[1]`` device word the kernels OR anomaly bits into."""
    prefill_row_tables: torch.Tensor | None = None
    """Optional int32 ``[n_prefill_tok, max_blocks]`` (see :func:`build_prefill_rows`): with it the prefill
    chunks run through the packed popcount kernel in one batched launch instead of per-sequence SDPA."""
    prefill_row_lens: torch.Tensor | None = None
    """int32 ``[n_prefill_tok]``: keys visible to each prefill token (context + position in chunk + 1)."""
    tables_settled: bool = False
    """The caller vouches that ``block_tables`` and ``seq_lens`` were complete before the launch that precedes the
    decode attention on the stream began (they are written at the head of the step).  The attention launch of
    :func:`fused_qkv_attention` may then overlap the tail of the LIF launch before it."""

    @property
    def num_prefills(self) -> int:
        return len(self.prefill_query_lens)

    def on(self, device: torch.device) -> "AttentionMetadata":
        """This metadata with its tensors on ``device`` (``self`` when they already are)."""
        if self.slot_mapping.device == device:
            return self
        mv = lambda t: None if t is None else t.to(device, non_blocking=True)
        return AttentionMetadata(
            slot_mapping=mv(self.slot_mapping), block_size=self.block_size,
            num_decode_tokens=self.num_decode_tokens, block_tables=mv(self.block_tables),
            seq_lens=mv(self.seq_lens), prefill_query_starts=self.prefill_query_starts,
            prefill_query_lens=self.prefill_query_lens, prefill_context_lens=self.prefill_context_lens,
            prefill_block_tables=[mv(t) for t in self.prefill_block_tables], status=mv(self.status),
            prefill_row_tables=mv(self.prefill_row_tables), prefill_row_lens=mv(self.prefill_row_lens),
            tables_settled=self.tables_settled)


def build_prefill_rows(meta: AttentionMetadata, pad_block: int = 0) -> AttentionMetadata:
    """Batched varlen prefill over the packed pool: every prefill token becomes one row of the decode kernel.

    Token ``i`` of a chunk with ``c`` cached tokens sees keys ``0 .. c + i`` of its sequence, i.e. it is a
    decode row of length ``c + i + 1`` over the sequence's block table; causal masking is the row length.
    The chunk's own K/V are written before attention runs, as for decode rows.  Fills ``prefill_row_tables``
    (each sequence's table repeated for its tokens, padded with ``pad_block``) and ``prefill_row_lens``; the
    prefill chunks must be contiguous and in order behind the decode tokens.  The reference runs one SDPA per
    sequence on unpacked spikes instead (``attention.py:161-178``)."""
    if not meta.num_prefills:
        return meta
    device = meta.slot_mapping.device
    width = max(int(t.numel()) for t in meta.prefill_block_tables)
    tables, lens = [], []
    expect = meta.num_decode_tokens
    for start, q_len, ctx, table in zip(meta.prefill_query_starts, meta.prefill_query_lens,
                                        meta.prefill_context_lens, meta.prefill_block_tables):
        if start != expect:
            raise ValueError("prefill chunks must be contiguous and ordered behind the decode tokens")
        expect = start + q_len
        if -(-(ctx + q_len) // meta.block_size) > table.numel():
            raise ValueError("block table shorter than the chunk's context")
        row = torch.full((width,), pad_block, dtype=torch.int32, device=device)
        row[: table.numel()] = table.to(device=device, dtype=torch.int32)
        tables.append(row.unsqueeze(0).expand(q_len, width))
        lens.append(torch.arange(ctx + 1, ctx + q_len + 1, dtype=torch.int32, device=device))
    meta.prefill_row_tables = torch.cat(tables).contiguous()
    meta.prefill_row_lens = torch.cat(lens)
    return meta


def _causal_offset_mask(query_len: int, total_len: int, device, dtype) -> torch.Tensor:
    mask = torch.full((query_len, total_len), float("-inf"), device=device, dtype=dtype)
    return torch.triu(mask, diagonal=total_len - query_len + 1)


def _flat_pool(pool: torch.Tensor) -> torch.Tensor:
    if pool.ndim != 4:
        raise ValueError("this path writes by flat slot index and needs a [T, H_kv, num_slots, W] pool")
    return pool


def _prefill_chunks(q_dense, k_cache, v_cache, meta, out, num_q_heads, num_kv_heads, head_dim):
    """q_dense ``[T, H_q, n_tok, D]`` (any strides): SDPA of every prefill chunk against its sequence's
    cached prefix, read back from the packed pool (attention.py:161-178 of the reference).  The reference
    loops over the sequences; here chunks of one shape (query length, total length) that lie next to each
    other in the batch go through one read-back launch per pool and one SDPA call with the sequences as
    leading batch entries: the same arithmetic per sequence, a fraction of the launches."""
    dtype, device = q_dense.dtype, q_dense.device
    T = q_dense.shape[0]
    i, n = 0, meta.num_prefills
    while i < n:
        start, q_len = meta.prefill_query_starts[i], meta.prefill_query_lens[i]
        total = meta.prefill_context_lens[i] + q_len
        j = i + 1
        while (j < n and meta.prefill_query_lens[j] == q_len and meta.prefill_context_lens[j] + q_len == total
               and meta.prefill_query_starts[j] == start + (j - i) * q_len):
            j += 1
        b = j - i
        need = -(-total // meta.block_size)
        mask = _causal_offset_mask(q_len, total, device, dtype)
        if b == 1:
            table = meta.prefill_block_tables[i]
            k_all = gather_kv_unpacked(k_cache, table, total, head_dim, meta.block_size, dtype, status=meta.status)
            v_all = gather_kv_unpacked(v_cache, table, total, head_dim, meta.block_size, dtype, status=meta.status)
            o = F.scaled_dot_product_attention(q_dense[:, :, start:start + q_len], k_all, v_all, attn_mask=mask,
                                               enable_gqa=num_q_heads != num_kv_heads)
            out[:, start:start + q_len] = o.permute(0, 2, 1, 3)
        else:
            tables = torch.stack([t[:need].to(device=device, dtype=torch.int32) for t in meta.prefill_block_tables[i:j]])
            k_all = gather_kv_unpacked_batch(k_cache, tables, total, head_dim, meta.block_size, dtype, status=meta.status)
            v_all = gather_kv_unpacked_batch(v_cache, tables, total, head_dim, meta.block_size, dtype, status=meta.status)
            # [T, H_q, b * q_len, D] -> [b * T, H_q, q_len, D], sequences leading
            q = q_dense[:, :, start:start + b * q_len].unflatten(2, (b, q_len)).permute(2, 0, 1, 3, 4).flatten(0, 1)
            o = F.scaled_dot_product_attention(q, k_all.flatten(0, 1), v_all.flatten(0, 1), attn_mask=mask,
                                               enable_gqa=num_q_heads != num_kv_heads)
            # [b * T, H_q, q_len, D] -> out[T, b * q_len, H_q, D]
            out[:, start:start + b * q_len] = o.unflatten(0, (b, T)).permute(1, 0, 3, 2, 4).flatten(1, 2)
        i = j


def paged_attention(q_spk, k_spk, v_spk, k_cache, v_cache, meta: AttentionMetadata,
                    num_q_heads: int, num_kv_heads: int, head_dim: int) -> torch.Tensor:
    """Spike attention over the paged cache from dense spikes ``[T, 1, H, n_tok, head_dim]``.

    Persists this step's K/V (packed, at ``meta.slot_mapping``), runs the decode rows through the packed
    popcount kernel and the prefill chunks through SDPA on unpacked spikes.  Returns
    ``[T, 1, n_tok, H_q * head_dim]``.
    """
    T, n_tok = q_spk.shape[0], q_spk.shape[3]
    dtype, device = q_spk.dtype, q_spk.device
    _flat_pool(k_cache).index_copy_(2, meta.slot_mapping, pack_spikes(k_spk.squeeze(1)))
    _flat_pool(v_cache).index_copy_(2, meta.slot_mapping, pack_spikes(v_spk.squeeze(1)))
    out = torch.empty((T, n_tok, num_q_heads, head_dim), device=device, dtype=dtype)
    n_dec = meta.num_decode_tokens
    if n_dec:
        q_dec = q_spk[:, 0, :, :n_dec, :].permute(0, 2, 1, 3)  # [T, n_dec, H_q, D], read in place
        paged_spike_attn_decode(pack_spikes(q_dec), k_cache, v_cache, meta.block_tables, meta.seq_lens,
                                head_dim=head_dim, block_size=meta.block_size, num_q_heads=num_q_heads,
                                num_kv_heads=num_kv_heads, out=out[:, :n_dec], status=meta.status)
    if meta.num_prefills and meta.prefill_row_tables is not None:
        n_pre = meta.prefill_row_lens.numel()
        q_pre = q_spk[:, 0, :, n_dec:n_dec + n_pre, :].permute(0, 2, 1, 3)
        paged_spike_attn_decode(pack_spikes(q_pre), k_cache, v_cache, meta.prefill_row_tables, meta.prefill_row_lens,
                                head_dim=head_dim, block_size=meta.block_size, num_q_heads=num_q_heads,
                                num_kv_heads=num_kv_heads, out=out[:, n_dec:n_dec + n_pre], status=meta.status)
    else:
        _prefill_chunks(q_spk[:, 0], k_cache, v_cache, meta, out, num_q_heads, num_kv_heads, head_dim)
    return out.view(T, 1, n_tok, num_q_heads * head_dim)


def fused_qkv_attention(qkv: torch.Tensor, lif_q, lif_k, lif_v, k_cache, v_cache, meta: AttentionMetadata,
                        num_q_heads: int, num_kv_heads: int, head_dim: int, reset_mode: int = 0,
                        rope: tuple[torch.Tensor, torch.Tensor] | None = None) -> torch.Tensor:
    """Attention from the projection outputs ``qkv [T, n_tok, (H_q + 2 H_kv) * head_dim]``.

    One launch runs the LIF recurrence of the q, k and v sites, packs the spikes and scatters K/V
    straight into the pools through ``meta.slot_mapping``; the decode rows then go to the popcount
    kernel.  Dense q spikes are produced only when the batch holds prefill chunks.  ``lif_*`` are
    ``(beta, threshold)`` pairs.  ``rope = (cos, sin)``, each ``[n_tok, head_dim]`` in ``qkv.dtype``, applies the
    rotary embedding to the q and k currents inside the same launch; without it ``qkv`` must already be
    rotated.  Returns ``[T, n_tok, H_q * head_dim]`` in ``qkv.dtype``.
    """
    T, n_tok, _ = qkv.shape
    dtype, device = qkv.dtype, qkv.device
    hq, hkv, d = num_q_heads, num_kv_heads, head_dim
    W = packed_width(d)
    xq = qkv[..., : hq * d].unflatten(-1, (hq, d))
    xk = qkv[..., hq * d:(hq + hkv) * d].unflatten(-1, (hkv, d))
    xv = qkv[..., (hq + hkv) * d:].unflatten(-1, (hkv, d))
    q_packed = torch.empty((T, n_tok, hq, W), dtype=torch.int32, device=device)
    q_dense = None
    packed_prefill = meta.num_prefills and meta.prefill_row_tables is not None
    if meta.num_prefills and not packed_prefill:
        q_dense = torch.empty((T, hq, n_tok, d), dtype=dtype, device=device)
    kc, vc = _flat_pool(k_cache), _flat_pool(v_cache)
    num_slots = kc.shape[2]
    cos, sin = rope if rope is not None else (None, None)
    lif_pack_scatter([
        LifSiteSpec(x=xq, beta=lif_q[0], threshold=lif_q[1], packed=q_packed, rope_cos=cos, rope_sin=sin,
                    packed_strides=(n_tok * hq * W, hq * W, W), dense=q_dense,
                    dense_strides=None if q_dense is None else (q_dense.stride(0), q_dense.stride(2), q_dense.stride(1))),
        LifSiteSpec(x=xk, beta=lif_k[0], threshold=lif_k[1], packed=kc, rope_cos=cos, rope_sin=sin,
                    packed_strides=(kc.stride(0), kc.stride(2), kc.stride(1)),
                    slot_mapping=meta.slot_mapping, num_rows=num_slots),
        LifSiteSpec(x=xv, beta=lif_v[0], threshold=lif_v[1], packed=vc,
                    packed_strides=(vc.stride(0), vc.stride(2), vc.stride(1)),
                    slot_mapping=meta.slot_mapping, num_rows=num_slots),
    ], reset_mode=reset_mode, status=meta.status)
    out = torch.empty((T, n_tok, hq, d), device=device, dtype=dtype)
    n_dec = meta.num_decode_tokens
    if n_dec:
        # directly behind the LIF launch: nothing but allocations in between
        paged_spike_attn_decode(q_packed[:, :n_dec], k_cache, v_cache, meta.block_tables, meta.seq_lens,
                                head_dim=d, block_size=meta.block_size, num_q_heads=hq, num_kv_heads=hkv,
                                out=out[:, :n_dec], status=meta.status, overlap_previous=meta.tables_settled)
    if packed_prefill:
        n_pre = meta.prefill_row_lens.numel()
        paged_spike_attn_decode(q_packed[:, n_dec:n_dec + n_pre], k_cache, v_cache, meta.prefill_row_tables,
                                meta.prefill_row_lens, head_dim=d, block_size=meta.block_size, num_q_heads=hq,
                                num_kv_heads=hkv, out=out[:, n_dec:n_dec + n_pre], status=meta.status)
    elif meta.num_prefills:
        _prefill_chunks(q_dense, k_cache, v_cache, meta, out, hq, hkv, d)
    return out.view(T, n_tok, hq * d)
