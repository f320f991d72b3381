"""Bit packing of spike tensors (CUDA).

Same operator surface as ``spikeinfer/kernels/packing.py`` of the reference
(``pack_spikes`` :84, ``unpack_spikes`` :136, ``packed_width`` :46,
``packed_bytes_per_token`` :155): bit ``i`` of word ``w`` holds channel ``32*w + i``,
words are ``int32`` whose sign bit is a value bit, and the tail of the last word is zero.
"""
from __future__ import annotations

import torch

from .. import _lib

BITS_PER_WORD = 32


def packed_width(num_channels: int) -> int:
    """Words needed to hold ``num_channels`` spikes (64 -> 2)."""
    return (num_channels + BITS_PER_WORD - 1) // BITS_PER_WORD


def packed_bytes_per_token(num_layers: int, num_timesteps: int, num_kv_heads: int, head_dim: int) -> int:
    """Bytes of packed K plus V one cached token costs over the whole model."""
    return 2 * num_layers * num_timesteps * num_kv_heads * packed_width(head_dim) * 4


def _leading_dims(x: torch.Tensor, first: int = 0):
    """Sizes/strides of ``x``'s dims ``first..-2`` with unit dims dropped and mergeable neighbours merged."""
    sizes, strides = [], []
    for size, stride in zip(x.shape[first:-1], x.stride()[first:-1]):
        if size == 1:
            continue
        if sizes and strides[-1] == stride * size:
            sizes[-1] *= size
            strides[-1] = stride
        else:
            sizes.append(size)
            strides.append(stride)
    return sizes, strides


def pack_spikes(x: torch.Tensor) -> torch.Tensor:
    """``[..., C]`` (anything nonzero is a spike) -> ``int32 [..., ceil(C/32)]``.

    Strided (e.g. permuted) inputs are read in place as long as the channel axis is
    contiguous; no ``.contiguous()`` copy is made for them.
    """
    _lib.require_cuda(x, "pack_spikes input")
    if x.dtype == torch.bool:
        x = x.view(torch.uint8)
    channels = x.shape[-1]
    out = torch.empty((*x.shape[:-1], packed_width(channels)), dtype=torch.int32, device=x.device)
    if out.numel() == 0:
        return out
    code = _lib.dtype_code(x.dtype)
    if x.stride(-1) != 1 and channels > 1:
        x = x.contiguous()
    sizes, strides = _leading_dims(x)
    if len(sizes) > 6:
        x = x.contiguous()
        sizes, strides = _leading_dims(x)
    lib = _lib.load()
    with torch.cuda.device(x.device):
        rc = lib.spk_pack(x.data_ptr(), code, len(sizes), _lib.i64_array(sizes), _lib.i64_array(strides),
                          channels, out.data_ptr(), _lib.current_stream(x.device))
    _lib.check(rc, "spk_pack")
    return out


def unpack_spikes(words: torch.Tensor, num_channels: int, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``int32 [..., W]`` -> ``[..., num_channels]`` of 0/1 in ``dtype``; inverse of :func:`pack_spikes`."""
    expected = packed_width(num_channels)
    if words.shape[-1] != expected:
        raise ValueError(f"expected {expected} words for {num_channels} channels, got {words.shape[-1]}")
    _lib.require_cuda(words, "unpack_spikes input")
    if words.dtype != torch.int32:
        raise TypeError(f"packed words must be int32, got {words.dtype}")
    words = words.contiguous()
    out = torch.empty((*words.shape[:-1], num_channels), dtype=dtype, device=words.device)
    if out.numel() == 0:
        return out
    rows = words.numel() // expected
    lib = _lib.load()
    with torch.cuda.device(words.device):
        rc = lib.spk_unpack(words.data_ptr(), rows, num_channels, out.data_ptr(), _lib.dtype_code(dtype),
                            _lib.current_stream(words.device))
    _lib.check(rc, "spk_unpack")
    return out
