"""Greedy sampling on the device (CUDA): the ``logits.argmax(dim=-1)`` of the reference's sampler
(``spikeinfer/engine/sampler.py:63-81``) as two small launches with fixed arguments, capturable in the decode
graph."""
from __future__ import annotations

import torch

from .. import _lib


def argmax_rows(logits: torch.Tensor, out: torch.Tensor | None = None,
                workspace: torch.Tensor | None = None) -> torch.Tensor:
    """``out[r] = logits[r].argmax()`` for ``logits [rows, vocab]`` (fp32, bf16 or fp16; unit stride along the
    vocabulary), with ``torch.argmax``'s rules: first index of the largest value, NaN above everything.

    ``out`` is int64 ``[rows]``; ``workspace`` a uint8 buffer of at least ``argmax_workspace_bytes(rows)`` bytes
    (pass both when the call is captured in a CUDA graph, so that nothing is allocated during capture)."""
    _lib.require_cuda(logits, "argmax_rows input")
    if logits.ndim != 2 or logits.stride(1) != 1:
        raise ValueError("logits must be [rows, vocab] with unit stride along the vocabulary")
    rows, cols = logits.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int64, device=logits.device)
    elif out.dtype != torch.int64 or out.numel() != rows or not out.is_contiguous() or out.device != logits.device:
        raise ValueError("out must be a contiguous int64 [rows] tensor on the device of logits")
    lib = _lib.load()
    need = lib.spk_argmax_workspace_bytes(rows)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=logits.device)
    elif workspace.numel() * workspace.element_size() < need or workspace.device != logits.device:
        raise ValueError(f"workspace must hold {need} bytes on the device of logits")
    with torch.cuda.device(logits.device):
        rc = lib.spk_argmax(logits.data_ptr(), _lib.dtype_code(logits.dtype), rows, cols, logits.stride(0),
                            out.data_ptr(), workspace.data_ptr(), workspace.numel() * workspace.element_size(),
                            _lib.current_stream(logits.device))
    _lib.check(rc, "spk_argmax")
    return out


def argmax_workspace_bytes(rows: int) -> int:
    return int(_lib.load().spk_argmax_workspace_bytes(rows))
