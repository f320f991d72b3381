"""Residual add + RMSNorm (CUDA), the two operators between the sublayers of a decoder layer
(``spikeinfer/modeling_fast.py:206-211`` with transformers' ``Qwen2RMSNorm``)."""
from __future__ import annotations

import torch

from .. import _lib


def add_rms_norm(h: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                 out: torch.Tensor | None = None) -> torch.Tensor:
    """``h += delta`` in place (skipped when ``delta`` is None), then returns ``weight * rmsnorm(h)``.

    ``h`` and ``delta`` are contiguous ``[..., hidden]`` in the same dtype; the variance is fp32 and the
    normalised value is rounded to the dtype before the weight multiplies it, as Qwen2RMSNorm does.
    """
    _lib.require_cuda(h, "add_rms_norm input")
    if not h.is_contiguous() or (delta is not None and (not delta.is_contiguous() or delta.shape != h.shape or delta.dtype != h.dtype)):
        raise ValueError("h and delta must be contiguous, same shape and dtype")
    hidden = h.shape[-1]
    if weight.dtype != h.dtype or weight.numel() != hidden or not weight.is_contiguous():
        raise ValueError("weight must be a contiguous [hidden] tensor in the dtype of h")
    if out is None:
        out = torch.empty_like(h)
    rows = h.numel() // hidden
    lib = _lib.load()
    with torch.cuda.device(h.device):
        rc = lib.spk_add_rmsnorm(h.data_ptr(), _lib.ptr(delta), weight.data_ptr(), eps, out.data_ptr(), rows, hidden,
                                 _lib.dtype_code(h.dtype), _lib.current_stream(h.device))
    _lib.check(rc, "spk_add_rmsnorm")
    return out
