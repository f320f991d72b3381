"""Fused multi-timestep LIF (CUDA): the reference operator and the fused pack/scatter form.

``lif_multistep`` keeps the signature, the assertions and the "no device sync" rule of
``spikeinfer/kernels/lif_triton.py:141-233``; ``validate_thresholds`` is :236-253.
``lif_pack_scatter`` is the added fused operator: LIF, bit-pack and (for K/V) the
slot-mapped write into the paged pool in one launch for up to four neuron sites.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from .. import _lib
from .packing import _leading_dims, packed_width

SUBTRACT_DELAYED = _lib.RESET_SUBTRACT_DELAYED
HARD_ZERO = _lib.RESET_HARD_ZERO


def _param(p: torch.Tensor, device: torch.device) -> torch.Tensor:
    p = p.detach()
    if p.dtype != torch.float32 or p.device != device or not p.is_contiguous():
        p = p.to(device=device, dtype=torch.float32).contiguous()
    return p


def lif_multistep(x, beta, threshold, mem0=None, out_dtype=None, return_membrane=False,
                  reset_mode: int = SUBTRACT_DELAYED):
    """T-step LIF over ``x [T, *mid, N]`` in one launch; ``beta``/``threshold`` are ``[N]``.

    Returns spikes ``[T, *mid, N]`` in ``out_dtype`` (default ``x.dtype``; ``torch.uint8`` allowed)
    and, if ``return_membrane``, the final fp32 membrane ``[*mid, N]``.  ``threshold > 0`` is a
    precondition checked once by :func:`validate_thresholds`, never here (a check would need a
    device-to-host sync, which is illegal during graph capture).  Permuted inputs whose channel
    axis is contiguous are read in place.
    """
    assert x.ndim >= 2, "expected [T, *mid, N]"
    N = x.shape[-1]
    assert beta.numel() == N and threshold.numel() == N, (
        f"beta/threshold must match trailing dim: got {beta.numel()}/{threshold.numel()} vs N={N}"
    )
    _lib.require_cuda(x, "lif_multistep input")
    out_dtype = out_dtype or x.dtype
    T = x.shape[0]
    mid_shape = tuple(x.shape[1:-1])
    if x.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        x = x.float()
    if x.stride(-1) != 1 and N > 1:
        x = x.contiguous()
    sizes, strides = _leading_dims(x, first=1)
    if len(sizes) > 6:
        x = x.contiguous()
        sizes, strides = _leading_dims(x, first=1)
    M = 1
    for s in mid_shape:
        M *= s

    dev = x.device
    beta = _param(beta, dev)
    threshold = _param(threshold, dev)
    spikes = torch.empty(x.shape, device=dev, dtype=out_dtype)
    u_out = torch.empty((*mid_shape, N), device=dev, dtype=torch.float32) if return_membrane else None
    u_in = None
    if mem0 is not None:
        u_in = mem0.reshape(M, N).to(device=dev, dtype=torch.float32).contiguous()
    if spikes.numel() or (return_membrane and M * N):
        lib = _lib.load()
        with torch.cuda.device(dev):
            rc = lib.spk_lif(x.data_ptr(), _lib.dtype_code(x.dtype), T, x.stride(0) if T > 0 else 0,
                             len(sizes), _lib.i64_array(sizes), _lib.i64_array(strides), N,
                             beta.data_ptr(), threshold.data_ptr(), _lib.ptr(u_in), spikes.data_ptr(),
                             _lib.dtype_code(out_dtype), _lib.ptr(u_out), reset_mode,
                             _lib.current_stream(dev))
        _lib.check(rc, "spk_lif")
    if return_membrane:
        return spikes, u_out
    return spikes


def validate_thresholds(model) -> bool:
    """Check ``threshold > 0`` at every LIF site of ``model`` (modules with a ``.lif.threshold``)."""
    bad = []
    for name, module in model.named_modules():
        lif = getattr(module, "lif", None)
        th = getattr(lif, "threshold", None) if lif is not None else None
        if th is not None and not bool(torch.all(th > 0)):
            bad.append(f"{name} (min={th.min().item():.4g})")
    if bad:
        raise ValueError("lif_multistep requires threshold > 0; violated at: " + ", ".join(bad))
    return True


@dataclass
class LifSiteSpec:
    """One neuron site of a fused launch.

    ``x``: currents ``[T, n_tok, H, N]`` (any strides with a contiguous channel axis).
    ``packed``: int32 destination addressed ``[t, row, h, w]`` through ``packed_strides``
    (element strides of t, row, h); ``row`` is ``slot_mapping[tok]`` if given, else ``tok``.
    ``dense``: optional 0/1 spike output addressed ``[t, tok, h, c]`` through ``dense_strides``.
    """

    x: torch.Tensor
    beta: torch.Tensor
    threshold: torch.Tensor
    packed: torch.Tensor | None = None
    packed_strides: tuple[int, int, int] | None = None
    slot_mapping: torch.Tensor | None = None
    num_rows: int = 0
    dense: torch.Tensor | None = None
    dense_strides: tuple[int, int, int] | None = None
    mem0: torch.Tensor | None = None
    mem_out: torch.Tensor | None = None
    rope_cos: torch.Tensor | None = None
    """Optional ``[n_tok, N]`` cos / sin (dtype of ``x``): rotary embedding applied to the currents first."""
    rope_sin: torch.Tensor | None = None
    mul: torch.Tensor | None = None
    """Optional ``[T, n_tok, H, N]`` (dtype of ``x``, any strides with a contiguous channel axis)."""
    gated: torch.Tensor | None = None
    """Output of the gated product ``spike ? mul : 0``, same shape and dtype as ``mul``."""


def lif_pack_scatter(sites: list[LifSiteSpec], reset_mode: int = SUBTRACT_DELAYED,
                     status: torch.Tensor | None = None) -> None:
    """Run LIF + bit-pack (+ slot-mapped scatter) for up to four sites in one launch."""
    if not 1 <= len(sites) <= _lib.MAX_LIF_SITES:
        raise ValueError(f"between 1 and {_lib.MAX_LIF_SITES} sites per launch, got {len(sites)}")
    T, n_tok = sites[0].x.shape[0], sites[0].x.shape[1]
    dev = sites[0].x.device
    arr = (_lib.LifSite * len(sites))()
    keep = []
    for i, s in enumerate(sites):
        x = s.x
        _lib.require_cuda(x, "lif_pack_scatter input")
        if x.ndim != 4 or x.shape[0] != T or x.shape[1] != n_tok:
            raise ValueError(f"site {i}: expected [T={T}, n_tok={n_tok}, H, N], got {tuple(x.shape)}")
        if x.stride(-1) != 1 and x.shape[-1] > 1:
            raise ValueError(f"site {i}: channel axis must be contiguous")
        H, N = x.shape[2], x.shape[3]
        if s.beta.numel() != N or s.threshold.numel() != N:
            raise ValueError(f"site {i}: beta/threshold must have N={N} elements")
        beta, th = _param(s.beta, dev), _param(s.threshold, dev)
        keep += [beta, th]
        e = arr[i]
        e.x, e.x_dtype, e.H, e.N = x.data_ptr(), _lib.dtype_code(x.dtype), H, N
        e.sx_t, e.sx_tok, e.sx_h = x.stride(0), x.stride(1), x.stride(2)
        e.beta, e.threshold = beta.data_ptr(), th.data_ptr()
        if s.mem0 is not None:
            if s.mem0.dtype != torch.float32 or not s.mem0.is_contiguous() or s.mem0.numel() != n_tok * H * N:
                raise ValueError(f"site {i}: mem0 must be contiguous fp32 [n_tok, H, N]")
            e.mem0 = s.mem0.data_ptr()
        if s.mem_out is not None:
            if s.mem_out.dtype != torch.float32 or not s.mem_out.is_contiguous() or s.mem_out.numel() != n_tok * H * N:
                raise ValueError(f"site {i}: mem_out must be contiguous fp32 [n_tok, H, N]")
            e.mem_out = s.mem_out.data_ptr()
        if s.packed is not None:
            if s.packed.dtype != torch.int32:
                raise TypeError(f"site {i}: packed destination must be int32")
            e.packed = s.packed.data_ptr()
            e.so_t, e.so_tok, e.so_h = s.packed_strides
            if s.slot_mapping is not None:
                if s.slot_mapping.dtype != torch.int64 or s.slot_mapping.numel() < n_tok:
                    raise ValueError(f"site {i}: slot_mapping must be int64 [n_tok]")
                e.slot_mapping = s.slot_mapping.data_ptr()
                e.num_rows = s.num_rows
        if s.dense is not None:
            e.dense = s.dense.data_ptr()
            e.dense_dtype = _lib.dtype_code(s.dense.dtype)
            e.sd_t, e.sd_tok, e.sd_h = s.dense_strides
        if s.rope_cos is not None:
            cos, sin = s.rope_cos, s.rope_sin
            if cos.dtype != x.dtype or sin.dtype != x.dtype or cos.shape != (n_tok, N) or sin.shape != (n_tok, N):
                raise ValueError(f"site {i}: rope cos/sin must be [n_tok, N] in the dtype of x")
            if cos.stride(1) != 1 or sin.stride(1) != 1 or cos.stride(0) != sin.stride(0):
                raise ValueError(f"site {i}: rope cos/sin must share a row stride and have contiguous rows")
            e.rope_cos, e.rope_sin, e.s_rope_tok = cos.data_ptr(), sin.data_ptr(), cos.stride(0)
        if s.gated is not None:
            for name, t in (("mul", s.mul), ("gated", s.gated)):
                if t is None or t.dtype != x.dtype or t.shape != x.shape or t.stride(3) != 1:
                    raise ValueError(f"site {i}: {name} must match x in shape and dtype with a contiguous channel axis")
            e.mul, e.gated = s.mul.data_ptr(), s.gated.data_ptr()
            e.sm_t, e.sm_tok, e.sm_h = s.mul.stride(0), s.mul.stride(1), s.mul.stride(2)
            e.sg_t, e.sg_tok, e.sg_h = s.gated.stride(0), s.gated.stride(1), s.gated.stride(2)
    if n_tok == 0 or T == 0:
        return
    lib = _lib.load()
    with torch.cuda.device(dev):
        rc = lib.spk_lif_pack_scatter(arr, len(sites), T, n_tok, reset_mode, _lib.ptr(status),
                                      _lib.current_stream(dev))
    _lib.check(rc, "spk_lif_pack_scatter")


def lif_pack(x: torch.Tensor, beta: torch.Tensor, threshold: torch.Tensor, *, dense_dtype=None,
             return_membrane: bool = False, reset_mode: int = SUBTRACT_DELAYED):
    """LIF + pack of ``x [T, n_tok, N]`` (e.g. the MLP gate): returns ``int32 [T, n_tok, ceil(N/32)]``
    and optionally the dense spikes and the final membrane, all from one read of ``x``."""
    T, n_tok, N = x.shape
    W = packed_width(N)
    packed = torch.empty((T, n_tok, W), dtype=torch.int32, device=x.device)
    dense = torch.empty((T, n_tok, N), dtype=dense_dtype, device=x.device) if dense_dtype else None
    mem = torch.empty((n_tok, N), dtype=torch.float32, device=x.device) if return_membrane else None
    site = LifSiteSpec(
        x=x.unsqueeze(2), beta=beta, threshold=threshold, packed=packed,
        packed_strides=(n_tok * W, W, 0), dense=dense,
        dense_strides=(n_tok * N, N, 0) if dense is not None else None, mem_out=mem,
    )
    lif_pack_scatter([site], reset_mode=reset_mode)
    return packed, dense, mem


def lif_gate_mul(gate: torch.Tensor, up: torch.Tensor, beta: torch.Tensor, threshold: torch.Tensor,
                 reset_mode: int = SUBTRACT_DELAYED) -> torch.Tensor:
    """``lif_multistep(gate) * up`` in one launch: ``[T, n_tok, N]`` currents and multiplicand (strided views of
    one GEMM output are fine) -> contiguous ``[T, n_tok, N]`` product; the dense spikes are never written."""
    T, n_tok, N = gate.shape
    out = torch.empty((T, n_tok, N), dtype=gate.dtype, device=gate.device)
    lif_pack_scatter([LifSiteSpec(x=gate.unsqueeze(2), beta=beta, threshold=threshold, mul=up.unsqueeze(2),
                                  gated=out.unsqueeze(2))], reset_mode=reset_mode)
    return out
