"""ctypes binding of ``libspikeinfer_b200.so`` (the C ABI declared in ``include/spikeinfer_b200.h``).

There is no fallback: if the library is missing or a call fails, the operators raise.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_uint32, c_void_p
from pathlib import Path

import torch

LIB_PATH = Path(os.environ.get("SPIKEINFER_B200_LIB") or Path(__file__).resolve().parent / "libspikeinfer_b200.so")

# element type codes (include/spikeinfer_b200.h)
F32, BF16, F16, U8, I32 = 0, 1, 2, 3, 4
RESET_SUBTRACT_DELAYED, RESET_HARD_ZERO = 0, 1

STATUS_BAD_BLOCK = 1 << 0
STATUS_BAD_SEQ_LEN = 1 << 1
STATUS_BAD_SLOT = 1 << 2
STATUS_POOL_EXHAUSTED = 1 << 3
STATUS_TABLE_FULL = 1 << 4
STATUS_FREE_LIST_OVERFLOW = 1 << 5
STATUS_ROW_BUSY = 1 << 6
STATUS_DEVICE_WAIT_EXPIRED = 1 << 7

MAX_LIF_SITES = 4

ATTN_FORM_AUTO, ATTN_FORM_GENERAL, ATTN_FORM_TCGEN05 = 0, 1, 2

_DTYPE_CODES = {
    torch.float32: F32,
    torch.bfloat16: BF16,
    torch.float16: F16,
    torch.uint8: U8,
    torch.int32: I32,
}


class SpkError(RuntimeError):
    """A C-ABI call returned a non-zero status."""


class LifSite(Structure):
    """Mirror of ``spk_lif_site``."""

    _fields_ = [
        ("x", c_void_p),
        ("x_dtype", c_int32),
        ("H", c_int32),
        ("N", c_int64),
        ("sx_t", c_int64),
        ("sx_tok", c_int64),
        ("sx_h", c_int64),
        ("beta", c_void_p),
        ("threshold", c_void_p),
        ("mem0", c_void_p),
        ("mem_out", c_void_p),
        ("packed", c_void_p),
        ("so_t", c_int64),
        ("so_tok", c_int64),
        ("so_h", c_int64),
        ("slot_mapping", c_void_p),
        ("num_rows", c_int64),
        ("dense", c_void_p),
        ("dense_dtype", c_int32),
        ("_pad", c_int32),
        ("sd_t", c_int64),
        ("sd_tok", c_int64),
        ("sd_h", c_int64),
        ("rope_cos", c_void_p),
        ("rope_sin", c_void_p),
        ("s_rope_tok", c_int64),
        ("mul", c_void_p),
        ("sm_t", c_int64),
        ("sm_tok", c_int64),
        ("sm_h", c_int64),
        ("gated", c_void_p),
        ("sg_t", c_int64),
        ("sg_tok", c_int64),
        ("sg_h", c_int64),
    ]


# name -> (restype, argtypes); every symbol include/spikeinfer_b200.h declares
I64P = POINTER(c_int64)
SIGNATURES = {
    "spk_version": (c_int, []),
    "spk_last_cuda_error": (c_int, []),
    "spk_error_string": (c_char_p, [c_int]),
    "spk_launch_count": (c_int64, []),
    "spk_nvtx_enabled": (c_int, []),
    "spk_attn_overlap_next_call": (c_int, []),
    "spk_pack": (c_int, [c_void_p, c_int, c_int, I64P, I64P, c_int64, c_void_p, c_void_p]),
    "spk_unpack": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int, c_void_p]),
    "spk_lif": (c_int, [c_void_p, c_int, c_int, c_int64, c_int, I64P, I64P, c_int64, c_void_p,
                        c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p]),
    "spk_lif_pack_scatter": (c_int, [POINTER(LifSite), c_int, c_int, c_int64, c_int, c_void_p, c_void_p]),
    "spk_add_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "spk_argmax_workspace_bytes": (c_int64, [c_int64]),
    "spk_argmax": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_void_p]),
    "spk_attn_decode_workspace_bytes": (c_int64, [c_int, c_int64, c_int, c_int, c_int, c_int, c_int64]),
    "spk_attn_decode": (c_int, [
        c_void_p, c_int64, c_int64, c_int64,
        c_void_p, c_int64, c_int64, c_int64, c_int64,
        c_void_p, c_int64, c_int64, c_int64, c_int64,
        c_void_p, c_int64, c_void_p,
        c_void_p, c_int, c_int64, c_int64, c_int64,
        c_int, c_int64, c_int, c_int, c_int, c_int, c_int64, c_int64, c_float,
        c_void_p, c_int64, c_void_p, c_void_p]),
    "spk_attn_decode_static_capacity": (c_int64, []),
    "spk_attn_decode_static": (c_int, [
        c_void_p, c_int64, c_int64, c_int64,
        c_void_p, c_int64, c_int64, c_int64, c_int64,
        c_void_p, c_int64, c_int64, c_int64, c_int64,
        c_void_p, c_int64, c_void_p,
        c_void_p, c_int, c_int64, c_int64, c_int64,
        c_int, c_int64, c_int, c_int, c_int, c_int, c_int64, c_int64, c_float,
        c_void_p, c_void_p]),
    "spk_qk_scores": (c_int, [
        c_void_p, c_int64, c_int64, c_int64,
        c_void_p, c_int64, c_int64, c_int64, c_int64,
        c_void_p, c_int64, c_void_p,
        c_void_p, c_int64, c_int, c_int64, c_int, c_int, c_int, c_int, c_int64, c_int64,
        c_void_p, c_void_p]),
    "spk_gather_kv_unpacked": (c_int, [
        c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int,
        c_int64, c_void_p, c_int, c_void_p, c_void_p]),
    "spk_gather_kv_unpacked_batch": (c_int, [
        c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int,
        c_int64, c_void_p, c_int, c_void_p, c_void_p]),
    "spk_meta_init": (c_int, [c_void_p, c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p]),
    "spk_meta_advance": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p,
                                 c_void_p]),
    "spk_attn_select_form": (c_int, [c_int]),
    "spk_meta_admit": (c_int, [c_int32, c_void_p, c_int32, c_int64, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32,
                               c_int32, c_void_p, c_void_p]),
    "spk_meta_take": (c_int, [c_void_p, c_void_p, c_int32, c_void_p, c_void_p, c_void_p]),
    "spk_meta_release": (c_int, [c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_int32, c_int32, c_int32, c_int32, c_int32, c_void_p, c_void_p]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library once and declare every entry point's signature."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise SpkError(
            f"{LIB_PATH} is missing: build it with `python -m spikeinfer_b200.build` "
            "(there is no fallback path)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(code: int, what: str) -> None:
    if code == 0:
        return
    lib = load()
    msg = lib.spk_error_string(code).decode()
    if code == -100:
        msg += f" [cudaError {lib.spk_last_cuda_error()}]"
    raise SpkError(f"{what}: {msg} ({code})")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODES[dtype]
    except KeyError:
        raise TypeError(f"{dtype} is not supported by the CUDA kernels") from None


def require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise SpkError(
            f"{name} is on {t.device}: spikeinfer_b200 operators run on CUDA tensors only "
            "(there is no CPU path)"
        )


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def current_stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def i64_array(values) -> ctypes.Array:
    values = list(values)
    return (c_int64 * max(len(values), 1))(*values)
