"""The C-ABI library: it builds, loads and exports exactly what include/spikeinfer_b200.h declares.
Host-side argument validation is exercised too; none of these calls launches a kernel."""
from __future__ import annotations

import ctypes
import dataclasses
import inspect
import json
import re
from pathlib import Path

from spikeinfer_b200 import _lib

HEADER = Path(__file__).resolve().parent.parent / "include" / "spikeinfer_b200.h"


def declared_symbols() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return re.findall(r"^\s*(?:const\s+char\s*\*|int64_t|int)\s+(spk_\w+)\s*\(", text, flags=re.M)


def test_header_and_binding_agree():
    names = declared_symbols()
    assert len(names) == len(set(names)) and len(names) >= 15
    assert set(names) == set(_lib.SIGNATURES)


def test_library_exports_every_declared_symbol(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared but not exported"


def test_version_and_error_strings(lib):
    assert lib.spk_version() == (0 << 16) | (1 << 8) | 0
    assert lib.spk_error_string(0) == b"ok"
    assert b"workspace" in lib.spk_error_string(-5)
    assert b"unknown" in lib.spk_error_string(-12345)
    assert lib.spk_last_cuda_error() == 0


def test_site_struct_layout():
    # 3 pointers/ints block + strides: must match `spk_lif_site` (all members 8-byte aligned)
    assert ctypes.sizeof(_lib.LifSite) == 8 + 4 + 4 + 8 + 24 + 32 + 8 + 24 + 8 + 8 + 8 + 4 + 4 + 24 + 24 + 32 + 32


def test_host_side_argument_checks(lib):
    one = _lib.i64_array([1])
    assert lib.spk_pack(None, _lib.F32, 1, one, one, 0, None, None) == -2       # no channels
    assert lib.spk_pack(None, 99, 1, one, one, 8, None, None) == -4             # null before dtype
    assert lib.spk_pack(1, 99, 1, one, one, 8, 1, None) == -1                   # bad dtype
    assert lib.spk_pack(None, _lib.F32, 7, one, one, 8, None, None) == -2       # too many dims
    assert lib.spk_unpack(None, 0, 8, None, _lib.F32, None) == 0                # empty is fine
    assert lib.spk_lif(None, _lib.F32, 4, 0, 1, one, one, 8, None, None, None, None, _lib.F32, None, 7, None) == -6
    assert lib.spk_lif_pack_scatter(None, 1, 4, 1, 0, None, None) == -4
    # attention: head_dim must be a multiple of 32 up to 128, block_size a power of two
    args = lambda hd, bs: (1, 0, 0, 0, 1, 0, 0, 0, 0, 1, 0, 0, 0, 0, 1, 0, 1, 1, _lib.F32, 0, 0, 0,
                           4, 2, 14, 2, hd, bs, 4, 8, 0.125, None, 0, None, None)
    assert lib.spk_attn_decode(*args(48, 16)) == -6
    assert lib.spk_attn_decode(*args(64, 12)) == -6
    assert lib.spk_attn_decode(*args(256, 16)) == -6
    # workspace of the streaming form: two partial records per worker warp, and only when a
    # sequence can be long enough (more than 256 keys) to be cut between warps.  Workers: one per eight 32-key
    # steps of the fully loaded batch, at most 148 SMs x 16 warps.
    record = (8 * 64 + 8) * 4                    # eight heads x 64 sums + 8 totals, fp32
    assert lib.spk_attn_decode_workspace_bytes(4, 64, 14, 2, 64, 16, 1) == 0
    assert lib.spk_attn_decode_workspace_bytes(4, 64, 14, 2, 64, 16, 16) == 0
    # tables of up to 768 keys are never cut (one warp walks such a row faster than a combine pass would cost)
    # (what is left at 48 pages are the two 512-key unit records per item of the selectable tcgen05 form)
    assert lib.spk_attn_decode_workspace_bytes(4, 64, 14, 2, 64, 16, 48) == 64 * 4 * 2 * 2 * record
    assert lib.spk_attn_decode_workspace_bytes(4, 64, 14, 2, 64, 16, 49) == (64 * 4 * 2 * 25 // 8) * 2 * record
    assert lib.spk_attn_decode_workspace_bytes(4, 64, 14, 2, 64, 16, 256) == 148 * 16 * 2 * record
    ws = lib.spk_attn_decode_workspace_bytes(4, 8, 14, 2, 64, 16, 256)
    assert ws == (8 * 4 * 2 * 128 // 8) * 2 * record
    assert lib.spk_attn_decode_workspace_bytes(4, 64, 14, 2, 48, 16, 256) == 0
    # workspace required but missing -> rejected on the host, nothing launched
    big = (1, 0, 0, 0, 1, 0, 0, 0, 0, 1, 0, 0, 0, 0, 1, 0, 1, 1, _lib.F32, 0, 0, 0,
           4, 8, 14, 2, 64, 16, 256, 8, 0.125, None, 0, None, None)
    assert lib.spk_attn_decode(*big) == -5
    # a softmax range the fp16 weight pairs cannot hold (head_dim * scale > 24) is refused
    wide = big[:-5] + (1.0, None, 0, None, None)
    assert lib.spk_attn_decode(*wide) == -6
    assert lib.spk_meta_advance(1, 1, 1, 1, 1, 1, 1, 1, None, 2048, 4, 0, 16, None, None) == -2
    # greedy sampling: shape, dtype, null and workspace checks happen before any launch
    assert lib.spk_argmax_workspace_bytes(0) == 0 and lib.spk_argmax_workspace_bytes(64) == 64 * 16 * 12
    assert lib.spk_argmax(1, _lib.BF16, 4, 0, 8, 1, 1, 1 << 20, None) == -2         # no columns
    assert lib.spk_argmax(1, _lib.BF16, 4, 16, 8, 1, 1, 1 << 20, None) == -2        # row stride below the width
    assert lib.spk_argmax(1, _lib.U8, 4, 16, 16, 1, 1, 1 << 20, None) == -1         # dtype
    assert lib.spk_argmax(None, _lib.F32, 0, 16, 16, None, None, 0, None) == 0      # no rows: nothing to do
    assert lib.spk_argmax(None, _lib.F32, 4, 16, 16, 1, 1, 1 << 20, None) == -4     # null logits
    assert lib.spk_argmax(1, _lib.F32, 4, 16, 16, 1, None, 0, None) == -5           # workspace missing
    assert lib.spk_argmax(1, _lib.F32, 70000, 16, 16, 1, 1, 1 << 30, None) == -7    # more rows than a grid dimension


def _params(fn):
    out = []
    for prm in inspect.signature(fn).parameters.values():
        has_default = prm.default is not inspect.Parameter.empty
        out.append(dict(name=prm.name, kind=prm.kind.name, has_default=has_default,
                        default=repr(prm.default) if has_default else None))
    return out


def test_operator_surface_matches_the_reference():
    """Drop-in conformance: every operator the reference's ``kernels`` package exports for this path exists here
    under the same name with the same leading parameters (name, order, kind, default); extra parameters are
    allowed only at the end and only with defaults.  ``AttentionMetadata`` keeps every public field, in order.
    The recorded surface comes from the reference itself (tests/golden/make_golden.py)."""
    from spikeinfer_b200 import attention, kernels

    surface = json.loads((Path(__file__).parent / "golden" / "interface.json").read_text())
    # the reference's own CPU restatements are its test oracles, not operators of the path: there is no CPU path here
    not_provided = {"lif_multistep_ref", "paged_spike_attn_decode_ref", "paged_spike_attn_decode_cpu"}
    checked = 0
    for name, entry in surface.items():
        if name in not_provided or name == "AttentionMetadata":
            continue
        where = attention if name == "paged_attention" else kernels
        assert hasattr(where, name), f"{name} is missing"
        mine = getattr(where, name)
        if "value" in entry:
            assert mine == entry["value"], name
            continue
        got, want = _params(mine), entry["params"]
        assert got[: len(want)] == want, f"{name}: {got[:len(want)]} != {want}"
        for extra in got[len(want):]:
            assert extra["has_default"], f"{name}: extra parameter {extra['name']} needs a default"
        checked += 1
    assert checked >= 8
    assert not_provided <= set(surface), "the reference's export list changed"
    mine = [f.name for f in dataclasses.fields(attention.AttentionMetadata)]
    theirs = [f["name"] for f in surface["AttentionMetadata"]["fields"] if f["public"]]
    assert mine[: len(theirs)] == theirs
    defaults = {f.name: (f.default is not dataclasses.MISSING or f.default_factory is not dataclasses.MISSING)
                for f in dataclasses.fields(attention.AttentionMetadata)}
    for f in surface["AttentionMetadata"]["fields"]:
        if f["public"]:
            assert defaults[f["name"]] == f["has_default"], f["name"]
    for extra in mine[len(theirs):]:
        assert defaults[extra], f"extra metadata field {extra} needs a default"


def test_nvtx_ranges_follow_the_environment():
    """SPK_NVTX switches the NVTX ranges of the entry points on; the default is off (one fresh process each)."""
    import os
    import subprocess
    import sys
    code = "from spikeinfer_b200 import _lib; print(_lib.load().spk_nvtx_enabled())"
    root = str(Path(__file__).resolve().parent.parent)
    for value, want in ((None, "0"), ("1", "1"), ("0", "0")):
        env = {k: v for k, v in os.environ.items() if k != "SPK_NVTX"}
        if value is not None:
            env["SPK_NVTX"] = value
        out = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True, check=True)
        assert out.stdout.strip().splitlines()[-1] == want
