"""Generate tests/golden/*.pt by running the reference's own CPU code on the seeded cases.

Run once in a container that has the reference checkout:
    python tests/golden/make_golden.py /path/to/reference

The reference package's ``__init__`` pulls in snntorch (absent here), so the kernel modules are
imported through empty parent-package objects that only carry ``__path__``; the modules used
(``kernels/*``, ``engine/block_manager.py``) depend on torch alone.  The fixtures are the
reference's OUTPUTS (plus a digest of the seeded inputs); no reference source is copied.
"""
from __future__ import annotations

import dataclasses
import importlib
import inspect
import json
import sys
import types
from pathlib import Path
from types import SimpleNamespace

import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import cases  # noqa: E402


def import_reference(ref_root: str):
    for name in ("spikeinfer", "spikeinfer.engine"):
        mod = types.ModuleType(name)
        mod.__path__ = [str(Path(ref_root) / name.replace(".", "/"))]
        sys.modules[name] = mod
    # sequence.py imports ..sampling_params, which is torch-free
    kernels = importlib.import_module("spikeinfer.kernels")
    cpu = importlib.import_module("spikeinfer.kernels.spike_attention_cpu")
    bm = importlib.import_module("spikeinfer.engine.block_manager")
    return kernels, cpu, bm


def describe_callable(fn) -> list[dict]:
    """Parameters of ``fn`` as plain data: name, kind, whether it has a default and the default's repr."""
    out = []
    for prm in inspect.signature(fn).parameters.values():
        has_default = prm.default is not inspect.Parameter.empty
        out.append(dict(name=prm.name, kind=prm.kind.name, has_default=has_default,
                        default=repr(prm.default) if has_default else None))
    return out


def record_interface(kernels, ref_root: str) -> None:
    """The operator surface a drop-in has to keep: every export of the reference's ``kernels`` package with its
    signature, ``paged_attention`` and the fields of ``AttentionMetadata``.  Written as JSON next to the fixtures."""
    surface = {}
    for name in kernels.__all__:
        obj = getattr(kernels, name)
        surface[name] = dict(params=describe_callable(obj)) if callable(obj) else dict(value=obj)
    attention = importlib.import_module("spikeinfer.attention")
    surface["paged_attention"] = dict(params=describe_callable(attention.paged_attention))
    fields = []
    for f in dataclasses.fields(attention.AttentionMetadata):
        has_default = f.default is not dataclasses.MISSING or f.default_factory is not dataclasses.MISSING
        fields.append(dict(name=f.name, has_default=has_default, public=not f.name.startswith("_")))
    surface["AttentionMetadata"] = dict(fields=fields)
    (HERE / "interface.json").write_text(json.dumps(surface, indent=1, sort_keys=True) + "\n")


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py /path/to/reference")
    ref_root = sys.argv[1]
    kernels, cpu, bm = import_reference(ref_root)
    torch.set_num_threads(4)
    record_interface(kernels, ref_root)

    # ---- packing -----------------------------------------------------------
    pack = {}
    for c in cases.PACK_CHANNELS:
        x = cases.pack_case(c)
        words = kernels.pack_spikes(x)
        assert torch.equal(kernels.unpack_spikes(words, c, torch.float32), x)
        pack[c] = dict(digest=cases.digest(x), words=words)
    pack["all_ones_32"] = kernels.pack_spikes(torch.ones(1, 32))
    pack["tail_33"] = kernels.pack_spikes(torch.ones(1, 33))
    pack["graded"] = kernels.pack_spikes(torch.tensor([[0.0, 0.5, 0.0, 2.0]]))
    pack["bytes_per_token_0p5b"] = kernels.packed_bytes_per_token(24, 4, 2, 64)
    torch.save(pack, HERE / "packing.pt")

    # ---- LIF (reference restatement lif_multistep_ref; CPU dispatch of lif_multistep) ----
    lif = {}
    for name, kw in cases.LIF_CASES.items():
        c = cases.lif_case(**kw)
        spikes, mem = kernels.lif_multistep_ref(c["x"], c["beta"], c["threshold"], mem0=c["mem0"],
                                                out_dtype=torch.uint8)
        spikes2, mem2 = kernels.lif_multistep(c["x"], c["beta"], c["threshold"], mem0=c["mem0"],
                                              out_dtype=torch.uint8, return_membrane=True)
        assert torch.equal(spikes, spikes2) and torch.equal(mem, mem2)
        lif[name] = dict(digest=cases.digest(c["x"].float(), c["beta"], c["threshold"]),
                         packed=kernels.pack_spikes(spikes), membrane=mem)
    c = cases.lif_boundary_case()
    spikes, mem = kernels.lif_multistep_ref(c["x"], c["beta"], c["threshold"], out_dtype=torch.uint8)
    lif["boundary"] = dict(digest=cases.digest(c["x"], c["beta"], c["threshold"]),
                           packed=kernels.pack_spikes(spikes), membrane=mem)
    torch.save(lif, HERE / "lif.pt")

    # ---- attention: both reference CPU forms, fp32 --------------------------
    attn = {}
    for name, kw in cases.ATTENTION_CASES.items():
        case = cases.attention_case(**kw)
        ref = kernels.paged_spike_attn_decode_ref(**case, dtype=torch.float32)
        fast = cpu.paged_spike_attn_decode_cpu(**case, dtype=torch.float32)
        torch.testing.assert_close(fast, ref, rtol=1e-5, atol=1e-6)
        attn[name] = dict(
            digest=cases.digest(case["q_packed"], case["k_cache"], case["v_cache"], case["block_tables"]),
            out_ref=ref,
        )
    # gather_kv_unpacked known answer on one case
    case = cases.attention_case(**cases.ATTENTION_CASES["ragged"])
    attn["gather_ragged_3"] = kernels.gather_kv_unpacked(
        case["k_cache"], case["block_tables"][3], 97, 64, 16, torch.float32).to(torch.uint8)
    attn["slot_matrix"] = cpu._slot_matrix(torch.tensor([[3, 1, 7], [5, 2, 0]], dtype=torch.int32), 10, 4)
    torch.save(attn, HERE / "attention.pt")

    # ---- block allocator trace ----------------------------------------------
    mgr = bm.BlockManager(num_blocks=12, block_size=4)
    seqs = [SimpleNamespace(num_computed_tokens=0, block_table=[]) for _ in range(3)]
    trace = []
    ok = [mgr.allocate(s, n) for s, n in zip(seqs, (5, 9, 2))]
    for s, n in zip(seqs, (5, 9, 2)):
        s.num_computed_tokens = n
    trace.append(dict(ok=ok, tables=[list(s.block_table) for s in seqs], free=list(mgr._free)))
    for step in range(6):  # six decode steps, every sequence grows by one token
        ok = [mgr.allocate(s, 1) for s in seqs]
        slots = [mgr.slot_mapping(s, s.num_computed_tokens, 1)[0] for s in seqs]
        for s in seqs:
            s.num_computed_tokens += 1
        trace.append(dict(ok=ok, tables=[list(s.block_table) for s in seqs], slots=slots, free=list(mgr._free)))
    mgr.free(seqs[1])
    trace.append(dict(tables=[list(s.block_table) for s in seqs], free=list(mgr._free)))
    ok = mgr.allocate(seqs[1], 6)
    trace.append(dict(ok=ok, tables=[list(s.block_table) for s in seqs], free=list(mgr._free)))
    seq = SimpleNamespace(num_computed_tokens=0, block_table=[5, 2, 7])
    known = [bm.BlockManager(8, 4).slot_mapping(seq, a, b) for a, b in ((0, 4), (4, 4), (8, 2), (3, 3))]
    torch.save(dict(trace=trace, slot_known=known), HERE / "block_manager.pt")

    for f in sorted(HERE.glob("*.pt")):
        print(f.name, f.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
