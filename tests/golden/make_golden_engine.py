"""Generate tests/golden/engine_tiny.pt: what the reference's own paged model path produces for the tiny
configuration (4 layers, hidden 256, 4/2 heads, head_dim 64, MLP 1024, vocab 32000, T=4, page 16,
4 prompts x 32 random ids, 16 greedy tokens) on CPU in fp32.

Run once where the reference checkout exists:  python tests/golden/make_golden_engine.py /path/to/reference

The reference imports snntorch only to hold the LIF parameters (its neuron is never stepped on the
engine path: spikeinfer/modeling_fast.py:32-34), so a stand-in module that registers ``beta`` /
``threshold`` and refuses to run is put on sys.path for this script.  The model's weights come from the
oracle's seeded ``init_weights`` and are loaded through ``load_state_dict``; the fixture stores only the
reference's OUTPUTS (tokens, logits samples, digests of the packed caches).
"""
from __future__ import annotations

import sys
import tempfile
from pathlib import Path
from types import SimpleNamespace

import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import cases  # noqa: E402
from oracle import model_oracle as mo  # noqa: E402

STUB = '''
import torch, torch.nn as nn
from . import surrogate
class Leaky(nn.Module):
    def __init__(self, beta, threshold=1.0, spike_grad=None, learn_beta=False, learn_threshold=False,
                 reset_mechanism="subtract", **kw):
        super().__init__()
        if isinstance(beta, torch.Tensor) and beta.device.type == "meta":
            raise RuntimeError("parameter holder cannot be built on meta")
        self.beta = nn.Parameter(torch.as_tensor(beta).clone(), requires_grad=learn_beta)
        self.threshold = nn.Parameter(torch.as_tensor(threshold).clone(), requires_grad=learn_threshold)
    def forward(self, *a, **k):
        raise NotImplementedError("parameter holder only")
'''

TINY = dict(vocab_size=32000, hidden_size=256, intermediate_size=1024, num_hidden_layers=4,
            num_attention_heads=4, num_key_value_heads=2, head_dim=64, T=4, rms_norm_eps=1e-6,
            rope_theta=1e6, tie_word_embeddings=True)
BLOCK_SIZE, NUM_BLOCKS, MAX_LEN, N_NEW = 16, 64, 256, 16


def prompts():
    g = cases.gen(1)
    return torch.randint(0, TINY["vocab_size"], (4, 32), generator=g).tolist()


def run_reference(ref_root: str, randomize: bool):
    from spikeinfer.attention import AttentionMetadata
    from spikeinfer.engine.block_manager import BlockManager
    from spikeinfer.engine.spike_cache import PagedSpikeCache
    from spikeinfer.modeling_fast import FastSpikingQwenForCausalLM
    from spikeinfer.reference.modeling_spiking_qwen import SpikingQwenConfig

    shape = mo.ModelShape(**TINY)
    w = mo.init_weights(shape, seed=0)
    if randomize:
        mo.randomize_lif(w, seed=1)
    cfg = SpikingQwenConfig(T=4, beta_init=0.9, threshold_init=1.0, vocab_size=shape.vocab_size,
                            hidden_size=shape.hidden_size, intermediate_size=shape.intermediate_size,
                            num_hidden_layers=shape.num_hidden_layers, num_attention_heads=shape.num_attention_heads,
                            num_key_value_heads=shape.num_key_value_heads, rope_theta=shape.rope_theta,
                            rms_norm_eps=shape.rms_norm_eps, tie_word_embeddings=True, max_position_embeddings=4096)
    model = FastSpikingQwenForCausalLM(cfg).eval()
    sd = dict(w)
    sd["lm_head.weight"] = w["model.embed_tokens.weight"]
    missing = model.load_state_dict(sd, strict=False)
    assert not missing.unexpected_keys, missing
    assert all("inv_freq" in k for k in missing.missing_keys), missing

    cache = PagedSpikeCache(shape.num_hidden_layers, shape.T, shape.num_key_value_heads, shape.head_dim,
                            NUM_BLOCKS, BLOCK_SIZE, device="cpu")
    mgr = BlockManager(cache.num_allocatable_blocks, BLOCK_SIZE)
    max_blocks = MAX_LEN // BLOCK_SIZE
    seqs, tokens = [], []
    ids, pos, slots, starts, lens, tabs, sample = [], [], [], [], [], [], []
    for p in prompts():
        s = SimpleNamespace(num_computed_tokens=0, block_table=[])
        assert mgr.allocate(s, len(p))
        starts.append(len(ids))
        ids += p
        pos += range(len(p))
        slots += mgr.slot_mapping(s, 0, len(p))
        lens.append(len(p))
        tabs.append(torch.tensor(s.block_table, dtype=torch.int32))
        sample.append(len(ids) - 1)
        s.num_computed_tokens = len(p)
        seqs.append(s)
        tokens.append(list(p))
    meta = AttentionMetadata(slot_mapping=torch.tensor(slots, dtype=torch.int64), block_size=BLOCK_SIZE,
                             prefill_query_starts=starts, prefill_query_lens=lens,
                             prefill_context_lens=[0] * len(lens), prefill_block_tables=tabs)
    logits_log = []
    with torch.no_grad():
        hidden = model.forward_paged(torch.tensor(ids), torch.tensor(pos), cache.layers, meta, T=4)
        logits = model.compute_logits(hidden, torch.tensor(sample)).float()
        logits_log.append(logits)
        for t, tok in zip(tokens, logits.argmax(-1).tolist()):
            t.append(tok)
        for _ in range(N_NEW - 1):
            for s in seqs:
                assert mgr.allocate(s, 1)
            slots = [mgr.slot_mapping(s, s.num_computed_tokens, 1)[0] for s in seqs]
            padded = [s.block_table + [cache.pad_block] * (max_blocks - len(s.block_table)) for s in seqs]
            meta = AttentionMetadata(
                slot_mapping=torch.tensor(slots, dtype=torch.int64), block_size=BLOCK_SIZE,
                num_decode_tokens=len(seqs), block_tables=torch.tensor(padded, dtype=torch.int32),
                seq_lens=torch.tensor([s.num_computed_tokens + 1 for s in seqs], dtype=torch.int32))
            hidden = model.forward_paged(torch.tensor([t[-1] for t in tokens]),
                                         torch.tensor([s.num_computed_tokens for s in seqs]), cache.layers, meta, T=4)
            logits = model.compute_logits(hidden).float()
            logits_log.append(logits)
            for s, t, tok in zip(seqs, tokens, logits.argmax(-1).tolist()):
                s.num_computed_tokens += 1
                t.append(tok)
    rates = [float((k != 0).float().mean()) for k in cache.k]
    return dict(
        tokens=[t[32:] for t in tokens],
        logits_first=logits_log[0][:, :64].clone(), logits_last=logits_log[-1][:, :64].clone(),
        logits_absmax=[float(l.abs().max()) for l in logits_log],
        top2_gap=[float((l.topk(2).values[:, 0] - l.topk(2).values[:, 1]).min()) for l in logits_log],
        k_digest=[cases.digest(k) for k in cache.k], v_digest=[cases.digest(v) for v in cache.v],
        k_popcount=[int(mo.orc.unpack_spikes(k, 64).sum()) for k in cache.k],
        tables=[list(s.block_table) for s in seqs], nonzero_word_rate=rates,
    )


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden_engine.py /path/to/reference")
    ref_root = sys.argv[1]
    with tempfile.TemporaryDirectory() as tmp:
        pkg = Path(tmp) / "snntorch"
        pkg.mkdir()
        (pkg / "__init__.py").write_text(STUB)
        (pkg / "surrogate.py").write_text("def fast_sigmoid(slope=25):\n    return None\n")
        sys.path.insert(0, tmp)
        sys.path.insert(0, ref_root)
        torch.set_num_threads(4)
        out = dict(config=TINY, block_size=BLOCK_SIZE, num_blocks=NUM_BLOCKS, max_len=MAX_LEN,
                   constant_lif=run_reference(ref_root, randomize=False),
                   random_lif=run_reference(ref_root, randomize=True))
    torch.save(out, HERE / "engine_tiny.pt")
    for k in ("constant_lif", "random_lif"):
        print(k, out[k]["tokens"][0][:8], out[k]["k_popcount"], [f"{g:.2e}" for g in out[k]["top2_gap"][:4]])
    print((HERE / "engine_tiny.pt").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
