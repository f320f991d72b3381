"""The CPU model oracle against what the reference's own paged model path produced (engine_tiny.pt):
greedy tokens, logits and the bit-packed K/V pools of every layer for the tiny configuration,
with constant and with randomised LIF parameters."""
from __future__ import annotations

import pytest
import torch

import cases
from oracle import model_oracle as mo


def tiny_prompts(vocab):
    return torch.randint(0, vocab, (4, 32), generator=cases.gen(1)).tolist()


@pytest.mark.parametrize("variant", ["constant_lif", "random_lif"])
def test_tiny_engine_matches_reference(variant, golden):
    torch.set_num_threads(4)  # the fixture was made with 4 threads; thread count changes GEMM blocking
    g = golden("engine_tiny")
    ref = g[variant]
    shape = mo.ModelShape(**g["config"])
    w = mo.init_weights(shape, seed=0)
    if variant == "random_lif":
        mo.randomize_lif(w, seed=1)
    run = mo.PagedRun(w, shape, g["num_blocks"], g["block_size"], g["max_len"])
    logits = [run.prefill(tiny_prompts(shape.vocab_size))]
    for _ in range(15):
        logits.append(run.decode())
    assert run.tables == ref["tables"]
    torch.testing.assert_close(logits[0][:, :64], ref["logits_first"], rtol=1e-4, atol=1e-5)
    assert [t[32:] for t in run.tokens] == ref["tokens"]
    torch.testing.assert_close(logits[-1][:, :64], ref["logits_last"], rtol=1e-4, atol=1e-5)
    # packed pools bit-identical to the reference's, layer by layer
    assert [cases.digest(k) for k in run.k] == ref["k_digest"]
    assert [cases.digest(v) for v in run.v] == ref["v_digest"]
