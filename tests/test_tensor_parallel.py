"""Head-sharded tensor parallelism: the sharding algebra on CPU, a 2-rank gloo all-reduce of the partial
projections, and (needs 2 GPUs) a 2-rank NCCL run of the engine against the single-GPU engine."""
from __future__ import annotations

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

import cases
from oracle import model_oracle as mo
from spikeinfer_b200.tensor_parallel import shard_config, shard_weights

SHAPE = dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=8,
             num_key_value_heads=4, head_dim=32)


def test_shard_shapes_and_coverage():
    shape = mo.ModelShape(**SHAPE)
    w = mo.init_weights(shape, seed=3)
    mo.randomize_lif(w, seed=4)
    local = shard_config(shape, 4)
    assert (local.num_attention_heads, local.num_key_value_heads, local.intermediate_size) == (2, 1, 64)
    shards = [shard_weights(w, shape, r, 4) for r in range(4)]
    p = "model.layers.1."
    assert shards[0][p + "self_attn.q_proj.weight"].shape == (2 * 32, 128)
    assert shards[0][p + "self_attn.o_proj.weight"].shape == (128, 2 * 32)
    assert torch.equal(torch.cat([s[p + "self_attn.k_proj.bias"] for s in shards]), w[p + "self_attn.k_proj.bias"])
    assert torch.equal(torch.cat([s[p + "mlp.lif_gate.lif.threshold"] for s in shards]), w[p + "mlp.lif_gate.lif.threshold"])
    assert torch.equal(shards[2][p + "self_attn.lif_q.lif.beta"], w[p + "self_attn.lif_q.lif.beta"])
    with pytest.raises(ValueError):
        shard_config(shape, 3)


def test_row_sharded_projections_sum_to_the_full_projection():
    shape = mo.ModelShape(**SHAPE)
    w = mo.init_weights(shape, seed=5)
    g = cases.gen(6)
    ctx = torch.randn(4, 7, 8 * 32, generator=g)
    act = torch.randn(4, 7, 256, generator=g)
    p = "model.layers.0."
    full_o = F.linear(ctx, w[p + "self_attn.o_proj.weight"])
    full_d = F.linear(act, w[p + "mlp.down_proj.weight"])
    part_o = part_d = 0
    for r in range(4):
        s = shard_weights(w, shape, r, 4)
        part_o = part_o + F.linear(ctx[..., r * 64:(r + 1) * 64], s[p + "self_attn.o_proj.weight"])
        part_d = part_d + F.linear(act[..., r * 64:(r + 1) * 64], s[p + "mlp.down_proj.weight"])
    torch.testing.assert_close(part_o, full_o, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(part_d, full_d, rtol=1e-5, atol=1e-6)


def _gloo_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    shape = mo.ModelShape(**SHAPE)
    w = mo.init_weights(shape, seed=5)
    s = shard_weights(w, shape, rank, world)
    ctx = torch.randn(4, 7, 8 * 32, generator=cases.gen(6))
    width = 8 * 32 // world
    part = F.linear(ctx[..., rank * width:(rank + 1) * width], s["model.layers.0.self_attn.o_proj.weight"])
    dist.all_reduce(part)
    full = F.linear(ctx, w["model.layers.0.self_attn.o_proj.weight"])
    q.put((rank, float((part - full).abs().max())))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_all_reduce_partial_projection():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 1000
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(err < 1e-5 for _, err in res)


def _nccl_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    # one NCCL communicator per process (the tensor-parallel group); the job-wide group is gloo
    dist.init_process_group("gloo", rank=rank, world_size=world)
    tp_group = dist.new_group(list(range(world)), backend="nccl")
    from spikeinfer_b200.engine.decode_engine import SpikeDecodeEngine
    from spikeinfer_b200.modeling import SpikingQwenConfig, SpikingQwenModel

    shape = mo.ModelShape(**SHAPE)
    w = mo.init_weights(shape, seed=7)
    mo.randomize_lif(w, seed=8)
    cfg = SpikingQwenConfig(**SHAPE)
    prompts = torch.randint(0, 512, (3, 20), generator=cases.gen(9)).tolist()

    def run(model):
        eng = SpikeDecodeEngine(model, num_blocks=32, block_size=16, max_num_seqs=4, max_model_len=64)
        rows = eng.add_requests(prompts)
        toks = [[int(eng.state.next_tokens[r])] for r in rows]
        for _ in range(6):
            eng.decode_step()
            for r in rows:
                toks[r].append(int(eng.state.next_tokens[r]))
        eng.state.check_status()
        return toks

    tp = run(SpikingQwenModel(shard_config(cfg, world), shard_weights(w, shape, rank, world), device=dev,
                              tp_group=tp_group))
    single = run(SpikingQwenModel(cfg, w, device=dev)) if rank == 0 else None
    q.put((rank, tp, single))
    torch.cuda.synchronize(dev)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.gpu
def test_two_gpu_tensor_parallel_engine_matches_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + os.getpid() % 1000
    procs = [ctx.Process(target=_nccl_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = {r: (tp, single) for r, tp, single in (q.get(timeout=300) for _ in procs)}
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert res[0][0] == res[1][0], "ranks of a group must sample identical tokens"
    same = sum(a == b for ta, tb in zip(res[0][0], res[0][1]) for a, b in zip(ta, tb))
    total = sum(len(t) for t in res[0][1])
    # the all-reduce changes the summation order, so a spike on a threshold may flip: token agreement, not bits
    assert same >= total - 1, f"{same}/{total} tokens agree with the single-GPU engine"


def _group_worker(rank, world, tp, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mine = None
    for g in range(world // tp):  # every rank creates every group, in the same order
        pg = dist.new_group(list(range(g * tp, (g + 1) * tp)), backend="gloo")
        if rank // tp == g:
            mine = pg
    # the row-sharded projection of test_row_sharded_projections_sum_to_the_full_projection, one shard per group rank;
    # each replica (group) works on its own input
    shape = mo.ModelShape(**SHAPE)
    w = mo.init_weights(shape, seed=7)
    replica, r = rank // tp, rank % tp
    x = torch.randn(5, shape.num_attention_heads * shape.head_dim, generator=cases.gen(40 + replica))
    full = torch.nn.functional.linear(x, w["model.layers.0.self_attn.o_proj.weight"])
    local = shard_weights(w, shape, r, tp)["model.layers.0.self_attn.o_proj.weight"]
    cols = x.shape[1] // tp
    part = torch.nn.functional.linear(x[:, r * cols:(r + 1) * cols], local)
    dist.all_reduce(part, group=mine)
    q.put((rank, dist.get_world_size(group=mine), float((part - full).abs().max())))
    dist.barrier()
    dist.destroy_process_group()


def test_two_groups_of_two_reduce_independently():
    """Four gloo ranks as two tensor-parallel groups of two (the 8-GPU form of the long-context configuration, scaled
    down): each group's all-reduce sums its own replica's partial projections and nothing else."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 1000
    procs = [ctx.Process(target=_group_worker, args=(r, 4, 2, port, q)) for r in range(4)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [r for r, _, _ in res] == [0, 1, 2, 3]
    for _, size, err in res:
        assert size == 2 and err < 1e-5
