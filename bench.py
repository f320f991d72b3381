"""Benchmark of the spiking decode hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline workload ("decode_0p5b_64req"): the spiking Qwen2.5-0.5B-shape model (24 layers, hidden 896,
14/2 heads, head_dim 64, MLP 4864, vocab 151936, tied embeddings, T=4, bf16 random-init weights,
thresholds calibrated to ~15 % q/k/v and ~5 % gate firing), 64 concurrent requests per GPU with
128-token random prompts, greedy decode, page size 16.  One step = one decode step of all 64 requests
(64 tokens) as a single CUDA-graph replay: on-GPU metadata advance, 24 layers, lm_head, argmax.

  value   decode tok/s with tokens looping on the device (inputs resident in HBM), K timed steps (the region of median
          duration among the repeats).
  spread  the same K steps repeated from the same batch state: median / min / max of every timed quantity.
  e2e     the same steps through ``SpikeDecodeEngine.step_host``: every step copies the input tokens
          from pinned host memory and reads the sampled tokens back.
  roofline  paged popcount attention at the kernel-level configuration the metric names (64 ragged sequences in
          [128, 4096], 14/2 heads, D 64, T 4, Bernoulli(0.2) bits, 16-token pages, bf16 out), timed with CUDA
          events over 24 distinct pools back to back (430 MB of K/V, larger than L2); achieved = algorithmic
          bytes / time per call against the measured HBM copy peak.  ``other_shapes``: the same for larger batches.
  roofline_lif  fused LIF + bit-pack (+ paged K/V write) at its kernel-level configuration, both reset rules.
  closed_loop  the reference's own serving protocol (spikeinfer/bench.py:29-116: N requests, C in flight, 128 in /
          64 out): prefill, admission, release and the host visits inside the clock; output tok/s, TTFT, ITL.
  open_loop  the same requests arriving as a Poisson process at 8 req/s (arrival-bound by construction).
  strong_scaling  64 requests in total over the N GPUs of the run (the headline is 64 per GPU).
  cpu_baseline  the CPU oracle port of the reference's paged model path, timed on this host's cores on
          a bounded sample of the same workload.

``--impl reference`` times that CPU port alone (the reference is pure Python/PyTorch; its CPU mode is
what a B200-less host runs) and prints the same line with ``"impl": "reference"``.

With N > 1 (launched under torchrun, one rank per GPU) every rank runs an independent replica with its
own 64 requests and page pool (requests shard, no collective on the data path); times are the max
over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
for _p in (str(ROOT), str(ROOT / "tests")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

METRIC = "decode_tok_per_s_0.5B_spiking_T4_64req"
UNIT = "tok/s"
N_REQ = 64
PROMPT_LEN = 128
BLOCK_SIZE = 16
FALLBACK_HBM_GBS = 6650.0


def stats(values: list[float], digits: int = 4) -> dict:
    return {"median": round(statistics.median(values), digits), "min": round(min(values), digits),
            "max": round(max(values), digits), "repeats": len(values)}


def measured_traffic(key: str):
    """DRAM bytes per launch of a kernel at a named workload, from the ncu capture summarised in
    profiles/dram_traffic.txt (lines ``key bytes``).  None when the kernel has no capture under that key, so a
    kernel that changed its name or shape without a new capture reports no traffic instead of a stale figure."""
    try:
        for line in (ROOT / "profiles" / "dram_traffic.txt").read_text().splitlines():
            parts = line.split()
            if len(parts) >= 2 and not line.startswith("#") and parts[0] == key:
                return float(parts[1])
    except OSError:
        pass
    return None


def hbm_peak():
    """(GB/s, "measured" | "fallback") from MEASURED_PEAKS.json."""
    path = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index = index
        self.samples: list[list[str]] = []
        self.proc: subprocess.Popen | None = None
        self.thread: threading.Thread | None = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return self
        def pump():
            for line in self.proc.stdout:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) == 6:
                    self.samples.append(parts)
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            # nvidia-smi needs up to a second or two before its first line on a host with eight GPUs: give it the
            # chance to deliver a sample (the GPU is still clocked up from the region that just ended)
            deadline = time.time() + 3.0
            time.sleep(0.15)
            while not self.samples and time.time() < deadline and self.proc.poll() is None:
                time.sleep(0.05)
            self.proc.terminate()  # the exact child started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        mhz, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for s in self.samples:
            try:
                mhz.append(float(s[0]))
                mx.append(float(s[1]))
            except ValueError:
                continue
            for name, flag in zip(names, s[2:]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not mhz:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(mhz), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(mhz)}


def dist_info():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# --------------------------------------------------------------------------- workload: model + engine
def random_weights_device(cfg, device, dtype, seed: int) -> dict:
    """Seeded normal(0, 0.02) weights generated on the device, keyed like the reference's state_dict."""
    g = torch.Generator(device=device).manual_seed(seed)
    mat = lambda *size: (torch.randn(size, generator=g, device=device, dtype=torch.float32) * 0.02).to(dtype)
    hq, hkv, d, hid, inter = (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.hidden_size,
                              cfg.intermediate_size)
    w = {"model.embed_tokens.weight": mat(cfg.vocab_size, hid), "model.norm.weight": torch.ones(hid, device=device, dtype=dtype)}
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        for name, rows in (("q", hq * d), ("k", hkv * d), ("v", hkv * d)):
            w[p + f"self_attn.{name}_proj.weight"] = mat(rows, hid)
            w[p + f"self_attn.{name}_proj.bias"] = torch.zeros(rows, device=device, dtype=dtype)
            w[p + f"self_attn.lif_{name}.lif.beta"] = torch.full((d,), 0.9, device=device)
            w[p + f"self_attn.lif_{name}.lif.threshold"] = torch.ones(d, device=device)
        w[p + "self_attn.o_proj.weight"] = mat(hid, hq * d)
        w[p + "mlp.gate_proj.weight"] = mat(inter, hid)
        w[p + "mlp.up_proj.weight"] = mat(inter, hid)
        w[p + "mlp.down_proj.weight"] = mat(hid, inter)
        w[p + "mlp.lif_gate.lif.beta"] = torch.full((inter,), 0.9, device=device)
        w[p + "mlp.lif_gate.lif.threshold"] = torch.ones(inter, device=device)
        w[p + "input_layernorm.weight"] = torch.ones(hid, device=device, dtype=dtype)
        w[p + "post_attention_layernorm.weight"] = torch.ones(hid, device=device, dtype=dtype)
    return w


def model_len(total_steps: int) -> int:
    """max_model_len of the workload: prompt + every decode step the run will take, rounded up to 256."""
    return -(-(PROMPT_LEN + total_steps + 2 * BLOCK_SIZE) // 256) * 256


def total_decode_steps(K: int, W: int) -> int:
    return 2 * (K + W) + 8  # device-timed and host-in-the-loop passes, plus slack


def build_model(device, seed: int):
    """0.5B-shape model with thresholds calibrated on 8 seeded prompts."""
    from spikeinfer_b200.calibrate import calibrate_thresholds
    from spikeinfer_b200.modeling import SpikingQwenConfig, SpikingQwenModel

    cfg = SpikingQwenConfig.qwen2_5_0p5b()
    weights = random_weights_device(cfg, device, torch.bfloat16, seed)
    model = SpikingQwenModel(cfg, weights, device=device)
    del weights
    g = torch.Generator(device="cpu").manual_seed(seed + 7)
    calib = torch.randint(0, cfg.vocab_size, (8, PROMPT_LEN), generator=g)
    rates = calibrate_thresholds(model, calib.to(device))
    model.validate_thresholds()
    return cfg, model, rates


def build_engine(model, prompts: torch.Tensor, max_len: int, device):
    """Engine with one decode row per prompt: prompts prefilled in groups of 16, decode graph captured.
    Returns (engine, launches of this library per decode step)."""
    from spikeinfer_b200 import _lib
    from spikeinfer_b200.engine.decode_engine import SpikeDecodeEngine

    n = prompts.shape[0]
    blocks_per_seq = -(-max_len // BLOCK_SIZE)
    engine = SpikeDecodeEngine(model, num_blocks=n * blocks_per_seq + 1, block_size=BLOCK_SIZE,
                               max_num_seqs=n, max_model_len=max_len)
    for s in range(0, n, 16):
        engine.add_requests(prompts[s:s + 16].tolist())
    lib = _lib.load()
    before = lib.spk_launch_count()
    engine.capture()
    launches_per_step = (lib.spk_launch_count() - before) // 5  # three warm-up passes and the two captured forms
    torch.cuda.synchronize(device)
    engine.state.check_status()
    return engine, launches_per_step


def job_prompts(cfg, seed: int, n_total: int) -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(seed + 1)
    return torch.randint(0, cfg.vocab_size, (n_total, PROMPT_LEN), generator=g)


# --------------------------------------------------------------------------- serving protocols (secondary keys)
OUT_LEN = 64


def percentile(values: list[float], q: float) -> float:
    v = sorted(values)
    return v[min(len(v) - 1, int(q * len(v)))]


def closed_loop(model, cfg, device, concurrency: int, n_requests: int, k: int = 9, packed_prefill: bool = False,
                seed: int = 77) -> dict:
    """The reference's closed-loop protocol (spikeinfer/bench.py:29-116): `concurrency` requests in flight, each
    replaced by the next one as soon as it finishes, 128 prompt tokens in, 64 greedy tokens out.  Everything is
    inside the clock: prefill (groups of up to 16 prompts), admission, the host visit that reads the tokens (one
    per k decode steps; the reference visits every step), release.  The engine holds `concurrency` rows and one
    decode graph per bucket of rows up to that (as the reference does); a step replays the smallest bucket that
    covers the batch."""
    from spikeinfer_b200.engine.decode_engine import SpikeDecodeEngine

    max_len = -(-(PROMPT_LEN + OUT_LEN + BLOCK_SIZE) // BLOCK_SIZE) * BLOCK_SIZE
    engine = SpikeDecodeEngine(model, num_blocks=concurrency * (max_len // BLOCK_SIZE) + 1, block_size=BLOCK_SIZE,
                               max_num_seqs=concurrency, max_model_len=max_len, packed_prefill=packed_prefill)
    g = torch.Generator(device="cpu").manual_seed(seed)
    prompts = torch.randint(0, cfg.vocab_size, (n_requests + 2, PROMPT_LEN), generator=g).tolist()
    sync = lambda: torch.cuda.synchronize(device)
    # warm-up, as the reference does (two requests): prefill kernels, graph capture
    rows = engine.add_requests(prompts[-2:][:min(2, concurrency)])
    engine.capture_all()
    engine.decode_steps(2)
    for r in rows:
        engine.release(r)
    sync()

    pending = list(range(n_requests))
    inflight: dict[int, list] = {}  # row -> [request, tokens produced, submit time, first-token time]
    ttft, itl, visits = [], [], 0
    t0 = time.perf_counter()
    freed_at = t0
    while pending or inflight:
        while pending and engine.free_rows:
            group = [pending.pop(0) for _ in range(min(16, len(pending), len(engine.free_rows)))]
            rows = engine.add_requests([prompts[i] for i in group])
            sync()
            now = time.perf_counter()
            for i, r in zip(group, rows):
                inflight[r] = [i, 1, freed_at, now]
                ttft.append(now - freed_at)
        steps = min(k, min(OUT_LEN - v[1] for v in inflight.values()))
        engine.decode_steps(steps)  # one host visit
        visits += 1
        now = time.perf_counter()
        for r in list(inflight):
            inflight[r][1] += steps
            if inflight[r][1] >= OUT_LEN:
                itl.append((now - inflight[r][3]) / (OUT_LEN - 1))
                engine.release(r)
                del inflight[r]
                freed_at = now
    sync()
    wall = time.perf_counter() - t0
    engine.state.check_status()
    return {"concurrency": concurrency, "requests": n_requests, "output_tok_per_s": round(n_requests * OUT_LEN / wall, 1),
            "ttft_ms_p50": round(percentile(ttft, 0.5) * 1e3, 2), "ttft_ms_p99": round(percentile(ttft, 0.99) * 1e3, 2),
            "itl_ms_mean": round(statistics.mean(itl) * 1e3, 4), "wall_s": round(wall, 3),
            "decode_steps_per_host_visit": k, "host_visits": visits,
            "prefill": "batched popcount kernel over the packed pool" if packed_prefill
                       else "SDPA on unpacked spikes, sequences of one shape in one call (the reference's arithmetic)"}


def open_loop(model, cfg, device, rate: float = 8.0, n_requests: int = 64, seed: int = 78) -> dict:
    """64 requests arriving as a Poisson process at `rate` per second, 128 in / 64 out, up to 64 rows.  The offered
    load is rate x 64 = 512 output tok/s, far below what one GPU decodes, so the run is ARRIVAL-BOUND: its
    throughput says nothing about the GPU; TTFT and inter-token latency do.  One host visit per decode step."""
    from spikeinfer_b200.engine.decode_engine import SpikeDecodeEngine

    max_len = -(-(PROMPT_LEN + OUT_LEN + BLOCK_SIZE) // BLOCK_SIZE) * BLOCK_SIZE
    engine = SpikeDecodeEngine(model, num_blocks=N_REQ * (max_len // BLOCK_SIZE) + 1, block_size=BLOCK_SIZE,
                               max_num_seqs=N_REQ, max_model_len=max_len)
    g = torch.Generator(device="cpu").manual_seed(seed)
    prompts = torch.randint(0, cfg.vocab_size, (n_requests + 1, PROMPT_LEN), generator=g).tolist()
    arrivals = torch.cumsum(torch.empty(n_requests).exponential_(rate, generator=g), 0).tolist()
    sync = lambda: torch.cuda.synchronize(device)
    rows = engine.add_requests(prompts[-1:])
    engine.capture_all()  # one graph per bucket of rows (1, 2, 4, ... 64): a step replays the smallest that covers the batch
    engine.decode_steps(2)
    engine.release(rows[0])
    sync()

    inflight: dict[int, list] = {}
    ttft, itl, nxt, done, busy_steps = [], [], 0, 0, 0
    t0 = time.perf_counter()
    while done < n_requests:
        now = time.perf_counter() - t0
        group = []
        while nxt < n_requests and arrivals[nxt] <= now and len(group) < len(engine.free_rows):
            group.append(nxt)
            nxt += 1
        if group:
            rows = engine.add_requests([prompts[i] for i in group])
            sync()
            now = time.perf_counter() - t0
            for i, r in zip(group, rows):
                inflight[r] = [i, 1, arrivals[i], now]
                ttft.append(now - arrivals[i])
        if inflight:
            engine.decode_steps(1)
            busy_steps += 1
            now = time.perf_counter() - t0
            for r in list(inflight):
                inflight[r][1] += 1
                if inflight[r][1] >= OUT_LEN:
                    itl.append((now - inflight[r][3]) / (OUT_LEN - 1))
                    engine.release(r)
                    del inflight[r]
                    done += 1
        elif nxt < n_requests:
            time.sleep(max(0.0, arrivals[nxt] - (time.perf_counter() - t0)))
    wall = time.perf_counter() - t0
    engine.state.check_status()
    return {"arrival_rate_req_per_s": rate, "requests": n_requests, "offered_output_tok_per_s": rate * OUT_LEN,
            "output_tok_per_s": round(n_requests * OUT_LEN / wall, 1), "arrival_bound": True,
            "ttft_ms_p50": round(percentile(ttft, 0.5) * 1e3, 2), "ttft_ms_p99": round(percentile(ttft, 0.99) * 1e3, 2),
            "itl_ms_mean": round(statistics.mean(itl) * 1e3, 4), "wall_s": round(wall, 2), "decode_steps": busy_steps}


# --------------------------------------------------------------------------- attention roofline (kernel level)
ATTN_KERNEL = "attn_stream_kernel<W=2,NB=1,dense>"  # what bf16 output at head_dim 64 launches (+ its combine pass)


ATTN_OVERLAP = False  # --attn-overlap sets it
ATTN_PAGE_MAJOR = False  # --attn-page-major sets it


def time_attention(device, lens, max_blocks, n_pools, iters, repeats, hd=64, hq=14, hkv=2, overlap=None) -> dict:
    """One call = the main kernel plus its combine pass over one pool; `n_pools` distinct pools back to back inside
    one CUDA graph (their K/V together exceed L2), `iters` replays per timed region, `repeats` regions.  With
    ATTN_OVERLAP a call may be placed while the previous call's combine pass still runs (programmatic dependent
    launch, as the attention launch of a decode step is placed behind the LIF launch before it; lengths and block
    tables never change here).  Off by default: behind a combine pass it does not pay (22.3 against 21.7 us)."""
    import cases
    from spikeinfer_b200 import kernels

    overlap = ATTN_OVERLAP if overlap is None else overlap
    case = cases.attention_case(seq_lens=lens, density=0.2, seed=2, spare_blocks=0, max_blocks=max_blocks,
                                head_dim=hd, num_q_heads=hq, num_kv_heads=hkv)
    d = {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in case.items()}
    if ATTN_PAGE_MAJOR:
        # one buffer [block, T, H_kv, K|V, slot, W] (a page's 2 KB contiguous); K and V as strided 5-D views of it
        def page_major(k, v):
            T_, H_, slots_, W_ = k.shape
            nb = slots_ // BLOCK_SIZE
            buf = torch.empty((nb, T_, H_, 2, BLOCK_SIZE, W_), dtype=k.dtype, device=device)
            buf[:, :, :, 0] = k.view(T_, H_, nb, BLOCK_SIZE, W_).permute(2, 0, 1, 3, 4)
            buf[:, :, :, 1] = v.view(T_, H_, nb, BLOCK_SIZE, W_).permute(2, 0, 1, 3, 4)
            return buf[:, :, :, 0].permute(1, 2, 0, 3, 4), buf[:, :, :, 1].permute(1, 2, 0, 3, 4)
        pools = [page_major(d["k_cache"], d["v_cache"]) for _ in range(n_pools)]
    else:
        pools = [(d["k_cache"].clone(), d["v_cache"].clone()) for _ in range(n_pools)]
    out = torch.empty(4, len(lens), hq, hd, dtype=torch.bfloat16, device=device)

    def run_all():
        for k, v in pools:
            kernels.paged_spike_attn_decode(d["q_packed"], k, v, d["block_tables"], d["seq_lens"], hd, BLOCK_SIZE,
                                            hq, hkv, out=out, overlap_previous=overlap)

    run_all()
    torch.cuda.synchronize(device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run_all()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize(device)
    us = []
    for _ in range(repeats):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(iters):
            graph.replay()
        stop.record()
        torch.cuda.synchronize(device)
        us.append(start.elapsed_time(stop) * 1e3 / (iters * n_pools))
    W = hd // 32
    n = len(lens)
    # algorithmic bytes of one call: K+V once per KV head, q, bf16 out, block-table entries, lengths
    alg = sum(lens) * 4 * hkv * 2 * W * 4 + 4 * n * hq * W * 4 + 4 * n * hq * hd * 2 \
        + sum(-(-l // BLOCK_SIZE) for l in lens) * 4 + n * 4
    peak, _ = hbm_peak()
    med = statistics.median(us)
    return {"us_per_call": stats(us, 2), "algorithmic_bytes": alg, "achieved_GBs": round(alg / med / 1e3, 1),
            "frac": round(alg / med / 1e3 / peak, 4), "pools": n_pools, "sum_keys": sum(lens),
            "overlaps_previous_call": overlap, "pool_layout": "page_major" if ATTN_PAGE_MAJOR else "reference"}


def attention_roofline(device, n_pools: int = 24, iters: int = 10, repeats: int = 5, extra: bool = True,
                       uniform: tuple[int, int] | None = None) -> dict:
    """`uniform` = (rows, keys): that many rows of equal length instead of the ragged configuration."""
    import math

    import cases

    if uniform is not None:
        rows, keys = uniform
        res = time_attention(device, [keys] * rows, -(-keys // BLOCK_SIZE), n_pools, iters, repeats)
        return {"kernel": ATTN_KERNEL, "workload": f"{rows} rows x {keys} keys, 14/2 heads, D64, T4, bf16 out, {n_pools} pools", **res}
    g = cases.gen(2)
    lens = torch.randint(128, 4097, (N_REQ,), generator=g).tolist()
    main = time_attention(device, lens, 4096 // BLOCK_SIZE, n_pools, iters, repeats)
    peak, which = hbm_peak()
    roof = {"bound": "hbm", "achieved": main["achieved_GBs"], "peak": peak, "unit": "GB/s", "frac": main["frac"],
            "peak_source": f"of {which}",
            # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel at this workload (ncu)
            "traffic": measured_traffic(ATTN_KERNEL + "@64x[128,4096]"),
            "kernel": ATTN_KERNEL + " (mma.sync m16n8k16 over V bits in place; equal step ranges per warp) + combine pass",
            "workload": "64 seqs ragged [128,4096] (sum %d keys), 14/2 heads, D64, T4, p=0.2, page 16, bf16 out, "
                        "%d distinct pools back to back" % (main["sum_keys"], n_pools),
            "us_per_launch": main["us_per_call"]["median"], "us_per_launch_spread": main["us_per_call"],
            "algorithmic_bytes": main["algorithmic_bytes"],
            "launch_overlap": "a call's prologue (lengths, step prefix, block-table entries) may run under the previous "
                              "call's combine pass" if ATTN_OVERLAP else "none"}
    if extra and not ATTN_OVERLAP:
        # the same calls launched the way the decode step launches them: each may be placed while the launch before
        # it (here the previous call's combine pass) still runs; lengths and tables are fixed, as the hint requires
        ov = time_attention(device, lens, 4096 // BLOCK_SIZE, n_pools, iters, repeats, overlap=True)
        roof["with_launch_overlap"] = {"us_per_launch": ov["us_per_call"], "achieved": ov["achieved_GBs"], "frac": ov["frac"]}
    if extra:
        g5 = cases.gen(5)
        lo, hi = math.log(1024.0), math.log(32768.0)
        ctx = torch.exp(torch.rand(64, generator=g5) * (hi - lo) + lo).long().clamp(1024, 32768).tolist()
        roof["other_shapes"] = {
            "256x4096_d64_14/2": time_attention(device, [4096] * 256, 256, 6, 5, repeats),
            "64x[1k,32k]loguniform_d128_7/1 (one tensor-parallel shard of the 7B shape)":
                time_attention(device, ctx, 2048, 4, 5, repeats, hd=128, hq=7, hkv=1),
        }
    return roof


def lif_roofline(device, n_tok: int = 8192, iters: int = 10, repeats: int = 5) -> dict:
    """Fused LIF + bit-pack (+ K/V scatter) at the kernel-level configuration: gate currents bf16
    [T=4, n_tok, 4864] -> packed bits + fp32 membrane, and k/v currents [4, n_tok, 2x64x2] scattered through
    a random slot permutation of a 16-token-page pool; both reset rules."""
    from spikeinfer_b200 import _lib, kernels

    T, N, Hkv, D = 4, 4864, 2, 64
    g = torch.Generator(device=device).manual_seed(3)
    gate = torch.randn((T, n_tok, N), generator=g, device=device).to(torch.bfloat16)
    kv = torch.randn((T, n_tok, 2 * Hkv * D), generator=g, device=device).to(torch.bfloat16)
    th = torch.rand(N, generator=g, device=device) + 0.5
    beta = torch.full((N,), 0.9, device=device)
    slots = torch.randperm(n_tok, generator=g, device=device)
    k_pool = torch.zeros((T, Hkv, n_tok, 2), dtype=torch.int32, device=device)
    v_pool = torch.zeros_like(k_pool)
    S = kernels.LifSiteSpec
    site = lambda x, pool: S(x=x, beta=beta[:D], threshold=th[:D], packed=pool,
                             packed_strides=(pool.stride(0), pool.stride(2), pool.stride(1)),
                             slot_mapping=slots, num_rows=n_tok)
    kv_sites = [site(kv[..., : Hkv * D].unflatten(-1, (Hkv, D)), k_pool), site(kv[..., Hkv * D:].unflatten(-1, (Hkv, D)), v_pool)]

    def timed(fn):
        # `iters` launches back to back inside one CUDA graph, so that the host's call overhead (above the k/v
        # launch's 20 us) stays out of the time; one replay per timed region
        for _ in range(3):
            fn()
        torch.cuda.synchronize(device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(iters):
                fn()
        graph.replay()
        us = []
        for _ in range(repeats):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize(device)
            start.record()
            graph.replay()
            stop.record()
            torch.cuda.synchronize(device)
            us.append(start.elapsed_time(stop) * 1e3 / iters)
        del graph
        return us

    peak, which = hbm_peak()

    def entry(us, alg):
        med = statistics.median(us)
        return {"us": stats(us, 1), "algorithmic_bytes": alg, "achieved_GBs": round(alg / med / 1e3, 1),
                "frac": round(alg / med / 1e3 / peak, 4)}

    out = {}
    for mode, tag in ((_lib.RESET_SUBTRACT_DELAYED, "subtract_delayed"), (_lib.RESET_HARD_ZERO, "hard_zero")):
        res = {}
        us = timed(lambda: kernels.lif_pack(gate, beta, th, return_membrane=True, reset_mode=mode))
        res["gate_pack_membrane"] = entry(us, gate.numel() * 2 + gate.numel() // 8 + n_tok * N * 4)
        us = timed(lambda: kernels.lif_pack(gate, beta, th, reset_mode=mode))
        res["gate_pack"] = entry(us, gate.numel() * 2 + gate.numel() // 8)
        us = timed(lambda: kernels.lif_pack_scatter(kv_sites, reset_mode=mode))
        res["kv_pack_scatter"] = entry(us, kv.numel() * 2 + kv.numel() // 8 + n_tok * 8)
        out[tag] = res
    out["bound"] = "hbm"
    out["peak"] = peak
    out["peak_source"] = f"of {which}"
    out["traffic_gate_pack_membrane"] = measured_traffic("lif_pack_scatter_vec_kernel@gate4x8192x4864+membrane")
    out["workload"] = (f"T=4, {n_tok} tokens, gate 4864 channels bf16, k/v 2 heads x 64, page 16; the gate tensor alone "
                       "exceeds L2; subtract_delayed is the reference's reset rule, hard_zero this library's own (parity unpinned)")
    return out


def step_kernels(device, repeats: int = 5, chain: int = 40) -> dict:
    """This library's kernels at the shapes of one decode layer of the headline workload (64 rows, T = 4, 0.5B
    shape), each `chain` times back to back inside one CUDA graph on warm operands, next to an empty-ish torch
    kernel and the four library GEMMs of the layer: what a launch costs when it is launch-latency-sized."""
    import torch.nn.functional as F

    import cases
    from spikeinfer_b200 import kernels

    T, n, Hq, Hkv, D, hid, inter = 4, N_REQ, 14, 2, 64, 896, 4864
    bf = torch.bfloat16
    g = torch.Generator(device=device).manual_seed(11)
    rnd = lambda *shape: torch.randn(shape, generator=g, device=device).to(bf)

    def timed(fn) -> dict:
        fn()
        torch.cuda.synchronize(device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(chain):
                fn()
        for _ in range(3):
            graph.replay()
        us = []
        for _ in range(repeats):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize(device)
            start.record()
            graph.replay()
            stop.record()
            torch.cuda.synchronize(device)
            us.append(start.elapsed_time(stop) * 1e3 / chain)
        return stats(us, 2)

    out = {}
    z = torch.zeros(32, device=device)
    out["empty_torch_kernel"] = timed(lambda: z.add_(1.0))
    h, dl, wn = rnd(T * n, hid), rnd(T * n, hid), torch.ones(hid, device=device, dtype=bf)
    out["add_rms_norm_256x896"] = timed(lambda: kernels.add_rms_norm(h, dl, wn, 1e-6))
    qkv = rnd(T, n, (Hq + 2 * Hkv) * D)
    beta, th = torch.full((D,), 0.9, device=device), torch.ones(D, device=device)
    cos, sin = rnd(n, D), rnd(n, D)
    slots = torch.randperm(4096, generator=g, device=device)[:n]
    kc = torch.zeros(T, Hkv, 4096, 2, dtype=torch.int32, device=device)
    vc = torch.zeros_like(kc)
    qp = torch.empty(T, n, Hq, 2, dtype=torch.int32, device=device)
    xq = qkv[..., : Hq * D].unflatten(-1, (Hq, D))
    xk = qkv[..., Hq * D:(Hq + Hkv) * D].unflatten(-1, (Hkv, D))
    xv = qkv[..., (Hq + Hkv) * D:].unflatten(-1, (Hkv, D))
    S = kernels.LifSiteSpec
    pool = lambda c: dict(packed=c, packed_strides=(c.stride(0), c.stride(2), c.stride(1)), slot_mapping=slots, num_rows=4096)
    sites = [S(x=xq, beta=beta, threshold=th, packed=qp, packed_strides=(n * Hq * 2, Hq * 2, 2), rope_cos=cos, rope_sin=sin),
             S(x=xk, beta=beta, threshold=th, rope_cos=cos, rope_sin=sin, **pool(kc)),
             S(x=xv, beta=beta, threshold=th, **pool(vc))]
    out["lif_qkv_rope_pack_scatter"] = timed(lambda: kernels.lif_pack_scatter(sites))
    case = cases.attention_case(seq_lens=[130 + (i % 70) for i in range(n)], density=0.15, seed=2, max_blocks=16)
    d = {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in case.items()}
    ctx = torch.empty(T, n, Hq, D, dtype=bf, device=device)
    out["attention_64_rows_130_to_199_keys"] = timed(lambda: kernels.paged_spike_attn_decode(**d, out=ctx))
    gu = rnd(T, n, 2 * inter)
    gb, gth = torch.full((inter,), 0.9, device=device), torch.ones(inter, device=device)
    out["lif_gate_times_up"] = timed(lambda: kernels.lif_gate_mul(gu[..., :inter], gu[..., inter:], gb, gth))
    x = rnd(T * n, hid)
    for name, N_, K_, bias in (("gemm_qkv", (Hq + 2 * Hkv) * D, hid, True), ("gemm_o", hid, hid, False),
                               ("gemm_gate_up", 2 * inter, hid, False), ("gemm_down", hid, inter, False)):
        a = x if K_ == hid else rnd(T * n, K_)
        w = (rnd(N_, K_).float() * 0.05).to(bf)
        b = rnd(N_) if bias else None
        out[name + "_library"] = timed(lambda: F.linear(a, w, b))
    return {"unit": "us per launch, median/min/max", "chain": chain, "kernels": out}


def run_kernel_bench(args) -> None:
    """Kernel-level configurations only (also the small cases the ncu captures under profiles/ run)."""
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    if args.attn_form != "auto":
        from spikeinfer_b200 import _lib

        form = {"general": _lib.ATTN_FORM_GENERAL, "tcgen05": _lib.ATTN_FORM_TCGEN05}[args.attn_form]
        _lib.check(_lib.load().spk_attn_select_form(form), "spk_attn_select_form")
    if args.kernel_bench == "step":
        res = step_kernels(device, repeats=args.repeats)
    elif args.kernel_bench == "attn":
        res = attention_roofline(device, n_pools=args.pools, iters=args.steps, repeats=args.repeats, extra=False,
                                 uniform=(args.rows, args.keys) if args.rows and args.keys else None)
    else:
        res = lif_roofline(device, n_tok=args.tokens, iters=args.steps, repeats=args.repeats)
    print(json.dumps({"kernel_bench": args.kernel_bench, **res}), flush=True)


# --------------------------------------------------------------------------- CPU port of the reference path
class CpuDecodeSample:
    """The oracle's CPU restatement of the reference's paged model path at the 0.5B shape (fp32, as the
    reference's pure-CPU mode), 64 requests at context 128.  The pools are filled with Bernoulli(0.15)
    bits instead of running a CPU prefill (which alone would take minutes); every timed step is a full
    decode step of all 64 requests: metadata build, 24 layers, lm_head, argmax."""

    def __init__(self, seed: int = 0, max_len: int = 512) -> None:
        from oracle import model_oracle as mo
        from oracle import torch_oracle as orc

        self.mo, self.orc = mo, orc
        self.shape = mo.ModelShape(vocab_size=151936, hidden_size=896, intermediate_size=4864, num_hidden_layers=24,
                                   num_attention_heads=14, num_key_value_heads=2, head_dim=64)
        self.w = mo.init_weights(self.shape, seed=seed)
        blocks_per_seq = max_len // BLOCK_SIZE
        self.run = mo.PagedRun(self.w, self.shape, N_REQ * blocks_per_seq + 1, BLOCK_SIZE, max_len)
        g = torch.Generator(device="cpu").manual_seed(seed + 1)
        for _ in range(N_REQ):
            table: list[int] = []
            assert self.run.mgr.allocate(table, 0, PROMPT_LEN)
            self.run.tables.append(table)
            self.run.computed.append(PROMPT_LEN)
            self.run.tokens.append([int(torch.randint(0, self.shape.vocab_size, (1,), generator=g))])
        for pool in self.run.k + self.run.v:
            bits = (torch.rand((*pool.shape[:3], 64), generator=g) < 0.15).to(torch.float32)
            pool.copy_(orc.pack_spikes(bits))

    def step(self) -> None:
        self.run.decode()


def time_cpu_steps(sample: CpuDecodeSample, steps: int, warmup: int) -> float:
    for _ in range(warmup):
        sample.step()
    t0 = time.perf_counter()
    for _ in range(steps):
        sample.step()
    return (time.perf_counter() - t0) / steps


def cpu_baseline(steps: int = 3, warmup: int = 1) -> dict:
    sample = CpuDecodeSample()
    sec = time_cpu_steps(sample, steps, warmup)
    return {"value": round(N_REQ / sec, 2), "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{steps} full decode steps of 64 requests at context 128 (fp32 weights, pools filled with "
                      f"Bernoulli(0.15) bits instead of a CPU prefill), {sec:.2f} s/step after {warmup} warm-up"}


# --------------------------------------------------------------------------- arms
def config_dict(world: int, max_len) -> dict:
    # identical in both arms: the reference arm times ONE replica's 64 requests on the host's cores whatever N is
    return {"workload": "decode_0p5b_64req: spiking Qwen2.5-0.5B shape, T=4, bf16, 64 concurrent requests per GPU, "
                        "128-token prompts, greedy decode, page 16, CUDA-graph decode step",
            "requests_per_gpu": N_REQ, "prompt_len": PROMPT_LEN, "block_size": BLOCK_SIZE, "max_model_len": max_len,
            "parallelism": f"{world} independent replica(s), requests sharded, no data-path collective",
            "l2": "inputs larger than L2: every step streams ~1 GB of weights plus the layers' pools"}


def run_own(args) -> None:
    import torch.distributed as dist

    rank, world, local = dist_info()
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    K, W = args.steps, max(args.warmup, 3)
    R = max(args.repeats, 1)
    from spikeinfer_b200.engine.replicas import max_over_ranks, shard_requests

    cfg, model, rates = build_model(device, seed=1234)
    all_prompts = job_prompts(cfg, 1234, N_REQ * world)
    mine = shard_requests(N_REQ * world, world, rank)  # this replica's share of the job's requests
    max_len = model_len(total_decode_steps(K, W))
    engine, launches_per_step = build_engine(model, all_prompts[mine.start:mine.stop], max_len, device)

    def timed_steps(eng) -> float:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        for _ in range(K):
            eng.decode_step()
        stop.record()
        barrier()
        return start.elapsed_time(stop)

    # ---- value: tokens stay on the device; the median region is the headline, all of them its spread -------
    with ClockSampler(local) as clocks:  # started ahead of the warm-up so that it is sampling when the clock starts
        for _ in range(W):
            engine.decode_step()
        torch.cuda.synchronize(device)
        snap = engine.snapshot()
        if args.profiler_range:
            torch.cuda.profiler.start()
        ms = timed_steps(engine)
        if args.profiler_range:
            torch.cuda.profiler.stop()
        regions = [ms]
        for _ in range(R - 1):
            engine.restore(snap)
            regions.append(timed_steps(engine))
    # ---- e2e: host-in-the-loop steps ---------------------------------------
    def timed_host_steps() -> float:
        barrier()
        t0 = time.perf_counter()
        for _ in range(K):
            host.copy_(engine.step_host(host))
        torch.cuda.synchronize(device)
        return (time.perf_counter() - t0) * 1e3

    host = engine.host_in
    engine.restore(snap)
    host.copy_(engine.state.next_tokens.cpu())
    for _ in range(W):
        host.copy_(engine.step_host(host))
    snap_host = engine.snapshot()
    e2e_regions = []
    for _ in range(R):
        engine.restore(snap_host)
        host.copy_(engine.state.next_tokens.cpu())
        e2e_regions.append(timed_host_steps())
    engine.state.check_status()
    # ---- strong scaling: 64 requests in the whole job ----------------------------------------------------
    strong_ms = None
    if world > 1 and N_REQ % world == 0:
        share = N_REQ // world
        small, _ = build_engine(model, all_prompts[rank * share:(rank + 1) * share], max_len, device)
        for _ in range(W):
            small.decode_step()
        strong_ms = timed_steps(small)
        del small

    reduced = max_over_ranks(regions + e2e_regions + ([strong_ms] if strong_ms is not None else []), device)
    regions, e2e_regions = reduced[:R], reduced[R:2 * R]
    # the region of median duration stands for the K timed steps (a single region can catch a stray host hiccup)
    ms, e2e_ms = statistics.median_low(regions), statistics.median_low(e2e_regions)

    if rank == 0:
        tok = N_REQ * K * world
        line = {
            "metric": METRIC, "value": round(tok / (ms * 1e-3), 1), "unit": UNIT, "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": round(ms / K, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_dict(world, max_len),
            "e2e": {"value": round(tok / (e2e_ms * 1e-3), 1), "unit": UNIT,
                    "h2d_bytes_per_step": N_REQ * 8, "d2h_bytes_per_step": N_REQ * 8,
                    "ms_per_step": round(e2e_ms / K, 4)},
            "spread": {"note": f"the same {K} steps repeated from the same batch state; value and e2e are the region of median duration",
                       "ms_per_step": stats([r / K for r in regions]),
                       "tok_per_s": stats([tok / (r * 1e-3) for r in regions], 1),
                       "e2e_ms_per_step": stats([r / K for r in e2e_regions]),
                       "e2e_tok_per_s": stats([tok / (r * 1e-3) for r in e2e_regions], 1)},
            "gpu_launches": launches_per_step * K,
            "gpu_launches_per_step": launches_per_step,
            "clocks": clocks.summary(),
            "firing_rates": {k: round(v, 3) for k, v in rates.items()},
        }
        if strong_ms is not None:
            strong_ms = reduced[2 * R]
            line["strong_scaling"] = {"requests_total": N_REQ, "requests_per_gpu": N_REQ // world,
                                      "tok_per_s": round(N_REQ * K / (strong_ms * 1e-3), 1),
                                      "ms_per_step": round(strong_ms / K, 4)}
        else:
            line["strong_scaling"] = {"requests_total": N_REQ, "requests_per_gpu": N_REQ,
                                      "tok_per_s": round(N_REQ * K / (ms * 1e-3), 1), "ms_per_step": round(ms / K, 4),
                                      "note": "one GPU: the headline itself"}
        del engine
        line["roofline"] = attention_roofline(device, repeats=R)
        line["roofline_lif"] = lif_roofline(device, repeats=R)
        if world == 1 and not args.no_serving:
            line["closed_loop"] = {
                "protocol": "N requests, C in flight, 128 prompt tokens, 64 greedy output tokens, ignore_eos; prefill, "
                            "admission, host visits and release inside the clock",
                "runs": [closed_loop(model, cfg, device, c, n) for c, n in ((64, 128), (32, 64), (8, 32), (1, 8))],
                "packed_prefill": closed_loop(model, cfg, device, 64, 128, packed_prefill=True)}
            line["open_loop"] = open_loop(model, cfg, device)
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline()
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_reference(args) -> None:
    """The reference's CPU implementation of the path (oracle port), all host threads, rank 0 only."""
    rank, world, _ = dist_info()
    if rank != 0:
        return
    # One host has one set of cores: the CPU arm is ONE replica's 64 requests on all of them, whatever N is
    # (under a multi-rank launcher the other ranks leave at once and the launcher's one-thread default is undone).
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    K = args.steps
    W = max(args.warmup, 3)  # the same clamp as the own arm, so that both arms print the same max_model_len
    max_len = model_len(total_decode_steps(K, W))
    W_cpu = max(min(args.warmup, 2), 1)  # a CPU step takes a third of a second: two warm-up steps settle it
    sample = CpuDecodeSample(max_len=max_len)
    sec = time_cpu_steps(sample, K, W_cpu)
    value = round(N_REQ / sec, 2)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": K,
        "warmup": W, "ms_per_step": round(sec * 1e3, 2), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config_dict(max(world, 1), max_len),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": "each step = one full decode step of ONE replica's 64 requests at context 128+ on "
                                   "all of this host's cores, whatever --gpus is (fp32, pools pre-filled with "
                                   f"Bernoulli(0.15) bits instead of a CPU prefill; {W_cpu} CPU warm-up steps)"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def make_tp_group(dist, rank: int, world: int, tp: int):
    """The NCCL group of `rank`'s tensor-parallel peers: ranks [g*tp, (g+1)*tp).  Every rank creates every group, in
    the same order, as torch.distributed requires; only its own is returned."""
    mine = None
    for g in range(world // tp):
        pg = dist.new_group(list(range(g * tp, (g + 1) * tp)), backend="nccl")
        if rank // tp == g:
            mine = pg
    return mine


def run_tp7b(args) -> None:
    """Secondary workload (the long-context tensor-parallel configuration): spiking Qwen2.5-7B shape (28 layers, hidden 3584, 28/4 heads,
    head_dim 128, MLP 18944, vocab 152064, T=4, bf16), 256 concurrent decode sequences per replica with ragged
    contexts log-uniform in [1k, 32k], head-sharded tensor parallel over min(N, 4) GPUs (NCCL all-reduce after
    o_proj and down_proj), N/4 replicas beyond that.  The pools are filled with random bits and the batch state
    is installed directly instead of prefilling 2.3 M tokens; every timed step is a full decode step."""
    import math

    import torch.distributed as dist

    from spikeinfer_b200 import _lib
    from spikeinfer_b200.engine.decode_engine import SpikeDecodeEngine
    from spikeinfer_b200.engine.replicas import max_over_ranks
    from spikeinfer_b200.modeling import SpikingQwenConfig, SpikingQwenModel
    from spikeinfer_b200.tensor_parallel import shard_config

    # In-switch reduction (NVLS) is left off: the all-reduce is captured in a CUDA graph here and a rank that
    # exits while bound to an NVLink multicast object can disturb its peers on shared machines.
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, world, local = dist_info()
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)

    def stage(msg):
        if args.verbose:
            print(f"[rank {rank}] {msg}", file=sys.stderr, flush=True)

    tp = args.tp_size or min(world, 4)
    if world % tp:
        raise SystemExit(f"world size {world} is not a multiple of the tensor-parallel size {tp}")
    group = None
    if world > 1:
        # Exactly ONE NCCL communicator per process: the tensor-parallel group's.  The job-wide group is gloo and
        # carries only host-side barriers and the max-reduce of the timings, after a device synchronise.  (With an
        # NCCL job-wide group next to NCCL sub-groups, the timing loop had collectives of two communicators in
        # flight on the same GPUs -- the job-wide barrier on its own internal stream, the sub-group's all-reduces
        # inside the replayed graph -- with no common order across ranks, which NCCL documents as deadlock-prone.)
        dist.init_process_group("gloo")
        group = make_tp_group(dist, rank, world, tp) if tp > 1 else None
    cfg = SpikingQwenConfig(vocab_size=152064, hidden_size=3584, intermediate_size=18944,
                            num_hidden_layers=args.tp_layers or 28, num_attention_heads=28, num_key_value_heads=4,
                            head_dim=128)
    lcfg = shard_config(cfg, tp)
    weights = random_weights_device(lcfg, device, torch.bfloat16, seed=100 + rank // tp)  # replicated parts differ per
    model = SpikingQwenModel(lcfg, weights, device=device, tp_group=group if tp > 1 else None)  # rank: irrelevant for timing
    del weights
    stage("model built")
    if tp > 1:  # first collective of the group outside any capture: communicator set-up happens here
        probe = torch.ones(1, device=device)
        dist.all_reduce(probe, group=group)
        torch.cuda.synchronize(device)
        stage(f"group all-reduce ok ({probe.item():.0f})")
    n_seq = args.tp_seqs
    g = torch.Generator(device="cpu").manual_seed(5 + rank // tp)
    lo, hi = math.log(1024.0), math.log(32768.0)
    ctx = torch.exp(torch.rand(n_seq, generator=g) * (hi - lo) + lo).long().clamp(1024, 32768).tolist()
    K, W = args.steps, max(args.warmup, 3)
    max_len = 32768 + 2 * (K + W) + 64
    blocks = sum(-(-(c + 2 * (K + W) + 16) // BLOCK_SIZE) for c in ctx) + 1
    engine = SpikeDecodeEngine(model, num_blocks=blocks, block_size=BLOCK_SIZE, max_num_seqs=n_seq, max_model_len=max_len)
    for k, v in engine.cache.layers:  # ~12.5 % set bits everywhere
        for pool in (k, v):
            r = torch.randint(-2**31, 2**31 - 1, (3, *pool.shape), dtype=torch.int32, device=device)
            pool.copy_(r[0] & r[1] & r[2])
            del r
    for row, c in enumerate(ctx):
        table = engine.state.take_blocks(-(-c // BLOCK_SIZE))
        engine.state.admit(row, table, c, row % cfg.vocab_size)
        engine.ledger.admit(row, c)
    engine.free_rows = []
    torch.cuda.synchronize(device)
    stage("pools filled, rows admitted")
    lib = _lib.load()
    before = lib.spk_launch_count()
    engine.capture()
    launches_per_step = (lib.spk_launch_count() - before) // 5  # three warm-up passes and the two captured forms
    torch.cuda.synchronize(device)
    stage("decode graph captured")

    def barrier():
        # device first, then the host-side (gloo) barrier: no NCCL collective besides the group's own is ever issued
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()

    with ClockSampler(local) as clocks:  # started ahead of the warm-up so that it is sampling when the clock starts
        for _ in range(W):
            engine.decode_step()
        torch.cuda.synchronize(device)
        stage("warm-up replays done")
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        stage("barrier passed")
        start.record()
        for _ in range(K):
            engine.decode_step()
        stop.record()
        barrier()
    stage("timed steps done")
    engine.state.check_status()
    (ms,) = max_over_ranks([start.elapsed_time(stop)], "cpu")  # host tensors: the job-wide group is gloo
    # share of the step spent in the all-reduces: the same replays with the reduction switched off cannot be
    # captured here (the graph holds them), so a separate loop times the bare collective on the step's tensor
    ar_us = None
    if tp > 1:
        buf = torch.zeros(lcfg.T * n_seq, cfg.hidden_size, dtype=torch.bfloat16, device=device)
        for _ in range(5):
            dist.all_reduce(buf, group=group)
        torch.cuda.synchronize(device)
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(20):
            dist.all_reduce(buf, group=group)
        a1.record()
        torch.cuda.synchronize(device)
        (ar_us,) = max_over_ranks([a0.elapsed_time(a1) * 1e3 / 20], "cpu")
    sum_ctx = sum(ctx)
    if rank == 0:
        kv_bytes = sum_ctx * lcfg.T * lcfg.num_key_value_heads * 2 * 4 * 4  # K+V words of one layer on one GPU
        print(json.dumps({
            "workload": "tp7b_256seq_longctx", "metric": "decode_tok_per_s_7B_spiking_T4", "unit": UNIT,
            "value": round(n_seq * (world // tp) * K / (ms * 1e-3), 1), "n_gpus": world, "tensor_parallel": tp,
            "replicas": world // tp, "steps": K, "warmup": W, "ms_per_step": round(ms / K, 3), "dtype": "bf16",
            "data": "synthetic (pools pre-filled with random bits, no prefill)", "sequences_per_replica": n_seq,
            "sum_context_tokens": sum_ctx, "attention_kv_bytes_per_layer_per_gpu": kv_bytes,
            "all_reduce_bytes_per_call": lcfg.T * n_seq * cfg.hidden_size * 2, "all_reduces_per_step": 2 * cfg.num_hidden_layers if tp > 1 else 0,
            "all_reduce_us_per_call_back_to_back": None if ar_us is None else round(ar_us, 1),
            "all_reduce_share_of_step": None if ar_us is None else round(ar_us * 2 * cfg.num_hidden_layers / (ms / K * 1e3), 3),
            "layers": cfg.num_hidden_layers,
            "gpu_launches_per_step": launches_per_step, "clocks": clocks.summary()}), flush=True)
    if world > 1:
        # the captured graph holds the communicator's kernels: release it before the group is torn down
        import gc

        dist.barrier()
        torch.cuda.synchronize(device)
        engine.graph = None
        del engine, model
        gc.collect()
        torch.cuda.synchronize(device)
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profiler-range", action="store_true",
                    help="bracket the timed decode steps with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    ap.add_argument("--kernel-bench", choices=["attn", "lif", "step"], default=None,
                    help="time only the kernel-level configuration of the attention or the LIF kernel")
    ap.add_argument("--attn-page-major", action="store_true",
                    help="kernel-level attention timing on the page-major pool layout [block, T, H_kv, K|V, slot, W]")
    ap.add_argument("--attn-overlap", action="store_true",
                    help="kernel-level attention timing with programmatic dependent launch between calls")
    ap.add_argument("--attn-form", choices=["auto", "general", "tcgen05"], default="auto",
                    help="form of the attention kernel for --kernel-bench attn (auto: what the library picks)")
    ap.add_argument("--pools", type=int, default=24, help="distinct K/V pools of --kernel-bench attn")
    ap.add_argument("--rows", type=int, default=0, help="--kernel-bench attn: this many rows of --keys keys each")
    ap.add_argument("--keys", type=int, default=0)
    ap.add_argument("--repeats", type=int, default=5, help="timed regions per quantity (median, min and max are reported)")
    ap.add_argument("--no-serving", action="store_true", help="skip the closed-loop / open-loop serving measurements")
    ap.add_argument("--tokens", type=int, default=8192, help="tokens of --kernel-bench lif")
    ap.add_argument("--workload", choices=["decode_0p5b", "tp7b"], default="decode_0p5b",
                    help="tp7b: the 7B-shape long-context tensor-parallel decode step (secondary line)")
    ap.add_argument("--tp-seqs", type=int, default=256, help="sequences per replica of --workload tp7b")
    ap.add_argument("--tp-size", type=int, default=0, help="tensor-parallel group size of --workload tp7b (default min(N, 4))")
    ap.add_argument("--tp-layers", type=int, default=0, help="layers of --workload tp7b (default 28)")
    ap.add_argument("--verbose", action="store_true", help="print progress of the set-up stages to stderr")
    args = ap.parse_args()
    global ATTN_OVERLAP, ATTN_PAGE_MAJOR
    ATTN_OVERLAP, ATTN_PAGE_MAJOR = args.attn_overlap, args.attn_page_major
    if args.workload == "tp7b" and args.impl == "own" and not args.kernel_bench:
        run_tp7b(args)
    elif args.kernel_bench:
        run_kernel_bench(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_own(args)


if __name__ == "__main__":
    main()
