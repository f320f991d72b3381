"""Continuous-batching decode runner: prefill in eager mode, decode steps as one CUDA-graph replay.

Plays the role of ``ModelRunner`` + ``CUDAGraphRunner`` of the reference
(``spikeinfer/engine/model_runner.py:143-215``, ``:218-287``) for the decode path, with two
differences: the per-step metadata is advanced on the GPU by ``DecodeBatchState.advance`` inside the
captured graph (no host-built tensors, no buffer copies at replay), and greedy sampling (argmax) is
captured too, so a step is a single graph launch that feeds itself.  Like the reference
(``model_runner.py:143-182``, ``config.py:118-126``) a step replays the smallest captured bucket of rows
that covers the batch: rows are handed out lowest first, a bucket of b rows runs rows 0..b-1, and a bucket
is captured the first time it is needed.  ``step_host`` is the
host-in-the-loop form (tokens cross PCIe both ways every step, as in the reference engine, which needs
them for detokenisation and stop checks).
"""
from __future__ import annotations

import torch

from ..attention import AttentionMetadata, build_prefill_rows
from ..kernels import argmax_rows, argmax_workspace_bytes
from ..modeling import SpikingQwenModel
from .batch_state import DecodeBatchState
from .block_ledger import BlockLedger, covering_bucket, row_buckets
from .spike_cache import PagedSpikeCache


class SpikeDecodeEngine:
    def __init__(self, model: SpikingQwenModel, num_blocks: int, block_size: int = 16, max_num_seqs: int = 64,
                 max_model_len: int = 4096, use_graph: bool = True, packed_prefill: bool = False,
                 graph_buckets: bool = True, short_context_keys: int = 768) -> None:
        c = model.config
        self.model = model
        self.device = model.device
        self.block_size = block_size
        self.max_num_seqs = max_num_seqs
        self.max_blocks = -(-max_model_len // block_size)
        if model.rope_table is None or model.rope_table.shape[0] < self.max_blocks * block_size:
            model.build_rope_table(self.max_blocks * block_size)
        self.cache = PagedSpikeCache(c.num_hidden_layers, c.T, c.num_key_value_heads, c.head_dim, num_blocks,
                                     block_size, device=self.device)
        self.state = DecodeBatchState(max_num_seqs, self.max_blocks, num_blocks, block_size, device=self.device)
        self.ledger = BlockLedger(num_blocks - 1, block_size, self.max_blocks)  # host count of the device free list
        self.use_graph = use_graph
        # row counts a step can run on: powers of two up to max_num_seqs, and max_num_seqs itself
        self.buckets = row_buckets(max_num_seqs) if graph_buckets else [max_num_seqs]
        self.graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self.host_graphs: dict[int, torch.cuda.CUDAGraph] = {}
        # While no row holds more than `short_context_keys` keys (the host knows: BlockLedger) a step is replayed from
        # graphs whose attention calls see only that many table entries: up to 768 keys the attention cuts no row,
        # so those calls have no combine pass, whatever max_model_len is.  0 pages = the tables are that short anyway.
        short = min(self.max_blocks, max(short_context_keys, 0) // block_size)
        self.short_blocks = short if 0 < short < self.max_blocks else 0
        self.short_graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self.short_host_graphs: dict[int, torch.cuda.CUDAGraph] = {}
        # True: prompts attend through the packed popcount kernel in one batched launch per layer (3x faster at
        # 64 prompts of 128 tokens, exact-score fp32 softmax).  False (default): one SDPA per sequence on unpacked
        # spikes in the model dtype, as the reference does; in bf16 that rounds the probabilities to bf16, so
        # the two differ at the 1e-2 level there, enough to flip near-tie tokens.  In fp32 they agree to 1e-5.
        self.packed_prefill = packed_prefill
        self.free_rows = list(range(max_num_seqs - 1, -1, -1))
        self.host_in = torch.zeros(max_num_seqs, dtype=torch.int64).pin_memory()
        self.host_out = torch.zeros(max_num_seqs, dtype=torch.int64).pin_memory()
        self.sample_ws = torch.empty(argmax_workspace_bytes(max_num_seqs), dtype=torch.uint8, device=self.device)
        self.token_log: torch.Tensor | None = None  # device log of decode_steps
        self.host_log: torch.Tensor | None = None

    # -- prefill ----------------------------------------------------------
    @torch.no_grad()
    def add_requests(self, prompts: list[list[int]]) -> list[int]:
        """Prefill ``prompts`` in one eager batch and install them as decode rows.  Returns the rows."""
        if len(prompts) > len(self.free_rows):
            raise RuntimeError("no free decode row")
        # admission control before anything is taken from the device list (the reference's scheduler asks
        # BlockManager.can_allocate first, spikeinfer/engine/scheduler.py:160): nothing is touched on refusal
        why = self.ledger.admission_error([len(p) for p in prompts])
        if why is not None:
            raise RuntimeError(f"cannot admit: {why}")
        bs, dev = self.block_size, self.device
        ids, pos, slot_parts, starts, lens, tables = [], [], [], [], [], []
        for p in prompts:
            n_blocks = -(-len(p) // bs)
            table = self.state.take_blocks(n_blocks)
            positions = torch.arange(len(p), device=dev)
            slot_parts.append(table.to(torch.int64)[positions // bs] * bs + positions % bs)
            starts.append(len(ids))
            ids += p
            pos.append(positions)
            lens.append(len(p))
            tables.append(table)
        meta = AttentionMetadata(
            slot_mapping=torch.cat(slot_parts), block_size=bs, prefill_query_starts=starts,
            prefill_query_lens=lens, prefill_context_lens=[0] * len(lens), prefill_block_tables=tables,
            status=self.state.status)
        if self.packed_prefill:
            build_prefill_rows(meta, pad_block=self.cache.pad_block)
        input_ids = torch.tensor(ids, dtype=torch.int64, device=dev)
        hidden = self.model.forward_paged(input_ids, torch.cat(pos), self.cache.layers, meta)
        last = torch.tensor([s + n - 1 for s, n in zip(starts, lens)], dtype=torch.int64, device=dev)
        first_tokens = self.model.compute_logits(hidden, last).argmax(dim=-1)
        rows = []
        for i, (table, n) in enumerate(zip(tables, lens)):
            row = self.free_rows.pop()
            self.state.admit(row, table, n, 0)
            self.ledger.admit(row, n)
            rows.append(row)
        idx = torch.tensor(rows, dtype=torch.int64, device=dev)
        self.state.next_tokens[idx] = first_tokens
        self.state.input_ids[idx] = first_tokens
        return rows

    def release(self, row: int) -> None:
        self.state.release(row)
        self.ledger.release(row)
        self.free_rows.append(row)
        self.free_rows.sort(reverse=True)  # lowest row first out: the batch stays within the smallest bucket

    # -- snapshots (benchmarks and tests: repeat the same steps from the same state) ---------------------
    def _state_tensors(self):
        st = self.state
        return (st.free_list, st._free_count, st.active, st.seq_lens, st.positions, st.slot_mapping, st.block_tables,
                st.input_ids, st.next_tokens)

    def snapshot(self) -> dict:
        """Batch state, block ledger and free rows as they are now (the pools are not copied: steps replayed
        from a snapshot rewrite the same slots with the same bits)."""
        return dict(tensors=[t.clone() for t in self._state_tensors()], free=self.ledger.free,
                    seq_lens=dict(self.ledger.seq_lens), free_rows=list(self.free_rows))

    def restore(self, snap: dict) -> None:
        for t, s in zip(self._state_tensors(), snap["tensors"]):
            t.copy_(s)
        self.ledger.free = snap["free"]
        self.ledger.seq_lens = dict(snap["seq_lens"])
        self.free_rows = list(snap["free_rows"])

    # -- decode -----------------------------------------------------------
    def _meta(self, rows: int, short: bool = False) -> AttentionMetadata:
        st = self.state
        tables = st.block_tables[:rows, :self.short_blocks] if short else st.block_tables[:rows]
        # tables and lengths are written by the metadata kernel at the head of the step, layers before any attention
        return AttentionMetadata(
            slot_mapping=st.slot_mapping[:rows], block_size=self.block_size, num_decode_tokens=rows,
            block_tables=tables, seq_lens=st.seq_lens[:rows], status=st.status, tables_settled=True)

    def short_context(self) -> bool:
        """True when the step about to run touches no more than the short tables hold in any row."""
        if not self.short_blocks:
            return False
        longest = max(self.ledger.seq_lens.values(), default=0) + 1  # the token being decoded included
        return longest <= self.short_blocks * self.block_size

    @property
    def meta(self) -> AttentionMetadata:
        """Decode metadata over all rows."""
        return self._meta(self.max_num_seqs)

    def _body(self, rows: int | None = None, short: bool = False) -> None:
        st = self.state
        rows = self.max_num_seqs if rows is None else rows
        st.advance(rows)
        hidden = self.model.forward_paged(st.input_ids[:rows], st.positions[:rows], self.cache.layers,
                                          self._meta(rows, short))
        logits = self.model.compute_logits(hidden)
        argmax_rows(logits, out=st.next_tokens[:rows], workspace=self.sample_ws)  # greedy, inside the graph

    def bucket_for_batch(self) -> int:
        """Smallest bucket that covers every admitted row (rows are handed out lowest first)."""
        return covering_bucket(self.buckets, self.ledger.seq_lens)

    @property
    def graph(self) -> torch.cuda.CUDAGraph | None:
        """The captured step over all rows (None before capture)."""
        return self.graphs.get(self.max_num_seqs)

    @graph.setter
    def graph(self, value) -> None:
        if value is not None:
            raise ValueError("assign None to drop the captured graphs")
        self.graphs.clear()
        self.host_graphs.clear()
        self.short_graphs.clear()
        self.short_host_graphs.clear()

    @torch.no_grad()
    def capture(self, rows: int | None = None, short: bool = False) -> None:
        """Capture one decode step over ``rows`` rows (default: all), with full or short tables.  Warm-up runs would
        advance real rows, so capture happens on a snapshot of the batch state and the pools' pad block only: the
        state is saved and restored.  All graphs share one memory pool (they never run at the same time)."""
        rows = self.max_num_seqs if rows is None else rows
        graphs, host_graphs = (self.short_graphs, self.short_host_graphs) if short else (self.graphs, self.host_graphs)
        st = self.state
        saved = [t.clone() for t in self._state_tensors()]
        active = st.active.clone()
        st.active.zero_()  # every row is a pad row during warm-up and capture: only the pad block is written
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(3):
                self._body(rows, short)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        any_graph = next(iter(self.graphs.values()), None) or next(iter(self.short_graphs.values()), None)
        with torch.cuda.graph(graph, pool=any_graph.pool() if any_graph is not None else None):
            self._body(rows, short)
        graphs[rows] = graph
        # the host-in-the-loop form of the same step: the token copies from and to pinned host memory are nodes of
        # the graph (fixed addresses: host_in, host_out), so a step is one launch and one wait on the host side
        host_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(host_graph, pool=graph.pool()):
            st.next_tokens[:rows].copy_(self.host_in[:rows], non_blocking=True)
            self._body(rows, short)
            self.host_out[:rows].copy_(st.next_tokens[:rows], non_blocking=True)
        host_graphs[rows] = host_graph
        for t, s in zip(self._state_tensors(), saved):
            t.copy_(s)
        st.active.copy_(active)

    def capture_all(self) -> None:
        """Capture every bucket now (largest first, so that the shared pool is sized once) instead of on first use."""
        for b in sorted(self.buckets, reverse=True):
            if b not in self.graphs:
                self.capture(b)
            if self.short_blocks and b not in self.short_graphs:
                self.capture(b, short=True)

    @torch.no_grad()
    def decode_step(self) -> None:
        """One token for every active row; tokens stay on the device (``state.next_tokens``)."""
        rows = self.bucket_for_batch()
        short = self.short_context()
        if self.use_graph:
            graphs = self.short_graphs if short else self.graphs
            if rows not in graphs:
                self.capture(rows, short)
            graphs[rows].replay()
        else:
            self._body(rows, short)
        self.ledger.advance()

    @torch.no_grad()
    def decode_steps(self, k: int) -> torch.Tensor:
        """``k`` decode steps per host visit: the steps are enqueued back to back (each feeds the next from
        ``state.next_tokens`` on the device), every step's tokens are kept in a device log, and the host
        waits once, for a single ``[k, max_num_seqs]`` copy.  The reference visits the host after every
        step (``sampler.py:81`` ``.tolist()``, ``llm_engine.py:359-387``); stop conditions are then checked on
        the returned block, so up to ``k - 1`` tokens per finished row are decoded in vain."""
        if k < 1:
            raise ValueError("k must be at least 1")
        if self.token_log is None or self.token_log.shape[0] < k:
            self.token_log = torch.zeros(k, self.state.next_tokens.numel(), dtype=torch.int64, device=self.device)
            self.host_log = torch.zeros(k, self.state.next_tokens.numel(), dtype=torch.int64).pin_memory()
        for i in range(k):
            self.decode_step()
            self.token_log[i].copy_(self.state.next_tokens, non_blocking=True)
        self.host_log[:k].copy_(self.token_log[:k], non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return self.host_log[:k]

    @torch.no_grad()
    def step_host(self, tokens_in: torch.Tensor | None = None) -> torch.Tensor:
        """Host-in-the-loop step: ``tokens_in`` (pinned int64 ``[max_num_seqs]``, the tokens to feed) is
        copied to the device, the step runs, and the sampled tokens are returned in pinned host memory."""
        if not self.use_graph or tokens_in is None:
            if tokens_in is not None:
                self.state.next_tokens.copy_(tokens_in, non_blocking=True)
            self.decode_step()
            self.host_out.copy_(self.state.next_tokens, non_blocking=True)
            torch.cuda.current_stream(self.device).synchronize()
            return self.host_out
        # one replay holds the copy in, the step and the copy out
        rows = self.bucket_for_batch()
        short = self.short_context()
        host_graphs = self.short_host_graphs if short else self.host_graphs
        if rows not in host_graphs:
            self.capture(rows, short)
        if tokens_in.data_ptr() != self.host_in.data_ptr():
            self.host_in.copy_(tokens_in)  # host to host: the graph reads the engine's own pinned buffer
        host_graphs[rows].replay()
        self.ledger.advance()
        torch.cuda.current_stream(self.device).synchronize()
        return self.host_out
