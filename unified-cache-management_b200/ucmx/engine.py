"""One decode step of sparse-KV retrieval for a ragged batch, layer by layer:
pool the newly filled blocks -> score every block of every request -> per-request top-k ->
gather the selected K and V blocks into a contiguous working set.

This is the sequence the reference spreads over ESA's hooks (ucm/sparse/esa/esa.py:286-399: start_retrieval,
wait_retrieval_and_start_load, block_repre_data, launch_transfer_task) with a CPU thread pool in the
middle; here every stage is a kernel on one stream and nothing leaves the device unless asked to.

Representatives are kept per layer in a bf16 table indexed by PHYSICAL block id, so the request's
block table is at once the slot list for scoring and the id map of the top-k output, and the
selected ids feed the gather directly.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from . import ops
from .workloads import KvShape, RaggedBatch


class DecodeRetrievalEngine:
    def __init__(self, shape: KvShape, batch: RaggedBatch, device: torch.device, *, n_layers: Optional[int] = None,
                 with_kv_pool: bool = True, heads_local: Optional[int] = None, seed: int = 0,
                 score_reduce=None, peer_exchange=None, order: int = ops.ORDER_SCORE_DESC, delta: bool = False,
                 overlap: bool = False):
        """heads_local: KV heads held by this rank under tensor parallelism (default: all).
        score_reduce: callable applied in place to the fp32 score vector between scoring and top-k
        (the tensor-parallel all-reduce); None on a single rank.
        peer_exchange: a parallel.PeerScoreExchange; partial scores then go into peer-mapped memory and are
        summed inside the top-k kernel instead of by score_reduce.
        order: order of the selected ids (best first, or ascending block position).
        delta: keep a resident working set per layer and request and move only the blocks that are new with respect
        to the previous step's selection (what ESA does, ucm/sparse/esa/esa.py:313-338): top-k of block positions in
        ascending order -> resident-set remap -> block-to-block move of the misses.
        overlap: scoring and selection of layer l+1 run on a second stream while layer l's blocks move (they do not
        depend on each other); the step is then bounded by the block moves alone."""
        self.shape, self.batch, self.device = shape, batch, device
        self.L = n_layers if n_layers is not None else shape.n_layers
        self.H = heads_local if heads_local is not None else shape.n_kv_heads
        self.Hq = shape.n_q_heads * self.H // shape.n_kv_heads
        self.D, self.T = shape.head_dim, shape.block_tokens
        self.score_reduce = score_reduce
        self.peer_exchange = peer_exchange
        self.order = ops.ORDER_INDEX_ASC if delta else order
        self.delta = delta
        self.overlap = bool(overlap) and with_kv_pool
        self._select_stream = torch.cuda.Stream(device=device) if self.overlap else None
        i32 = dict(dtype=torch.int32, device=device)
        self.offsets = torch.from_numpy(batch.offsets).to(device)
        self.k_per_req = torch.from_numpy(batch.k_per_req).to(device)
        self.k_offsets = torch.from_numpy(batch.k_offsets).to(device)
        self.block_table = torch.from_numpy(batch.block_table).to(device)
        # physical id of each request's newest block (the one a decode step may have just filled)
        last = torch.from_numpy(batch.offsets[1:] - 1).long().to(device)
        self.new_block_ids = self.block_table[last].contiguous()
        g = torch.Generator(device=device).manual_seed(seed)
        self.gen = g
        E = self.H * self.D
        # representatives of every layer stay resident: [L, n_slots, H, 1, D] bf16
        self.rep_tables = torch.empty((self.L, batch.n_slots, self.H, 1, self.D), dtype=torch.bfloat16, device=device)
        for l in range(self.L):
            self.rep_tables[l].copy_((torch.randn((batch.n_slots, self.H, 1, self.D), generator=g, device=device) * 0.0884)
                                     .to(torch.bfloat16))
        self.kv_pool = None
        if with_kv_pool:
            # one layer's paged K and V pool, reused for every layer: [2, n_slots, T, H, D] bf16
            self.kv_pool = torch.empty((2, batch.n_slots, self.T, self.H, self.D), dtype=torch.bfloat16, device=device)
            chunk = 1024
            for p in range(2):
                for s in range(0, batch.n_slots, chunk):
                    e = min(s + chunk, batch.n_slots)
                    self.kv_pool[p, s:e].copy_(torch.randn((e - s, self.T, self.H, self.D), generator=g, device=device)
                                               .to(torch.bfloat16))
            self.staging = torch.empty((batch.total_k, 2, self.T * E * 2), dtype=torch.uint8, device=device)
        self.qbar = torch.empty((batch.n_req, E), dtype=torch.float32, device=device)
        self.scores = torch.empty((batch.total,), dtype=torch.float32, device=device)
        self.sel_ids = torch.full((self.L, batch.total_k), -1, **i32)
        self.sel_scores = torch.zeros((self.L, batch.total_k), dtype=torch.float32, device=device)
        self.sel_counts = torch.zeros((self.L, batch.n_req), **i32)
        self.out_stride = max(batch.max_k, 1)
        # host side of the end-to-end path
        self.q_dev = torch.empty((self.L, batch.n_req, self.Hq, self.D), dtype=torch.bfloat16, device=device)
        self.q_host: Optional[torch.Tensor] = None
        self.sel_host: Optional[torch.Tensor] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.host_graph: Optional[torch.cuda.CUDAGraph] = None
        self.launches_per_step = self.L * (3 if with_kv_pool else 2) + (1 if with_kv_pool else 0)
        self._pool_all = None
        if delta:
            if not with_kv_pool:
                raise ValueError("the delta step moves blocks: it needs the K/V pool")
            # resident working set: request r owns slots [k_offsets[r], k_offsets[r+1]) of `staging` in every layer
            n = batch.total_k
            self.slot_phys = torch.arange(n, **i32)
            self.slot_logical = torch.full((self.L, n), -1, **i32)
            self.slot_free = torch.ones((self.L, n), dtype=torch.uint8, device=device)
            self.remap_out = [(torch.full((n,), -1, **i32), torch.full((n,), -1, **i32), torch.full((n,), -1, **i32),
                               torch.zeros((batch.n_req,), **i32)) for _ in range(self.L)]
            self.moves = ops.MoveList(n, device)
            self.max_logical = int(batch.blocks_per_req.max())
            self.launches_per_step = self.L * 4 + 1

    # ---------------------------------------------------------------------------------- stages
    def make_queries(self) -> torch.Tensor:
        q = torch.randn((self.L, self.batch.n_req, self.Hq, self.D), generator=self.gen, device=self.device)
        self.q_dev.copy_(q.to(torch.bfloat16))
        return self.q_dev

    def pool_all_layers(self) -> None:
        """Representatives of the blocks that filled up since the last step, for every layer, in one launch: the
        rows go to slot `layer * n_slots + block id` of the stacked tables.  (Blocks fill between steps, so this
        need not wait for the layers to come round one by one.)"""
        if self._pool_all is None:
            ns = self.batch.n_slots
            ids = self.new_block_ids.repeat(self.L).contiguous()
            slots = (torch.arange(self.L, device=self.device, dtype=torch.int64)[:, None] * ns
                     + self.new_block_ids.long()[None, :]).reshape(-1).to(torch.int32).contiguous()
            self._pool_all = (ids, slots, self.rep_tables.view(self.L * ns, self.H, 1, self.D))
        ids, slots, table = self._pool_all
        ops.pool_blocks(self.kv_pool[0], ids, out_slots=slots, out_bf16=table)

    def pool_layer(self, layer: int) -> None:
        ops.pool_blocks(self.kv_pool[0], self.new_block_ids, out_slots=self.new_block_ids,
                        out_bf16=self.rep_tables[layer])

    def prefill_pool_all(self, layer: int) -> None:
        """Representatives of every block of the pool (what the last prefill chunk does)."""
        ops.pool_blocks(self.kv_pool[0], self.block_table, out_slots=self.block_table, out_bf16=self.rep_tables[layer])

    def score_layer(self, layer: int, early: bool = False) -> None:
        """early: the kernel ahead in the stream writes none of the scoring inputs (it is the previous layer's top-k or
        block move), so the scoring kernel may begin under its tail; it stores its scores only after that kernel's end."""
        if self.peer_exchange is not None:
            # the partial scores go straight into every rank's inbox; nothing is kept locally
            ops.score_dot_query(self.rep_tables[layer], self.offsets, self.q_dev[layer], total=self.batch.total,
                                slot_ids=self.block_table, n_kv_heads=self.H, exchange=self.peer_exchange)
            return
        ops.score_dot_query(self.rep_tables[layer], self.offsets, self.q_dev[layer], total=self.batch.total,
                            slot_ids=self.block_table, n_kv_heads=self.H, out=self.scores, early=early)
        if self.score_reduce is not None:
            self.score_reduce(self.scores)

    def topk_layer(self, layer: int) -> None:
        id_map = None if self.delta else self.block_table      # the delta step selects block positions, not pool ids
        if self.peer_exchange is not None:
            self.peer_exchange.topk(self.offsets, self.k_per_req, total=self.batch.total, out_stride=self.out_stride,
                                    order=self.order,
                                    id_map=id_map, out_offsets=self.k_offsets, out_idx=self.sel_ids[layer],
                                    out_scores=self.sel_scores[layer], out_counts=self.sel_counts[layer])
            return
        ops.topk_ragged(self.scores, self.offsets, self.k_per_req, out_stride=self.out_stride,
                        order=self.order, id_map=id_map, out_offsets=self.k_offsets,
                        out_idx=self.sel_ids[layer], out_scores=self.sel_scores[layer],
                        out_counts=self.sel_counts[layer])

    def gather_layer(self, layer: int) -> None:
        if self.delta:
            self.remap_layer(layer)
            self.move_layer(layer)
            return
        ops.gather_blocks([self.kv_pool[0], self.kv_pool[1]], self.sel_ids[layer], self.staging)

    def remap_layer(self, layer: int) -> None:
        """Which resident slot serves each selected block, and the (pool block -> resident slot) list of the misses."""
        ops.remap_resident(self.slot_logical[layer], self.slot_free[layer], self.slot_phys, self.k_offsets,
                           self.sel_ids[layer], self.k_offsets, max_logical=self.max_logical, max_slots=self.out_stride,
                           sel_counts=self.sel_counts[layer], src_map=self.block_table, src_map_offsets=self.offsets,
                           moves=self.moves, out=self.remap_out[layer])

    def move_layer(self, layer: int) -> None:
        ops.move_blocks([self.kv_pool[0], self.kv_pool[1]], self.moves, [self.staging[:, 0], self.staging[:, 1]])

    def drift_queries(self, rho: float = 0.98) -> None:
        """Next decode step's queries: a seeded random walk, q <- rho*q + sqrt(1-rho^2)*noise, so that consecutive
        selections overlap the way consecutive decode steps of one sequence do."""
        noise = torch.randn(self.q_dev.shape, generator=self.gen, device=self.device)
        self.q_dev.copy_((self.q_dev.float() * rho + noise * (1.0 - rho * rho) ** 0.5).to(torch.bfloat16))

    def loads_of_last_step(self) -> int:
        return int(sum(int(o[3].sum().item()) for o in self.remap_out))

    def layer_step(self, layer: int, gather_events=None, early: bool = False) -> None:
        """Score, select and gather one layer (pooling of new blocks is done for all layers at the start of a step).
        gather_events: an optional (before, after) pair of CUDA events recorded around the gather launch."""
        self.score_layer(layer, early=early)
        self.topk_layer(layer)
        if self.kv_pool is not None:
            if gather_events is not None:
                gather_events[0].record()
            self.gather_layer(layer)
            if gather_events is not None:
                gather_events[1].record()

    # ------------------------------------------------------------------------------------ steps
    @property
    def exchanges_scores(self) -> bool:
        return self.peer_exchange is not None or self.score_reduce is not None

    def all_layers(self, gather_events=None) -> None:
        """The launches of one step after pooling.  A single rank goes layer by layer.  Tensor-parallel ranks score one
        layer ahead: layer l+1's partial scores are computed and exchanged before layer l's blocks move, so the exchange
        (and whatever the ranks have drifted apart) is over long before layer l+1's top-k asks for the sums, instead of
        being waited for once per layer.  (Queries of all layers are known when the step starts: retrieval works on the
        previous decode step's queries, ucm/sparse/esa/esa.py:286-339.)  The peer exchange allows it: the top-k of a
        layer still follows that layer's scoring with no other scoring in between, and a rank can only be two rounds
        ahead of another after a top-k that waited for that rank's previous round."""
        if self.overlap:
            self._all_layers_two_streams(gather_events)
            return
        if not self.exchanges_scores:
            for l in range(self.L):
                self.layer_step(l, None if gather_events is None else gather_events[l], early=l > 0 and gather_events is None)
            return
        self.score_layer(0)
        for l in range(self.L):
            self.topk_layer(l)
            if l + 1 < self.L:
                self.score_layer(l + 1)
            if self.kv_pool is not None:
                if gather_events is not None:
                    gather_events[l][0].record()
                self.gather_layer(l)
                if gather_events is not None:
                    gather_events[l][1].record()

    def _all_layers_two_streams(self, gather_events=None) -> None:
        """Selection (score + top-k, with the exchange under tensor parallelism) on a stream of its own, one layer ahead of
        the block moves on the current stream.  Each layer has its own selection buffers, so layer l+1 may be selected
        while layer l's blocks move; the moves wait for their layer's selection through an event.  Works inside a graph
        capture (the second stream forks from and joins the capturing one)."""
        main = torch.cuda.current_stream(self.device)
        side = self._select_stream
        fork = torch.cuda.Event()
        fork.record(main)
        side.wait_event(fork)
        selected = [torch.cuda.Event() for _ in range(self.L)]
        with torch.cuda.stream(side):
            self.score_layer(0)
            self.topk_layer(0)
            selected[0].record(side)
        for l in range(self.L):
            if l + 1 < self.L:
                with torch.cuda.stream(side):
                    # behind layer l's top-k on this stream.  (Not in the delta step: there the scoring, started
                    # that much sooner, takes HBM time from the short move beside it - 1.90 against 1.79 ms per step.)
                    self.score_layer(l + 1, early=not self.delta)
                    self.topk_layer(l + 1)
                    selected[l + 1].record(side)
            main.wait_event(selected[l])
            if gather_events is not None:
                gather_events[l][0].record()
            self.gather_layer(l)
            if gather_events is not None:
                gather_events[l][1].record()
        main.wait_stream(side)

    def step(self) -> None:
        """All layers, inputs and outputs resident on the device."""
        if self.graph is not None:
            self.graph.replay()
            return
        if self.kv_pool is not None:
            self.pool_all_layers()
        self.all_layers()

    def capture(self, gather_events=None) -> torch.cuda.CUDAGraph:
        """Record the whole step once into a CUDA graph and return it.  Without events the graph also becomes the
        one step() replays.
        gather_events: optional list of one (before, after) pair of events per layer, created with
        torch.cuda.Event(enable_timing=True, external=True); they become event-record nodes of the graph, so after
        a replay they hold the times of that replay's gather launches.  (Such nodes cost about 6 us each, which
        is why the instrumented graph is a separate one.)"""
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            if self.kv_pool is not None:
                self.pool_all_layers()
            self.all_layers()               # warm up lazily initialised state outside capture
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            if self.kv_pool is not None:
                self.pool_all_layers()
            self.all_layers(gather_events)
        if gather_events is None:
            self.graph = graph
        return graph

    def alloc_host(self) -> None:
        self.q_host = torch.empty(self.q_dev.shape, dtype=torch.bfloat16).pin_memory()
        self.q_host.copy_(self.q_dev)
        self.sel_host = torch.empty(self.sel_ids.shape, dtype=torch.int32).pin_memory()
        self.cnt_host = torch.empty(self.sel_counts.shape, dtype=torch.int32).pin_memory()
        self._copy_stream = torch.cuda.Stream(device=self.device)
        self._q_ready = [torch.cuda.Event() for _ in range(self.L)]
        self._layer_done = [torch.cuda.Event() for _ in range(self.L)]

    def _enqueue_host_step(self, main: torch.cuda.Stream) -> None:
        """The end-to-end step as stream work, without the final wait: the copies run on their own stream; layer
        l's kernels wait for the event of their own queries only, and its results leave while layer l+1 computes,
        so the host link works beside the kernels instead of between them."""
        cs = self._copy_stream
        cs.wait_stream(main)                               # earlier work on the buffers has finished
        with torch.cuda.stream(cs):
            for l in range(self.L):
                self.q_dev[l].copy_(self.q_host[l], non_blocking=True)
                self._q_ready[l].record(cs)
        if self.kv_pool is not None:
            self.pool_all_layers()
        if self.overlap:
            # selection on its own stream, as in all_layers: layer l+1 is scored and selected (and its ids leave for
            # the host) while layer l's blocks move
            side = self._select_stream
            pooled = torch.cuda.Event()
            pooled.record(main)
            side.wait_event(pooled)
            for l in range(self.L):
                with torch.cuda.stream(side):
                    side.wait_event(self._q_ready[l])
                    self.score_layer(l)
                    self.topk_layer(l)
                    self._layer_done[l].record(side)
                with torch.cuda.stream(cs):
                    cs.wait_event(self._layer_done[l])
                    self.sel_host[l].copy_(self.sel_ids[l], non_blocking=True)
                    self.cnt_host[l].copy_(self.sel_counts[l], non_blocking=True)
                main.wait_event(self._layer_done[l])
                if self.kv_pool is not None:
                    self.gather_layer(l)
            main.wait_stream(side)
            main.wait_stream(cs)
            return
        for l in range(self.L):
            main.wait_event(self._q_ready[l])
            self.layer_step(l)
            self._layer_done[l].record(main)
            with torch.cuda.stream(cs):
                cs.wait_event(self._layer_done[l])
                self.sel_host[l].copy_(self.sel_ids[l], non_blocking=True)
                self.cnt_host[l].copy_(self.sel_counts[l], non_blocking=True)
        main.wait_stream(cs)

    def capture_host(self) -> None:
        """Record the end-to-end step - host-to-device copies, kernels, device-to-host copies, on both streams -
        into one CUDA graph; step_host() then replays it.  The pinned host buffers are part of the graph, so the
        caller keeps writing queries into q_host and reading selections from sel_host / cnt_host."""
        if self.score_reduce is not None or self.peer_exchange is not None:
            raise RuntimeError("the captured end-to-end step covers the single-rank path only")
        for _ in range(2):                                 # lazily initialised state is set up outside capture
            self.step_host()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._enqueue_host_step(torch.cuda.current_stream(self.device))
        self.host_graph = graph

    def step_host(self) -> torch.Tensor:
        """End to end with host buffers: each layer's queries come from pinned host memory and its
        selected block ids and counts go back to pinned host memory; returns after a final sync."""
        main = torch.cuda.current_stream(self.device)
        if self.host_graph is not None:
            self.host_graph.replay()
        else:
            self._enqueue_host_step(main)
        main.synchronize()
        return self.sel_host

    @property
    def h2d_bytes_per_step(self) -> int:
        return self.q_dev.numel() * 2

    @property
    def d2h_bytes_per_step(self) -> int:
        return self.sel_ids.numel() * 4 + self.sel_counts.numel() * 4

    # ------------------------------------------------------------------- algorithmic byte counts
    def bytes_score_layer(self) -> int:
        E = self.H * self.D
        return self.batch.total * (E * 2 + 4 + 4)          # rep row + slot id + score

    def bytes_gather_layer(self) -> int:
        return 2 * self.batch.total_k * 2 * self.T * self.H * self.D * 2   # K and V, read + write

    def bytes_pool_layer(self) -> int:
        E = self.H * self.D
        return self.batch.n_req * (self.T * E * 2 + E * 2)

    def tokens_scored_per_step(self) -> int:
        return self.batch.total * self.T * self.L
