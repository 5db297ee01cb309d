"""Drop-in for the reference's `gsa_offload_ops` module: the `CalKpreAndTopk` object GSA drives
(ucm/sparse/gsa/offload_ops/src/pybinds.cpp:9-26, cal_kpre_and_topk.cpp:7-263; called from
ucm/sparse/gsa/gsa.py:497-501, 616-654, 809, 914-954).

The reference object owns a copy thread and a calculate thread: `add_copy_req` queues a layer's
decode queries, the copy thread moves them to fp32 host memory, and once layer 0 is there the
calculate thread walks the layers, spinning on per-layer ready flags, and runs
TopkBlockSelector::SelectTopKBS (per request: group-mean query, per-block score = sum over KV heads
of the best representative, forced first/last windows, ascending indices) into the top-k cache.
`is_calculate_finish` reads the flag of the last layer.

Here a layer's work is enqueued on a private CUDA stream the moment its queries arrive: one ragged
scoring launch and one ragged top-k launch serve every decode request of the batch, writing straight
into the top-k cache rows; `is_calculate_finish` is an event query.  No host thread takes part.
Method names, argument meaning and the order in which GSA calls them are the reference's.
Representative caches and query caches are device tensors (the reference keeps both in host memory):
    kpre cache of a layer   [slots, n_kpre, kv_heads, head_size] - with n_kpre == 1, which is all GSA ever sets
                            (gsa.py:500), that is also the [slot, kv_head, rep, d] layout the kernels read
    q_cache[layer]          [max_bs, q_heads, head_size] fp32
    top-k cache of a layer  [bs, max_blocks] int32, on the device or in host memory (pinned for asynchronous copies)
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from . import ops

START_WINDOW, END_WINDOW = 1, 2          # TopkBlockSelector's defaults (select_topk_block.h:20)


class CalKpreAndTopk:
    def __init__(self, layer_num: int, block_size: int, max_bs: int, num_heads: int, head_size: int, *,
                 device: Optional[torch.device] = None):
        self.layer_num, self.block_size, self.max_bs = int(layer_num), int(block_size), int(max_bs)
        self.q_num_heads, self.head_size = int(num_heads), int(head_size)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.q_cache: List[torch.Tensor] = [torch.zeros((max_bs, num_heads, head_size), dtype=torch.float32, device=self.device)
                                            for _ in range(layer_num)]
        self.k_cache: List[torch.Tensor] = []               # kept for interface parity; the reference never fills it either
        self.k_num_heads, self.num_kpre = 0, 1
        self._kpre: List[torch.Tensor] = []
        self._topk: List[torch.Tensor] = []
        self._topk_lens: List[int] = []
        self._cal_topk_idx: List[int] = []
        self._is_decode: List[bool] = []
        self._slot_mapping: List[List[int]] = []
        self._calc_block_table = None
        self._calc_slot_mapping: List[int] = []
        self._need_topk = False
        self._need_kpre = False
        self._plan = None                                    # device-side batch description, rebuilt when the parameters change
        self._stream = torch.cuda.Stream(device=self.device)
        self._done = [None] * layer_num                      # event of each layer's last enqueued work
        self._pending_host: list = []                        # results on their way to host-side top-k caches
        self.start_window, self.end_window = START_WINDOW, END_WINDOW

    # ------------------------------------------------------------------ parameters (same names as the reference)
    def set_kpre_method_param(self, num_heads: int, num_kpre: int) -> None:
        self.k_num_heads, self.num_kpre = int(num_heads), int(num_kpre)
        self._plan = None

    def set_kpre_cache(self, kpre_cache: Sequence[torch.Tensor]) -> None:
        for t in kpre_cache:
            if not t.is_cuda or t.dtype not in (torch.bfloat16, torch.float32) or not t.is_contiguous():
                raise ValueError("kpre caches must be contiguous CUDA tensors, bf16 or fp32")
        if self.num_kpre != 1 and len(kpre_cache) and kpre_cache[0].dim() == 4 and kpre_cache[0].shape[1] == self.num_kpre:
            raise ValueError("with more than one representative per block the cache must be laid out "
                             "[slot, kv_head, rep, head_size]")
        self._kpre = list(kpre_cache)

    def set_topk_cache(self, topk_cache: Sequence[torch.Tensor], topk_lens: Sequence[int]) -> None:
        self._topk = list(topk_cache)
        self._topk_lens = [int(v) for v in topk_lens]
        self._plan = None

    def set_common_param(self, cal_topk_idx: Sequence[int], is_decode: Sequence[bool]) -> None:
        self._cal_topk_idx = [int(v) for v in cal_topk_idx]
        self._is_decode = [bool(v) for v in is_decode]
        self._plan = None

    def set_topk_param(self, repre_slot_mapping: Sequence[Sequence[int]]) -> None:
        self._need_topk = True
        self._slot_mapping = [list(m) for m in repre_slot_mapping]
        self._plan = None

    def set_kpre_param(self, calc_kpre_block_table, calc_repre_slot_mapping: Sequence[int]) -> None:
        self._calc_block_table = calc_kpre_block_table
        self._calc_slot_mapping = [int(v) for v in calc_repre_slot_mapping]

    def set_kpre_data_ready(self, layer_idx: int) -> bool:
        """The reference's calculate thread only waits for this flag (its own pooling call is commented out,
        cal_kpre_and_topk.cpp:193: the representatives are written by GSA.copy_k); here there is nothing to wait for."""
        if layer_idx == 0:
            self._need_kpre = True
        return True

    def set_topk_data_ready(self, layer_idx: int) -> None:
        """The queries of `layer_idx` are in q_cache: score and select that layer now (stream-ordered)."""
        if self._need_topk:
            self._calculate_topk(layer_idx)
        if layer_idx == self.layer_num - 1:
            self._need_topk = False                          # ResetReady (cal_kpre_and_topk.cpp:243-257)
            self._need_kpre = False

    def add_copy_req(self, need_cal_kpre: bool, layer_idx: int, locations: Sequence[int], tensor: torch.Tensor) -> None:
        """locations non-empty: `tensor` holds one query row per batch entry ([bs, q_heads, head_size], any float
        type); rows whose location is not -1 go into q_cache[layer] as fp32 (CopyData, cal_kpre_and_topk.cpp:134-160)
        and the layer's top-k is started.  locations empty: a key-cache notification - representatives are already
        in the kpre cache by then, so only the layer's readiness is noted."""
        if layer_idx == 0 and len(locations):
            self._need_kpre = bool(need_cal_kpre)
        if len(locations):
            cur = torch.cuda.current_stream(self.device)
            self._stream.wait_stream(cur)                    # the caller filled `tensor` on its stream
            rows = [i for i, loc in enumerate(locations) if loc != -1]
            with torch.cuda.stream(self._stream):
                if rows:
                    if len(rows) == len(locations):
                        self.q_cache[layer_idx][: len(rows)].copy_(tensor[: len(rows)], non_blocking=True)
                    else:
                        idx = torch.tensor(rows, dtype=torch.int64, device=self.device)
                        self.q_cache[layer_idx].index_copy_(0, idx, tensor.index_select(0, idx).to(torch.float32))
            tensor.record_stream(self._stream)
            self.set_topk_data_ready(layer_idx)
        else:
            self.set_kpre_data_ready(layer_idx)

    def is_calculate_finish(self) -> bool:
        ev = self._done[self.layer_num - 1]
        done = True if ev is None else bool(ev.query())
        if done:
            self._flush_host()
        return done

    def wait(self) -> None:
        """Block until everything enqueued so far has run (the reference has no such call; tests use it)."""
        self._stream.synchronize()
        self._flush_host()

    def _flush_host(self) -> None:
        for layer, host, p in self._pending_host:
            cache = self._topk[layer]
            h = host.numpy()
            for j, i in enumerate(p["dec"]):
                n = min(int(p["n_out"][j]), cache.shape[1])
                cache[i, :n] = torch.from_numpy(h[j, :n].copy()).to(cache.dtype)
        self._pending_host = []

    # ------------------------------------------------------------------ the calculation
    def _build_plan(self):
        """CalculateTopk's gathering of pointers (cal_kpre_and_topk.cpp:219-241) as device arrays: one ragged
        candidate list (the representative slots of every decode request), k per request, the q_cache row and the
        top-k cache row of each."""
        dec = [i for i, d in enumerate(self._is_decode) if d]
        if len(dec) != len(self._cal_topk_idx) or len(dec) != len(self._topk_lens):
            raise ValueError("set_common_param / set_topk_cache disagree on the number of decode requests")
        counts = np.asarray([len(self._slot_mapping[i]) for i in dec], np.int32)
        off = np.zeros(len(dec) + 1, np.int32)
        off[1:] = np.cumsum(counts)
        slots = (np.concatenate([np.asarray(self._slot_mapping[i], np.int32) for i in dec])
                 if len(dec) else np.zeros(0, np.int32))
        ks = np.asarray(self._topk_lens, np.int32)
        # TopKImpl writes numBlock indices when the selection degenerates to the identity (k >= n, windows >= n, k == 0)
        width = int(max(1, ks.max() if len(ks) else 1, counts.max() if len(counts) else 1))
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(self.device)  # noqa: E731
        n_out = np.asarray([int(c) if _identity(int(c), int(k), self.start_window, self.end_window) else int(k)
                            for c, k in zip(counts, ks)], np.int32)
        mask = np.arange(width)[None, :] < n_out[:, None]
        return dict(dec=dec, off=t(off), slots=t(slots), ks=t(ks), total=int(off[-1]), width=width, n_out=n_out,
                    q_rows=torch.tensor(self._cal_topk_idx, dtype=torch.int64, device=self.device),
                    dec_rows=torch.tensor(dec, dtype=torch.int64, device=self.device), mask=t(mask))

    def _calculate_topk(self, layer: int) -> None:
        if not self._kpre or not self._topk:
            raise RuntimeError("set_kpre_cache and set_topk_cache come before the first query")
        if self._plan is None:
            self._plan = self._build_plan()
        p = self._plan
        with torch.cuda.stream(self._stream):
            if p["total"] > 0:
                table = self._kpre[layer]
                n_slots = table.shape[0]
                reps = table.view(n_slots, self.k_num_heads, self.num_kpre, self.head_size)
                q = self.q_cache[layer].index_select(0, p["q_rows"])            # [n_dec, q_heads, head_size] fp32
                g = self.q_num_heads // self.k_num_heads
                # ComputeQHeadMean (select_topk_block.cpp:101-114): mean of each KV head's query heads, in fp32
                qbar = q.view(len(p["dec"]), self.k_num_heads, g, self.head_size).mean(dim=2).reshape(len(p["dec"]), -1).contiguous()
                scores = ops.score_dot(reps, p["off"], qbar, total=p["total"], slot_ids=p["slots"], n_kv_heads=self.k_num_heads,
                                       head_dim=self.head_size, n_rep=self.num_kpre)
                sel, _, cnt = ops.topk_ragged(scores, p["off"], p["ks"], out_stride=p["width"], start_win=self.start_window,
                                              end_win=self.end_window, window_mode=ops.WIN_FORCE, order=ops.ORDER_INDEX_ASC,
                                              want_scores=False)
                sel = sel.view(len(p["dec"]), p["width"])
                cache = self._topk[layer]
                width = min(p["width"], cache.shape[1])
                if cache.is_cuda:
                    # one masked write for the whole batch: entries beyond a request's result keep what they held
                    rows = cache.index_select(0, p["dec_rows"])[:, :width]
                    merged = torch.where(p["mask"][:, :width], sel[:, :width].to(cache.dtype), rows)
                    cache[:, :width].index_copy_(0, p["dec_rows"], merged)
                else:
                    # a host-side cache: the result travels through pinned memory and is written into the cache when
                    # the layer's event has fired (is_calculate_finish / wait), as the reference's flag promises
                    host = torch.empty(sel.shape, dtype=torch.int32).pin_memory()
                    host.copy_(sel, non_blocking=True)
                    self._pending_host.append((layer, host, p))
            ev = torch.cuda.Event()
            ev.record(self._stream)
            self._done[layer] = ev


def _identity(n: int, k: int, start: int, end: int) -> bool:
    return start + end >= n or k >= n or k == 0
