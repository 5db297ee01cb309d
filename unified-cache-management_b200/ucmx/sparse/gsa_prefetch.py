"""The per-layer block tables GSA hands to attention, kept on the device.

The reference builds them on the host: GSAPrefetchBase holds `[layers, max_bs, max_blocks]` int32 tensors
(`use_block_table`, `block_table_len`, `gsa_seq_len`, the prefetch lists; ucm/sparse/gsa/prefetch/prefetch_engine.py:252-299),
GSAPrefetchEngineC walks std::maps per request and layer to find which selected blocks are resident, hands free HBM
blocks to the misses and rewrites the tables (ucm/sparse/gsa/prefetch/src/kvcache_pre.cpp:206-322), and
`model_input_del` slices the rows of the running batch out for the attention metadata (prefetch_engine.py:120-166).

Here the same tables are device tensors and one ragged launch of the resident-set remap kernel serves every
(layer, request) pair of a step: the freshly selected block positions go in, the block table rows, their lengths, the
sequence lengths and the (block to load -> HBM block) lists come out, and nothing visits the host in between.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import ops


class GSAPrefetchTables:
    def __init__(self, n_layers: int, max_bs: int, max_blocks: int, max_slots: int, block_size: int, device: torch.device):
        """max_blocks: logical blocks a request can have; max_slots: HBM blocks a request keeps per layer."""
        self.L, self.max_bs, self.max_blocks, self.max_slots = n_layers, max_bs, max_blocks, max_slots
        self.block_size, self.device = block_size, device
        i32 = dict(dtype=torch.int32, device=device)
        # the reference's tables (prefetch_engine.py:252-299), here on the device
        self.use_block_table = torch.zeros((n_layers, max_bs, max_slots), **i32)     # HBM block serving each selected position
        self.block_table_len = torch.zeros((n_layers, max_bs), **i32)
        self.gsa_seq_len = torch.zeros((n_layers, max_bs), **i32)
        self.prefetch_blocks = torch.full((n_layers, max_bs, max_slots), -1, **i32)  # HBM blocks that are being filled
        self.prefetch_logical = torch.full((n_layers, max_bs, max_slots), -1, **i32)  # with these logical blocks
        self.prefetch_block_len = torch.zeros((n_layers, max_bs), **i32)
        # resident-set state of every (layer, batch row): mBlocksMap / mDocsTables / mFreeBlock as flat arrays
        self.slot_phys = torch.zeros((n_layers, max_bs, max_slots), **i32)
        self.slot_logical = torch.full((n_layers, max_bs, max_slots), -1, **i32)
        self.slot_free = torch.ones((n_layers, max_bs, max_slots), dtype=torch.uint8, device=device)
        n = n_layers * max_bs
        self._slot_offsets = (torch.arange(n + 1, device=device, dtype=torch.int64) * max_slots).to(torch.int32)
        self._sel = torch.full((n_layers, max_bs, max_slots), -1, **i32)
        self._sel_counts = torch.full((n_layers, max_bs), -1, **i32)
        self.rows: Dict[object, int] = {}                # request id -> batch row
        self._n_slots_of_row = [0] * max_bs

    # -------------------------------------------------------------------------------- request life cycle
    def add_request(self, req_id, hbm_blocks: Sequence[int], resident: Optional[Sequence[int]] = None) -> int:
        """A request starts sparse decoding with these HBM blocks (ascending physical ids, the same in every layer).
        resident[i]: the logical block HBM block i holds already (-1: nothing, the block is free); default all free
        (add_blocks_map / set_blocks_map of the reference engine)."""
        free_rows = [b for b in range(self.max_bs) if b not in self.rows.values()]
        if not free_rows:
            raise RuntimeError("no free batch row")
        if len(hbm_blocks) > self.max_slots:
            raise ValueError("more HBM blocks than max_slots")
        row = free_rows[0]
        self.rows[req_id] = row
        ns = len(hbm_blocks)
        phys = np.full(self.max_slots, -1, np.int32)                   # a negative id: the slot does not exist
        phys[:ns] = np.sort(np.asarray(hbm_blocks, np.int32))
        order = np.argsort(np.asarray(hbm_blocks, np.int32), kind="stable")
        logical = np.full(self.max_slots, -1, np.int32)
        free = np.zeros(self.max_slots, np.uint8)
        free[:ns] = 1
        if resident is not None:
            res = np.asarray(resident, np.int32)[order]
            logical[:ns] = res
            free[:ns] = (res < 0).astype(np.uint8)
        t = lambda a: torch.from_numpy(a).to(self.device)  # noqa: E731
        self.slot_phys[:, row] = t(phys)
        self.slot_logical[:, row] = t(logical)
        self.slot_free[:, row] = t(free)
        self.block_table_len[:, row] = 0
        self._n_slots_of_row[row] = ns
        return row

    def del_request(self, req_id) -> None:
        """del_blocks_map: the row can be reused."""
        row = self.rows.pop(req_id, None)
        if row is not None:
            self.slot_logical[:, row] = -1
            self.slot_free[:, row] = 1
            self.block_table_len[:, row] = 0
            self._n_slots_of_row[row] = 0

    # -------------------------------------------------------------------------------- one prefetch round
    def run_prefetch(self, req_ids: Sequence, topk: torch.Tensor, topk_lens: Sequence[int], seq_lens: Sequence[int]):
        """run_async_prefetch_bs for the whole batch and every layer in one launch.

        topk: int32 [layers, len(req_ids), width] - the selected block positions of each request and layer, ascending
        (what CalKpreAndTopk leaves in the top-k cache); topk_lens[i] of them count; seq_lens[i]: tokens of request i.
        Afterwards use_block_table / block_table_len / gsa_seq_len / prefetch_* hold the new rows; returns the load
        lists (logical block, HBM block, count) as [layers, max_bs, max_slots] / [layers, max_bs] views."""
        rows = [self.rows[r] for r in req_ids]
        width = topk.shape[2]
        if topk.shape[0] != self.L or topk.shape[1] != len(rows) or width > self.max_slots:
            raise ValueError("topk must be [layers, requests, <= max_slots]")
        rows_t = torch.tensor(rows, dtype=torch.int64, device=self.device)
        lens = torch.tensor([int(v) for v in topk_lens], dtype=torch.int32, device=self.device)
        self._sel_counts.fill_(-1)                            # rows that are not in this batch sit the round out
        self._sel_counts[:, rows_t] = lens[None, :]
        self._sel[:, rows_t, :width] = topk.to(torch.int32)
        n = self.L * self.max_bs
        table, ll, lp, lc = ops.remap_resident(self.slot_logical.view(-1), self.slot_free.view(-1), self.slot_phys.view(-1),
                                               self._slot_offsets, self._sel.view(-1), self._slot_offsets,
                                               max_logical=self.max_blocks, max_slots=self.max_slots,
                                               sel_counts=self._sel_counts.view(-1),
                                               out=(self.use_block_table.view(-1), self.prefetch_logical.view(-1),
                                                    self.prefetch_blocks.view(-1), self.prefetch_block_len.view(-1)))
        # lengths: one block-table entry per selected position; the last selected block is the request's last block,
        # so its fill level carries over into the sparse sequence length (gsa.py:672-686)
        seq = torch.tensor([int(v) for v in seq_lens], dtype=torch.int64, device=self.device)
        self.block_table_len[:, rows_t] = lens[None, :]
        tail = seq - ((seq - 1) // self.block_size) * self.block_size
        self.gsa_seq_len[:, rows_t] = ((lens.to(torch.int64) - 1) * self.block_size + tail).to(torch.int32)[None, :]
        return self.prefetch_logical, self.prefetch_blocks, self.prefetch_block_len

    def model_input_del(self, req_ids: Sequence) -> dict:
        """What attention gets for the running batch: one block table and one sequence-length vector per layer
        (model_input_del, prefetch_engine.py:152-166: `block_tables_mp`, `gsa_seq_len`)."""
        rows_t = torch.tensor([self.rows[r] for r in req_ids], dtype=torch.int64, device=self.device)
        bt = self.use_block_table.index_select(1, rows_t)
        sl = self.gsa_seq_len.index_select(1, rows_t)
        return {"block_tables_mp": list(bt.unbind(0)), "gsa_seq_len": list(sl.unbind(0)),
                "block_table_len": list(self.block_table_len.index_select(1, rows_t).unbind(0))}
