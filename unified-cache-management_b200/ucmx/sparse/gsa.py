"""GSA-style retrieval (windowed top-k over mean-pooled block representatives) on the device.

The reference's GSA (ucm/sparse/gsa/gsa.py) keeps per-layer "kpre" caches of block representatives
(copy_k, :634-654), copies the decode queries out (copy_q, :616-632), scores blocks on CPU threads
with TopkBlockSelector (ucm/sparse/gsa/offload_ops/src/select_topk_block.cpp: per KV head the best
of a block's n_rep representatives against the group-mean query, summed over heads; the first
`start` and last `end` blocks forced; ascending indices out) and then swaps the attention
metadata's block table and sequence lengths for the selected blocks (attention_begin, :656-686).

Here the same three steps are kernels: pool_blocks fills the kpre table, score_dot (n_rep aware) and
topk_ragged (forced windows, ascending order, id map = the request's physical blocks) produce,
directly, the per-request row of selected PHYSICAL block ids, i.e. the rewritten block table, and
the matching sequence lengths.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import numpy as np
import torch

from .. import ops
from .base import INVALID_SLOT, UcmSparseBase, UcmSparseMetadata, UcmSparseRole

DEFAULT_BLOCK_SIZE = 128
MIN_TOPK_LEN = 32
MAX_TOPK_LEN = 48
MAX_BS = 256
LOCAL_WINDOW_SZ = MIN_TOPK_LEN - 1


def compute_topk_len(raw_seq_len: int) -> int:
    """Blocks kept for a request of raw_seq_len blocks (ucm/sparse/utils.py:30-36): 30 %, clamped to [32, 48]."""
    topk_len = int(raw_seq_len * 0.3)
    if topk_len < MIN_TOPK_LEN:
        topk_len = min(MIN_TOPK_LEN, raw_seq_len)
    elif topk_len > MAX_TOPK_LEN:
        topk_len = MAX_TOPK_LEN
    return topk_len


class GSAMetaData(UcmSparseMetadata):
    def __init__(self):
        self.req_ids: List[Any] = []
        self.block_ids: List[List[int]] = []      # physical block ids of each request, logical order
        self.seq_lens: List[int] = []
        self.query_rows: List[int] = []


class GSA(UcmSparseBase):
    def __init__(self, vllm_config: Any, role: UcmSparseRole):
        super().__init__(vllm_config, role)
        self.block_size = vllm_config.cache_config.block_size
        self.n_layers = vllm_config.model_config.hf_config.num_hidden_layers
        self.num_kv_heads = vllm_config.model_config.get_num_kv_heads(vllm_config.parallel_config)
        self.head_size = vllm_config.model_config.get_head_size()
        cfg = vllm_config.kv_transfer_config.kv_connector_extra_config.get("ucm_sparse_config", {}).get("GSA", {}) or {}
        self.n_rep = int(cfg.get("max_norm_num", 1))
        self.start_window = int(cfg.get("start_window", 1))      # TopkBlockSelector defaults (select_topk_block.h:20)
        self.end_window = int(cfg.get("end_window", 2))
        # "offload": the CPU library's weights, sum over KV heads of the max over representatives against the
        # group-mean query (select_topk_block.cpp:53-76); "device": the weights of the reference's on-GPU
        # path, mean over query heads of each head's max (gsa.py:386-412).  They rank alike with one representative.
        self.score_variant = str(cfg.get("score_variant", "offload"))
        self.kv_caches: Dict[str, torch.Tensor] = {}
        self.kpre: List[Optional[torch.Tensor]] = [None] * self.n_layers
        self.pooled: List[set] = [set() for _ in range(self.n_layers)]
        self.block_tables: List[Optional[torch.Tensor]] = [None] * self.n_layers
        self.gsa_seq_len: List[Optional[torch.Tensor]] = [None] * self.n_layers

    @staticmethod
    def layer_id_of(layer_name: str) -> int:
        return int(layer_name.split(".")[2])

    def register_kv_caches(self, kv_caches: Dict[str, torch.Tensor]):
        self.kv_caches.update(kv_caches)

    def _k(self, layer_name, forward_context) -> torch.Tensor:
        if forward_context is not None and getattr(forward_context, "no_compile_layers", None):
            return forward_context.no_compile_layers[layer_name].kv_cache[forward_context.virtual_engine][0]
        return self.kv_caches[layer_name][0]

    def _table(self, layer: int, k_cache: torch.Tensor) -> torch.Tensor:
        if self.kpre[layer] is None:
            self.kpre[layer] = torch.zeros((k_cache.shape[0], self.num_kv_heads, self.n_rep, self.head_size),
                                           dtype=torch.bfloat16, device=k_cache.device)
        return self.kpre[layer]

    def _i32(self, v, device):
        return torch.from_numpy(np.ascontiguousarray(v, dtype=np.int32)).to(device)

    def copy_k(self, layer_name: str, forward_context, block_ids: List[int]) -> None:
        """Representatives of freshly filled blocks (gsa.py:634-654); the table is indexed by physical block."""
        if not block_ids:
            return
        layer = self.layer_id_of(layer_name)
        k_cache = self._k(layer_name, forward_context)
        ids = self._i32(block_ids, k_cache.device)
        table = self._table(layer, k_cache)
        modes = ["mean"] if self.n_rep == 1 else ["mean", "max", "min"][: self.n_rep]
        for r, mode in enumerate(modes):
            ops.pool_blocks(k_cache, ids, mode=mode, out_slots=ids, out_bf16=table, n_rep=self.n_rep, rep_index=r)
        self.pooled[layer].update(block_ids)

    def cal_topk(self, layer_name: str, forward_context, query: torch.Tensor) -> None:
        """Score, select and emit this layer's block table and sequence lengths for the bound batch."""
        md: GSAMetaData = self._get_sparse_metadata()
        layer = self.layer_id_of(layer_name)
        k_cache = self._k(layer_name, forward_context)
        dev = k_cache.device
        counts = np.asarray([len(b) for b in md.block_ids], np.int32)
        ks = np.asarray([compute_topk_len(int(c)) for c in counts], np.int32)
        off = np.zeros(len(counts) + 1, np.int32)
        off[1:] = np.cumsum(counts)
        phys = np.concatenate([np.asarray(b, np.int32) for b in md.block_ids]) if len(counts) else np.zeros(0, np.int32)
        d_off, d_phys = self._i32(off, dev), self._i32(phys, dev)
        rows = torch.from_numpy(np.asarray(md.query_rows, np.int64)).to(dev)
        if self.score_variant == "device":
            scores = ops.score_dot_heads(self._table(layer, k_cache), d_off, query.index_select(0, rows).contiguous(),
                                         total=int(off[-1]), slot_ids=d_phys)
        else:
            qbar = ops.query_group_mean(query.index_select(0, rows), self.num_kv_heads, round_bf16=False)
            scores = ops.score_dot(self._table(layer, k_cache), d_off, qbar, total=int(off[-1]), slot_ids=d_phys,
                                   n_kv_heads=self.num_kv_heads, head_dim=self.head_size, n_rep=self.n_rep)
        width = int(max(1, ks.max() if len(ks) else 1, ))
        width = max(width, int(counts.max()) if len(counts) else 1) if (counts <= ks).any() else width
        table, _, cnt = ops.topk_ragged(scores, d_off, self._i32(ks, dev), out_stride=width, start_win=self.start_window,
                                        end_win=self.end_window, window_mode=ops.WIN_FORCE, order=ops.ORDER_INDEX_ASC,
                                        id_map=d_phys, want_scores=False)
        # the last selected block is the request's last block: its fill level carries over
        seq = torch.from_numpy(np.asarray(md.seq_lens, np.int64)).to(dev)
        full = torch.from_numpy(counts.astype(np.int64)).to(dev)
        tail = seq - (full - 1) * self.block_size
        self.block_tables[layer] = table
        self.gsa_seq_len[layer] = ((cnt.to(torch.int64) - 1) * self.block_size + tail).to(torch.int32)

    def attention_begin(self, query, key, value, layer_name, forward_context) -> None:
        """Swap in the selected blocks (gsa.py:656-686)."""
        layer = self.layer_id_of(layer_name)
        self.cal_topk(layer_name, forward_context, query)
        md = getattr(forward_context, "attn_metadata", None)
        if isinstance(md, dict):
            md = md[layer_name]
        if md is not None:
            md.block_table = self.block_tables[layer]
            md.seq_lens = self.gsa_seq_len[layer]

    def request_begin(self, request_id, prompt_token_ids):
        pass

    def estimate_num_slots_sparsed(self, request) -> int:
        return INVALID_SLOT
