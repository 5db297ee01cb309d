"""KVStar multi-step retrieval behind the UcmSparseBase hooks, on the device.

Follows the reference's flow (ucm/sparse/kvstar/multistep.py): at the end of prefill every full prompt
block is dumped to the store and gets a block representation - the channels with the largest mean
magnitude per KV head are kept, runs of `blk_repre_inner_token_merge` tokens are averaged
(extract_block_repre, :279-316) - and the queries of the last `retrieval_stride` prompt tokens form the
first query group (query_offload_info, :103-129).  During decode each step's query joins the current
group; once per stride the group votes (softmax over all positions of the request's middle blocks, summed
per block: KVStar::Execute) and the winners are loaded into the HBM blocks between the init window and
the local window (load_retrieve_result_async, :411-450).

Two things differ.  The vote runs on the GPU (ops.kvstar_scores + ops.topk_ragged, one launch each for
all requests due in the step) instead of on a CPU thread pool fed with host copies of the queries and
representations.  And because the vote then takes microseconds, its result is used in the step that
asks for it; the reference, hiding CPU latency, applies a group's result two strides later.  The channel
selection at the end of prefill is a one-off reduction left to torch, as in the reference.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Union

import numpy as np
import torch

from .. import ops
from ..store.dramstore import store_offset
from .base import INVALID_SLOT, UcmSparseBase, UcmSparseMetadata, UcmSparseRole
from .esa import ReprePool

ReqType = Union[str, int]

DEFAULTS = {"init_window_sz": 1, "local_window_sz": 2, "sparse_ratio": 0.25, "retrieval_stride": 8,
            "blk_repre_dim_prune_ratio": 0.25, "blk_repre_inner_token_merge": 2}


@dataclass
class ReqMeta:
    request_id: ReqType
    index_in_batch: int
    num_prompt_tokens: int
    num_output_tokens: int
    num_scheduled_tokens: int
    num_computed_tokens: int
    num_sparsed_tokens: int
    vllm_block_ids: List[int]
    query_start_loc: int = 0
    query_len: int = 1

    @property
    def step(self) -> int:
        return self.num_output_tokens

    @property
    def is_prefill(self) -> bool:
        return self.num_output_tokens == 0

    @property
    def is_last_chunk(self) -> bool:
        return self.num_computed_tokens + self.num_scheduled_tokens >= self.num_prompt_tokens


class KVStarMultiStepSparseMetaData(UcmSparseMetadata):
    def __init__(self):
        self.requests: List[ReqMeta] = []
        self.finished_req_ids: List[ReqType] = []

    def add_request(self, *args, **kwargs) -> None:
        self.requests.append(ReqMeta(*args, **kwargs))


def block_hash(request_id, block_id) -> str:
    return f"req_{request_id}_blk_{block_id}"


class _ReqState:
    def __init__(self, n_layers: int, stride: int):
        self.slots: List[int] = []                                   # table slots of the prompt blocks (shared by layers)
        self.n_blocks = 0                                            # full prompt blocks
        self.pruned: List[Optional[torch.Tensor]] = [None] * n_layers  # int64 [H, d_pruned] per layer
        self.group: List[List[Optional[torch.Tensor]]] = [[None] * stride for _ in range(n_layers)]
        self.windows: List[Optional[tuple]] = [None] * n_layers


class KVStarMultiStep(UcmSparseBase):
    def __init__(self, vllm_config: Any, role: UcmSparseRole, store=None):
        super().__init__(vllm_config, role)
        self.rank = vllm_config.parallel_config.rank
        self.tp_size = vllm_config.parallel_config.tensor_parallel_size
        self.block_size = vllm_config.cache_config.block_size
        self.n_layers = vllm_config.model_config.hf_config.num_hidden_layers
        self.num_kv_heads = vllm_config.model_config.get_num_kv_heads(vllm_config.parallel_config)
        self.head_size = vllm_config.model_config.get_head_size()
        extra = vllm_config.kv_transfer_config.kv_connector_extra_config
        cfg = dict(DEFAULTS)
        cfg.update(extra.get("ucm_sparse_config", {}).get("KVStarMultiStep", {}) or {})
        self.cfg = cfg
        self.init_window_sz = int(cfg["init_window_sz"])
        self.local_window_sz = int(cfg["local_window_sz"])
        self.stride = int(cfg["retrieval_stride"])
        self.merge = int(cfg["blk_repre_inner_token_merge"])
        ratio = float(cfg["blk_repre_dim_prune_ratio"])
        self.d_pruned = self.head_size if ratio >= 0.98 else round(self.head_size * ratio)
        self.store = store if store is not None else getattr(vllm_config, "ucm_store", None)
        self.req_states: Dict[ReqType, _ReqState] = {}
        self.kv_caches: Dict[str, torch.Tensor] = {}
        if role == UcmSparseRole.WORKER:
            self.num_slots = (vllm_config.model_config.max_model_len * vllm_config.scheduler_config.max_num_seqs
                              // self.block_size)
            self.pool = ReprePool(self.num_slots)
            self.tables: List[Optional[torch.Tensor]] = [None] * self.n_layers
            self._tasks: List[list] = [[] for _ in range(self.n_layers)]

    @staticmethod
    def layer_id_of(layer_name: str) -> int:
        return int(layer_name.split(".")[2])

    def register_kv_caches(self, kv_caches: Dict[str, torch.Tensor]):
        self.kv_caches.update(kv_caches)

    def _kv(self, layer_name, forward_context):
        if forward_context is not None and getattr(forward_context, "no_compile_layers", None):
            kv = forward_context.no_compile_layers[layer_name].kv_cache[forward_context.virtual_engine]
        else:
            kv = self.kv_caches[layer_name]
        return kv[0], kv[1]

    def _table(self, layer: int, device) -> torch.Tensor:
        if self.tables[layer] is None:
            self.tables[layer] = torch.zeros((self.num_slots, self.block_size // self.merge, self.num_kv_heads, self.d_pruned),
                                             dtype=torch.float16, device=device)
        return self.tables[layer]

    def _i32(self, v, device):
        return torch.from_numpy(np.ascontiguousarray(v, dtype=np.int32)).to(device)

    def _state(self, rid) -> _ReqState:
        st = self.req_states.get(rid)
        if st is None:
            st = _ReqState(self.n_layers, self.stride)
            self.req_states[rid] = st
        return st

    def _transfer(self, kind: str, layer: int, hashes: List[str], hbm_ids: List[int], k_cache, v_cache) -> None:
        if not hashes or self.store is None:
            return
        fn = getattr(self.store, kind)
        shape = (self.block_size, self.num_kv_heads, self.head_size)
        prec = k_cache.element_size()
        ok = store_offset(shape, self.rank, self.tp_size, prec, layer, False)
        ov = store_offset(shape, self.rank, self.tp_size, prec, layer, True)
        n = len(hashes)
        self._tasks[layer].append(fn(hashes, [ok] * n, [k_cache[i] for i in hbm_ids]))
        self._tasks[layer].append(fn(hashes, [ov] * n, [v_cache[i] for i in hbm_ids]))

    def _wait(self, layer: int) -> int:
        rc = 0
        for t in self._tasks[layer]:
            rc |= self.store.wait(t)
        self._tasks[layer] = []
        return rc

    def pruned_channels(self, k_blocks: torch.Tensor) -> torch.Tensor:
        """The d_pruned channels of every KV head with the largest mean magnitude over the request's prompt
        (multistep.py:284-297).  k_blocks: [n, S, h, d] of the cache's dtype."""
        n, S, h, d = k_blocks.shape
        absmean = k_blocks.reshape(n * S, h, d).to(torch.float32).abs().mean(dim=0)
        return torch.topk(absmean, k=self.d_pruned, dim=-1)[1].contiguous()

    # ------------------------------------------------------------------ hooks
    def _offload_prefill_queries(self, m: ReqMeta, st: _ReqState, layer: int, query: torch.Tensor) -> None:
        """Queries of the last `stride` prompt tokens become the first group (query_offload_info)."""
        end = m.num_computed_tokens + m.num_scheduled_tokens
        if end < m.num_prompt_tokens - self.stride:
            return
        end_in_group = self.stride - (m.num_prompt_tokens - end)
        n_valid = min(end_in_group, m.num_scheduled_tokens)
        first = end_in_group - n_valid
        rows = query[m.query_start_loc + m.query_len - n_valid: m.query_start_loc + m.query_len]
        for i in range(n_valid):
            st.group[layer][first + i] = rows[i].clone()

    def attention_begin(self, query, key, value, layer_name, forward_context) -> None:
        layer = self.layer_id_of(layer_name)
        md = self._get_sparse_metadata()
        due = []
        for m in md.requests:
            st = self._state(m.request_id)
            if m.is_prefill:
                self._offload_prefill_queries(m, st, layer, query)
                continue
            if st.n_blocks <= self.init_window_sz + self.local_window_sz or st.pruned[layer] is None:
                continue
            if m.step % self.stride == 1:
                due.append((m, st))
            else:
                st.group[layer][(m.step - 1) % self.stride] = query[m.query_start_loc].clone()
        if due:
            self._retrieve_and_load(layer, due, query, layer_name, forward_context)
        for m, st in due:                                   # the query of this step opens the next group
            st.group[layer] = [None] * self.stride
            st.group[layer][0] = query[m.query_start_loc].clone()

    def _retrieve_and_load(self, layer, due, query, layer_name, forward_context) -> None:
        k_cache, v_cache = self._kv(layer_name, forward_context)
        dev = k_cache.device
        self._wait(layer)
        groups, q_counts, counts, ks, slots, targets, pruned = [], [], [], [], [], [], []
        for m, st in due:
            if m.step == 1 and st.windows[layer] is not None:
                init, local = st.windows[layer]              # prepare_init_and_local_window
                b = m.vllm_block_ids
                k_cache[b[: self.init_window_sz]] = init[0]
                v_cache[b[: self.init_window_sz]] = init[1]
                if local is not None:
                    k_cache[b[-local[0].shape[0]:]] = local[0]
                    v_cache[b[-local[0].shape[0]:]] = local[1]
            qs = [x for x in st.group[layer] if x is not None]
            groups.extend(qs)
            q_counts.append(len(qs))
            mid = st.slots[self.init_window_sz: st.n_blocks - self.local_window_sz]
            n_keep = math.ceil(len(mid) * float(self.cfg["sparse_ratio"]))
            tgt = m.vllm_block_ids[self.init_window_sz: n_keep + self.init_window_sz]   # get_retrieve_candidate_block_ids
            counts.append(len(mid))
            ks.append(len(tgt) if qs else 0)
            slots.extend(mid)
            targets.append(tgt)
            pruned.append(st.pruned[layer])
        if not groups or not slots:
            return
        off = np.zeros(len(due) + 1, np.int32)
        off[1:] = np.cumsum(counts)
        qoff = np.zeros(len(due) + 1, np.int32)
        qoff[1:] = np.cumsum(q_counts)
        q = torch.stack(groups).to(torch.float16).contiguous()           # the reference casts the group to half as well
        pr = None if self.d_pruned == self.head_size else torch.stack(pruned).contiguous()
        d_off = self._i32(off, dev)
        votes = ops.kvstar_scores(self._table(layer, dev), d_off, q, self._i32(qoff, dev), total=int(off[-1]),
                                  max_q_tokens=self.stride, slot_ids=self._i32(slots, dev), pruned_index=pr)
        width = int(max(1, max(ks)))
        idx, _, cnt = ops.topk_ragged(votes, d_off, self._i32(ks, dev), out_stride=width, order=ops.ORDER_SCORE_DESC,
                                      want_scores=False)
        idx_h, cnt_h = idx.cpu().numpy(), cnt.cpu().numpy()
        hashes, hbm = [], []
        for i, (m, st) in enumerate(due):
            chosen = idx_h[i, : cnt_h[i]]
            n = min(len(chosen), len(targets[i]))
            hashes.extend(block_hash(m.request_id, int(b) + self.init_window_sz) for b in chosen[:n])
            hbm.extend(targets[i][:n])
        self._transfer("load", layer, hashes, hbm, k_cache, v_cache)
        self._wait(layer)

    def attention_finished(self, query, key, value, attn_output, layer_name, forward_context) -> None:
        layer = self.layer_id_of(layer_name)
        k_cache, v_cache = self._kv(layer_name, forward_context)
        dev = k_cache.device
        for m in self._get_sparse_metadata().requests:
            if not (m.is_prefill and m.is_last_chunk):
                continue
            st = self._state(m.request_id)
            n_full = m.num_prompt_tokens // self.block_size
            st.n_blocks = n_full
            if n_full == 0:
                continue
            while len(st.slots) < n_full:
                st.slots.extend(self.pool.allocate(1))
            b = m.vllm_block_ids[:n_full]
            self._transfer("dump", layer, [block_hash(m.request_id, i) for i in range(n_full)], b, k_cache, v_cache)
            ids = self._i32(b, dev)
            st.pruned[layer] = None if self.d_pruned == self.head_size else self.pruned_channels(k_cache[ids.long()])
            ops.kvstar_block_repre(k_cache, ids, merge=self.merge, pruned_index=st.pruned[layer],
                                   out_slots=self._i32(st.slots[:n_full], dev), out=self._table(layer, dev))
            if self.d_pruned == self.head_size:
                st.pruned[layer] = torch.arange(self.head_size, device=dev).repeat(self.num_kv_heads, 1)   # marks "ready"
            # keep copies of the init and local windows (and of a trailing partial block): their HBM blocks may be
            # reused before decode starts
            b_all = m.vllm_block_ids[: math.ceil(m.num_prompt_tokens / self.block_size)]
            n_tail = min(self.local_window_sz + (len(b_all) - n_full), len(b_all) - min(self.init_window_sz, len(b_all)))
            init = (k_cache[b_all[: self.init_window_sz]].clone(), v_cache[b_all[: self.init_window_sz]].clone())
            local = (k_cache[b_all[-n_tail:]].clone(), v_cache[b_all[-n_tail:]].clone()) if n_tail > 0 else None
            st.windows[layer] = (init, local)
            self._wait(layer)

    # ------------------------------------------------------------------ scheduler / bookkeeping
    def request_begin(self, request_id, prompt_token_ids):
        pass

    def request_finished_in_worker(self, request_id):
        st = self.req_states.pop(request_id, None)
        if st is not None:
            self.pool.free(st.slots)

    def estimate_num_slots_sparsed(self, request) -> int:
        """Slots a decode step needs once the middle of the prompt is sparsified (multistep.py:775-814)."""
        if request.num_output_tokens == 0:
            return INVALID_SLOT
        bs = self.block_size
        n_full = request.num_prompt_tokens // bs
        fixed = min(self.init_window_sz + self.local_window_sz, n_full)
        saved = math.ceil((n_full - fixed) * float(self.cfg["sparse_ratio"]))
        dense_total = math.ceil(request.num_tokens / bs)
        budget = dense_total - (n_full - saved - fixed)
        tail = request.num_tokens % bs
        return (budget - 1) * bs + tail if tail else budget * bs
