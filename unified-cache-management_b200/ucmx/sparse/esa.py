"""ESA (extract-and-select attention) behind the UcmSparseBase hooks, on the device.

Control flow, request bookkeeping and the meaning of every configuration key follow the reference
(ucm/sparse/esa/esa.py): mean-pooled block representatives are built when the last prefill chunk of
a request has run (block_repre_data, :353-364), every `retrieval_stride` decode steps the query is
scored against them (start_retrieval, :286-301), the best `sparse_ratio` of the blocks is selected,
and the blocks that are new with respect to the previous selection are loaded from the KV store
into the HBM blocks the request kept (wait_retrieval_and_start_load, :303-339).

What differs is where the work happens.  The reference keeps fp32 representatives in host memory,
moves every query to the CPU and scores it on a thread pool, one request at a time.  Here the
representatives of a layer are one bf16 table in HBM, and each hook call handles ALL requests of the
batch that need the same action with one launch: one pooling launch for every request that finished
prefill, one fused score launch and one top-k launch for every request that retrieves, one store
load (K and V) for the whole layer.  Only the selected block indices return to the host, because
the store is addressed by block hash strings there.
"""
from __future__ import annotations

import hashlib
import math
import pickle
from dataclasses import dataclass
from functools import lru_cache
from typing import Any, Dict, List, Optional, Union

import numpy as np
import torch

from .. import ops
from ..store.dramstore import store_offset
from .base import INVALID_SLOT, UcmSparseBase, UcmSparseMetadata, UcmSparseRole

ReqType = Union[str, int]


class ReprePool:
    """Slots of the representative table (ucm/sparse/esa/esa.py:34-48).  One pool serves every layer:
    a request's blocks take the same slots in each layer's table, so one slot list per request
    describes the candidates of all layers."""

    def __init__(self, num_slots: int):
        self.free_slots = list(range(num_slots - 1, -1, -1))
        self.allocated = set()

    def allocate(self, num_new_slots: int) -> List[int]:
        assert len(self.free_slots) >= num_new_slots, "Not enough free slots"
        out = [self.free_slots.pop() for _ in range(num_new_slots)]
        self.allocated.update(out)
        return out

    def free(self, slots) -> None:
        for s in slots:
            if s in self.allocated:
                self.allocated.discard(s)
                self.free_slots.append(s)


@dataclass
class ReqMeta:
    request_id: ReqType
    index_in_batch: int
    num_scheduled_tokens: int
    num_computed_tokens: int
    vllm_block_ids: List[int]
    query_start_loc: int
    prompt_token_ids: List[int]
    output_token_ids: List[int]

    @property
    def step(self) -> int:
        return len(self.output_token_ids)

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def num_output_tokens(self) -> int:
        return len(self.output_token_ids)

    @property
    def is_prefill(self) -> bool:
        return self.num_output_tokens == 0

    @property
    def is_last_chunk(self) -> bool:
        return self.num_computed_tokens + self.num_scheduled_tokens >= self.num_prompt_tokens


class ESASparseMetaData(UcmSparseMetadata):
    def __init__(self):
        self.requests: List[ReqMeta] = []
        self.finished_req_ids: List[ReqType] = []

    def add_request(self, request_id, index_in_batch, num_scheduled_tokens, num_computed_tokens, vllm_block_ids,
                    query_start_loc, prompt_token_ids, output_token_ids) -> None:
        self.requests.append(ReqMeta(request_id, index_in_batch, num_scheduled_tokens, num_computed_tokens,
                                     list(vllm_block_ids), int(query_start_loc), prompt_token_ids, output_token_ids))


@lru_cache(maxsize=None)
def md5(value) -> int:
    return int.from_bytes(hashlib.md5(pickle.dumps(value, protocol=pickle.HIGHEST_PROTOCOL)).digest(), byteorder="big")


def block_hash_func(parent_block_hash, curr_block_token_ids) -> int:
    """Chained block hash (ucm/sparse/esa/esa.py:138-150)."""
    if not parent_block_hash:
        parent_block_hash = md5("UCMHASHSEED")
    return md5((parent_block_hash, tuple(curr_block_token_ids)))


def block_hashes_of(token_ids: List[int], block_size: int) -> List[str]:
    out, parent = [], None
    for start in range(0, len(token_ids), block_size):
        chunk = token_ids[start:start + block_size]
        if len(chunk) < block_size:
            break
        parent = block_hash_func(parent, tuple(chunk))
        out.append(str(parent))
    return out


def sparse_prefill_range(num_prompt_tokens: int, block_size: int, local_window_sz: int) -> int:
    """How many leading blocks of the prompt get a representative (esa.py:341-351)."""
    if num_prompt_tokens % block_size == 0:
        return num_prompt_tokens // block_size - local_window_sz
    return math.floor(num_prompt_tokens / block_size) - (local_window_sz - 1)


class ReqState:
    """Per-request state shared by all layers, plus the per-layer selection history."""

    def __init__(self, meta: ReqMeta, block_size: int, cfg: dict, n_layers: int):
        self.meta = meta
        self.slots: List[int] = []
        self.block_hashes = block_hashes_of(meta.prompt_token_ids, block_size)
        self.sparse_range = max(sparse_prefill_range(meta.num_prompt_tokens, block_size, cfg["local_window_sz"]), 0)
        self.top_k = int(self.sparse_range * cfg["sparse_ratio"])
        self.repre_layers = set()                                   # layers whose representatives exist
        self.pre_topk: List[Dict[int, str]] = [dict() for _ in range(n_layers)]  # HBM block -> hash, per layer
        # retrieval under way per layer: (record shared by the requests launched together, this request's row in it).
        # The reference keeps a retrieval_task per request and layer (ReqStatePerLayer, ucm/sparse/esa/esa.py:157-170).
        self.pending: List[Optional[tuple]] = [None] * n_layers


class ESA(UcmSparseBase):
    def __init__(self, vllm_config: Any, role: UcmSparseRole, store=None):
        super().__init__(vllm_config, role)
        self.rank = vllm_config.parallel_config.rank
        self.tp_size = vllm_config.parallel_config.tensor_parallel_size
        self.esa_cfg = vllm_config.kv_transfer_config.kv_connector_extra_config["ucm_sparse_config"]["ESA"]
        self.block_size = vllm_config.cache_config.block_size
        self.n_layers = vllm_config.model_config.hf_config.num_hidden_layers
        self.num_kv_heads = vllm_config.model_config.get_num_kv_heads(vllm_config.parallel_config)
        self.head_size = vllm_config.model_config.get_head_size()
        self.store = store if store is not None else getattr(vllm_config, "ucm_store", None)
        self.req_states: Dict[ReqType, ReqState] = {}
        self.kv_caches: Dict[str, torch.Tensor] = {}
        if role == UcmSparseRole.WORKER:
            self.num_slots = (vllm_config.model_config.max_model_len * vllm_config.scheduler_config.max_num_seqs
                              // self.block_size)
            self.pool = ReprePool(self.num_slots)
            self.tables: List[Optional[torch.Tensor]] = [None] * self.n_layers
            self.device: Optional[torch.device] = None
            self._pinned_free: List[torch.Tensor] = []
            self._load_tasks: List[list] = [[] for _ in range(self.n_layers)]
            self._csr_cache: Optional[tuple] = None

    # ------------------------------------------------------------------ helpers
    @staticmethod
    def layer_id_of(layer_name: str) -> int:
        return int(layer_name.split(".")[2])

    def register_kv_caches(self, kv_caches: Dict[str, torch.Tensor]):
        self.kv_caches.update(kv_caches)

    def _kv(self, layer_name: str, forward_context):
        if forward_context is not None and getattr(forward_context, "no_compile_layers", None):
            attn = forward_context.no_compile_layers[layer_name]
            kv = attn.kv_cache[forward_context.virtual_engine]
        else:
            kv = self.kv_caches[layer_name]
        return kv[0], kv[1]

    def _table(self, layer: int, device: torch.device) -> torch.Tensor:
        if self.tables[layer] is None:
            self.device = device
            self.tables[layer] = torch.zeros((self.num_slots, self.num_kv_heads, 1, self.head_size),
                                             dtype=torch.bfloat16, device=device)
        return self.tables[layer]

    def _state(self, meta: ReqMeta) -> ReqState:
        st = self.req_states.get(meta.request_id)
        if st is None:
            st = ReqState(meta, self.block_size, self.esa_cfg, self.n_layers)
            self.req_states[meta.request_id] = st
        st.meta = meta
        return st

    def _i32(self, values, device) -> torch.Tensor:
        return torch.from_numpy(np.ascontiguousarray(values, dtype=np.int32)).to(device)

    # ------------------------------------------------------------------ the three actions, batched
    def _save_representatives(self, layer: int, states: List[ReqState], k_cache: torch.Tensor) -> None:
        """block_repre_data for every request that just finished prefill: one pooling launch."""
        ids, slots = [], []
        for st in states:
            if st.sparse_range <= 0:
                continue
            if not st.slots:
                st.slots = self.pool.allocate(st.sparse_range)
            ids.extend(st.meta.vllm_block_ids[:st.sparse_range])
            slots.extend(st.slots)
            st.repre_layers.add(layer)
        if ids:
            ops.pool_blocks(k_cache, self._i32(ids, k_cache.device), out_slots=self._i32(slots, k_cache.device),
                            out_bf16=self._table(layer, k_cache.device))

    def _csr(self, states: List[ReqState], device: torch.device):
        key = tuple((st.meta.request_id, len(st.slots), st.top_k, st.meta.query_start_loc) for st in states)
        if self._csr_cache is not None and self._csr_cache[0] == key:
            return self._csr_cache[1]
        counts = np.asarray([len(st.slots) for st in states], np.int32)
        ks = np.asarray([min(st.top_k, len(st.slots)) for st in states], np.int32)
        off = np.zeros(len(states) + 1, np.int32)
        off[1:] = np.cumsum(counts)
        koff = np.zeros(len(states) + 1, np.int32)
        koff[1:] = np.cumsum(ks)
        slots = np.concatenate([np.asarray(st.slots, np.int32) for st in states]) if len(states) else np.zeros(0, np.int32)
        rows = np.asarray([st.meta.query_start_loc for st in states], np.int64)
        pack = dict(off=self._i32(off, device), koff=self._i32(koff, device), ks=self._i32(ks, device),
                    slots=self._i32(slots, device), rows=torch.from_numpy(rows).to(device), total=int(off[-1]),
                    total_k=int(koff[-1]), max_k=int(ks.max()) if len(ks) else 0, koff_host=koff)
        self._csr_cache = (key, pack)
        return pack

    def _take_pinned(self, n: int) -> torch.Tensor:
        for i, t in enumerate(self._pinned_free):
            if t.numel() >= n:
                return self._pinned_free.pop(i)
        return torch.empty((max(n, 1024),), dtype=torch.int32).pin_memory()

    def _drop_pending(self, st: ReqState, layer: int) -> None:
        """Forget a request's retrieval under way; the record's host buffer is reused once nobody refers to it."""
        p = st.pending[layer]
        st.pending[layer] = None
        if p is not None:
            rec = p[0]
            rec["refs"] -= 1
            if rec["refs"] == 0:
                self._pinned_free.append(rec["host"])

    def _start_retrieval(self, layer: int, states: List[ReqState], query: torch.Tensor) -> None:
        """start_retrieval for every request that retrieves this step: one score and one top-k launch.  Each of
        these requests gets its own pending entry; entries of requests that are at another step are left alone."""
        states = [st for st in states if st.slots and st.top_k > 0 and layer in st.repre_layers]
        if not states:
            return
        dev = query.device
        c = self._csr(states, dev)
        q = query.index_select(0, c["rows"])                          # [n_req, n_q_heads, head_size], one decode token each
        scores = ops.score_dot_query(self._table(layer, dev), c["off"], q, total=c["total"], slot_ids=c["slots"],
                                     n_kv_heads=self.num_kv_heads)
        sel = torch.full((max(c["total_k"], 1),), -1, dtype=torch.int32, device=dev)
        cnt = torch.zeros((len(states),), dtype=torch.int32, device=dev)
        # positions inside the request's slot list = relative block indices (slots are allocated in block order)
        ops.topk_ragged(scores, c["off"], c["ks"], out_stride=max(c["max_k"], 1), order=ops.ORDER_SCORE_DESC,
                        out_offsets=c["koff"], out_idx=sel, out_counts=cnt, want_scores=False)
        host = self._take_pinned(sel.numel())
        host[: sel.numel()].copy_(sel, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        rec = dict(koff=c["koff_host"], host=host, event=ev, refs=len(states))
        for i, st in enumerate(states):
            self._drop_pending(st, layer)                             # a retrieval that was never collected
            st.pending[layer] = (rec, i)

    def _wait_retrieval_and_start_load(self, layer: int, states: List[ReqState], k_cache: torch.Tensor,
                                       v_cache: torch.Tensor) -> None:
        """wait_retrieval_and_start_load for the requests that are due in this layer: each one's own retrieval
        result, the delta against its previous selection (esa.py:313-334), then ONE load of K and ONE of V for
        the new blocks of all of them."""
        hashes: List[str] = []
        hbm_ids: List[int] = []
        for st in states:
            p = st.pending[layer]
            if p is None:
                continue
            rec, i = p
            rec["event"].synchronize()
            rel = rec["host"].numpy()[rec["koff"][i]: rec["koff"][i + 1]].copy()
            self._drop_pending(st, layer)
            sel_hashes = [st.block_hashes[int(j)] for j in rel]
            top_k = len(sel_hashes)
            sparse_vllm_block_ids = st.meta.vllm_block_ids[:top_k]
            pre = st.pre_topk[layer]
            if not pre:
                diff_ids, diff_hashes = list(sparse_vllm_block_ids), list(sel_hashes)
                st.pre_topk[layer] = dict(zip(sparse_vllm_block_ids, sel_hashes))
            else:
                wanted = set(sel_hashes)
                matched = {}
                for b in sparse_vllm_block_ids:
                    h = pre.get(b)
                    if h is not None and h in wanted:
                        matched[b] = h
                        wanted.discard(h)
                diff_ids = [b for b in sparse_vllm_block_ids if b not in matched]
                diff_hashes = [h for h in sel_hashes if h in wanted]
                st.pre_topk[layer] = matched
                for b, h in zip(diff_ids, diff_hashes):
                    st.pre_topk[layer][b] = h
            hashes.extend(diff_hashes)
            hbm_ids.extend(diff_ids[: len(diff_hashes)])
        if hashes and self.store is not None:
            self._launch_transfer_task("load", layer, hashes, hbm_ids, k_cache, v_cache)

    def _launch_transfer_task(self, transfer_type: str, layer: int, block_hashes: List[str], vllm_block_ids: List[int],
                              k_cache: torch.Tensor, v_cache: torch.Tensor) -> None:
        """launch_transfer_task (esa.py:222-263): K and V slices of the given HBM blocks, at the byte
        offsets of this layer and rank inside the stored block."""
        fn = getattr(self.store, transfer_type)
        shape = (self.block_size, self.num_kv_heads, self.head_size)
        precision = k_cache.element_size()
        off_k = store_offset(shape, self.rank, self.tp_size, precision, layer, False)
        off_v = store_offset(shape, self.rank, self.tp_size, precision, layer, True)
        n = len(block_hashes)
        self._load_tasks[layer].append(fn(block_hashes, [off_k] * n, [k_cache[i] for i in vllm_block_ids]))
        self._load_tasks[layer].append(fn(block_hashes, [off_v] * n, [v_cache[i] for i in vllm_block_ids]))

    def _wait_transfer_task_done(self, layer: int) -> int:
        rc = 0
        for t in self._load_tasks[layer]:
            rc |= self.store.wait(t)
        self._load_tasks[layer] = []
        return rc

    # ------------------------------------------------------------------ hooks (ucm/sparse/esa/esa.py:366-399,467-494)
    def attention_begin(self, query, key, value, layer_name, forward_context) -> None:
        layer = self.layer_id_of(layer_name)
        stride = self.esa_cfg["retrieval_stride"]
        metas = self._get_sparse_metadata().requests
        at_one = [self._state(m) for m in metas if m.step % stride == 1]
        if not at_one:
            return
        k_cache, v_cache = self._kv(layer_name, forward_context)
        first = [st for st in at_one if st.meta.step == 1]
        if first:
            self._start_retrieval(layer, first, query)
            self._wait_retrieval_and_start_load(layer, first, k_cache, v_cache)
        self._wait_transfer_task_done(layer)

    def attention_finished(self, query, key, value, attn_output, layer_name, forward_context) -> None:
        layer = self.layer_id_of(layer_name)
        stride = self.esa_cfg["retrieval_stride"]
        metas = self._get_sparse_metadata().requests
        k_cache, v_cache = self._kv(layer_name, forward_context)
        save = [self._state(m) for m in metas if m.is_prefill and m.is_last_chunk]
        if save:
            self._save_representatives(layer, save, k_cache)
        decode = [self._state(m) for m in metas if not (m.is_prefill and m.is_last_chunk) and m.step != 0]
        retrieve = [st for st in decode if st.meta.step % stride == 2]
        if retrieve:
            self._start_retrieval(layer, retrieve, query)
        due = [st for st in decode if st.meta.step % stride == 0]
        if due:
            self._wait_retrieval_and_start_load(layer, due, k_cache, v_cache)

    # ------------------------------------------------------------------ scheduler / bookkeeping
    def is_sparsed_request(self, req) -> bool:
        return len(req.prompt_token_ids) >= self.block_size * self.esa_cfg["min_blocks"]

    def build_sparse_meta(self, scheduler_output, requests, input_batch, attn_metadata) -> UcmSparseMetadata:
        sparse_meta = ESASparseMetaData()
        if isinstance(attn_metadata, dict):
            attn_metadata = next(iter(attn_metadata.values()))
        for req_id, num_scheduled_tokens in scheduler_output.num_scheduled_tokens.items():
            req = requests[req_id]
            if not self.is_sparsed_request(req):
                continue
            idx = input_batch.req_id_to_index[req_id]
            sparse_meta.add_request(req_id, idx, num_scheduled_tokens, req.num_computed_tokens, req.block_ids[0],
                                    attn_metadata.query_start_loc[idx], req.prompt_token_ids, req.output_token_ids)
        self._sparse_metadata = sparse_meta
        return sparse_meta

    def request_begin(self, request_id: ReqType, prompt_token_ids: List[int]):
        pass

    def request_finished_in_worker(self, request_id: ReqType):
        st = self.req_states.pop(request_id, None)
        if st is not None:
            for layer in range(self.n_layers):
                self._drop_pending(st, layer)
            self.pool.free(st.slots)
            self._csr_cache = None

    def estimate_num_slots_sparsed(self, request) -> int:
        if request.num_output_tokens == 0 or not self.is_sparsed_request(request):
            return INVALID_SLOT
        prompt_len, output_len, bs = request.num_prompt_tokens, request.num_output_tokens, self.block_size
        lw = self.esa_cfg["local_window_sz"]
        flaw = prompt_len % bs
        if flaw == 0:
            sparse_range = prompt_len // bs - lw
            local_window = bs * lw + output_len
        else:
            sparse_range = math.floor(prompt_len / bs) - (lw - 1)
            local_window = flaw + bs * (lw - 1) + output_len
        return int(sparse_range * self.esa_cfg["sparse_ratio"]) * bs + local_window

    def allocate_slots(self, request, num_slots_sparsed, coordinator, block_pool, kv_cache_groups):
        """Shrink the request's block list to what sparse decoding needs (esa.py:557-587)."""
        num_blocks_need = math.ceil(num_slots_sparsed / self.block_size)
        allocated = coordinator.get_blocks(request.request_id)[0]
        n_orig = len(allocated)
        kept, returned = [], []
        for i, block in enumerate(allocated):
            (kept if i >= n_orig - num_blocks_need else returned).append(block)
            block_pool._maybe_evict_cached_block(block)
        block_pool.free_blocks(returned)
        coordinator.single_type_managers[0].req_to_blocks[request.request_id] = kept
        new_computed = tuple([] for _ in range(len(kv_cache_groups)))
        need = coordinator.get_num_blocks_to_allocate(request_id=request.request_id, num_tokens=num_slots_sparsed,
                                                      new_computed_blocks=new_computed)
        if need > block_pool.get_num_free_blocks():
            return None
        coordinator.allocate_new_blocks(request.request_id, num_slots_sparsed)
        return kept
