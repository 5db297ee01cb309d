"""KVComp (hash-code retrieval) behind the UcmSparseBase hooks, on the device.

Follows the reference's flow (ucm/sparse/kvcomp/kvcomp.py): every full block a request produces is
dumped to the DRAM store and gets per-token 128-bit sign-hash codes (save_blocks, :320-347); every
RETRIEVAL_STRIDE decode steps the hashed query is scored against the codes of the middle blocks
(all but the init window and the local window), the best blocks are chosen (retrieval, :202-258)
and loaded into the HBM blocks between the two windows (attention_begin, :361-388).

The reference unpacks codes to +-1 fp16 and contracts them with an einsum per request; here the
codes of a layer live packed in one table, and scoring (XOR + popcount) and top-k run as one launch
each for all requests of the batch.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Union

import numpy as np
import torch

from .. import ops
from ..hash_encoder import HashEncoder
from ..store.dramstore import store_offset
from .base import INVALID_SLOT, UcmSparseBase, UcmSparseMetadata, UcmSparseRole
from .esa import ReprePool

ReqType = Union[str, int]

INIT_WINDOW_SZ = 1
LOCAL_WINDOW_SZ = 2
SPARSE_RATIO = 0.3
RETRIEVAL_STRIDE = 4


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

    @property
    def step(self) -> int:
        return self.num_output_tokens

    @property
    def is_prefill(self) -> bool:
        return self.num_output_tokens == 0

    @property
    def is_last_chunk(self) -> bool:
        return self.num_computed_tokens + self.num_scheduled_tokens >= self.num_prompt_tokens


class KvCompSparseMetaData(UcmSparseMetadata):
    def __init__(self):
        self.requests: List[ReqMeta] = []
        self.finished_req_ids: List[ReqType] = []

    def add_request(self, *args, **kwargs) -> None:
        self.requests.append(ReqMeta(*args, **kwargs))


def block_hash(request_id, block_id) -> str:
    return f"req_{request_id}_blk_{block_id}"


class _ReqState:
    def __init__(self, n_layers: int):
        self.slots: List[int] = []                  # code-table slots, one per dumped block (shared by layers)
        self.dumped = [0] * n_layers                # blocks hashed so far, per layer
        self.windows: List[Optional[tuple]] = [None] * n_layers


class KvComp(UcmSparseBase):
    def __init__(self, vllm_config: Any, role: UcmSparseRole, store=None):
        super().__init__(vllm_config, role)
        self.rank = vllm_config.parallel_config.rank
        self.tp_size = vllm_config.parallel_config.tensor_parallel_size
        self.block_size = vllm_config.cache_config.block_size
        self.n_layers = vllm_config.model_config.hf_config.num_hidden_layers
        self.num_kv_heads = vllm_config.model_config.get_num_kv_heads(vllm_config.parallel_config)
        self.head_size = vllm_config.model_config.get_head_size()
        extra = vllm_config.kv_transfer_config.kv_connector_extra_config
        cfg = extra.get("ucm_sparse_config", {}).get("KvComp", {}) or {}
        self.hash_bits = int(cfg.get("hash_bits", 128))
        self.init_window_sz = int(cfg.get("init_window_sz", INIT_WINDOW_SZ))
        self.local_window_sz = int(cfg.get("local_window_sz", LOCAL_WINDOW_SZ))
        self.retrieval_stride = int(cfg.get("retrieval_stride", RETRIEVAL_STRIDE))
        self.cross_head = bool(cfg.get("cross_head", True))   # the reference's einsum pairs every q head with every k head
        self.store = store if store is not None else getattr(vllm_config, "ucm_store", None)
        self.req_states: Dict[ReqType, _ReqState] = {}
        self.kv_caches: Dict[str, torch.Tensor] = {}
        self.hash_encoder: Optional[HashEncoder] = None
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

    def _encoder(self, device) -> HashEncoder:
        if self.hash_encoder is None:
            self.hash_encoder = HashEncoder(self.head_size, self.hash_bits, torch.bfloat16, device)
        return self.hash_encoder

    def _table(self, layer: int, device) -> torch.Tensor:
        if self.tables[layer] is None:
            self.tables[layer] = torch.zeros((self.num_slots, self.num_kv_heads, self.block_size, self.hash_bits // 8),
                                             dtype=torch.uint8, device=device)
        return self.tables[layer]

    def _i32(self, v, device):
        return torch.from_numpy(np.ascontiguousarray(v, dtype=np.int32)).to(device)

    def _state(self, rid) -> _ReqState:
        st = self.req_states.get(rid)
        if st is None:
            st = _ReqState(self.n_layers)
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

    # ------------------------------------------------------------------ hooks
    def attention_finished(self, query, key, value, attn_output, layer_name, forward_context) -> None:
        layer = self.layer_id_of(layer_name)
        k_cache, v_cache = self._kv(layer_name, forward_context)
        dev = k_cache.device
        ids, slots, hashes = [], [], []
        last_chunk = []
        for m in self._get_sparse_metadata().requests:
            st = self._state(m.request_id)
            full = (m.num_computed_tokens + m.num_scheduled_tokens) // self.block_size
            need = full - st.dumped[layer]
            if need > 0:
                first = st.dumped[layer]
                while len(st.slots) < first + need:
                    st.slots.extend(self.pool.allocate(1))
                src = m.vllm_block_ids[first:first + need] if m.is_prefill else m.vllm_block_ids[-1:] * need
                ids.extend(src)
                slots.extend(st.slots[first:first + need])
                hashes.extend(block_hash(m.request_id, b) for b in range(first, first + need))
                st.dumped[layer] = first + need
            if m.is_prefill and m.is_last_chunk:
                last_chunk.append((m, st))
        if ids:
            self._transfer("dump", layer, hashes, ids, k_cache, v_cache)
            ops.hash_encode_blocks(k_cache, self._i32(ids, dev), self._encoder(dev).hash_weights,
                                   out_slots=self._i32(slots, dev), head_major=True, out=self._table(layer, dev))
        for m, st in last_chunk:
            # keep copies of the init and local windows: their HBM blocks may be reused before decode starts
            b = m.vllm_block_ids
            init = (k_cache[b[: self.init_window_sz]].clone(), v_cache[b[: self.init_window_sz]].clone())
            n_local = min(self.local_window_sz, len(b[self.init_window_sz:]))
            local = (k_cache[b[-n_local:]].clone(), v_cache[b[-n_local:]].clone()) if n_local > 0 else None
            st.windows[layer] = (init, local)
        if last_chunk:
            self._wait(layer)

    def attention_begin(self, query, key, value, layer_name, forward_context) -> None:
        layer = self.layer_id_of(layer_name)
        metas = [m for m in self._get_sparse_metadata().requests if m.step % self.retrieval_stride == 1]
        if not metas:
            return
        k_cache, v_cache = self._kv(layer_name, forward_context)
        dev = k_cache.device
        self._wait(layer)
        for m in metas:
            st = self._state(m.request_id)
            if m.step == 1 and st.windows[layer] is not None:
                init, local = st.windows[layer]
                b = m.vllm_block_ids
                k_cache[b[: self.init_window_sz]] = init[0]
                v_cache[b[: self.init_window_sz]] = init[1]
                if local is not None:
                    k_cache[b[-local[0].shape[0]:]] = local[0]
                    v_cache[b[-local[0].shape[0]:]] = local[1]
        # one Hamming-score launch and one top-k launch for the whole batch
        states = [self._state(m.request_id) for m in metas]
        counts = np.asarray([st.dumped[layer] for st in states], np.int32)
        targets = [m.vllm_block_ids[self.init_window_sz: -self.local_window_sz] for m in metas]
        ks = np.asarray([len(t) for t in targets], np.int32)
        off = np.zeros(len(metas) + 1, np.int32)
        off[1:] = np.cumsum(counts)
        width = int(max(1, counts.max() if len(counts) else 1))
        slots = np.concatenate([np.asarray(st.slots[:c], np.int32) for st, c in zip(states, counts)])
        rows = torch.from_numpy(np.asarray([m.query_start_loc for m in metas], np.int64)).to(dev)
        q = query.index_select(0, rows)                                    # [n_req, n_q_heads, head_size]
        qbar = ops.query_group_mean(q, self.num_kv_heads)                  # bf16-rounded group mean, as the reference takes it
        q_codes = self._encoder(dev).compute_hash(qbar.view(len(metas), self.num_kv_heads, self.head_size).to(torch.bfloat16))
        d_off = self._i32(off, dev)
        scores = ops.score_hamming(self._table(layer, dev), d_off, q_codes, total=int(off[-1]),
                                   slot_ids=self._i32(slots, dev), cross_head=self.cross_head)
        idx, _, cnt = ops.topk_ragged(scores, d_off, self._i32(ks, dev), out_stride=width, start_win=self.init_window_sz,
                                      end_win=self.local_window_sz - 1, window_mode=ops.WIN_EXCLUDE,
                                      order=ops.ORDER_INDEX_ASC, want_scores=False)
        idx_h, cnt_h = idx.cpu().numpy(), cnt.cpu().numpy()
        hashes, hbm = [], []
        for i, m in enumerate(metas):
            chosen = idx_h[i, : cnt_h[i]]
            n = min(len(chosen), len(targets[i]))
            hashes.extend(block_hash(m.request_id, int(b)) for b in chosen[:n])
            hbm.extend(targets[i][:n])
        self._transfer("load", layer, hashes, hbm, k_cache, v_cache)
        self._wait(layer)

    # ------------------------------------------------------------------ scheduler / bookkeeping
    def request_begin(self, request_id, prompt_token_ids):
        pass

    def request_finished_in_worker(self, request_id):
        st = self.req_states.pop(request_id, None)
        if st is not None:
            self.pool.free(st.slots)

    def estimate_num_slots_sparsed(self, request) -> int:
        if request.num_output_tokens == 0:
            return INVALID_SLOT
        n_blocks = request.num_prompt_tokens // self.block_size
        if n_blocks <= self.init_window_sz + self.local_window_sz:
            return INVALID_SLOT
        mid = n_blocks - self.init_window_sz - self.local_window_sz
        keep = self.init_window_sz + int(mid * SPARSE_RATIO) + self.local_window_sz
        return keep * self.block_size + request.num_prompt_tokens % self.block_size + request.num_output_tokens
