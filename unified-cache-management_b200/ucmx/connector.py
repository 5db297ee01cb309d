"""Worker side of the KV connector: layer-wise load and dump of prefix-cache blocks through a
UcmKVStoreBase, batched per layer.

Method names, metadata classes, stored-block layout (`DataOffset`) and the results of every call
follow the reference's UnifiedCacheConnectorV1 (ucm/integration/vllm/uc_connector.py:87-522).  The
scheduler side of that class (hash matching, block bookkeeping: uc_connector.py:527-830) is control
plane and is not reproduced here.

What differs is how the transfers are described.  The reference builds one tensor view per block and
layer in Python (`get_tensor_and_offset_layerwise`, :203-227), submits one K task and one V task per
request and layer for loads (:275-293) and one task PER BLOCK and layer for dumps (:409-424).  Here a
layer's work for all requests is one address table: block addresses are `base + id * stride` computed
with numpy, K and V go in the same submission, and the store moves the whole table in one batched
transfer (`fetch_data` / `dump_data`).  The price is granularity of failure reporting: when a batched
task fails, every request (for loads) or block (for dumps) that took part in it is reported failed.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Set, Tuple

import numpy as np
import torch

from .store.factory import UcmConnectorFactory
from .store.ucmstore import Task, UcmKVStoreBase


@dataclass
class ReqMeta:
    request_id: str
    load_blocks: List[Tuple[str, int]] = field(default_factory=list)   # (block hash, vLLM block id)
    dump_blocks: List[Tuple[str, int]] = field(default_factory=list)
    load_async: bool = False


@dataclass
class UCConnectorV1Metadata:
    requests: List[ReqMeta] = field(default_factory=list)


def _extract_layer_index(layer_name: str) -> Optional[int]:
    for chunk in layer_name.split("."):
        if chunk.isdigit():
            return int(chunk)
    return None


class UnifiedCacheConnectorV1:
    """`vllm_config` is read through the same attribute paths as the reference does
    (cache_config.block_size, parallel_config.tensor_parallel_size, model_config.get_num_layers(...),
    model_config.dtype.itemsize, model_config.get_num_kv_heads(...), model_config.get_head_size(),
    model_config.is_deepseek_mla, kv_transfer_config.kv_role / kv_connector_extra_config), so either a
    vLLM config or a plain namespace with those fields works.  role: "worker" or "scheduler"."""

    def __init__(self, vllm_config: Any, role: str = "worker", rank: int = 0, store: Optional[UcmKVStoreBase] = None):
        mc, pc = vllm_config.model_config, vllm_config.parallel_config
        self.block_size = vllm_config.cache_config.block_size
        self.total_tp_size = pc.tensor_parallel_size
        self.rank = -1 if role == "scheduler" else rank
        self.is_mla = bool(getattr(mc, "is_deepseek_mla", False))
        self.num_layers = mc.get_num_layers(pc)
        self.element_size = mc.dtype.itemsize
        self.num_head = mc.get_num_kv_heads(pc)
        self.head_size = mc.get_head_size()
        ktc = vllm_config.kv_transfer_config
        self.kv_role = getattr(ktc, "kv_role", "kv_both")
        extra = dict(getattr(ktc, "kv_connector_extra_config", {}) or {})
        self.use_layerwise = bool(extra.get("use_layerwise", True))
        self.kv_caches: Dict[str, torch.Tensor] = {}
        self.dump_tasks: Dict[str, Dict[str, List[Task]]] = {}
        self.layerwise_load_tasks: Dict[str, Dict[str, Tuple[Task, Optional[Task]]]] = {}
        self._need_load_reqs: Dict[str, List[Task]] = {}
        self._load_failed_reqs: Set[str] = set()
        self._load_req_to_blocks: Dict[str, Set[int]] = {}
        self._metadata: Optional[UCConnectorV1Metadata] = None
        self.current_layer = 0
        if store is not None:
            self.connector = store
        elif "ucm_connector_name" in extra:
            config = dict(extra.get("ucm_connector_config", {}))
            config["device"] = self.rank
            config["role"] = "scheduler" if role == "scheduler" else "worker"
            base = self.block_size * self.element_size * self.head_size
            config["kv_block_size"] = base * self.num_layers * (1 if self.is_mla else self.num_head * self.total_tp_size * 2)
            config["io_size"] = base * (1 if self.is_mla else self.num_head)
            self.connector = UcmConnectorFactory.create_connector(extra["ucm_connector_name"], config)
        else:
            raise TypeError("no storage connector.")

    # ------------------------------------------------------------------ metadata plumbing
    def bind_connector_metadata(self, metadata: UCConnectorV1Metadata) -> None:
        self._metadata = metadata

    def _get_connector_metadata(self) -> UCConnectorV1Metadata:
        assert self._metadata is not None, "bind_connector_metadata was not called"
        return self._metadata

    def clear_connector_metadata(self) -> None:
        self._load_failed_reqs.clear()
        self._load_req_to_blocks.clear()
        self._metadata = None

    def register_kv_caches(self, kv_caches: Dict[str, torch.Tensor]) -> None:
        """layer name -> [2, num_blocks, block_size, num_kv_heads, head_size] (MLA: [num_blocks, block_size, head_size])."""
        self.kv_caches = dict(kv_caches)

    def _init_kv_caches_from_forward_context(self, forward_context: Any) -> None:
        for layer_name, attn_layer in forward_context.no_compile_layers.items():
            if hasattr(attn_layer, "kv_cache") and layer_name not in self.kv_caches:
                self.kv_caches[layer_name] = attn_layer.kv_cache[forward_context.virtual_engine]

    # ------------------------------------------------------------------ stored-block layout
    def DataOffset(self, kv_layer, rank, layer_id, is_v) -> int:
        """Byte offset of this rank's K (or V) slice of a layer inside a stored block (uc_connector.py:168-201)."""
        elem = kv_layer[0].element_size()
        k_sz = (kv_layer[0][0].numel() if not self.is_mla else kv_layer[0].numel()) * elem
        v_sz = (kv_layer[1][0].numel() if not self.is_mla else 0) * elem
        layer_size = (k_sz + v_sz) * (self.total_tp_size if not self.is_mla else 1)
        if is_v:
            return int(self.DataOffset(kv_layer, rank, layer_id, False) + k_sz)
        if self.is_mla:
            return int(layer_size * layer_id)
        return int(layer_size * layer_id + layer_size / self.total_tp_size * self.rank)

    def get_tensor_and_offset_layerwise(self, vllm_block_ids: List[int], kv_layer: torch.Tensor, layer_name: str):
        """The reference's per-block description (kept for callers that want tensors): K views then V views."""
        layer_id = _extract_layer_index(layer_name)
        k_off = self.DataOffset(kv_layer, self.rank, layer_id, False)
        if self.is_mla:
            return [kv_layer[b] for b in vllm_block_ids], [k_off] * len(vllm_block_ids)
        v_off = self.DataOffset(kv_layer, self.rank, layer_id, True)
        n = len(vllm_block_ids)
        return ([kv_layer[0][b] for b in vllm_block_ids] + [kv_layer[1][b] for b in vllm_block_ids], [k_off] * n + [v_off] * n)

    def _layer_table(self, storage_ids: List[str], vllm_ids: np.ndarray, kv_layer: torch.Tensor, layer_name: str):
        """One layer's transfer as flat lists: block hashes, offsets in the stored block, device addresses, sizes."""
        layer_id = _extract_layer_index(layer_name)
        k_off = self.DataOffset(kv_layer, self.rank, layer_id, False)
        if self.is_mla:
            stride = kv_layer.stride(0) * kv_layer.element_size()
            size = kv_layer[0].numel() * kv_layer.element_size()
            addrs = kv_layer.data_ptr() + vllm_ids * stride
            return list(storage_ids), [k_off] * len(storage_ids), addrs.tolist(), [size] * len(storage_ids)
        v_off = self.DataOffset(kv_layer, self.rank, layer_id, True)
        stride = kv_layer.stride(1) * kv_layer.element_size()
        size = kv_layer[0][0].numel() * kv_layer.element_size()
        k_addr = kv_layer[0].data_ptr() + vllm_ids * stride
        v_addr = kv_layer[1].data_ptr() + vllm_ids * stride
        n = len(storage_ids)
        return (list(storage_ids) * 2, [k_off] * n + [v_off] * n, np.concatenate([k_addr, v_addr]).tolist(), [size] * (2 * n))

    def _wait(self, task: Task) -> int:
        """A batched task serves several requests or blocks but may be waited on only once: the status is
        remembered on the task."""
        status = getattr(task, "_ucmx_status", None)
        if status is None:
            status = self.connector.wait(task)
            task._ucmx_status = status
        return status

    # ------------------------------------------------------------------ loads
    def start_load_kv(self, forward_context: Any = None, **kwargs) -> None:
        metadata = self._get_connector_metadata()
        if not self.kv_caches and forward_context is not None:
            self._init_kv_caches_from_forward_context(forward_context)
        self.layerwise_load_tasks.clear()
        self.current_layer = 0
        for load_async in (False, True):
            reqs = [r for r in metadata.requests if r.load_blocks and bool(r.load_async) == load_async]
            if not reqs:
                continue
            storage_ids = [b[0] for r in reqs for b in r.load_blocks]
            vllm_ids = np.asarray([b[1] for r in reqs for b in r.load_blocks], dtype=np.int64)
            for r in reqs:
                self._load_req_to_blocks.setdefault(r.request_id, set()).update(b[1] for b in r.load_blocks)
            for layer_name, kv_layer in self.kv_caches.items():
                task = self.connector.fetch_data(*self._layer_table(storage_ids, vllm_ids, kv_layer, layer_name))
                for r in reqs:
                    if load_async:
                        self._need_load_reqs.setdefault(r.request_id, []).append(task)
                    else:
                        self.layerwise_load_tasks.setdefault(r.request_id, {})[layer_name] = (task, None)
        if not self.use_layerwise:
            for request_id, layer_to_task in self.layerwise_load_tasks.items():
                if any(self._wait(t) != 0 for t, _ in layer_to_task.values()):
                    self._load_failed_reqs.add(request_id)

    def wait_for_layer_load(self, layer_name: str) -> None:
        if not self.use_layerwise:
            return
        assert self.current_layer < self.num_layers, "The current layer should be less than total layers!"
        for request_id, layer_to_task in self.layerwise_load_tasks.items():
            if request_id in self._load_failed_reqs:
                continue
            task, _ = layer_to_task[layer_name]
            if self._wait(task) != 0:
                self._load_failed_reqs.add(request_id)

    def get_finished(self, finished_req_ids: Set[str]):
        """(None, ids of requests whose asynchronous loads have ended, successfully or not)."""
        done: Set[str] = set()
        for req_id, tasks in self._need_load_reqs.items():
            if req_id in self._load_failed_reqs:
                done.add(req_id)
                continue
            unfinished = []
            for task in tasks:
                status = getattr(task, "_ucmx_status", None)
                if status is not None:
                    if status != 0:
                        self._load_failed_reqs.add(req_id)
                        break
                    continue
                ret, finish = self.connector.check(task)
                if ret != 0:
                    self._load_failed_reqs.add(req_id)
                    break
                if not finish:
                    unfinished.append(task)
                    continue
                if self._wait(task) != 0:
                    self._load_failed_reqs.add(req_id)
                    break
            if unfinished:
                self._need_load_reqs[req_id] = unfinished
                continue
            done.add(req_id)
        for req_id in done:
            self._need_load_reqs.pop(req_id, None)
        return None, done

    def get_block_ids_with_load_errors(self) -> Set[int]:
        out: Set[int] = set()
        for req_id in self._load_failed_reqs:
            out |= self._load_req_to_blocks.get(req_id, set())
        return out

    # ------------------------------------------------------------------ dumps
    def _dump_layer(self, layer_name: str, kv_layer: torch.Tensor, reqs: List[ReqMeta]) -> None:
        storage_ids = [b[0] for r in reqs for b in r.dump_blocks]
        vllm_ids = np.asarray([b[1] for r in reqs for b in r.dump_blocks], dtype=np.int64)
        task = self.connector.dump_data(*self._layer_table(storage_ids, vllm_ids, kv_layer, layer_name))
        for r in reqs:
            per_block = self.dump_tasks.setdefault(r.request_id, {})
            for block_id, _ in r.dump_blocks:
                per_block.setdefault(block_id, []).append(task)

    def save_kv_layer(self, layer_name: str, kv_layer: torch.Tensor, attn_metadata: Any = None, **kwargs) -> None:
        if self.is_mla and self.rank != 0:
            return
        self.current_layer += 1
        if self.kv_role == "kv_consumer" or not self.use_layerwise:
            return
        reqs = [r for r in self._get_connector_metadata().requests if r.dump_blocks and not r.load_async]
        if not reqs:
            return
        base = kv_layer if self.is_mla else kv_layer[0]
        if base.is_cuda:
            torch.cuda.current_stream(base.device).synchronize()     # the layer's KV must have been written
        self._dump_layer(layer_name, kv_layer, reqs)

    def wait_for_save(self) -> Optional[Dict[str, List[str]]]:
        if self.kv_role == "kv_consumer":
            return None
        if not self.use_layerwise:
            reqs = [r for r in self._get_connector_metadata().requests if r.dump_blocks]
            if reqs:
                for layer_name, kv_layer in self.kv_caches.items():
                    self._dump_layer(layer_name, kv_layer, reqs)
        success: Dict[str, List[str]] = {}
        for request_id, per_block in self.dump_tasks.items():
            for block_id, tasks in per_block.items():
                if any(self._wait(t) != 0 for t in tasks):
                    continue
                success.setdefault(request_id, []).append(block_id)
        self.dump_tasks.clear()
        return success if success else None
