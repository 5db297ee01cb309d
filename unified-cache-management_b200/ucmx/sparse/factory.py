"""Lazy name -> class registry of sparse methods (ucm/sparse/factory.py:12-52)."""
from __future__ import annotations

import importlib
from typing import Callable, Dict

from .base import UcmSparseBase, UcmSparseRole


class UcmSparseFactory:
    _registry: Dict[str, Callable[[], type]] = {}

    @classmethod
    def register_sparse_method(cls, name: str, module_path: str, class_name: str) -> None:
        if name in cls._registry:
            raise ValueError(f"Sparse attention method '{name}' is already registered.")

        def loader():
            return getattr(importlib.import_module(module_path), class_name)

        cls._registry[name] = loader

    @classmethod
    def create_sparse_method(cls, config, role: UcmSparseRole) -> UcmSparseBase:
        ucm_cfg = config.kv_transfer_config.kv_connector_extra_config.get("ucm_sparse_config")
        name, _ = next(iter(ucm_cfg.items()))
        if name not in cls._registry:
            raise ValueError(f"Unsupported sparse method type: {name}")
        klass = cls._registry[name]()
        assert issubclass(klass, UcmSparseBase)
        return klass(config, role)


UcmSparseFactory.register_sparse_method("ESA", "ucmx.sparse.esa", "ESA")
UcmSparseFactory.register_sparse_method("KvComp", "ucmx.sparse.kvcomp", "KvComp")
UcmSparseFactory.register_sparse_method("GSA", "ucmx.sparse.gsa", "GSA")
UcmSparseFactory.register_sparse_method("KVStarMultiStep", "ucmx.sparse.kvstar", "KVStarMultiStep")
