"""Name -> store class registry (ucm/store/factory.py:35-70)."""
from __future__ import annotations

import importlib
from typing import Callable, Dict

from .ucmstore import UcmKVStoreBase


class UcmConnectorFactory:
    _registry: Dict[str, Callable[[], type]] = {}

    @classmethod
    def register_connector(cls, name: str, module_path: str, class_name: str) -> None:
        if name in cls._registry:
            raise ValueError(f"Connector '{name}' is already registered.")

        def loader():
            return getattr(importlib.import_module(module_path), class_name)

        cls._registry[name] = loader

    @classmethod
    def create_connector(cls, connector_name: str, config: dict) -> UcmKVStoreBase:
        if connector_name not in cls._registry:
            raise ValueError(f"Unsupported connector type: {connector_name}")
        return cls._registry[connector_name]()(config)


UcmConnectorFactory.register_connector("UcmDramStore", "ucmx.store.dramstore", "UcmDramStore")
UcmConnectorFactory.register_connector("UcmNfsStore", "ucmx.store.nfsstore", "UcmNfsStore")
