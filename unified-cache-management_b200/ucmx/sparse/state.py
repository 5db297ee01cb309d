"""Process-wide sparse agent (ucm/sparse/state.py:20-76): one instance per process, created on first
use from the configuration, looked up by the hooks."""
from __future__ import annotations

from typing import Optional

from .base import UcmSparseBase, UcmSparseRole
from .factory import UcmSparseFactory

_UCM_SPARSE_AGENT: Optional[UcmSparseBase] = None


def ensure_ucm_sparse_initialized(vllm_config, role: UcmSparseRole = UcmSparseRole.WORKER) -> None:
    global _UCM_SPARSE_AGENT
    if vllm_config.kv_transfer_config is None:
        return
    if "ucm_sparse_config" not in vllm_config.kv_transfer_config.kv_connector_extra_config:
        return
    if _UCM_SPARSE_AGENT is None:
        _UCM_SPARSE_AGENT = UcmSparseFactory.create_sparse_method(vllm_config, role=role)


def get_ucm_sparse() -> UcmSparseBase:
    if _UCM_SPARSE_AGENT is None:
        raise RuntimeError("UCM sparse agent is not initialized")
    return _UCM_SPARSE_AGENT


def has_ucm_sparse() -> bool:
    return _UCM_SPARSE_AGENT is not None


def reset_ucm_sparse() -> None:
    """Drop the agent (tests)."""
    global _UCM_SPARSE_AGENT
    _UCM_SPARSE_AGENT = None
