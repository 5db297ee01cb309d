"""The store interface the sparse algorithms and the KV connector program against.

Same methods, arguments and return conventions as the reference's UcmKVStoreBase
(ucm/store/ucmstore.py:39-204): blocks are named by strings (vLLM block hashes), a transfer is
described by parallel lists (block id, byte offset inside the stored block, device tensor) and
returns a Task; wait(task) == 0 means success.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Dict, List, Tuple

import torch


class Task:
    """Handle of one asynchronous transfer."""


class UcmKVStoreBase(ABC):
    def __init__(self, config: Dict):
        self.config = config

    @abstractmethod
    def cc_store(self) -> int:
        """Address of the native store object (0 when there is none)."""

    @abstractmethod
    def create(self, block_ids: List[str]) -> List[int]:
        """Reserve space for blocks; one status per block, 0 = ok."""

    @abstractmethod
    def lookup(self, block_ids: List[str]) -> List[bool]:
        """Which of these blocks can be loaded."""

    @abstractmethod
    def prefetch(self, block_ids: List[str]) -> None:
        """Hint that these blocks will be loaded soon."""

    @abstractmethod
    def load(self, block_ids: List[str], offset: List[int], dst_tensor: List[torch.Tensor]) -> Task:
        """Start copying stored slices into device tensors."""

    @abstractmethod
    def dump(self, block_ids: List[str], offset: List[int], src_tensor: List[torch.Tensor]) -> Task:
        """Start copying device tensors into the store."""

    @abstractmethod
    def fetch_data(self, block_ids: List[str], offset: List[int], dst_addr: List[int], size: List[int]) -> Task:
        """load() on raw device addresses."""

    @abstractmethod
    def dump_data(self, block_ids: List[str], offset: List[int], src_addr: List[int], size: List[int]) -> Task:
        """dump() on raw device addresses."""

    @abstractmethod
    def wait(self, task: Task) -> int:
        """Block until the task is done; 0 = success."""

    @abstractmethod
    def commit(self, block_ids: List[str], is_success: bool = True) -> None:
        """Make dumped blocks visible (or release them when is_success is False)."""

    @abstractmethod
    def check(self, task: Task) -> Tuple[int, bool]:
        """(status, finished) without blocking."""
