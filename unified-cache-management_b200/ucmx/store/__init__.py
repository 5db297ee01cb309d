"""KV store interface of the reference (ucm/store) backed by the batched gather/scatter kernels."""
from .ucmstore import Task, UcmKVStoreBase  # noqa: F401
