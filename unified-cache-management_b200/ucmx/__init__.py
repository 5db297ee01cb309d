"""ucmx — B200 (sm_100a) implementation of UCM's sparse-KV retrieval and block-transfer hot path.

Layers, bottom up:
  _native   ctypes binding of libucmx.so (the C ABI in include/ucmx.h); raises if it is not built
  ops       tensor-level calls: pool_blocks, hash_encode, score_dot, score_hamming, topk_ragged,
            gather_blocks / scatter_blocks
  retrieval RetrievalWorkerBackend / RetrievalWorker, the ESA native back-end's interface
  hash_encoder  HashEncoder, KVComp's encoder interface
  sparse    UcmSparseBase hooks, factory and the ESA / KvComp / GSA-style retrievers
  store     UcmKVStoreBase, tasks, pinned ring and the DRAM store built on gather/scatter
"""
from . import _native  # noqa: F401  (fails loudly when the CUDA library is missing)
from . import ops  # noqa: F401

__all__ = ["ops"]
__version__ = "0.1.0"
