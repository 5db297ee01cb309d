"""Seeded synthetic workloads with the shapes of the benchmark configurations.

No dataset is involved anywhere: keys, queries and codes are normal random tensors, context
lengths are drawn uniformly, block tables are random permutations.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass
class KvShape:
    n_q_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    block_tokens: int = 128
    n_layers: int = 32

    @property
    def row_elems(self) -> int:
        return self.n_kv_heads * self.head_dim

    @property
    def slice_bytes(self) -> int:            # one block of K (or V) of one layer, bf16
        return self.block_tokens * self.row_elems * 2


LLAMA3_8B = KvShape()
QWEN2_72B_LIKE = KvShape(n_q_heads=64, n_kv_heads=8, head_dim=128, block_tokens=128, n_layers=80)


@dataclass
class RaggedBatch:
    blocks_per_req: np.ndarray      # int32 [n_req]
    offsets: np.ndarray             # int32 [n_req+1]
    k_per_req: np.ndarray           # int32 [n_req]
    k_offsets: np.ndarray           # int32 [n_req+1], prefix sum of k_per_req
    block_table: np.ndarray         # int32 [total]: physical block of every logical block, CSR order
    n_slots: int                    # physical blocks in the pool

    @property
    def n_req(self) -> int:
        return len(self.blocks_per_req)

    @property
    def total(self) -> int:
        return int(self.offsets[-1])

    @property
    def total_k(self) -> int:
        return int(self.k_offsets[-1])

    @property
    def max_k(self) -> int:
        return int(self.k_per_req.max()) if len(self.k_per_req) else 0


def _prefix(v: np.ndarray) -> np.ndarray:
    off = np.zeros(len(v) + 1, np.int32)
    off[1:] = np.cumsum(v)
    return off


def ragged_decode_batch(seed: int = 2002, n_req: int = 64, min_ctx: int = 8192, max_ctx: int = 131072,
                        block_tokens: int = 128, ratio: float = 0.05, min_k: int = 16, table_seed=None) -> RaggedBatch:
    """Requests with context lengths uniform in [min_ctx, max_ctx], rounded up to whole blocks; a paged
    pool with exactly one slot per block and a randomly permuted block table; k = max(min_k, ceil(ratio*n)).
    table_seed: a separate seed for the block table, so that several ranks can hold batches of the same request
    lengths (the same amount of work) over different tables."""
    rng = np.random.default_rng(seed)
    ctx = rng.integers(min_ctx, max_ctx + 1, n_req)
    blocks = ((ctx + block_tokens - 1) // block_tokens).astype(np.int32)
    offsets = _prefix(blocks)
    k = np.maximum(min_k, np.ceil(ratio * blocks - 1e-9)).astype(np.int32)
    k = np.minimum(k, blocks)
    total = int(offsets[-1])
    table = (rng if table_seed is None else np.random.default_rng(table_seed)).permutation(total).astype(np.int32)
    return RaggedBatch(blocks, offsets, k, _prefix(k), table, total)


def fixed_batch(n_req: int, blocks: int, k: int, seed: int = 5005) -> RaggedBatch:
    """n_req requests of `blocks` blocks each, k selected per request (the long-context case)."""
    rng = np.random.default_rng(seed)
    b = np.full(n_req, blocks, np.int32)
    kk = np.full(n_req, k, np.int32)
    total = n_req * blocks
    return RaggedBatch(b, _prefix(b), kk, _prefix(kk), rng.permutation(total).astype(np.int32), total)
