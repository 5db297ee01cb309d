"""HashEncoder with the interface of the reference (ucm/sparse/kvcomp/hash_encoder.py:35-219):
sign-bit hash codes packed 8 bits per uint8, LSB first.  compute_hash runs the CUDA kernel
(ucmx_hash_encode); there is no CPU path, so `device` must be a CUDA device.  The projection is
evaluated as an fp32 fused multiply-add chain over the input dimension, so results are reproducible
bit for bit across runs and batch sizes (the reference's library GEMM does not promise that).
"""
from __future__ import annotations

import torch

from . import ops


class HashEncoder:
    def __init__(self, input_dim: int, hash_bits: int, dtype: torch.dtype, device: torch.device) -> None:
        self.input_dim = input_dim
        if hash_bits % 8 != 0:
            raise ValueError("hash_bits must be a multiple of 8")
        self.hash_bits = hash_bits
        self.hash_numbers = hash_bits // 8
        self.dtype = dtype
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ValueError("HashEncoder runs on a CUDA device only")
        if dtype != torch.bfloat16:
            raise ValueError("hash weights are kept in bfloat16 (the KV cache dtype of this path)")
        self.hash_weights = torch.normal(mean=0, std=2, size=(input_dim, hash_bits), dtype=torch.float32,
                                         device=self.device).to(dtype)
        self.bit_masks = torch.pow(2, torch.arange(8, dtype=torch.uint8, device=self.device)).view(1, 1, 8)

    def set_hash_weight(self, hash_weights: torch.Tensor) -> None:
        if hash_weights.shape != (self.input_dim, self.hash_bits):
            raise ValueError(f"hash_weights shape {hash_weights.shape} does not match required shape "
                             f"{(self.input_dim, self.hash_bits)}")
        if hash_weights.dtype != self.dtype:
            raise ValueError(f"hash_weights dtype {hash_weights.dtype} does not match required dtype {self.dtype}")
        if hash_weights.device != self.device:
            raise ValueError(f"hash_weights device {hash_weights.device} does not match required device {self.device}")
        self.hash_weights.copy_(hash_weights)

    def compute_hash(self, x: torch.Tensor) -> torch.Tensor:
        """x: (..., input_dim) -> uint8 (..., hash_bits // 8)."""
        if x.shape[-1] != self.input_dim:
            raise ValueError(f"x must be of shape (..., {self.input_dim}), but got {x.shape}")
        if x.device != self.device:
            raise ValueError(f"x device {x.device} does not match required device {self.device}")
        if x.dtype != self.dtype:
            x = x.to(self.dtype)
        return ops.hash_encode(x, self.hash_weights)

    def _unpack_hash(self, packed_codes: torch.Tensor) -> torch.Tensor:
        """uint8 (..., hash_numbers) -> float16 (..., hash_bits) of +1/-1.  Kept for interface parity and
        debugging; scoring does not need it (ops.score_hamming works on the packed codes)."""
        if packed_codes.shape[-1] != self.hash_numbers:
            raise ValueError(f"packed_codes must be of shape (..., {self.hash_numbers}), but got {packed_codes.shape}")
        if packed_codes.device != self.device:
            raise ValueError(f"packed_codes device {packed_codes.device} does not match required device {self.device}")
        if packed_codes.dtype != torch.uint8:
            raise ValueError(f"packed_codes dtype {packed_codes.dtype} is not torch.uint8")
        bits = (packed_codes.unsqueeze(-1) & self.bit_masks.view(*([1] * (packed_codes.dim() - 1)), 1, 8)) > 0
        out = (bits.to(torch.float16) * 2 - 1)
        return out.reshape(*packed_codes.shape[:-1], self.hash_bits)
