"""The tensor-core (tcgen05) sign-hash encoder against the CPU checker and against the CUDA-core
kernel: bit-exact, including vectors built so that projections cancel to (nearly) zero, where the
sign is decided by the exact fused-multiply-add chain rather than by the tensor core."""
import os

import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev_bf16(u16):
    return torch.from_numpy(np.ascontiguousarray(u16).view(np.int16)).to(DEV).view(torch.bfloat16)


def test_paged_llama_shape_bit_exact(oracle):
    from ucmx import ops
    rng = np.random.default_rng(101)
    w = H.randn_bf16(rng, (128, 128), 2.0)
    k = H.randn_bf16(rng, (9, 128, 8, 128))
    ids = np.array([8, 0, 3, 3, 5, 7], np.int32)
    want = oracle.hash_encode(k[ids], w)                                   # [6, 128, 8, 16]
    got = ops.hash_encode_blocks(dev_bf16(k), torch.from_numpy(ids).to(DEV), dev_bf16(w), head_major=False)
    assert np.array_equal(got.cpu().numpy(), want)
    slots = np.array([4, 2, 0, 1, 5, 3], np.int32)
    out = torch.zeros((6, 8, 128, 16), dtype=torch.uint8, device=DEV)
    ops.hash_encode_blocks(dev_bf16(k), torch.from_numpy(ids).to(DEV), dev_bf16(w), out_slots=torch.from_numpy(slots).to(DEV), out=out)
    assert np.array_equal(out.cpu().numpy()[slots], want.transpose(0, 2, 1, 3))
    from ucmx import _native
    assert _native.device_error() == 0


def test_cancelling_projections_take_the_exact_path(oracle):
    from ucmx import ops
    rng = np.random.default_rng(102)
    n = 4096
    x = H.bf16_to_f32(H.randn_bf16(rng, (n, 128)))
    w = H.bf16_to_f32(H.randn_bf16(rng, (128, 128), 2.0))
    # second half of every vector mirrors the first with opposite sign, and for half of the columns the
    # weights repeat, so those projections cancel exactly in exact arithmetic
    x[:, 64:] = -x[:, :64]
    w[64:, ::2] = w[:64, ::2]
    # a few rows with a tiny leftover so that the true sum is a small non-zero number
    x[::7, 127] = H.bf16_to_f32(H.f32_to_bf16(x[::7, 127] * 1.0078125))
    x16, w16 = H.f32_to_bf16(x), H.f32_to_bf16(w)
    want = oracle.hash_encode(x16, w16)
    got = ops.hash_encode(dev_bf16(x16), dev_bf16(w16)).cpu().numpy()
    assert np.array_equal(got, want)
    margins = oracle.hash_project(x16[:64], w16)
    assert np.abs(margins[:, ::2]).max() < 0.25 < np.abs(margins[:, 1::2]).std()   # cancelling columns sit at rounding-noise level


def test_large_batch_matches_the_checker(oracle):
    """A batch large enough to keep every SM busy for many tiles, a size that is no multiple of the tile, against
    the CPU checker's FMA chain bit for bit."""
    from ucmx import ops
    rng = np.random.default_rng(103)
    x16 = H.randn_bf16(rng, (200_003, 128))
    w16 = H.randn_bf16(rng, (128, 128), 2.0)
    got = ops.hash_encode(dev_bf16(x16), dev_bf16(w16)).cpu().numpy()
    assert np.array_equal(got, oracle.hash_encode(x16, w16))
    assert 0.45 < float(np.unpackbits(got[:10000]).mean()) < 0.55


def test_zero_and_tiny_vectors(oracle):
    """Rows of zeros (every projection is exactly zero: all bits 0; they take no exact chain at all) and rows whose
    squares underflow (every bit of them goes through the exact chain)."""
    from ucmx import ops
    rng = np.random.default_rng(104)
    n = 128 * 20
    x = H.bf16_to_f32(H.randn_bf16(rng, (n, 128)))
    x[5:300] = 0.0
    x[300:420] *= 1e-24
    x[420:500] *= 1e-36
    x[1000, :64] = 0.0
    w16 = H.randn_bf16(rng, (128, 128), 2.0)
    x16 = H.f32_to_bf16(x)
    want = oracle.hash_encode(x16, w16)
    got = ops.hash_encode(dev_bf16(x16), dev_bf16(w16)).cpu().numpy()
    assert np.array_equal(got, want)
    assert not want[5:300].any()


def test_repeated_runs_are_identical(oracle):
    """The code words settled by the fixer warp and those stored by the epilogue never overlap: a dozen runs of a
    batch large enough to keep every SM busy give the same bytes, and those are the checker's."""
    from ucmx import ops
    rng = np.random.default_rng(105)
    x16 = H.randn_bf16(rng, (150_000, 128))
    w16 = H.randn_bf16(rng, (128, 128), 2.0)
    x, w = dev_bf16(x16), dev_bf16(w16)
    ref = torch.from_numpy(oracle.hash_encode(x16, w16)).to(DEV)
    for rep in range(12):
        got = ops.hash_encode(x, w)
        bad = (got.view(torch.int32) != ref.view(torch.int32)).nonzero()
        assert bad.numel() == 0, f"run {rep}: {bad.shape[0]} words differ, first (row, word): {bad[:8].tolist()}"


def test_every_bit_doubtful_on_every_sm(oracle):
    """Every bit of every vector is doubtful (squares underflow, so no tensor-core sign is trusted) and every thread
    block gets many tiles: the fixer warps' queue (128 words a tile) overflows in each of them, so most words are
    settled by the epilogue warps' pooled fallback.  Same bytes as the checker either way."""
    from ucmx import ops
    rng = np.random.default_rng(106)
    n = 148 * 8 * 128
    x = H.bf16_to_f32(H.randn_bf16(rng, (n, 128))) * 1e-24
    x16, w16 = H.f32_to_bf16(x), H.randn_bf16(rng, (128, 128), 2.0)
    got = ops.hash_encode(dev_bf16(x16), dev_bf16(w16)).cpu().numpy()
    assert np.array_equal(got, oracle.hash_encode(x16, w16))
    from ucmx import _native
    assert _native.device_error() == 0


def test_two_and_a_half_million_vectors(oracle):
    """2.5 million vectors (19 532 tiles, 66 per thread block).  The input is a 100 000-vector batch repeated 25 times,
    so the checker runs once."""
    from ucmx import ops
    rng = np.random.default_rng(107)
    base16 = H.randn_bf16(rng, (100_000, 128))
    w16 = H.randn_bf16(rng, (128, 128), 2.0)
    x = dev_bf16(base16).repeat(25, 1).contiguous()
    got = ops.hash_encode(x, dev_bf16(w16)).view(25, 100_000, 16)
    want = torch.from_numpy(oracle.hash_encode(base16, w16)).to(DEV)
    assert bool((got == want.unsqueeze(0)).all())


def test_outlier_channels_and_unwritten_blocks(oracle):
    """Keys whose channels differ in scale by orders of magnitude (the margin test is relative to the row norm, so the
    small channels' contributions sit far below it), in a paged cache half of whose blocks were never written."""
    from ucmx import ops
    rng = np.random.default_rng(108)
    scale = np.exp(rng.standard_normal(128) * 1.5).astype(np.float32)
    k = H.bf16_to_f32(H.randn_bf16(rng, (24, 128, 8, 128))) * scale
    k[12:] = 0.0
    k[3, 64:] = 0.0
    k16, w16 = H.f32_to_bf16(k), H.randn_bf16(rng, (128, 128), 2.0)
    ids = rng.permutation(24).astype(np.int32)
    got = ops.hash_encode_blocks(dev_bf16(k16), torch.from_numpy(ids).to(DEV), dev_bf16(w16), head_major=False).cpu().numpy()
    want = oracle.hash_encode(k16[ids], w16)
    assert np.array_equal(got, want)
    assert not want[ids >= 12].any()
