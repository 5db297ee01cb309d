"""ucmx_retrieve_topk_noalloc: score + top-k for callers that may not allocate device memory
(code running inside a serving engine's forward pass, when the engine already owns nearly all of
HBM and a cudaMalloc could fail or stall the device).  The scores between the two kernels sit in
an array built into the library, so the call allocates nothing.

Checked here, through the C ABI, against the two existing entry points (ucmx_score_dot then
ucmx_topk_ragged with a caller-owned score buffer): same selected ids, same counts, same scores bit
for bit, since both routes run the same kernels - and against the CPU checker's restatement of the
reference's scoring loop and partial_sort.  Two different batches are sent one after the other
to show that what the first call left in the shared array does not leak into the second.  The
property the entry point exists for is checked as well: the device's free memory and the bytes
held by torch's allocator are the same before and after a call whose outputs already exist.
This file sorts last on purpose: a run that stops at the first failure has then already run
everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _dev(a, dtype=None):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=dtype)).to(DEV)


def _ptr(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


def _both_routes(N, reps, off, slots, q, ks, koff, n_kv_heads, head_dim):
    n_req = len(ks)
    n_slots = reps.shape[0]
    total = int(off[-1])
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    d_off, d_slots, d_q, d_k, d_koff = _dev(off), _dev(slots), _dev(q), _dev(ks), _dev(koff)
    stride = int(ks.max())
    outs = []
    for route in ("noalloc", "existing"):
        idx = torch.full((int(koff[-1]),), -7, dtype=torch.int32, device=DEV)
        sc = torch.full((int(koff[-1]),), -7.0, dtype=torch.float32, device=DEV)
        cnt = torch.full((n_req,), -7, dtype=torch.int32, device=DEV)
        if route == "noalloc":
            st = N.lib.ucmx_retrieve_topk_noalloc(_ptr(reps), N.DT_BF16, n_slots, n_kv_heads, 1, head_dim, _ptr(d_off),
                                                  _ptr(d_slots), _ptr(d_q), n_req, total, 1.0, _ptr(d_k), 0, 0,
                                                  N.WIN_NONE, N.ORDER_SCORE_DESC, _ptr(d_slots), stride, _ptr(d_koff),
                                                  _ptr(idx), _ptr(sc), _ptr(cnt), stream)
            assert st == N.OK, N.last_error()
        else:
            scores = torch.empty((total,), dtype=torch.float32, device=DEV)
            st = N.lib.ucmx_score_dot(_ptr(reps), N.DT_BF16, n_slots, n_kv_heads, 1, head_dim, _ptr(d_off), _ptr(d_slots),
                                      _ptr(d_q), n_req, total, 1.0, _ptr(scores), None, stream)
            assert st == N.OK, N.last_error()
            st = N.lib.ucmx_topk_ragged(_ptr(scores), N.DT_F32, _ptr(d_off), _ptr(d_k), n_req, 0, 0, N.WIN_NONE,
                                        N.ORDER_SCORE_DESC, _ptr(d_slots), stride, _ptr(d_koff), _ptr(idx), _ptr(sc),
                                        _ptr(cnt), stream)
            assert st == N.OK, N.last_error()
        torch.cuda.synchronize()
        outs.append((idx.cpu().numpy(), sc.cpu().numpy(), cnt.cpu().numpy()))
    return outs


def test_noalloc_matches_existing_entry_points_twice_in_a_row(oracle):
    from ucmx import _native as N
    rng = np.random.default_rng(71)
    n_slots, Hkv, D = 3000, 8, 128
    reps16 = H.randn_bf16(rng, (n_slots, Hkv * D), 0.09)
    reps = torch.from_numpy(reps16.view(np.int16)).to(DEV).view(torch.bfloat16)
    # two batches of different size and raggedness: the second is smaller, so stale scores of the
    # first call remain in the shared array beyond its end
    for counts, kfrac in (([700, 64, 1, 1200, 333], 0.1), ([90, 0, 256], 0.25)):
        off = H.ragged_offsets(counts)
        slots = rng.integers(0, n_slots, int(off[-1])).astype(np.int32)
        q = H.bf16_to_f32(H.randn_bf16(rng, (len(counts), Hkv * D)))
        ks = np.maximum(1, np.ceil(np.array(counts) * kfrac)).astype(np.int32)
        ks = np.minimum(ks, np.maximum(np.array(counts), 1)).astype(np.int32)
        koff = H.ragged_offsets(ks)
        (i1, s1, c1), (i2, s2, c2) = _both_routes(N, reps, off, slots, q, ks, koff, Hkv, D)
        assert np.array_equal(c1, c2)
        assert np.array_equal(i1, i2)
        assert np.array_equal(s1, s2)          # tolerance: none needed, the kernels are the same
        assert c1.sum() == sum(min(k, n) for k, n in zip(ks, counts))
        # and the reference's arithmetic: fp32 dot over the row, then the k best (ties to the lower position)
        ref = oracle.score_dot_esa(H.bf16_to_f32(reps16), off, slots, q)
        for r, n in enumerate(counts):
            want_ids, want_sc = oracle.topk_esa(ref[off[r]:off[r + 1]], int(ks[r]), slots[off[r]:off[r + 1]])
            got_sc = s1[koff[r]:koff[r] + c1[r]]
            np.testing.assert_allclose(got_sc, want_sc, rtol=1e-3, atol=1e-3 * float(np.abs(ref).std()))
            # identical sets unless two candidates tie at the cut within the score tolerance
            got_ids = i1[koff[r]:koff[r] + c1[r]]
            if not np.array_equal(np.sort(got_ids), np.sort(want_ids)):
                cut = want_sc[-1]
                odd = np.setxor1d(got_ids, want_ids)
                sc_of = {int(s): float(v) for s, v in zip(slots[off[r]:off[r + 1]], ref[off[r]:off[r + 1]])}
                assert all(abs(sc_of[int(o)] - cut) <= 1e-3 * abs(cut) + 1e-6 for o in odd)


def test_noalloc_allocates_no_device_memory():
    """Free device memory and torch's own allocation count do not move across a call (outputs made beforehand)."""
    from ucmx import _native as N
    rng = np.random.default_rng(72)
    n_slots, Hkv, D = 2048, 8, 128
    reps = torch.from_numpy(H.randn_bf16(rng, (n_slots, Hkv * D), 0.09).view(np.int16)).to(DEV).view(torch.bfloat16)
    counts = [900, 40, 513]
    off = H.ragged_offsets(counts)
    total = int(off[-1])
    d_off, d_slots = _dev(off), _dev(rng.integers(0, n_slots, total).astype(np.int32))
    d_q = _dev(H.bf16_to_f32(H.randn_bf16(rng, (3, Hkv * D))))
    ks = np.array([64, 8, 32], np.int32)
    d_k, d_koff = _dev(ks), _dev(H.ragged_offsets(ks))
    idx = torch.full((int(ks.sum()),), -7, dtype=torch.int32, device=DEV)
    sc = torch.zeros((int(ks.sum()),), dtype=torch.float32, device=DEV)
    cnt = torch.zeros((3,), dtype=torch.int32, device=DEV)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call():
        st = N.lib.ucmx_retrieve_topk_noalloc(_ptr(reps), N.DT_BF16, n_slots, Hkv, 1, D, _ptr(d_off), _ptr(d_slots),
                                              _ptr(d_q), 3, total, 1.0, _ptr(d_k), 0, 0, N.WIN_NONE, N.ORDER_SCORE_DESC,
                                              _ptr(d_slots), int(ks.max()), _ptr(d_koff), _ptr(idx), _ptr(sc), _ptr(cnt),
                                              stream)
        assert st == N.OK, N.last_error()

    call()                                  # the first call on a device looks up the scratch address
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    held0, reserved0 = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0
    assert torch.cuda.memory_allocated() == held0 and torch.cuda.memory_reserved() == reserved0
    assert cnt.cpu().tolist() == [64, 8, 32]


def test_noalloc_rejects_batches_beyond_its_scratch():
    from ucmx import _native as N
    limit = N.lib.ucmx_noalloc_max_candidates()
    assert limit == 1 << 20
    st = N.lib.ucmx_retrieve_topk_noalloc(None, N.DT_BF16, 0, 8, 1, 128, None, None, None, 1, limit + 1, 1.0, None, 0, 0,
                                          N.WIN_NONE, N.ORDER_SCORE_DESC, None, 1, None, None, None, None, None)
    assert st == N.EUNSUPPORTED
    assert "1048576" in N.last_error()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs a second GPU")
def test_noalloc_on_a_second_device(oracle):
    """The scratch array's address is looked up per device: a call with the second GPU current uses that GPU's copy
    and returns the checker's selection."""
    from ucmx import _native as N
    rng = np.random.default_rng(73)
    dev = "cuda:1"
    n_slots, Hkv, D = 1500, 8, 128
    reps16 = H.randn_bf16(rng, (n_slots, Hkv * D), 0.09)
    counts = [400, 31, 270]
    off = H.ragged_offsets(counts)
    total = int(off[-1])
    slots = rng.integers(0, n_slots, total).astype(np.int32)
    q = H.bf16_to_f32(H.randn_bf16(rng, (3, Hkv * D)))
    ks = np.array([40, 4, 27], np.int32)
    koff = H.ragged_offsets(ks)
    with torch.cuda.device(dev):
        to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)   # noqa: E731
        reps = to(reps16.view(np.int16)).view(torch.bfloat16)
        d_off, d_slots, d_q, d_k, d_koff = to(off), to(slots), to(q), to(ks), to(koff)
        idx = torch.full((int(ks.sum()),), -7, dtype=torch.int32, device=dev)
        sc = torch.zeros((int(ks.sum()),), dtype=torch.float32, device=dev)
        cnt = torch.zeros((3,), dtype=torch.int32, device=dev)
        stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        st = N.lib.ucmx_retrieve_topk_noalloc(_ptr(reps), N.DT_BF16, n_slots, Hkv, 1, D, _ptr(d_off), _ptr(d_slots),
                                              _ptr(d_q), 3, total, 1.0, _ptr(d_k), 0, 0, N.WIN_NONE, N.ORDER_SCORE_DESC,
                                              _ptr(d_slots), int(ks.max()), _ptr(d_koff), _ptr(idx), _ptr(sc), _ptr(cnt),
                                              stream)
        assert st == N.OK, N.last_error()
        torch.cuda.synchronize(dev)
    assert cnt.cpu().tolist() == [40, 4, 27]
    ref = oracle.score_dot_esa(H.bf16_to_f32(reps16), off, slots, q)
    got = idx.cpu().numpy()
    for r in range(3):
        want_ids, _ = oracle.topk_esa(ref[off[r]:off[r + 1]], int(ks[r]), slots[off[r]:off[r + 1]])
        assert np.array_equal(np.sort(got[koff[r]:koff[r + 1]]), np.sort(want_ids))
