"""Edge cases: empty and degenerate batches, sizes at the limits of each kernel's fast path, ids at the end
of large tables, many requests, and argument errors (which must come back as status codes, never as faults)."""
import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev_i32(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)


def dev_bf16(u16):
    return torch.from_numpy(np.ascontiguousarray(u16).view(np.int16)).to(DEV).view(torch.bfloat16)


def test_empty_batches_are_no_ops():
    from ucmx import ops
    z = dev_i32(np.zeros(0))
    reps = torch.zeros((4, 8, 1, 128), dtype=torch.bfloat16, device=DEV)
    off0 = dev_i32([0])
    assert ops.score_dot(reps, off0, torch.zeros((0, 1024), device=DEV), total=0, n_kv_heads=8, head_dim=128).numel() == 0
    idx, sc, cnt = ops.topk_ragged(torch.zeros(0, device=DEV), off0, z, out_stride=4)
    assert idx.shape == (0, 4) and cnt.numel() == 0
    # requests that own no candidates, and k = 0
    off = dev_i32([0, 0, 5, 5])
    s = torch.arange(5, dtype=torch.float32, device=DEV)
    idx, sc, cnt = ops.topk_ragged(s, off, dev_i32([3, 0, 2]), out_stride=3)
    assert cnt.tolist() == [0, 0, 0] or cnt.tolist() == [0, 0, 0]
    idx, sc, cnt = ops.topk_ragged(s, off, dev_i32([3, 2, 2]), out_stride=3)
    assert cnt.tolist() == [0, 2, 0] and idx[1, :2].tolist() == [4, 3]
    pool = torch.zeros((4, 4096), dtype=torch.uint8, device=DEV)
    ops.gather_blocks([pool], z, torch.zeros(16, dtype=torch.uint8, device=DEV))
    ops.scatter_blocks([pool], z, torch.zeros(16, dtype=torch.uint8, device=DEV))
    assert ops.hash_encode(torch.zeros((0, 128), dtype=torch.bfloat16, device=DEV),
                           torch.zeros((128, 128), dtype=torch.bfloat16, device=DEV)).shape == (0, 16)
    torch.cuda.synchronize()


def test_topk_large_request_and_wide_k(oracle):
    from ucmx import ops
    rng = np.random.default_rng(121)
    counts = [65536, 9000]
    off = H.ragged_offsets(counts)
    s = rng.standard_normal(int(off[-1])).astype(np.float32)
    s[100:200] = s[100]                                             # a run of ties inside the big request
    ks = np.array([8192, 4097], np.int32)
    idx, sc, cnt = ops.topk_ragged(torch.from_numpy(s).to(DEV), dev_i32(off), dev_i32(ks), out_stride=8192)
    idx, cnt = idx.cpu().numpy(), cnt.cpu().numpy()
    for r in range(2):
        want, _ = oracle.topk_esa(s[off[r]:off[r + 1]], int(ks[r]))
        assert cnt[r] == ks[r] and np.array_equal(idx[r, :cnt[r]], want)
    # ascending order has no limit on k
    idx, _, cnt = ops.topk_ragged(torch.from_numpy(s).to(DEV), dev_i32(off), dev_i32([40000, 9000]), out_stride=40000,
                                  order=ops.ORDER_INDEX_ASC, want_scores=False)
    want, _ = oracle.topk_esa(s[:65536], 40000)
    assert np.array_equal(idx[0, :40000].cpu().numpy(), np.sort(want)) and cnt.tolist() == [40000, 9000]
    from ucmx import _native as N
    st = N.lib.ucmx_topk_ragged(1, N.DT_F32, 1, 1, 1, 0, 0, 0, N.ORDER_SCORE_DESC, None, 8193, None, 1, None, 1, None)
    assert st == N.EUNSUPPORTED                                     # score-descending output is limited to k <= 8192


def test_many_requests_use_the_global_offset_path(oracle):
    from ucmx import ops
    rng = np.random.default_rng(122)
    n_req = 3000                                                    # more than the shared-memory offset table holds
    counts = rng.integers(0, 6, n_req)
    off = H.ragged_offsets(counts)
    total = int(off[-1])
    reps16 = H.randn_bf16(rng, (500, 256), 0.1)
    slots = rng.integers(0, 500, total).astype(np.int32)
    q = H.bf16_to_f32(H.randn_bf16(rng, (n_req, 256)))
    got = ops.score_dot(dev_bf16(reps16), dev_i32(off), torch.from_numpy(q).to(DEV), total=total, slot_ids=dev_i32(slots),
                        n_kv_heads=2, head_dim=128).cpu().numpy()
    ref = oracle.score_dot_esa(H.bf16_to_f32(reps16), off, slots, q)
    np.testing.assert_allclose(got, ref, rtol=1e-3, atol=1e-3 * float(ref.std()))
    q16 = H.randn_bf16(rng, (n_req, 4, 128))
    fused = ops.score_dot_query(dev_bf16(reps16), dev_i32(off), dev_bf16(q16), total=total, slot_ids=dev_i32(slots), n_kv_heads=2)
    ref2 = oracle.score_dot_esa(H.bf16_to_f32(reps16), off, slots, oracle.query_group_mean(q16, 2, True))
    np.testing.assert_allclose(fused.cpu().numpy(), ref2, rtol=1e-3, atol=1e-3 * float(ref2.std()))


def test_ids_at_the_end_of_a_large_pool(oracle):
    """Block ids near the top of a pool whose byte offsets exceed 2^32."""
    from ucmx import ops
    nb = 17000                                                      # 17000 * 262144 B = 4.46 GB > 2^32
    k = torch.zeros((nb, 128, 8, 128), dtype=torch.bfloat16, device=DEV)
    rng = np.random.default_rng(123)
    hot = np.array([nb - 1, nb - 7, 16385, 3], np.int32)
    blocks = H.randn_bf16(rng, (4, 128, 8, 128))
    k[torch.from_numpy(hot).long().to(DEV)] = dev_bf16(blocks)
    reps = ops.pool_blocks(k, dev_i32(hot))
    want = H.f32_to_bf16(oracle.pool_blocks(blocks, np.arange(4, dtype=np.int32), 0, True))
    assert np.array_equal(reps.view(torch.int16).cpu().numpy().view(np.uint16).reshape(4, -1), want)
    st = torch.zeros(4 * 262144, dtype=torch.uint8, device=DEV)
    ops.gather_blocks([k], dev_i32(hot), st)
    assert np.array_equal(st.cpu().numpy().view(np.uint16).reshape(4, -1), blocks.reshape(4, -1))
    w = H.randn_bf16(rng, (128, 128), 2.0)
    codes = ops.hash_encode_blocks(k, dev_i32(hot), dev_bf16(w), head_major=False)
    assert np.array_equal(codes.cpu().numpy(), oracle.hash_encode(blocks, w))
    del k


def test_argument_errors_are_status_codes():
    from ucmx import _native as N
    from ucmx import ops
    k = torch.zeros((4, 16, 2, 64), dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError):
        ops.pool_blocks(k.float(), dev_i32([0]))                                    # not bf16
    with pytest.raises(ValueError):
        ops.pool_blocks(k, torch.zeros(2, dtype=torch.int64, device=DEV))           # ids must be int32
    with pytest.raises(ValueError):
        ops.pool_blocks(k.cpu(), dev_i32([0]))                                      # no CPU path
    with pytest.raises(N.UcmxError) as e:
        ops.pool_blocks(k, dev_i32([0]), n_rep=2, rep_index=2)
    assert e.value.status == N.EPARAM
    pool = torch.zeros((4, 1000), dtype=torch.uint8, device=DEV)                    # slice not a multiple of 16
    with pytest.raises(N.UcmxError):
        ops.gather_blocks([pool], dev_i32([0]), torch.zeros(1000, dtype=torch.uint8, device=DEV))
    with pytest.raises(ValueError):
        ops.gather_blocks([pool[:, :992]], dev_i32([0]), torch.zeros(992, dtype=torch.uint8))   # pageable host memory
    with pytest.raises(N.UcmxError):
        ops.score_hamming(torch.zeros((2, 2, 4, 16), dtype=torch.uint8, device=DEV), dev_i32([0, 2]),
                          torch.zeros((1, 3, 16), dtype=torch.uint8, device=DEV), total=2, cross_head=False)
    # the context is still healthy
    assert ops.pool_blocks(k, dev_i32([1, 2])).shape == (2, 2, 1, 64)
    assert N.device_error() == 0


def test_topk_ties_cut_inside_a_threads_run(oracle):
    """A few distinct score values over requests far larger than the thread block: every thread owns a run of
    positions, the threshold value occurs thousands of times and only its first few positions may be taken."""
    from ucmx import ops
    rng = np.random.default_rng(123)
    counts = [7000, 1025, 4096, 33]
    off = H.ragged_offsets(counts)
    s = rng.choice(np.array([-1.5, 0.0, 0.25, 0.25, 3.0], np.float32), int(off[-1])).astype(np.float32)
    d_s = torch.from_numpy(s).to(DEV)
    for ks in ([300, 200, 2048, 7], [6999, 1, 4095, 33], [129, 1024, 257, 0]):
        k = np.asarray(ks, np.int32)
        idx, sc, cnt = ops.topk_ragged(d_s, dev_i32(off), dev_i32(k), out_stride=7000 if max(ks) > 2048 else 2048,
                                       order=ops.ORDER_INDEX_ASC)
        idx, sc, cnt = idx.cpu().numpy(), sc.cpu().numpy(), cnt.cpu().numpy()
        for r, n in enumerate(counts):
            seg = s[off[r]:off[r + 1]]
            want, _ = oracle.topk_esa(seg, int(k[r]))
            want = np.sort(want)
            assert cnt[r] == len(want) and np.array_equal(idx[r, :cnt[r]], want), (ks, r)
            assert np.array_equal(sc[r, :cnt[r]], seg[want])
        if max(ks) <= 8192:
            idx, _, cnt = ops.topk_ragged(d_s, dev_i32(off), dev_i32(k), out_stride=max(max(ks), 1), want_scores=False)
            idx, cnt = idx.cpu().numpy(), cnt.cpu().numpy()
            for r in range(len(counts)):
                want, _ = oracle.topk_esa(s[off[r]:off[r + 1]], int(k[r]))
                assert np.array_equal(idx[r, :cnt[r]], want), (ks, r, "score order")
        # forced windows on top (GSA)
        idx, _, cnt = ops.topk_ragged(d_s, dev_i32(off), dev_i32(k), out_stride=7000, start_win=3, end_win=5,
                                      window_mode=ops.WIN_FORCE, order=ops.ORDER_INDEX_ASC, want_scores=False)
        idx, cnt = idx.cpu().numpy(), cnt.cpu().numpy()
        for r in range(len(counts)):
            want = oracle.topk_gsa(s[off[r]:off[r + 1]], int(k[r]), 3, 5, cap=7000)
            assert cnt[r] == len(want) and np.array_equal(idx[r, :cnt[r]], want), (ks, r, "windows")
