"""Exchange of partial block scores through peer-mapped memory: delivered by the scoring kernel, summed
inside the top-k kernel.

On one GPU several "ranks" are emulated in ONE process: each gets its own buffer on the device,
all ranks score (which also raises their flags) first and only then do the top-k kernels run, so no
kernel ever waits for another one that is not yet complete.  With two or more GPUs the real thing runs in
child processes over symmetric memory and is compared with the NCCL all-reduce route."""
import os
import sys

import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def dev_i32(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)


def dev_bf16(u16):
    return torch.from_numpy(np.ascontiguousarray(u16).view(np.int16)).to(DEV).view(torch.bfloat16)


@pytest.mark.parametrize("world", [4, 8])        # two heads per rank: 512-byte rows; one head: the narrow-row kernel
def test_emulated_ranks_on_one_gpu(oracle, world):
    from ucmx import _native, ops
    from ucmx.parallel import PeerScoreExchange, head_range
    rng = np.random.default_rng(111)
    Hkv, D, n_slots = 8, 128, 700
    reps16 = H.randn_bf16(rng, (n_slots, Hkv, D), 0.09)
    counts = [300, 0, 91, 256]
    off = H.ragged_offsets(counts)
    total = int(off[-1])
    slots = rng.integers(0, n_slots, total).astype(np.int32)
    q = H.bf16_to_f32(H.randn_bf16(rng, (len(counts), Hkv, D)))
    ks = np.array([30, 3, 9, 25], np.int32)
    koff = H.ragged_offsets(np.minimum(ks, counts))
    bufs = [torch.zeros(PeerScoreExchange.words_needed(world, total), dtype=torch.float32, device=DEV) for _ in range(world)]
    ex = [PeerScoreExchange([b.data_ptr() for b in bufs], r, total, torch.device(DEV), bufs[r]) for r in range(world)]
    d_off, d_slots, d_k, d_koff = dev_i32(off), dev_i32(slots), dev_i32(ks), dev_i32(koff)
    full = oracle.score_dot_esa(H.bf16_to_f32(reps16).reshape(n_slots, -1), off, slots, q.reshape(len(counts), -1))
    for rnd in range(3):                                                  # three rounds: both halves, growing round numbers
        scale = float(rnd + 1)
        for r in range(world):
            lo, hi = head_range(Hkv, r, world)
            table = dev_bf16(np.ascontiguousarray(reps16[:, lo:hi]))
            qr = torch.from_numpy(np.ascontiguousarray(q[:, lo:hi].reshape(len(counts), -1))).to(DEV)
            ops.score_dot(table, d_off, qr, total=total, slot_ids=d_slots, n_kv_heads=hi - lo, head_dim=D, scale=scale,
                          exchange=ex[r])
        sels = []
        for r in range(world):
            idx = torch.full((int(koff[-1]),), -1, dtype=torch.int32, device=DEV)
            cnt = torch.zeros((len(counts),), dtype=torch.int32, device=DEV)
            ex[r].topk(d_off, d_k, total=total, out_stride=int(ks.max()), order=ops.ORDER_SCORE_DESC, out_idx=idx,
                       out_counts=cnt, id_map=d_slots, out_offsets=d_koff)
            sels.append((idx.cpu().numpy(), cnt.cpu().numpy(), ex[r].summed.cpu().numpy()))
        for r in range(1, world):                                          # every rank: identical bits
            assert np.array_equal(sels[r][0], sels[0][0]) and np.array_equal(sels[r][2], sels[0][2])
        np.testing.assert_allclose(sels[0][2], scale * full, rtol=1e-3, atol=1e-3 * scale * float(np.abs(full).std()))
        for i in range(len(counts)):
            want, _ = oracle.topk_esa(sels[0][2][off[i]:off[i + 1]], int(ks[i]), slots[off[i]:off[i + 1]])
            assert np.array_equal(sels[0][0][koff[i]:koff[i + 1]], want)
    assert _native.device_error() == 0


def test_wide_rows_and_replay_from_a_cuda_graph(oracle):
    """Two emulated ranks with 2 KiB rows each (the copy-engine scoring kernel with the raw query folded in); the
    round counter lives in the exchange buffer, so score + top-k of both ranks is captured once and replayed."""
    from ucmx import _native, ops
    from ucmx.parallel import PeerScoreExchange, head_range
    rng = np.random.default_rng(112)
    world, Hkv, Hq, D, n_slots = 2, 16, 32, 128, 900
    reps16 = H.randn_bf16(rng, (n_slots, Hkv, D), 0.09)
    counts = [500, 37, 240]
    off = H.ragged_offsets(counts)
    total = int(off[-1])
    slots = rng.integers(0, n_slots, total).astype(np.int32)
    q16 = H.randn_bf16(rng, (len(counts), Hq, D))
    ks = np.array([40, 5, 12], np.int32)
    koff = H.ragged_offsets(ks)
    dev = torch.device(DEV)
    bufs = [torch.zeros(PeerScoreExchange.words_needed(world, total), dtype=torch.float32, device=DEV) for _ in range(world)]
    ex = [PeerScoreExchange([b.data_ptr() for b in bufs], r, total, dev, bufs[r]) for r in range(world)]
    d_off, d_slots, d_k, d_koff = dev_i32(off), dev_i32(slots), dev_i32(ks), dev_i32(koff)
    tables, queries = [], []
    for r in range(world):
        lo, hi = head_range(Hkv, r, world)
        tables.append(dev_bf16(np.ascontiguousarray(reps16[:, lo:hi])))
        queries.append(dev_bf16(np.ascontiguousarray(q16[:, lo * 2:hi * 2])))      # two query heads per KV head
    idx = [torch.full((int(koff[-1]),), -1, dtype=torch.int32, device=DEV) for _ in range(world)]
    cnt = [torch.zeros((len(counts),), dtype=torch.int32, device=DEV) for _ in range(world)]

    def one_round():
        for r in range(world):
            ops.score_dot_query(tables[r], d_off, queries[r], total=total, slot_ids=d_slots, n_kv_heads=Hkv // world,
                                exchange=ex[r])
        for r in range(world):
            ex[r].topk(d_off, d_k, total=total, out_stride=int(ks.max()), order=ops.ORDER_SCORE_DESC, out_idx=idx[r],
                       out_counts=cnt[r], id_map=d_slots, out_offsets=d_koff)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        one_round()                                             # sets up lazily initialised state outside the capture
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    qbar = oracle.query_group_mean(q16, Hkv, True)
    full = oracle.score_dot_esa(H.bf16_to_f32(reps16).reshape(n_slots, -1), off, slots, qbar)
    want = np.concatenate([oracle.topk_esa(full[off[i]:off[i + 1]], int(ks[i]), slots[off[i]:off[i + 1]])[0]
                           for i in range(len(counts))])
    first = idx[0].cpu().numpy().copy()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        one_round()
    for _ in range(3):                                          # odd and even rounds: both halves of the inbox
        for t in idx:
            t.fill_(-1)
        graph.replay()
        torch.cuda.synchronize()
        for r in range(world):
            assert np.array_equal(idx[r].cpu().numpy(), first)
    np.testing.assert_allclose(ex[0].summed.cpu().numpy(), full, rtol=1e-3, atol=1e-3 * float(np.abs(full).std()))
    # the sums differ from the checker's by rounding only; where that does not reorder anything the ids agree
    assert (np.sort(first) == np.sort(want)).mean() > 0.97
    assert _native.device_error() == 0


def test_missing_signal_is_reported_not_hung():
    """A peer that never delivers: the bounded wait gives up, records code 4 and the kernel returns."""
    from ucmx import _native, ops
    from ucmx.parallel import PeerScoreExchange
    total = 64
    dev = torch.device(DEV)
    bufs = [torch.zeros(PeerScoreExchange.words_needed(2, total), dtype=torch.float32, device=DEV) for _ in range(2)]
    ex0 = PeerScoreExchange([b.data_ptr() for b in bufs], 0, total, dev, bufs[0])
    table = torch.ones((total, 1, 1, 128), dtype=torch.bfloat16, device=DEV)
    q = torch.ones((1, 128), dtype=torch.float32, device=DEV)
    ops.score_dot(table, dev_i32([0, total]), q, total=total, n_kv_heads=1, head_dim=128, exchange=ex0)   # rank 1 stays silent
    idx = torch.full((4,), -1, dtype=torch.int32, device=DEV)
    cnt = torch.zeros((1,), dtype=torch.int32, device=DEV)
    _native.device_error()
    ex0.topk(dev_i32([0, total]), dev_i32([4]), total=total, out_stride=4, order=ops.ORDER_SCORE_DESC, out_idx=idx,
             out_counts=cnt)
    torch.cuda.synchronize()
    assert _native.device_error() == 4
    assert cnt.item() == 4                                     # the context is intact and the kernel completed


def _two_gpu_worker(rank, world, port, out_dir):
    for p in (ROOT, os.path.join(ROOT, "unified-cache-management_b200"), HERE):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    dev = torch.device(f"cuda:{rank}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from ucmx import ops
    from ucmx.parallel import PeerScoreExchange, ScoreAllReduce, head_range
    rng = np.random.default_rng(5005)
    Hkv, D, n_slots = 8, 128, 2000
    reps16 = H.randn_bf16(rng, (n_slots, Hkv, D), 0.09)
    counts = [1200, 64, 700]
    off = H.ragged_offsets(counts)
    total = int(off[-1])
    slots = rng.integers(0, n_slots, total).astype(np.int32)
    q = H.bf16_to_f32(H.randn_bf16(rng, (3, Hkv, D)))
    ks = np.array([100, 16, 50], np.int32)
    koff = H.ragged_offsets(ks)
    lo, hi = head_range(Hkv, rank, world)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)  # noqa: E731
    table = t(reps16[:, lo:hi].view(np.int16)).view(torch.bfloat16)
    qr = t(q[:, lo:hi].reshape(3, -1))
    d_off, d_slots, d_k, d_koff = t(off), t(slots), t(ks), t(koff)
    ex = PeerScoreExchange.create(total, dev)
    res = []
    for rnd in range(4):
        ops.score_dot(table, d_off, qr, total=total, slot_ids=d_slots, n_kv_heads=hi - lo, head_dim=D, exchange=ex)
        idx = torch.full((int(koff[-1]),), -1, dtype=torch.int32, device=dev)
        cnt = torch.zeros((3,), dtype=torch.int32, device=dev)
        ex.topk(d_off, d_k, total=total, out_stride=100, order=ops.ORDER_SCORE_DESC, out_idx=idx, out_counts=cnt,
                id_map=d_slots, out_offsets=d_koff)
        res.append(idx.cpu().numpy())
    # the library route: all-reduce between the two kernels
    part = ops.score_dot(table, d_off, qr, total=total, slot_ids=d_slots, n_kv_heads=hi - lo, head_dim=D)
    ScoreAllReduce()(part)
    idx2 = torch.full((int(koff[-1]),), -1, dtype=torch.int32, device=dev)
    cnt2 = torch.zeros((3,), dtype=torch.int32, device=dev)
    ops.topk_ragged(part, d_off, d_k, out_stride=100, order=ops.ORDER_SCORE_DESC, id_map=d_slots, out_offsets=d_koff,
                    out_idx=idx2, out_counts=cnt2, want_scores=False)
    from ucmx import _native
    np.savez(os.path.join(out_dir, f"r{rank}.npz"), peer=np.stack(res), nccl=idx2.cpu().numpy(),
             summed=ex.summed.cpu().numpy(), reduced=part.cpu().numpy(), err=_native.device_error())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_symmetric_memory_matches_nccl(tmp_path):
    import torch.multiprocessing as mp
    port = 29600 + (os.getpid() % 1000)
    mp.spawn(_two_gpu_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    a, b = np.load(tmp_path / "r0.npz"), np.load(tmp_path / "r1.npz")
    assert a["err"] == 0 and b["err"] == 0
    assert np.array_equal(a["peer"], b["peer"]) and np.array_equal(a["summed"], b["summed"])
    for rnd in range(4):
        assert np.array_equal(a["peer"][rnd], a["peer"][0])
    np.testing.assert_allclose(a["summed"], a["reduced"], rtol=1e-5, atol=1e-6)
    same = (np.sort(a["peer"][0]) == np.sort(a["nccl"])).mean()
    assert same > 0.99
