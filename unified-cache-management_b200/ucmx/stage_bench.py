"""Per-kernel throughput at the benchmark configurations' sizes (run: python -m ucmx.stage_bench [names]).

Each kernel is timed alone with CUDA events over back-to-back launches that were queued while the
GPU was busy (so host launch cost does not show), on inputs larger than L2 or rotated so that every
launch reads cold data.  Prints one JSON object: microseconds per launch and GB/s of algorithmic
bytes (what the kernel must read and write, not what the memory system moved).
  hamming   config 3: 64-request ragged batch, 128-bit codes, 16 KiB per block, both head pairings
  hash      config 3: sign-hash encoding of paged key blocks (exact FMA chain)
  offload   config 4: gather 4096 blocks of K and V of one layer to pinned host memory and scatter
            4096 back, direct (kernel writes host memory) and staged (device compaction + one DMA)
  pool      config 1/2: pooling a whole pool, and the 64-block decode case
  kvstar    (only when named) KVStar softmax-vote scoring of the 64-request ragged batch: 8 query tokens x 32 heads per
            request against fp16 representations [64 positions, 8 heads, 32 kept channels] per block (32 KiB); the
            tensor-core kernel, the row statistics and the vote kernel timed together, and the CUDA-core kernel beside it
  connector (only when named) prefix-cache dump and load of 256 blocks x 32 layers (4 GiB) through the host-memory store:
            this connector's one address table per layer against the reference's call pattern (one dump per block,
            layer and K/V with a tensor view; one K and one V load per request and layer); wall-clock GB/s
  filestore (only when named) file-per-block store: dump 256 blocks x 16 K/V layer slices of 256 KiB (1 GiB) from
            HBM to block files under $UCMX_STORE_DIR (default: the temp dir) and load them back; wall-clock GB/s,
            bounded by that directory's file system; also with one slice per launch (the reference's granularity)
"""
from __future__ import annotations

import json
import sys

import torch

from . import ops
from .workloads import LLAMA3_8B, ragged_decode_batch


def _time(fn, iters, reps=3):
    best = float("inf")
    for _ in range(reps):
        torch.cuda.synchronize()
        torch.cuda._sleep(int(2e9 * 0.003))
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(iters):
            fn(i)
        b.record()
        torch.cuda.synchronize()
        best = min(best, a.elapsed_time(b) * 1e3 / iters)
    return best


def main(argv):
    which = argv or ["hamming", "hash", "offload", "pool"]
    dev = torch.device("cuda:0")
    shape = LLAMA3_8B
    batch = ragged_decode_batch(seed=3003)
    g = torch.Generator(device=dev).manual_seed(3003)
    off = torch.from_numpy(batch.offsets).to(dev)
    table = torch.from_numpy(batch.block_table).to(dev)
    out = {"blocks": batch.total}
    T, H, D = shape.block_tokens, shape.n_kv_heads, shape.head_dim

    if "hamming" in which:
        n_tables = 3                                             # 3 x 547 MB rotate through L2
        codes = [torch.randint(0, 256, (batch.n_slots, H, T, 16), generator=g, device=dev, dtype=torch.uint8)
                 for _ in range(n_tables)]
        qc = torch.randint(0, 256, (batch.n_req, H, 16), generator=g, device=dev, dtype=torch.uint8)
        scores = torch.empty((batch.total,), dtype=torch.int32, device=dev)
        nbytes = batch.total * (H * T * 16 + 8)
        for name, cross in (("hamming_cross_head", True), ("hamming_matched_head", False)):
            t = _time(lambda i: ops.score_hamming(codes[i % n_tables], off, qc, total=batch.total, slot_ids=table,
                                                  cross_head=cross, out=scores), iters=6)
            out[name] = {"us": t, "gbs": nbytes / t / 1e3}
        del codes

    if "hash" in which:
        nb = 2048
        k = torch.randn((nb, T, H, D), generator=g, device=dev).to(torch.bfloat16)
        w = (torch.randn((D, 128), generator=g, device=dev) * 2).to(torch.bfloat16)
        ids = torch.randperm(nb, generator=g, device=dev).to(torch.int32)
        codes = torch.empty((nb, H, T, 16), dtype=torch.uint8, device=dev)
        t = _time(lambda i: ops.hash_encode_blocks(k, ids, w, out=codes), iters=2)
        flops = nb * T * H * 2.0 * D * 128
        out["hash_encode_blocks"] = {"us": t, "gbs": nb * (T * H * D * 2 + T * H * 16) / t / 1e3, "tflops": flops / t / 1e6,
                                     "blocks": nb}
        del k, codes

    if "offload" in which:
        n_slots, n = 8192, 4096
        kv = torch.empty((2, n_slots, T, H, D), dtype=torch.bfloat16, device=dev)
        for p in range(2):
            for s in range(0, n_slots, 1024):
                kv[p, s:s + 1024].copy_(torch.randn((1024, T, H, D), generator=g, device=dev).to(torch.bfloat16))
        perm = torch.randperm(n_slots, generator=g, device=dev).to(torch.int32)
        src_ids, dst_ids = perm[:n].contiguous(), perm[n:].contiguous()
        payload = n * 2 * shape.slice_bytes                      # 2 GiB
        host = torch.empty(payload, dtype=torch.uint8).pin_memory()
        stage = torch.empty(payload, dtype=torch.uint8, device=dev)
        planes = [kv[0], kv[1]]
        res = {}
        res["gather_device_staging"] = _time(lambda i: ops.gather_blocks(planes, src_ids, stage), iters=4)
        res["scatter_device_staging"] = _time(lambda i: ops.scatter_blocks(planes, dst_ids, stage), iters=4)
        res["d2h_direct"] = _time(lambda i: ops.gather_blocks(planes, src_ids, host), iters=2, reps=2)
        res["h2d_direct"] = _time(lambda i: ops.scatter_blocks(planes, dst_ids, host), iters=2, reps=2)

        def d2h_staged(i):
            ops.gather_blocks(planes, src_ids, stage)
            host.copy_(stage, non_blocking=True)

        def h2d_staged(i):
            stage.copy_(host, non_blocking=True)
            ops.scatter_blocks(planes, dst_ids, stage)

        res["d2h_staged"] = _time(d2h_staged, iters=2, reps=2)
        res["h2d_staged"] = _time(h2d_staged, iters=2, reps=2)
        res["memcpy_d2h_pinned"] = _time(lambda i: host.copy_(stage, non_blocking=True), iters=2, reps=2)
        res["memcpy_h2d_pinned"] = _time(lambda i: stage.copy_(host, non_blocking=True), iters=2, reps=2)

        # what the reference does: one cudaMemcpyAsync per 256 KiB slice (dramstore_connector.py:129-132,161-164)
        hv = host.view(n, 2, shape.slice_bytes)
        ids_h = src_ids.cpu().tolist()
        kvb = kv.view(torch.uint8).view(2, n_slots, shape.slice_bytes)

        def per_block_d2h(i):
            for j, b in enumerate(ids_h):
                hv[j, 0].copy_(kvb[0, b], non_blocking=True)
                hv[j, 1].copy_(kvb[1, b], non_blocking=True)

        torch.cuda.synchronize()
        a, bev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        per_block_d2h(0)
        bev.record()
        torch.cuda.synchronize()
        res["per_block_memcpy_d2h"] = a.elapsed_time(bev) * 1e3
        out["offload"] = {k2: {"us": v, "gbs_payload": payload / v / 1e3} for k2, v in res.items()}
        out["offload"]["payload_bytes"] = payload
        # round trip is bit exact
        ops.gather_blocks(planes, src_ids, host)
        ops.scatter_blocks(planes, dst_ids, host)
        torch.cuda.synchronize()
        out["offload"]["roundtrip_exact"] = bool(torch.equal(kv[:, dst_ids.long()], kv[:, src_ids.long()]))
        del kv, stage, host

    if "pool" in which:
        nb = 8192                                                # 2 GiB of K
        k = torch.empty((nb, T, H, D), dtype=torch.bfloat16, device=dev)
        for s in range(0, nb, 1024):
            k[s:s + 1024].copy_(torch.randn((1024, T, H, D), generator=g, device=dev).to(torch.bfloat16))
        reps = torch.empty((nb, H, 1, D), dtype=torch.bfloat16, device=dev)
        ids = torch.randperm(nb, generator=g, device=dev).to(torch.int32)
        for mode in ("mean", "max"):
            t = _time(lambda i: ops.pool_blocks(k, ids, mode=mode, out_slots=ids, out_bf16=reps), iters=4)
            out[f"pool_{mode}_whole_pool"] = {"us": t, "gbs": nb * (shape.slice_bytes + 2048) / t / 1e3}
        sets = [ids[i * 64:(i + 1) * 64].contiguous() for i in range(16)]
        t = _time(lambda i: ops.pool_blocks(k, sets[i % 16], out_slots=sets[i % 16], out_bf16=reps), iters=16)
        out["pool_mean_64_blocks"] = {"us": t, "gbs": 64 * (shape.slice_bytes + 2048) / t / 1e3}
    if "kvstar" in which:
        import os
        Mp, dp, xq, Hq = 64, 32, 8, shape.n_q_heads
        nb = batch.total
        reps = torch.empty((nb, Mp, H, dp), dtype=torch.float16, device=dev)
        for s in range(0, nb, 2048):
            e = min(nb, s + 2048)
            reps[s:e].copy_((torch.randn((e - s, Mp, H, dp), generator=g, device=dev) * 0.6).to(torch.float16))
        nreq = batch.n_req
        q = torch.randn((nreq * xq, Hq, D), generator=g, device=dev).to(torch.float16)
        qoff = (torch.arange(nreq + 1, device=dev) * xq).to(torch.int32)
        pr = torch.stack([torch.stack([torch.randperm(D, generator=g, device=dev)[:dp] for _ in range(H)])
                          for _ in range(nreq)]).contiguous()
        ws = torch.empty((ops.kvstar_workspace_bytes(nb, nreq, xq, Hq, H),), dtype=torch.uint8, device=dev)
        votes = torch.empty((nb,), dtype=torch.float32, device=dev)

        def run(i):
            ops.kvstar_scores(reps, off, q, qoff, total=nb, max_q_tokens=xq, slot_ids=table, pruned_index=pr,
                              workspace=ws, out=votes)
        t = _time(run, iters=4)
        nbytes = nb * (Mp * H * dp * 2 + 4)
        flops = 2.0 * xq * Hq * dp * Mp * nb
        res = {"us": t, "gbs": nbytes / t / 1e3, "tflops_useful": flops / t / 1e6, "exps_per_us": xq * Hq * Mp * nb / t}
        ref_votes = votes.clone()
        os.environ["UCMX_KVSTAR_NO_TC"] = "1"
        try:
            t2 = _time(run, iters=1, reps=1)
        finally:
            os.environ.pop("UCMX_KVSTAR_NO_TC", None)
        torch.cuda.synchronize()
        res["cuda_core_us"] = t2
        res["max_rel_diff_between_kernels"] = float(((votes - ref_votes).abs() / ref_votes.abs().clamp_min(1e-6)).max())
        out["kvstar"] = res
        del reps, ws

    if "connector" in which:
        import time
        import types

        from .connector import ReqMeta, UCConnectorV1Metadata, UnifiedCacheConnectorV1
        Lc, nbc, nblk = 32, 320, 256
        mc = types.SimpleNamespace(dtype=torch.bfloat16, is_deepseek_mla=False, get_num_layers=lambda pc: Lc,
                                   get_num_kv_heads=lambda pc: H, get_head_size=lambda: D)
        cfg = types.SimpleNamespace(
            model_config=mc, parallel_config=types.SimpleNamespace(tensor_parallel_size=1),
            cache_config=types.SimpleNamespace(block_size=T),
            kv_transfer_config=types.SimpleNamespace(kv_role="kv_both", kv_connector_extra_config={
                "ucm_connector_name": "UcmDramStore", "ucm_connector_config": {"max_cache_size": 5 << 30}}))
        kvc = {f"model.layers.{l}.attn": torch.empty((2, nbc, T, H, D), dtype=torch.bfloat16, device=dev).normal_(generator=g)
               for l in range(Lc)}
        hs = [f"{i:032x}" for i in range(nblk)]
        ids = torch.randperm(nbc, generator=g, device=dev)[:nblk].tolist()
        reqs = [ReqMeta(f"r{r}", dump_blocks=list(zip(hs[r * 32:(r + 1) * 32], ids[r * 32:(r + 1) * 32]))) for r in range(8)]
        nbytes = nblk * Lc * 2 * shape.slice_bytes
        res = {"bytes": nbytes}
        for name in ("table_per_layer", "reference_call_pattern"):
            conn = UnifiedCacheConnectorV1(cfg, "worker", rank=0)
            conn.register_kv_caches(kvc)
            conn.bind_connector_metadata(UCConnectorV1Metadata(reqs))
            conn.connector._ensure_slab()           # page-locking 5 GiB is a one-time cost of the store, not of a dump
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            if name == "table_per_layer":
                for lname, layer in kvc.items():
                    conn.save_kv_layer(lname, layer)
                ok = conn.wait_for_save()
            else:
                tasks = []
                for lname, layer in kvc.items():
                    for r in reqs:
                        tensors, offsets = conn.get_tensor_and_offset_layerwise([b[1] for b in r.dump_blocks], layer, lname)
                        torch.cuda.current_stream().synchronize()
                        for bid, o, tns in zip([b[0] for b in r.dump_blocks] * 2, offsets, tensors):
                            tasks.append(conn.connector.dump([bid], [o], [tns]))
                ok = all(conn.connector.wait(tk) == 0 for tk in tasks)
            t1 = time.perf_counter()
            conn.connector.commit(hs, True)
            # load everything back into other slots
            dst = torch.randperm(nbc, generator=g, device=dev)[:nblk].tolist()
            lreqs = [ReqMeta(f"l{r}", load_blocks=list(zip(hs[r * 32:(r + 1) * 32], dst[r * 32:(r + 1) * 32]))) for r in range(8)]
            conn.bind_connector_metadata(UCConnectorV1Metadata(lreqs))
            torch.cuda.synchronize()
            t2 = time.perf_counter()
            if name == "table_per_layer":
                conn.start_load_kv()
                for lname in kvc:
                    conn.wait_for_layer_load(lname)
            else:
                tasks = []
                for r in lreqs:
                    for lname, layer in kvc.items():
                        tensors, offsets = conn.get_tensor_and_offset_layerwise([b[1] for b in r.load_blocks], layer, lname)
                        n = len(r.load_blocks)
                        tasks.append(conn.connector.load([b[0] for b in r.load_blocks], offsets[:n], tensors[:n]))
                        tasks.append(conn.connector.load([b[0] for b in r.load_blocks], offsets[n:], tensors[n:]))
                assert all(conn.connector.wait(tk) == 0 for tk in tasks)
            torch.cuda.synchronize()
            t3 = time.perf_counter()
            res[name] = {"dump_ms": (t1 - t0) * 1e3, "dump_gbs": nbytes / (t1 - t0) / 1e9, "load_ms": (t3 - t2) * 1e3,
                         "load_gbs": nbytes / (t3 - t2) / 1e9, "ok": bool(ok)}
            conn.connector.close()
        out["connector"] = res
        del kvc

    if "filestore" in which:
        import os
        import shutil
        import tempfile
        import time

        import numpy as np

        from .store.nfsstore import UcmNfsStore
        nblk, nsl = 256, 16
        sl = shape.slice_bytes
        cache = torch.empty((nblk * nsl, sl), dtype=torch.uint8, device=dev)
        cache.random_(0, 256, generator=g)
        back = torch.zeros_like(cache)
        rng = np.random.default_rng(4004)
        ids = [rng.integers(1, 256, size=32, dtype=np.uint8).tobytes() for _ in range(nblk)]
        bl = [b for b in ids for _ in range(nsl)]
        offs = [j * sl for _ in ids for j in range(nsl)]
        res = {"bytes": nblk * nsl * sl}
        for name, slots in (("grouped", 16), ("one_slice_per_launch", 2)):
            root = tempfile.mkdtemp(dir=os.environ.get("UCMX_STORE_DIR"))
            try:
                store = UcmNfsStore({"storage_backends": root, "kv_block_size": nsl * sl, "role": "worker", "device": 0,
                                     "io_size": sl, "buffer_number": slots, "stream_number": 8})
                store.create(ids)
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                st_d = store.wait(store.dump(bl, offs, list(cache)))
                t1 = time.perf_counter()
                store.commit(ids, True)
                t2 = time.perf_counter()
                st_l = store.wait(store.load(bl, offs, list(back)))
                t3 = time.perf_counter()
                torch.cuda.synchronize()
                res[name] = {"dump_gbs": res["bytes"] / (t1 - t0) / 1e9, "load_gbs": res["bytes"] / (t3 - t2) / 1e9,
                             "status": [st_d, st_l], "exact": bool(torch.equal(back, cache))}
                back.zero_()
                store.close()
            finally:
                shutil.rmtree(root, ignore_errors=True)
        out["filestore"] = res
    print(json.dumps(out))


if __name__ == "__main__":
    main(sys.argv[1:])
