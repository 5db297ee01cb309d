"""Benchmark of the decode-step sparse-KV retrieval path (pool -> score -> top-k -> gather).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-graph]

Workload (default): 64 decode requests with context lengths uniform in [8192, 131072] tokens
(seeded, rounded up to 128-token blocks), Llama-3-8B KV shapes (32 query heads, 8 KV heads,
head_dim 128, bf16), a paged K/V pool with a randomly permuted block table, top-k = 5 % of each
request's blocks (at least 16), all 32 layers per step.  A step is, for every layer: pool the 64
newest blocks, score every block of every request, select the per-request top-k and gather the
selected K and V blocks into a contiguous working set.  All data is synthetic (seeded normal).

One JSON line is printed by rank 0.  `value` = KV tokens scored per second over all GPUs with every
input resident in HBM; `e2e` = the same with queries coming from pinned host memory and the selected
block ids going back to it each layer.  With N > 1 each rank runs its own batch (data parallel over
requests, no data-path collective): weak scaling.

`--impl reference` times the reference's own CPU retrieval (its compiled RetrievalWorkerBackend:
fp32 dot scores + partial_sort top-k) on the host cores for the same batch, on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "unified-cache-management_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

METRIC = "decode_step_retrieval_scored_kv_tokens_per_s"
UNIT = "tokens/s"
FALLBACK_HBM_GBS = 6650.0

# DRAM bytes per launch of the dominant kernel (xfer_bulk_kernel gathering one layer's selected K and
# V blocks) over its algorithmic bytes, from a one-pass ncu capture of this benchmark at full size
# (profiles/xfer_bulk_gather_full_size_traffic.md): reads 955.28 MB = the payload, writes 895.5 MB (the
# last ~57 MB are still dirty in L2 when the kernel ends), against 2 x 955.25 MB.
NCU_GATHER_TRAFFIC_PER_ALGORITHMIC_BYTE = 0.969


def env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as fh:
                d = json.load(fh)
            return float(d["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(prefix="ucmx_clocks_", suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-f", self.path], stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        try:
            self.proc.terminate()
            self.proc.wait(timeout=5)
        except Exception:
            pass
        try:
            rows = [ln.strip().split(",") for ln in open(self.path) if ln.strip()]
            os.remove(self.path)
        except Exception:
            return out
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(names, r[2:6]):
                if v.strip().lower() == "active":
                    reasons.add(name)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


# ------------------------------------------------------------------------------------ reference arm

def reference_cpu_run(batch, layers_per_step: int, steps: int, warmup: int, distinct_tables: int = 4):
    """The reference's CPU retrieval for this batch: one RetrievalWorkerBackend per layer table, one
    submit per request (what ESA does, ucm/sparse/esa/esa.py:286-301), all in flight at once, so
    that every host core its thread pool owns has work.  Returns (tokens_per_s, sec_per_step, cores)."""
    import numpy as np
    from oracle import oracle as orc
    rb = orc.ref_retrieval_backend()
    rng = np.random.default_rng(2002)
    dim = 1024
    n_tables = min(distinct_tables, layers_per_step)
    backends = []
    for _ in range(n_tables):
        data = orc.bf16_to_f32(orc.f32_to_bf16(rng.standard_normal((batch.n_slots, dim), dtype=np.float32) * np.float32(0.0884)))
        backends.append((rb.RetrievalWorkerBackend(data), data))
    queries = orc.bf16_to_f32(orc.f32_to_bf16(rng.standard_normal((layers_per_step, batch.n_req, dim), dtype=np.float32)))
    slot_lists = [np.ascontiguousarray(batch.block_table[batch.offsets[r]:batch.offsets[r + 1]][None, :]) for r in range(batch.n_req)]

    def one_step():
        for l in range(layers_per_step):
            be = backends[l % n_tables][0]
            rids = [be.submit(queries[l, r:r + 1], int(batch.k_per_req[r]), slot_lists[r]) for r in range(batch.n_req)]
            for rid in rids:
                be.wait(rid)
                be.get_result(rid)

    for _ in range(warmup):
        one_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    tokens = batch.total * 128 * layers_per_step
    return tokens / dt, dt, os.cpu_count()


def run_reference(args, rank: int):
    if rank != 0:
        return
    from ucmx.workloads import ragged_decode_batch
    from oracle import oracle as orc
    base = {"impl": "reference", "metric": METRIC, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic"}
    if not orc.have_ref():
        base["unavailable"] = "oracle/_ref (the compiled reference CPU sources) is not present on this machine"
        print(json.dumps(base))
        return
    batch = ragged_decode_batch(seed=2002)
    layers = 8
    tps, dt, cores = reference_cpu_run(batch, layers, args.steps, args.warmup)
    base.update({
        "value": tps, "ms_per_step": dt * 1e3,
        "config": workload_config(batch, extra={"sample": f"{layers} of 32 layers per step"}),
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cores, "kind": "reference",
                         "sample": f"{layers} of 32 layers of the 64-request batch per step, score + top-k only "
                                   "(RetrievalWorkerBackend, one submit per request, all in flight)"},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    })
    print(json.dumps(base))


def run_offload(args, rank, world, local_rank, dev, barrier):
    """Configuration 4: per step and GPU, gather 4096 randomly chosen K and V blocks of one layer (2 GiB) into
    pinned host memory and scatter 4096 blocks back into randomly chosen free slots.  Device side: one
    compaction kernel per direction; host link: one DMA per direction.  Weak scaling (every GPU moves its own)."""
    import torch
    import torch.distributed as dist
    from ucmx import _native, ops
    from ucmx.workloads import LLAMA3_8B as shape
    from ucmx.store.numa import bind_to_device_node
    numa_node = None if os.environ.get("UCMX_NO_NUMA_BIND") else bind_to_device_node(local_rank)   # before page-locking
    g = torch.Generator(device=dev).manual_seed(4004 + rank)
    n_slots, n = 8192, 4096
    T, H, D = shape.block_tokens, shape.n_kv_heads, shape.head_dim
    kv = torch.empty((2, n_slots, T, H, D), dtype=torch.bfloat16, device=dev)
    for p in range(2):
        for s in range(0, n_slots, 1024):
            kv[p, s:s + 1024].copy_(torch.randn((1024, T, H, D), generator=g, device=dev).to(torch.bfloat16))
    perm = torch.randperm(n_slots, generator=g, device=dev).to(torch.int32)
    src_ids, dst_ids = perm[:n].contiguous(), perm[n:].contiguous()
    payload = n * 2 * shape.slice_bytes
    host = torch.empty(payload, dtype=torch.uint8).pin_memory()
    stage = torch.empty(payload, dtype=torch.uint8, device=dev)
    planes = [kv[0], kv[1]]

    def step():
        ops.gather_blocks(planes, src_ids, stage)
        host.copy_(stage, non_blocking=True)
        stage.copy_(host, non_blocking=True)
        ops.scatter_blocks(planes, dst_ids, stage)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    launches_before = _native.launch_count
    barrier()
    torch.cuda.synchronize()
    sampler.start()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        step()
    b.record()
    torch.cuda.synchronize()
    barrier()
    clocks = sampler.stop()
    ms = a.elapsed_time(b)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    exact = bool(torch.equal(kv[:, dst_ids.long()], kv[:, src_ids.long()]))
    if rank == 0:
        gbs = 2.0 * payload * world * args.steps / (ms * 1e-3) / 1e9
        print(json.dumps({
            "metric": "kv_block_offload_bytes_per_s", "value": gbs, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {"workload": "KV block offload: per GPU and step 4096 random K+V blocks of one Llama-3-8B layer (2 GiB) "
                                   "gathered to pinned host memory and 4096 scattered back into free slots",
                       "payload_bytes_per_direction_per_gpu": payload, "route": "device compaction + one DMA per direction", "numa_node_of_rank0": numa_node},
            "per_gpu_gbs_each_direction": payload * args.steps / (ms * 1e-3) / 1e9 * 2 / 2, "roundtrip_exact": exact,
            "gpu_launches": _native.launch_count - launches_before, "clocks": clocks}))


def workload_config(batch, extra=None):
    cfg = {
        "workload": "ESA batched decode, 64 requests, ctx U[8192,131072] tokens, Llama-3-8B KV (32q/8kv heads, "
                    "head_dim 128, block 128), paged pool with permuted block table, top-k 5% (min 16), 32 layers/step",
        "n_req": int(batch.n_req), "blocks_total_per_layer": int(batch.total), "selected_per_layer": int(batch.total_k),
        "layers": 32, "stages": "pool(64 new blocks of each of the 32 layers, one launch per step) + per layer score+topk+gather(K,V of selected)",
        "l2_policy": "inputs larger than L2: 2.3 GB of representatives and an 18 GB K/V pool are cycled per step",
        "parallelism": "dp over requests: every GPU serves 64 requests of these lengths over its own block table and data",
    }
    if extra:
        cfg.update(extra)
    return cfg


# ----------------------------------------------------------------------------------------- our arm

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="launch the step call by call instead of replaying its CUDA graph")
    ap.add_argument("--no-e2e-graph", action="store_true", help="end-to-end step launched call by call instead of replayed from its CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--layers", type=int, default=None, help=argparse.SUPPRESS)
    ap.add_argument("--workload", default="decode64", choices=["decode64", "tp-long", "offload"],
                    help="decode64: the 64-request ragged decode batch, data parallel over requests (default); "
                         "tp-long: 8 requests of 1 048 576 tokens, KV heads split over the GPUs with an all-reduce of "
                         "block scores before top-k; offload: every GPU moves 4096 random K+V blocks of one layer (2 GiB) to "
                         "pinned host memory and 4096 back into free slots per step")
    ap.add_argument("--allreduce", default="nccl", choices=["nccl", "peer"],
                    help="tp-long only: how partial block scores are summed over ranks - a NCCL all-reduce between the "
                         "scoring and top-k kernels, or peer-memory loads inside the top-k kernel")
    ap.add_argument("--profile-case", action="store_true",
                    help="small case for profiler captures: 8 requests, 2 layers, 1 warm-up + 1 step, no host legs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    n_req = 64
    tp = args.workload == "tp-long"
    if args.layers is None:
        args.layers = 16 if tp else 32
    if args.profile_case:
        args.layers, args.steps, args.warmup, args.no_cpu_baseline, n_req = 2, 1, 1, True, 8

    rank = env_int("RANK", 0)
    world = env_int("WORLD_SIZE", 1)
    local_rank = env_int("LOCAL_RANK", 0)

    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    from ucmx import _native
    from ucmx.engine import DecodeRetrievalEngine
    from ucmx.parallel import PeerScoreExchange, ScoreAllReduce, head_range
    from ucmx.workloads import LLAMA3_8B, QWEN2_72B_LIKE, fixed_batch, ragged_decode_batch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local_rank])

    if args.workload == "offload":
        run_offload(args, rank, world, local_rank, dev, barrier)
        if world > 1:
            dist.destroy_process_group()
        return

    if tp:
        # every rank sees the same 8 requests and block tables and holds n_kv_heads/world of the heads
        shape = QWEN2_72B_LIKE
        batch = fixed_batch(8, 8192, 2048, seed=5005)
        lo, hi = head_range(shape.n_kv_heads, rank, world)
        peer = PeerScoreExchange.create(batch.total, dev) if (world > 1 and args.allreduce == "peer") else None
        eng = DecodeRetrievalEngine(shape, batch, dev, n_layers=args.layers, seed=1000 + rank, heads_local=hi - lo,
                                    score_reduce=ScoreAllReduce() if (world > 1 and peer is None) else None,
                                    peer_exchange=peer)
    else:
        shape = LLAMA3_8B
        # weak scaling: every rank serves requests of the same lengths (the same work per GPU) over its own block
        # table, keys and queries
        batch = ragged_decode_batch(seed=2002, n_req=n_req, table_seed=None if rank == 0 else 7007 + rank)
        eng = DecodeRetrievalEngine(shape, batch, dev, n_layers=args.layers, seed=1000 + rank)
    eng.make_queries()
    torch.cuda.synchronize()

    # prefill-time pooling of the whole pool (layer 0's table is really pooled), timed on its own
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    eng.prefill_pool_all(0)
    torch.cuda.synchronize()
    e0.record()
    eng.prefill_pool_all(0)
    e1.record()
    torch.cuda.synchronize()
    prefill_ms = e0.elapsed_time(e1)
    row_bytes = eng.H * eng.D * 2
    prefill_gbs = batch.total * (eng.T * row_bytes + row_bytes) / prefill_ms / 1e6

    # The step is replayed from a CUDA graph unless --no-graph (or a tensor-parallel run, whose exchange is driven
    # from the host).  The gather launches are timed by events around them.  An event record costs about 6 us of
    # stream time, call by call and as a graph node alike, so in graph mode the last of the K timed steps replays
    # a second graph that has an event pair around each of its gathers and the other K-1 replay the plain one;
    # call by call, every fourth gather launch of every step carries a pair.
    use_graph = not args.no_graph and not tp and not args.profile_case
    timed_graph = None
    if use_graph:
        gev = [(torch.cuda.Event(enable_timing=True, external=True), torch.cuda.Event(enable_timing=True, external=True))
               for _ in range(eng.L)]
        timed_graph = eng.capture(gather_events=gev)
        eng.capture()
        timed_graph.replay()
    for _ in range(args.warmup):
        eng.step()
    torch.cuda.synchronize()

    # ---- timed region: K steps, device-resident inputs; the gather launches carry their own events
    every = 1 if args.profile_case else 4
    if not use_graph:
        gev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
               for _ in range(args.steps * ((eng.L + every - 1) // every))]
    sampler = ClockSampler(local_rank)
    launches_before = _native.launch_count
    barrier()
    torch.cuda.synchronize()
    sampler.start()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    if use_graph:
        for _ in range(args.steps - 1):
            eng.step()
        timed_graph.replay()
    else:
        gi = 0
        for _ in range(args.steps):
            eng.pool_all_layers()
            for l in range(eng.L):
                eng.score_layer(l)
                eng.topk_layer(l)
                if l % every == 0:
                    a, b = gev[gi]
                    gi += 1
                    a.record()
                    eng.gather_layer(l)
                    b.record()
                else:
                    eng.gather_layer(l)
    t_end.record()
    torch.cuda.synchronize()
    barrier()
    clocks = sampler.stop()
    launches = (_native.launch_count - launches_before) if not use_graph else eng.launches_per_step * args.steps
    elapsed_ms = t_start.elapsed_time(t_end)
    if world > 1:
        t = torch.tensor([elapsed_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    tokens_per_step_all = eng.tokens_scored_per_step() * world   # same batch size on every rank (weak scaling)
    if tp:
        tokens_per_step_all = eng.tokens_scored_per_step()       # one batch shared by all ranks (strong scaling)
    elif world > 1:
        tt = torch.tensor([float(eng.tokens_scored_per_step())], dtype=torch.float64, device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.SUM)
        tokens_per_step_all = float(tt.item())
    value = tokens_per_step_all / (ms_per_step * 1e-3)

    gather_ms = [a.elapsed_time(b) for a, b in gev]
    gather_avg_ms = statistics.fmean(gather_ms) if gather_ms else None

    # ---- per-stage breakdown (separate instrumented pass, same inputs)
    stage_names = ("pool", "score", "topk", "gather")
    acc = {s: [] for s in stage_names}
    evs = []
    pool_marks = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    eng.pool_all_layers()                      # one launch for the new blocks of all layers; the second one is timed
    pool_marks[0].record()
    eng.pool_all_layers()
    pool_marks[1].record()
    for l in range(eng.L):
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        marks[0].record()
        marks[1].record()
        eng.score_layer(l)
        marks[2].record()
        eng.topk_layer(l)
        marks[3].record()
        eng.gather_layer(l)
        marks[4].record()
        evs.append(marks)
    torch.cuda.synchronize()
    for marks in evs:
        for i, s in enumerate(stage_names):
            acc[s].append(marks[i].elapsed_time(marks[i + 1]) * 1e3)
    stages_us = {s: statistics.median(v) for s, v in acc.items()}
    stages_us["pool"] = pool_marks[0].elapsed_time(pool_marks[1]) * 1e3 / eng.L
    retrieval_us = stages_us["pool"] + stages_us["score"] + stages_us["topk"]

    # ---- end to end with host buffers
    eng.graph = None
    e2e_s = float("nan")
    if not args.profile_case:
        eng.alloc_host()
        if not tp and not args.no_e2e_graph:
            eng.capture_host()                 # copies and kernels of both streams in one graph; step_host() replays it
        for _ in range(2):
            eng.step_host()
        barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            eng.step_host()
        torch.cuda.synchronize()
        e2e_s = (time.perf_counter() - t0) / args.steps
    if world > 1:
        t = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = tokens_per_step_all / e2e_s

    peak, peak_kind = measured_peaks()
    roofline = None
    if gather_avg_ms:
        achieved = eng.bytes_gather_layer() / (gather_avg_ms * 1e-3) / 1e9
        traffic = None
        if NCU_GATHER_TRAFFIC_PER_ALGORITHMIC_BYTE is not None:
            traffic = eng.bytes_gather_layer() * NCU_GATHER_TRAFFIC_PER_ALGORITHMIC_BYTE
        roofline = {"kernel": "xfer_bulk_kernel (gather of selected K,V blocks, one layer)", "bound": "hbm",
                    "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                    "traffic": traffic, "algorithmic_bytes_per_launch": eng.bytes_gather_layer(),
                    "avg_launch_us": gather_avg_ms * 1e3, "launches_timed": len(gather_ms)}
    stage_gbs = {
        "score": eng.bytes_score_layer() / (stages_us["score"] * 1e-6) / 1e9,
        "gather": eng.bytes_gather_layer() / (stages_us["gather"] * 1e-6) / 1e9,
        "pool_decode": eng.bytes_pool_layer() / (stages_us["pool"] * 1e-6) / 1e9,
        "pool_prefill": prefill_gbs,
    }

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and not tp:
        try:
            from oracle import oracle as orc
            if orc.have_ref():
                tps, dt, cores = reference_cpu_run(batch, 8, 10, 1)
                cpu_baseline = {"value": tps, "unit": UNIT, "cores": cores, "kind": "reference",
                                "sample": "10 timed passes over 8 of the 32 layers of the same 64-request batch, "
                                          "score + top-k only (compiled RetrievalWorkerBackend, one submit per request)",
                                "ms_per_layer": dt * 1e3 / 8}
            else:
                cpu_baseline = {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "reference",
                                "sample": "oracle/_ref not present"}
        except Exception as exc:  # the baseline must never take the benchmark down
            cpu_baseline = {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "reference",
                            "sample": f"failed: {exc}"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong" if tp else "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": workload_config(batch, extra={"cuda_graph": use_graph, "layers": eng.L}) if not tp else {
                "workload": "long-context sharded retrieval: 8 requests x 1 048 576 tokens (8192 blocks each), Qwen2-72B-like "
                            "KV (64q/8kv heads, head_dim 128), KV heads split over the GPUs, fp32 all-reduce of 65 536 block "
                            "scores before top-k 2048, gather of the selected K,V head slices",
                "layers": eng.L, "tp": world, "heads_per_rank": eng.H, "parallelism": f"tp{world} over KV heads", "allreduce": args.allreduce if world > 1 else "none",
                "l2_policy": "inputs larger than L2 per step", "cuda_graph": use_graph},
            "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"],
                       "samples": clocks["samples"]},
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_s * 1e3,
                    "h2d_bytes_per_step": eng.h2d_bytes_per_step, "d2h_bytes_per_step": eng.d2h_bytes_per_step,
                    "cuda_graph": eng.host_graph is not None},
            "gpu_launches": int(launches),
            "roofline": roofline,
            "cpu_baseline": cpu_baseline,
            "stages_us_per_layer": stages_us,
            "retrieval_us_per_layer": retrieval_us,
            "stage_gbs": stage_gbs,
            "device_error": _native.device_error(),
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
