"""Benchmark of the decode-step sparse-KV retrieval path (pool -> score -> top-k -> gather).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload (decode64): 64 decode requests with context lengths uniform in [8192, 131072] tokens
(seeded, rounded up to 128-token blocks), Llama-3-8B KV shapes (32 query heads, 8 KV heads,
head_dim 128, bf16), a paged K/V pool with a randomly permuted block table, top-k = 5 % of each
request's blocks (at least 16), all 32 layers per step.  A step is, for every layer: pool the 64
newest blocks, score every block of every request, select the per-request top-k and gather the
selected K and V blocks into a contiguous working set.  All data is synthetic (seeded normal).

One JSON line is printed by rank 0.
  value            KV tokens scored per second over all GPUs with every input resident in HBM
  e2e              the same count of tokens per second through the reference's own retrieval object
                   (RetrievalWorkerBackend: numpy query and index lists in, numpy indices and scores out, one
                   submit per request, the way ESA calls it) - what `--impl reference` times on the host cores
  e2e_full_step    the whole step with queries coming from pinned host memory and the selected ids going back
  retrieval_only   score + top-k per layer, ours (graph nodes, no event overhead) beside the reference's
  parity_at_bench_config   one layer of this very batch checked against the compiled reference
  tp_long          the long-context case with KV heads split over the GPUs (all-reduce of block scores before
                   top-k); on one GPU its single-rank time
With N > 1 each rank runs its own batch (data parallel over requests, no data-path collective): weak scaling.

Other workloads print their own JSON line: decode64-delta (remap + delta load instead of the full gather),
tp-long, offload, hamming, hash, pool, kvstar, connector, filestore.

`--impl reference` times the reference's own CPU retrieval (its compiled RetrievalWorkerBackend: fp32 dot scores
+ partial_sort top-k) on the host cores for the same batch, all 32 layers per step.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "unified-cache-management_b200")

METRIC = "decode_step_retrieval_scored_kv_tokens_per_s"
UNIT = "tokens/s"
FALLBACK_HBM_GBS = 6650.0
N_PLUGIN_TABLES = 4          # distinct representative tables the retrieval objects of both arms cycle through

# DRAM traffic of one launch of the gather kernel, from an ncu capture (dram__bytes_read.sum + dram__bytes_write.sum)
# of the --profile-case batch (274 blocks, 143.65 MB of payload): reads = the payload (143.71 MB), writes = the
# payload minus what is still dirty in L2 when the kernel ends (84.0-87.0 MB written: 58.6 MB on average stay behind,
# about half of the 126 MB L2).  Reads grow with the blocks moved, the residue does not (an earlier full-size capture
# showed the same 57 MB), so a full launch moves its algorithmic bytes minus that residue.
GATHER_L2_DIRTY_RESIDUE_BYTES = 58.6e6
GATHER_TRAFFIC_SOURCE = ("ncu dram__bytes_read+write of xfer_bulk_kernel on the --profile-case batch: reads = payload, "
                         "writes = payload - 58.6 MB still dirty in L2; scaled to this launch by blocks moved")


def env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def load_workloads():
    """The seeded batch generators, loaded by file so that the reference arm maps none of the repo's native code."""
    spec = importlib.util.spec_from_file_location("ucmx_workloads", os.path.join(PKG, "ucmx", "workloads.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ucmx_workloads"] = mod
    spec.loader.exec_module(mod)
    return mod


def use_package():
    for p in (ROOT, PKG):
        if p not in sys.path:
            sys.path.insert(0, p)


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
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs.  nvidia-smi takes a while to
    deliver its first line (longer than a short timed region), so it is started ahead of the warm-up steps, waited
    for, and the lines are picked by their time stamps: those between begin() and stop(), else - a timed region
    shorter than the sampling period - those of the warm-up steps of the same workload just before it."""

    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None
        self.t_begin = None

    def start(self, wait_s: float = 3.0):
        try:
            fd, self.path = tempfile.mkstemp(prefix="ucmx_clocks_", suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "25", "-f", self.path], stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
            t0 = time.time()
            while time.time() - t0 < wait_s and os.path.getsize(self.path) == 0:     # until the first line is there
                time.sleep(0.01)
        except Exception:
            self.proc = None

    def begin(self):
        """The timed region starts now."""
        self.t_begin = time.time()

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        t_end = time.time()
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
        import datetime
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        parsed = []
        for r in rows:
            if len(r) < 7:
                continue
            try:
                ts = datetime.datetime.strptime(r[0].strip(), "%Y/%m/%d %H:%M:%S.%f").timestamp()
                parsed.append((ts, float(r[1]), float(r[2]), [n for n, v in zip(names, r[3:7]) if v.strip().lower() == "active"]))
            except ValueError:
                continue
        begin = self.t_begin if self.t_begin is not None else 0.0
        window = "timed region"
        picked = [x for x in parsed if begin <= x[0] <= t_end]
        if not picked:
            window = "warm-up steps just before the timed region (the region is shorter than the sampling period)"
            picked = [x for x in parsed if begin - 0.25 <= x[0] <= t_end + 0.05]
        if picked:
            out.update(sm_mhz=statistics.median(x[1] for x in picked), sm_max_mhz=max(x[2] for x in picked),
                       reasons=sorted({n for x in picked for n in x[3]}), samples=len(picked), window=window)
        return out


def workload_config(batch):
    """The same dictionary in both arms."""
    return {
        "workload": "ESA batched decode, 64 requests, ctx U[8192,131072] tokens, Llama-3-8B KV (32q/8kv heads, "
                    "head_dim 128, block 128), paged pool with permuted block table, top-k 5% (min 16), 32 layers/step",
        "n_req": int(batch.n_req), "blocks_total_per_layer": int(batch.total), "selected_per_layer": int(batch.total_k),
        "layers": 32,
        "l2_policy": "inputs larger than L2: 2.3 GB of representatives (and an 18 GB K/V pool) are cycled per step",
        "parallelism": "dp over requests: every GPU serves 64 requests of these lengths over its own block table and data",
    }


# ------------------------------------------------------------- inputs of the retrieval objects (both arms)

def plugin_inputs(batch, layers: int, seed: int = 2002):
    """What the reference's RetrievalWorkerBackend is fed: fp32 representative tables (bf16-rounded values, as ESA
    stores them), one fp32 query row per request and layer, one slot list per request, k per request."""
    import numpy as np
    rng = np.random.default_rng(seed)
    dim = 1024

    def bf16_round(a):
        u = a.view(np.uint32)
        u = (u + 0x7fff + ((u >> 16) & 1)) & np.uint32(0xffff0000)
        return u.view(np.float32)

    tables = [bf16_round(rng.standard_normal((batch.n_slots, dim), dtype=np.float32) * np.float32(0.0884))
              for _ in range(min(N_PLUGIN_TABLES, layers))]
    queries = bf16_round(rng.standard_normal((layers, batch.n_req, dim), dtype=np.float32))
    slot_lists = [np.ascontiguousarray(batch.block_table[batch.offsets[r]:batch.offsets[r + 1]][None, :])
                  for r in range(batch.n_req)]
    ks = [int(k) for k in batch.k_per_req]
    return tables, queries, slot_lists, ks


def plugin_layer_pass(backends, queries, slot_lists, ks, layers):
    """ESA's call pattern (ucm/sparse/esa/esa.py:286-339): per layer one submit per request, all in flight, then
    wait and collect each."""
    n_req = len(ks)
    nb = len(backends)
    last = None
    for l in range(layers):
        be = backends[l % nb]
        q = queries[l]
        rids = [be.submit(q[r:r + 1], ks[r], slot_lists[r]) for r in range(n_req)]
        for rid in rids:
            be.wait(rid)
            last = be.get_result(rid)
    return last


def plugin_layer_pass_batched(backends, queries, padded_idx, kmax, layers):
    """The other way the object can be called: one submit carrying the whole batch (index matrix padded with -1)."""
    nb = len(backends)
    for l in range(layers):
        be = backends[l % nb]
        rid = be.submit(queries[l], kmax, padded_idx)
        be.wait(rid)
        be.get_result(rid)


def time_plugin(backends, queries, slot_lists, ks, layers, steps, warmup):
    for _ in range(warmup):
        plugin_layer_pass(backends, queries, slot_lists, ks, layers)
    t0 = time.perf_counter()
    for _ in range(steps):
        plugin_layer_pass(backends, queries, slot_lists, ks, layers)
    return (time.perf_counter() - t0) / max(steps, 1)


def padded_index_matrix(slot_lists):
    import numpy as np
    width = max(s.shape[1] for s in slot_lists)
    m = np.full((len(slot_lists), width), -1, np.int32)
    for r, s in enumerate(slot_lists):
        m[r, :s.shape[1]] = s[0]
    return m


# ------------------------------------------------------------------------------------ reference arm

def run_reference(args, rank: int):
    """The reference's compiled RetrievalWorkerBackend on the host cores.  Imports nothing of the package."""
    if rank != 0:
        return
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    W = load_workloads()
    from oracle import oracle as orc
    base = {"impl": "reference", "metric": METRIC, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic"}
    if not orc.have_ref():
        base["unavailable"] = "oracle/_ref (the compiled reference CPU sources) is not present on this machine"
        print(json.dumps(base))
        return
    rb = orc.ref_retrieval_backend()
    batch = W.ragged_decode_batch(seed=2002)
    layers = 32
    tables, queries, slot_lists, ks = plugin_inputs(batch, layers)
    backends = [rb.RetrievalWorkerBackend(t) for t in tables]
    dt = time_plugin(backends, queries, slot_lists, ks, layers, args.steps, args.warmup)
    tokens = batch.total * 128 * layers
    tps = tokens / dt
    sample = ("all 32 layers of the 64-request batch per step, score + top-k (the reference has no CPU pooling or block "
              "transfer on this path): RetrievalWorkerBackend, one submit per request, all in flight")
    base.update({
        "value": tps, "ms_per_step": dt * 1e3, "config": workload_config(batch),
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": os.cpu_count(), "kind": "reference", "sample": sample,
                         "ms_per_layer": dt * 1e3 / layers},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    })
    print(json.dumps(base))


def reference_baseline(batch, plug, budget_s: float = 12.0):
    """cpu_baseline of our arm: the compiled reference on this box's host cores, same inputs as our retrieval
    object gets, as many passes over the 32 layers as fit the budget (at least 3)."""
    from oracle import oracle as orc
    if not orc.have_ref():
        return {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "reference", "sample": "oracle/_ref not present"}, None
    rb = orc.ref_retrieval_backend()
    tables, queries, slot_lists, ks = plug
    layers = queries.shape[0]
    backends = [rb.RetrievalWorkerBackend(t) for t in tables]
    plugin_layer_pass(backends, queries, slot_lists, ks, layers)            # warm-up
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < 3 or (time.perf_counter() < t_end and len(times) < 40):
        t0 = time.perf_counter()
        plugin_layer_pass(backends, queries, slot_lists, ks, layers)
        times.append(time.perf_counter() - t0)
    dt = statistics.median(times)
    t0 = time.perf_counter()
    plugin_layer_pass_batched(backends, queries, padded_index_matrix(slot_lists), max(ks), layers)
    dt_batched = time.perf_counter() - t0
    tps = batch.total * 128 * layers / dt
    out = {"value": tps, "unit": UNIT, "cores": os.cpu_count(), "kind": "reference",
           "sample": f"{len(times)} passes over all 32 layers of the same 64-request batch, score + top-k only (compiled "
                     "RetrievalWorkerBackend, one submit per request, all in flight; median pass)",
           "ms_per_layer": dt * 1e3 / layers, "ms_per_layer_one_batched_submit": dt_batched * 1e3 / layers}
    return out, backends


def cpu_baseline_legs():
    """The other CPU paths of the reference, each timed on a bounded sample of its own configuration."""
    import numpy as np
    legs = {}
    try:
        from oracle import oracle as orc
        if orc.have_ref():
            # GSA: SelectTopKBS semantics for one request of config 1 (256 blocks, 32q/8kv heads, k 64, windows 2/4):
            # q head mean + dot scores (OpenMP, 16 threads hard-coded in the reference) + stable_sort top-k
            rng = np.random.default_rng(1001)
            reps = rng.standard_normal((256, 8, 1, 128), dtype=np.float32)
            q = rng.standard_normal((32, 128), dtype=np.float32)
            orc.ref_gsa_select_topk(q, reps, 8, 32, 1, 128, 2, 4, 64)
            t0 = time.perf_counter()
            n = 0
            while time.perf_counter() - t0 < 2.0:
                orc.ref_gsa_select_topk(q, reps, 8, 32, 1, 128, 2, 4, 64)
                n += 1
            per = (time.perf_counter() - t0) / n
            legs["gsa_select_topk_config1"] = {"us_per_request": per * 1e6, "kind": "reference",
                                               "threads": "OpenMP, 16 as set by the reference's source",
                                               "cores": os.cpu_count(), "sample": f"{n} calls, 256 blocks, k 64, windows 2/4"}
            k32 = rng.standard_normal((64, 8, 128, 128), dtype=np.float32)      # [blocks, heads, tokens, dim], its own layout
            t0 = time.perf_counter()
            n = 0
            while time.perf_counter() - t0 < 2.0:
                orc.ref_gsa_k_repre(k32)
                n += 1
            per = (time.perf_counter() - t0) / n
            legs["gsa_k_repre_64_blocks"] = {"us_per_call": per * 1e6, "gbs": k32.nbytes / per / 1e9, "kind": "reference",
                                             "threads": "OpenMP, 32 as set by the reference's source", "cores": os.cpu_count(),
                                             "sample": f"{n} calls of ComputeKRepre over 64 fp32 blocks"}
    except Exception as exc:
        legs["gsa_error"] = str(exc)
    try:
        # KVComp on CPU torch, the reference's expressions (hash_encoder.py:119-157,199-212; kvcomp.py:239-253):
        # sign of a bf16 matmul, unpack to +-1 fp16, einsum over every (query head, key head) pair, sum, top-k
        import torch
        torch.manual_seed(3003)
        n_blocks, H, T, D, bits = 256, 8, 128, 128, 128
        keys = torch.randn((n_blocks, T, H, D)).to(torch.bfloat16)
        w = torch.randn((D, bits)).to(torch.bfloat16)
        qv = torch.randn((1, H, D)).to(torch.bfloat16)
        pw = (2 ** torch.arange(8, dtype=torch.int32)).to(torch.uint8)

        def encode(x):
            b = (torch.matmul(x, w) > 0).to(torch.uint8).reshape(*x.shape[:-1], bits // 8, 8)
            return (b * pw).sum(-1).to(torch.uint8)

        def unpack(c):
            b = ((c.unsqueeze(-1) >> torch.arange(8, dtype=torch.uint8)) & 1).reshape(*c.shape[:-1], bits)
            return b.to(torch.float32) * 2 - 1            # (the reference uses fp16; CPU torch has no fp16 einsum)

        t0 = time.perf_counter()
        codes = encode(keys).permute(0, 2, 1, 3).contiguous()            # [n, H, T, 16]
        t_hash = time.perf_counter() - t0
        t0 = time.perf_counter()
        qc = unpack(encode(qv))
        kc = unpack(codes)
        s = torch.einsum("tid,njsd->tijsn", qc, kc).sum(dim=(0, 1, 2, 3))
        torch.topk(s[1:-2], 26)
        t_score = time.perf_counter() - t0
        legs["kvcomp_cpu_torch_256_blocks"] = {"hash_ms": t_hash * 1e3, "score_topk_ms": t_score * 1e3, "kind": "port",
                                               "threads": torch.get_num_threads(), "cores": os.cpu_count(),
                                               "sample": "one request of 256 blocks (config 3 has 33 391): codes of the keys, then "
                                                         "unpack + einsum + top-k 10%"}
    except Exception as exc:
        legs["kvcomp_error"] = str(exc)
    return legs


# ----------------------------------------------------------------------------------- parity at bench size

def parity_at_bench_config(eng, batch, layer: int):
    """One layer of the timed batch against the reference itself: the engine's representative table (widened to
    fp32) and bf16-rounded query means go through the compiled RetrievalWorkerBackend, request by request; the
    selected sets must be equal except where scores tie at the cut within 1e-3, scores within 1e-3 relative."""
    import numpy as np
    import torch
    from oracle import oracle as orc
    table = eng.rep_tables[layer].reshape(batch.n_slots, -1).float().cpu().numpy()
    q16 = eng.q_dev[layer].view(torch.int16).cpu().numpy().view(np.uint16)
    qbar = orc.query_group_mean(q16, eng.H, True)
    sel = eng.sel_ids[layer].cpu().numpy()
    sel_sc = eng.sel_scores[layer].cpu().numpy()
    cnt = eng.sel_counts[layer].cpu().numpy()
    kind = "reference" if orc.have_ref() else "port"
    be = orc.ref_retrieval_backend().RetrievalWorkerBackend(table) if kind == "reference" else None
    sets_equal, tie_only, max_rel = 0, 0, 0.0
    scale = float(np.abs(sel_sc[sel_sc > -1e30]).mean()) if sel_sc.size else 1.0
    for r in range(batch.n_req):
        lo, hi = int(batch.offsets[r]), int(batch.offsets[r + 1])
        slots = np.ascontiguousarray(batch.block_table[lo:hi][None, :])
        k = int(batch.k_per_req[r])
        if be is not None:
            rid = be.submit(np.ascontiguousarray(qbar[r:r + 1]), k, slots)
            be.wait(rid)
            res = be.get_result(rid)
            want_ids, want_sc = res["indices"][0], res["scores"][0]
        else:
            s = orc.score_dot_esa(table, np.array([0, hi - lo], np.int32), slots[0], qbar[r:r + 1])
            want_ids, want_sc = orc.topk_esa(s, k, slots[0])
        o = int(batch.k_offsets[r])
        got_ids, got_sc = sel[o:o + cnt[r]], sel_sc[o:o + cnt[r]]
        if len(got_ids) != len(want_ids):
            continue
        max_rel = max(max_rel, float(np.max(np.abs(np.sort(got_sc)[::-1] - np.sort(want_sc)[::-1])) / scale))
        if np.array_equal(np.sort(got_ids), np.sort(want_ids)):
            sets_equal += 1
            continue
        odd = np.setxor1d(got_ids, want_ids)
        sc_of = dict(zip(want_ids.tolist(), want_sc.tolist()))
        sc_of.update(zip(got_ids.tolist(), got_sc.tolist()))
        cut = float(want_sc[-1])
        if all(abs(sc_of[int(b)] - cut) <= 1e-3 * max(abs(cut), scale) for b in odd):
            tie_only += 1
    ok = (sets_equal + tie_only == batch.n_req) and max_rel <= 1e-3
    return {"layer": layer, "checked_against": kind, "requests": int(batch.n_req), "sets_equal": sets_equal,
            "sets_differ_only_on_ties_within_1e-3": tie_only, "max_rel_score_diff": max_rel, "ok": bool(ok)}


# --------------------------------------------------------------------------------- tensor-parallel case

def run_tp_long(args, rank, world, local_rank, dev, barrier, *, layers, steps, warmup, allreduce):
    """Configuration 5: 8 requests of 1 048 576 tokens (8192 blocks each), Qwen2-72B-like KV shape, KV heads split over
    the ranks, the sum of the ranks' partial block scores before top-k 2048, gather of the selected K,V head slices.
    Returns the numbers as a dictionary (rank 0; None elsewhere)."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from ucmx import _native, ops
    from ucmx.engine import DecodeRetrievalEngine
    from ucmx.parallel import PeerScoreExchange, ScoreAllReduce, head_range
    W = sys.modules["ucmx_workloads"] if "ucmx_workloads" in sys.modules else load_workloads()
    shape = W.QWEN2_72B_LIKE
    batch = W.fixed_batch(8, 8192, 2048, seed=5005)
    lo, hi = head_range(shape.n_kv_heads, rank, world)
    peer = PeerScoreExchange.create(batch.total, dev) if (world > 1 and allreduce == "peer") else None
    use_graph_overlap = world == 1 or peer is not None    # selection of layer l+1 on a second stream beside layer l's block moves
    eng = DecodeRetrievalEngine(shape, batch, dev, n_layers=layers, seed=1000 + rank, heads_local=hi - lo,
                                score_reduce=ScoreAllReduce() if (world > 1 and peer is None) else None,
                                peer_exchange=peer, order=ops.ORDER_INDEX_ASC, overlap=use_graph_overlap)
    # every rank must hold the same queries' head slices of the same requests; seeds differ per rank, which is fine
    # for timing, and for the identity check below only the SUMS matter (they are formed from all ranks' parts)
    eng.make_queries()
    torch.cuda.synchronize()
    use_graph = world == 1 or peer is not None            # the NCCL route is driven call by call
    if use_graph:
        eng.capture()
    for _ in range(max(warmup, 3)):
        eng.step()
    torch.cuda.synchronize()
    barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        eng.step()
    b.record()
    torch.cuda.synchronize()
    barrier()
    ms = a.elapsed_time(b) / steps
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    # per-stage times, launched call by call with events (rank-local; the exchange wait shows up in top-k)
    eng.graph = None
    marks = []
    for l in range(eng.L):
        m = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        m[0].record()
        eng.score_layer(l)
        m[1].record()
        eng.topk_layer(l)
        m[2].record()
        eng.gather_layer(l)
        m[3].record()
        marks.append(m)
    torch.cuda.synchronize()
    med = lambda i: statistics.median(m[i].elapsed_time(m[i + 1]) * 1e3 for m in marks)  # noqa: E731
    stages = {"score_us": med(0), "topk_with_exchange_us": med(1), "gather_us": med(2)}
    # identical selections on every rank, and agreement with the library route (NCCL all-reduce between the kernels)
    identical, agree = None, None
    if world > 1:
        mine = eng.sel_ids[0].clone()
        allsel = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allsel, mine)
        identical = all(bool(torch.equal(allsel[0], s)) for s in allsel)
        part = torch.empty((batch.total,), dtype=torch.float32, device=dev)
        ops.score_dot_query(eng.rep_tables[0], eng.offsets, eng.q_dev[0], total=batch.total, slot_ids=eng.block_table,
                            n_kv_heads=eng.H, out=part)
        dist.all_reduce(part, op=dist.ReduceOp.SUM)
        idx2 = torch.full_like(mine, -1)
        cnt2 = torch.zeros((batch.n_req,), dtype=torch.int32, device=dev)
        ops.topk_ragged(part, eng.offsets, eng.k_per_req, out_stride=eng.out_stride, order=ops.ORDER_INDEX_ASC,
                        id_map=eng.block_table, out_offsets=eng.k_offsets, out_idx=idx2, out_counts=cnt2, want_scores=False)
        agree = float((torch.sort(idx2).values == torch.sort(mine).values).float().mean().item())
    err = _native.device_error()
    out = None
    if rank == 0:
        out = {"ms_per_step": ms, "us_per_layer": ms * 1e3 / eng.L, "layers": eng.L, "tp": world, "heads_per_rank": eng.H,
               "allreduce": ("fused into the scoring and top-k kernels over peer memory" if peer is not None
                             else ("nccl all_reduce between the kernels" if world > 1 else "none")),
               "cuda_graph": use_graph, "order": "block position ascending", **stages,
               "stage_times_note": "launched call by call with an event pair each: every stage time includes the host's launch "
                                   "latency (10-40 us), which the replayed step does not pay",
               "scored_tokens_per_s": eng.tokens_scored_per_step() / (ms * 1e-3),
               "gather_gbs": eng.bytes_gather_layer() / (stages["gather_us"] * 1e-6) / 1e9,
               "tp_selection_identical": identical, "agreement_with_nccl_route": agree, "device_error": err}
    del eng
    torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------------------- offload (config 4)

def run_offload(args, rank, world, local_rank, dev, barrier):
    """Configuration 4: per step and GPU, gather 4096 randomly chosen K and V blocks of one layer (2 GiB) into
    pinned host memory and scatter 4096 blocks back into randomly chosen free slots.  Device side: one
    compaction kernel per direction; host link: one DMA per direction.  Weak scaling (every GPU moves its own)."""
    import torch
    import torch.distributed as dist
    from ucmx import _native, ops
    from ucmx.store.numa import bind_to_device_node
    shape = load_workloads().LLAMA3_8B
    numa_node = bind_to_device_node(local_rank)   # before page-locking
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

    # The step in sixteen pieces on two streams: while piece c comes back over the link and is scattered, piece c+1 is
    # gathered and goes out - the link is full duplex, and the two halves of a round trip only depend on each other piece
    # by piece.  (One piece after the other on one stream takes twice as long: `serial_ms_per_step`.)
    n_pieces = 16
    per = n // n_pieces
    piece_bytes = per * 2 * shape.slice_bytes
    s_out, s_in = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    src_p = [src_ids[c * per:(c + 1) * per].contiguous() for c in range(n_pieces)]
    dst_p = [dst_ids[c * per:(c + 1) * per].contiguous() for c in range(n_pieces)]
    host_p = [host[c * piece_bytes:(c + 1) * piece_bytes] for c in range(n_pieces)]
    out_buf = [stage[i * piece_bytes:(i + 1) * piece_bytes] for i in range(2)]
    in_buf = [stage[(2 + i) * piece_bytes:(3 + i) * piece_bytes] for i in range(2)]
    left = [torch.cuda.Event() for _ in range(n_pieces)]

    def step_serial():
        ops.gather_blocks(planes, src_ids, stage)
        host.copy_(stage, non_blocking=True)
        stage.copy_(host, non_blocking=True)
        ops.scatter_blocks(planes, dst_ids, stage)

    def step():
        main = torch.cuda.current_stream(dev)
        s_out.wait_stream(main)
        s_in.wait_stream(main)
        for c in range(n_pieces):
            with torch.cuda.stream(s_out):
                ops.gather_blocks(planes, src_p[c], out_buf[c & 1])
                host_p[c].copy_(out_buf[c & 1], non_blocking=True)
                left[c].record(s_out)
            with torch.cuda.stream(s_in):
                s_in.wait_event(left[c])
                in_buf[c & 1].copy_(host_p[c], non_blocking=True)
                ops.scatter_blocks(planes, dst_p[c], in_buf[c & 1])
        main.wait_stream(s_out)
        main.wait_stream(s_in)

    def timed(fn, iters):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / iters

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    serial_ms = timed(step_serial, 2)
    # the host link's own rate in this very run, per GPU: one pinned memcpy of the payload each way
    link_d2h = payload / timed(lambda: host.copy_(stage, non_blocking=True), 2) / 1e6
    link_h2d = payload / timed(lambda: stage.copy_(host, non_blocking=True), 2) / 1e6
    sampler = ClockSampler(local_rank)
    launches_before = _native.launch_count
    sampler.start()
    barrier()
    torch.cuda.synchronize()
    sampler.begin()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        step()
    b.record()
    torch.cuda.synchronize()
    barrier()
    clocks = sampler.stop()
    ms = a.elapsed_time(b)
    link = torch.tensor([link_d2h, link_h2d], dtype=torch.float64, device=dev)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.all_reduce(link, op=dist.ReduceOp.MIN)
    exact = bool(torch.equal(kv[:, dst_ids.long()], kv[:, src_ids.long()]))
    # the reference's way on the same data: one cudaMemcpyAsync per 256 KiB slice (dramstore_connector.py:129-132)
    per_slice = None
    if rank == 0:
        hv = host.view(n, 2, shape.slice_bytes)
        ids_h = src_ids.cpu().tolist()
        kvb = kv.view(torch.uint8).view(2, n_slots, shape.slice_bytes)

        def loop():
            for j, blk in enumerate(ids_h):
                hv[j, 0].copy_(kvb[0, blk], non_blocking=True)
                hv[j, 1].copy_(kvb[1, blk], non_blocking=True)
        per_slice = payload / timed(loop, 1) / 1e6
    if rank == 0:
        gbs = 2.0 * payload * world * args.steps / (ms * 1e-3) / 1e9
        per_gpu = payload * args.steps / (ms * 1e-3) / 1e9 * 2 / 2
        link_min = float(link.min().item())
        print(json.dumps({
            "metric": "kv_block_offload_bytes_per_s", "value": gbs, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {"workload": "KV block offload: per GPU and step 4096 random K+V blocks of one Llama-3-8B layer (2 GiB) "
                                   "gathered to pinned host memory and 4096 scattered back into free slots",
                       "payload_bytes_per_direction_per_gpu": payload,
                       "route": "device compaction + DMA in sixteen pieces, the two directions on two streams (full duplex)",
                       "numa_node_of_rank0": numa_node},
            "per_gpu_gbs_each_direction": per_gpu, "roundtrip_exact": exact, "serial_ms_per_step": serial_ms,
            "roofline": {"kernel": "host link (one pinned DMA per direction after device-side compaction)", "bound": "host link",
                         "achieved": per_gpu, "peak": link_min, "peak_kind": "pinned cudaMemcpyAsync of the same payload, measured "
                         "in this run (slowest direction, slowest rank)", "unit": "GB/s", "frac": per_gpu / link_min, "traffic": None},
            "pinned_memcpy_gbs_min_over_ranks": {"d2h": float(link[0].item()), "h2d": float(link[1].item())},
            "cpu_baseline": {"value": per_slice, "unit": "GB/s", "cores": 1, "kind": "port",
                             "sample": "the reference's transfer loop on the same blocks: one cudaMemcpyAsync per 256 KiB slice "
                                       "(device to pinned host, 8192 copies)"},
            "gpu_launches": _native.launch_count - launches_before, "clocks": clocks}))


# ------------------------------------------------------------------------ single-kernel workloads

def _time_launches(fn, iters, reps=3):
    """Microseconds per launch: launches queued behind a busy GPU, best of `reps`."""
    import torch
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


def run_kernel_workload(args, dev):
    """score | hamming | hash | pool | gsa | kvstar | connector | filestore: one kernel (or one call path) of the other benchmark
    configurations, timed alone on inputs larger than L2 (or rotated over several tables)."""
    import numpy as np
    import torch
    from ucmx import _native, ops
    W = load_workloads()
    shape = W.LLAMA3_8B
    batch = W.ragged_decode_batch(seed=3003)
    g = torch.Generator(device=dev).manual_seed(3003)
    off = torch.from_numpy(batch.offsets).to(dev)
    table = torch.from_numpy(batch.block_table).to(dev)
    T, H, D = shape.block_tokens, shape.n_kv_heads, shape.head_dim
    peak, peak_kind = measured_peaks()
    name = args.workload
    launches_before = _native.launch_count
    line = {"n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "data": "synthetic"}

    def roofline(kernel, nbytes, us):
        gbs = nbytes / us / 1e3
        return {"kernel": kernel, "bound": "hbm", "achieved": gbs, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                "frac": gbs / peak, "traffic": None, "algorithmic_bytes_per_launch": nbytes, "avg_launch_us": us}

    if name == "hamming":
        n_tables = 3                                             # 3 x 547 MB rotate through L2
        codes = [torch.randint(0, 256, (batch.n_slots, H, T, 16), generator=g, device=dev, dtype=torch.uint8)
                 for _ in range(n_tables)]
        qc = torch.randint(0, 256, (batch.n_req, H, 16), generator=g, device=dev, dtype=torch.uint8)
        scores = torch.empty((batch.total,), dtype=torch.int32, device=dev)
        nbytes = batch.total * (H * T * 16 + 8)
        res = {}
        for key, cross in (("cross_head", True), ("matched_head", False)):
            res[key] = _time_launches(lambda i: ops.score_hamming(codes[i % n_tables], off, qc, total=batch.total, slot_ids=table,
                                                                  cross_head=cross, out=scores), iters=6)
        line.update(metric="hamming_scored_kv_tokens_per_s", unit=UNIT, value=batch.total * T / (res["cross_head"] * 1e-6),
                    ms_per_step=res["cross_head"] * 1e-3, dtype="u32",
                    config={"workload": "KVComp Hamming scoring, the 64-request ragged batch, 128-bit codes, 16 KiB per block, "
                                        "every (query head, key head) pair as the reference's einsum sums them",
                            "blocks": int(batch.total), "l2_policy": "three 547 MB code tables in rotation"},
                    roofline=roofline("score_hamming_kernel<all pairs>", nbytes, res["cross_head"]),
                    matched_head={"us": res["matched_head"], "gbs": nbytes / res["matched_head"] / 1e3,
                                  "frac": nbytes / res["matched_head"] / 1e3 / peak})
    elif name == "hash":
        nb = 2048
        k = torch.randn((nb, T, H, D), generator=g, device=dev).to(torch.bfloat16)
        w = (torch.randn((D, 128), generator=g, device=dev) * 2).to(torch.bfloat16)
        ids = torch.randperm(nb, generator=g, device=dev).to(torch.int32)
        codes = torch.empty((nb, H, T, 16), dtype=torch.uint8, device=dev)
        us = _time_launches(lambda i: ops.hash_encode_blocks(k, ids, w, out=codes), iters=4)
        nbytes = nb * (T * H * D * 2 + T * H * 16)
        line.update(metric="hash_encoded_kv_tokens_per_s", unit=UNIT, value=nb * T / (us * 1e-6), ms_per_step=us * 1e-3,
                    dtype="bf16 x bf16 -> fp32 sign bits",
                    config={"workload": "KVComp sign-hash codes of 2048 paged key blocks (0.5 GiB), 128 bits per token and head",
                            "blocks": nb, "l2_policy": "input larger than L2"},
                    roofline=roofline("hash_encode_tc_kernel", nbytes, us), tflops=nb * T * H * 2.0 * D * 128 / us / 1e6)
    elif name == "pool":
        nb = 8192                                                # 2 GiB of K
        k = torch.empty((nb, T, H, D), dtype=torch.bfloat16, device=dev)
        for s in range(0, nb, 1024):
            k[s:s + 1024].copy_(torch.randn((1024, T, H, D), generator=g, device=dev).to(torch.bfloat16))
        reps = torch.empty((nb, H, 1, D), dtype=torch.bfloat16, device=dev)
        ids = torch.randperm(nb, generator=g, device=dev).to(torch.int32)
        res = {m: _time_launches(lambda i: ops.pool_blocks(k, ids, mode=m, out_slots=ids, out_bf16=reps), iters=4)
               for m in ("mean", "max")}
        sets = [ids[i * 64:(i + 1) * 64].contiguous() for i in range(16)]
        small = _time_launches(lambda i: ops.pool_blocks(k, sets[i % 16], out_slots=sets[i % 16], out_bf16=reps), iters=16)
        nbytes = nb * (shape.slice_bytes + 2048)
        line.update(metric="pooled_kv_tokens_per_s", unit=UNIT, value=nb * T / (res["mean"] * 1e-6), ms_per_step=res["mean"] * 1e-3,
                    dtype="bf16", config={"workload": "mean pooling of a whole pool of 8192 key blocks (2 GiB)", "blocks": nb,
                                          "l2_policy": "input larger than L2"},
                    roofline=roofline("pool_blocks_kernel<mean>", nbytes, res["mean"]),
                    max_pooling={"us": res["max"], "gbs": nbytes / res["max"] / 1e3},
                    decode_64_blocks={"us": small, "gbs": 64 * (shape.slice_bytes + 2048) / small / 1e3})
    elif name == "score":
        # the headline batch's scoring kernel on its own: 33 391 rows of 2 KiB per launch out of three tables in rotation
        # (a launch reads 68 MB; the next launch's table is not in L2), with the query mean folded in and with fp32 queries
        n_tables = 3
        reps = [(torch.randn((batch.n_slots, H, 1, D), generator=g, device=dev) * 0.0884).to(torch.bfloat16) for _ in range(n_tables)]
        q = torch.randn((batch.n_req, shape.n_q_heads, D), generator=g, device=dev).to(torch.bfloat16)
        qbar = ops.query_group_mean(q, H)
        scores = torch.empty((batch.total,), dtype=torch.float32, device=dev)
        nbytes = batch.total * (H * D * 2 + 8)

        def graph_us(fn, n=24):
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                fn(0)
            torch.cuda.current_stream(dev).wait_stream(side)
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                for i in range(n):
                    fn(i)
            best = float("inf")
            for _ in range(5):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                gr.replay()
                b.record()
                torch.cuda.synchronize()
                best = min(best, a.elapsed_time(b) * 1e3 / n)
            return best

        def fused(early):
            return lambda i: ops.score_dot_query(reps[i % n_tables], off, q, total=batch.total, slot_ids=table, n_kv_heads=H,
                                                 out=scores, early=early and i > 0)

        def f32q(early):
            return lambda i: ops.score_dot(reps[i % n_tables], off, qbar, total=batch.total, slot_ids=table, n_kv_heads=H,
                                           head_dim=D, out=scores, early=early and i > 0)

        # every launch after the first one of a graph begins under the tail of the launch ahead (it reads its inputs
        # at once and waits for that launch's end before its first store), as the scoring of layer l+1 does behind
        # layer l's top-k inside a step; `serial` is the same graph with plain launches
        us_fused, us_f32q = graph_us(fused(True)), graph_us(f32q(True))
        us_fused_serial, us_f32q_serial = graph_us(fused(False)), graph_us(f32q(False))
        line.update(metric="scored_kv_tokens_per_s", unit=UNIT, value=batch.total * T / (us_fused * 1e-6), ms_per_step=us_fused * 1e-3,
                    dtype="bf16", config={"workload": "dot scoring of the 64-request ragged batch, one launch per graph node, "
                                                      "each launch allowed to begin under the tail of the one ahead",
                                          "blocks": int(batch.total), "l2_policy": "three 73 MB tables in rotation"},
                    roofline=roofline("score_dot_ring_kernel<bf16, 32, query mean folded in>", nbytes, us_fused),
                    fp32_queries={"kernel": "score_dot_ring_kernel<bf16, 32>", "us": us_f32q, "gbs": nbytes / us_f32q / 1e3,
                                  "frac": nbytes / us_f32q / 1e3 / peak},
                    serial={"us": us_fused_serial, "frac": nbytes / us_fused_serial / 1e3 / peak,
                            "fp32_queries_us": us_f32q_serial, "fp32_queries_frac": nbytes / us_f32q_serial / 1e3 / peak})
    elif name == "gsa":
        # GSA's two scoring forms on the 64-request batch with two representatives per head (config 1's pooling, at
        # config 2's size): sum over heads of the best representative's dot product (host-side SelectTopKBS semantics,
        # the row-ring kernel with the maximum over representatives in its reduction) and the device-side block weights of
        # gsa.py:386-412 (score_dot_heads_rows_kernel)
        R = 2
        n_tables = 3
        reps = [(torch.randn((batch.n_slots, H, R, D), generator=g, device=dev) * 0.0884).to(torch.bfloat16) for _ in range(n_tables)]
        q = torch.randn((batch.n_req, shape.n_q_heads, D), generator=g, device=dev).to(torch.bfloat16)
        qbar = ops.query_group_mean(q, H)
        scores = torch.empty((batch.total,), dtype=torch.float32, device=dev)
        nbytes = batch.total * (H * R * D * 2 + 8)
        us_gen = _time_launches(lambda i: ops.score_dot(reps[i % n_tables], off, qbar, total=batch.total, slot_ids=table,
                                                        n_kv_heads=H, head_dim=D, n_rep=R, out=scores), iters=12)
        us_heads = _time_launches(lambda i: ops.score_dot_heads(reps[i % n_tables], off, q, total=batch.total, slot_ids=table,
                                                                out=scores), iters=12)
        line.update(metric="gsa_scored_kv_tokens_per_s", unit=UNIT, value=batch.total * T / (us_gen * 1e-6), ms_per_step=us_gen * 1e-3,
                    dtype="bf16", config={"workload": "GSA scoring with two representatives per head, the 64-request ragged batch",
                                          "blocks": int(batch.total), "l2_policy": "three 137 MB tables in rotation"},
                    roofline=roofline("score_dot_ring_kernel<bf16, 4 KiB rows, 2 representatives per head>", nbytes, us_gen),
                    per_head_weights={"kernel": "score_dot_heads_rows_kernel<8 loads, 2 representatives, 4 query heads per KV head>", "us": us_heads, "gbs": nbytes / us_heads / 1e3,
                                      "frac": nbytes / us_heads / 1e3 / peak})
    elif name == "kvstar":
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
        us = _time_launches(lambda i: ops.kvstar_scores(reps, off, q, qoff, total=nb, max_q_tokens=xq, slot_ids=table,
                                                        pruned_index=pr, workspace=ws, out=votes), iters=4)
        nbytes = nb * (Mp * H * dp * 2 + 4)
        line.update(metric="kvstar_voted_blocks_per_s", unit="blocks/s", value=nb / (us * 1e-6), ms_per_step=us * 1e-3, dtype="f16",
                    config={"workload": "KVStar softmax-vote scoring, the 64-request ragged batch, 8 query tokens x 32 heads per "
                                        "request, fp16 representations of 64 positions x 8 heads x 32 kept channels per block",
                            "blocks": int(nb), "l2_policy": "1.2 GB of representations per launch"},
                    roofline=roofline("kvstar partial (tcgen05) + stats + vote kernels", nbytes, us),
                    tflops_useful=2.0 * xq * Hq * dp * Mp * nb / us / 1e6)
    elif name == "connector":
        line.update(_connector_case(dev, g, shape))
    elif name == "filestore":
        line.update(_filestore_case(dev, g, shape))
    line["gpu_launches"] = _native.launch_count - launches_before
    line["device_error"] = _native.device_error()
    print(json.dumps(line))


def _connector_case(dev, g, shape):
    """Prefix-cache dump and load of 256 blocks x 32 layers (4 GiB) through the host-memory store: one address table
    per layer against the reference's call pattern (one dump per block, layer and K/V with a tensor view; one K and
    one V load per request and layer).  Wall clock."""
    import types

    import torch
    from ucmx.connector import ReqMeta, UCConnectorV1Metadata, UnifiedCacheConnectorV1
    T, H, D = shape.block_tokens, shape.n_kv_heads, shape.head_dim
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
    res = {}
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
    ours, ref = res["table_per_layer"], res["reference_call_pattern"]
    return {"metric": "prefix_cache_dump_bytes_per_s", "unit": "GB/s", "value": ours["dump_gbs"], "ms_per_step": ours["dump_ms"],
            "dtype": "u8", "config": {"workload": "connector dump + load of 256 blocks x 32 layers (4 GiB) through the host-memory "
                                                  "store, one address table per layer", "bytes": nbytes},
            "load_gbs": ours["load_gbs"], "ok": ours["ok"],
            "roofline": {"kernel": "xfer_plain_kernel over the host link", "bound": "host link", "achieved": ours["dump_gbs"],
                         "peak": None, "unit": "GB/s", "frac": None, "traffic": None},
            "cpu_baseline": {"value": ref["dump_gbs"], "unit": "GB/s", "cores": 1, "kind": "port",
                             "sample": "the reference's call pattern on the same store: one dump per block, layer and K/V",
                             "load_gbs": ref["load_gbs"]}}


def _filestore_case(dev, g, shape):
    """File-per-block store: dump 256 blocks x 16 K/V layer slices of 256 KiB (1 GiB) from HBM to block files under
    $UCMX_STORE_DIR (default: the temp dir) and load them back; wall clock, bounded by that file system; also with
    one slice per launch (the reference's granularity)."""
    import shutil

    import numpy as np
    import torch
    from ucmx.store.nfsstore import UcmNfsStore
    nblk, nsl = 256, 16
    sl = shape.slice_bytes
    cache = torch.empty((nblk * nsl, sl), dtype=torch.uint8, device=dev)
    cache.random_(0, 256, generator=g)
    back = torch.zeros_like(cache)
    rng = np.random.default_rng(4004)
    ids = [rng.integers(1, 256, size=32, dtype=np.uint8).tobytes() for _ in range(nblk)]
    bl = [b for b in ids for _ in range(nsl)]
    offs = [j * sl for _ in ids for j in range(nsl)]
    nbytes = nblk * nsl * sl
    res = {}
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
            res[name] = {"dump_gbs": nbytes / (t1 - t0) / 1e9, "load_gbs": nbytes / (t3 - t2) / 1e9,
                         "status": [st_d, st_l], "exact": bool(torch.equal(back, cache))}
            back.zero_()
            store.close()
        finally:
            shutil.rmtree(root, ignore_errors=True)
    ours, ref = res["grouped"], res["one_slice_per_launch"]
    return {"metric": "block_file_dump_bytes_per_s", "unit": "GB/s", "value": ours["dump_gbs"], "ms_per_step": nbytes / ours["dump_gbs"] / 1e6,
            "dtype": "u8", "config": {"workload": "file-per-block store: 256 blocks x 16 slices of 256 KiB (1 GiB) HBM -> files -> HBM",
                                      "bytes": nbytes, "directory": os.environ.get("UCMX_STORE_DIR") or tempfile.gettempdir()},
            "load_gbs": ours["load_gbs"], "exact": ours["exact"], "status": ours["status"],
            "roofline": {"kernel": "file system + host link", "bound": "file system", "achieved": ours["dump_gbs"], "peak": None,
                         "unit": "GB/s", "frac": None, "traffic": None},
            "cpu_baseline": {"value": ref["dump_gbs"], "unit": "GB/s", "cores": 8, "kind": "port",
                             "sample": "one slice per launch, the reference's granularity", "load_gbs": ref["load_gbs"]}}


# ----------------------------------------------------------------------------------------- our arm

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="launch the step call by call instead of replaying its CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="headline numbers only: no parity check, plug-in timing or tp_long object")
    ap.add_argument("--layers", type=int, default=None, help=argparse.SUPPRESS)
    ap.add_argument("--workload", default="decode64",
                    choices=["decode64", "decode64-delta", "tp-long", "offload", "score", "hamming", "hash", "pool", "gsa", "kvstar",
                             "connector", "filestore"],
                    help="decode64: the 64-request ragged decode batch, data parallel over requests (default); "
                         "decode64-delta: the same batch with a resident working set per request and layer - queries drift "
                         "from step to step and only the newly selected blocks are moved; "
                         "tp-long: 8 requests of 1 048 576 tokens, KV heads split over the GPUs with the sum of block scores "
                         "over ranks before top-k; offload: every GPU moves 4096 random K+V blocks of one layer (2 GiB) to "
                         "pinned host memory and 4096 back into free slots per step; the rest time one kernel or call path "
                         "of the other configurations on one GPU")
    ap.add_argument("--allreduce", default="peer", choices=["nccl", "peer"],
                    help="tp-long only: how partial block scores are summed over ranks - inside the scoring and top-k "
                         "kernels over peer memory, or a NCCL all-reduce between them")
    ap.add_argument("--profile-case", action="store_true",
                    help="small case for profiler captures: 8 requests, 2 layers, 1 warm-up + 1 step, no host legs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = env_int("RANK", 0)
    world = env_int("WORLD_SIZE", 1)
    local_rank = env_int("LOCAL_RANK", 0)

    if args.impl == "reference":
        run_reference(args, rank)
        return

    use_package()
    import torch
    import torch.distributed as dist
    from ucmx import _native, ops
    from ucmx.engine import DecodeRetrievalEngine
    W = load_workloads()

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

    def finish():
        if world > 1:
            dist.destroy_process_group()

    if args.workload == "offload":
        run_offload(args, rank, world, local_rank, dev, barrier)
        return finish()
    if args.workload in ("score", "hamming", "hash", "pool", "gsa", "kvstar", "connector", "filestore"):
        if rank == 0:
            run_kernel_workload(args, dev)
        return finish()
    if args.workload == "tp-long":
        layers = args.layers or 16
        res = run_tp_long(args, rank, world, local_rank, dev, barrier, layers=layers, steps=args.steps, warmup=args.warmup,
                          allreduce=args.allreduce)
        if rank == 0:
            peak, peak_kind = measured_peaks()
            gather_bytes = res["gather_gbs"] * 1e9 * res["gather_us"] * 1e-6          # per rank and layer
            layer_gbs = gather_bytes / (res["us_per_layer"] * 1e-6) / 1e9
            roofline = {"kernel": "xfer_bulk_kernel (gather of the selected K,V head slices, one layer, one rank)", "bound": "hbm",
                        "achieved": layer_gbs, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": layer_gbs / peak,
                        "traffic": None, "algorithmic_bytes_per_launch": gather_bytes,
                        "note": "a lower bound: the gather's bytes over the WHOLE layer time of the replayed step (scoring, exchange "
                                "and top-k of the next layer run beside the gather on a second stream)"}
            print(json.dumps({
                "roofline": roofline,
                "metric": METRIC, "value": res["scored_tokens_per_s"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": "long-context sharded retrieval: 8 requests x 1 048 576 tokens (8192 blocks each), Qwen2-72B-like "
                                       "KV (64q/8kv heads, head_dim 128), KV heads split over the GPUs, sum of 65 536 fp32 block "
                                       "scores over ranks before top-k 2048, gather of the selected K,V head slices",
                           "layers": layers, "parallelism": f"tp{world} over KV heads", "l2_policy": "inputs larger than L2 per step"},
                "tp_long": res, "device_error": res["device_error"]}))
        return finish()

    # ------------------------------------------------------------------ decode64 and decode64-delta
    delta = args.workload == "decode64-delta"
    n_req = 64
    if args.layers is None:
        args.layers = 32
    if args.profile_case:
        args.layers, args.steps, args.warmup, args.no_cpu_baseline, args.no_extras, n_req = 2, 1, 1, True, True, 8
    shape = W.LLAMA3_8B
    # weak scaling: every rank serves requests of the same lengths (the same work per GPU) over its own block
    # table, keys and queries
    batch = W.ragged_decode_batch(seed=2002, n_req=n_req, table_seed=None if rank == 0 else 7007 + rank)
    eng = DecodeRetrievalEngine(shape, batch, dev, n_layers=args.layers, seed=1000 + rank, delta=delta, overlap=True)
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

    # The step is replayed from a CUDA graph unless --no-graph.  The gather launches are timed by events around
    # them.  An event record costs several microseconds of stream time, call by call and as a graph node alike, so
    # in graph mode the last of the K timed steps replays a second graph that has an event pair around each of its
    # gathers and the other K-1 replay the plain one; call by call, every fourth gather launch carries a pair.
    use_graph = not args.no_graph and not args.profile_case
    timed_graph = None
    if use_graph:
        gev = [(torch.cuda.Event(enable_timing=True, external=True), torch.cuda.Event(enable_timing=True, external=True))
               for _ in range(eng.L)]
        timed_graph = eng.capture(gather_events=gev)
        eng.capture()
        timed_graph.replay()

    def one_step():
        if delta:
            eng.drift_queries()            # the next decode step's queries (device-side, part of the step's input)
        eng.step()

    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(args.warmup):
        one_step()
    torch.cuda.synchronize()

    # ---- timed region: K steps, device-resident inputs; the gather launches carry their own events
    every = 1 if args.profile_case else 4
    if not use_graph:
        gev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
               for _ in range(args.steps * ((eng.L + every - 1) // every))]
    launches_before = _native.launch_count
    loads = []
    barrier()
    torch.cuda.synchronize()
    sampler.begin()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    if use_graph:
        for _ in range(args.steps - 1):
            one_step()
        if delta:
            eng.drift_queries()
        timed_graph.replay()
    else:
        gi = 0
        for _ in range(args.steps):
            if delta:
                eng.drift_queries()
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
    tokens_per_step_all = float(eng.tokens_scored_per_step())
    if world > 1:
        tt = torch.tensor([tokens_per_step_all], dtype=torch.float64, device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.SUM)
        tokens_per_step_all = float(tt.item())
    value = tokens_per_step_all / (ms_per_step * 1e-3)
    gather_ms = [a.elapsed_time(b) for a, b in gev]
    gather_avg_ms = statistics.fmean(gather_ms) if gather_ms else None
    if delta:
        loads.append(eng.loads_of_last_step())

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

    # ---- score + top-k alone as graph nodes: no event records between the kernels
    retrieval_graph_us = None
    if not args.profile_case:
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            eng.score_layer(0)
            eng.topk_layer(0)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for l in range(eng.L):
                eng.score_layer(l, early=l > 0 and not eng.exchanges_scores)   # under the previous layer's top-k
                eng.topk_layer(l)
        best = float("inf")
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            gr.replay()
            b.record()
            torch.cuda.synchronize()
            best = min(best, a.elapsed_time(b) * 1e3 / eng.L)
        retrieval_graph_us = best
        del gr

    peak, peak_kind = measured_peaks()
    roofline = None
    moved_bytes = eng.bytes_gather_layer()
    if delta and loads:
        moved_bytes = 2 * 2 * eng.T * eng.H * eng.D * 2 * loads[-1] / eng.L      # K and V, read + write, per layer
    if gather_avg_ms:
        achieved = moved_bytes / (gather_avg_ms * 1e-3) / 1e9
        roofline = {"kernel": ("remap_resident_kernel + xfer_bulk_kernel (delta load of one layer)" if delta
                               else "xfer_bulk_kernel (gather of selected K,V blocks, one layer)"), "bound": "hbm",
                    "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                    "traffic": None if delta else moved_bytes - GATHER_L2_DIRTY_RESIDUE_BYTES,
                    "traffic_source": None if delta else GATHER_TRAFFIC_SOURCE,
                    "algorithmic_bytes_per_launch": moved_bytes, "avg_launch_us": gather_avg_ms * 1e3,
                    "launches_timed": len(gather_ms)}
        if eng.overlap and not delta:
            roofline["note"] = ("timed inside the step, where the next layer's scoring and top-k run beside the gather on a "
                                "second stream and share HBM with it; alone (stages_us_per_layer.gather) a launch takes "
                                f"{stages_us['gather']:.1f} us = {moved_bytes / (stages_us['gather'] * 1e-6) / 1e9 / peak:.3f} of the peak")
    stage_gbs = {
        "score": eng.bytes_score_layer() / (stages_us["score"] * 1e-6) / 1e9,
        "gather": moved_bytes / (stages_us["gather"] * 1e-6) / 1e9,
        "pool_decode": eng.bytes_pool_layer() / (stages_us["pool"] * 1e-6) / 1e9,
        "pool_prefill": prefill_gbs,
    }
    if retrieval_graph_us:
        stage_gbs["score_plus_topk_as_graph_nodes"] = eng.bytes_score_layer() / (retrieval_graph_us * 1e-6) / 1e9

    extras = not args.no_extras and not args.profile_case
    parity = None
    if extras and not delta and rank == 0:
        try:
            parity = parity_at_bench_config(eng, batch, layer=min(5, eng.L - 1))
        except Exception as exc:
            parity = {"ok": False, "error": str(exc)}

    # ---- the whole step end to end with host buffers (queries in, selected ids out)
    e2e_full = None
    if not args.profile_case and not delta:
        eng.graph = None
        eng.alloc_host()
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
        e2e_full = {"value": tokens_per_step_all / e2e_s, "unit": UNIT, "ms_per_step": e2e_s * 1e3,
                    "h2d_bytes_per_step": eng.h2d_bytes_per_step, "d2h_bytes_per_step": eng.d2h_bytes_per_step,
                    "what": "pool + score + top-k + gather, queries from pinned host memory, selected ids back to it, "
                            "both streams replayed from one CUDA graph"}
    h2d_full, d2h_full = eng.h2d_bytes_per_step, eng.d2h_bytes_per_step
    L_eng = eng.L
    launches_per_step = eng.launches_per_step
    tokens_one_rank = float(eng.tokens_scored_per_step())
    del eng, timed_graph
    torch.cuda.empty_cache()

    # ---- end to end through the reference's own object: host arrays in, host arrays out, one submit per request
    e2e = None
    e2e_plugin = None
    cpu_baseline = None
    ref_backends = None
    if not args.profile_case and not delta:
        from ucmx.retrieval import RetrievalWorkerBackend
        plug = plugin_inputs(batch, L_eng)
        tables, queries, slot_lists, ks = plug
        backends = [RetrievalWorkerBackend(t, device=local_rank, table_dtype="bf16") for t in tables]
        launches0 = sum(b.launches for b in backends)
        barrier()
        dt = time_plugin(backends, queries, slot_lists, ks, L_eng, args.steps, 2)
        plugin_launches = sum(b.launches for b in backends) - launches0
        if world > 1:
            t = torch.tensor([dt], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        idx_bytes = sum(s.nbytes for s in slot_lists)
        e2e = {"value": tokens_per_step_all / dt, "unit": UNIT, "ms_per_step": dt * 1e3,
               "h2d_bytes_per_step": L_eng * (batch.n_req * 4096 + idx_bytes + 3 * 4 * (batch.n_req + 1)),
               "d2h_bytes_per_step": L_eng * (4 * batch.n_req + 8 * batch.total_k),
               "path": "ucmx.retrieval.RetrievalWorkerBackend over ucmx_retrieval_*: numpy query and slot list in, numpy "
                       "indices and scores out; per layer one submit per request, then wait + get_result for each "
                       "(score + top-k, the work the reference's object does)",
               "gpu_launches_per_step": plugin_launches // (args.steps + 2)}
        padded = padded_index_matrix(slot_lists)
        plugin_layer_pass_batched(backends, queries, padded, max(ks), L_eng)
        t0 = time.perf_counter()
        for _ in range(3):
            plugin_layer_pass_batched(backends, queries, padded, max(ks), L_eng)
        dtb = (time.perf_counter() - t0) / 3
        e2e_plugin = {"per_request_submit_ms_per_layer": dt * 1e3 / L_eng, "batched_submit_ms_per_layer": dtb * 1e3 / L_eng}
        if rank == 0 and world == 1 and not args.no_cpu_baseline:
            try:
                cpu_baseline, ref_backends = reference_baseline(batch, plug)
                if cpu_baseline.get("ms_per_layer"):
                    e2e_plugin["reference_per_request_submit_ms_per_layer"] = cpu_baseline["ms_per_layer"]
                    e2e_plugin["reference_batched_submit_ms_per_layer"] = cpu_baseline["ms_per_layer_one_batched_submit"]
            except Exception as exc:  # the baseline must never take the benchmark down
                cpu_baseline = {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "reference",
                                "sample": f"failed: {exc}"}
        for b in backends:
            b.close()
        del backends, ref_backends
        torch.cuda.empty_cache()

    retrieval_only = None
    if retrieval_graph_us:
        retrieval_only = {"ours_us_per_layer": retrieval_graph_us,
                          "ours": "score + top-k of all 64 requests as two graph nodes per layer, inputs resident",
                          "reference_us_per_layer": (cpu_baseline["ms_per_layer"] * 1e3
                                                     if cpu_baseline and cpu_baseline.get("ms_per_layer") else None)}

    legs = cpu_baseline_legs() if (extras and rank == 0 and world == 1 and not args.no_cpu_baseline and not delta) else None

    # ---- the tensor-parallel case beside it
    tp_long = None
    if extras and not delta:
        tp_steps, tp_layers = min(args.steps, 10), 16
        if world > 1:
            tp_long = run_tp_long(args, rank, world, local_rank, dev, barrier, layers=tp_layers, steps=tp_steps, warmup=3,
                                  allreduce="peer")
            nccl = run_tp_long(args, rank, world, local_rank, dev, barrier, layers=tp_layers, steps=tp_steps, warmup=3,
                               allreduce="nccl")
            if rank == 0:
                tp_long["nccl_route"] = {k: nccl[k] for k in ("ms_per_step", "score_us", "topk_with_exchange_us", "gather_us")}
        # the single-rank time of the same batch: rank 0 alone (the others wait at the barrier below)
        if rank == 0:
            solo = run_tp_long(args, 0, 1, local_rank, dev, lambda: None, layers=tp_layers, steps=min(tp_steps, 5), warmup=3,
                               allreduce="none")
            if tp_long is None:
                tp_long = solo
            else:
                tp_long["tp1_ms_per_step"] = solo["ms_per_step"]
                tp_long["strong_efficiency_vs_tp1"] = solo["ms_per_step"] / (tp_long["ms_per_step"] * world)
        barrier()

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": workload_config(batch),
            "cuda_graph": use_graph,
            "schedule": "score + top-k of layer l+1 on a second stream beside the block moves of layer l (same graph)",
            "stages": ("pool(64 new blocks of each of the 32 layers, one launch per step) + per layer score + top-k + "
                       + ("remap + move of newly selected K,V blocks" if delta else "gather(K,V of selected)")),
            "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"],
                       "samples": clocks["samples"]},
            "e2e": e2e if e2e is not None else e2e_full,
            "e2e_full_step": e2e_full,
            "e2e_plugin": e2e_plugin,
            "gpu_launches": int(launches),
            "roofline": roofline,
            "cpu_baseline": cpu_baseline,
            "cpu_baseline_legs": legs,
            "retrieval_only": retrieval_only,
            "parity_at_bench_config": parity,
            "stages_us_per_layer": stages_us,
            "retrieval_us_per_layer": retrieval_us,
            "retrieval_us_per_layer_note": "pool + score + top-k of the instrumented pass; each stage carries an event pair "
                                           "(several microseconds); retrieval_only.ours_us_per_layer has none",
            "stage_gbs": stage_gbs,
            "tp_long": tp_long,
            "device_error": _native.device_error(),
        }
        if delta:
            line["config"] = dict(line["config"], workload=line["config"]["workload"] + "; resident working set per request and "
                                  "layer, queries drift as a random walk (rho 0.98), only newly selected blocks are moved")
            line["delta"] = {"selected_per_layer": int(batch.total_k), "loaded_per_layer": loads[-1] / L_eng,
                             "hit_rate": 1.0 - loads[-1] / (L_eng * batch.total_k), "us_per_layer": ms_per_step * 1e3 / L_eng,
                             "target_us_per_layer": 150.0, "bytes_moved_per_layer": moved_bytes}
        if parity is not None and not parity.get("ok", False):
            print(json.dumps(line))
            finish()
            raise SystemExit("parity_at_bench_config failed: " + json.dumps(parity))
        print(json.dumps(line))
    finish()


if __name__ == "__main__":
    main()
