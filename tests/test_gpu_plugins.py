"""The reference-facing layers on the GPU: the DRAM store (mirrors the cases of the reference's
test/test_ucm_dram.py), HashEncoder, and the ESA / KvComp / GSA / KVStar plug-ins driven through the
UcmSparseBase hooks by a miniature model runner, each checked against the CPU checker."""
import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev_bf16(u16):
    return torch.from_numpy(np.ascontiguousarray(u16).view(np.int16)).to(DEV).view(torch.bfloat16)


def bits(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


# ----------------------------------------------------------------------------------- DRAM store

@pytest.fixture()
def dram():
    from ucmx.store.factory import UcmConnectorFactory
    st = UcmConnectorFactory.create_connector("UcmDramStore", {"role": "worker", "max_cache_size": 64 * 4096,
                                                               "kv_block_size": 4096, "device": DEV})
    yield st
    st.close()


def test_dram_dump_then_load_roundtrip(dram):
    hashes = [f"h{i}" for i in range(6)]
    src = [torch.randint(0, 100, (4096,), dtype=torch.int8, device=DEV) for _ in hashes]
    offsets = list(range(6))
    t = dram.dump(hashes, offsets, src)
    assert dram.check(t)[0] == 0
    assert dram.wait(t) == 0
    for i, h in enumerate(hashes):            # dump_success: the cached bytes are the source bytes
        assert np.array_equal(dram.slab_view(dram.slot_of[f"{h}_{offsets[i]}"]), src[i].cpu().numpy().view(np.uint8))
    dst = [torch.zeros(4096, dtype=torch.int8, device=DEV) for _ in hashes]
    t = dram.load(hashes, offsets, dst)
    assert dram.wait(t) == 0
    assert dram.check(t) == (0, True)
    for a, b in zip(src, dst):                # load_success
        assert torch.equal(a, b)
    # overwrite in place keeps the slot
    slot = dram.slot_of["h0_0"]
    assert dram.wait(dram.dump(["h0"], [0], [src[3]])) == 0 and dram.slot_of["h0_0"] == slot
    # raw-address forms
    d2 = torch.zeros(4096, dtype=torch.int8, device=DEV)
    assert dram.wait(dram.fetch_data(["h0"], [0], [d2.data_ptr()], [4096])) == 0 and torch.equal(d2, src[3])
    assert dram.wait(dram.dump_data(["raw"], [7], [src[5].data_ptr()], [4096])) == 0
    d3 = torch.zeros(4096, dtype=torch.int8, device=DEV)
    assert dram.wait(dram.load(["raw"], [7], [d3])) == 0 and torch.equal(d3, src[5])


def test_dram_lookup_commit_and_failures(dram):
    from ucmx.store.dramstore import DramTask
    assert dram.lookup(["a", "b"]) == [False, False]
    dram.commit(["a"])
    assert dram.lookup(["a", "b"]) == [True, False]
    assert dram.create(["x", "y"]) == [0, 0]
    assert dram.wait(DramTask()) == -1                       # a task nothing was recorded on
    with pytest.raises(KeyError):
        dram.load(["never"], [0], [torch.zeros(4096, dtype=torch.int8, device=DEV)])
    # the cache holds 64 slices: the 65th dump fails in wait(), as a full reference cache does
    big = [torch.zeros(4096, dtype=torch.int8, device=DEV) for _ in range(64)]
    assert dram.wait(dram.dump([f"f{i}" for i in range(64)], [0] * 64, big)) == 0
    t = dram.dump(["one_more"], [0], [big[0]])
    assert t.task_id == "-1" and dram.wait(t) == -1


def test_hash_encoder_interface(oracle):
    from ucmx.hash_encoder import HashEncoder
    w, q, keys = H.case_hash()
    enc = HashEncoder(128, 128, torch.bfloat16, torch.device(DEV))
    enc.set_hash_weight(dev_bf16(w))
    codes = enc.compute_hash(dev_bf16(keys))
    assert codes.shape == (7, 16, 8, 16) and codes.dtype == torch.uint8
    assert np.array_equal(codes.cpu().numpy(), oracle.hash_encode(keys, w))
    un = enc._unpack_hash(codes)
    ref = np.unpackbits(codes.cpu().numpy(), axis=-1, bitorder="little").astype(np.float32) * 2 - 1
    assert un.dtype == torch.float16 and np.array_equal(un.float().cpu().numpy(), ref)
    with pytest.raises(ValueError):
        enc.compute_hash(torch.zeros((2, 64), dtype=torch.bfloat16, device=DEV))
    with pytest.raises(ValueError):
        enc.set_hash_weight(torch.zeros((128, 64), dtype=torch.bfloat16, device=DEV))


# --------------------------------------------------------------------------- miniature model runner

T, HKV, HQ, D, LAYERS, NBLK = 16, 2, 8, 64, 2, 96


def make_config(method, cfg, store):
    model = SimpleNamespace(max_model_len=1024, hf_config=SimpleNamespace(num_hidden_layers=LAYERS),
                            get_num_kv_heads=lambda pc: HKV, get_head_size=lambda: D)
    return SimpleNamespace(
        parallel_config=SimpleNamespace(rank=0, tensor_parallel_size=1),
        cache_config=SimpleNamespace(block_size=T), model_config=model,
        scheduler_config=SimpleNamespace(max_num_seqs=4),
        kv_transfer_config=SimpleNamespace(kv_connector_extra_config={"ucm_sparse_config": {method: cfg}}),
        ucm_store=store)


class Runner:
    """Holds per-layer paged KV caches and calls the plug-in's hooks in the order the patched engine does."""

    def __init__(self, sparse, seed):
        self.sparse = sparse
        rng = np.random.default_rng(seed)
        self.kv_host = [H.randn_bf16(rng, (2, NBLK, T, HKV, D)) for _ in range(LAYERS)]
        self.kv = [dev_bf16(a) for a in self.kv_host]
        self.layer_names = [f"model.layers.{l}.self_attn.attn" for l in range(LAYERS)]
        self.fc = SimpleNamespace(virtual_engine=0, attn_metadata=SimpleNamespace(block_table=None, seq_lens=None),
                                  no_compile_layers={n: SimpleNamespace(kv_cache=[self.kv[l]])
                                                     for l, n in enumerate(self.layer_names)})
        self.rng = rng

    def step(self, metas, queries_per_layer, meta_obj):
        meta_obj.requests = metas
        self.sparse.bind_sparse_metadata(meta_obj)
        for l, name in enumerate(self.layer_names):
            q = queries_per_layer[l]
            self.sparse.attention_begin(q, None, None, name, self.fc)
            self.sparse.attention_finished(q, None, None, None, name, self.fc)
        self.sparse.clear_sparse_metadata()


def test_esa_hooks_select_and_load_the_right_blocks(oracle):
    from ucmx.sparse.base import UcmSparseRole
    from ucmx.sparse.esa import ESA, ESASparseMetaData, ReqMeta, block_hashes_of
    from ucmx.sparse.factory import UcmSparseFactory
    from ucmx.store.dramstore import UcmDramStore, store_offset

    slice_bytes = T * HKV * D * 2
    store = UcmDramStore({"role": "worker", "max_cache_size": 512 * slice_bytes, "kv_block_size": slice_bytes, "device": DEV})
    cfg = {"init_window_sz": 1, "local_window_sz": 2, "min_blocks": 4, "sparse_ratio": 0.3, "retrieval_stride": 3}
    esa = UcmSparseFactory.create_sparse_method(make_config("ESA", cfg, store), UcmSparseRole.WORKER)
    assert isinstance(esa, ESA)
    run = Runner(esa, seed=81)
    rng = run.rng
    prompts = {"A": list(rng.integers(0, 1000, 20 * T)), "B": list(rng.integers(0, 1000, 33 * T + 5))}
    prefill_blocks = {"A": list(range(0, 20)), "B": list(range(20, 54))}        # B: 33 full + 1 partial
    sparse_range = {"A": 18, "B": 32}
    top_k = {"A": 5, "B": 9}
    hashes = {r: block_hashes_of(prompts[r], T) for r in prompts}

    # ---- prefill (single chunk): representatives are built in attention_finished
    metas = [ReqMeta(r, i, len(prompts[r]), 0, prefill_blocks[r], 0, prompts[r], []) for i, r in enumerate(prompts)]
    qs = [dev_bf16(H.randn_bf16(rng, (len(prompts["A"]) + len(prompts["B"]), HQ, D))) for _ in range(LAYERS)]
    run.step(metas, qs, ESASparseMetaData())
    for r in prompts:
        assert len(esa.req_states[r].slots) == sparse_range[r] and esa.req_states[r].top_k == top_k[r]
    for l in range(LAYERS):
        for r in prompts:
            want = H.f32_to_bf16(oracle.pool_blocks(run.kv_host[l][0], np.asarray(prefill_blocks[r][:sparse_range[r]], np.int32), 0, True))
            got = bits(esa.tables[l][torch.tensor(esa.req_states[r].slots, device=DEV)]).reshape(sparse_range[r], -1)
            assert np.array_equal(got, want)

    # ---- what the KV connector does after prefill: every full block goes to the store
    for l in range(LAYERS):
        for r in prompts:
            n = len(hashes[r])
            ok = store_offset((T, HKV, D), 0, 1, 2, l, False)
            ov = store_offset((T, HKV, D), 0, 1, 2, l, True)
            assert store.wait(store.dump(hashes[r], [ok] * n, [run.kv[l][0][b] for b in prefill_blocks[r][:n]])) == 0
            assert store.wait(store.dump(hashes[r], [ov] * n, [run.kv[l][1][b] for b in prefill_blocks[r][:n]])) == 0
    # ---- the scheduler shrinks each request to top_k + local-window blocks; take fresh (zeroed) HBM blocks
    decode_blocks = {"A": list(range(60, 60 + 5 + 2)), "B": list(range(70, 70 + 9 + 3))}
    for l in range(LAYERS):
        for r in prompts:
            run.kv[l][:, decode_blocks[r]] = 0

    def expected(l, r, q_tok_u16):
        reps = oracle.pool_blocks(run.kv_host[l][0], np.asarray(prefill_blocks[r][:sparse_range[r]], np.int32), 0, True)
        qbar = oracle.query_group_mean(q_tok_u16[None], HKV, True)
        s = oracle.score_dot_esa(reps, np.array([0, len(reps)], np.int32), None, qbar)
        idx, _ = oracle.topk_esa(s, top_k[r])
        return {hashes[r][int(i)] for i in idx}

    def check_loaded(l, r, want_hashes):
        held = esa.req_states[r].pre_topk[l]
        assert set(held.values()) == want_hashes and set(held) == set(decode_blocks[r][:top_k[r]])
        for blk, h in held.items():
            src = prefill_blocks[r][hashes[r].index(h)]
            assert torch.equal(run.kv[l][0][blk], dev_bf16(run.kv_host[l][0][src]))
            assert torch.equal(run.kv[l][1][blk], dev_bf16(run.kv_host[l][1][src]))

    outs = {r: [] for r in prompts}
    q_hist = {}
    loads_before = None
    for step in range(1, 5):
        for r in prompts:
            outs[r].append(step)
        metas = [ReqMeta(r, i, 1, len(prompts[r]) + step - 1, decode_blocks[r], i, prompts[r], list(outs[r]))
                 for i, r in enumerate(prompts)]
        q_u16 = [H.randn_bf16(rng, (2, HQ, D)) for _ in range(LAYERS)]
        q_hist[step] = q_u16
        run.step(metas, [dev_bf16(q) for q in q_u16], ESASparseMetaData())
        if step == 1:       # retrieval, load and wait all happen inside attention_begin of step 1
            for l in range(LAYERS):
                for i, r in enumerate(prompts):
                    check_loaded(l, r, expected(l, r, q_u16[l][i]))
            loads_before = {(l, r): dict(esa.req_states[r].pre_topk[l]) for l in range(LAYERS) for r in prompts}
        if step == 4:       # retrieved with the step-2 query, delta-loaded at step 3, waited for at step 4
            for l in range(LAYERS):
                for i, r in enumerate(prompts):
                    want = expected(l, r, q_hist[2][l][i])
                    check_loaded(l, r, want)
                    # blocks selected both times were not moved
                    before = loads_before[(l, r)]
                    for blk, h in esa.req_states[r].pre_topk[l].items():
                        if h in set(before.values()) and before.get(blk) == h:
                            assert True
                    kept = {h for h in want if h in set(before.values())}
                    assert all(before_blk in esa.req_states[r].pre_topk[l] and esa.req_states[r].pre_topk[l][before_blk] == h
                               for before_blk, h in before.items() if h in kept)
    esa.request_finished_in_worker("A")
    assert "A" not in esa.req_states and len(esa.pool.allocated) == sparse_range["B"]
    store.close()


def test_esa_requests_at_different_decode_steps(oracle):
    """Continuous batching: request B starts decoding one iteration after request A, so with stride 3 A collects a
    retrieval in the very iteration in which B starts one (and the other way round an iteration later).  Each
    request must get its own selection, from the query of its own step 2, loaded at its own step 3."""
    from ucmx.sparse.base import UcmSparseRole
    from ucmx.sparse.esa import ESA, ESASparseMetaData, ReqMeta, block_hashes_of
    from ucmx.store.dramstore import UcmDramStore, store_offset

    slice_bytes = T * HKV * D * 2
    store = UcmDramStore({"role": "worker", "max_cache_size": 512 * slice_bytes, "kv_block_size": slice_bytes, "device": DEV})
    cfg = {"init_window_sz": 1, "local_window_sz": 2, "min_blocks": 4, "sparse_ratio": 0.3, "retrieval_stride": 3}
    esa = ESA(make_config("ESA", cfg, store), UcmSparseRole.WORKER)
    run = Runner(esa, seed=83)
    rng = run.rng
    prompts = {"A": list(rng.integers(0, 1000, 22 * T)), "B": list(rng.integers(0, 1000, 30 * T))}
    prefill_blocks = {"A": list(range(0, 22)), "B": list(range(22, 52))}
    sparse_range = {"A": 20, "B": 28}
    top_k = {"A": 6, "B": 8}
    decode_blocks = {"A": list(range(60, 60 + 6 + 2)), "B": list(range(70, 70 + 8 + 2))}
    hashes = {r: block_hashes_of(prompts[r], T) for r in prompts}

    def dump_to_store(r):
        for l in range(LAYERS):
            n = len(hashes[r])
            ok = store_offset((T, HKV, D), 0, 1, 2, l, False)
            ov = store_offset((T, HKV, D), 0, 1, 2, l, True)
            assert store.wait(store.dump(hashes[r], [ok] * n, [run.kv[l][0][b] for b in prefill_blocks[r][:n]])) == 0
            assert store.wait(store.dump(hashes[r], [ov] * n, [run.kv[l][1][b] for b in prefill_blocks[r][:n]])) == 0
            run.kv[l][:, decode_blocks[r]] = 0

    def expected(l, r, q_tok_u16):
        reps = oracle.pool_blocks(run.kv_host[l][0], np.asarray(prefill_blocks[r][:sparse_range[r]], np.int32), 0, True)
        qbar = oracle.query_group_mean(q_tok_u16[None], HKV, True)
        s = oracle.score_dot_esa(reps, np.array([0, len(reps)], np.int32), None, qbar)
        idx, _ = oracle.topk_esa(s, top_k[r])
        return {hashes[r][int(i)] for i in idx}

    def check_loaded(l, r, want_hashes):
        held = esa.req_states[r].pre_topk[l]
        assert set(held.values()) == want_hashes and set(held) == set(decode_blocks[r][:top_k[r]])
        for blk, h in held.items():
            src = prefill_blocks[r][hashes[r].index(h)]
            assert torch.equal(run.kv[l][0][blk], dev_bf16(run.kv_host[l][0][src]))

    out = {"A": [], "B": []}
    q_of = {"A": {}, "B": {}}          # request -> its decode step -> per-layer query row (uint16)
    # iteration 0: A prefills.  iteration i >= 1: A is at decode step i; B prefills in iteration 1 and is at step i-1 after.
    n_a = len(prompts["A"])
    run.step([ReqMeta("A", 0, n_a, 0, prefill_blocks["A"], 0, prompts["A"], [])],
             [dev_bf16(H.randn_bf16(rng, (n_a, HQ, D))) for _ in range(LAYERS)], ESASparseMetaData())
    dump_to_store("A")
    for it in range(1, 7):
        out["A"].append(it)
        metas = [ReqMeta("A", 0, 1, n_a + it - 1, decode_blocks["A"], 0, prompts["A"], list(out["A"]))]
        if it == 1:
            n_b = len(prompts["B"])
            metas.append(ReqMeta("B", 1, n_b, 0, prefill_blocks["B"], 1, prompts["B"], []))
            rows = 1 + n_b
        else:
            out["B"].append(it - 1)
            metas.append(ReqMeta("B", 1, 1, len(prompts["B"]) + it - 2, decode_blocks["B"], 1, prompts["B"], list(out["B"])))
            rows = 2
        q_u16 = [H.randn_bf16(rng, (rows, HQ, D)) for _ in range(LAYERS)]
        q_of["A"][it] = [q[0] for q in q_u16]
        if it >= 2:
            q_of["B"][it - 1] = [q[1] for q in q_u16]
        run.step(metas, [dev_bf16(q) for q in q_u16], ESASparseMetaData())
        if it == 1:
            dump_to_store("B")
        # a request's selection is in place after its step 1 (query of step 1) and after its steps 3 and 6 (query of steps 2 and 5)
        for r, step in (("A", it), ("B", it - 1)):
            src_step = {1: 1, 3: 2, 4: 2, 6: 5}.get(step)
            if src_step is None:
                continue
            if step in (3, 6):                      # loads were launched in this iteration; they are waited for at the next step
                esa._wait_transfer_task_done(0), esa._wait_transfer_task_done(1)
            for l in range(LAYERS):
                check_loaded(l, r, expected(l, r, q_of[r][src_step][l]))
    store.close()


def test_kvcomp_hooks_select_and_load(oracle):
    from ucmx.sparse.base import UcmSparseRole
    from ucmx.sparse.kvcomp import KvComp, KvCompSparseMetaData, ReqMeta, block_hash
    from ucmx.store.dramstore import UcmDramStore

    slice_bytes = T * HKV * D * 2
    store = UcmDramStore({"role": "worker", "max_cache_size": 512 * slice_bytes, "kv_block_size": slice_bytes, "device": DEV})
    kc = KvComp(make_config("KvComp", {"hash_bits": 128}, store), UcmSparseRole.WORKER)
    run = Runner(kc, seed=82)
    rng = run.rng
    n_blocks = {"A": 12, "B": 30}
    prefill_blocks = {"A": list(range(0, 12)), "B": list(range(12, 42))}
    metas = [ReqMeta(r, i, n_blocks[r] * T, 0, n_blocks[r] * T, 0, 0, prefill_blocks[r], 0) for i, r in enumerate(n_blocks)]
    qs = [dev_bf16(H.randn_bf16(rng, (4, HQ, D))) for _ in range(LAYERS)]
    run.step(metas, qs, KvCompSparseMetaData())
    w16 = bits(kc.hash_encoder.hash_weights)
    for l in range(LAYERS):
        for r in n_blocks:
            want = oracle.hash_encode(run.kv_host[l][0][prefill_blocks[r]], w16).transpose(0, 2, 1, 3)   # [n, H, T, 16]
            got = kc.tables[l][torch.tensor(kc.req_states[r].slots, device=DEV)].cpu().numpy()
            assert np.array_equal(got, want)
            assert store.lookup([block_hash(r, 0)]) == [False]                 # dumped, not yet committed
            assert f"{block_hash(r, n_blocks[r] - 1)}_0" in store.slot_of

    # decode step 1: kept blocks = init window + selected middle + local window
    k_mid = {"A": 3, "B": 8}
    decode_blocks = {"A": list(range(50, 50 + 1 + 3 + 2)), "B": list(range(60, 60 + 1 + 8 + 2))}
    for l in range(LAYERS):
        for r in n_blocks:
            run.kv[l][:, decode_blocks[r]] = 0
    metas = [ReqMeta(r, i, n_blocks[r] * T, 1, 1, n_blocks[r] * T, 0, decode_blocks[r], i) for i, r in enumerate(n_blocks)]
    q_u16 = [H.randn_bf16(rng, (2, HQ, D)) for _ in range(LAYERS)]
    run.step(metas, [dev_bf16(q) for q in q_u16], KvCompSparseMetaData())
    for l in range(LAYERS):
        for i, r in enumerate(n_blocks):
            codes = oracle.hash_encode(run.kv_host[l][0][prefill_blocks[r]], w16).transpose(0, 2, 1, 3)
            qbar = H.f32_to_bf16(oracle.query_group_mean(q_u16[l][i][None], HKV, True)).reshape(1, HKV, D)
            qc = oracle.hash_encode(qbar, w16)
            s = oracle.score_hamming(np.ascontiguousarray(codes), np.array([0, n_blocks[r]], np.int32), None, qc, True)
            chosen = oracle.topk_kvcomp(s, k_mid[r], 1, 2)
            targets = decode_blocks[r][1:-2]
            for dst, src_rel in zip(targets, chosen):
                src = prefill_blocks[r][int(src_rel)]
                assert torch.equal(run.kv[l][0][dst], dev_bf16(run.kv_host[l][0][src]))
                assert torch.equal(run.kv[l][1][dst], dev_bf16(run.kv_host[l][1][src]))
            # the windows were restored from the copies taken at the end of prefill
            assert torch.equal(run.kv[l][0][decode_blocks[r][0]], dev_bf16(run.kv_host[l][0][prefill_blocks[r][0]]))
            assert torch.equal(run.kv[l][1][decode_blocks[r][-1]], dev_bf16(run.kv_host[l][1][prefill_blocks[r][-1]]))
    store.close()


def test_kvstar_multistep_hooks_vote_and_load(oracle):
    """Prefill builds pruned fp16 representations and the first query group; decode step 1 loads the blocks
    that group votes for, and the next stride's group (decode queries 1..8) decides at step 9."""
    from ucmx.sparse.base import UcmSparseRole
    from ucmx.sparse.factory import UcmSparseFactory
    from ucmx.sparse.kvstar import KVStarMultiStep, KVStarMultiStepSparseMetaData, ReqMeta, block_hash
    from ucmx.store.dramstore import UcmDramStore

    slice_bytes = T * HKV * D * 2
    store = UcmDramStore({"role": "worker", "max_cache_size": 512 * slice_bytes, "kv_block_size": slice_bytes, "device": DEV})
    cfg = {"retrieval_stride": 8, "sparse_ratio": 0.25, "blk_repre_dim_prune_ratio": 0.25, "blk_repre_inner_token_merge": 2}
    ks = UcmSparseFactory.create_sparse_method(make_config("KVStarMultiStep", cfg, store), UcmSparseRole.WORKER)
    assert isinstance(ks, KVStarMultiStep) and ks.d_pruned == D // 4
    run = Runner(ks, seed=84)
    rng = run.rng
    n_tok = {"A": 12 * T, "B": 30 * T + 5}
    n_full = {"A": 12, "B": 30}
    prefill_blocks = {"A": list(range(0, 12)), "B": list(range(12, 43))}           # B ends in a partial block
    starts = {"A": 0, "B": n_tok["A"]}
    metas = [ReqMeta(r, i, n_tok[r], 0, n_tok[r], 0, 0, prefill_blocks[r], starts[r], n_tok[r]) for i, r in enumerate(n_tok)]
    q_pre = [H.randn_bf16(rng, (n_tok["A"] + n_tok["B"], HQ, D)) for _ in range(LAYERS)]
    run.step(metas, [dev_bf16(q) for q in q_pre], KVStarMultiStepSparseMetaData())

    pruned, reps = {}, {}
    for l in range(LAYERS):
        for r in n_tok:
            k = H.bf16_to_f32(run.kv_host[l][0][prefill_blocks[r][: n_full[r]]]).reshape(-1, HKV, D)
            want_channels = np.argsort(-np.abs(k).astype(np.float64).mean(0), axis=-1)[:, : D // 4]
            pr = ks.req_states[r].pruned[l].cpu().numpy()
            assert [set(a) for a in pr] == [set(a) for a in want_channels]
            pruned[l, r] = pr
            want = oracle.kvstar_block_repre(run.kv_host[l][0], np.asarray(prefill_blocks[r][: n_full[r]], np.int32), pr, 2)
            got = ks.tables[l][torch.tensor(ks.req_states[r].slots, device=DEV)].view(torch.int16).cpu().numpy().view(np.uint16)
            assert np.array_equal(got, want)
            reps[l, r] = want
            assert f"{block_hash(r, n_full[r] - 1)}_0" in store.slot_of

    def half_bits(q_u16):
        return H.f32_to_f16_bits(H.bf16_to_f32(q_u16))

    def check(l, r, group_u16, targets):
        mid = reps[l, r][1: n_full[r] - 2]
        s = oracle.kvstar_scores(half_bits(group_u16), mid, pruned[l, r])
        k = len(targets)
        best = np.sort(s)[::-1][:k]
        srcs = []
        for dst in targets:
            hit = [j for j in range(len(mid)) if torch.equal(run.kv[l][0][dst], dev_bf16(run.kv_host[l][0][prefill_blocks[r][1 + j]]))]
            assert len(hit) == 1
            assert torch.equal(run.kv[l][1][dst], dev_bf16(run.kv_host[l][1][prefill_blocks[r][1 + hit[0]]]))
            srcs.append(hit[0])
        assert len(set(srcs)) == k
        np.testing.assert_allclose(s[srcs], best, rtol=2e-3)           # the k largest votes, in descending order

    k_mid = {"A": 3, "B": 7}                                                       # ceil(9 / 4), ceil(27 / 4)
    decode_blocks = {"A": list(range(50, 50 + 1 + 3 + 2)), "B": list(range(60, 60 + 1 + 7 + 3))}
    for l in range(LAYERS):
        for r in n_tok:
            run.kv[l][:, decode_blocks[r]] = 0
    q_dec = {}
    for step in range(1, 10):
        metas = [ReqMeta(r, i, n_tok[r], step, 1, n_tok[r] + step - 1, 0, decode_blocks[r], i, 1) for i, r in enumerate(n_tok)]
        q_dec[step] = [H.randn_bf16(rng, (2, HQ, D)) for _ in range(LAYERS)]
        if step == 9:
            for l in range(LAYERS):
                for r in n_tok:
                    run.kv[l][:, decode_blocks[r][1: 1 + k_mid[r]]] = 0
        run.step(metas, [dev_bf16(q) for q in q_dec[step]], KVStarMultiStepSparseMetaData())
        for l in range(LAYERS):
            for i, r in enumerate(n_tok):
                targets = decode_blocks[r][1: 1 + k_mid[r]]
                if step == 1:
                    check(l, r, q_pre[l][starts[r] + n_tok[r] - 8: starts[r] + n_tok[r]], targets)
                    assert torch.equal(run.kv[l][0][decode_blocks[r][0]], dev_bf16(run.kv_host[l][0][prefill_blocks[r][0]]))
                    assert torch.equal(run.kv[l][1][decode_blocks[r][-1]], dev_bf16(run.kv_host[l][1][prefill_blocks[r][-1]]))
                if step == 9:
                    check(l, r, np.stack([q_dec[t][l][i] for t in range(1, 9)]), targets)
    ks.request_finished_in_worker("A")
    assert "A" not in ks.req_states and len(ks.pool.allocated) == n_full["B"]
    store.close()


def test_gsa_block_table_rewrite(oracle):
    from ucmx.sparse.base import UcmSparseRole
    from ucmx.sparse.gsa import GSA, GSAMetaData, compute_topk_len

    for n_rep in (1, 3):
        gsa = GSA(make_config("GSA", {"max_norm_num": n_rep, "start_window": 1, "end_window": 2}, None), UcmSparseRole.WORKER)
        run = Runner(gsa, seed=83 + n_rep)
        rng = run.rng
        blocks = {"A": list(rng.permutation(NBLK)[:40]), "B": list(rng.permutation(NBLK)[:70])}
        md = GSAMetaData()
        md.req_ids = list(blocks)
        md.block_ids = [[int(b) for b in blocks[r]] for r in blocks]
        md.seq_lens = [40 * T - 3, 70 * T]
        md.query_rows = [0, 1]
        gsa.bind_sparse_metadata(md)
        all_ids = sorted({int(b) for r in blocks for b in blocks[r]})
        q_u16 = H.randn_bf16(rng, (2, HQ, D))
        for l, name in enumerate(run.layer_names):
            gsa.copy_k(name, run.fc, all_ids)
            gsa.attention_begin(dev_bf16(q_u16), None, None, name, run.fc)
            table = run.fc.attn_metadata.block_table.cpu().numpy()
            seq = run.fc.attn_metadata.seq_lens.cpu().numpy()
            modes = [0] if n_rep == 1 else [0, 1, 2]
            for i, r in enumerate(blocks):
                ids = np.asarray(blocks[r], np.int32)
                reps = np.stack([oracle.pool_blocks(run.kv_host[l][0], ids, m, True).reshape(len(ids), HKV, D) for m in modes], 2)
                qm = oracle.query_group_mean(q_u16[i][None], HKV, False)
                s = oracle.score_dot_gsa(reps, HKV, n_rep, D, np.array([0, len(ids)], np.int32), None, qm)
                k = compute_topk_len(len(ids))
                sel = oracle.topk_gsa(s, k, 1, 2)
                assert np.array_equal(table[i, :len(sel)], ids[sel])
                tail = md.seq_lens[i] - (len(ids) - 1) * T
                assert seq[i] == (len(sel) - 1) * T + tail
