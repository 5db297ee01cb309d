"""Regenerates tests/golden/golden.npz from the reference itself (run in a container that has the
UCM checkout at $UCM_REFERENCE and oracle/_ref built by `make -C oracle ref`).

Outputs only are stored; the inputs are re-created from seeds by tests/helpers.py.
Sources of each vector:
  pool_*      torch CPU `k_cache[ids].mean(1)` in bf16 (ucm/sparse/esa/esa.py:265-266) and the
              amax/amin/sum siblings for the max/min/sum representative variants
  qmean       torch CPU `query.view(ntok, kvH, -1, D).mean(2)` in bf16 (esa.py:291-293)
  esa_*       the compiled ucm/sparse/esa/retrieval/cpy/retrieval_backend.cpp (oracle/_ref)
  gsa_*       the compiled ucm/sparse/gsa/offload_ops sources (oracle/_ref/libgsa_ref.so)
  hash_*      ucm/sparse/kvcomp/hash_encoder.py imported from the checkout, on CPU in bf16
  kvcomp_*    the scoring expression of ucm/sparse/kvcomp/kvcomp.py:239-254 applied to those codes
  offset_*    get_offset executed from the text of ucm/sparse/esa/esa.py:123-135
"""
import ast
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import helpers as H  # noqa: E402
from oracle import oracle as orc  # noqa: E402

REF = orc.reference_root()
if REF is None:
    raise SystemExit("set UCM_REFERENCE to a checkout of the reference project")
sys.path.insert(0, REF)


def bf(u16):
    return torch.from_numpy(u16.view(np.int16).copy()).view(torch.bfloat16)


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def main():
    out = {}

    k, ids = H.case_pool()
    kt = bf(k)
    sel = kt[torch.from_numpy(ids).long()]
    out["pool_mean"] = bits(sel.mean(1))
    out["pool_max"] = bits(sel.amax(1))
    out["pool_min"] = bits(sel.amin(1))
    out["pool_sum"] = bits(sel.sum(1))

    q = H.case_qmean()
    qt = bf(q)
    out["qmean"] = qt.view(5, 8, -1, 128).mean(2).reshape(5, -1).to(torch.float32).numpy()

    rb = orc.ref_retrieval_backend()
    data, query, idx, topk = H.case_esa()
    backend = rb.RetrievalWorkerBackend(data)
    rid = backend.submit(query, topk, idx)
    backend.wait(rid)
    res = backend.get_result(rid)
    out["esa_indices"] = np.asarray(res["indices"], np.int32)
    out["esa_scores"] = np.asarray(res["scores"], np.float32)
    del backend

    for n_rep in (1, 3):
        qg, reps, p = H.case_gsa(n_rep=n_rep)
        out[f"gsa_topk_r{n_rep}"] = orc.ref_gsa_select_topk(qg, reps, 8, 32, n_rep, 128, p["start"], p["end"], p["k"])[: p["k"]]
        qm = orc.ref_gsa_q_head_mean(qg, 8)
        out[f"gsa_qmean_r{n_rep}"] = qm
        out[f"gsa_scores_r{n_rep}"] = orc.ref_gsa_scores(qm, reps, 8, n_rep, 128)
    # K representatives by the reference's native KRepreComputer (fp32, [n, H, T, D] layout)
    kf = H.bf16_to_f32(k[ids]).transpose(0, 2, 1, 3).copy()
    out["gsa_krepre"] = orc.ref_gsa_k_repre(kf)

    from ucm.sparse.kvcomp.hash_encoder import HashEncoder
    w, hq, keys = H.case_hash()
    enc = HashEncoder(128, 128, torch.bfloat16, torch.device("cpu"))
    enc.set_hash_weight(bf(w))
    q_codes = enc.compute_hash(bf(hq))                      # [1, 8, 16]
    k_codes = enc.compute_hash(bf(keys))                    # [7, 16, 8, 16]
    out["hash_q_codes"] = q_codes.numpy()
    out["hash_k_codes"] = k_codes.numpy()
    block_repre = k_codes.transpose(1, 2).contiguous()      # [n, H, T, 16] as kvcomp.py:342 keeps it
    uq = enc._unpack_hash(q_codes)
    uk = enc._unpack_hash(block_repre)
    s = torch.einsum("tid,njsd->tijsn", uq, uk)
    s = s.sum(dim=tuple(range(s.ndim - 1)))
    out["kvcomp_scores_all"] = s.to(torch.float32).numpy().astype(np.int32)
    # the retrieval range and top-k of kvcomp.py:225-254 with init window 1, local window 2
    mid = block_repre[1 : block_repre.shape[0] - 2 + 1]
    sm = torch.einsum("tid,njsd->tijsn", uq, enc._unpack_hash(mid))
    sm = sm.sum(dim=tuple(range(sm.ndim - 1)))
    top = torch.topk(sm, 3).indices.sort().values + 1
    out["kvcomp_topk"] = top.numpy().astype(np.int32)

    src = open(os.path.join(REF, "ucm/sparse/esa/esa.py")).read()
    fn = [n for n in ast.parse(src).body if isinstance(n, ast.FunctionDef) and n.name == "get_offset"][0]
    fn.decorator_list = []
    ns = {}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), "esa.get_offset", "exec"), ns)
    rows = []
    for rank, tp, layer, is_v in [(0, 1, 0, False), (0, 1, 3, True), (1, 2, 5, False), (3, 4, 31, True), (7, 8, 17, False)]:
        rows.append([rank, tp, layer, int(is_v), ns["get_offset"]((128, 8 // tp, 128), rank, tp, 2, layer, is_v, False)])
    out["offset_cases"] = np.asarray(rows, np.int64)

    np.savez_compressed(os.path.join(HERE, "golden.npz"), **out)
    for k_, v in out.items():
        print(k_, v.shape, v.dtype)


if __name__ == "__main__":
    main()
