"""Records GSA's device-side block weights, computed with the reference's own torch expressions
(cal_topk, ucm/sparse/gsa/gsa.py:386-412) on CPU in bf16 as the reference runs them, for the seeded case
of tests/helpers.py, into tests/golden/gsa_heads.npz.  The table is passed in the reference's layout
[slot, n_rep, kv_heads, D].

    python tests/golden/make_gsa_heads_golden.py
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(os.path.dirname(HERE)))
import helpers as H  # noqa: E402


def bf(u16):
    return torch.from_numpy(u16.view(np.int16).copy()).view(torch.bfloat16)


def main():
    reps, q, off, ids, inc, exc = H.case_gsa_heads()
    n_slots, kvH, R, D = reps.shape
    Hq = q.shape[1]
    kpre = bf(reps).permute(0, 2, 1, 3).contiguous()              # [slot, n_rep, kv_heads, D]
    out = np.zeros(int(off[-1]), np.float32)
    for r, (a, b) in enumerate(zip(off[:-1], off[1:])):
        # one request at a time (the reference pads requests to a common block count; the arithmetic per block is this)
        q_decode = bf(q)[r:r + 1]
        kpre_need = kpre[torch.from_numpy(ids[a:b]).long()]
        max_norm_num = kpre_need.shape[1]
        # every KV head serves its group of query heads (the reference's expand + reshape to att_num_heads)
        kpre_out = kpre_need.unsqueeze(3).expand(-1, -1, -1, Hq // kvH, -1).reshape(1, -1, Hq, D)
        blk_num = kpre_out.shape[1] // max_norm_num
        qk = torch.einsum("bij,bmij->bim", q_decode, kpre_out)
        w, _ = torch.max(qk.reshape(1, Hq, blk_num, max_norm_num), dim=-1)
        w = w.mean(1)
        w.masked_fill_(torch.from_numpy(inc[a:b]).view(1, -1) == 1, float("inf"))
        w.masked_fill_(torch.from_numpy(exc[a:b]).view(1, -1) == 1, float("-inf"))
        out[a:b] = w[0].float().numpy()
    np.savez_compressed(os.path.join(HERE, "gsa_heads.npz"), weights=out)
    print("wrote gsa_heads.npz", out[:6])


if __name__ == "__main__":
    main()
