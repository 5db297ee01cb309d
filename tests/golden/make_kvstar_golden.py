"""Records what the reference's KVStar code returns on the seeded cases of tests/helpers.py into
tests/golden/kvstar.npz (outputs only; the inputs are re-created from seeds).

  <case>_avx2    the blocks KVStar::Execute selects in the AVX2 build an x86 host runs (sorted; that
                 build returns them in no particular order)
  <case>_rank    the complete ranking of all blocks from the portable scalar build (top-k = n)
  repre_m<c>     extract_block_repre's arithmetic (ucm/sparse/kvstar/multistep.py:300-314,495-499) in torch
                 on CPU: channel selection, mean over `c` merged tokens in bf16, cast to half

    python tests/golden/make_kvstar_golden.py      # needs oracle/_ref built from a UCM checkout
"""
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


def main():
    out = {}
    for name in H.KVSTAR_CASES:
        q, reps, pruned, k = H.case_kvstar(name)
        out[name + "_avx2"] = np.sort(orc.ref_kvstar_topk(q, reps, pruned, k))
        out[name + "_rank"] = orc.ref_kvstar_topk(q, reps, pruned, reps.shape[0], scalar=True)
    for merge in (2, 4):
        k, ids, pruned = H.case_kvstar_repre(merge=merge)
        kc = torch.from_numpy(k.view(np.int16).copy()).view(torch.bfloat16)[torch.from_numpy(ids).long()]
        n, S, h, d = kc.shape
        dp = pruned.shape[1]
        kp = torch.zeros_like(kc[:, :, :, :dp])
        for i_h in range(h):
            kp[:, :, i_h, :] = kc[:, :, i_h, torch.from_numpy(pruned[i_h])]
        rep = kp.reshape(n, S // merge, merge, h, dp).mean(dim=2).to(torch.float16)
        out[f"repre_m{merge}"] = rep.contiguous().view(torch.int16).numpy().view(np.uint16).copy()
    np.savez_compressed(os.path.join(HERE, "kvstar.npz"), **out)
    print("wrote kvstar.npz:", sorted(out))


if __name__ == "__main__":
    main()
