"""Records what the reference's GSA prefetch engine (ucm/sparse/gsa/prefetch/src/kvcache_pre.cpp, compiled
unmodified by `make -C oracle ref`) does with seeded selection rounds, into tests/golden/remap_rounds.json:
block tables, load lists, free lists and block maps of every layer after every round.

    python tests/golden/make_remap_golden.py
"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import helpers as H  # noqa: E402
from oracle import oracle  # noqa: E402


def main():
    cases = []
    for name in H.REMAP_SCENARIOS:
        sc = H.remap_scenario(name)
        got = oracle.ref_prefetch_rounds(sc["n_layers"], sc["block_table"], sc["owned_idx"], sc["free_idx"], sc["rounds"],
                                         idx_dtype=sc["idx_dtype"])
        cases.append({"name": name, "rounds": got})
    with open(os.path.join(HERE, "remap_rounds.json"), "w") as f:
        json.dump(cases, f, separators=(",", ":"))
    print("wrote", len(cases), "scenarios")


if __name__ == "__main__":
    main()
