"""Seeded inputs shared by the golden-vector generator and the tests (numpy only, so that the
same bits come out on every machine). bf16 tensors are carried as uint16 bit patterns."""
import numpy as np


def f32_to_bf16(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    return ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)


def bf16_to_f32(h):
    return (np.ascontiguousarray(h, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def randn_bf16(rng, shape, scale=1.0):
    return f32_to_bf16(rng.standard_normal(shape, dtype=np.float32) * np.float32(scale))


def bf16_ulp_distance(a_u16, b_u16):
    """Distance in bf16 steps between two bf16 bit arrays (sign-magnitude aware)."""
    def key(u):
        u = u.astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)
    return np.abs(key(a_u16) - key(b_u16))


def ragged_offsets(counts):
    off = np.zeros(len(counts) + 1, np.int32)
    off[1:] = np.cumsum(counts)
    return off


# ---- the fixed small cases behind tests/golden/golden.npz ---------------------------------------

def case_pool(seed=1001):
    rng = np.random.default_rng(seed)
    k = randn_bf16(rng, (12, 128, 8, 128))
    ids = rng.permutation(12)[:9].astype(np.int32)
    return k, ids


def case_qmean(seed=1002):
    rng = np.random.default_rng(seed)
    return randn_bf16(rng, (5, 32, 128))


def case_esa(seed=1003):
    rng = np.random.default_rng(seed)
    data = bf16_to_f32(randn_bf16(rng, (300, 1024), 0.09))
    query = bf16_to_f32(randn_bf16(rng, (3, 1024)))
    idx = np.full((3, 100), -1, np.int32)
    for r, n in enumerate((100, 37, 64)):
        idx[r, :n] = rng.permutation(300)[:n]
    return data, query, idx, 16


def case_gsa(seed=1004, n_rep=1):
    rng = np.random.default_rng(seed + n_rep)
    reps = bf16_to_f32(randn_bf16(rng, (40, 8, n_rep, 128), 0.09))
    q = bf16_to_f32(randn_bf16(rng, (32, 128)))
    return q, reps, dict(start=2, end=4, k=12)


def case_hash(seed=1005):
    rng = np.random.default_rng(seed)
    w = randn_bf16(rng, (128, 128), 2.0)           # HashEncoder draws N(0, std=2)
    q = randn_bf16(rng, (1, 8, 128))                # one decode token, 8 (group-mean) heads
    keys = randn_bf16(rng, (7, 16, 8, 128))         # 7 blocks of 16 tokens, 8 kv heads
    return w, q, keys


def f32_to_f16_bits(x):
    return np.ascontiguousarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


KVSTAR_CASES = {
    # name: (seed, x tokens, Hq, H, d_orig, d_pruned, M positions per block, n blocks, top-k)
    "llama": (6001, 8, 32, 8, 128, 32, 64, 96, 24),          # tensor-core shape: 4 heads per instruction, 2 groups
    "qwen": (6002, 8, 64, 8, 128, 32, 64, 80, 20),           # 8-way groups: 2 heads per instruction, 4 groups
    "short_group": (6003, 5, 32, 8, 128, 32, 32, 70, 18),    # 20 query rows per head padded to 32
    "odd": (6004, 3, 6, 2, 40, 24, 10, 37, 9),               # a shape only the CUDA-core kernel takes
    "unpruned": (6005, 2, 8, 4, 64, 64, 32, 41, 10),         # no channel list: d_pruned == d_orig
}


def case_kvstar(name):
    """Query group (half bits [x, Hq, d]), block representations (half bits [n, M, H, d_pruned]) and the
    kept-channel list (int64 [H, d_pruned] or None) of one KVStar retrieval."""
    seed, x, Hq, H, D, dp, M, n, k = KVSTAR_CASES[name]
    rng = np.random.default_rng(seed)
    q = f32_to_f16_bits(rng.standard_normal((x, Hq, D), dtype=np.float32))
    reps = f32_to_f16_bits(rng.standard_normal((n, M, H, dp), dtype=np.float32) * np.float32(0.6))
    pruned = None if dp == D else np.stack([rng.permutation(D)[:dp] for _ in range(H)]).astype(np.int64)
    return q, reps, pruned, k


def case_kvstar_repre(seed=6101, merge=2, dp=32):
    rng = np.random.default_rng(seed + merge)
    k = randn_bf16(rng, (7, 128, 8, 128))
    ids = rng.permutation(7)[:5].astype(np.int32)
    pruned = np.stack([rng.permutation(128)[:dp] for _ in range(8)]).astype(np.int64)
    return k, ids, pruned


def case_gsa_heads(seed=7001):
    """GSA device-side scoring: 3 requests over a shared table with 3 representatives per block and head."""
    rng = np.random.default_rng(seed)
    H, Hq, D, R, n_slots = 8, 32, 128, 3, 90
    reps = randn_bf16(rng, (n_slots, H, R, D), 0.3)
    q = randn_bf16(rng, (3, Hq, D))
    counts = [40, 7, 33]
    off = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    ids = rng.permutation(n_slots)[:off[-1]].astype(np.int32)
    inc = np.zeros(off[-1], np.uint8)
    exc = np.zeros(off[-1], np.uint8)
    for a, b in zip(off[:-1], off[1:]):
        inc[a:a + 2] = 1          # the first blocks are always kept
        inc[b - 1] = 1            # and the newest one
        exc[a + 4] = 1
    exc[off[1] - 1] = 1           # flagged both ways: exclude wins
    return reps, q, off, ids, inc, exc


# ---------------------------------------------------------------- resident-set remap scenarios
REMAP_SCENARIOS = {
    # name: (seed, layers, logical blocks, resident at start, on the free list at start, selected per round, rounds,
    #        ascending selections, index dtype)
    "steady": (7101, 3, 64, 24, 6, 16, 6, True, "int32"),
    "free_list_runs_out": (7102, 2, 48, 12, 2, 10, 4, True, "int32"),        # more misses than free blocks
    "all_hits_then_all_misses": (7103, 2, 40, 10, 4, 6, 3, True, "int64"),
    "unsorted_selection": (7104, 2, 64, 20, 8, 12, 5, False, "int64"),
    "one_block": (7105, 1, 8, 1, 1, 1, 4, True, "int32"),
}


def remap_scenario(name):
    """Seeded inputs of one life cycle of a request in the prefetch engine.  The blocks on the initial free list
    are given in ascending physical order - the order every later free list has."""
    seed, L, n_logical, n_owned, n_free, k, n_rounds, ascending, idx_dtype = REMAP_SCENARIOS[name]
    rng = np.random.default_rng(seed)
    block_table = [int(x) for x in rng.permutation(4 * n_logical)[:n_logical] + 1]
    owned = sorted(int(x) for x in rng.permutation(n_logical)[:n_owned])
    free_idx = sorted((int(x) for x in rng.permutation(owned)[:n_free]), key=lambda i: block_table[i])
    rounds = []
    for r in range(n_rounds):
        sel = np.stack([rng.permutation(n_logical)[:k] for _ in range(L)])
        if name == "all_hits_then_all_misses":
            held = [i for i in owned if i not in free_idx]
            sel = np.stack([np.asarray(held[:k]) if r == 0 else
                            np.asarray([i for i in range(n_logical) if i not in owned][r * k: (r + 1) * k]) for _ in range(L)])
        if ascending:
            sel = np.sort(sel, axis=1)
        rounds.append(sel.astype(np.int64))
    return {"n_layers": L, "block_table": block_table, "owned_idx": owned, "free_idx": free_idx, "rounds": rounds,
            "idx_dtype": idx_dtype}


def remap_replay(oracle, sc):
    """The scenario through the CPU checker, in the shape oracle.ref_prefetch_rounds returns."""
    bt = sc["block_table"]
    order = sorted(sc["owned_idx"], key=lambda i: bt[i])
    phys = np.asarray([bt[i] for i in order], np.int32)
    out = []
    logical = [np.asarray(order, np.int32) for _ in range(sc["n_layers"])]
    free = [np.asarray([1 if i in sc["free_idx"] else 0 for i in order], np.uint8) for _ in range(sc["n_layers"])]
    for sel in sc["rounds"]:
        res = {"table": [], "load_blocks": [], "miss_idx": [], "free": [], "blocks_map": []}
        for l in range(sc["n_layers"]):
            before = set(int(x) for x in logical[l])
            logical[l], free[l], table, ll, lp = oracle.remap_resident(logical[l], free[l], phys, sel[l].astype(np.int32))
            pairs = sorted((int(s), int(t)) for s, t in zip(sel[l], table) if t >= 0)      # the engine lists by logical index
            res["table"].append([t for _, t in pairs])
            res["load_blocks"].append([int(x) for x in lp])
            assert [int(x) for x in ll] == [int(s) for s in sel[l] if int(s) not in before][: len(ll)]
            res["miss_idx"].append([int(s) for s in sel[l] if int(s) not in before])
            res["free"].append([int(p) for p, f in zip(phys, free[l]) if f])
            res["blocks_map"].append({int(p): int(x) for p, x in zip(phys, logical[l])})
        out.append(res)
    return out
