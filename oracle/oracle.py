"""numpy front-end of the CPU checker (oracle/ucm_oracle.c and, when built, oracle/_ref).

TEST INFRASTRUCTURE ONLY.  The shipped package never imports this module; the test-suite, the
smoke check and the benchmark's CPU-baseline leg do.  Each function forwards to the C restatement
whose comment names the reference lines it follows.  bf16 arrays are carried as numpy uint16.
"""
from __future__ import annotations

import ctypes as C
import importlib.util
import os
import subprocess
import sys

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libucm_oracle.so")
_REF_DIR = os.path.join(_HERE, "_ref")

POOL_MEAN, POOL_MAX, POOL_MIN, POOL_SUM = 0, 1, 2, 3


def reference_root():
    """Where a checkout of the reference project lies: $UCM_REFERENCE, else a directory named `reference` beside this
    repository; None when there is none (the GPU box: only the prebuilt oracle/_ref travels)."""
    cand = os.environ.get("UCM_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return cand if os.path.isdir(os.path.join(cand, "ucm")) else None


def build(ref: bool = True) -> None:
    """Compile the C restatement, and the reference's own CPU sources when a checkout is present."""
    targets = ["oracle"]
    root = reference_root() if ref else None
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    cmd = ["make", "-s", "-C", _HERE] + targets
    if root:
        cmd += ["ref", "REF=" + root]
    subprocess.run(cmd, check=True, env=env)


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build(ref=False)
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_bf16_round.restype = C.c_float
        _lib.orc_bf16_round.argtypes = [C.c_float]
        _lib.orc_store_offset.restype = C.c_int64
        for n in ("orc_topk_esa", "orc_topk_gsa", "orc_topk_kvcomp", "orc_remap_resident"):
            getattr(_lib, n).restype = C.c_int32
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    return None if a is None else np.ascontiguousarray(a, dtype=dt)


# ---------------------------------------------------------------- bf16 helpers

def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    return ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)


def bf16_to_f32(h: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(h, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# --------------------------------------------------------------------- stages

def pool_blocks(k_u16, block_ids, mode=POOL_MEAN, round_bf16=True):
    """k_u16: uint16 [num_blocks, T, H, D] (dense paged cache). Returns fp32 [n, H*D]."""
    k = _c(k_u16, np.uint16)
    nb, T, H, D = k.shape
    ids = _c(block_ids, np.int32)
    out = np.empty((len(ids), H * D), np.float32)
    lib().orc_pool_blocks(_p(k), C.c_int64(T * H * D), C.c_int64(H * D), C.c_int32(T),
                          C.c_int32(H), C.c_int32(D), _p(ids), C.c_int32(len(ids)),
                          C.c_int32(mode), C.c_int32(int(round_bf16)), _p(out))
    return out


def query_group_mean(q_u16, n_kv_heads, round_bf16=True):
    """q_u16: uint16 [n_tok, Hq, D]. Returns fp32 [n_tok, n_kv_heads*D]."""
    q = _c(q_u16, np.uint16)
    nt, Hq, D = q.shape
    out = np.empty((nt, n_kv_heads * D), np.float32)
    lib().orc_query_group_mean(_p(q), C.c_int32(nt), C.c_int32(Hq), C.c_int32(n_kv_heads),
                               C.c_int32(D), C.c_int64(Hq * D), C.c_int32(int(round_bf16)), _p(out))
    return out


def score_dot_esa(data_f32, req_offsets, slot_ids, q_f32):
    data = _c(data_f32, np.float32)
    off = _c(req_offsets, np.int32)
    sl = _c(slot_ids, np.int32)
    q = _c(q_f32, np.float32)
    out = np.empty(int(off[-1]), np.float32)
    lib().orc_score_dot_esa(_p(data), C.c_int32(data.shape[1]), _p(off), _p(sl), _p(q),
                            C.c_int32(len(off) - 1), _p(out))
    return out


def score_dot_gsa(reps_f32, n_kv_heads, n_rep, head_dim, req_offsets, slot_ids, q_f32):
    reps = _c(reps_f32, np.float32)
    off = _c(req_offsets, np.int32)
    sl = _c(slot_ids, np.int32)
    q = _c(q_f32, np.float32)
    out = np.empty(int(off[-1]), np.float32)
    lib().orc_score_dot_gsa(_p(reps), C.c_int32(n_kv_heads), C.c_int32(n_rep), C.c_int32(head_dim),
                            _p(off), _p(sl), _p(q), C.c_int32(len(off) - 1), _p(out))
    return out


def topk_esa(scores, k, id_map=None):
    s = _c(scores, np.float32)
    m = _c(id_map, np.int32)
    n = len(s)
    idx = np.empty(max(min(k, n), 1), np.int32)
    sc = np.empty(max(min(k, n), 1), np.float32)
    cnt = lib().orc_topk_esa(_p(s), C.c_int32(n), C.c_int32(k), _p(m), _p(idx), _p(sc))
    return idx[:cnt], sc[:cnt]


def topk_gsa(scores, k, start, end, cap=None):
    s = _c(scores, np.float32)
    n = len(s)
    cap = n if cap is None else cap
    idx = np.empty(max(cap, 1), np.int32)
    cnt = lib().orc_topk_gsa(_p(s), C.c_int32(n), C.c_int32(k), C.c_int32(start), C.c_int32(end),
                             C.c_int32(cap), _p(idx))
    return idx[:cnt]


def topk_kvcomp(scores_i32, k, init_win=1, local_win=2):
    s = _c(scores_i32, np.int32)
    n = len(s)
    idx = np.empty(max(n, 1), np.int32)
    cnt = lib().orc_topk_kvcomp(_p(s), C.c_int32(n), C.c_int32(k), C.c_int32(init_win),
                                C.c_int32(local_win), _p(idx))
    return idx[:cnt]


def hash_encode(x_u16, w_u16):
    """x_u16: uint16 [..., dim]; w_u16: uint16 [dim, bits]. Returns uint8 [..., bits/8]."""
    x = _c(x_u16, np.uint16)
    w = _c(w_u16, np.uint16)
    dim, bits = w.shape
    nv = x.size // dim
    out = np.empty(x.shape[:-1] + (bits // 8,), np.uint8)
    lib().orc_hash_encode(_p(x), C.c_int64(nv), _p(w), C.c_int32(dim), C.c_int32(bits), _p(out))
    return out


def hash_project(x_u16, w_u16):
    x = _c(x_u16, np.uint16)
    w = _c(w_u16, np.uint16)
    dim, bits = w.shape
    nv = x.size // dim
    out = np.empty(x.shape[:-1] + (bits,), np.float32)
    lib().orc_hash_project(_p(x), C.c_int64(nv), _p(w), C.c_int32(dim), C.c_int32(bits), _p(out))
    return out


def score_hamming(codes_u8, req_offsets, slot_ids, q_codes_u8, cross_head=True):
    """codes_u8: uint8 [slots, H, T, bits/8]; q_codes_u8: uint8 [n_req, Hq, bits/8]."""
    codes = _c(codes_u8, np.uint8)
    _, H, T, nb = codes.shape
    qc = _c(q_codes_u8, np.uint8)
    off = _c(req_offsets, np.int32)
    sl = _c(slot_ids, np.int32)
    out = np.empty(int(off[-1]), np.int32)
    lib().orc_score_hamming(_p(codes), C.c_int32(H), C.c_int32(T), C.c_int32(nb * 8), _p(off),
                            _p(sl), _p(qc), C.c_int32(qc.shape[1]), C.c_int32(len(off) - 1),
                            C.c_int32(int(cross_head)), _p(out))
    return out


def _plane_array(planes):
    arr = (C.c_void_p * len(planes))()
    for i, p in enumerate(planes):
        arr[i] = p.ctypes.data
    return arr


def gather_blocks(planes, block_ids, slice_bytes, block_stride):
    """planes: list of uint8 arrays (one per K/V plane). Returns uint8 [n, n_planes, slice_bytes]."""
    ids = _c(block_ids, np.int32)
    out = np.empty((len(ids), len(planes), slice_bytes), np.uint8)
    lib().orc_gather_blocks(_plane_array(planes), C.c_int32(len(planes)), C.c_int64(block_stride),
                            _p(ids), C.c_int32(len(ids)), C.c_int64(slice_bytes), _p(out))
    return out


def scatter_blocks(planes, block_ids, slice_bytes, block_stride, staging):
    ids = _c(block_ids, np.int32)
    st = _c(staging, np.uint8)
    lib().orc_scatter_blocks(_plane_array(planes), C.c_int32(len(planes)), C.c_int64(block_stride),
                             _p(ids), C.c_int32(len(ids)), C.c_int64(slice_bytes), _p(st))


def remap_resident(slot_logical, slot_free, slot_phys, selected):
    """One round for one request. Returns (slot_logical', slot_free', table, load_logical, load_phys)."""
    res = _c(slot_logical, np.int32).copy()
    fr = _c(slot_free, np.uint8).copy()
    sl = _c(slot_phys, np.int32)
    sel = _c(selected, np.int32)
    table = np.empty(max(len(sel), 1), np.int32)
    ll = np.empty(max(len(sel), 1), np.int32)
    lp = np.empty(max(len(sel), 1), np.int32)
    n = lib().orc_remap_resident(_p(res), _p(fr), _p(sl), C.c_int32(len(sl)), _p(sel), C.c_int32(len(sel)),
                                 _p(table), _p(ll), _p(lp))
    return res, fr, table[:len(sel)], ll[:n], lp[:n]


def store_offset(block_tokens, heads_per_rank, head_dim, rank, tp_size, elem_bytes, layer, is_v,
                 is_mla=False):
    return int(lib().orc_store_offset(C.c_int32(block_tokens), C.c_int32(heads_per_rank),
                                      C.c_int32(head_dim), C.c_int32(rank), C.c_int32(tp_size),
                                      C.c_int32(elem_bytes), C.c_int32(layer), C.c_int32(int(is_v)),
                                      C.c_int32(int(is_mla))))


def score_dot_gsa_heads(reps_f32, req_offsets, slot_ids, q_bf16, include_mask=None, exclude_mask=None):
    """GSA's device-side weights: mean over query heads of the per-head maximum over a block's representatives.
    reps_f32 [n_slots, H, n_rep, D] fp32; q_bf16 uint16 bits [n_req, Hq, D]."""
    reps = _c(reps_f32, np.float32)
    off = _c(req_offsets, np.int32)
    ids = _c(slot_ids, np.int32)
    q = _c(q_bf16, np.uint16)
    inc = _c(include_mask, np.uint8)
    exc = _c(exclude_mask, np.uint8)
    n_slots, H, n_rep, D = reps.shape
    n_req, Hq, _ = q.shape
    out = np.empty(int(off[-1]), np.float32)
    vp = lambda a: None if a is None else a.ctypes.data_as(C.c_void_p)
    lib().orc_score_dot_gsa_heads(vp(reps), C.c_int32(H), C.c_int32(n_rep), C.c_int32(D), vp(off), vp(ids), C.c_int32(n_req),
                                  vp(q), C.c_int32(Hq), vp(inc), vp(exc), vp(out))
    return out


# ------------------------------------------------------------------------- KVStar

def f32_to_f16_bits(x: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def kvstar_block_repre(k_bf16, ids, pruned, merge):
    """k_bf16: uint16 bf16 bits [num_blocks, T, H, D]; pruned: int64 [H, d_pruned] or None.
    Returns half bits [n, T/merge, H, d_pruned]."""
    k = _c(k_bf16, np.uint16)
    nb, T, H, D = k.shape
    ids = _c(ids, np.int32)
    pr = _c(pruned, np.int64)
    dp = D if pr is None else pr.shape[1]
    out = np.empty((len(ids), T // merge, H, dp), np.uint16)
    lib().orc_kvstar_block_repre(k.ctypes.data_as(C.c_void_p), C.c_int64(T * H * D), C.c_int64(H * D), C.c_int32(T),
                                 C.c_int32(H), C.c_int32(D), ids.ctypes.data_as(C.c_void_p), C.c_int32(len(ids)),
                                 None if pr is None else pr.ctypes.data_as(C.c_void_p), C.c_int32(dp), C.c_int32(merge),
                                 out.ctypes.data_as(C.c_void_p))
    return out


def kvstar_scores(q_f16, reps_f16, pruned=None):
    """q_f16: half bits [x, Hq, d_orig]; reps_f16: half bits [n, M, H, d_pruned]. Returns float32 [n]."""
    q = _c(q_f16, np.uint16)
    r = _c(reps_f16, np.uint16)
    pr = _c(pruned, np.int64)
    x, Hq, d_orig = q.shape
    n, M, H, dp = r.shape
    scratch = np.empty(x * Hq * n * M, np.float32)
    out = np.empty(n, np.float32)
    lib().orc_kvstar_scores(q.ctypes.data_as(C.c_void_p), C.c_int32(x), C.c_int32(Hq), C.c_int32(d_orig),
                            r.ctypes.data_as(C.c_void_p), C.c_int32(n), C.c_int32(M), C.c_int32(H), C.c_int32(dp),
                            None if pr is None else pr.ctypes.data_as(C.c_void_p), scratch.ctypes.data_as(C.c_void_p),
                            out.ctypes.data_as(C.c_void_p))
    return out


def kvstar_topk(scores, k):
    s = _c(scores, np.float32)
    out = np.empty(max(min(k, len(s)), 0), np.int64)
    cnt = lib().orc_kvstar_topk(s.ctypes.data_as(C.c_void_p), C.c_int32(len(s)), C.c_int32(k), out.ctypes.data_as(C.c_void_p))
    return out[:cnt]


# ------------------------------------------------------- the compiled reference

def have_ref() -> bool:
    return (os.path.isdir(_REF_DIR)
            and any(f.startswith("retrieval_backend") for f in os.listdir(_REF_DIR))
            and os.path.exists(os.path.join(_REF_DIR, "libgsa_ref.so")))


def ref_retrieval_backend():
    """The reference's ESA pybind11 module (retrieval_backend.cpp), compiled unmodified."""
    name = [f for f in os.listdir(_REF_DIR) if f.startswith("retrieval_backend")][0]
    spec = importlib.util.spec_from_file_location("retrieval_backend", os.path.join(_REF_DIR, name))
    mod = importlib.util.module_from_spec(spec)
    sys.modules.setdefault("retrieval_backend", mod)
    spec.loader.exec_module(mod)
    return mod


def have_prefetch_ref() -> bool:
    return os.path.isdir(_REF_DIR) and any(f.startswith("gsa_prefetch") for f in os.listdir(_REF_DIR))


def ref_gsa_prefetch():
    """The reference's GSA prefetch engine (ucm/sparse/gsa/prefetch/src/kvcache_pre.cpp + pybinds.cpp), compiled
    unmodified into its own Python module."""
    import torch  # noqa: F401  (the module links against libtorch)
    if "gsa_prefetch" in sys.modules:
        return sys.modules["gsa_prefetch"]
    name = [f for f in os.listdir(_REF_DIR) if f.startswith("gsa_prefetch")][0]
    spec = importlib.util.spec_from_file_location("gsa_prefetch", os.path.join(_REF_DIR, name))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["gsa_prefetch"] = mod
    spec.loader.exec_module(mod)
    return mod


def ref_prefetch_rounds(n_layers, block_table, owned_idx, free_idx, rounds, req_id=7, bs_index=1, idx_dtype="int32"):
    """Runs the reference engine for one request through several selection rounds, the way
    ucm/sparse/gsa/prefetch/prefetch_engine.py drives it (:88-94 construction, :329-379 first state, :203-233 a round).

    block_table[i]: physical block of logical block i; owned_idx: the logical blocks resident at the start
    (set_blocks_map's selectIndex); free_idx: those of them whose blocks start on the free list, in list order;
    rounds: list of integer arrays [n_layers, k] - the selected logical blocks of every layer.
    Returns one dict per round with, per layer: the block table the engine wrote, its load list (blocks, logical
    indices of all misses), the free list it left behind and its block -> logical map."""
    import time

    import torch
    mod = ref_gsa_prefetch()
    max_bs, max_len = bs_index + 2, len(block_table) + 4
    free_block = torch.zeros((n_layers, max_bs, max_len), dtype=torch.int32)
    free_len = torch.zeros((n_layers, max_bs), dtype=torch.int32)
    tables = [torch.zeros((n_layers, max_bs, max_len), dtype=torch.int32) for _ in range(2)]
    table_len = [torch.zeros((n_layers, max_bs), dtype=torch.int32) for _ in range(2)]
    eng = mod.GSAPrefetchEngineC(free_block, tables[0], free_len, table_len[0], False)
    eng.set_blocks_map(req_id, [int(b) for b in block_table], [int(i) for i in owned_idx])
    free_block[:, bs_index, : len(free_idx)] = torch.tensor([int(block_table[i]) for i in free_idx], dtype=torch.int32)
    free_len[:, bs_index] = len(free_idx)
    out = []
    for step, sel in enumerate(rounds):
        sel = np.asarray(sel)
        k = sel.shape[1]
        buf = torch.zeros((n_layers, 1, max_len), dtype=getattr(torch, idx_dtype))
        buf[:, 0, :k] = torch.from_numpy(sel.astype(np.int64))
        t, tl = tables[step % 2], table_len[step % 2]            # the caller alternates two tables (:205-214)
        eng.set_blocks_table_info(t, tl, buf, step)
        eng.run_async_prefetch_bs([req_id], [k], [bs_index], 0)
        deadline = time.time() + 30
        while not eng.get_prefetch_status():
            if time.time() > deadline:
                raise RuntimeError("reference prefetch engine did not finish")
            time.sleep(0.001)
        loads, misses, bmap = eng.obtain_load_blocks(), eng.obtain_miss_idxs(), eng.obtain_blocks_map()
        out.append({
            "table": [t[l, bs_index, : int(tl[l, bs_index])].tolist() for l in range(n_layers)],
            "load_blocks": [list(loads[0][l]) for l in range(n_layers)],
            "miss_idx": [list(misses[0][l]) for l in range(n_layers)],
            "free": [free_block[l, bs_index, : int(free_len[l, bs_index])].tolist() for l in range(n_layers)],
            "blocks_map": [{int(b): int(i) for b, i in bmap[req_id][l].items()} for l in range(n_layers)],
        })
    return out


_nfs = None


def have_nfs_ref() -> bool:
    return os.path.exists(os.path.join(_REF_DIR, "libnfs_ref.so"))


def ref_nfs() -> C.CDLL:
    """The reference's NFS-store space manager and file helpers (space_manager.cc,
    space_shard_layout.cc, space_shard_temp_layout.cc, file.cc, posix_file.cc) behind nfs_ref_shim.cpp."""
    global _nfs
    if _nfs is None:
        L = C.CDLL(os.path.join(_REF_DIR, "libnfs_ref.so"))
        L.nfsref_create.restype = C.c_void_p
        L.nfsref_create.argtypes = [C.c_char_p, C.c_size_t, C.c_int, C.POINTER(C.c_int)]
        L.nfsref_destroy.argtypes = [C.c_void_p]
        L.nfsref_new_block.argtypes = [C.c_void_p, C.c_char_p, C.c_size_t]
        L.nfsref_lookup_block.argtypes = [C.c_void_p, C.c_char_p, C.c_size_t]
        L.nfsref_commit_block.argtypes = [C.c_void_p, C.c_char_p, C.c_size_t, C.c_int]
        L.nfsref_data_path.argtypes = [C.c_void_p, C.c_char_p, C.c_size_t, C.c_int, C.c_char_p, C.c_size_t]
        L.nfsref_write.argtypes = [C.c_char_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_int]
        L.nfsref_read.argtypes = [C.c_char_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_int]
        _nfs = L
    return _nfs


class RefSpaceManager:
    """Thin object over ref_nfs(): the reference's SpaceManager on a set of backend directories."""

    def __init__(self, backends: str, block_size: int, temp_dir: bool = False):
        st = C.c_int(0)
        self.h = ref_nfs().nfsref_create(backends.encode(), block_size, int(temp_dir), C.byref(st))
        self.status = st.value
        if not self.h:
            raise RuntimeError(f"reference SpaceManager::Setup failed with {st.value}")

    def new_block(self, bid: bytes) -> int:
        return ref_nfs().nfsref_new_block(self.h, bid, len(bid))

    def commit(self, bid: bytes, success: bool = True) -> int:
        return ref_nfs().nfsref_commit_block(self.h, bid, len(bid), int(success))

    def lookup(self, bid: bytes) -> bool:
        return bool(ref_nfs().nfsref_lookup_block(self.h, bid, len(bid)))

    def path(self, bid: bytes, activated: bool) -> str:
        buf = C.create_string_buffer(4096)
        ref_nfs().nfsref_data_path(self.h, bid, len(bid), int(activated), buf, 4096)
        return buf.value.decode()

    @staticmethod
    def write(path: str, offset: int, data: np.ndarray, direct: bool = False) -> int:
        return ref_nfs().nfsref_write(path.encode(), offset, data.nbytes, data.ctypes.data, int(direct))

    @staticmethod
    def read(path: str, offset: int, out: np.ndarray, direct: bool = False) -> int:
        return ref_nfs().nfsref_read(path.encode(), offset, out.nbytes, out.ctypes.data, int(direct))


def have_kvstar_ref() -> bool:
    return all(os.path.exists(os.path.join(_REF_DIR, f)) for f in ("libkvstar_ref.so", "libkvstar_ref_scalar.so"))


_kvstar = {}


def ref_kvstar_topk(q_f16, reps_f16, pruned, topk, scalar=False):
    """KVStar::Execute of the reference (simd_compute_kernel.cpp) on one request: the selected block
    indices, in the order the reference returns them (scalar build: best first; AVX2 build: any order)."""
    name = "libkvstar_ref_scalar.so" if scalar else "libkvstar_ref.so"
    if name not in _kvstar:
        _kvstar[name] = C.CDLL(os.path.join(_REF_DIR, name))
    q = _c(q_f16, np.uint16)
    r = _c(reps_f16, np.uint16)
    pr = _c(pruned, np.int64)
    x, Hq, d_orig = q.shape
    n, M, H, dp = r.shape
    out = np.empty(max(topk, 1), np.int64)
    cnt = _kvstar[name].kvstar_ref_execute(q.ctypes.data_as(C.c_void_p), C.c_int64(x), C.c_int64(Hq), C.c_int64(d_orig),
                                           r.ctypes.data_as(C.c_void_p), C.c_int64(n), C.c_int64(M), C.c_int64(H),
                                           C.c_int64(dp), None if pr is None else pr.ctypes.data_as(C.c_void_p),
                                           C.c_int(topk), out.ctypes.data_as(C.c_void_p))
    if cnt < 0:
        raise RuntimeError("the reference kernel threw")
    return out[:cnt]


_gsa = None


def ref_gsa() -> C.CDLL:
    """The reference's GSA offload arithmetic (vec_product/k_repre/select_topk_block)."""
    global _gsa
    if _gsa is None:
        _gsa = C.CDLL(os.path.join(_REF_DIR, "libgsa_ref.so"))
    return _gsa


def ref_gsa_k_repre(k_f32):
    """k_f32: fp32 [n, H, T, D] (the layout the reference's KRepreComputer takes)."""
    k = _c(k_f32, np.float32)
    n, H, T, D = k.shape
    out = np.empty((n, H * D), np.float32)
    ref_gsa().gsa_ref_k_repre(_p(k), C.c_int64(H * T * D), C.c_uint32(n), C.c_uint32(H),
                              C.c_uint32(T), C.c_uint32(D), _p(out))
    return out


def ref_gsa_scores(q_mean_f32, reps_f32, n_kv_heads, n_rep, head_dim):
    q = _c(q_mean_f32, np.float32)
    reps = _c(reps_f32, np.float32)
    nb = reps.size // (n_kv_heads * n_rep * head_dim)
    out = np.empty(nb, np.float32)
    ref_gsa().gsa_ref_scores(_p(q), _p(reps), C.c_uint32(nb), C.c_uint32(n_kv_heads),
                             C.c_uint32(n_rep), C.c_uint32(head_dim), _p(out))
    return out


def ref_gsa_select_topk(q_f32, reps_f32, n_kv_heads, n_q_heads, n_rep, head_dim, start, end, k):
    q = _c(q_f32, np.float32).copy()
    reps = _c(reps_f32, np.float32)
    nb = reps.size // (n_kv_heads * n_rep * head_dim)
    out = np.full(max(nb, k), -1, np.int32)
    ref_gsa().gsa_ref_select_topk(_p(q), _p(reps), C.c_uint32(nb), C.c_uint32(n_kv_heads),
                                  C.c_uint32(n_q_heads), C.c_uint32(n_rep), C.c_uint32(head_dim),
                                  C.c_uint32(start), C.c_uint32(end), C.c_uint32(k), _p(out))
    return out


def ref_gsa_q_head_mean(q_f32, n_kv_heads):
    q = _c(q_f32, np.float32).copy()
    Hq, D = q.shape
    ref_gsa().gsa_ref_q_head_mean(_p(q), C.c_uint32(n_kv_heads), C.c_uint32(Hq), C.c_uint32(D))
    return q[:n_kv_heads].copy()
