"""ctypes binding of libucmx.so, the C ABI declared in include/ucmx.h.

There is no fallback: if the library is missing or does not export a declared symbol, importing
this module raises.  Build it with `python unified-cache-management_b200/build.py`.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_lib", "libucmx.so")

OK = 0
ERROR = -1
EPARAM = -50000
EOOM = -50001
EOSERROR = -50002
EDUPLICATE = -50003
ENOOBJ = -50005
EUNSUPPORTED = -50008

DT_BF16, DT_F32, DT_I32 = 0, 1, 2
POOL_MEAN, POOL_MAX, POOL_MIN, POOL_SUM = 0, 1, 2, 3
WIN_NONE, WIN_FORCE, WIN_EXCLUDE = 0, 1, 2
ORDER_SCORE_DESC, ORDER_INDEX_ASC = 0, 1

_STATUS_NAMES = {
    OK: "OK", ERROR: "ERROR", EPARAM: "EPARAM", EOOM: "EOOM", EOSERROR: "EOSERROR", EDUPLICATE: "EDUPLICATE",
    ENOOBJ: "ENOOBJ", EUNSUPPORTED: "EUNSUPPORTED",
}


class UcmxError(RuntimeError):
    def __init__(self, fn: str, status: int, detail: str = ""):
        self.status = status
        name = _STATUS_NAMES.get(status, str(status))
        super().__init__(f"{fn} failed with {name} ({status})" + (f": {detail}" if detail else ""))


class KvGeometry(C.Structure):
    _fields_ = [
        ("block_stride", C.c_int64),
        ("token_stride", C.c_int64),
        ("block_tokens", C.c_int32),
        ("n_kv_heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("reserved", C.c_int32),
    ]


_vp, _i32, _i64, _f32, _sz = C.c_void_p, C.c_int32, C.c_int64, C.c_float, C.c_size_t
_pvp = C.POINTER(C.c_void_p)
_pi32 = C.POINTER(C.c_int32)

# name -> argtypes; every entry returns int32 unless listed in _RESTYPES
SIGNATURES = {
    "ucmx_version": [],
    "ucmx_set_early_start": [_i32],
    "ucmx_compiled_arch": [],
    "ucmx_last_error": [],
    "ucmx_device_error": [_pi32, _i32],
    "ucmx_pool_blocks": [_vp, C.POINTER(KvGeometry), _vp, _vp, _i64, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp],
    "ucmx_hash_encode": [_vp, _i64, _i64, _vp, _i32, _i32, _vp, _vp],
    "ucmx_hash_encode_blocks": [_vp, C.POINTER(KvGeometry), _vp, _vp, _i64, _i32, _vp, _i32, _i32, _vp, _vp],
    "ucmx_query_group_mean": [_vp, _i32, _i32, _i32, _i32, _i64, _i32, _vp, _vp],
    "ucmx_score_dot": [_vp, _i32, _i64, _i32, _i32, _i32, _vp, _vp, _vp, _i32, _i32, _f32, _vp, _vp, _vp],
    "ucmx_score_dot_query": [_vp, _i32, _i64, _i32, _i32, _vp, _vp, _vp, _i32, _i64, _i32, _i32, _i32, _f32, _vp, _vp, _vp],
    "ucmx_score_dot_heads": [_vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp, _i32, _i64, _i32, _i32, _vp, _vp, _vp, _vp],
    "ucmx_score_hamming": [_vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp],
    "ucmx_topk_ragged": [_vp, _i32, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _i32, _vp, _vp, _vp, _vp, _vp],
    "ucmx_peer_exchange_bytes": [_i32, _i64],
    "ucmx_topk_ragged_peer_sum": [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _i32, _vp, _vp, _vp, _vp,
                                  _vp],
    "ucmx_remap_resident": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp],
    "ucmx_retrieve_topk_noalloc": [_vp, _i32, _i64, _i32, _i32, _i32, _vp, _vp, _vp, _i32, _i32, _f32, _vp, _i32, _i32, _i32,
                                   _i32, _vp, _i32, _vp, _vp, _vp, _vp, _vp],
    "ucmx_noalloc_max_candidates": [],
    "ucmx_gather_blocks": [_pvp, _i32, _i64, _i64, _vp, _i32, _i64, _vp, _i32, _vp],
    "ucmx_scatter_blocks": [_pvp, _i32, _i64, _i64, _vp, _i32, _i64, _vp, _i32, _vp],
    "ucmx_move_blocks": [_pvp, _pvp, _i32, _i64, _i64, _vp, _i64, _i64, _vp, _i32, _vp, _i64, _vp],
    "ucmx_copy_batch": [_vp, _vp, _i32, _i64, _i32, _vp],
    "ucmx_memcpy_async": [_vp, _vp, _i64, _vp],
    "ucmx_ring_create": [_sz, _sz, _pvp],
    "ucmx_ring_acquire": [_vp, _pvp, _pi32],
    "ucmx_ring_release": [_vp, _i32],
    "ucmx_ring_base": [_vp, _pvp, C.POINTER(_sz), C.POINTER(_sz)],
    "ucmx_ring_destroy": [_vp],
    "ucmx_task_create": [_pvp],
    "ucmx_task_record": [_vp, _vp],
    "ucmx_task_check": [_vp, _pi32],
    "ucmx_task_wait": [_vp, _i64],
    "ucmx_task_destroy": [_vp],
    "ucmx_retrieval_create": [_vp, _i64, _i32, _i32, _i32, _pvp],
    "ucmx_retrieval_update_rows": [_vp, _vp, _i32, _vp],
    "ucmx_retrieval_table": [_vp, _pvp, _pi32],
    "ucmx_retrieval_submit": [_vp, _vp, _i32, _i32, _i32, _vp, _i32, _pi32],
    "ucmx_retrieval_flush": [_vp],
    "ucmx_retrieval_launches": [_vp, C.POINTER(C.c_int64)],
    "ucmx_retrieval_poll": [_vp, _i32, _pi32],
    "ucmx_retrieval_wait": [_vp, _i32],
    "ucmx_retrieval_result_shape": [_vp, _i32, _pi32, _pi32],
    "ucmx_retrieval_get_result": [_vp, _i32, _vp, _vp],
    "ucmx_retrieval_destroy": [_vp],
    "ucmx_fstore_create": [C.c_char_p, _sz, _i32, _i32, _i32, _sz, _sz, _sz, _sz, _pvp],
    "ucmx_fstore_destroy": [_vp],
    "ucmx_fstore_path": [_vp, C.c_char_p, _sz, _i32, C.c_char_p, _sz],
    "ucmx_fstore_alloc": [_vp, C.c_char_p, _sz],
    "ucmx_fstore_lookup": [_vp, C.c_char_p, _sz, _pi32],
    "ucmx_fstore_commit": [_vp, C.c_char_p, _sz, _i32],
    "ucmx_fstore_submit": [_vp, _i32, _i32, C.POINTER(C.c_char_p), C.POINTER(_sz), C.POINTER(_sz),
                           C.POINTER(C.c_size_t), C.POINTER(_sz), _sz, C.POINTER(_sz)],
    "ucmx_fstore_wait": [_vp, _sz],
    "ucmx_fstore_check": [_vp, _sz, _pi32],
    "ucmx_kvstar_block_repre": [_vp, C.POINTER(KvGeometry), _vp, _vp, _i64, _i32, _vp, _i32, _i32, _vp, _vp],
    "ucmx_kvstar_kernel_choice": [_i32, _i32, _i32, _i32, _i32, _i32],
    "ucmx_kvstar_workspace_bytes": [_i32, _i32, _i32, _i32, _i32],
    "ucmx_kvstar_scores": [_vp, _i32, _i32, _i32, _i32, _vp, _vp, _i32, _i32, _vp, _vp, _i32, _i32, _i32, _vp, _vp, _sz,
                           _vp, _vp],
}
_RESTYPES = {"ucmx_last_error": C.c_char_p, "ucmx_kvstar_workspace_bytes": C.c_size_t,
             "ucmx_peer_exchange_bytes": C.c_size_t}


class RemapMoves(C.Structure):
    """ucmx_remap_moves: the packed (pool block -> HBM block) move list a remap round writes for ucmx_move_blocks."""
    _fields_ = [("src_map", C.c_void_p), ("src_map_offsets", C.c_void_p), ("move_src", C.c_void_p),
                ("move_dst", C.c_void_p), ("move_count", C.c_void_p)]


class PeerExchange(C.Structure):
    """ucmx_peer_exchange: where a tensor-parallel rank's partial scores go."""
    _fields_ = [("bases", C.c_void_p), ("world", C.c_int32), ("my_rank", C.c_int32), ("n_scores", C.c_int64)]


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: the CUDA extension has not been built "
            "(run `python unified-cache-management_b200/build.py`). There is no CPU fallback."
        )
    lib = C.CDLL(LIB_PATH)
    for name, argtypes in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:  # pragma: no cover - a stale build
            raise ImportError(f"{LIB_PATH} does not export {name}; rebuild it") from e
        fn.argtypes = argtypes
        fn.restype = _RESTYPES.get(name, C.c_int32)
    return lib


lib = _load()
launch_count = 0  # kernels launched through this binding (each checked call below launches >= 1)


def last_error() -> str:
    s = lib.ucmx_last_error()
    return s.decode() if s else ""


def check(fn_name: str, status: int, launches: int = 1) -> None:
    global launch_count
    if status != OK:
        raise UcmxError(fn_name, status, last_error())
    launch_count += launches


def device_error(clear: bool = True) -> int:
    code = C.c_int32(0)
    st = lib.ucmx_device_error(C.byref(code), 1 if clear else 0)
    if st != OK:
        raise UcmxError("ucmx_device_error", st)
    return code.value
