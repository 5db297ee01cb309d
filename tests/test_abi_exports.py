"""The C-ABI library loads and exports every function include/ucmx.h declares (no GPU needed)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared():
    text = open(os.path.join(ROOT, "include", "ucmx.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ucmx_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_path():
    names = declared()
    for must in ("ucmx_pool_blocks", "ucmx_hash_encode", "ucmx_score_dot", "ucmx_score_hamming",
                 "ucmx_topk_ragged", "ucmx_gather_blocks", "ucmx_scatter_blocks", "ucmx_retrieval_submit"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from ucmx import _native
    lib = ctypes.CDLL(_native.LIB_PATH)
    missing = [n for n in declared() if not hasattr(lib, n)]
    assert not missing, missing
    assert set(declared()) == set(_native.SIGNATURES), set(declared()) ^ set(_native.SIGNATURES)
    assert lib.ucmx_compiled_arch() == 100


def test_parameter_errors_need_no_gpu():
    from ucmx import _native as N
    # argument validation happens before any CUDA call
    assert N.lib.ucmx_pool_blocks(None, None, None, None, 1, 1, 0, 1, 1, 0, None, None, None) == N.EPARAM
    assert N.lib.ucmx_topk_ragged(None, 1, None, None, 3, 0, 0, 0, 0, None, 4, None, None, None, None, None) == N.EPARAM
    assert N.lib.ucmx_score_dot(None, 0, 0, 8, 1, 128, None, None, None, 0, 0, 1.0, None, None, None) == N.OK  # empty batch
    assert N.lib.ucmx_ring_release(None, 0) == N.EPARAM


def test_early_start_switch_is_per_thread_and_returns_the_previous_setting():
    import threading
    from ucmx import _native as N
    assert N.lib.ucmx_set_early_start(1) == 0
    seen = []
    t = threading.Thread(target=lambda: seen.append(N.lib.ucmx_set_early_start(0)))
    t.start()
    t.join()
    assert seen == [0]                       # another thread has its own setting
    assert N.lib.ucmx_set_early_start(0) == 1
    assert N.lib.ucmx_set_early_start(0) == 0
