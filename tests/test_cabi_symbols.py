"""The C-ABI library loads without a GPU and exports every function that
include/katsu_cuda.h declares; the ctypes table covers the same set."""
import ctypes
import os
import re

from katsu_b200 import cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "katsu_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(katsu_cuda_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_groups():
    names = declared_functions()
    for must in ("katsu_cuda_init", "katsu_cuda_conv2d_fwd", "katsu_cuda_conv2d_bwd", "katsu_cuda_matmul_fwd",
                 "katsu_cuda_matmul_bwd", "katsu_cuda_allreduce_sum", "katsu_cuda_sum"):
        assert must in names


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(cabi.LIB_PATH)
    missing = [name for name in declared_functions() if not hasattr(lib, name)]
    assert not missing, missing


def test_ctypes_table_matches_header():
    table = set(cabi.SIGNATURES) | {"katsu_cuda_last_error_string"}
    assert table == set(declared_functions())


def test_no_device_is_reported_not_hidden():
    """Without a GPU the context cannot be created and says so (no CPU path)."""
    lib = cabi.load()
    count = ctypes.c_int32(-1)
    rc = lib.katsu_cuda_device_count(ctypes.byref(count))
    if rc == cabi.OK and count.value > 0:
        return  # a GPU is present; nothing to check here
    handle = ctypes.c_void_p()
    rc = lib.katsu_cuda_init(0, ctypes.byref(handle))
    assert rc == cabi.ERR_NO_DEVICE
    assert lib.katsu_cuda_last_error_string()
