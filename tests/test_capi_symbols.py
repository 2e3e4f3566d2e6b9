"""CPU checks of the C-ABI boundary: the library builds, loads, exports exactly the symbols
include/cuvdia.h declares, checks preconditions before touching CUDA, and fails loudly (no
fallback) when no device is present."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def capi():
    from cuv_b200 import build, _capi
    build.build()
    return _capi


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "cuvdia.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"CUVDIA_API\s+[\w\s\*]+?\b(cuvdia_\w+)\s*\(", text)))


def test_header_symbols_all_exported_and_bound(capi):
    names = declared_symbols()
    assert len(names) >= 12
    L = capi.lib()
    for n in names:
        assert hasattr(L, n), n + " is declared in include/cuvdia.h but not exported"
    assert sorted(capi.SIGNATURES) == names


def test_error_strings(capi):
    L = capi.lib()
    assert L.cuvdia_error_string(0) == b"success"
    assert b"precondition" in L.cuvdia_error_string(capi.ERR_INVALID)


def test_preconditions_checked_before_cuda(capi):
    L = capi.lib()
    plan = ctypes.c_void_p()
    offs = np.array([0, 1, 1], dtype=np.int32)
    op = offs.ctypes.data_as(ctypes.POINTER(ctypes.c_int))
    assert L.cuvdia_plan_create(ctypes.byref(plan), 8, 8, 0, 8, 1, op) == capi.ERR_INVALID
    assert L.cuvdia_last_error_message() == b"num_dia > 0"
    assert L.cuvdia_plan_create(ctypes.byref(plan), 8, 8, 2, 8, 0, op) == capi.ERR_INVALID
    assert L.cuvdia_last_error_message() == b"row_fact > 0"
    assert L.cuvdia_plan_create(ctypes.byref(plan), 8, 8, 2, 4, 1, op) == capi.ERR_INVALID
    assert L.cuvdia_last_error_message() == b"stride >= h"
    assert L.cuvdia_prod_f32(None, None, None, 0, None, 0, 0, b"n", b"n", 1.0, 0.0, 0, None) == capi.ERR_INVALID
    assert L.cuvdia_reduce_f32(None, None, 1, 1, 0, 0, 1.0, 0.0, None) == capi.ERR_INVALID
    assert L.cuvdia_plan_destroy(None) == 0
    # the entry points of the device-drawn uniform numbers: a draw descriptor is required and its fields are ranged
    d = capi.Draw(1, 0, 0)
    buf = ctypes.c_void_p(16)                            # never dereferenced: the checks come before any CUDA call
    for fn in (L.cuvdia_uniform_f32, L.cuvdia_rnd_binarize_f32):
        assert fn(buf, 8, 8, 1, None, 0, None) == capi.ERR_INVALID
        assert fn(None, 8, 8, 1, ctypes.byref(d), 0, None) == capi.ERR_INVALID
        assert fn(buf, 4, 8, 1, ctypes.byref(d), 0, None) == capi.ERR_INVALID          # ld < rows
        assert fn(buf, 8, 8, 1, ctypes.byref(d), 65536, None) == capi.ERR_INVALID      # draw index of 16 bits
        assert fn(buf, 8, 8, 1, ctypes.byref(capi.Draw(1, 1 << 32, 0)), 0, None) == capi.ERR_INVALID
        assert fn(buf, 8, 8, 1, ctypes.byref(capi.Draw(1, 0, -1)), 0, None) == capi.ERR_INVALID
        assert fn(buf, 8, 8, 0, ctypes.byref(d), 0, None) == 0                         # no columns: nothing to do


def test_no_cpu_fallback(capi):
    """Without a CUDA device a compute call must fail with a CUDA error, never compute on the CPU."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    L = capi.lib()
    plan = ctypes.c_void_p()
    offs = np.array([0, 1], dtype=np.int32)
    rc = L.cuvdia_plan_create(ctypes.byref(plan), 8, 8, 2, 8, 1, offs.ctypes.data_as(ctypes.POINTER(ctypes.c_int)))
    assert rc == capi.ERR_CUDA and not plan.value
    with pytest.raises(capi.CuvDiaError):
        capi.check(rc)


def test_product_package_does_not_use_the_oracle():
    for dirpath, _, files in os.walk(os.path.join(ROOT, "cuv_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".hpp")):
                assert "oracle" not in open(os.path.join(dirpath, f)).read().lower(), f
