"""The C++ template surface (include/cuv/*.hpp over libcuvdia.so): it must compile and link without a
GPU, and on a GPU its test program - CUV's own DIA tests restated - must pass."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "build", "test_cuv_surface")


def build_exe():
    from cuv_b200 import build
    build.build()
    subprocess.check_call(["make", "-C", os.path.join(ROOT, "tests", "cpp"), "-s"])
    return EXE


def test_surface_compiles_and_links():
    exe = build_exe()
    assert os.path.exists(exe)
    # every host-side template of the path resolves: no unresolved cuv:: symbol is left for run time
    out = subprocess.run(["nm", "-C", "-u", exe], capture_output=True, text=True).stdout
    assert "cuv::" not in out


@pytest.mark.gpu
def test_surface_program_passes_on_gpu():
    exe = EXE if os.path.exists(EXE) else build_exe()
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    print(r.stdout, r.stderr)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "0 failed" in r.stdout
