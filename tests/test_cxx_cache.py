"""chromofold::CompressedKvCache, the reference's C++ cache class re-stated as a header-only front of the adapter ABI
(include/chromofold_b200/compressed_kv_cache.hpp): a C++ program is compiled against the header and the shared
library, as a maintainer's code would be, and run."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SOURCE = os.path.join(ROOT, "tests", "cxx", "compressed_kv_cache_check.cpp")


def _build(native, where):
    native.lib()                                   # the library must be there
    gxx = shutil.which("g++")
    assert gxx, "g++ is needed to build the C++ check"
    exe = os.path.join(str(where), "compressed_kv_cache_check")
    libdir = os.path.dirname(native.LIB_PATH)
    cmd = [gxx, "-std=c++17", "-O1", "-Wall", "-Werror", "-I" + os.path.join(ROOT, "include"), SOURCE, "-o", exe,
           "-L" + libdir, "-lchromofold_b200", "-Wl,-rpath," + libdir]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr
    return exe


def test_cxx_cache_contract(native, tmp_path):
    exe = _build(native, tmp_path)
    proc = subprocess.run([exe, "contract"], capture_output=True, text=True, timeout=120)
    assert proc.returncode == 0 and "contract ok" in proc.stdout, proc.stderr


@pytest.mark.gpu
def test_cxx_cache_equals_the_adapter(native, tmp_path):
    exe = _build(native, tmp_path)
    proc = subprocess.run([exe, "gpu"], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0 and "gpu ok" in proc.stdout, proc.stdout + proc.stderr
