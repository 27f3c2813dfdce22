"""CPU-side checks of the boundary: the library loads without a GPU, exports every symbol the
header declares, and refuses to open a device that is not there (no CPU fallback)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from vectorstorekit_b200 import build, _lib
    build.build_library()
    return _lib.load()


def _declared():
    text = open(os.path.join(ROOT, "include", "vsk_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vsk_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    from vectorstorekit_b200 import _lib
    names = _declared()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in vsk_cuda.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), set(names) ^ set(_lib.SIGNATURES)


def test_header_compiles_as_c():
    import subprocess, tempfile
    with tempfile.TemporaryDirectory() as t:
        src = os.path.join(t, "t.c")
        open(src, "w").write('#include "vsk_cuda.h"\nint main(void){return VSK_OK;}\n')
        subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-c", src,
                        "-o", os.path.join(t, "t.o")], check=True)


def test_status_strings(lib):
    assert lib.vsk_status_string(0) == b"ok"
    assert lib.vsk_status_string(9) == b"empty input"


def test_no_cpu_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    assert lib.vsk_open(0, C.byref(h)) == 1  # VSK_ERR_DEVICE_NOT_AVAILABLE
    import vectorstorekit_b200 as vsk
    with pytest.raises(vsk.DeviceNotAvailable):
        vsk.CUDAAcceleratorStrategy().initialize()


def test_product_does_not_import_oracle():
    pkg = os.path.join(ROOT, "vectorstorekit_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".hpp", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower().replace("oracle/", "oracle/") or "import oracle" not in text


def test_unsupported_metric_raises():
    import vectorstorekit_b200 as vsk
    from vectorstorekit_b200.engine import _metric_id
    with pytest.raises(vsk.UnsupportedOperation):
        _metric_id(vsk.DistanceMetric.hamming)
    assert _metric_id("cosine") == 1


def _build_host_mirror(tmp):
    import subprocess
    exe = os.path.join(tmp, "host_mirror_test")
    subprocess.run(["g++", "-std=c++17", "-O1", os.path.join(ROOT, "tests", "host_mirror_test.cpp"), "-o", exe,
                    "-L", os.path.join(ROOT, "vectorstorekit_b200"), "-lvsk_cuda",
                    "-Wl,-rpath," + os.path.join(ROOT, "vectorstorekit_b200")], check=True)
    return exe


def test_cpp_host_mirror_compiles_and_refuses_without_gpu(lib, tmp_path):
    import subprocess
    import torch
    exe = _build_host_mirror(str(tmp_path))
    out = subprocess.run([exe], capture_output=True, text=True)
    assert out.returncode == 0, out
    assert out.stdout.strip() == ("ok" if torch.cuda.is_available() else "no-device")
