"""The checked build variant (``libvsk_cuda_checked.so``): every global load, store and atomic of every kernel goes
through a range test against the buffers the library allocated and the buffers the caller announced.  It stands in
for compute-sanitizer's memcheck where that tool cannot run.  The first test re-runs the known-answer tests, the odd
small shapes and the per-kernel parity suites in a child process with VSK_CHECKED=1; tests/conftest.py then fails any
test during which an access was refused.  The second (which only runs inside that child process) is the positive
control: one read just past a buffer's announced end is refused and reported, and nothing faults."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHECKED = os.environ.get("VSK_CHECKED", "0") not in ("", "0")

SUITES = ["tests/test_gpu_checked.py", "tests/test_gpu_odd_shapes.py", "tests/test_gpu_flat.py",
          "tests/test_gpu_stream_scan.py", "tests/test_gpu_filters.py", "tests/test_gpu_ivf_sq8.py",
          "tests/test_gpu_pq.py", "tests/test_gpu_image.py", "tests/test_gpu_store.py"]


@pytest.mark.skipif(CHECKED, reason="this is the child process")
def test_parity_suites_under_the_checked_build():
    lib = os.path.join(ROOT, "vectorstorekit_b200", "libvsk_cuda_checked.so")
    assert os.path.exists(lib), "build it with `python -m vectorstorekit_b200.build --checked`"
    env = dict(os.environ, VSK_CHECKED="1")
    r = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-m", "gpu", "-p", "no:cacheprovider"] + SUITES,
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=3000)
    tail = "\n".join(r.stdout.strip().splitlines()[-25:])
    assert r.returncode == 0, f"checked run failed:\n{tail}\n{r.stderr[-2000:]}"
    assert " passed" in tail


@pytest.mark.skipif(not CHECKED, reason="needs the checked build (VSK_CHECKED=1)")
@pytest.mark.expects_refused_access
def test_a_read_past_the_announced_end_is_refused_and_reported():
    import vectorstorekit_b200 as vsk
    dev = vsk.CUDAComputeDevice(0)
    try:
        assert dev._lib.vsk_checked_build() == 1
        dev.checked_faults()                         # clear
        dev.checked_selftest()
        count, addr, info = dev.checked_faults()
        assert count == 1 and (info & 0xff) == 4 and not (info & 0x100) and not (info & 0x200), (count, hex(addr), info)
        assert dev.checked_faults()[0] == 0          # reading resets
        # the context is intact: a search right after
        import numpy as np
        x = np.eye(8, dtype=np.float32)
        ix = vsk.FlatIndex(dev, 8, "euclidean")
        ix.add(x)
        d, i = ix.batchSearch(x[:2], 1)
        assert i[:, 0].tolist() == [0, 1]
        ix.close()
        assert dev.checked_faults()[0] == 0
    finally:
        dev.close()


@pytest.mark.skipif(CHECKED, reason="the normal library")
def test_the_normal_library_answers_that_it_is_not_checked():
    import vectorstorekit_b200 as vsk
    dev = vsk.CUDAComputeDevice(0)
    try:
        assert dev._lib.vsk_checked_build() == 0
        assert dev.checked_faults() == (0, 0, 0)
        with pytest.raises(vsk.UnsupportedOperation):
            dev.checked_selftest()
    finally:
        dev.close()
