import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")
    config.addinivalue_line("markers", "expects_refused_access: the test makes the checked build refuse an access")


@pytest.fixture(scope="session")
def cpu_oracle():
    import oracle

    return oracle.CpuOracle()


@pytest.fixture(scope="session")
def metal_ref():
    import oracle

    if not oracle.MetalRef.available():
        pytest.skip("reference shader build (oracle/_ref) not present")
    return oracle.MetalRef()


# Under the checked build variant (VSK_CHECKED=1: every global access of every kernel is range-tested, see
# vectorstorekit_b200/ptx_check.py) every GPU test also asserts that no access was refused while it ran.
_checked_dev = None


@pytest.fixture(autouse=True)
def _no_refused_access_under_the_checked_build(request):
    yield
    from vectorstorekit_b200 import _lib
    if not _lib.CHECKED or request.node.get_closest_marker("gpu") is None:
        return
    global _checked_dev
    if _checked_dev is None:
        import vectorstorekit_b200 as vsk
        _checked_dev = vsk.CUDAComputeDevice(0)
    count, addr, info = _checked_dev.checked_faults()
    if request.node.get_closest_marker("expects_refused_access") is None:
        assert count == 0, (f"{count} accesses refused by the checked build; first: address {addr:#x}, "
                            f"{info & 0xff} bytes, {'write' if info & 0x100 else 'read'}"
                            f"{', misaligned' if info & 0x200 else ''}")
