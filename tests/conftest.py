import glob
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


# a container may see every core of a big host while being allowed a few: keep the OpenMP runtimes modest
os.environ.setdefault("OMP_WAIT_POLICY", "PASSIVE")
if "OMP_NUM_THREADS" not in os.environ:
    try:
        os.environ["OMP_NUM_THREADS"] = str(min(16, len(os.sched_getaffinity(0))))
    except AttributeError:
        os.environ["OMP_NUM_THREADS"] = "8"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(autouse=True)
def _stack_dump_if_stuck():
    """If a test sits in one call for two minutes, the Python stacks of all threads go to stderr (the run goes on)."""
    import faulthandler
    faulthandler.dump_traceback_later(120, exit=False)
    yield
    faulthandler.cancel_dump_traceback_later()


def golden_cases(prefix):
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, prefix + "*.npz")))


def load_golden(name):
    return dict(np.load(os.path.join(GOLDEN, name + ".npz"), allow_pickle=False))


@pytest.fixture(scope="session")
def port():
    from oracle import oracle as orc
    orc.build()
    return orc.Port()


@pytest.fixture(scope="session")
def reference():
    from oracle import oracle as orc
    if not orc.Reference.available():
        pytest.skip("oracle/_ref was not built here (needs the reference sources at build time)")
    return orc.Reference()


@pytest.fixture(scope="session")
def checker():
    """The strongest CPU checker present: the compiled reference operators, else the C restatement."""
    from oracle import oracle as orc
    orc.build()
    return orc.best()


def same_bits(a, b):
    """fp32 equality that treats +0 and -0 as equal (relu / leaky_relu may differ in the sign of zero)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    return a.shape == b.shape and bool(np.all((a.view(np.int32) == b.view(np.int32)) | ((a == 0) & (b == 0))))
