import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    # GPU tests never silently pass on a box without a GPU: they are skipped with a reason,
    # and on a GPU box a missing CUDA library is an error, not a skip.
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    """A fixture file as a dict of torch tensors; bf16 payloads come back as bf16."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    bf16 = bool(z["bf16"]) if "bf16" in z.files else False
    out = {}
    for k in z.files:
        if k == "bf16":
            continue
        t = torch.from_numpy(np.ascontiguousarray(z[k]))
        if bf16 and t.dtype == torch.int16:
            t = t.view(torch.bfloat16)
        out[k] = t
    out["_bf16"] = bf16
    return out


def golden_names(prefix):
    return sorted(f[:-4] for f in os.listdir(GOLDEN) if f.startswith(prefix) and f.endswith(".npz"))


def bits(t):
    """Bit pattern view for exact comparison of floating tensors (NaN-safe, sign-of-zero-safe)."""
    t = t.detach().cpu().contiguous()
    return t.view(torch.int32) if t.dtype == torch.float32 else t.view(torch.int16)


@pytest.fixture(scope="session")
def cuda_lib():
    """The built CUDA library; on a GPU box its absence is a failure."""
    from robogoat_b200 import _lib
    return _lib.load()


# bulk-copy waits that tests made run out on purpose (RC_OPT_BULK_WAIT_LIMIT = 0); any other event is a failure
DELIBERATE_BULK_TIMEOUTS = [0]


def bulk_wait_timeouts(lib) -> int:
    import ctypes
    n = ctypes.c_uint32(0)
    assert lib.rc_bulk_wait_timeouts(0, ctypes.byref(n)) == 0
    return int(n.value)


@pytest.fixture(scope="session", autouse=True)
def no_unexpected_bulk_wait_timeouts():
    """At the end of a GPU session: the staged kernel's bounded wait fired only where a test asked it to."""
    yield
    if torch.cuda.is_available():
        from robogoat_b200 import _lib
        assert bulk_wait_timeouts(_lib.load()) == DELIBERATE_BULK_TIMEOUTS[0]


@pytest.fixture(params=["staged-block", "row-gather"])
def kernel_choice(request, cuda_lib):
    """Runs a test once with the TMA-staged block kernel allowed (it is used where shapes qualify)
    and once with the row-gather kernel forced; both must produce the same bits."""
    cuda_lib.rc_set_option(0, 1 if request.param == "staged-block" else 0)
    yield request.param
    cuda_lib.rc_set_option(0, 1)
