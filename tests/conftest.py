import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def pkg():
    import __graft_entry__ as entry
    p = entry.load_package()
    if not p.cu32.LIB_PATH.exists():
        entry.build()
    return p


@pytest.fixture(scope="session")
def O():
    from oracle import oracle
    oracle.build()
    return oracle


@pytest.fixture(scope="session")
def golden():
    sys.path.insert(0, str(ROOT / "tests" / "golden"))
    import make_golden
    return make_golden


@pytest.fixture(scope="session")
def cuda(pkg):
    """torch with cuda:0 selected; the library must be the thing that runs."""
    import torch
    assert torch.cuda.is_available(), "gpu-marked test without a CUDA device"
    torch.cuda.set_device(0)
    pkg.cu32.load()
    return torch


@pytest.fixture(autouse=True)
def _default_tuning(request):
    """GPU tests that change tuning knobs must not leak them into later tests."""
    yield
    if "gpu" in request.keywords:
        import __graft_entry__ as entry
        p = entry.load_package()
        p.cu32.tune("tile", -1)
        p.cu32.tune("kc", DEFAULT_KC["kc"])
        p.cu32.tune("kc_fast", DEFAULT_KC["kc_fast"])
        for key in ("ring_raw", "ring_lo", "store_bufs", "arrive_release", "sm_reserve", "gather"):
            p.cu32.tune(key, 0)
        p.cu32.tune("phase_overlap", 1)
        p.cu32.tune("rep_lazy", 1)
        p.cu32.tune("ring_fixed", 1)
        p.cu32.tune("phase_fused", 1)
        p.cu32.tune("ring_paired", 1)


DEFAULT_KC = {"kc": 2, "kc_fast": 4}
