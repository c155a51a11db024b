import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")
    config.addinivalue_line("markers", "multigpu: needs at least two CUDA devices")
    config.addinivalue_line("markers", "first_device_run: a blocking test whose path now rides kernels that have not run on a device yet")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        n = 0
    skip_gpu = pytest.mark.skip(reason="no CUDA device")
    skip_multi = pytest.mark.skip(reason="needs >= 2 CUDA devices")
    for item in items:
        if "gpu" in item.keywords and n == 0:
            item.add_marker(skip_gpu)
        if "multigpu" in item.keywords and n < 2:
            item.add_marker(skip_multi)
    # Kernels that have never run on a device (their tests carry a non-strict expected-failure mark) go last: should
    # one of them lose the context, every test of a kernel that is known to work has already run and been recorded.
    # Blocking tests whose path now includes such kernels run after the plain ones and before those.
    def rank(it):
        if "gpu" not in it.keywords:
            return 0
        if it.get_closest_marker("xfail") is not None:
            return 2
        return 1 if it.get_closest_marker("first_device_run") is not None else 0
    items.sort(key=rank)


# ---- required-case gate ----------------------------------------------------------------------------------------------
_outcomes = {}


def pytest_runtest_logreport(report):
    if report.when == "call" or (report.when == "setup" and report.skipped):
        kind = "skipped" if report.skipped and not hasattr(report, "wasxfail") else report.outcome
        if hasattr(report, "wasxfail"):
            kind = "xfailed" if report.skipped else "xpassed"
        _outcomes[report.nodeid] = kind


def _cuda_devices() -> int:
    try:
        import torch
        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        return 0


def pytest_sessionfinish(session, exitstatus):
    """A required case that was selected but did not really run (skipped, expected failure, unexpected pass under a
    non-strict mark) fails the run."""
    from required_cases import CPU, GPU
    required = list(CPU) + (list(GPU) if _cuda_devices() > 0 else [])
    bad = sorted((nid, kind) for nid, kind in _outcomes.items()
                 if kind in ("skipped", "xfailed", "xpassed") and any(nid.startswith(p) for p in required))
    if bad:
        tr = session.config.pluginmanager.get_plugin("terminalreporter")
        msg = "required cases did not run: " + ", ".join(f"{n} ({k})" for n, k in bad[:20])
        if tr is not None:
            tr.write_line(msg, red=True)
        else:
            print(msg)
        if session.exitstatus == 0:
            session.exitstatus = 1
