"""Shared pytest configuration: the `gpu` marker and the repo root on sys.path.

`-m "not gpu"` covers the CPU oracle against the reference's known answers, the host-side
logic and the C-ABI export check; `-m gpu` holds the kernel-vs-oracle parity tests, which all
go through the C ABI of libb200tp.so.
"""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU and the built CUDA library")


def pytest_terminal_summary(terminalreporter):
    """Worst observed error of every tolerance class the parity tests recorded (tests/_worst.py)."""
    import importlib
    worst = sys.modules.get("_worst") or importlib.import_module("_worst")   # the module object the tests filled
    WORST = worst.WORST
    if not WORST:
        return
    tr = terminalreporter
    tr.write_sep("-", "worst observed error / tolerance per class")
    for name in sorted(WORST):
        value, tol, n = WORST[name]
        tr.write_line(f"{name:58s} {value:10.3e} / {tol:8.1e}  ({100 * value / tol:5.1f} % of the tolerance, {n} checks)")


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)
