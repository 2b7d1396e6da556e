import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def engine():
    """One libprad_cuda context for the whole GPU session (fails loudly without a GPU)."""
    from parallelreverseautodiff_b200.engine import Engine

    eng = Engine(0)
    yield eng
    eng.close()


def pytest_terminal_summary(terminalreporter):
    """Share of each stated tolerance that the comparisons of this run used (err / limit)."""
    try:
        from util import HEADROOM
    except ImportError:
        return
    rows = [(k, v) for k, v in HEADROOM.items() if v > 0]
    if not rows:
        return
    terminalreporter.write_line("tolerance used (max err / limit) per comparison:")
    for k, v in sorted(rows, key=lambda kv: -kv[1]):
        terminalreporter.write_line(f"  {v:8.4f}  {k}")
