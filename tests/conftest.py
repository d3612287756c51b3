import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def pkg():
    import __graft_entry__ as g
    return g


@pytest.fixture(scope="session")
def oracle_mod():
    import oracle
    oracle.lib()
    return oracle


def pytest_terminal_summary(terminalreporter):
    """Prints the largest floor-relative error |a-b| / max(|b|, 1e-3 max|b|) the parity cases of this run
    recorded, per math mode (the bars are 1e-4 for 3xTF32 and 5e-3 for plain TF32)."""
    try:
        import helpers
    except ImportError:
        return
    worst = helpers.worst_floor_rel()
    if worst:
        terminalreporter.write_line("parity: max floor-relative error (tau = 1e-3) over %d recorded cases: %s" % (
            len(helpers._REPORT), ", ".join("%s %.3e" % kv for kv in sorted(worst.items()))))
