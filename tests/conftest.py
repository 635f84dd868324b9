import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle binding (builds oracle/liboracle.so on first use)."""
    from oracle import binding
    binding.lib()
    return binding


@pytest.fixture(scope="session")
def tcab_lib():
    """libtcab.so through ctypes; built in-tree if missing (never substituted)."""
    from tcacomp_b200 import _lib, build
    if not os.path.exists(_lib.LIB_PATH):
        build.build()
    return _lib.load()


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    return torch.device("cuda:0")


# Parity counts of the full-size configuration checks: how many elements were compared with the oracle and how
# many of them were accepted only through the oracle's own distance to the fp64 value (oracle/checks.py).
# Printed after the run so that the effect of the two-sided criterion is visible in every log.
PARITY_COUNTS = {}


@pytest.fixture(scope="session")
def parity_counts():
    return PARITY_COUNTS


def pytest_terminal_summary(terminalreporter):
    if PARITY_COUNTS:
        terminalreporter.write_line("parity counts (elements compared with the oracle / accepted only through the "
                                    "oracle-to-fp64 term):")
        for name, rep in PARITY_COUNTS.items():
            terminalreporter.write_line(f"  {name}: {rep}")
