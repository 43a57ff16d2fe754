import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "nsa-test_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "cuda: marker name used by the reference project's own tests")


def pytest_terminal_summary(terminalreporter):
    """Print what the parity comparisons achieved (not only that they passed): block-id agreement counts and the
    largest error of every tensor compared through tests.util.close()."""
    try:
        from tests import util
    except Exception:
        return
    tr = terminalreporter
    if util.INDEX_LOG:
        tr.write_line("block-id agreement with the oracle (rows = B*G*T; rows may differ only inside the ambiguity set):")
        for where, rows, amb, mism, outside in util.INDEX_LOG:
            tr.write_line(f"  {where}: rows {rows}, ambiguous {amb}, differing {mism}, differing outside the ambiguity set {outside}")
    if util.PARITY_LOG:
        tr.write_line("achieved parity errors (max-abs | largest reference magnitude | bound):")
        for where, name, err, ref_max, tol in util.PARITY_LOG:
            tr.write_line(f"  {where}: {name}: {err:.3e} | {ref_max:.3e} | {tol:.3e}")
