import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (run on the B200 box)")


@pytest.fixture(scope="session")
def built_library():
    """The in-tree CUDA library, (re)built if its sources are newer."""
    from hydraserve_b200 import build

    return build.build()


def pytest_terminal_summary(terminalreporter):
    """How many rows each parity comparison covered, how many of them were rounding-sensitive
    (allowed to move by the few elements noise can move a cut) and how many had a top-p cut
    inside a group of equal scores.  Also written to $HS_PARITY_REPORT when that is set."""
    from tests import parity

    if not parity.COUNTS:
        return
    lines = ["case | rows | rounding-sensitive | tie-split"]
    lines += [f"{name} | {rows} | {sensitive} | {split}" for name, rows, sensitive, split in parity.COUNTS]
    terminalreporter.write_sep("-", "parity row counts")
    for line in lines:
        terminalreporter.write_line(line)
    path = os.environ.get("HS_PARITY_REPORT")
    if path:
        Path(path).write_text("\n".join(lines) + "\n")
