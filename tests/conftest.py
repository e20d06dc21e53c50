import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# under pytest-xdist every worker gets its own slice of the GPUs (before anything initialises CUDA)
from arctic_platform_b200.testing_utils import partition_gpus_for_xdist  # noqa: E402

partition_gpus_for_xdist()


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_addoption(parser):
    from arctic_platform_b200.testing_utils import pytest_addoption_shared
    pytest_addoption_shared(parser)


def pytest_terminal_summary(terminalreporter):
    make_reports = terminalreporter.config.getoption("--make-reports", default=False)
    if make_reports:
        from arctic_platform_b200.testing_utils import pytest_terminal_summary_main
        pytest_terminal_summary_main(terminalreporter, id=make_reports, root=str(ROOT / "reports"))
