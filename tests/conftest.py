import json
import os
import sys

import pytest
import torch

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


from tests.helpers import TINY, make_model_folder  # noqa: E402


@pytest.fixture(scope="session")
def tiny_folders(tmp_path_factory):
    out = {}
    for name, (cfg, seed, page, sharpen) in TINY.items():
        d = tmp_path_factory.mktemp(f"tiny_{name}")
        out[name] = make_model_folder(d, cfg, seed, sharpen)
    return out


@pytest.fixture(autouse=True)
def no_wait_ran_out(request):
    """After every GPU test: no kernel of the package reported a bounded wait that ran out
    (a result made by such a launch is not valid, whatever the tolerances said)."""
    yield
    if "gpu" in request.keywords and torch.cuda.is_available():
        from paged_batch_engine_b200.csrc import ops
        ops.raise_on_kernel_status(torch.device("cuda:0"))
