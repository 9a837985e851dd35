import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    # GPU tests fail loudly on a box without a device instead of passing silently.
    pass


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders with random weights for the tiny configurations, made once
    per session in a temporary folder."""
    from util import TINY, make_model_dir
    root = tmp_path_factory.mktemp("models")
    out = {}
    for name, spec in TINY.items():
        out[name] = make_model_dir(str(root / name), spec["config"], spec["seed"])
        out[name + "_sharp"] = make_model_dir(str(root / (name + "_sharp")), spec["config"], spec["seed"] + 100,
                                              sharpen=4.0)
    return out
