import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders of the tiny configurations, written once a session into a temporary folder."""
    from tiny_configs import CONFIGS, make_model_dir

    root = tmp_path_factory.mktemp("models")
    return {name: make_model_dir(name, str(root)) for name in CONFIGS}


@pytest.fixture(scope="session")
def plain_models(model_dirs):
    from plain_lfm2 import PlainLfm2

    return {name: PlainLfm2(d) for name, d in model_dirs.items()}
