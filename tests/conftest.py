import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders of the two tiny configurations, made once per run in a temporary folder."""
    from tests.helpers import make_model_dir

    root = tmp_path_factory.mktemp("models")
    return {
        "tiny_a": make_model_dir(root / "tiny_a", "tiny_a", seed=0, norm_noise=0.1),
        "tiny_b": make_model_dir(root / "tiny_b", "tiny_b", seed=1, norm_noise=0.0),
        "tiny_c": make_model_dir(root / "tiny_c", "tiny_c", seed=2, norm_noise=0.05),
    }
