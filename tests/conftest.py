import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


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
def tiny_a_dir(tmp_path_factory):
    from tests.helpers import TINY_A, make_model_dir

    return make_model_dir(tmp_path_factory.mktemp("tiny_a"), TINY_A)


@pytest.fixture(scope="session")
def tiny_b_dir(tmp_path_factory):
    from tests.helpers import TINY_B, make_model_dir

    return make_model_dir(tmp_path_factory.mktemp("tiny_b"), TINY_B)


@pytest.fixture(scope="session")
def tiny_c_dir(tmp_path_factory):
    from tests.helpers import TINY_C, make_model_dir

    return make_model_dir(tmp_path_factory.mktemp("tiny_c"), TINY_C)
