import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    # the file whose name sorts last must also run last, whatever order the files were given in
    items.sort(key=lambda it: (os.path.basename(str(it.fspath)).startswith("test_zz"),))


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders of the tiny configurations, written once per session into a temporary folder."""
    import tiny_models
    base = tmp_path_factory.mktemp("models")
    return tiny_models.write_all(str(base))
