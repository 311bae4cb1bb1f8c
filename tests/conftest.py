import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle_lib():
    from oracle import graph
    graph.build()
    return graph.lib()


@pytest.fixture(scope="session")
def models_dir(tmp_path_factory):
    """Directory of freshly written model packs (what $LLIS_MODELS_DIR points at)."""
    from paella_b200 import packer
    d = tmp_path_factory.mktemp("models")
    packer.write_all(str(d))
    return str(d)
