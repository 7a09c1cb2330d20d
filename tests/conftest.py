import os
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if REPO not in sys.path:
    sys.path.insert(0, REPO)
if os.path.dirname(os.path.abspath(__file__)) not in sys.path:
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 GPU (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import flat_oracle
    flat_oracle.build()
    return flat_oracle


@pytest.fixture(scope="session")
def fm():
    import faiss_metal_b200
    return faiss_metal_b200


@pytest.fixture(scope="session")
def res(fm):
    r = fm.StandardB200Resources(0)
    yield r
    r.close()


SELECT_MODES = {
    # which optimistic selection stages of the tensor path are allowed (b200f_set_selection_mode)
    "filter": 1,            # threshold filter wherever the shard allows a pilot sample
    "no_filter": 2,
    "matrix_or_fused": 3,
}


@pytest.fixture(params=list(SELECT_MODES))
def select_mode(request, fm):
    L = fm.lib()
    old = L.b200f_get_selection_mode()
    assert L.b200f_set_selection_mode(SELECT_MODES[request.param]) == 0
    yield request.param
    assert L.b200f_set_selection_mode(old) == 0
