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
    # which optimistic selection stages of the tensor path are allowed (environment switches of
    # the library, read at every call)
    "filter": {"B200F_FILTER": "1"},   # threshold filter wherever the shard allows a pilot sample
    "no_filter": {"B200F_NO_FILTER": "1"},
    "matrix_or_fused": {"B200F_NO_FILTER": "1", "B200F_NO_LISTS": "1"},
}


@pytest.fixture(params=list(SELECT_MODES))
def select_mode(request):
    import os
    env = SELECT_MODES[request.param]
    old = {k: os.environ.get(k) for k in ("B200F_FILTER", "B200F_NO_FILTER", "B200F_NO_LISTS")}
    for k in old:
        os.environ.pop(k, None)
    os.environ.update(env)
    yield request.param
    for k, v in old.items():
        os.environ.pop(k, None)
        if v is not None:
            os.environ[k] = v
