import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, 'tests', 'golden')):
    if p not in sys.path:
        sys.path.insert(0, p)


os.environ.setdefault('SBL_REFERENCE_ROOT', os.path.join(os.path.dirname(ROOT), 'reference'))


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (run with -m gpu on a B200)')


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason='no CUDA device')
    for item in items:
        if 'gpu' in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope='session')
def sbl_lib():
    """Builds (if stale) and loads the C-ABI library."""
    import os
    from fly_b200 import build, _cabi
    try:
        build.build()
    except RuntimeError as exc:
        if 'nvcc not found' in str(exc) and not os.path.exists(build.LIB_PATH):
            pytest.skip('no nvcc and no prebuilt library on this machine')
        if not os.path.exists(build.LIB_PATH):
            raise
    return _cabi.load()
