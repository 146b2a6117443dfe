import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


# property-based tests: the same examples on every run (a failure found once stays found; no surprise on another box),
# no wall-clock limits (the boxes that run the suite differ a lot in speed)
try:
    from hypothesis import HealthCheck, settings as _hyp_settings
    _hyp_settings.register_profile("repo", derandomize=True, deadline=None,
                                   suppress_health_check=[HealthCheck.too_slow, HealthCheck.data_too_large])
    _hyp_settings.load_profile("repo")
except ImportError:          # the property-based tests then fail at import, which names the missing package
    pass


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
