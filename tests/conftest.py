import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")
    # Property tests draw the same examples on every run (a gate must not depend on the day's seed) and keep no example
    # database in the tree; HYPOTHESIS_SEED=random explores new ones by hand.
    try:
        from hypothesis import settings
        explore = os.environ.get("HYPOTHESIS_SEED", "") == "random"
        settings.register_profile("repo", derandomize=not explore, deadline=None, database=None, print_blob=True)
        settings.load_profile("repo")
    except ImportError:
        pass


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
