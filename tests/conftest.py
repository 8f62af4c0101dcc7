import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "kv_retention: a GPU test that wants the KV pool to retain published pages (off for the others)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has = torch.cuda.is_available()
    except Exception:
        has = False
    if has:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


@pytest.fixture(autouse=True)
def _bit_exact_repeats_on_the_gpu(request, monkeypatch):
    """GPU tests compare a repeated prompt token for token with its first run.  That needs the same compute path both times, so
    the KV pool's retention of published pages is off for them (servers they launch inherit the variable); a test that is about
    retention asks for it with ``@pytest.mark.kv_retention``."""
    if "gpu" in request.keywords and "kv_retention" not in request.keywords:
        monkeypatch.setenv("B200_KV_RETAIN", "0")
