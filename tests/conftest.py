import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


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
def tiny_qwen3_path(tmp_path_factory):
    from tensorsharp_b200.models import synth
    p = str(tmp_path_factory.mktemp("models") / "tiny_qwen3_q8.gguf")
    synth.write_qwen3(p, **synth.QWEN3_TINY, device="cpu")
    return p
