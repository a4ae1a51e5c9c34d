import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs at least one CUDA GPU (run on the B200 box)")
    config.addinivalue_line("markers", "multigpu(n): needs at least n CUDA GPUs")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        gpus = torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        gpus = 0
    for item in items:
        marker = item.get_closest_marker("multigpu")
        if marker is not None:
            item.add_marker(pytest.mark.gpu)
            need = marker.args[0] if marker.args else 2
            if gpus < need:
                item.add_marker(pytest.mark.skip(reason=f"needs {need} GPUs, found {gpus}"))
        elif item.get_closest_marker("gpu") is not None and gpus < 1:
            item.add_marker(pytest.mark.skip(reason="needs a CUDA GPU"))
