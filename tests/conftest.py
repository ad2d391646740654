"""Shared fixtures.  Tests that need a GPU carry ``@pytest.mark.gpu``; everything else runs on a CPU."""

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(Path(__file__).resolve().parent))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """Tiny random model folders (config.json + model.safetensors), made once per session in a
    temporary folder.  ``model_folders(name, dtype)`` returns the path."""
    import torch

    from tiny_configs import TINY, tiny_config
    from zephyr_b200.weights import write_random_model

    made = {}

    def get(name: str, dtype: str = "bfloat16") -> Path:
        key = (name, dtype)
        if key not in made:
            folder = tmp_path_factory.mktemp(f"{name}_{dtype}")
            write_random_model(tiny_config(name), TINY[name]["seed"], folder,
                               dtype=getattr(torch, dtype))
            made[key] = folder
        return made[key]

    return get


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)
