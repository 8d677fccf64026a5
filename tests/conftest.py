import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device of compute capability 10.x")


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders of the tiny configurations, written once per session into a
    temporary folder: name -> (path, config, page_size)."""
    from tiny_configs import ALL
    from vosti_b200.weights import write_random_model

    out = {}
    for name, (config, seed, page) in ALL.items():
        folder = tmp_path_factory.mktemp(f"tiny_{name}")
        write_random_model(folder, config, seed)
        out[name] = (str(folder), config, page)
    return out


@pytest.fixture(scope="session")
def plain_models(model_dirs):
    """name -> (config, float32 tensors) as the plain implementation reads them."""
    import plain_qwen3 as plain

    return {name: plain.load_model(path) for name, (path, _, _) in model_dirs.items()}
