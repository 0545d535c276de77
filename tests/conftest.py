import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for entry in (str(ROOT), str(ROOT / "tests")):
    if entry not in sys.path:
        sys.path.insert(0, entry)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """Model folders (config.json + model.safetensors, float32) of the tiny configurations."""
    from tiny_configs import SEEDS, TINY_CONFIGS
    from tinyvllm_b200.weights.random_init import write_model_folder

    folders = {}
    for name, config in TINY_CONFIGS.items():
        folders[name] = write_model_folder(tmp_path_factory.mktemp(f"tiny_{name}"), config, SEEDS[name])
    return folders
