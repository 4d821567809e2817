import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    # tests/test_zz_* files go last whatever the collection order was
    items.sort(key=lambda item: (os.path.basename(str(item.fspath)).startswith("test_zz"),))


@pytest.fixture(scope="session")
def tiny_folders(tmp_path_factory):
    """Model folders (config.json + model.safetensors, bfloat16 values) of the tiny configurations,
    made with the random-weights mode in a temporary folder."""
    import torch
    from tiny_configs import TINY
    from llmserver_b200.config import Qwen3Config
    from llmserver_b200.weights import write_model_folder
    import llmserver_b200.models  # noqa: F401  registers the architecture

    root = tmp_path_factory.mktemp("models")
    folders = {}
    for name, (raw, seed) in TINY.items():
        folders[name] = write_model_folder(Qwen3Config.from_dict(raw), str(root / name), seed, torch.bfloat16)
    return folders
