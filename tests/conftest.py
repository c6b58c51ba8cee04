import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:  # noqa: BLE001
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """Folders of the tiny random models, made on demand: ``get(name, store_dtype)``."""
    from tests.helpers import TINY, make_model_folder

    made = {}

    def get(name: str, store: str = "bfloat16", seed: int = 0) -> str:
        key = (name, store, seed)
        if key not in made:
            folder = tmp_path_factory.mktemp(f"tiny_{name}_{store}_{seed}")
            made[key] = make_model_folder(str(folder), TINY[name], store, seed)
        return made[key]

    return get
