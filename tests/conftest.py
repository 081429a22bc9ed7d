import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (B200)")
    config.addinivalue_line("markers", "multigpu: needs at least two CUDA GPUs")
    config.addinivalue_line("markers", "slow: long-running CPU test")


def _gpu_count():
    try:
        import torch

        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        return 0


def pytest_collection_modifyitems(config, items):
    n = _gpu_count()
    for item in items:
        if "gpu" in item.keywords and n == 0:
            item.add_marker(pytest.mark.skip(reason="no CUDA device"))
        if "multigpu" in item.keywords and n < 2:
            item.add_marker(pytest.mark.skip(reason="needs two CUDA devices"))


@pytest.fixture(scope="session")
def native_lib():
    from glm_tpu_b200.csrc.build import build

    build()
    from glm_tpu_b200.ops import native

    return native


def scaled(seconds: float) -> float:
    """A subprocess timeout of a test, stretched by ``GLM_B200_TEST_TIMEOUT_SCALE`` (a slow or shared machine sets it above 1)."""
    from glm_tpu_b200 import envs

    return seconds * envs.GLM_B200_TEST_TIMEOUT_SCALE
