import os
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (ROOT, HERE):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    """Tests marked gpu are skipped where there is no CUDA device."""
    try:
        import torch
        have = torch.cuda.is_available()
    except Exception:
        have = False
    if have:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """Model folders of the tiny configurations, written once per session with the random-weights mode."""
    from tiny_configs import SEED_A, SEED_B, SEED_C, SEED_D, TINY_A, TINY_B, TINY_C, TINY_D, WEIGHTS
    from tinyserve_llm_b200.weights import write_random_model

    out = {}
    for name, raw, seed in (("a", TINY_A, SEED_A), ("b", TINY_B, SEED_B), ("c", TINY_C, SEED_C),
                            ("d", TINY_D, SEED_D)):
        folder = tmp_path_factory.mktemp(f"tiny_{name}")
        write_random_model(str(folder), raw, seed, **WEIGHTS)
        out[name] = str(folder)
    return out
