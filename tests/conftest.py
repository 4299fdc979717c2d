import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    """GPU tests are skipped where there is no GPU, so a plain `pytest tests` stays green on
    a CPU box; `-m gpu` on a GPU box runs them."""
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter):
    """The largest error of each dtype and configuration against the oracle, relative to the
    oracle's largest logit: what the tolerances in helpers.py were set from."""
    try:
        from helpers import OBSERVED
    except Exception:
        return
    if OBSERVED:
        terminalreporter.write_line("largest observed error / largest reference magnitude:")
        for (dtype, what), v in sorted(OBSERVED.items()):
            terminalreporter.write_line(f"  {dtype:9s} {what:24s} {v:.3e}")


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """Factory: folder of a tiny random model (written once per configuration and seed)."""
    from helpers import write_folder
    made = {}

    def get(name: str, seed: int = 0, std: float = 0.02, **overrides) -> str:
        key = (name, seed, std, tuple(sorted(overrides.items())))
        if key not in made:
            folder = str(tmp_path_factory.mktemp(f"{name}-s{seed}"))
            write_folder(folder, name, seed, std=std, **overrides)
            made[key] = folder
        return made[key]

    return get
