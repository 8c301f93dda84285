import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
TESTS = os.path.dirname(os.path.abspath(__file__))
if TESTS not in sys.path:
    sys.path.insert(0, TESTS)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
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


@pytest.fixture(autouse=True)
def seeded(request):
    """Every test draws its random inputs from a seed of its own name, whatever ran before it."""
    import zlib
    import torch
    torch.manual_seed(zlib.crc32(request.node.nodeid.encode()))
    yield


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Tiny model folders (config.json + model.safetensors), made once per session in a temp folder."""
    import configs
    from gesso_b200.weights import write_random_model
    out = {}
    for name, (cfg, seed, style) in configs.TINY.items():
        d = str(tmp_path_factory.mktemp(f"model_{name}"))
        write_random_model(d, cfg, seed, dtype="bfloat16", style=style)
        out[name] = d
    return out


@pytest.fixture(scope="session")
def plain_models(model_dirs):
    from plain_lfm2 import PlainModel
    return {name: PlainModel(d) for name, d in model_dirs.items()}
