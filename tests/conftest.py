import os
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (ROOT, HERE):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """Writes tiny random model folders on demand: get(config, seed=1, dtype="bfloat16") -> path."""
    import torch
    from gemmars_b200.weights import write_random_model
    made = {}

    def get(cfg, seed=1, dtype="bfloat16"):
        key = (id(cfg), seed, dtype)
        if key not in made:
            d = tmp_path_factory.mktemp("model")
            write_random_model(str(d), cfg, seed, torch.bfloat16 if dtype == "bfloat16" else torch.float32)
            made[key] = str(d)
        return made[key]

    return get
