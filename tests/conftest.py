import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def model_dir(tmp_path_factory):
    """Directory for model files regenerated from their seeds (cached across tests of a session)."""
    d = Path(os.environ.get("SMX_MODEL_CACHE", "")) if os.environ.get("SMX_MODEL_CACHE") else tmp_path_factory.mktemp("models")
    d.mkdir(parents=True, exist_ok=True)
    return d


@pytest.fixture(scope="session")
def model_file(model_dir):
    """``model_file(name, **spec_overrides)`` -> (path to JSON, model dict, spec)."""
    from symmetrix_b200.modelgen.generate import generate_model, named_spec, write_json

    cache = {}

    def get(name, **over):
        key = (name, tuple(sorted(over.items())))
        if key not in cache:
            spec = named_spec(name, **over)
            model = generate_model(spec)
            tag = "_".join(f"{k}{v}" for k, v in sorted(over.items()))
            path = model_dir / f"{name}_{tag}.json"
            write_json(model, path)
            cache[key] = (path, model, spec)
        return cache[key]

    return get
