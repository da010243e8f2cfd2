import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def backend():
    """One library context on cuda:0 with the arena reserved."""
    import torch
    from cleffa_b200 import OmniBackend

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    torch.cuda.init()
    b = OmniBackend(0)
    b.reserve(1, n_layer=4)
    yield b
    b.close()


@pytest.fixture(scope="session")
def weights0():
    """Seed-0 random-init weights on the host (configuration 1)."""
    from oracle import omni_oracle as orc

    return orc.make_weights(0)


@pytest.fixture(scope="session")
def bound0(backend, weights0):
    """Seed-0 weights uploaded as layer 0."""
    backend.bind_layer(0, *weights0)
    return backend
