import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# The unmodified reference package the provider is tested through: installed (copied) from the
# checkout into baseline/_ref where a checkout exists, and found there on machines without one.
from intent_b200 import build as _build

_installed = _build.install_reference()
REFERENCE_PYTHON = _installed if _installed is not None else ROOT / "baseline" / "_ref"
HAS_REFERENCE = (REFERENCE_PYTHON / "intent" / "__init__.py").is_file()


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu on the GPU box")
    config.addinivalue_line("markers", "reference: needs the reference checkout to be importable")


def pytest_collection_modifyitems(config, items):
    has_gpu = torch.cuda.is_available()
    for item in items:
        if "gpu" in item.keywords and not has_gpu:
            item.add_marker(pytest.mark.skip(reason="no CUDA device in this environment"))


@pytest.fixture(scope="session", autouse=True)
def built():
    """Native pieces are built in-tree before any test uses them (no-op when fresh)."""
    from intent_b200 import build
    import oracle
    build.build_all()
    oracle.build()


def relative_error(actual: torch.Tensor, expected: torch.Tensor) -> float:
    """max |a - e| / (|e| + rms(e)).  `relative_error(a, e) <= tol` is the usual mixed
    test |a - e| <= tol * |e| + atol with atol = tol * rms(e): entries near zero are
    measured against the scale of the data instead of dividing by (almost) nothing."""
    a = actual.detach().double().cpu()
    e = expected.detach().double().cpu()
    if e.numel() == 0:
        return 0.0
    floor = e.pow(2).mean().sqrt().clamp_min(1e-30)
    return ((a - e).abs() / (e.abs() + floor)).max().item()


@pytest.fixture
def rel():
    return relative_error
