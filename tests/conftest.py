import json
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    """What the reference's own example programs wrote back (tests/golden/make_golden.py)."""
    return json.loads((ROOT / "tests" / "golden" / "reference_outputs.json").read_text())["programs"]


@pytest.fixture(scope="session")
def ctx():
    """One aiehlc context on cuda:0 for the whole session (GPU tests only)."""
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device; aiehlc_b200 has no CPU path"
    from aiehlc_b200.ops import Context
    c = Context(0)
    yield c
    assert c.sync() == 0
    c.close()
