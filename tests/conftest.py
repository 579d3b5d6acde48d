import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
if str(ROOT / "tests") not in sys.path:
    sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


GOLDEN_FIXTURE = ROOT / "tests" / "golden" / "qwen-tiny"


def reference_checkout_fixture_dir():
    """Folder of the qwen-tiny fixture inside a checkout of the reference project, or None.

    Looked up through SPROUT_REFERENCE_DIR, else as a ``reference`` checkout beside this
    repository.
    """
    base = os.environ.get("SPROUT_REFERENCE_DIR")
    base = Path(base) if base else ROOT.parent / "reference"
    path = base / "test" / "fixtures" / "qwen-tiny"
    return path if (path / "reference.json").exists() else None


def reference_fixture_dir():
    """The reference project's qwen-tiny fixture: from a checkout of the reference when one is
    at hand, else the byte-identical copy of its data files under tests/golden/qwen-tiny."""
    return reference_checkout_fixture_dir() or (GOLDEN_FIXTURE if (GOLDEN_FIXTURE / "reference.json").exists() else None)


@pytest.fixture(scope="session")
def fixture_dir():
    path = reference_fixture_dir()
    if path is None:
        pytest.skip("reference fixture folder not found")
    return path
