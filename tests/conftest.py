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


def reference_fixture_dir():
    """Folder of the reference project's qwen-tiny fixture, or None.

    Looked up through SPROUT_REFERENCE_DIR, else as a ``reference`` checkout
    beside this repository.
    """
    base = os.environ.get("SPROUT_REFERENCE_DIR")
    base = Path(base) if base else ROOT.parent / "reference"
    path = base / "test" / "fixtures" / "qwen-tiny"
    return path if (path / "reference.json").exists() else None


@pytest.fixture(scope="session")
def fixture_dir():
    path = reference_fixture_dir()
    if path is None:
        pytest.skip("reference fixture folder not found")
    return path
