import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = ROOT / "tests" / "golden"
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def golden_names(prefix: str):
    return sorted(path.stem[len(prefix):] for path in GOLDEN.glob(f"{prefix}*.npz") if path.stem != "lattice_units")


def load_golden(stem: str) -> dict:
    with np.load(GOLDEN / f"{stem}.npz", allow_pickle=False) as data:
        return {key: data[key] for key in data.files}


def buffers_of(record: dict) -> dict:
    return {key[4:]: value for key, value in record.items() if key.startswith("buf_")}


@pytest.fixture(scope="session")
def oracle_module():
    import oracle

    oracle.build()
    return oracle
