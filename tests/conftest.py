from __future__ import annotations

import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O

    O.build()
    return O


@pytest.fixture(scope="session")
def rb():
    """The package with libretro_b200.so built (compiling needs nvcc, not a GPU)."""
    import retrograd_b200
    from retrograd_b200 import build as B

    if not retrograd_b200.LIB_PATH.exists() or os.environ.get("RB200_REBUILD"):
        B.build()
    retrograd_b200.load_library()
    return retrograd_b200


@pytest.fixture(scope="session")
def models(rb, tmp_path_factory):
    """Seeded synthetic GGUF models, written once per session."""
    root = tmp_path_factory.mktemp("models")
    cache: dict[str, Path] = {}

    def get(name: str, **spec) -> Path:
        if name not in cache:
            path = root / f"{name}.gguf"
            rb.synth_gguf(path, **spec)
            cache[name] = path
        return cache[name]

    return get


# The tiny CPU-runnable model: llama-style decoder, Q8_0 (ffn_down rows of 688 cannot hold whole
# Q8_0 blocks and are stored as F16, which the synthesiser does for any indivisible row).
C1_SPEC = dict(arch="llama", layers=2, d=256, heads=4, kv_heads=4, ff=688, vocab=4096, dtype="q8_0", seed=20261125)


@pytest.fixture(scope="session")
def c1_model(models):
    return models("c1", **C1_SPEC)
