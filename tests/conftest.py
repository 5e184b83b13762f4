import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "transformers5-qwen3.5-recipe_b200"
for p in (str(ROOT), str(PKG)):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def lib():
    """The C-ABI library; built on demand when the tree has no libb2g.so yet."""
    from b2g import _lib

    if not _lib.LIB_PATH.exists():
        sys.path.insert(0, str(PKG / "csrc"))
        import build as _build

        _build.build()
    return _lib.load()


@pytest.fixture(scope="session")
def cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    from b2g import ops

    yield torch.device("cuda", 0)
    torch.cuda.synchronize()
    ops.check_status()
