import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def reference_root():
    """Directory that holds the reference's ``xlstm`` package, or None.  Looked up at run time: the environment
    variable XLSTM_REFERENCE first, then an installed copy under ``baseline/_ref`` of this checkout (made with
    ``pip install --no-deps --target baseline/_ref <reference checkout>``; it is not part of the history)."""
    for cand in (os.environ.get("XLSTM_REFERENCE"), os.path.join(ROOT, "baseline", "_ref")):
        if cand and os.path.isdir(os.path.join(cand, "xlstm")):
            return cand
    return None


def import_reference():
    """Put the reference on sys.path (after installing this package's mLSTM backend module, which the reference's
    xlstm_large/model.py imports) and return its root; skips the calling test when no copy is present."""
    root = reference_root()
    if root is None:
        pytest.skip("reference package not found (set XLSTM_REFERENCE or install it under baseline/_ref)")
    from xlstm_b200.integration import install_mlstm_backend
    assert install_mlstm_backend() in ("shim", "registered")
    if root not in sys.path:
        sys.path.insert(0, root)
    return root


def load_golden(name):
    d = np.load(os.path.join(GOLDEN, name + ".npz"))
    return {k: torch.from_numpy(d[k]) for k in d.files}


def rel_l2(a, b):
    a = a.double().flatten()
    b = b.double().flatten()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))
