import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def _load_npz(name):
    import numpy as np
    flat = np.load(os.path.join(GOLDEN, name))
    cases = {}
    for key in flat.files:
        case, field = key.split("/", 1)
        cases.setdefault(case, {})[field] = flat[key]
    return cases


@pytest.fixture(scope="session")
def metadata_golden():
    return _load_npz("metadata_golden.npz")


@pytest.fixture(scope="session")
def attention_golden():
    return _load_npz("attention_golden.npz")


def unpack_golden_metadata(case):
    """Golden metadata back in the reference's dtypes/shapes (int64, bool, int64)."""
    import numpy as np
    import torch
    bm, ma = int(case["block_m"]), int(case["max_ancestors"])
    ai = torch.from_numpy(case["ancestor_idx"].astype(np.int64))
    li = torch.from_numpy(case["leaf_idx"].astype(np.int64))
    am = np.unpackbits(case["ancestor_mask_bits"], axis=2)[:, :, :ma].astype(bool)
    return ai, torch.from_numpy(am), li, bm, ma


@pytest.fixture(scope="session")
def built_lib():
    """Path of the C-ABI library, built first when it is missing or stale and nvcc is here."""
    from fstattention_b200 import build as fst_build
    if not fst_build.up_to_date():
        try:
            fst_build.build()
        except RuntimeError:
            if not os.path.exists(fst_build.LIB):
                raise
    return fst_build.LIB
