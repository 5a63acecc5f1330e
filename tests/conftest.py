import json
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name: str):
    """Returns (meta, tensors) of a small golden case: 16-bit inputs restored
    to torch tensors, fp32 reference outputs as torch tensors."""
    z = np.load(GOLDEN / f"{name}.npz")
    meta = json.loads(bytes(z["meta"]).decode())
    dtype = getattr(torch, meta["dtype"])
    out = {}
    for key in z.files:
        if key == "meta":
            continue
        arr = z[key]
        if arr.dtype == np.uint16:
            out[key] = torch.from_numpy(arr.view(np.int16).copy()).view(dtype)
        else:
            out[key] = torch.from_numpy(arr.copy())
    return meta, out


SMALL_GOLDEN = ["rope_s33_d128_bf16", "rope_s129_d256_bf16", "norope_s33_d128_bf16", "rope_s40_d128_fp16"]
