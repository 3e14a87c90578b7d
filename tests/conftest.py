import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    """Golden vectors written by tests/golden/make_golden.py (outputs of the unmodified
    reference under Triton's interpreter).  bf16 tensors are stored as raw int16 bits."""
    data = dict(np.load(os.path.join(GOLDEN_DIR, name + ".npz")))
    bf16 = "bf16" in name
    out = {}
    for k, v in data.items():
        if v.dtype.kind in "US":
            out[k] = v
            continue
        t = torch.from_numpy(v)
        if bf16 and t.dtype == torch.int16:
            t = t.view(torch.bfloat16)
        out[k] = t
    return out


def golden_names(prefix):
    return sorted(f[:-4] for f in os.listdir(GOLDEN_DIR) if f.startswith(prefix) and f.endswith(".npz"))


def ulp_tolerance(ref, dtype, n_ulp=1.0, floor=0.0):
    """Elementwise tolerance of n_ulp units in the last place of `dtype` at |ref|."""
    mant = {torch.float16: 10, torch.bfloat16: 7, torch.float32: 23}[dtype]
    mag = ref.float().abs().clamp_min(2.0**-14)
    ulp = torch.exp2(torch.floor(torch.log2(mag)) - mant)
    return (n_ulp * ulp).clamp_min(floor)


TINY = dict(vocab_size=1024, block_size=128, n_layer=2, n_head=4, n_embd=128, dropout=0.1)
