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


def load_golden(name):
    """read a fixture written by tests/golden/make_golden.py back into torch tensors"""
    out = {}
    with np.load(os.path.join(GOLDEN, name + ".npz")) as z:
        for k in z.files:
            a = torch.from_numpy(z[k])
            if k.endswith("__bf16"):
                out[k[:-6]] = a.view(torch.bfloat16)
            elif k.endswith("__e4m3"):
                out[k[:-6]] = a.view(torch.float8_e4m3fn)
            else:
                out[k] = a
    return out


@pytest.fixture(scope="session")
def golden():
    return load_golden


def rel_rms_err(got, ref):
    """max abs error relative to the RMS of the reference output: the tolerance measure of the hot path
    (bf16 outputs: <= 2e-2)"""
    got, ref = got.float(), ref.float()
    rms = ref.square().mean().sqrt().clamp_min(1e-30)
    return ((got - ref).abs().max() / rms).item()


def assert_parity(got, ref, tol=2e-2):
    """hot-path tolerance for bf16 outputs: |got - ref| <= tol * RMS(ref), where an element may also differ by one
    bf16 rounding step of its own magnitude (2^-7 |ref|): both sides round fp32 sums that differ in their last bits,
    and on a heavy-tailed output a single rounding flip of an outlier is larger than tol * RMS."""
    got, ref = got.float(), ref.float()
    rms = ref.square().mean().sqrt().clamp_min(1e-30)
    allowed = torch.maximum(tol * rms, ref.abs() * 2.0 ** -7)
    bad = (got - ref).abs() > allowed
    assert not bad.any(), (f"{int(bad.sum())} of {bad.numel()} elements outside tolerance; worst "
                           f"{((got - ref).abs() / rms).max().item():.3e} of RMS")
