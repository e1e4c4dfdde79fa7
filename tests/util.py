"""Helpers shared by the tests: package loader and torch<->numpy conversions."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402

# Parity tolerance for attention outputs computed in bf16 / fp16 against the fp32 oracle on the
# same (already rounded) inputs: max-abs <= 2e-2 and mean-abs <= 2e-3.
MAX_ABS_TOL = 2e-2
MEAN_ABS_TOL = 2e-3
# fp32 CUDA path against the fp32 oracle (the reference's own tests use 1e-5 on tiny cases).
F32_TOL = 2e-5


def nvk():
    return entry.load_package()


def workloads():
    import importlib
    entry.load_package()
    return importlib.import_module("benchmarks.workloads")


def to_dev(a, dtype=None, device="cuda"):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(a)).to(device)
    return t.to(dtype) if dtype is not None else t


def to_np(t):
    return t.detach().float().cpu().numpy()


def assert_attention_close(actual, expected, half=True):
    err = np.abs(np.asarray(actual, dtype=np.float64) - np.asarray(expected, dtype=np.float64))
    if half:
        assert err.max() <= MAX_ABS_TOL, f"max-abs {err.max():.4e} > {MAX_ABS_TOL}"
        assert err.mean() <= MEAN_ABS_TOL, f"mean-abs {err.mean():.4e} > {MEAN_ABS_TOL}"
    else:
        assert err.max() <= F32_TOL, f"max-abs {err.max():.4e} > {F32_TOL}"
