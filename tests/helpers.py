"""Shared helpers for the parity tests."""
from __future__ import annotations

import os

import numpy as np
import torch

import cases

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_golden(name: str) -> dict:
    with np.load(os.path.join(GOLDEN_DIR, name + ".npz")) as f:
        return {k: torch.from_numpy(f[k]) for k in f.files}


def rms(t: torch.Tensor) -> float:
    return float(t.double().pow(2).mean().sqrt())


def err_stats(got: torch.Tensor, ref: torch.Tensor) -> tuple[float, float]:
    """(max-abs error / RMS(ref), RMS error / RMS(ref))."""
    got, ref = got.double().cpu(), ref.double().cpu()
    r = rms(ref) + 1e-30
    d = got - ref
    return float(d.abs().max()) / r, float(d.pow(2).mean().sqrt()) / r


def compare_pair_output(got: torch.Tensor, gold: dict, key: str = "out"):
    """Compare a (B,N,N,C) result with a golden entry stored whole or thinned."""
    if key in gold:
        return err_stats(got, gold[key])
    s = cases.SUB_STRIDE
    return err_stats(got[:, ::s, ::s], gold[key + "_sub"])
