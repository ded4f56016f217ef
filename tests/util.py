"""Helpers shared by the parity tests."""
from __future__ import annotations

import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# Tolerances on the normalised error max|out - ref| / max|ref| (the bar set for this path:
# 1e-5 for float32 state and outputs, 2e-2 for bfloat16 activations).
TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2}


def load_golden(name: str) -> dict:
  with np.load(os.path.join(GOLDEN_DIR, name + ".npz")) as z:
    return {k: z[k] for k in z.files}


def as_f32(t) -> torch.Tensor:
  if isinstance(t, np.ndarray):
    return torch.from_numpy(t).float()
  return t.detach().to("cpu", torch.float32)


def norm_err(out, ref) -> float:
  """max|out - ref| / max(|ref|, tiny); NaN anywhere counts as infinite error."""
  o, r = as_f32(out), as_f32(ref)
  assert o.shape == r.shape, (o.shape, r.shape)
  if o.numel() == 0:
    return 0.0
  d = (o - r).abs()
  if torch.isnan(d).any():
    return float("inf")
  return float(d.max() / r.abs().max().clamp_min(1e-30))


def assert_close(out, ref, tol: float, what: str = ""):
  e = norm_err(out, ref)
  assert e <= tol, f"{what}: normalised max error {e:.3e} > {tol:.1e}"
  return e
