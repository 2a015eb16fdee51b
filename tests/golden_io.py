"""Loaders for the committed golden vectors (tests/golden/*.npz)."""

import json
from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"


def _json(arr):
    return json.loads(bytes(arr.tolist()).decode())


def load_gradient_parity():
    """Returns (config dict, weights {name: f32 [out,in]}, adapters, cases dict, expected)."""
    z = np.load(GOLDEN / "gradient_parity.npz")
    cfg = _json(z["config_json"])
    cases = _json(z["cases_json"])
    weights = {k[len("model/"):]: z[k] for k in z.files if k.startswith("model/")}
    adapters = {k[len("adapter/"):]: z[k] for k in z.files if k.startswith("adapter/")}
    expected = {k[len("expected/"):]: z[k] for k in z.files if k.startswith("expected/")}
    return cfg, weights, adapters, cases, expected


def load_qwen2_family():
    z = np.load(GOLDEN / "qwen2_family.npz")
    cfg = _json(z["config_json"])
    cases = _json(z["cases_json"])
    weights = {k[len("model/"):]: z[k] for k in z.files if k.startswith("model/")}
    expected = {k[len("expected/"):]: z[k] for k in z.files if k.startswith("expected/")}
    return cfg, weights, cases, expected


def within(got, exp, atol=1e-4, rtol=1e-3):
    """The reference's parity rule: |got - exp| <= atol + rtol * |exp| elementwise."""
    got = np.asarray(got, dtype=np.float64)
    exp = np.asarray(exp, dtype=np.float64)
    assert got.shape == exp.shape, (got.shape, exp.shape)
    err = np.abs(got - exp)
    tol = atol + rtol * np.abs(exp)
    bad = err > tol
    return (not bad.any()), float(err.max()) if err.size else 0.0


def to_torch(d):
    return {k: torch.tensor(np.asarray(v)) for k, v in d.items()}
