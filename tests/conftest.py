"""pytest configuration: the `gpu` marker, import of the hyphen-named package, golden-fixture loading."""

from __future__ import annotations

import importlib
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

REPO = Path(__file__).resolve().parent.parent
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))

GOLDEN = Path(__file__).resolve().parent / "golden"
PACKAGE = "int8-kvcache_b200"

# payload dtypes of the uint16-encoded arrays in the golden files
_BF16_KEYS = {"query", "key", "value", "out_loop_bf16", "out_loop_quantize_q_bf16", "out_unquantised_bf16"}
_FP16_KEYS = {"k", "v"}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def package(sub: str = ""):
    return importlib.import_module(PACKAGE + (("." + sub) if sub else ""))


def load_golden(name: str) -> dict:
    """Golden .npz -> dict of CPU tensors (uint16 payloads reinterpreted as bf16/fp16)."""
    raw = np.load(GOLDEN / f"{name}.npz")
    out = {}
    for k in raw.files:
        a = raw[k]
        if a.dtype == np.uint16:
            t = torch.from_numpy(a.view(np.int16).copy())
            out[k] = t.view(torch.float16 if (k in _FP16_KEYS and name == "real_layer27") else torch.bfloat16)
        else:
            out[k] = torch.from_numpy(a.copy())
    return out


@pytest.fixture(scope="session")
def kv():
    return package()


@pytest.fixture(scope="session")
def workloads():
    return package("workloads")


def cosine(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.double().reshape(-1)
    b = b.double().reshape(-1)
    return float((a @ b) / (a.norm() * b.norm()).clamp_min(1e-300))


def max_abs(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.double() - b.double()).abs().max())
