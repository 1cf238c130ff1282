"""Kernel-vs-reference comparison (crates/orion-cuda/src/lib.rs:188-317)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import numpy as np

from .errors import InternalError


@dataclass(frozen=True)
class Tolerance:
    """lib.rs:188-224: a value matches when abs OR rel holds; non-finite only bit-for-bit."""
    abs: float
    rel: float

    def matches(self, expected: float, actual: float) -> bool:
        e, a = np.float32(expected), np.float32(actual)
        if not math.isfinite(e) or not math.isfinite(a):
            return e.view(np.uint32) == a.view(np.uint32)
        diff = abs(float(e) - float(a))
        return diff <= self.abs or diff <= self.rel * abs(float(e))


Tolerance.F32 = Tolerance(1e-5, 1e-5)
Tolerance.F16 = Tolerance(1e-2, 1e-2)


@dataclass
class ValidationReport:
    kernel: str
    elements: int
    mismatches: int
    max_abs_error: float
    max_rel_error: float
    worst_index: Optional[int]

    def passed(self) -> bool:
        return self.mismatches == 0

    def render(self) -> str:
        if self.passed():
            return (f"{self.kernel}: PASS ({self.elements} elements, max abs {self.max_abs_error:.3e}, "
                    f"max rel {self.max_rel_error:.3e})")
        return (f"{self.kernel}: FAIL — {self.mismatches}/{self.elements} elements differ (max abs "
                f"{self.max_abs_error:.3e}, max rel {self.max_rel_error:.3e}, worst at {self.worst_index})")


def validate(kernel: str, expected, actual, tol: Tolerance) -> ValidationReport:
    """lib.rs:269-317, vectorised."""
    e = np.asarray(expected, dtype=np.float32).ravel()
    a = np.asarray(actual, dtype=np.float32).ravel()
    if e.size != a.size:
        raise InternalError(f"validation shape mismatch for {kernel}: reference has {e.size} elements, "
                            f"kernel produced {a.size}")
    finite = np.isfinite(e) & np.isfinite(a)
    diff = np.abs(e.astype(np.float64) - a.astype(np.float64))
    ok_finite = (diff <= tol.abs) | (diff <= tol.rel * np.abs(e.astype(np.float64)))
    ok_other = e.view(np.uint32) == a.view(np.uint32)
    ok = np.where(finite, ok_finite, ok_other)
    d = np.where(finite, diff, 0.0)
    eps = float(np.finfo(np.float32).eps)
    with np.errstate(divide="ignore", invalid="ignore"):
        rel = np.where(finite & (np.abs(e) > eps), d / np.abs(e.astype(np.float64)), 0.0)
    worst = int(np.argmax(d)) if d.size and float(d.max()) > 0 else None
    return ValidationReport(kernel, int(e.size), int((~ok).sum()), float(d.max()) if d.size else 0.0,
                            float(rel.max()) if rel.size else 0.0, worst)
