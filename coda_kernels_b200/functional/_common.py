"""Pieces shared by the fused-linear autograd wrappers."""

from __future__ import annotations

from ..ops import linear_backward  # noqa: F401  (re-exported: the shared backward of ``pre = x @ weight^T``)
