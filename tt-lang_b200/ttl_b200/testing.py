"""Comparison helpers programs import as `sim.testing` (python/sim/testing.py:11-21)."""

from __future__ import annotations

import torch

from .ttnn import Tensor


def assert_pcc(tensor_a: Tensor, tensor_b: Tensor, rtol: float = 1e-5, atol: float = 1e-8) -> None:
    assert tensor_a.shape == tensor_b.shape, "Tensors must have the same shape"
    assert tensor_a.dtype == tensor_b.dtype, "Tensors must have the same dtype"
    close = torch.isclose(tensor_a._tensor, tensor_b._tensor, rtol=rtol, atol=atol)
    assert bool(close.all().item()), "Tensor values are not close enough"
