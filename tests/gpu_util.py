"""Bridges between the numpy world of the oracle and device tensors for the GPU parity tests."""
from __future__ import annotations

import numpy as np
import torch

import oracle
from nml_b200 import ops

TORCH_DTYPE = {oracle.F16: torch.float16, oracle.BF16: torch.bfloat16}


def to_device_bits(bits: np.ndarray, dtype: int) -> torch.Tensor:
    """uint16 bit patterns -> f16/bf16 device tensor."""
    t = torch.from_numpy(np.ascontiguousarray(bits).view(np.int16).copy())
    return t.view(TORCH_DTYPE[dtype]).cuda()


def from_device_bits(tensor: torch.Tensor) -> np.ndarray:
    return tensor.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def device_f32(tensor: torch.Tensor) -> np.ndarray:
    return tensor.detach().float().cpu().numpy()


def parameter(name: str, triple, width: int, dtype: int) -> ops.NvFp4Parameter:
    payload, scales, g = triple
    shape = tuple(payload.shape[:-1]) + (width,)
    return ops.NvFp4Parameter.nvfp4(
        name, shape, TORCH_DTYPE[dtype], torch.from_numpy(np.ascontiguousarray(payload)).cuda(),
        torch.from_numpy(np.ascontiguousarray(scales)).cuda(),
        torch.tensor(float(g), dtype=torch.float32).cuda())


def assert_gemm_close(actual_f32: np.ndarray, expected_f32: np.ndarray, what: str = ""):
    """The GEMM parity bar: max relative error <= 2e-2 and mean relative error <= 2e-3
    against the f32-accumulated oracle output (denominator floored at 1% of its RMS)."""
    m = oracle.error_metrics(actual_f32, expected_f32)
    assert m["max_rel"] <= 2e-2 and m["mean_rel"] <= 2e-3, (what, m)
    return m


def assert_layer_close(actual_f32: np.ndarray, expected_f32: np.ndarray, what: str = "",
                       mean_bar: float = 2e-3):
    """The bar for outputs of the whole routed layer (after the k-way sum of rows that were
    narrowed to the activation dtype).  The mean relative error keeps the GEMM bar (<= 2e-3).
    The elementwise bound is the reference's own one for this operator, |a - e| <= t + t |e|
    with t = 6e-2 for bf16 (crates/nml/tests/nvfp4_contract.rs:510-534): a one-ulp difference
    in one narrowed term is 2^-8 of that term, and the sum of the k terms can be far smaller
    than the term, so a max *relative* error has no fixed bound here."""
    m = oracle.error_metrics(actual_f32, expected_f32)
    assert m["mean_rel"] <= mean_bar and m["max_mixed"] <= 6e-2 and m["norm_rel"] <= 5e-3, (
        what, m)
    return m
