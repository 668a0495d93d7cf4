"""Shared input builders for the parity tests (seeded, torch-version independent)."""
from __future__ import annotations

import numpy as np

import oracle


def rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


def bf16_bits(values: np.ndarray) -> np.ndarray:
    return oracle.from_f32(np.asarray(values, np.float32), oracle.BF16)


def bf16_round(values: np.ndarray) -> np.ndarray:
    return oracle.to_f32(bf16_bits(values), oracle.BF16)


def make_weight(seed: int, shape, std: float = 0.02):
    """bf16 N(0, std) source -> NVFP4 recipe-v2 triple (payload, scales, g)."""
    source = bf16_round(rng(seed).standard_normal(shape).astype(np.float32) * std)
    return oracle.quantize_tensor(source)


def make_activation(seed: int, shape, std: float = 1.0, dtype: int = oracle.BF16):
    """Returns (bits uint16, f32 view of the same rounded values)."""
    values = rng(seed).standard_normal(shape).astype(np.float32) * std
    bits = oracle.from_f32(values, dtype)
    return bits, oracle.to_f32(bits, dtype)


class Lcg:
    """The generator of crates/nml-kernel-nvfp4/tests/cpu_contract.rs:346-357."""

    def __init__(self, state: int = 0x4E4D4C4E56465034):
        self.state = state

    def unit(self) -> np.float32:
        self.state = (self.state * 6364136223846793005 + 1442695040888963407) & (2**64 - 1)
        return np.float32(np.float32((self.state >> 40) & 0xFFFFFFFF) / np.float32((1 << 24) - 1))

    def values(self, count: int, magnitude: float) -> np.ndarray:
        return np.array([(self.unit() * np.float32(2.0) - np.float32(1.0)) * np.float32(magnitude)
                         for _ in range(count)], np.float32)
