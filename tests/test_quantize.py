"""The torch quantizer used to make benchmark-size synthetic weights is byte-identical to the
parity oracle (and, through the golden fixtures, to the reference's Python quantizer)."""
import numpy as np
import pytest
import torch

import oracle
from helpers import bf16_round, rng
from nml_b200 import quantize as q


def compare(values: np.ndarray):
    payload, scales, g = q.quantize(torch.from_numpy(values))
    ep, es, eg = oracle.quantize_tensor(values)
    assert np.float32(g.item()) == eg
    assert np.array_equal(payload.numpy(), ep)
    assert np.array_equal(scales.numpy(), es)


@pytest.mark.parametrize("shape,std", [((64, 2880), 0.02), ((7, 17), 1.0), ((3, 5, 33), 0.02),
                                       ((4, 16), 0.0), ((9, 48), 3.0)])
def test_matches_oracle_bytes(shape, std):
    compare(bf16_round(rng(sum(shape)).standard_normal(shape).astype(np.float32) * std))


def test_boundary_values_and_tiny_blocks():
    # values exactly on every E2M1 rounding boundary, both signs, plus blocks whose scale
    # rounds to a subnormal code or to zero next to a large outlier
    values = np.zeros((4, 32), np.float32)
    values[0, :16] = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75,
                      -2.5, -3.5, -5.0, -6.0]
    values[0, 16:] = 6.0
    values[1, :] = 1e-6
    values[2, :16] = np.linspace(-2e-3, 2e-3, 16)
    values[3, 5] = 2688.0
    compare(values)


@pytest.mark.parametrize("name", ["normal_8x64", "odd_width_5x17", "wide_range_6x80",
                                  "experts_3x10x48", "zero_blocks_4x32"])
def test_matches_reference_quantizer_fixture(golden, name):
    source = oracle.to_f32(golden[f"{name}.source_bf16"], oracle.BF16)
    payload, scales, g = q.quantize(torch.from_numpy(source))
    assert np.float32(g.item()) == golden[f"{name}.global"]
    assert np.array_equal(payload.numpy(), golden[f"{name}.payload"])
    assert np.array_equal(scales.numpy(), golden[f"{name}.scales"])


def test_e4m3_encode_matches_oracle_on_dense_grid():
    values = np.concatenate([np.linspace(0, 500, 20001), np.logspace(-6, 2.7, 5000)]).astype(
        np.float32)
    got = q.encode_e4m3fn(torch.from_numpy(values)).numpy()
    want = np.array([oracle.encode_e4m3fn_scale(float(v)) for v in values], np.uint8)
    assert np.array_equal(got, want)
