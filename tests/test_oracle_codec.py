"""Pins the CPU oracle's codec to the reference's known-answer tests and to the
outputs of the reference's Python quantizer/decoder (golden fixtures)."""
import numpy as np
import pytest

import oracle


def f32_bits(x):
    return np.float32(x).view(np.uint32)


def test_e2m1_all_sixteen_codes_bit_exact():
    # crates/nml-parameter/tests/parameter_contract.rs:84-94
    expected = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0,
                -6.0]
    for code, value in enumerate(expected):
        assert f32_bits(oracle.decode_e2m1(code)) == f32_bits(value), hex(code)


def test_e4m3fn_scale_known_answers_and_rejections():
    # crates/nml-parameter/tests/parameter_contract.rs:96-104
    assert oracle.decode_e4m3fn_scale(0x00) == 0.0
    assert oracle.decode_e4m3fn_scale(0x01) == 2.0 ** -9
    assert oracle.decode_e4m3fn_scale(0x38) == 1.0
    assert oracle.decode_e4m3fn_scale(0x7E) == 448.0
    for bad in (0x7F, 0x80, 0xFF):
        with pytest.raises(ValueError):
            oracle.decode_e4m3fn_scale(bad)


def test_e4m3fn_encode_round_trips_every_valid_code():
    for bits in range(0x7F):
        assert oracle.encode_e4m3fn_scale(oracle.decode_e4m3fn_scale(bits)) == bits
    assert oracle.encode_e4m3fn_scale(1e9) == 0x7E  # saturates at 448
    # exact midpoint between 1.0 (0x38, even) and 1.125 (0x39): ties to the even code
    assert oracle.encode_e4m3fn_scale(1.0625) == 0x38
    assert oracle.encode_e4m3fn_scale(1.1875) == 0x3A


def test_e2m1_encode_thresholds_tie_to_even_code():
    # tools/nvfp4/convert.py:24,388-397: boundaries 0.25 .75 1.25 1.75 2.5 3.5 5
    cases = {0.25: 0, 0.75: 2, 1.25: 2, 1.75: 4, 2.5: 4, 3.5: 6, 5.0: 6, 100.0: 7, 0.2: 0,
             0.26: 1}
    for value, code in cases.items():
        assert oracle.encode_e2m1(value) == code, value
        assert oracle.encode_e2m1(-value) == (code | 8), value
    assert oracle.encode_e2m1(-0.0) == 8


def test_row_codec_low_nibble_first_and_padding():
    # crates/nml-parameter/tests/parameter_contract.rs:106-131
    values = np.array([-6.0, -4.0, -3.0, -2.0, -1.5, -1.0, -0.5, -0.0, 0.0, 0.5, 1.0, 1.5, 2.0,
                       3.0, 4.0, 6.0, 0.0], np.float32)
    g = oracle.global_scale(values)
    assert g == np.float32(1.0 / 448.0)
    payload, scales = oracle.quantize_row(values, g)
    assert list(scales) == [0x7E, 0x00]
    assert payload[0] == 0xEF and payload[7] == 0x76 and payload[8] == 0x00
    decoded = oracle.dequantize_row(payload, scales, g, values.size)
    assert np.array_equal(decoded.view(np.uint32), values.view(np.uint32))
    invalid = payload.copy()
    invalid[-1] = 0x10
    with pytest.raises(ValueError):
        oracle.dequantize_row(invalid, scales, g, values.size)


def test_weight_validation_rejections():
    # crates/nml-kernel-nvfp4/src/lib.rs:128-176
    values = np.linspace(-3, 3, 34, dtype=np.float32).reshape(2, 17)
    payload, scales, g = oracle.quantize_tensor(values)
    assert oracle.validate_weight(payload, scales, g, 2, 17) == 0
    assert oracle.validate_weight(payload, scales, 0.0, 2, 17) == 1
    assert oracle.validate_weight(payload, scales, float("inf"), 2, 17) == 1
    bad = payload.copy(); bad[0, -1] |= 0x10
    assert oracle.validate_weight(bad, scales, g, 2, 17) == 2
    bad = scales.copy(); bad[1, 0] = 0x7F
    assert oracle.validate_weight(payload, bad, g, 2, 17) == 3
    bad = scales.copy(); bad[0, 0] = 0x00
    assert oracle.validate_weight(payload, bad, g, 2, 17) == 4


CASES = ["normal_8x64", "odd_width_5x17", "width_33", "experts_3x10x48", "zero_blocks_4x32",
         "all_zero_2x16", "wide_range_6x80", "gpt_oss_row_2x2880"]


@pytest.mark.parametrize("name", CASES)
def test_quantizer_matches_reference_python_quantizer_bytes(golden, name):
    source = oracle.to_f32(golden[f"{name}.source_bf16"], oracle.BF16)
    payload, scales, g = oracle.quantize_tensor(source)
    assert np.float32(g) == golden[f"{name}.global"]
    assert np.array_equal(payload, golden[f"{name}.payload"])
    assert np.array_equal(scales, golden[f"{name}.scales"])


@pytest.mark.parametrize("name", CASES)
def test_decoder_matches_reference_spec_decoder_bits(golden, name):
    payload, scales = golden[f"{name}.payload"], golden[f"{name}.scales"]
    g = golden[f"{name}.global"]
    expected = golden[f"{name}.decoded"]
    width = expected.shape[-1]
    decoded = oracle.dequantize_tensor(payload, scales, g, width)
    assert np.array_equal(decoded.view(np.uint32), expected.view(np.uint32))
    flat_p = payload.reshape(-1, payload.shape[-1])
    flat_s = scales.reshape(-1, scales.shape[-1])
    assert oracle.validate_weight(flat_p, flat_s, g, flat_p.shape[0], width) == 0


def test_fixture_projection_matches_reference_tool(golden):
    # tools/nvfp4/extract_fixture.py:95-110: exact (fsum) projection of the fixed input
    x = golden["fixture_input_2880"]
    payload = golden["gpt_oss_row_2x2880.payload"]
    scales = golden["gpt_oss_row_2x2880.scales"]
    g = golden["gpt_oss_row_2x2880.global"]
    y64 = oracle.linear(x[None, :], payload, scales, g, mode=1)[0]
    y32 = oracle.linear(x[None, :], payload, scales, g, mode=0)[0]
    expected = golden["fixture_projection_2x2880"]
    assert np.allclose(y64, expected, rtol=1e-6, atol=1e-7)
    assert np.allclose(y32, expected, rtol=2e-5, atol=2e-5)


def test_bf16_and_f16_narrowing_round_to_nearest_even():
    import torch
    values = np.concatenate([
        np.random.default_rng(1).standard_normal(4096).astype(np.float32) * 3,
        np.array([0.0, -0.0, 1.00390625, 1.01171875, 65504.0, 65520.0, 1e-8, 6e-8, 5.96e-8,
                  3.0e-5, float("inf"), -float("inf")], np.float32)])
    t = torch.from_numpy(values)
    for dtype, torch_dtype in ((oracle.BF16, torch.bfloat16), (oracle.F16, torch.float16)):
        bits = oracle.from_f32(values, dtype)
        expected = t.to(torch_dtype).view(torch.int16).numpy().view(np.uint16)
        assert np.array_equal(bits, expected)
        back = oracle.to_f32(bits, dtype)
        assert np.array_equal(back, t.to(torch_dtype).float().numpy())
