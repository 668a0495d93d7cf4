"""The routed layer for hosts that cannot provide scratch memory.

Some callers of this library cannot allocate device memory when they call it: an XLA
custom-call handler sees only the operand and result buffers the compiler planned, and a
serving runtime may forbid cudaMalloc after start-up.  `nml_nvfp4_sm100_routed_swiglu_static`
serves them by keeping the layer's intermediates in a fixed 8 MiB array inside the library
instead of in a caller-provided workspace.

This test drives that entry point through the C ABI and requires its output to equal, bit
for bit (both run the same kernels), the output of `nml_nvfp4_sm100_routed_swiglu` with a
caller-provided workspace, and to agree with the CPU oracle's evaluation of the layer.  It does so on two calls in a row with different inputs and a
different token count, so that anything the first call leaves in the shared array would
show up in the second.  It also checks the size limit.  The file sorts last so that a run
stopping at the first failure has already run every other test; it passes alone in a fresh
process as well.
"""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from helpers import make_activation, make_weight, rng

pytestmark = pytest.mark.gpu


def host_inputs(tokens, H, E, I, k, seed):
    """The layer's inputs as the oracle takes them (weights as triples, f32 views)."""
    dtype = oracle.BF16
    gate, down = make_weight(seed, (E, 2 * I, H)), make_weight(seed + 1, (E, H, I))
    gate_bias = make_activation(seed + 2, (E, 2 * I), 0.02)
    down_bias = make_activation(seed + 3, (E, H), 0.02)
    hidden = make_activation(seed + 4, (tokens, H))
    logits = rng(seed + 5).standard_normal((tokens, E)).astype(np.float32)
    ids, _, w16 = oracle.route(logits, k, dtype)
    ids[0, 0] = -1  # one masked route
    return gate, down, gate_bias, down_bias, hidden, ids, w16


def build_request(tokens, H, E, I, k, seed, workspace=None):
    from nml_b200 import _abi
    import gpu_util as gu
    dtype = oracle.BF16
    gate_t, down_t, gate_b, down_b, hidden_b, ids, w16 = host_inputs(tokens, H, E, I, k, seed)
    gate = gu.parameter("gate", gate_t, H, dtype)
    down = gu.parameter("down", down_t, I, dtype)
    gate_bias = gu.to_device_bits(gate_b[0], dtype)
    down_bias = gu.to_device_bits(down_b[0], dtype)
    hidden = gu.to_device_bits(hidden_b[0], dtype)
    d_ids = torch.from_numpy(ids).cuda()
    d_w = gu.to_device_bits(w16, dtype)
    out = torch.full((tokens, H), float("nan"), dtype=torch.bfloat16, device="cuda")
    keep = [gate, down, gate_bias, down_bias, hidden, d_ids, d_w, out, workspace]
    request = _abi.RoutedSwiglu(
        hidden=hidden.data_ptr(), expert_ids=d_ids.data_ptr(), routing_weights=d_w.data_ptr(),
        gate_payload=gate.payload.data_ptr(), gate_scales=gate.block_scales.data_ptr(),
        gate_global=gate.global_scale.data_ptr(), gate_bias=gate_bias.data_ptr(),
        down_payload=down.payload.data_ptr(), down_scales=down.block_scales.data_ptr(),
        down_global=down.global_scale.data_ptr(), down_bias=down_bias.data_ptr(),
        output=out.data_ptr(),
        workspace=None if workspace is None else workspace.data_ptr(),
        workspace_bytes=0 if workspace is None else workspace.numel(), stream=0x1,
        tokens=tokens, hidden_size=H, intermediate_size=I, experts=E, experts_per_token=k,
        expert_offset=0, dtype=_abi.BF16)
    return request, out, keep


def test_static_scratch_entry_point_matches_workspace_entry_point_twice():
    from nml_b200 import _abi
    import gpu_util as gu
    lib = _abi.load()
    for tokens, seed in ((48, 21), (7, 33)):  # two calls in a row, second one smaller
        H, E, I, k = 256, 8, 128, 2
        size = lib.nml_nvfp4_sm100_routed_swiglu_workspace_bytes(tokens, H, I, E, k)
        assert 0 < size <= _abi.STATIC_SCRATCH_BYTES
        workspace = torch.empty(size, dtype=torch.uint8, device="cuda")
        expected_request, expected, keep_a = build_request(tokens, H, E, I, k, seed, workspace)
        _abi.call("nml_nvfp4_sm100_routed_swiglu", expected_request)
        static_request, actual, keep_b = build_request(tokens, H, E, I, k, seed)
        _abi.call("nml_nvfp4_sm100_routed_swiglu_static", static_request)
        torch.cuda.synchronize()
        assert _abi.device_status(0x1) == 0
        assert not torch.isnan(actual.float()).any()
        assert np.array_equal(gu.from_device_bits(actual), gu.from_device_bits(expected))
        # and against the CPU oracle's layer (f32 between the projections; the device narrows
        # there like the reference's device path, so the bar is the norm-wise one of the
        # other layer-level tests)
        gate_t, down_t, gate_b, down_b, hidden_b, ids, w16 = host_inputs(tokens, H, E, I, k, seed)
        weights = np.where(ids < 0, 0, oracle.to_f32(w16, oracle.BF16))
        e_layer = oracle.routed_clamped_swiglu(hidden_b[1], np.where(ids < 0, 0, ids), weights,
                                               gate_t, gate_b[1], down_t, down_b[1])
        metrics = oracle.error_metrics(gu.device_f32(actual), e_layer)
        assert metrics["norm_rel"] <= 1e-2, metrics


def test_static_scratch_entry_point_rejects_oversized_requests():
    from nml_b200 import _abi
    # 4096 tokens at GPT-OSS widths need ~190 MB of intermediates: far beyond the 8 MiB array.
    # Validation happens before any pointer is touched, so placeholder addresses suffice.
    fake = 0x1000
    request = _abi.RoutedSwiglu(
        hidden=fake, expert_ids=fake, routing_weights=fake, gate_payload=fake, gate_scales=fake,
        gate_global=fake, gate_bias=fake, down_payload=fake, down_scales=fake, down_global=fake,
        down_bias=fake, output=fake, workspace=None, workspace_bytes=0, stream=0x1, tokens=4096,
        hidden_size=2880, intermediate_size=2880, experts=32, experts_per_token=4,
        expert_offset=0, dtype=_abi.BF16)
    with pytest.raises(_abi.NvFp4Error) as error:
        _abi.call("nml_nvfp4_sm100_routed_swiglu_static", request)
    assert error.value.code == _abi.INVALID_ARGUMENT
    assert "static scratch holds 8388608" in error.value.message
