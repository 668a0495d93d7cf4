"""The weight-streaming kernels (few activation rows) through the C ABI against the oracle.

Dense: every row count from 1 to 16 and the multi-group row counts up to 64, both activation
dtypes, tail tiles (output counts that are not multiples of 16), every K split the planner
produces, fused Q/K/V.  Grouped: decode-size routed batches in both schedule forms.  The bar
is the GEMM bar of gpu_util.assert_gemm_close; runs are deterministic bit for bit.

bf16 activations reach the f16 tensor-core path through a per-slice power-of-two rescale;
the cases with extreme magnitudes pin that it is exact where it has to be."""
import numpy as np
import pytest
import torch

import oracle
from helpers import make_activation, make_weight, rng

pytestmark = pytest.mark.gpu


def stream_linear(x_bits, triple, K, dtype, bias_bits=None):
    from nml_b200 import ops, _abi
    import gpu_util as gu
    weight = gu.parameter("w", triple, K, dtype)
    x = gu.to_device_bits(x_bits, dtype)
    bias = None if bias_bits is None else gu.to_device_bits(bias_bits, dtype)
    previous = _abi.set_kernel_policy(_abi.POLICY_STREAM)
    try:
        y = ops.linear(x, weight, bias)
        again = ops.linear(x, weight, bias)
        torch.cuda.synchronize()
        assert _abi.last_linear_kernel() == "stream"
    finally:
        _abi.set_kernel_policy(previous)
    assert _abi.device_status(0x1) == 0
    assert torch.equal(y.view(torch.int16), again.view(torch.int16))  # deterministic
    return y


@pytest.mark.parametrize("dtype", [oracle.BF16, oracle.F16])
@pytest.mark.parametrize("M,K,N,bias", [
    (1, 64, 16, False), (1, 2880, 2880, True), (2, 2880, 640, False), (3, 128, 20, True),
    (5, 1024, 132, False), (7, 4096, 2880, True), (8, 2880, 5760, False), (9, 192, 48, True),
    (12, 2880, 5120, False), (16, 2880, 2884, True), (16, 4096, 2880, False),
    (15, 3072, 36, True), (16, 960, 4, False), (4, 2880, 100000, False)])
def test_dense_rows_up_to_16(M, K, N, bias, dtype):
    import gpu_util as gu
    triple = make_weight(500 + M + N, (N, K))
    x_bits, x32 = make_activation(600 + M + K, (M, K), dtype=dtype)
    bias_bits = bias32 = None
    if bias:
        bias_bits, bias32 = make_activation(700 + N, (N,), std=0.5, dtype=dtype)
    y = stream_linear(x_bits, triple, K, dtype, bias_bits)
    rows = np.arange(M)
    expected = oracle.linear(x32[rows], *triple, bias32)
    gu.assert_gemm_close(gu.device_f32(y), expected, f"stream M={M} K={K} N={N}")


@pytest.mark.parametrize("M,K,N", [(17, 2880, 2880), (33, 4096, 2880), (64, 2880, 5760),
                                   (48, 512, 200)])
def test_dense_several_groups_of_16_rows(M, K, N):
    import gpu_util as gu
    triple = make_weight(800 + M, (N, K))
    x_bits, x32 = make_activation(801 + M, (M, K))
    bias_bits, bias32 = make_activation(802 + M, (N,), std=0.5)
    y = stream_linear(x_bits, triple, K, oracle.BF16, bias_bits)
    gu.assert_gemm_close(gu.device_f32(y), oracle.linear(x32, *triple, bias32), f"M={M}")


def test_bf16_rescale_is_exact_over_extreme_magnitudes():
    # rows scaled by powers of two far outside the f16 range, a zero row, and one row mixing
    # large and small elements: the result must scale exactly with the row
    import gpu_util as gu
    M, K, N = 8, 2880, 256
    triple = make_weight(900, (N, K))
    base_bits, base = make_activation(901, (1, K))
    factors = np.array([2.0 ** 100, 2.0 ** -100, 1.0, 2.0 ** 30, 0.0, 2.0 ** -60, 3.0, 2.0 ** 60],
                       np.float32)
    x32 = (base * factors[:, None]).astype(np.float32)
    x32[6, ::2] *= np.float32(2.0 ** -20)  # small elements beside large ones
    x_bits = oracle.from_f32(x32, oracle.BF16)
    x32 = oracle.to_f32(x_bits, oracle.BF16)
    y = gu.device_f32(stream_linear(x_bits, triple, K, oracle.BF16))
    expected = oracle.linear(x32, *triple, None)
    assert np.isfinite(y).all()
    assert (y[4] == 0).all()
    for row in (0, 1, 2, 3, 5, 6, 7):
        gu.assert_gemm_close(y[row:row + 1], expected[row:row + 1], f"row {row}")
    # rows 0..3, 5 and 7 are the same activations up to an exact power of two
    unit = y[2]
    for row, power in ((0, 100), (1, -100), (3, 30), (5, -60), (7, 60)):
        assert np.array_equal(y[row], oracle.to_f32(oracle.from_f32(
            unit * np.float32(2.0 ** power), oracle.BF16), oracle.BF16)), row


@pytest.mark.parametrize("dtype", [oracle.BF16, oracle.F16])
@pytest.mark.parametrize("M", [1, 8, 16, 40])
def test_fused_qkv_on_the_streaming_kernel(M, dtype):
    # one launch walks the tiles of three weights; every tile is computed exactly as in a
    # launch of its own weight, so the results equal three separate calls bit for bit
    from nml_b200 import ops, _abi
    import gpu_util as gu
    K, outputs = 2880, (4096, 512, 520)
    x_bits, x32 = make_activation(1000 + M, (M, K), dtype=dtype)
    x = gu.to_device_bits(x_bits, dtype)
    triples = [make_weight(1010 + i, (n, K)) for i, n in enumerate(outputs)]
    weights = [gu.parameter(f"w{i}", t, K, dtype) for i, t in enumerate(triples)]
    bias_bits, bias32 = make_activation(1020, (outputs[0],), std=0.5, dtype=dtype)
    biases = [gu.to_device_bits(bias_bits, dtype), None, None]
    fused = ops.linear_qkv(x, weights[0], biases[0], weights[1], biases[1], weights[2], biases[2])
    torch.cuda.synchronize()
    assert _abi.last_linear_kernel() == "stream"
    for i in range(3):
        single = ops.linear(x, weights[i], biases[i])
        torch.cuda.synchronize()
        assert torch.equal(fused[i].view(torch.int16), single.view(torch.int16)), i
        expected = oracle.linear(x32, *triples[i], bias32 if i == 0 else None)
        gu.assert_gemm_close(gu.device_f32(fused[i]), expected, f"projection {i}")
    assert _abi.device_status(0x1) == 0


@pytest.mark.parametrize("policy_name", ["POLICY_SIMT", "POLICY_UMMA", "POLICY_UMMA_SMEM",
                                         "POLICY_STREAM"])
@pytest.mark.parametrize("dtype", [oracle.BF16, oracle.F16])
def test_invalid_scale_bytes_poison_their_rows_with_nan(policy_name, dtype):
    # crates/nml-kernel-nvfp4/src/turing_adapter.cu:35-40: scale bytes with the sign bit set, or
    # 0x7f, decode to NaN on the device (the CPU path rejects the weight instead,
    # crates/nml-kernel-nvfp4/src/lib.rs:158-176).  Every kernel family must poison exactly the
    # rows that hold such a byte.
    from nml_b200 import ops, _abi
    import gpu_util as gu
    M, K, N = 4, 256, 160
    payload, scales, g = make_weight(1100, (N, K))
    scales = scales.copy()
    payload = payload.copy()
    poisoned = {3: 0x7f, 40: 0x80, 77: 0xff, 130: 0x9c}
    for row, byte in poisoned.items():
        scales[row, (row * 5) % (K // 16)] = byte
    payload[40, :] = 0  # zero codes do not hide the poison: NaN * 0 is NaN
    x_bits, x32 = make_activation(1101, (M, K), dtype=dtype)
    weight = gu.parameter("w", (payload, scales, g), K, dtype)
    previous = _abi.set_kernel_policy(getattr(_abi, policy_name))
    try:
        y = gu.device_f32(ops.linear(gu.to_device_bits(x_bits, dtype), weight))
    finally:
        _abi.set_kernel_policy(previous)
    assert _abi.device_status(0x1) == 0
    bad = np.zeros(N, bool)
    bad[list(poisoned)] = True
    assert np.isnan(y[:, bad]).all()
    assert np.isfinite(y[:, ~bad]).all()
    clean = scales.copy()
    clean[bad] = 0x38
    expected = oracle.linear(x32, payload, clean, g, None)
    gu.assert_gemm_close(y[:, ~bad], expected[:, ~bad], policy_name)


def run_routed_stream(tokens, H, E, I, k, dtype, seed, mask=None):
    """Both projections on the streaming kernel, each against the oracle on its own inputs,
    and the orchestrated layer (which selects the same kernels) against them bit for bit."""
    from nml_b200 import ops, _abi
    import gpu_util as gu
    from test_gpu_moe import make_experts
    gate, down, (gb_bits, gb), (db_bits, db) = make_experts(seed, E, H, I, dtype)
    x_bits, x = make_activation(seed + 9, (tokens, H), 1.0, dtype)
    logits = (rng(seed + 10).standard_normal((tokens, E)) * 0.6).astype(np.float32)
    ids, _, w16 = oracle.route(logits, k, dtype, active=mask)
    w = oracle.to_f32(w16, dtype)
    gate_p, down_p = gu.parameter("gate_up", gate, H, dtype), gu.parameter("down", down, I, dtype)
    d_x, d_gb, d_db = (gu.to_device_bits(b, dtype) for b in (x_bits, gb_bits, db_bits))
    d_ids, d_w = torch.from_numpy(ids).cuda(), gu.to_device_bits(w16, dtype)
    previous = _abi.set_kernel_policy(_abi.POLICY_STREAM)
    try:
        plan = ops.moe_assignment_plan(d_ids.reshape(-1), E)
        activated = ops.expert_gate_up(d_x, plan, gate_p, d_gb, k)
        weighted = ops.expert_down(activated, plan, down_p, d_db, d_w.reshape(-1), k)
        torch.cuda.synchronize()
    finally:
        _abi.set_kernel_policy(previous)
    fused = ops.routed_experts(d_x, d_ids, d_w, gate_p, d_gb, down_p, d_db)  # automatic choice
    combined = ops.combine(weighted, tokens, k, d_ids.reshape(-1), E, 0)
    torch.cuda.synchronize()
    assert _abi.device_status(0x1) == 0
    valid = ids.ravel() >= 0
    e_act = oracle.expert_gate_up(x, ids.ravel(), k, gate, gb)
    gu.assert_gemm_close(gu.device_f32(activated)[valid], e_act[valid], "gate_up")
    e_weighted = oracle.expert_down(gu.device_f32(activated), ids.ravel(), w.ravel(), down, db)
    gu.assert_gemm_close(gu.device_f32(weighted)[valid], e_weighted[valid], "down")
    assert (gu.device_f32(activated)[~valid] == 0).all()  # unscheduled routes are not written
    assert np.array_equal(gu.from_device_bits(fused), gu.from_device_bits(combined))


@pytest.mark.parametrize("tokens,E,k,H,I,dtype", [
    (1, 8, 4, 512, 384, oracle.BF16),       # sparse schedule form: one route per block
    (2, 32, 4, 2880, 2880, oracle.BF16),    # sparse form at GPT-OSS widths
    (6, 8, 4, 512, 384, oracle.F16),        # dense form, a few slots per expert
    (24, 8, 4, 512, 384, oracle.BF16),      # ~12 slots per expert, some experts over 16
    (64, 32, 4, 2880, 2880, oracle.BF16),   # the decode batch of the end-to-end configuration
    (16, 4, 2, 4096, 1024, oracle.BF16),    # K = 4096: sixteen compute warps, padded rows
])
def test_routed_experts_streaming_kernel(tokens, E, k, H, I, dtype):
    mask = None
    if tokens >= 16:
        mask = np.ones(tokens, np.uint8)
        mask[rng(tokens).integers(0, tokens, max(1, tokens // 9))] = 0
    run_routed_stream(tokens, H, E, I, k, dtype, seed=tokens + E + H, mask=mask)


def test_routed_streaming_kernel_with_expert_offset_skips_foreign_blocks():
    # expert-parallel form of the kernel ABI: global ids in the schedule, local weights
    from nml_b200 import ops, _abi
    import gpu_util as gu
    from test_gpu_moe import make_experts
    dtype = oracle.BF16
    E, local, offset, H, I, k, tokens = 8, 4, 4, 256, 128, 2, 24
    gate, down, (gb_bits, gb), (db_bits, db) = make_experts(1200, E, H, I, dtype)
    x_bits, x = make_activation(1201, (tokens, H), 1.0, dtype)
    logits = (rng(1202).standard_normal((tokens, E)) * 0.6).astype(np.float32)
    ids, _, w16 = oracle.route(logits, k, dtype)
    sl = slice(offset, offset + local)
    gate_l = gu.parameter("gate", (gate[0][sl], gate[1][sl], gate[2]), H, dtype)
    down_l = gu.parameter("down", (down[0][sl], down[1][sl], down[2]), I, dtype)
    d_x = gu.to_device_bits(x_bits, dtype)
    d_ids = torch.from_numpy(ids).cuda()
    d_offset = torch.tensor(offset, dtype=torch.int32).cuda()
    plan = ops.moe_assignment_plan(d_ids.reshape(-1), E)
    previous = _abi.set_kernel_policy(_abi.POLICY_STREAM)
    try:
        act = ops.expert_gate_up(d_x, plan, gate_l, gu.to_device_bits(gb_bits[sl], dtype), k,
                                 expert_offset=d_offset)
        out = ops.expert_down(act, plan, down_l, gu.to_device_bits(db_bits[sl], dtype),
                              gu.to_device_bits(w16, dtype).reshape(-1), k,
                              expert_offset=d_offset, use_active_blocks=False)
        torch.cuda.synchronize()
    finally:
        _abi.set_kernel_policy(previous)
    assert _abi.device_status(0x1) == 0
    act32, out32 = gu.device_f32(act), gu.device_f32(out)
    is_local = (ids.ravel() >= offset) & (ids.ravel() < offset + local)
    e_act = oracle.expert_gate_up(x, ids.ravel(), k, gate, gb)
    gu.assert_gemm_close(act32[is_local], e_act[is_local], "gate_up")
    assert (act32[~is_local] == 0).all() and (out32[~is_local] == 0).all()
    e_out = oracle.expert_down(act32, ids.ravel(), oracle.to_f32(w16, dtype).ravel(), down, db)
    gu.assert_gemm_close(out32[is_local], e_out[is_local], "down")
